// fluke_sm100_all.cu -- the single sm_100a translation unit of the library: the kernel
// sources are included here so they share one copy of the device status word and of the
// tcgen05/TMA helpers, and the library needs no relocatable device code.
#include "rowwise_sm100.cu"
#include "gemm_sm100.cu"
#include "lstm_sm100.cu"
#include "lstm_persist_sm100.cu"
#include "lstm_cluster_sm100.cu"
#include "lstm_noalloc_sm100.cu"
#include "stack_sm100.cu"
