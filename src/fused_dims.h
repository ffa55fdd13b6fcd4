/* fused_dims.h -- the one transformer shape the fused kernels accept; fluke_*_select returns
 * NULL for anything else so the caller keeps its fp16 path (reference: src/fused_dims.h:8-11). */
#ifndef FLUKE_SRC_FUSED_DIMS_H
#define FLUKE_SRC_FUSED_DIMS_H

#define FLUKE_SUP_D_MODEL 512
#define FLUKE_SUP_DIM_FF 2048
#define FLUKE_SUP_NHEAD 8
#define FLUKE_SUP_HEAD_DIM 64

#endif
