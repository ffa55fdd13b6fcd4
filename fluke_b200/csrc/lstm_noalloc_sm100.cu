// lstm_noalloc_sm100.cu -- a factored-LSTM layer entry point for callers that cannot allocate
// device memory.
//
// Some hosts of this library may not call cudaMalloc at the point where they run a layer:
// plug-ins that are handed device pointers but own no allocator, services whose memory budget
// is fixed at start-up, and code in regions where the CUDA allocator must not be called. fluke_factored_lstm_layer_i8_gpu asks such a caller for a workspace it has no
// way to provide. The variant below takes the same layer description, ignores its workspace
// fields and keeps the intermediate tensors (hh_down [B,R] and x_down [T,B,R], f16) in a fixed
// 4 MiB array that is part of the library image, so nothing is allocated -- by this function or
// by anything it calls -- at any time.
//
// What to know before using it:
//  * Size limit. The layer must fit the built-in array:
//    fluke_factored_lstm_layer_workspace(T,B,H,R) <= FLUKE_LSTM_NOALLOC_SCRATCH_BYTES (4 MiB),
//    e.g. 1024 chunks x 14 timesteps, or 128 chunks x 126 timesteps, at rank 128 (the workspace
//    is 256 bytes x (T + 1) per chunk plus 1 KB). Larger layers are refused with a message on
//    stderr and a non-zero return; nothing is launched. Long sequences can be run as several
//    calls, the state (c, h) carries over.
//  * Cost. Every GPU on which the library is loaded holds the 4 MiB until the process exits,
//    whether or not this entry point is ever called.
//  * First call per device. It looks up the device address of the array (the array's name in
//    host code is only a host-side handle, not something a kernel can dereference) and caches
//    it, and the kernels it launches are configured on their first use. Make the first call on
//    a device -- with the layer shape (B, H, R) and the fluke_set_lstm_persistent mode that later
//    calls will use, since those choose the kernels -- before any stream capture begins, with the
//    device current.
//  * One layer at a time per device. All calls share the one array; it still holds the previous
//    call's intermediates when the next call starts. That is harmless -- every element a layer
//    reads has been written by the same call first, and rows past B are never read from memory
//    -- so nothing is cleared. But two calls whose kernels overlap on the GPU (different
//    streams, or different host threads) race on the array and corrupt each other.
#include <fluke/fluke.h>

#include "fluke_sm100.h"

#include <cuda_runtime.h>
#include <stdio.h>

extern "C" int fluke_host_note_error(int code);  // src/nn_gpu.c: records the last error text

namespace {

static __device__ __align__(256) unsigned char g_lstm_noalloc_scratch[FLUKE_LSTM_NOALLOC_SCRATCH_BYTES];

// Device address of the array on the current device, resolved once per device.
int noalloc_scratch_ptr(void **out) {
    static void *cached[64] = {nullptr};
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return (int)e;
    if (dev < 0 || dev >= 64) return (int)cudaErrorInvalidDevice;
    if (!cached[dev]) {
        void *p = nullptr;
        e = cudaGetSymbolAddress(&p, g_lstm_noalloc_scratch);
        if (e != cudaSuccess) return (int)e;
        cached[dev] = p;
    }
    *out = cached[dev];
    return 0;
}

}  // namespace

extern "C" int fluke_factored_lstm_layer_i8_noalloc_gpu(const fluke_flstm_layer_t *layer) {
    if (!layer) return -1;
    const size_t need = fluke_sm100_lstm_layer_workspace(layer->T, layer->B, layer->H, layer->R);
    if (need == 0) return fluke_host_note_error((int)cudaErrorInvalidValue);
    if (need > (size_t)FLUKE_LSTM_NOALLOC_SCRATCH_BYTES) {
        fprintf(stderr,
                "[fluke] fluke_factored_lstm_layer_i8_noalloc_gpu: T=%d B=%d R=%d needs %zu bytes of "
                "intermediates, the built-in buffer holds %zu; split the sequence or use "
                "fluke_factored_lstm_layer_i8_gpu with a workspace\n",
                layer->T, layer->B, layer->R, need, (size_t)FLUKE_LSTM_NOALLOC_SCRATCH_BYTES);
        return fluke_host_note_error((int)cudaErrorInvalidValue);
    }
    void *scratch = nullptr;
    int rc = noalloc_scratch_ptr(&scratch);
    if (rc) return fluke_host_note_error(rc);
    fluke_flstm_layer_t l = *layer;
    l.workspace = scratch;
    l.workspace_bytes = (size_t)FLUKE_LSTM_NOALLOC_SCRATCH_BYTES;
    return fluke_host_note_error(fluke_sm100_lstm_layer(&l, fluke_get_stream()));
}
