// mma_peak_sm100.cu -- issue-rate probe for tcgen05.mma: the measured tensor-pipe ceiling that
// the GEMM-class kernels of this library are compared against (the pool's measured peaks only
// cover bf16 through cuBLAS). Every SM runs one CTA that issues `iters` back-to-back MMAs of
// shape 128 x N x 32 bytes on operand tiles resident in shared memory (contents irrelevant:
// zeros) and times them with clock64; no global traffic is involved.
// Built on its own into lib/libfluke_probe.so (`make probe cuda=1`) for the benchmark; it is not
// part of libfluke.
#include "fluke_sm100.h"
#include "sm100_ptx.cuh"

namespace fluke_sm100 {
namespace {

template <int KIND>
__global__ void __launch_bounds__(64, 1) mma_peak_kernel(int n, int iters, long long *cycles) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *sa = smem;                 // 128 rows x 128 B
    uint8_t *sb = smem + 16384;         // 256 rows x 128 B
    uint64_t *bar = reinterpret_cast<uint64_t *>(smem + 16384 + 32768);
    uint32_t *slot = reinterpret_cast<uint32_t *>(smem + 16384 + 32768 + 8);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + 16384 + 32768 + 16);
    for (int i = threadIdx.x; i < (16384 + 32768) / 16; i += blockDim.x)
        reinterpret_cast<uint4 *>(smem)[i] = make_uint4(0, 0, 0, 0);
    if (threadIdx.x == 0) {
        mbar_init(bar, 1);
        *abort_flag = 0;
        fence_barrier_init();
    }
    fence_proxy_async_smem();
    if (threadIdx.x < 32) tmem_alloc(slot, 256);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem = *slot;
    if (threadIdx.x == 0) {
        const uint32_t idesc = (KIND == kKindI8 ? 2u : 1u) << 4 | (KIND == kKindI8 ? 1u : 0u) << 7 |
                               (KIND == kKindI8 ? 1u : 0u) << 10 | (uint32_t(n >> 3) << 17) | (8u << 24);
        const uint64_t ad = make_smem_desc_sw128(smem_u32(sa)), bd = make_smem_desc_sw128(smem_u32(sb));
        const long long t0 = clock64();
        for (int i = 0; i < iters; ++i) tc_mma<KIND>(tmem, ad + uint64_t(2 * (i & 3)), bd + uint64_t(2 * (i & 3)), idesc, 1u);
        tc_commit(bar);
        mbar_wait(bar, 0, abort_flag, 70);
        cycles[blockIdx.x] = clock64() - t0;
    }
    tc_fence_before_sync();
    __syncthreads();
    if (threadIdx.x < 32) {
        tc_fence_after_sync();
        tmem_dealloc(tmem, 256);
    }
}

}  // namespace
}  // namespace fluke_sm100

// kind: 0 int8, 1 e4m3, 2 f16. Fills cycles_dev[0 .. n_sms) (device memory) with the SM-clock
// cycles each CTA needed for `iters` MMAs of 128 x n x (32 bytes of K).
extern "C" int fluke_sm100_mma_peak(int kind, int n, int iters, void *cycles_dev, int n_ctas, void *stream) {
    using namespace fluke_sm100;
    if (n < 16 || n > 256 || n % 16 || iters < 1) return (int)cudaErrorInvalidValue;
    const int smem = 16384 + 32768 + 64 + 1024;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    long long *c = static_cast<long long *>(cycles_dev);
    cudaError_t e;
    if (kind == 0) {
        e = cudaFuncSetAttribute(mma_peak_kernel<kKindI8>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e == cudaSuccess) mma_peak_kernel<kKindI8><<<n_ctas, 64, smem, s>>>(n, iters, c);
    } else if (kind == 1) {
        e = cudaFuncSetAttribute(mma_peak_kernel<kKindF8>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e == cudaSuccess) mma_peak_kernel<kKindF8><<<n_ctas, 64, smem, s>>>(n, iters, c);
    } else {
        e = cudaFuncSetAttribute(mma_peak_kernel<kKindF16>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e == cudaSuccess) mma_peak_kernel<kKindF16><<<n_ctas, 64, smem, s>>>(n, iters, c);
    }
    if (e != cudaSuccess) return (int)e;
    return (int)cudaGetLastError();
}
