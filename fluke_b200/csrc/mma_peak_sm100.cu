// mma_peak_sm100.cu -- issue-rate probe for tcgen05.mma: the measured tensor-pipe ceiling that
// the GEMM-class kernels of this library are compared against (the pool's measured peaks only
// cover bf16 through cuBLAS). Every SM runs one CTA that issues `iters` back-to-back MMAs of
// shape 128 x N x 32 bytes on operand tiles resident in shared memory and times them with
// clock64 and the global nanosecond timer; no global traffic is involved. The operand tiles are
// zeros (pattern 0: the issue rate at whatever clock an idle data path allows) or pseudo-random
// bytes (pattern 1: the data path toggles, the board's power limit pulls the SM clock down within
// tens of microseconds, and the figure is what the tensor pipe sustains under that limit).
// A second kernel samples the SM clock from inside the GPU (cycle counter against the
// nanosecond timer) while other kernels run: nvidia-smi's 100 ms samples cannot see the clock
// of a burst of a few milliseconds.
// Built on its own into lib/libfluke_probe.so (`make probe cuda=1`) for the benchmark; it is not
// part of libfluke.
#include "fluke_sm100.h"
#include "sm100_ptx.cuh"

namespace fluke_sm100 {
namespace {

__device__ __forceinline__ long long global_ns() {
    long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}

template <int KIND>
__global__ void __launch_bounds__(64, 1) mma_peak_kernel(int n, int iters, int pattern, long long *cycles) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint8_t *sa = smem;                 // 128 rows x 128 B
    uint8_t *sb = smem + 16384;         // 256 rows x 128 B
    uint64_t *bar = reinterpret_cast<uint64_t *>(smem + 16384 + 32768);
    uint32_t *slot = reinterpret_cast<uint32_t *>(smem + 16384 + 32768 + 8);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + 16384 + 32768 + 16);
    for (int i = threadIdx.x; i < (16384 + 32768) / 16; i += blockDim.x) {
        uint4 v = make_uint4(0, 0, 0, 0);
        if (pattern) {
            // xorshift words; bit 6 of every byte cleared so that no e4m3 or f16 element has an
            // all-ones exponent (the accumulators stay finite-ish; the values do not matter)
            uint32_t x = 0x9E3779B9u * uint32_t(i + 1) + 0x7F4A7C15u * (blockIdx.x + 1);
            uint32_t w[4];
            for (int k = 0; k < 4; ++k) {
                x ^= x << 13; x ^= x >> 17; x ^= x << 5;
                w[k] = x & 0xBFBFBFBFu;
            }
            v = make_uint4(w[0], w[1], w[2], w[3]);
        }
        reinterpret_cast<uint4 *>(smem)[i] = v;
    }
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
        const long long t0 = clock64(), n0 = global_ns();
        // the first MMA overwrites the accumulator, the rest accumulate
        for (int i = 0; i < iters; ++i)
            tc_mma<KIND>(tmem, ad + uint64_t(2 * (i & 3)), bd + uint64_t(2 * (i & 3)), idesc, i ? 1u : 0u);
        tc_commit(bar);
        mbar_wait(bar, 0, abort_flag, 70);
        cycles[2 * blockIdx.x] = clock64() - t0;
        cycles[2 * blockIdx.x + 1] = global_ns() - n0;
    }
    tc_fence_before_sync();
    __syncthreads();
    if (threadIdx.x < 32) {
        tc_fence_after_sync();
        tmem_dealloc(tmem, 256);
    }
}

// One thread: `n` samples of (cycle counter, nanosecond timer), `gap_ns` apart.
__global__ void clock_sample_kernel(long long *out, int n, int gap_ns) {
    for (int i = 0; i < n; ++i) {
        const long long c = clock64(), t = global_ns();
        out[2 * i] = c;
        out[2 * i + 1] = t;
        long long t1 = t;
        while (t1 - t < gap_ns) t1 = global_ns();
    }
}

}  // namespace
}  // namespace fluke_sm100

// Samples the SM clock from one thread of one CTA for n * gap_ns nanoseconds: out_dev receives n
// pairs (cycles, nanoseconds); successive differences give the clock. Launch it on a stream of
// its own BEFORE the work to be observed, which must leave one SM free or share SMs with small CTAs.
extern "C" int fluke_sm100_clock_samples(void *out_dev, int n, int gap_ns, void *stream) {
    if (n < 2 || n > (1 << 20) || gap_ns < 1000) return (int)cudaErrorInvalidValue;
    fluke_sm100::clock_sample_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(static_cast<long long *>(out_dev), n, gap_ns);
    return (int)cudaGetLastError();
}

// kind: 0 int8, 1 e4m3, 2 f16; pattern: 0 zero operands, 1 pseudo-random operands. Fills
// cycles_dev[0 .. 2 n_ctas) (device memory) with, per CTA, the SM-clock cycles and the nanoseconds
// it needed for `iters` MMAs of 128 x n x (32 bytes of K).
extern "C" int fluke_sm100_mma_peak(int kind, int n, int iters, int pattern, void *cycles_dev, int n_ctas, void *stream) {
    using namespace fluke_sm100;
    if (n < 16 || n > 256 || n % 16 || iters < 1) return (int)cudaErrorInvalidValue;
    const int smem = 16384 + 32768 + 64 + 1024;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    long long *c = static_cast<long long *>(cycles_dev);
    cudaError_t e;
    if (kind == 0) {
        e = cudaFuncSetAttribute(mma_peak_kernel<kKindI8>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e == cudaSuccess) mma_peak_kernel<kKindI8><<<n_ctas, 64, smem, s>>>(n, iters, pattern, c);
    } else if (kind == 1) {
        e = cudaFuncSetAttribute(mma_peak_kernel<kKindF8>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e == cudaSuccess) mma_peak_kernel<kKindF8><<<n_ctas, 64, smem, s>>>(n, iters, pattern, c);
    } else {
        e = cudaFuncSetAttribute(mma_peak_kernel<kKindF16>, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        if (e == cudaSuccess) mma_peak_kernel<kKindF16><<<n_ctas, 64, smem, s>>>(n, iters, pattern, c);
    }
    if (e != cudaSuccess) return (int)e;
    return (int)cudaGetLastError();
}
