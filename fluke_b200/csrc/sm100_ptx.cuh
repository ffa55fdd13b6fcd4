// sm100_ptx.cuh -- inline-PTX building blocks for the sm_100a kernels: mbarriers with
// bounded waits, TMA tile copies, tensor-memory allocation, tcgen05 MMA issue/commit and
// tensor-memory loads, plus the shared-memory and instruction descriptors they consume.
#pragma once

#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace fluke_sm100 {

// ---------------------------------------------------------------------------------------
// Device status word (see fluke_sm100_read_status). Set once by the first wait that gives up.
// ---------------------------------------------------------------------------------------
__device__ unsigned int g_status = 0;

// Cycle budget of any single wait (about a second at B200 clocks). Kernels in this library
// wait for at most a few hundred microseconds when healthy.
constexpr long long kWaitCycleLimit = 1ll << 31;

__device__ __forceinline__ void report_timeout(unsigned int site) {
    atomicCAS(&g_status, 0u, 1u | (site << 8));
}

// Time stamps for stage tables: compiled in only with -DFLUKE_SM100_TRACE. `p` is the kernel's
// parameter block with a `trace` pointer.
#ifdef FLUKE_SM100_TRACE
#define FLUKE_STAMP(cond, slot, now) \
    do { if (p.trace && (cond)) p.trace[(slot)] = (now); } while (0)
#else
#define FLUKE_STAMP(cond, slot, now) do {} while (0)
#endif

// ---------------------------------------------------------------------------------------
// Addresses, election, fences
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t smem_u32(const void *p) {
    return static_cast<uint32_t>(__cvta_generic_to_shared(p));
}

// True in exactly one lane of a converged warp.
__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile(
        "{\n"
        ".reg .pred P;\n"
        "elect.sync _|P, 0xffffffff;\n"
        "selp.u32 %0, 1, 0, P;\n"
        "}\n"
        : "=r"(pred));
    return pred != 0;
}

// Per-warpgroup register budget (all four warps of the warpgroup execute it together).
template <int N>
__device__ __forceinline__ void reg_alloc() {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 %0;" ::"n"(N));
}
template <int N>
__device__ __forceinline__ void reg_dealloc() {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 %0;" ::"n"(N));
}

// Orders generic-proxy shared-memory writes before later async-proxy (TMA, tcgen05) reads.
__device__ __forceinline__ void fence_proxy_async_smem() {
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
// Same for global memory written with ordinary stores and later read by TMA.
__device__ __forceinline__ void fence_proxy_async_all() {
    asm volatile("fence.proxy.async;" ::: "memory");
}
__device__ __forceinline__ void fence_barrier_init() {
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}

// ---------------------------------------------------------------------------------------
// mbarrier
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t arrivals) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(arrivals)
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_arrive_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)),
                 "r"(bytes)
                 : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint64_t *bar, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n"
        ".reg .pred P;\n"
        "mbarrier.try_wait.parity.shared::cta.b64 P, [%1], %2;\n"
        "selp.u32 %0, 1, 0, P;\n"
        "}\n"
        : "=r"(done)
        : "r"(smem_u32(bar)), "r"(parity)
        : "memory");
    return done != 0;
}

// Waits for the phase with the given parity to complete. Gives up after `limit` cycles
// (kWaitCycleLimit in every kernel of the library): records `site` in the status word, raises
// *abort_flag (shared memory, seen by the other roles of the CTA) and returns false. A raised
// abort flag also ends the wait.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, volatile int *abort_flag,
                                          unsigned int site, long long limit = kWaitCycleLimit) {
    if (mbar_try_wait(bar, parity)) return true;
    const long long t0 = clock64();
    for (;;) {
#pragma unroll 1
        for (int i = 0; i < 64; ++i)
            if (mbar_try_wait(bar, parity)) return true;
        if (*abort_flag) return false;
        if (clock64() - t0 > limit) {
            report_timeout(site);
            *abort_flag = 1;
            return false;
        }
    }
}

// ---------------------------------------------------------------------------------------
// Counters in global memory that CTAs of one launch hand data over with
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ unsigned int ld_acquire_u32(const unsigned int *p) {
    unsigned int v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ unsigned int ld_relaxed_u32(const unsigned int *p) {
    unsigned int v;
    asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// Waits until *flag >= target. Gives up when `limit` cycles have passed or another CTA has raised
// the global abort word; then raises both abort flags and returns false (a timeout also records
// `site` in the status word).
__device__ __forceinline__ bool wait_counter(const unsigned int *flag, unsigned int target,
                                             unsigned int *g_abort, volatile int *abort_flag,
                                             unsigned int site, long long limit = kWaitCycleLimit) {
    const long long t0 = clock64();
    unsigned int spins = 0;
    for (;;) {
        // poll with relaxed loads; one acquire fence orders the data reads after the sighting
        if (ld_relaxed_u32(flag) >= target) {
            asm volatile("fence.acq_rel.gpu;" ::: "memory");
            return true;
        }
        if (*abort_flag) return false;
        if ((++spins & 63u) == 0u) {
            const bool late = clock64() - t0 > limit;
            if (late || ld_acquire_u32(g_abort) != 0u) {
                if (late) report_timeout(site);
                *abort_flag = 1;
                atomicExch(g_abort, 1u);
                return false;
            }
        }
    }
}

// ---------------------------------------------------------------------------------------
// TMA (cp.async.bulk.tensor), 2-D and 3-D tiles; loads complete on an mbarrier, stores are
// tracked with bulk groups.
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap *m) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(reinterpret_cast<uint64_t>(m)) : "memory");
}
__device__ __forceinline__ void tma_load_2d(void *smem_dst, const CUtensorMap *m, uint64_t *bar,
                                            int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)),
          "r"(c0), "r"(c1)
        : "memory");
}
__device__ __forceinline__ void tma_load_4d(void *smem_dst, const CUtensorMap *m, uint64_t *bar,
                                            int c0, int c1, int c2, int c3) {
    asm volatile(
        "cp.async.bulk.tensor.4d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5, %6}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)),
          "r"(c0), "r"(c1), "r"(c2), "r"(c3)
        : "memory");
}
__device__ __forceinline__ void tma_load_3d(void *smem_dst, const CUtensorMap *m, uint64_t *bar,
                                            int c0, int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes"
        " [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(bar)),
          "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}
// Brings a box into L2 only (no shared-memory destination, nothing to wait for).
__device__ __forceinline__ void tma_prefetch_l2_3d(const CUtensorMap *m, int c0, int c1, int c2) {
    asm volatile("cp.async.bulk.prefetch.tensor.3d.L2.global [%0, {%1, %2, %3}];"
                 ::"l"(reinterpret_cast<uint64_t>(m)), "r"(c0), "r"(c1), "r"(c2)
                 : "memory");
}
__device__ __forceinline__ void tma_store_2d(const CUtensorMap *m, const void *smem_src, int c0,
                                             int c1) {
    asm volatile("cp.async.bulk.tensor.2d.global.shared::cta.bulk_group [%0, {%2, %3}], [%1];"
                 ::"l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(smem_src)), "r"(c0), "r"(c1)
                 : "memory");
}
__device__ __forceinline__ void tma_store_3d(const CUtensorMap *m, const void *smem_src, int c0,
                                             int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.global.shared::cta.bulk_group [%0, {%2, %3, %4}], [%1];"
        ::"l"(reinterpret_cast<uint64_t>(m)), "r"(smem_u32(smem_src)), "r"(c0), "r"(c1), "r"(c2)
        : "memory");
}
__device__ __forceinline__ void tma_store_commit() {
    asm volatile("cp.async.bulk.commit_group;" ::: "memory");
}
// Blocks until at most N of this thread's bulk groups still READ their shared-memory source.
template <int N>
__device__ __forceinline__ void tma_store_wait_read() {
    asm volatile("cp.async.bulk.wait_group.read %0;" ::"n"(N) : "memory");
}
// Blocks until at most N bulk groups are incomplete (writes performed).
template <int N>
__device__ __forceinline__ void tma_store_wait_all() {
    asm volatile("cp.async.bulk.wait_group %0;" ::"n"(N) : "memory");
}

// ---------------------------------------------------------------------------------------
// Tensor memory (TMEM) and tcgen05
// ---------------------------------------------------------------------------------------
// One full warp allocates `cols` (power of two, 32..512) columns; the base address lands in
// *smem_slot.
__device__ __forceinline__ void tmem_alloc(uint32_t *smem_slot, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(
                     smem_u32(smem_slot)),
                 "r"(cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols)
                 : "memory");
}
__device__ __forceinline__ void tc_fence_before_sync() {
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_after_sync() {
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
}
// Arrives once on `bar` when every MMA issued so far by this thread has finished.
__device__ __forceinline__ void tc_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                     smem_u32(bar))
                 : "memory");
}

enum MmaKind { kKindI8 = 0, kKindF8 = 1, kKindF16 = 2 };

// D[tmem] (+)= A[smem] * B[smem]^T; `accumulate` == 0 overwrites D.
template <int KIND>
__device__ __forceinline__ void tc_mma(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc,
                                       uint32_t idesc, uint32_t accumulate) {
    if constexpr (KIND == kKindI8) {
        asm volatile(
            "{\n.reg .pred P;\nsetp.ne.b32 P, %4, 0;\n"
            "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, P;\n}\n"
            ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
            : "memory");
    } else if constexpr (KIND == kKindF8) {
        asm volatile(
            "{\n.reg .pred P;\nsetp.ne.b32 P, %4, 0;\n"
            "tcgen05.mma.cta_group::1.kind::f8f6f4 [%0], %1, %2, %3, P;\n}\n"
            ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
            : "memory");
    } else {
        asm volatile(
            "{\n.reg .pred P;\nsetp.ne.b32 P, %4, 0;\n"
            "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, P;\n}\n"
            ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
            : "memory");
    }
}

// Instruction descriptor for a dense, K-major x K-major MMA of shape M x N (x 32 bytes of K).
//   bits [4,6) accumulator format, [7,10) A format, [10,13) B format, 15/16 A/B major
//   (0 = K), [17,23) N/8, [24,29) M/16.
template <int KIND>
__host__ __device__ constexpr uint32_t make_idesc(int M, int N) {
    const uint32_t c_fmt = (KIND == kKindI8) ? 2u : 1u;   // S32 : F32
    const uint32_t ab_fmt = (KIND == kKindI8) ? 1u : 0u;  // S8 : (E4M3 | F16)
    return (c_fmt << 4) | (ab_fmt << 7) | (ab_fmt << 10) | (uint32_t(N >> 3) << 17) |
           (uint32_t(M >> 4) << 24);
}

// Shared-memory matrix descriptor of a K-major tile stored as rows of 128 bytes in the
// 128-byte swizzle (what a TMA load with CU_TENSOR_MAP_SWIZZLE_128B writes): groups of
// 8 rows are 1024 bytes apart. `byte_addr` is the shared-window address of the first row
// (1024-byte aligned tile; +32 bytes per further K step of the same rows).
__device__ __forceinline__ uint64_t make_smem_desc_sw128(uint32_t byte_addr) {
    uint64_t d = 0;
    d |= uint64_t((byte_addr & 0x3FFFFu) >> 4);  // start address
    d |= uint64_t(1) << 16;                      // leading byte offset (unused when swizzled)
    d |= uint64_t(1024 >> 4) << 32;              // stride byte offset: 8 rows x 128 B
    d |= uint64_t(1) << 46;                      // descriptor version of sm_100
    d |= uint64_t(2) << 61;                      // layout: 128-byte swizzle
    return d;
}

// 32 lanes x 32 columns of 32-bit cells: thread i of the warp receives row (lane base + i),
// columns [col, col+32). The warp may only touch lanes 32*(warp_id%4) .. +31.
__device__ __forceinline__ void tmem_ld_32x32(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
          "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
          "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_32x16(uint32_t taddr, uint32_t (&r)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}
// 16 lanes x 256 bits, repeated over 8 groups of 8 columns: thread (g = lane/4, t = lane%4) of
// the warp receives in r[4j .. 4j+3] the 32-bit cells (row g, columns 8j+2t, 8j+2t+1) and
// (row g+8, the same two columns) of the 16 lanes starting at the address's lane.
__device__ __forceinline__ void tmem_ld_16x256_x8(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.16x256b.x8.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]),
          "=r"(r[7]), "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]),
          "=r"(r[14]), "=r"(r[15]), "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]),
          "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]), "=r"(r[25]),
          "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() {
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// Packed pairs of f32: one instruction per two IEEE round-to-nearest results (each half is
// bit-identical to the scalar add.rn / mul.rn / fma.rn). The rounding mode is spelled out: without
// it the assembler may merge a multiplication with a following addition into one fused operation.
// Even so, do not feed mul2 straight into add2 where the two roundings matter: that pair was
// observed to behave as one fused multiply-add; write fma2(mul2(a, b), one, c) instead.
__device__ __forceinline__ float2 add2(float2 a, float2 b) {
    float2 c;
    asm("add.rn.f32x2 %0, %1, %2;"
        : "=l"(reinterpret_cast<uint64_t &>(c))
        : "l"(reinterpret_cast<const uint64_t &>(a)), "l"(reinterpret_cast<const uint64_t &>(b)));
    return c;
}
__device__ __forceinline__ float2 mul2(float2 a, float2 b) {
    float2 c;
    asm("mul.rn.f32x2 %0, %1, %2;"
        : "=l"(reinterpret_cast<uint64_t &>(c))
        : "l"(reinterpret_cast<const uint64_t &>(a)), "l"(reinterpret_cast<const uint64_t &>(b)));
    return c;
}
__device__ __forceinline__ float2 fma2(float2 a, float2 b, float2 c) {
    float2 d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;"
        : "=l"(reinterpret_cast<uint64_t &>(d))
        : "l"(reinterpret_cast<const uint64_t &>(a)), "l"(reinterpret_cast<const uint64_t &>(b)),
          "l"(reinterpret_cast<const uint64_t &>(c)));
    return d;
}

// Byte offset of 16-byte chunk `chunk16` of row `row` inside a tile of 128-byte rows stored in
// the 128-byte swizzle (the layout TMA reads for a store and writes for a load).
__device__ __forceinline__ uint32_t sw128_offset(uint32_t row, uint32_t chunk16) {
    return row * 128u + ((chunk16 ^ (row & 7u)) << 4);
}

}  // namespace fluke_sm100
