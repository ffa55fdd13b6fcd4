// lstm_cluster_sm100.cu -- the recurrence of a factored-LSTM layer with one thread-block
// CLUSTER per 128-chunk row tile; hidden state and its projection travel between the CTAs of
// the cluster through distributed shared memory and never touch L2.
//
// A cluster is H/64 gate CTAs plus four projection CTAs (at most 12 + 4 = 16):
//
//   gate CTA     64 hidden units. Its four gate weight blocks [4*64, 2R] f16 stay in shared
//                memory, the cell state of its units in registers. Per step: TMA-load the
//                x_down tile and issue that half of the contraction at once; when the four
//                projection CTAs have delivered hh_down (four 128 x 32 f16 blocks, pushed
//                straight into this CTA's operand buffer) issue the other half; gates, cell
//                update, int8 hidden slice; the slice goes to h_out[t] in global memory and, as
//                one contiguous 8 KB block, into the operand buffers of the four projection CTAs.
//   projection   32 of the R = 128 down-projection columns; its int8 weight rows stay in shared
//   CTA          memory. Per step: as the gate CTAs' slices arrive (each is one 64-byte K block
//                of the operand), tcgen05 kind::i8 contraction over H, scale, round to f16 (as
//                the two-kernel form does) and push the 128 x 32 block to every gate CTA.
//
// The pushes are bulk asynchronous copies (shared::cta -> shared::cluster) that complete on an
// mbarrier of the receiving CTA, like a TMA load: the receiver arms the barrier with the byte
// count, waits (bounded) and feeds the data to tcgen05.mma without touching it. Operand blocks
// that are exchanged use 64-byte rows in the 64-byte swizzle so that one sender's part is one
// contiguous block of the receiver's operand.
//
// A buffer is only overwritten after its reader has provably finished: a gate CTA sends h_t only
// after it has received all of hh_t, which every projection CTA sends only after its contraction
// over h_{t-1} has completed, and vice versa. No CTA leaves before all have reached the final
// cluster barrier.
//
// Arithmetic is that of lstm_step_kernel and of the dequant GEMM epilogue, with the same two
// deviations as the L2-exchange kernel (x_down half accumulated first, fast tanh).
#include <fluke/fluke.h>

#include "fluke_sm100.h"
#include "sm100_ptx.cuh"
#include "tma_host.cuh"

#include <cuda_fp16.h>

namespace fluke_sm100 {
namespace {

constexpr int kCThreads = 576;     // warp 0 loader, warp 1 MMA issuer, warps 2-17 epilogue
constexpr int kCEpiWarps = 16;     // gate CTA: four per TMEM lane quadrant, 16 units each
constexpr int kCUnits = 64;        // hidden units per gate CTA
constexpr int kCWorkers = 4;       // projection CTAs per tile
constexpr int kCWorkerCols = 32;   // projection columns each of them owns
constexpr int kCRank = 128;        // factor rank the kernel is built for
constexpr int kCMaxSlices = 12;    // H <= 768
constexpr int kCTmemCols = 256;

struct ClusterDev {
    int T, B, H;
    int b_stride;              // chunks per timestep plane of h_out (the full batch)
    int reverse;
    int n_slices;              // H / 64 = gate CTAs per cluster
    const float *bias;         // [4H]
    const float *dn_scale;     // [R]
    float *c;                  // [B,H]
    int8_t *h_out;             // [T,B,H]
    long long *trace;          // trace builds only: [T][8] nanosecond stamps of tile 0's first gate and projection CTA
};

struct ClusterSmem {
    // gate role
    static constexpr int kWKB = 4 * kCUnits * 128;            // one 128-byte K block of the four gate slices
    static constexpr int kOffW = 0;                            // 4 K blocks: 0,1 hh half; 2,3 x half
    static constexpr int kOffAhh = 4 * kWKB;                   // 4 blocks [128 x 64 B], one per projection CTA
    static constexpr int kOffX = kOffAhh + 4 * 8192;           // 2 K blocks [128 x 128 B]
    static constexpr int kOffHs = kOffX + 2 * 16384;           // outgoing h slice [128 x 64 B]
    static constexpr int kOffBias = kOffHs + 8192;             // 4 x 64 floats
    static constexpr int kGateBytes = kOffBias + 4 * kCUnits * 4;
    // projection role
    static constexpr int kDnKB = kCWorkerCols * 128;           // 32 weight rows x 128 B
    static constexpr int kOffDn = 0;                           // up to 6 K blocks of 128 B
    static constexpr int kOffH = 24576;                        // up to 12 blocks [128 x 64 B], one per gate CTA
    static constexpr int kOffOut = kOffH + kCMaxSlices * 8192; // outgoing hh block [128 x 64 B]
    static constexpr int kWorkerBytes = kOffOut + 8192;
    static constexpr int kData = kGateBytes > kWorkerBytes ? kGateBytes : kWorkerBytes;
    static constexpr int kOffBars = (kData + 15) / 16 * 16;
    // barriers, at the same offsets in every CTA so that a peer's barrier is this CTA's address
    // mapped to the peer's rank
    static constexpr int kBarOnce = 0, kBarAccFull = 1, kBarAccEmpty = 2, kBarX = 3, kBarEpi = 4,
                         kBarAhh = 5 /* [4] */, kBarH = 9 /* [12] */, kNumBars = 21;
    static constexpr int kOffMisc = kOffBars + kNumBars * 8;
    static constexpr int kDynamic = kOffMisc + 16 + 1024;
    static_assert(kDynamic <= 232448, "shared memory budget of one CTA exceeded");
};

// Byte offset of 16-byte chunk `chunk16` (0..3) of row `row` in a tile of 64-byte rows stored in
// the 64-byte swizzle (tile base aligned to 512 bytes).
__device__ __forceinline__ uint32_t sw64_offset(uint32_t row, uint32_t chunk16) {
    return row * 64u + ((chunk16 ^ ((row >> 1) & 3u)) << 4);
}

// Shared-memory matrix descriptor of a K-major tile of 64-byte rows in the 64-byte swizzle:
// groups of 8 rows are 512 bytes apart.
__device__ __forceinline__ uint64_t make_smem_desc_sw64(uint32_t byte_addr) {
    uint64_t d = 0;
    d |= uint64_t((byte_addr & 0x3FFFFu) >> 4);
    d |= uint64_t(1) << 16;
    d |= uint64_t(512 >> 4) << 32;
    d |= uint64_t(1) << 46;
    d |= uint64_t(4) << 61;  // layout: 64-byte swizzle
    return d;
}

__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// The address, in the cluster's shared window, of this CTA's shared address `local` in CTA `rank`.
__device__ __forceinline__ uint32_t map_to_rank(uint32_t local, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(local), "r"(rank));
    return r;
}
// Asynchronous copy of `bytes` (multiple of 16) from this CTA's shared memory into a peer's;
// completes `bytes` of the transaction count of the peer's mbarrier.
__device__ __forceinline__ void push_to_peer(uint32_t dst_cluster, const void *src, uint32_t bytes,
                                             uint32_t bar_cluster) {
    asm volatile(
        "cp.async.bulk.shared::cluster.shared::cta.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
        ::"r"(dst_cluster), "r"(smem_u32(src)), "r"(bytes), "r"(bar_cluster)
        : "memory");
}
__device__ __forceinline__ long long global_ns() {
    long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;" ::: "memory");
    asm volatile("barrier.cluster.wait.acquire.aligned;" ::: "memory");
}

__global__ void __launch_bounds__(kCThreads, 1)
lstm_cluster_kernel(const __grid_constant__ CUtensorMap tm_w0, const __grid_constant__ CUtensorMap tm_w1,
                    const __grid_constant__ CUtensorMap tm_w2, const __grid_constant__ CUtensorMap tm_w3,
                    const __grid_constant__ CUtensorMap tm_x,    // x_down [T,B,R] f16, boxes 128 x 64
                    const __grid_constant__ CUtensorMap tm_dn,   // dn_hh  [R,H]   int8, boxes 32 x 128
                    const __grid_constant__ CUtensorMap tm_h0,   // h_0    [1,B,H] int8, boxes 128 x 64, 64-byte swizzle
                    const ClusterDev p) {
    using L = ClusterSmem;
    extern __shared__ uint8_t smem_raw[];
    // every CTA of the cluster computes the same offset, so peers' buffers are at the same
    // shared-window offsets as this CTA's
    uint8_t *smem = reinterpret_cast<uint8_t *>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + L::kOffBars);
    uint64_t *bar_once = &bars[L::kBarOnce];           // resident weights loaded
    uint64_t *bar_acc_full = &bars[L::kBarAccFull];    // MMAs of the step finished
    uint64_t *bar_acc_empty = &bars[L::kBarAccEmpty];  // epilogue finished reading the accumulator
    uint64_t *bar_x = &bars[L::kBarX];                 // gate: x_down tile landed
    uint64_t *bar_epi = &bars[L::kBarEpi];             // epilogue warps have staged their part
    uint64_t *bar_ahh = &bars[L::kBarAhh];             // gate [4]: hh_down block of projection CTA j landed
    uint64_t *bar_h = &bars[L::kBarH];                 // projection [12]: h slice of gate CTA j landed
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + L::kOffMisc);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + L::kOffMisc + 4);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int cluster_size = p.n_slices + kCWorkers;
    const int rank = int(cluster_ctarank());
    const int tile = blockIdx.x / cluster_size;
    const bool is_gate = rank < p.n_slices;
    const int m0 = tile * 128;

    if (threadIdx.x == 0) {
        mbar_init(bar_once, 1);
        mbar_init(bar_acc_full, 1);
        mbar_init(bar_acc_empty, is_gate ? kCEpiWarps : 4);
        mbar_init(bar_x, 1);
        mbar_init(bar_epi, is_gate ? kCEpiWarps : 4);
        for (int j = 0; j < 4; ++j) mbar_init(&bar_ahh[j], 1);
        for (int j = 0; j < kCMaxSlices; ++j) mbar_init(&bar_h[j], 1);
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 1) tmem_alloc(tmem_slot, kCTmemCols);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    // every barrier of the cluster is initialised before any CTA may push to a peer
    cluster_sync_all();
    const uint32_t tmem_base = *tmem_slot;

    auto time_of = [&](int i) { return p.reverse ? p.T - 1 - i : i; };

    if (is_gate) {
        const int n0 = rank * kCUnits;
        if (warp == 0) {
            // ------------------------------ gate: loader (one thread) -------------------
            if (elect_one()) {
                mbar_arrive_expect_tx(bar_once, 4 * L::kWKB);
                for (int kb = 0; kb < 4; ++kb) {
                    uint8_t *sw = smem + L::kOffW + kb * L::kWKB;
                    tma_load_2d(sw + 0 * kCUnits * 128, &tm_w0, bar_once, kb * 64, n0);
                    tma_load_2d(sw + 1 * kCUnits * 128, &tm_w1, bar_once, kb * 64, n0);
                    tma_load_2d(sw + 2 * kCUnits * 128, &tm_w2, bar_once, kb * 64, n0);
                    tma_load_2d(sw + 3 * kCUnits * 128, &tm_w3, bar_once, kb * 64, n0);
                }
                bool ok = true;
                for (int i = 0; i < p.T && ok; ++i) {
                    // MMAs of the previous step are done: the x buffer is free
                    if (i > 0) ok = mbar_wait(bar_acc_full, (i - 1) & 1, abort_flag, 70);
                    if (!ok) break;
                    uint8_t *sx = smem + L::kOffX;
                    mbar_arrive_expect_tx(bar_x, 32768);
                    tma_load_3d(sx, &tm_x, bar_x, 0, m0, time_of(i));
                    tma_load_3d(sx + 16384, &tm_x, bar_x, 64, m0, time_of(i));
                }
            }
            __syncwarp();
        } else if (warp == 1) {
            // ------------------------------ gate: MMA issuer (one thread) ---------------
            if (elect_one()) {
                constexpr uint32_t kIdesc = make_idesc<kKindF16>(128, 4 * kCUnits);
                for (int j = 0; j < kCWorkers; ++j) mbar_arrive_expect_tx(&bar_ahh[j], 8192);
                bool ok = mbar_wait(bar_once, 0, abort_flag, 71);
                for (int i = 0; i < p.T && ok; ++i) {
                    if (i > 0) ok = mbar_wait(bar_acc_empty, (i - 1) & 1, abort_flag, 72);
                    if (!ok) break;
                    ok = mbar_wait(bar_x, i & 1, abort_flag, 73);
                    if (!ok) break;
                    tc_fence_after_sync();
                    for (int kb = 0; kb < 2; ++kb) {  // x_down half: W K blocks 2, 3
                        const uint64_t ad = make_smem_desc_sw128(smem_u32(smem + L::kOffX + kb * 16384));
                        const uint64_t bd = make_smem_desc_sw128(smem_u32(smem + L::kOffW + (2 + kb) * L::kWKB));
#pragma unroll
                        for (int k = 0; k < 4; ++k)
                            tc_mma<kKindF16>(tmem_base, ad + uint64_t(2 * k), bd + uint64_t(2 * k), kIdesc,
                                             (kb | k) != 0 ? 1u : 0u);
                    }
                    for (int j = 0; j < kCWorkers && ok; ++j) {  // hh_down half, block j = columns 32j..32j+31
                        ok = mbar_wait(&bar_ahh[j], i & 1, abort_flag, 74);
                        if (!ok) break;
                        if (i + 1 < p.T) mbar_arrive_expect_tx(&bar_ahh[j], 8192);  // arm the next step
                        tc_fence_after_sync();
                        const uint64_t ad = make_smem_desc_sw64(smem_u32(smem + L::kOffAhh + j * 8192));
                        const uint64_t bd = make_smem_desc_sw128(smem_u32(smem + L::kOffW + (j >> 1) * L::kWKB)) +
                                            uint64_t((j & 1) * 4);
#pragma unroll
                        for (int k = 0; k < 2; ++k)
                            tc_mma<kKindF16>(tmem_base, ad + uint64_t(2 * k), bd + uint64_t(2 * k), kIdesc, 1u);
                    }
                    if (ok) tc_commit(bar_acc_full);
                    FLUKE_STAMP(blockIdx.x == 0, i * 8 + 0, global_ns());
                }
            }
            __syncwarp();
        } else {
            // ------------------------------ gate: epilogue ------------------------------
            const int e = warp - 2;
            const int q = warp & 3;   // TMEM lane quadrant of this warp
            const int ug = e >> 2;    // which 16 of the CTA's 64 units
            float *sbias = reinterpret_cast<float *>(smem + L::kOffBias);
            for (int j = threadIdx.x - 64; j < 4 * kCUnits; j += kCEpiWarps * 32)
                sbias[j] = __ldg(p.bias + (j / kCUnits) * p.H + n0 + (j % kCUnits));
            bool ok = warps_barrier(bar_epi, 0, lane, abort_flag);  // biases staged
            const int row = m0 + q * 32 + lane;
            const bool row_ok = row < p.B;
            float2 c2[8];  // the cell state of the thread's 16 units, as pairs of adjacent units
            if (row_ok) {
#pragma unroll
                for (int v = 0; v < 4; ++v) {
                    const float4 c4 = *reinterpret_cast<const float4 *>(p.c + int64_t(row) * p.H + n0 + ug * 16 + 4 * v);
                    c2[2 * v] = make_float2(c4.x, c4.y);
                    c2[2 * v + 1] = make_float2(c4.z, c4.w);
                }
            } else {
#pragma unroll
                for (int v = 0; v < 8; ++v) c2[v] = make_float2(0.f, 0.f);
            }
            const uint32_t t_row = tmem_base + (uint32_t(q * 32) << 16) + ug * 16;
            uint8_t *shs = smem + L::kOffHs;
            for (int i = 0; i < p.T && ok; ++i) {
                ok = mbar_wait(bar_acc_full, i & 1, abort_flag, 75);
                if (!ok) break;
                FLUKE_STAMP(blockIdx.x == 0 && threadIdx.x == 64, i * 8 + 1, global_ns());
                tc_fence_after_sync();
                uint32_t packed[4] = {0u, 0u, 0u, 0u};
#pragma unroll
                for (int half = 0; half < 2; ++half) {  // 8 units at a time keeps the register count down
                    uint32_t gi[8], gf[8], gg[8], go[8];
                    tmem_ld_32x8(t_row + 0 * kCUnits + half * 8, gi);
                    tmem_ld_32x8(t_row + 1 * kCUnits + half * 8, gf);
                    tmem_ld_32x8(t_row + 2 * kCUnits + half * 8, gg);
                    tmem_ld_32x8(t_row + 3 * kCUnits + half * 8, go);
                    tmem_ld_wait();
                    if (half == 1) {
                        // all TMEM reads of this step are done: the next step's MMAs may overwrite
                        tc_fence_before_sync();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(bar_acc_empty);
                    }
#pragma unroll
                    for (int v = 0; v < 2; ++v) {
                        const int u = ug * 16 + half * 8 + 4 * v;
                        const float4 bi = *reinterpret_cast<const float4 *>(sbias + 0 * kCUnits + u);
                        const float4 bf = *reinterpret_cast<const float4 *>(sbias + 1 * kCUnits + u);
                        const float4 bg = *reinterpret_cast<const float4 *>(sbias + 2 * kCUnits + u);
                        const float4 bo = *reinterpret_cast<const float4 *>(sbias + 3 * kCUnits + u);
                        const int x = 4 * v, cp = half * 4 + 2 * v;
                        const uint32_t lo = lstm_cell_pair(gi[x], gi[x + 1], gf[x], gf[x + 1], gg[x], gg[x + 1], go[x], go[x + 1],
                                                           make_float2(bi.x, bi.y), make_float2(bf.x, bf.y),
                                                           make_float2(bg.x, bg.y), make_float2(bo.x, bo.y), c2[cp]);
                        const uint32_t hi = lstm_cell_pair(gi[x + 2], gi[x + 3], gf[x + 2], gf[x + 3], gg[x + 2], gg[x + 3],
                                                           go[x + 2], go[x + 3], make_float2(bi.z, bi.w), make_float2(bf.z, bf.w),
                                                           make_float2(bg.z, bg.w), make_float2(bo.z, bo.w), c2[cp + 1]);
                        packed[half * 2 + v] = lo | (hi << 16);
                    }
                }
                const uint4 hv = make_uint4(packed[0], packed[1], packed[2], packed[3]);
                if (i + 1 < p.T) {
                    // the slice of h_t, as the projection CTAs' operand block (64-byte swizzle)
                    *reinterpret_cast<uint4 *>(shs + sw64_offset(q * 32 + lane, ug)) = hv;
                    fence_proxy_async_smem();
                    ok = warps_barrier(bar_epi, (i + 1) & 1, lane, abort_flag);
                    if (ok && e == 0 && lane == 0) {
                        FLUKE_STAMP(blockIdx.x == 0, i * 8 + 2, global_ns());
                        const uint32_t dst = smem_u32(smem + L::kOffH + rank * 8192);
                        const uint32_t bar = smem_u32(&bar_h[rank]);
                        for (int wk = 0; wk < kCWorkers; ++wk)
                            push_to_peer(map_to_rank(dst, p.n_slices + wk), shs, 8192,
                                         map_to_rank(bar, p.n_slices + wk));
                        FLUKE_STAMP(blockIdx.x == 0, i * 8 + 3, global_ns());
                    }
                }
                if (row_ok)
                    *reinterpret_cast<uint4 *>(p.h_out + (int64_t(time_of(i)) * p.b_stride + row) * p.H + n0 + ug * 16) = hv;
            }
            if (row_ok) {
#pragma unroll
                for (int v = 0; v < 4; ++v)
                    *reinterpret_cast<float4 *>(p.c + int64_t(row) * p.H + n0 + ug * 16 + 4 * v) =
                        make_float4(c2[2 * v].x, c2[2 * v].y, c2[2 * v + 1].x, c2[2 * v + 1].y);
            }
        }
    } else {
        const int widx = rank - p.n_slices;       // which projection CTA of the tile
        const int r0 = widx * kCWorkerCols;       // its projection columns
        const int nkb_dn = (p.H + 127) / 128;
        if (warp == 0) {
            // ------------------------------ projection: loader (one thread) -------------
            if (elect_one()) {
                mbar_arrive_expect_tx(bar_once, nkb_dn * L::kDnKB);
                for (int kb = 0; kb < nkb_dn; ++kb)
                    tma_load_2d(smem + L::kOffDn + kb * L::kDnKB, &tm_dn, bar_once, kb * 128, r0);
                // step 0 projects the layer's initial hidden state, fetched from global memory
                for (int j = 0; j < p.n_slices; ++j) {
                    mbar_arrive_expect_tx(&bar_h[j], 8192);
                    tma_load_3d(smem + L::kOffH + j * 8192, &tm_h0, &bar_h[j], j * 64, m0, 0);
                }
            }
            __syncwarp();
        } else if (warp == 1) {
            // ------------------------------ projection: MMA issuer (one thread) ---------
            if (elect_one()) {
                constexpr uint32_t kIdesc = make_idesc<kKindI8>(128, kCWorkerCols);
                bool ok = mbar_wait(bar_once, 0, abort_flag, 80);
                for (int i = 0; i < p.T && ok; ++i) {
                    if (i > 0) ok = mbar_wait(bar_acc_empty, (i - 1) & 1, abort_flag, 81);
                    for (int j = 0; j < p.n_slices && ok; ++j) {
                        ok = mbar_wait(&bar_h[j], i & 1, abort_flag, 82);
                        if (!ok) break;
                        if (i + 1 < p.T) mbar_arrive_expect_tx(&bar_h[j], 8192);  // arm the next step
                        tc_fence_after_sync();
                        const uint64_t ad = make_smem_desc_sw64(smem_u32(smem + L::kOffH + j * 8192));
                        const uint64_t bd = make_smem_desc_sw128(smem_u32(smem + L::kOffDn + (j >> 1) * L::kDnKB)) +
                                            uint64_t((j & 1) * 4);
#pragma unroll
                        for (int k = 0; k < 2; ++k)
                            tc_mma<kKindI8>(tmem_base, ad + uint64_t(2 * k), bd + uint64_t(2 * k), kIdesc,
                                            (j | k) != 0 ? 1u : 0u);
                    }
                    if (ok) tc_commit(bar_acc_full);
                    FLUKE_STAMP(int(blockIdx.x) == p.n_slices, i * 8 + 4, global_ns());
                }
            }
            __syncwarp();
        } else if (warp < 6) {
            // ------------------------------ projection: epilogue (four warps) -----------
            const int q = warp & 3;
            float sc[32];
#pragma unroll
            for (int v = 0; v < 8; ++v) {
                const float4 s4 = __ldg(reinterpret_cast<const float4 *>(p.dn_scale + r0) + v);
                // same operand order as the dequant GEMM epilogue: sa * sb
                sc[4 * v] = (1.0f / 127.0f) * s4.x; sc[4 * v + 1] = (1.0f / 127.0f) * s4.y;
                sc[4 * v + 2] = (1.0f / 127.0f) * s4.z; sc[4 * v + 3] = (1.0f / 127.0f) * s4.w;
            }
            const uint32_t t_row = tmem_base + (uint32_t(q * 32) << 16);
            uint8_t *sout = smem + L::kOffOut;
            bool ok = true;
            for (int i = 0; i < p.T && ok; ++i) {
                ok = mbar_wait(bar_acc_full, i & 1, abort_flag, 83);
                if (!ok) break;
                FLUKE_STAMP(int(blockIdx.x) == p.n_slices && threadIdx.x == 64, i * 8 + 5, global_ns());
                tc_fence_after_sync();
                uint32_t acc[32];
                tmem_ld_32x32(t_row, acc);
                tmem_ld_wait();
                tc_fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar_acc_empty);
#pragma unroll
                for (int v = 0; v < 4; ++v) {
                    uint32_t w[4];
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        const int x = 8 * v + 2 * j;
                        const __half2 h2 = __floats2half2_rn(float(int(acc[x])) * sc[x],
                                                             float(int(acc[x + 1])) * sc[x + 1]);
                        w[j] = *reinterpret_cast<const uint32_t *>(&h2);
                    }
                    // the gate CTAs' operand block (64-byte swizzle): 8 columns per 16-byte chunk
                    *reinterpret_cast<uint4 *>(sout + sw64_offset(q * 32 + lane, v)) = make_uint4(w[0], w[1], w[2], w[3]);
                }
                fence_proxy_async_smem();
                ok = warps_barrier(bar_epi, i & 1, lane, abort_flag);
                if (ok && warp == 2 && lane == 0) {
                    FLUKE_STAMP(int(blockIdx.x) == p.n_slices, i * 8 + 6, global_ns());
                    const uint32_t dst = smem_u32(smem + L::kOffAhh + widx * 8192);
                    const uint32_t bar = smem_u32(&bar_ahh[widx]);
                    for (int s = 0; s < p.n_slices; ++s)
                        push_to_peer(map_to_rank(dst, s), sout, 8192, map_to_rank(bar, s));
                    FLUKE_STAMP(int(blockIdx.x) == p.n_slices, i * 8 + 7, global_ns());
                }
            }
        }
    }

    // Nobody leaves (and frees shared memory that a peer's copy may still target or read) before
    // every CTA of the cluster is done.
    tc_fence_before_sync();
    __syncthreads();
    cluster_sync_all();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, kCTmemCols);
    }
}

// ---- host side ---------------------------------------------------------------------------------

// Number of clusters of `cluster_size` CTAs of the kernel that the device can hold at once
// (0: none, the kernel cannot be used).
int cluster_capacity(int cluster_size) {
    static int ready[64][17];  // per device and size: 0 unknown, n + 1 known, -1 none
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64 || cluster_size < 1 || cluster_size > 16) return -1;
    if (ready[dev][cluster_size] == 0) {
        int ok = 1, n_clusters = 0;
        if (cudaFuncSetAttribute(lstm_cluster_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 ClusterSmem::kDynamic) != cudaSuccess)
            ok = -1;
        if (ok == 1 && cudaFuncSetAttribute(lstm_cluster_kernel, cudaFuncAttributeNonPortableClusterSizeAllowed,
                                            1) != cudaSuccess)
            ok = -1;
        if (ok == 1) {
            cudaLaunchConfig_t cfg = {};
            cfg.gridDim = dim3(cluster_size);
            cfg.blockDim = dim3(kCThreads);
            cfg.dynamicSmemBytes = ClusterSmem::kDynamic;
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeClusterDimension;
            attr[0].val.clusterDim.x = cluster_size;
            attr[0].val.clusterDim.y = 1;
            attr[0].val.clusterDim.z = 1;
            cfg.attrs = attr;
            cfg.numAttrs = 1;
            if (cudaOccupancyMaxActiveClusters(&n_clusters, lstm_cluster_kernel, &cfg) != cudaSuccess || n_clusters < 1)
                ok = -1;
        }
        cudaGetLastError();  // a refused attribute must not linger as the thread's last error
        ready[dev][cluster_size] = ok == 1 ? n_clusters + 1 : -1;
    }
    return ready[dev][cluster_size] > 0 ? ready[dev][cluster_size] - 1 : 0;
}

}  // namespace
}  // namespace fluke_sm100

// How many row tiles (clusters) of a layer with hidden size H run at the same time; 0 when the
// cluster form is not available for H on this device.
extern "C" int fluke_sm100_lstm_cluster_capacity(int H) {
    using namespace fluke_sm100;
    if (H < 0) return cluster_capacity(-H);  // probe: capacity for a cluster size given directly
    if (H <= 0 || H % kCUnits || H / kCUnits > kCMaxSlices) return 0;
    return cluster_capacity(H / kCUnits + kCWorkers);
}

// Runs the recurrence of one layer (x_down already computed) with one cluster per row tile.
// Returns -2 when the shape or the device is not covered, or when the layer has more row tiles
// than clusters fit on the device at once and `allow_waves` is 0 (the tiles would run in several
// rounds; the caller may prefer another form).
extern "C" int fluke_sm100_lstm_layer_cluster(const void *layer, const void *x_down_, int allow_waves,
                                              void *stream_) {
    using namespace fluke_sm100;
    const fluke_flstm_layer_t *l = static_cast<const fluke_flstm_layer_t *>(layer);
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (l->R != kCRank || l->H % kCUnits || l->H / kCUnits > kCMaxSlices) return -2;
    const int T = l->T, B = l->B, H = l->H, R = l->R;
    const int n_slices = H / kCUnits, cluster_size = n_slices + kCWorkers;
    const int capacity = cluster_capacity(cluster_size);
    if (capacity < 1) return -2;
    if (!allow_waves && (B + 127) / 128 > capacity) return -2;
    const __half *x_down = static_cast<const __half *>(x_down_);

    ClusterDev p;
    p.T = T; p.B = B; p.H = H; p.b_stride = B; p.reverse = l->reverse; p.n_slices = n_slices;
    p.bias = static_cast<const float *>(l->bias_f32);
    p.dn_scale = static_cast<const float *>(l->dn_hh_scale);
    p.c = static_cast<float *>(l->c_f32);
    p.h_out = static_cast<int8_t *>(l->h_out_i8);
    p.trace = trace_buffer();

    CUtensorMap tm_w[4], tm_x, tm_dn, tm_h0;
    int rc;
    for (int g = 0; g < 4; ++g) {
        const __half *w = static_cast<const __half *>(l->w_up_f16) + size_t(g) * H * 2 * R;
        rc = make_tmap_2d(&tm_w[g], CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, w, H, 2 * R, uint64_t(2 * R) * 2, kCUnits, 64, true);
        if (rc) return rc;
    }
    rc = make_tmap_3d(&tm_x, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, x_down, T, B, R, uint64_t(R) * 2,
                      uint64_t(B) * R * 2, 128, 64, true);
    if (rc) return rc;
    rc = make_tmap_2d(&tm_dn, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, l->dn_hh_i8, R, H, H, kCWorkerCols, 128, true);
    if (rc) return rc;
    rc = make_tmap_3d_sw(&tm_h0, CU_TENSOR_MAP_DATA_TYPE_UINT8, l->h_i8, 1, B, H, H, uint64_t(B) * H, 128, 64,
                         CU_TENSOR_MAP_SWIZZLE_64B);
    if (rc) return rc;

    const int n_tiles = (B + 127) / 128;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(n_tiles * cluster_size);
    cfg.blockDim = dim3(kCThreads);
    cfg.dynamicSmemBytes = ClusterSmem::kDynamic;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = cluster_size;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return (int)cudaLaunchKernelEx(&cfg, lstm_cluster_kernel, tm_w[0], tm_w[1], tm_w[2], tm_w[3], tm_x, tm_dn,
                                   tm_h0, p);
}
