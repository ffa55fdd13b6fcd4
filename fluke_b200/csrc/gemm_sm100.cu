// gemm_sm100.cu -- the tcgen05 GEMM family of the quantized transformer path on sm_100a.
//
// One persistent, warp-specialised, WEIGHT-STATIONARY kernel template computes
// out = epilogue(A @ B^T) for K-major 8-bit operands (int8 -> int32 via kind::i8,
// e4m3 -> f32 via kind::f8f6f4). A CTA owns one N tile of the weight for its whole life: the
// tile (all of K, up to 128 KB) is TMA-loaded into shared memory once, and the CTA then streams
// the M tiles assigned to it, so per output tile only the 128 x K activation block crosses
// L2 -> SM (the activations are what is large; the weights of this path are at most 2 MB).
//
// 384 threads in three warpgroups; after set-up the first gives most of its registers to the
// other two (setmaxnreg):
//
//   warp 0      TMA producer (one thread): the resident weight tile once, then
//               128-byte-swizzled 128 x 128-byte A blocks into a ring of four stages; it also
//               pulls the A tile three steps ahead into L2
//   warp 1      MMA issuer (one thread): tcgen05.mma 128 x BN x 32B from shared-memory
//               descriptors into one of two accumulator buffers in tensor memory
//   warps 2-3   idle
//   warps 4-11  epilogue: two warps per TMEM lane quadrant, each owning half of the tile's
//               columns: tcgen05.ld, dequant / rotary / SiLU in packed f32x2 arithmetic, f16
//               pack, swizzled smem staging, TMA tile store
//
// The two accumulator buffers let the epilogue of tile i overlap the MMAs of tile i+1; no
// accumulator or f16 intermediate ever reaches HBM. Per-column and per-position factors live in
// registers wherever the data layout allows it: the SiLU and dequant epilogues read tensor
// memory in the 16-lane x 256-bit shape, in which a thread keeps the same 16 columns for the
// whole kernel (their weight scales are loaded once); the rotary epilogue keeps thread = row
// and, with tiles aligned to the sequences, holds the row's sin/cos values across tiles.
// It replaces TensorOpGemmI8 (cute/ampere/gemm/gemm_i8_quant.py:344-757), TensorOpGemmI8Rotary
// (cute/ampere/rotary/gemm_i8_rotary.py:151-472) and TensorOpDualGemmI8Silu
// (cute/ampere/dual_gemm_silu/dual_gemm_i8_silu.py:150-523) of the reference, and follows
// their epilogue arithmetic: acc*(sa*sb) for the base GEMM (:617,:750), (acc*sa)*sb for the
// rotary (:411-435) and SiLU (:478-487) kernels.
#include "fluke_sm100.h"
#include "sm100_ptx.cuh"
#include "tma_host.cuh"

#include <cuda_fp16.h>

namespace fluke_sm100 {

namespace {

constexpr int kBlockM = 128;          // rows per tile = TMEM lanes
constexpr int kBlockKBytes = 128;     // K bytes per TMA box = one swizzle row
constexpr int kUmmaKBytes = 32;       // K bytes per tcgen05.mma
constexpr int kPrefetchTiles = 3;     // how many tiles ahead the activations are pulled into L2
constexpr int kNumThreads = 384;       // three warpgroups: {TMA, MMA, 2 idle warps}, 2 x epilogue
constexpr int kEpilogueWarp0 = 4;
constexpr int kRegsLight = 64;         // registers per thread of warpgroup 0 after set-up
constexpr int kRegsEpilogue = 216;     // and of the two epilogue warpgroups
constexpr int kEpilogueWarps = 8;
constexpr int kStageRows = 32;        // rows per epilogue warp
constexpr int kStagingBytes = kStageRows * 128;
constexpr int kWeightBytes = 128 * 1024;  // resident weight tile: BN_MMA rows x K bytes

struct GemmDev {
    int M, N, K;
    int num_m_tiles, num_n_tiles, num_k_blocks;
    int ctas_per_n;          // CTAs that share one N tile (they split the M tiles)
    const float *scale_a;
    float const_scale_a;
    const float *scale_b;
    const float *scale_b2;
    const float *sin_tab;
    const float *cos_tab;
    int seqlen;
    int qk_cols;
    int a_plane;  // plane of the 3-D A tensor map this launch reads
    // ROTARY with whole sequences (M = n_seq * seqlen, seqlen >= 128): tiles are aligned to the
    // sequences (seq_tiles per sequence, the last one shifted up to end at the sequence end) and a
    // CTA takes a contiguous run of the list ordered by (tile-in-sequence, sequence), so the rows
    // of successive tiles keep their positions and their sin/cos values stay in registers.
    int seq_tiles;  // 0: plain tiling, tile t covers rows [128 t, 128 t + 128)
    int n_seq;
    int items_per_cta;
};

struct TrueTag { static constexpr bool value = true; };
struct FalseTag { static constexpr bool value = false; };

// The work list of a CTA: items w_begin, w_begin + w_step, ... < w_end; item -> first row.
struct TileIter {
    int w_begin, w_end, w_step;
    __device__ __forceinline__ TileIter(const GemmDev &p, int m_first) {
        if (p.seq_tiles > 0) {
            w_begin = m_first * p.items_per_cta;
            w_end = min(p.seq_tiles * p.n_seq, w_begin + p.items_per_cta);
            w_step = 1;
        } else {
            w_begin = m_first;
            w_end = p.num_m_tiles;
            w_step = p.ctas_per_n;
        }
    }
    // tile-in-sequence index (seq mode only)
    __device__ __forceinline__ static int seq_index(const GemmDev &p, int w) { return w / p.n_seq; }
    __device__ __forceinline__ static int seq_pos0(const GemmDev &p, int s) {
        return min(s * kBlockM, p.seqlen - kBlockM);
    }
    __device__ __forceinline__ static int row0(const GemmDev &p, int w) {
        if (p.seq_tiles > 0) {
            const int s = w / p.n_seq;
            return (w - s * p.n_seq) * p.seqlen + seq_pos0(p, s);
        }
        return w * kBlockM;
    }
};

template <int EPI, int BN_MMA, int STAGES>
struct SmemLayout {
    static constexpr int kMaxKBlocks = kWeightBytes / (BN_MMA * kBlockKBytes);  // 4 (BN 256) or 8 (BN 128)
    static constexpr int kABytes = kBlockM * kBlockKBytes;        // one K block of an A tile = one ring stage
    static constexpr int kBBytes = BN_MMA * kBlockKBytes;         // one K block of the weight tile
    static constexpr int kOffW = 0;
    static constexpr int kOffA = kWeightBytes;
    static constexpr int kOffStaging = kOffA + STAGES * kABytes;
    static constexpr int kOffBars = kOffStaging + kEpilogueWarps * kStagingBytes;
    static constexpr int kNumBars = 2 * STAGES + 5;
    static constexpr int kOffMisc = kOffBars + kNumBars * 8;
    static constexpr int kTotal = kOffMisc + 16;
    static constexpr int kDynamic = kTotal + 1024;  // slack for manual 1024-byte alignment
    static_assert(kDynamic <= 232448, "shared memory budget of one CTA exceeded");
};

__device__ __forceinline__ uint32_t pack_half2(float lo, float hi) {
    __half2 h = __floats2half2_rn(lo, hi);
    return *reinterpret_cast<uint32_t *>(&h);
}

__device__ __forceinline__ float tanh_approx(float x) {
    float y;
    asm("tanh.approx.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

template <int KIND>
__device__ __forceinline__ float acc_to_float(uint32_t bits) {
    if constexpr (KIND == kKindI8) return static_cast<float>(static_cast<int>(bits));
    else return __uint_as_float(bits);
}
template <int KIND>
__device__ __forceinline__ float2 acc_to_float2(uint32_t a, uint32_t b) {
    return make_float2(acc_to_float<KIND>(a), acc_to_float<KIND>(b));
}

// Four 8 x 8 matrices of 16-bit elements, each thread giving its fragment of every matrix (the
// two adjacent elements 2t, 2t+1 of row g) in one register: lane i supplies the shared-memory
// address of row i % 8 of matrix i / 8 (16 bytes per row).
__device__ __forceinline__ void stmatrix_x4(const void *row_addr, const uint32_t (&r)[4]) {
    asm volatile("stmatrix.sync.aligned.m8n8.x4.shared.b16 [%0], {%1, %2, %3, %4};"
                 ::"r"(smem_u32(row_addr)), "r"(r[0]), "r"(r[1]), "r"(r[2]), "r"(r[3])
                 : "memory");
}

// Writes one 128-byte row (8 x 16-byte chunks held in v[0..31]) into a swizzled staging tile.
__device__ __forceinline__ void stage_row(uint8_t *staging, uint32_t row, const uint32_t (&v)[32]) {
#pragma unroll
    for (uint32_t ch = 0; ch < 8; ++ch) {
        uint4 q = make_uint4(v[4 * ch], v[4 * ch + 1], v[4 * ch + 2], v[4 * ch + 3]);
        *reinterpret_cast<uint4 *>(staging + sw128_offset(row, ch)) = q;
    }
}

template <int KIND, int EPI, int BN_MMA, int STAGES>
__global__ void __launch_bounds__(kNumThreads, 1)
gemm_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b,
            const __grid_constant__ CUtensorMap tm_b2, const __grid_constant__ CUtensorMap tm_out,
            const GemmDev p) {
    using L = SmemLayout<EPI, BN_MMA, STAGES>;
    constexpr bool kDual = (EPI == FLUKE_SM100_EPI_SILU);
    constexpr int BN_OUT = kDual ? BN_MMA / 2 : BN_MMA;  // output columns per tile
    constexpr int kWarpCols = BN_OUT / 2;                // output columns per epilogue warp
    constexpr uint32_t kTmemCols = 2 * BN_MMA;  // two accumulator buffers (256 or 512)
    constexpr uint32_t kIdesc = make_idesc<KIND>(kBlockM, BN_MMA);

    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + L::kOffBars);
    uint64_t *full_bar = bars;
    uint64_t *empty_bar = bars + STAGES;
    uint64_t *tfull_bar = bars + 2 * STAGES;
    uint64_t *tempty_bar = bars + 2 * STAGES + 2;
    uint64_t *w_bar = bars + 2 * STAGES + 4;      // resident weight tile loaded
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + L::kOffMisc);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + L::kOffMisc + 4);

    const int warp = threadIdx.x >> 5;
    const int lane = threadIdx.x & 31;
    const int n_tile = blockIdx.x % p.num_n_tiles;
    const int m_first = blockIdx.x / p.num_n_tiles;
    const int n0 = n_tile * BN_OUT;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], 1);
        }
        for (int s = 0; s < 2; ++s) {
            mbar_init(&tfull_bar[s], 1);
            mbar_init(&tempty_bar[s], kEpilogueWarps);
        }
        mbar_init(w_bar, 1);
        *abort_flag = 0;
        fence_barrier_init();
        tma_prefetch_desc(&tm_a);
        tma_prefetch_desc(&tm_b);
        if (kDual) tma_prefetch_desc(&tm_b2);
        tma_prefetch_desc(&tm_out);
    }
    if (warp == 1) tmem_alloc(tmem_slot, kTmemCols);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    // The launch gives every thread 65536 / 384 registers; the loader and issuer need few, the
    // epilogue threads hold a whole row segment plus rotary tables: each role branch below
    // starts by resizing its warpgroup's share.

    if (warp < kEpilogueWarp0) reg_dealloc<kRegsLight>();
    if (warp == 0) {
        // ------------------------------ TMA producer (one thread) ------------------
        if (elect_one()) {
            mbar_arrive_expect_tx(w_bar, uint32_t(p.num_k_blocks) * L::kBBytes);
            for (int kb = 0; kb < p.num_k_blocks; ++kb) {
                uint8_t *sb = smem + L::kOffW + kb * L::kBBytes;
                if constexpr (kDual) {
                    tma_load_2d(sb, &tm_b, w_bar, kb * kBlockKBytes, n0);
                    tma_load_2d(sb + L::kBBytes / 2, &tm_b2, w_bar, kb * kBlockKBytes, n0);
                } else {
                    tma_load_2d(sb, &tm_b, w_bar, kb * kBlockKBytes, n0);
                }
            }
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            const TileIter it(p, m_first);
            // The CTAs that share an activation tile reach it at about the same time, so without
            // help every tile load would pay the HBM latency. One of them (chosen by the tile
            // index) asks for the tile kPrefetchTiles steps ahead to be brought into L2. With a
            // single N tile nothing is shared and the ring alone covers the latency.
            auto prefetch_tile = [&](int w) {
                if (p.num_n_tiles > 1 && w < it.w_end && (w % p.num_n_tiles) == n_tile) {
                    const int m0 = TileIter::row0(p, w);
                    for (int kb = 0; kb < p.num_k_blocks; ++kb)
                        tma_prefetch_l2_3d(&tm_a, kb * kBlockKBytes, m0, p.a_plane);
                }
            };
            for (int d = 0; d < kPrefetchTiles; ++d) prefetch_tile(it.w_begin + d * it.w_step);
            for (int w = it.w_begin; w < it.w_end && ok; w += it.w_step) {
                const int m0 = TileIter::row0(p, w);
                prefetch_tile(w + kPrefetchTiles * it.w_step);
                for (int kb = 0; kb < p.num_k_blocks; ++kb) {
                    ok = mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag, 1);
                    if (!ok) break;
                    mbar_arrive_expect_tx(&full_bar[stage], L::kABytes);
                    tma_load_3d(smem + L::kOffA + stage * L::kABytes, &tm_a, &full_bar[stage],
                                kb * kBlockKBytes, m0, p.a_plane);
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
            }
            if (!ok) {
                // Give loads that are still in flight a bounded chance to land before the CTA's
                // shared memory is released.
                const long long t0 = clock64();
                while (clock64() - t0 < (1ll << 22)) { }
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        // ------------------------------ MMA issuer (one thread) --------------------
        if (elect_one()) {
            int stage = 0;
            uint32_t phase = 0;
            int local = 0;
            bool ok = mbar_wait(w_bar, 0, abort_flag, 6);
            const TileIter it(p, m_first);
            for (int w = it.w_begin; w < it.w_end && ok; w += it.w_step, ++local) {
                const int acc = local & 1;
                const uint32_t acc_phase = (local >> 1) & 1;
                ok = mbar_wait(&tempty_bar[acc], acc_phase ^ 1u, abort_flag, 2);
                if (!ok) break;
                tc_fence_after_sync();
                const uint32_t d_tmem = tmem_base + acc * BN_MMA;
                for (int kb = 0; kb < p.num_k_blocks; ++kb) {
                    ok = mbar_wait(&full_bar[stage], phase, abort_flag, 3);
                    if (!ok) break;
                    tc_fence_after_sync();
                    const uint64_t adesc =
                        make_smem_desc_sw128(smem_u32(smem + L::kOffA + stage * L::kABytes));
                    const uint64_t bdesc =
                        make_smem_desc_sw128(smem_u32(smem + L::kOffW + kb * L::kBBytes));
#pragma unroll
                    for (int k = 0; k < kBlockKBytes / kUmmaKBytes; ++k) {
                        tc_mma<KIND>(d_tmem, adesc + uint64_t(k * (kUmmaKBytes >> 4)),
                                     bdesc + uint64_t(k * (kUmmaKBytes >> 4)), kIdesc,
                                     (kb | k) != 0 ? 1u : 0u);
                    }
                    tc_commit(&empty_bar[stage]);
                    if (kb == p.num_k_blocks - 1) tc_commit(&tfull_bar[acc]);
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
            }
        }
        __syncwarp();
    } else if (warp >= kEpilogueWarp0) {
        // ------------------------------ epilogue ----------------------------------
        // Accumulators leave tensor memory in the 16-lane x 256-bit shape: per load a thread
        // (g = lane / 4, t = lane % 4) receives, for each group j of 8 columns, the columns
        // 8j + 2t and 8j + 2t + 1 of rows g and g + 8 of the 16 addressed lanes. Two loads
        // (lane offsets 0 and 16) cover the warp's quadrant, so a thread works on four rows
        // (g + 8k) and on a quarter of the warp's columns. Those columns never change while the
        // CTA lives (it owns one N tile), which lets every per-column factor of the epilogue --
        // the weight scales, and with sequence-aligned tiling the rotary sin/cos values -- stay
        // in registers: the epilogue reads no table from shared memory.
        reg_alloc<kRegsEpilogue>();
        const int q = warp & 3;                           // TMEM lane quadrant this warp may read
        const int ch = (warp - kEpilogueWarp0) >> 2;      // which of the quadrant's two warps
        const int g8 = lane >> 2, t4 = lane & 3;
        uint8_t *staging = smem + L::kOffStaging + (warp - kEpilogueWarp0) * kStagingBytes;
        const TileIter it(p, m_first);
        int local = 0;
        bool ok = true;

        // row scales of the thread's four rows of the tile that starts at row m0
        auto load_sa = [&](int m0, float (&sa)[4]) {
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const int row = m0 + q * 32 + g8 + 8 * k;
                sa[k] = p.scale_a ? (row < p.M ? __ldg(p.scale_a + row) : 0.f) : p.const_scale_a;
            }
        };

        if constexpr (EPI == FLUKE_SM100_EPI_RAW) {
            // 32-bit accumulators, no scaling: thread = row, 32 columns per store
            for (int w = it.w_begin; w < it.w_end && ok; w += it.w_step, ++local) {
                const int m0 = TileIter::row0(p, w);
                const int acc = local & 1;
                const uint32_t acc_phase = (local >> 1) & 1;
                ok = mbar_wait(&tfull_bar[acc], acc_phase, abort_flag, 4);
                if (!ok) break;
                tc_fence_after_sync();
                const uint32_t t_row = tmem_base + (uint32_t(q * 32) << 16) + acc * BN_MMA;
                constexpr int kChunks = kWarpCols / 32;
#pragma unroll 1
                for (int chunk = 0; chunk < kChunks; ++chunk) {
                    const int c0 = ch * kWarpCols + chunk * 32;
                    const bool chunk_ok = n0 + c0 < p.N;
                    uint32_t outw[32];
                    if (chunk_ok) {
                        tmem_ld_32x32(t_row + c0, outw);
                        tmem_ld_wait();
                    }
                    if (chunk == kChunks - 1) {
                        tc_fence_before_sync();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&tempty_bar[acc]);
                    }
                    if (!chunk_ok) continue;
                    if (lane == 0) tma_store_wait_read<0>();
                    __syncwarp();
                    stage_row(staging, lane, outw);
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        tma_store_2d(&tm_out, staging, n0 + c0, m0 + q * 32);
                        tma_store_commit();
                    }
                }
            }
        } else if constexpr (EPI == FLUKE_SM100_EPI_ROTARY) {
            // A tile is four heads; warp `ch` owns heads 2*ch and 2*ch+1. Accumulators come in the
            // 16-lane x 256-bit layout: a thread holds columns 8j + 2t, +1 (j = 0..7) of a head for
            // rows g + 8k (k = 0..3) of its quadrant, so both halves of a rotation pair (columns i
            // and i + 32: j and j + 4) are its own, its 32 column scales never change (registers),
            // and it needs 16 sin and 16 cos pairs: rows g + 8k x pair indices 8j + 2t, +1 (j < 4).
            // Those stay in registers too: with sequence-aligned tiling they are loaded once per
            // run of tiles with the same tile-in-sequence index, otherwise at the start of every
            // tile. The epilogue reads nothing from shared memory; its outputs, which are 8 x 8
            // matrix fragments in this layout, go to the staging tile four matrices per
            // instruction (stmatrix).
            static_assert(BN_OUT == 256, "two heads per epilogue warp");
            const bool rotate = n0 < p.qk_cols;
            float2 sc[2][8];
#pragma unroll
            for (int h2 = 0; h2 < 2; ++h2)
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    sc[h2][j] = __ldg(reinterpret_cast<const float2 *>(p.scale_b + n0 + (2 * ch + h2) * 64 + 8 * j + 2 * t4));
            float2 sn2[4][4], cs2[4][4];  // [row k][pair group j]
            auto load_tables = [&](int k, int pos) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    sn2[k][j] = __ldg(reinterpret_cast<const float2 *>(p.sin_tab + pos * 32 + 8 * j + 2 * t4));
                    cs2[k][j] = __ldg(reinterpret_cast<const float2 *>(p.cos_tab + pos * 32 + 8 * j + 2 * t4));
                }
            };
            // stmatrix: lane i gives the address of row i % 8 of matrix i / 8
            const uint32_t st_row = lane & 7, st_mat = lane >> 3;
            const bool seq_mode = p.seq_tiles > 0;
            int cur_s = -1;
            float sa_next[4];
            if (it.w_begin < it.w_end) load_sa(TileIter::row0(p, it.w_begin), sa_next);
            for (int w = it.w_begin; w < it.w_end && ok; w += it.w_step, ++local) {
                const int m0 = TileIter::row0(p, w);
                const int acc = local & 1;
                const uint32_t acc_phase = (local >> 1) & 1;
                float2 sa2[4];
#pragma unroll
                for (int k = 0; k < 4; ++k) sa2[k] = make_float2(sa_next[k], sa_next[k]);
                if (w + it.w_step < it.w_end) load_sa(TileIter::row0(p, w + it.w_step), sa_next);
                if (rotate) {
                    if (seq_mode) {
                        // the positions only change when the tile-in-sequence index does
                        const int s_idx = TileIter::seq_index(p, w);
                        if (s_idx != cur_s) {
                            cur_s = s_idx;
#pragma unroll
                            for (int k = 0; k < 4; ++k) load_tables(k, TileIter::seq_pos0(p, s_idx) + q * 32 + g8 + 8 * k);
                        }
                    } else {
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            const int grow = m0 + q * 32 + g8 + 8 * k;
                            load_tables(k, grow < p.M ? grow % p.seqlen : 0);
                        }
                    }
                }

                ok = mbar_wait(&tfull_bar[acc], acc_phase, abort_flag, 4);
                if (!ok) break;
                tc_fence_after_sync();
                const uint32_t t_base = tmem_base + (uint32_t(q * 32) << 16) + acc * BN_MMA;

                // One head: 64 columns x the quadrant's 32 rows, two loads of 16 rows. kRot is a
                // type so that the rotation is compiled in or out of the inner loop.
                auto head_math = [&](auto rot_tag, int h2) {
                    constexpr bool kRot = decltype(rot_tag)::value;
                    const int c0 = (2 * ch + h2) * 64;  // first column of the head inside the tile
#pragma unroll
                    for (int hr = 0; hr < 2; ++hr) {  // rows g, g+8 then g+16, g+24
                        uint32_t a[32];
                        tmem_ld_16x256_x8(t_base + (uint32_t(16 * hr) << 16) + c0, a);
                        tmem_ld_wait();
                        if (h2 == 1 && hr == 1) {
                            // Every TMEM read of this accumulator is done: hand it back to the MMA
                            // warp before the arithmetic and the store.
                            tc_fence_before_sync();
                            __syncwarp();
                            if (lane == 0) mbar_arrive(&tempty_bar[acc]);
                        }
                        if (hr == 0) {
                            // the store of the previous head must have read the staging tile
                            if (lane == 0) tma_store_wait_read<0>();
                            __syncwarp();
                        }
#pragma unroll
                        for (int k2 = 0; k2 < 2; ++k2) {
                            const int k = 2 * hr + k2;
                            uint32_t wlo[4], whi[4];
#pragma unroll
                            for (int j = 0; j < 4; ++j) {
                                // (acc*sa)*sb, then the rotation in a fixed operation order (no
                                // compiler-chosen contraction): lo' = fma(x0, cos, -(x1*sin)),
                                // hi' = fma(x0, sin, x1*cos)
                                const float2 x0 = mul2(mul2(acc_to_float2<KIND>(a[4 * j + 2 * k2], a[4 * j + 2 * k2 + 1]), sa2[k]), sc[h2][j]);
                                const float2 x1 = mul2(mul2(acc_to_float2<KIND>(a[4 * (j + 4) + 2 * k2], a[4 * (j + 4) + 2 * k2 + 1]), sa2[k]),
                                                       sc[h2][j + 4]);
                                float2 o_lo = x0, o_hi = x1;
                                if constexpr (kRot) {
                                    const float2 m = mul2(x1, sn2[k][j]);
                                    o_lo = fma2(x0, cs2[k][j], make_float2(-m.x, -m.y));
                                    o_hi = fma2(x0, sn2[k][j], mul2(x1, cs2[k][j]));
                                }
                                wlo[j] = pack_half2(o_lo.x, o_lo.y);
                                whi[j] = pack_half2(o_hi.x, o_hi.y);
                            }
                            // rows 8k .. 8k+7 of the quadrant: column chunks 0-3, then 4-7
                            stmatrix_x4(staging + sw128_offset(8 * k + st_row, st_mat), wlo);
                            stmatrix_x4(staging + sw128_offset(8 * k + st_row, 4 + st_mat), whi);
                        }
                    }
                    fence_proxy_async_smem();
                    __syncwarp();
                    if (lane == 0) {
                        tma_store_2d(&tm_out, staging, n0 + c0, m0 + q * 32);
                        tma_store_commit();
                    }
                };
#pragma unroll
                for (int h2 = 0; h2 < 2; ++h2) {
                    if (rotate) head_math(TrueTag{}, h2);
                    else head_math(FalseTag{}, h2);
                }
            }
        } else {
            // SILU: warp `ch` owns output columns [64 ch, 64 ch + 64) of the tile's 128: gate
            // accumulators at those columns, up accumulators 128 columns further.
            // DEQUANT / DEQUANT2: columns [64 ch, 64 ch + 64) of the tile's 128.
            static_assert(BN_OUT == 128, "64 output columns per epilogue warp");
            const int c0 = ch * 64;
            const bool cols_ok = n0 + c0 < p.N;  // N % 64 == 0: the warp's columns are all in or all out
            float2 sc[8], sc_up[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int col = n0 + c0 + 8 * j + 2 * t4;
                sc[j] = cols_ok ? __ldg(reinterpret_cast<const float2 *>(p.scale_b + col)) : make_float2(0.f, 0.f);
                if constexpr (kDual) {
                    // the epilogue works on gate/2: halving the scale is exact
                    sc[j] = make_float2(0.5f * sc[j].x, 0.5f * sc[j].y);
                    sc_up[j] = cols_ok ? __ldg(reinterpret_cast<const float2 *>(p.scale_b2 + col)) : make_float2(0.f, 0.f);
                }
            }
            float sa_next[4];
            if (it.w_begin < it.w_end) load_sa(TileIter::row0(p, it.w_begin), sa_next);
            for (int w = it.w_begin; w < it.w_end && ok; w += it.w_step, ++local) {
                const int m0 = TileIter::row0(p, w);
                const int acc = local & 1;
                const uint32_t acc_phase = (local >> 1) & 1;
                float2 sa2[4];
#pragma unroll
                for (int k = 0; k < 4; ++k) sa2[k] = make_float2(sa_next[k], sa_next[k]);
                if (w + it.w_step < it.w_end) load_sa(TileIter::row0(p, w + it.w_step), sa_next);

                ok = mbar_wait(&tfull_bar[acc], acc_phase, abort_flag, 4);
                if (!ok) break;
                tc_fence_after_sync();
                const uint32_t t_base = tmem_base + (uint32_t(q * 32) << 16) + acc * BN_MMA + c0;
#pragma unroll
                for (int hr = 0; hr < 2; ++hr) {  // rows g, g+8 then g+16, g+24
                    uint32_t a[32], u[32];
                    if (cols_ok) {
                        tmem_ld_16x256_x8(t_base + (uint32_t(16 * hr) << 16), a);
                        if constexpr (kDual) tmem_ld_16x256_x8(t_base + (uint32_t(16 * hr) << 16) + BN_OUT, u);
                        tmem_ld_wait();
                    }
                    if (hr == 1) {
                        // Every TMEM read of this accumulator is done: hand it back to the MMA
                        // warp before the arithmetic and the store.
                        tc_fence_before_sync();
                        __syncwarp();
                        if (lane == 0) mbar_arrive(&tempty_bar[acc]);
                    }
                    if (!cols_ok) continue;
                    if (hr == 0) {
                        // the store of the previous tile must have read the staging tile
                        if (lane == 0) tma_store_wait_read<0>();
                        __syncwarp();
                    }
#pragma unroll
                    for (int k2 = 0; k2 < 2; ++k2) {
                        const int k = 2 * hr + k2;
                        uint32_t wv[8];
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            const float2 v = acc_to_float2<KIND>(a[4 * j + 2 * k2], a[4 * j + 2 * k2 + 1]);
                            float2 o;
                            if constexpr (EPI == FLUKE_SM100_EPI_SILU) {
                                // h = gate/2 = (acc_g*sa)*(sg/2); silu(gate) = gate *
                                // (0.5*tanh(h)+0.5) = h*tanh(h) + h
                                const float2 h = mul2(mul2(v, sa2[k]), sc[j]);
                                const float2 up = mul2(mul2(acc_to_float2<KIND>(u[4 * j + 2 * k2], u[4 * j + 2 * k2 + 1]), sa2[k]), sc_up[j]);
                                const float2 t = make_float2(tanh_approx(h.x), tanh_approx(h.y));
                                o = mul2(fma2(h, t, h), up);
                            } else if constexpr (EPI == FLUKE_SM100_EPI_DEQUANT) {
                                o = mul2(v, mul2(sa2[k], sc[j]));
                            } else {
                                o = mul2(mul2(v, sa2[k]), sc[j]);
                            }
                            wv[j] = pack_half2(o.x, o.y);
                        }
                        // the eight 8 x 8 fragments of rows 8k .. 8k+7: four matrices per instruction
                        const uint32_t lo4[4] = {wv[0], wv[1], wv[2], wv[3]}, hi4[4] = {wv[4], wv[5], wv[6], wv[7]};
                        stmatrix_x4(staging + sw128_offset(8 * k + (lane & 7), lane >> 3), lo4);
                        stmatrix_x4(staging + sw128_offset(8 * k + (lane & 7), 4 + (lane >> 3)), hi4);
                    }
                }
                if (!cols_ok) continue;
                fence_proxy_async_smem();
                __syncwarp();
                if (lane == 0) {
                    tma_store_2d(&tm_out, staging, n0 + c0, m0 + q * 32);
                    tma_store_commit();
                }
            }
        }
        if (lane == 0) tma_store_wait_all<0>();
        __syncwarp();
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        __syncwarp();
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

// ------------------------------------------------------------------------------------------
// ------------------------------------------------------------------------------------------
// Host side: a GemmPlan holds the tensor maps and kernel parameters of one problem; building
// it costs four cuTensorMapEncodeTiled calls, launching it costs one kernel launch. Loops that
// re-run the same GEMM on another plane of a 3-D A tensor (the LSTM down-projection per
// timestep) build the plan once and only change `a_plane`.
// ------------------------------------------------------------------------------------------

struct GemmPlan {
    CUtensorMap tm_a, tm_b, tm_b2, tm_out;
    GemmDev p;
    int grid;
};

inline int device_sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) dev = 0;
    if (!cached[dev]) cudaDeviceGetAttribute(&cached[dev], cudaDevAttrMultiProcessorCount, dev);
    return cached[dev];
}

// Raises the dynamic shared-memory limit of KERNEL once per device. The kernel is a template
// argument so that every instantiation keeps its own "done" flags.
template <auto KERNEL>
int configure_smem(int bytes) {
    static bool done[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) dev = 0;
    if (!done[dev]) {
        cudaError_t e =
            cudaFuncSetAttribute(KERNEL, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
        if (e != cudaSuccess) return (int)e;
        done[dev] = true;
    }
    return 0;
}

// `a_planes` > 1 describes A as [a_planes, M, K] (plane stride M*K bytes).
template <int KIND, int EPI, int BN_MMA, int STAGES>
int plan_build(const fluke_sm100_gemm_t *g, int a_planes, GemmPlan *plan) {
    constexpr bool kDual = (EPI == FLUKE_SM100_EPI_SILU);
    constexpr int BN_OUT = kDual ? BN_MMA / 2 : BN_MMA;
    constexpr bool kRaw = (EPI == FLUKE_SM100_EPI_RAW);
    int rc;
    rc = make_tmap_3d(&plan->tm_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, g->a, a_planes, g->M, g->K,
                      g->K, uint64_t(g->M) * g->K, kBlockM, kBlockKBytes, true);
    if (rc) return rc;
    rc = make_tmap_2d(&plan->tm_b, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, g->b, g->N, g->K, g->K,
                      BN_OUT, kBlockKBytes, true);
    if (rc) return rc;
    plan->tm_b2 = plan->tm_b;
    if (kDual) {
        rc = make_tmap_2d(&plan->tm_b2, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, g->b2, g->N, g->K,
                          g->K, BN_OUT, kBlockKBytes, true);
        if (rc) return rc;
    }
    if (kRaw) {
        rc = make_tmap_2d(&plan->tm_out,
                          KIND == kKindI8 ? CU_TENSOR_MAP_DATA_TYPE_INT32
                                          : CU_TENSOR_MAP_DATA_TYPE_FLOAT32,
                          4, g->out, g->M, g->N, uint64_t(g->ld_out) * 4, kStageRows, 32, true);
    } else {
        rc = make_tmap_2d(&plan->tm_out, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, g->out, g->M, g->N,
                          uint64_t(g->ld_out) * 2, kStageRows, 64, true);
    }
    if (rc) return rc;

    GemmDev &p = plan->p;
    p.M = g->M; p.N = g->N; p.K = g->K;
    p.num_m_tiles = (g->M + kBlockM - 1) / kBlockM;
    p.num_n_tiles = (g->N + BN_OUT - 1) / BN_OUT;
    p.num_k_blocks = (g->K + kBlockKBytes - 1) / kBlockKBytes;
    p.scale_a = g->scale_a; p.const_scale_a = g->const_scale_a;
    p.scale_b = g->scale_b; p.scale_b2 = g->scale_b2;
    p.sin_tab = g->sin_tab; p.cos_tab = g->cos_tab;
    p.seqlen = g->seqlen > 0 ? g->seqlen : 1;
    p.qk_cols = g->qk_cols;
    p.a_plane = 0;
    // weight-stationary schedule: every N tile gets the same number of CTAs, which split the
    // M tiles between them
    const int sms = device_sm_count();
    if (p.num_n_tiles > sms || p.num_k_blocks > SmemLayout<EPI, BN_MMA, STAGES>::kMaxKBlocks)
        return (int)cudaErrorInvalidValue;  // N tile count / K beyond what one resident tile covers
    p.seq_tiles = 0; p.n_seq = 0; p.items_per_cta = 0;
    int items = p.num_m_tiles;
    if (EPI == FLUKE_SM100_EPI_ROTARY && p.seqlen >= kBlockM && g->M % p.seqlen == 0) {
        p.seq_tiles = (p.seqlen + kBlockM - 1) / kBlockM;
        p.n_seq = g->M / p.seqlen;
        items = p.seq_tiles * p.n_seq;
    }
    int per_n = sms / p.num_n_tiles;
    if (per_n > items) per_n = items;
    if (per_n < 1) per_n = 1;
    if (p.seq_tiles > 0) {
        p.items_per_cta = (items + per_n - 1) / per_n;
        per_n = (items + p.items_per_cta - 1) / p.items_per_cta;  // no CTA without work
    }
    p.ctas_per_n = per_n;
    plan->grid = p.num_m_tiles > 0 ? per_n * p.num_n_tiles : 0;
    return 0;
}

template <int KIND, int EPI, int BN_MMA, int STAGES>
int plan_launch(const GemmPlan &plan, int a_plane, cudaStream_t stream) {
    using L = SmemLayout<EPI, BN_MMA, STAGES>;
    auto kernel = gemm_kernel<KIND, EPI, BN_MMA, STAGES>;
    int rc = configure_smem<gemm_kernel<KIND, EPI, BN_MMA, STAGES>>(L::kDynamic);
    if (rc) return rc;
    if (plan.grid == 0) return 0;
    GemmDev p = plan.p;
    p.a_plane = a_plane;
    kernel<<<plan.grid, kNumThreads, L::kDynamic, stream>>>(plan.tm_a, plan.tm_b, plan.tm_b2,
                                                            plan.tm_out, p);
    return (int)cudaGetLastError();
}

template <int KIND, int EPI, int BN_MMA, int STAGES>
int launch(const fluke_sm100_gemm_t *g, cudaStream_t stream) {
    if (g->M == 0) return 0;
    GemmPlan plan;
    int rc = plan_build<KIND, EPI, BN_MMA, STAGES>(g, 1, &plan);
    if (rc) return rc;
    return plan_launch<KIND, EPI, BN_MMA, STAGES>(plan, 0, stream);
}

// Tile shapes: 128 x 128 (K up to 1024 resident) for the plain GEMMs; 128 x 256 (one UMMA of
// N = 256 per K step, K up to 512 resident) for the two fused transformer kernels. Beside the
// resident weight tile and 32 KB of store staging there is room for a ring of four 16 KB
// activation stages.
constexpr int kPlainBN = 128, kFusedBN = 256;
constexpr int kPlainStages = 4, kFusedStages = 4, kSiluStages = 4;

template <int KIND>
int dispatch(const fluke_sm100_gemm_t *g, cudaStream_t s) {
    switch (g->epilogue) {
        case FLUKE_SM100_EPI_RAW:
            return launch<KIND, FLUKE_SM100_EPI_RAW, kPlainBN, kPlainStages>(g, s);
        case FLUKE_SM100_EPI_DEQUANT:
            return launch<KIND, FLUKE_SM100_EPI_DEQUANT, kPlainBN, kPlainStages>(g, s);
        case FLUKE_SM100_EPI_DEQUANT2:
            return launch<KIND, FLUKE_SM100_EPI_DEQUANT2, kPlainBN, kPlainStages>(g, s);
        case FLUKE_SM100_EPI_ROTARY:
            return launch<KIND, FLUKE_SM100_EPI_ROTARY, kFusedBN, kFusedStages>(g, s);
        case FLUKE_SM100_EPI_SILU:
            return launch<KIND, FLUKE_SM100_EPI_SILU, kFusedBN, kSiluStages>(g, s);
        default:
            return (int)cudaErrorInvalidValue;
    }
}

}  // namespace
}  // namespace fluke_sm100

// The epilogue reads scale_b and stores output in 64-column chunks, so N must be a multiple
// of 64 (all weights of the path are); K only needs the 16-byte TMA row alignment.
extern "C" int fluke_sm100_gemm(const fluke_sm100_gemm_t *g, void *stream) {
    using namespace fluke_sm100;
    if (!g || g->M < 0 || g->N <= 0 || g->K <= 0) return (int)cudaErrorInvalidValue;
    // the weight tile of a CTA stays resident: K <= 1024 bytes (plain) / 512 bytes (fused kernels)
    if (g->K > ((g->epilogue == FLUKE_SM100_EPI_ROTARY || g->epilogue == FLUKE_SM100_EPI_SILU) ? 512 : 1024))
        return (int)cudaErrorInvalidValue;
    if (g->K % 16 != 0 || g->N % 64 != 0) return (int)cudaErrorInvalidValue;
    if (g->epilogue == FLUKE_SM100_EPI_ROTARY && (g->qk_cols % 256 != 0 || g->N % 256 != 0))
        return (int)cudaErrorInvalidValue;
    if (g->epilogue == FLUKE_SM100_EPI_SILU && g->N % 128 != 0) return (int)cudaErrorInvalidValue;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (g->kind == FLUKE_SM100_KIND_I8) return dispatch<kKindI8>(g, s);
    if (g->kind == FLUKE_SM100_KIND_F8) return dispatch<kKindF8>(g, s);
    return (int)cudaErrorInvalidValue;
}


extern "C" int fluke_sm100_compute_capability(int device_index) {
    int major = 0, minor = 0;
    if (cudaDeviceGetAttribute(&major, cudaDevAttrComputeCapabilityMajor, device_index) !=
            cudaSuccess ||
        cudaDeviceGetAttribute(&minor, cudaDevAttrComputeCapabilityMinor, device_index) !=
            cudaSuccess)
        return -1;
    return major * 10 + minor;
}

extern "C" int fluke_sm100_malloc(void **ptr, size_t bytes) {
    return (int)cudaMalloc(ptr, bytes);
}
// Waits for the device's outstanding work before releasing (cudaFree does), so a kernel still
// reading the block finishes first.
extern "C" int fluke_sm100_free(void *ptr) {
    return (int)cudaFree(ptr);
}
extern "C" int fluke_sm100_current_device(void) {
    int dev = -1;
    return cudaGetDevice(&dev) == cudaSuccess ? dev : -1;
}

extern "C" const char *fluke_sm100_error_string(int code) {
    return cudaGetErrorString(static_cast<cudaError_t>(code));
}

extern "C" int fluke_sm100_read_status(unsigned int *status_out, int reset) {
    unsigned int v = 0;
    cudaError_t e = cudaMemcpyFromSymbol(&v, fluke_sm100::g_status, sizeof(v));
    if (e != cudaSuccess) return (int)e;
    if (status_out) *status_out = v;
    if (reset && v != 0) {
        const unsigned int zero = 0;
        e = cudaMemcpyToSymbol(fluke_sm100::g_status, &zero, sizeof(zero));
    }
    return (int)e;
}
