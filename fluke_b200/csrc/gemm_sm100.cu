// gemm_sm100.cu -- the tcgen05 GEMM family of the quantized transformer path on sm_100a.
//
// One persistent, warp-specialised, WEIGHT-STATIONARY kernel template computes
// out = epilogue(A @ B^T) for K-major 8-bit operands (int8 -> int32 via kind::i8,
// e4m3 -> f32 via kind::f8f6f4). A CTA owns one N tile of the weight for its whole life: the
// tile (all of K, up to 128 KB) is TMA-loaded into shared memory once, and the CTA then streams
// the M tiles assigned to it, so per output tile only the 128 x K activation block crosses
// L2 -> SM (the activations are what is large; the weights of this path are at most 2 MB).
//
//   warp 0      TMA producer: the resident weight tile once, then 128-byte-swizzled A blocks
//               into a ring of shared-memory stages
//   warp 1      MMA issuer: tcgen05.mma 128 x BN x 32B from shared-memory descriptors into one
//               of two accumulator buffers in tensor memory
//   warps 2-9   epilogue: two warps per TMEM lane quadrant, each owning half of the tile's
//               columns: tcgen05.ld (thread = output row), dequant / rotary / SiLU in
//               registers, f16 pack, swizzled smem staging, TMA tile store
//
// The two accumulator buffers let the epilogue of tile i overlap the MMAs of tile i+1; no
// accumulator or f16 intermediate ever reaches HBM. The rotary tables of a tile's 128 rows are
// staged once per tile in shared memory (coalesced loads, swizzled rows); the weight scales of
// the CTA's N tile are staged once per launch.
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
constexpr int kBlockKBytes = 128;     // K bytes per stage = one swizzle row
constexpr int kUmmaKBytes = 32;       // K bytes per tcgen05.mma
constexpr int kNumThreads = 320;
constexpr int kEpilogueWarp0 = 2;
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
};


template <int EPI, int BN_MMA, int STAGES>
struct SmemLayout {
    static constexpr bool kRotary = (EPI == FLUKE_SM100_EPI_ROTARY);
    static constexpr int kMaxKBlocks = kWeightBytes / (BN_MMA * kBlockKBytes);  // 4 (BN 256) or 8 (BN 128)
    static constexpr int kABytes = kBlockM * kBlockKBytes;
    static constexpr int kBBytes = BN_MMA * kBlockKBytes;   // one K block of the weight tile
    static constexpr int kOffW = 0;
    static constexpr int kOffA = kWeightBytes;
    static constexpr int kOffStaging = kOffA + STAGES * kABytes;
    static constexpr int kOffTables = kOffStaging + kEpilogueWarps * kStagingBytes;
    static constexpr int kOffScaleB = kOffTables + (kRotary ? 4 * 8192 : 0);  // per quadrant: sin 4 KB | cos 4 KB
    static constexpr int kOffBars = kOffScaleB + (EPI == FLUKE_SM100_EPI_SILU ? 0 : BN_MMA * 4);
    static constexpr int kNumBars = 2 * STAGES + 5 + 8;
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

// Writes one 128-byte row (8 x 16-byte chunks held in v[0..31]) into a swizzled staging tile.
__device__ __forceinline__ void stage_row(uint8_t *staging, uint32_t row, const uint32_t (&v)[32]) {
#pragma unroll
    for (uint32_t ch = 0; ch < 8; ++ch) {
        uint4 q = make_uint4(v[4 * ch], v[4 * ch + 1], v[4 * ch + 2], v[4 * ch + 3]);
        *reinterpret_cast<uint4 *>(staging + sw128_offset(row, ch)) = q;
    }
}

// Bounded barrier between the two epilogue warps of a lane quadrant (one arrival per warp).
__device__ __forceinline__ bool pair_barrier(uint64_t *bar, uint32_t parity, int lane,
                                             volatile int *abort_flag) {
    __syncwarp();
    if (lane == 0) mbar_arrive(bar);
    return mbar_wait(bar, parity, abort_flag, 5);
}

__device__ __forceinline__ void ld4(const float *p, float (&v)[4]) {
    const float4 t = *reinterpret_cast<const float4 *>(p);
    v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
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
    uint64_t *w_bar = bars + 2 * STAGES + 4;          // resident weight tile loaded
    uint64_t *tab_full_bar = bars + 2 * STAGES + 5;   // [4] tables of the quadrant are staged
    uint64_t *tab_empty_bar = bars + 2 * STAGES + 9;  // [4] both warps are done reading them
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + L::kOffMisc);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + L::kOffMisc + 4);
    float *sbs = reinterpret_cast<float *>(smem + L::kOffScaleB);  // weight scales of this N tile

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
        for (int s = 0; s < 4; ++s) {
            mbar_init(&tab_full_bar[s], 2);
            mbar_init(&tab_empty_bar[s], 2);
        }
        *abort_flag = 0;
        fence_barrier_init();
        tma_prefetch_desc(&tm_a);
        tma_prefetch_desc(&tm_b);
        if (kDual) tma_prefetch_desc(&tm_b2);
        tma_prefetch_desc(&tm_out);
    }
    if (warp == 1) tmem_alloc(tmem_slot, kTmemCols);
    if (warp >= kEpilogueWarp0) {
        // weight scales of the tile's columns (zeros past N), read by every epilogue thread
        if constexpr (EPI != FLUKE_SM100_EPI_RAW && EPI != FLUKE_SM100_EPI_SILU) {
            for (int j = threadIdx.x - 64; j < BN_MMA; j += kEpilogueWarps * 32) {
                float v;
                if (kDual) {
                    const int col = n0 + (j % BN_OUT);
                    v = col < p.N ? __ldg((j < BN_OUT ? p.scale_b : p.scale_b2) + col) : 0.f;
                } else {
                    v = n0 + j < p.N ? __ldg(p.scale_b + n0 + j) : 0.f;
                }
                sbs[j] = v;
            }
        }
    }
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        // ------------------------------ TMA producer ------------------------------
        if (lane == 0) {
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
        }
        __syncwarp();
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        for (int mt = m_first; mt < p.num_m_tiles && ok; mt += p.ctas_per_n) {
            const int m0 = mt * kBlockM;
            for (int kb = 0; kb < p.num_k_blocks; ++kb) {
                ok = mbar_wait(&empty_bar[stage], phase ^ 1u, abort_flag, 1);
                if (!ok) break;
                if (lane == 0) {
                    mbar_arrive_expect_tx(&full_bar[stage], L::kABytes);
                    tma_load_3d(smem + L::kOffA + stage * L::kABytes, &tm_a, &full_bar[stage],
                                kb * kBlockKBytes, m0, p.a_plane);
                }
                __syncwarp();
                if (++stage == STAGES) { stage = 0; phase ^= 1u; }
            }
        }
        if (!ok) {
            // Give loads that are still in flight a bounded chance to land before the CTA's
            // shared memory is released.
            const long long t0 = clock64();
            while (clock64() - t0 < (1ll << 22)) { }
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer --------------------------------
        int stage = 0;
        uint32_t phase = 0;
        int local = 0;
        bool ok = mbar_wait(w_bar, 0, abort_flag, 6);
        for (int mt = m_first; mt < p.num_m_tiles && ok; mt += p.ctas_per_n, ++local) {
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
                if (lane == 0) {
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
                }
                __syncwarp();
                if (++stage == STAGES) { stage = 0; phase ^= 1u; }
            }
        }
    } else {
        // ------------------------------ epilogue ----------------------------------
        const int q = warp & 3;                           // TMEM lane quadrant this warp may read
        const int ch = (warp - kEpilogueWarp0) >> 2;      // which half of the tile's columns
        uint8_t *staging = smem + L::kOffStaging + (warp - kEpilogueWarp0) * kStagingBytes;
        uint8_t *tables = smem + L::kOffTables + q * 8192;  // ROTARY only
        const bool rotate = (EPI == FLUKE_SM100_EPI_ROTARY) && n0 < p.qk_cols;
        int local = 0;
        uint32_t tab_phase = 0;
        bool ok = true;
        for (int mt = m_first; mt < p.num_m_tiles && ok; mt += p.ctas_per_n, ++local) {
            const int m0 = mt * kBlockM;
            const int acc = local & 1;
            const uint32_t acc_phase = (local >> 1) & 1;
            const int row = m0 + q * 32 + lane;
            const bool row_ok = row < p.M;

            float sa = 0.f;
            if constexpr (EPI != FLUKE_SM100_EPI_RAW) {
                sa = p.scale_a ? (row_ok ? __ldg(p.scale_a + row) : 0.f) : p.const_scale_a;
            }

            // Rotary tables of the quadrant's 32 rows, staged once per tile: warp ch = 0 copies
            // the sin rows, ch = 1 the cos rows (coalesced 16-byte loads, swizzled 128-byte rows).
            if constexpr (EPI == FLUKE_SM100_EPI_ROTARY) {
                if (rotate) {
                    const float *src = ch == 0 ? p.sin_tab : p.cos_tab;
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const int id = j * 32 + lane;
                        const int r = id >> 3, cc = id & 7;
                        const int grow = m0 + q * 32 + r;
                        const int pos = grow < p.M ? grow % p.seqlen : 0;
                        const float4 v = __ldg(reinterpret_cast<const float4 *>(src + pos * 32) + cc);
                        *reinterpret_cast<float4 *>(tables + ch * 4096 + sw128_offset(r, cc)) = v;
                    }
                    ok = pair_barrier(&tab_full_bar[q], tab_phase, lane, abort_flag);
                    if (!ok) break;
                }
            }

            ok = mbar_wait(&tfull_bar[acc], acc_phase, abort_flag, 4);
            if (!ok) break;
            tc_fence_after_sync();
            const uint32_t t_row = tmem_base + (uint32_t(q * 32) << 16) + acc * BN_MMA;

            constexpr int kChunkCols = (EPI == FLUKE_SM100_EPI_RAW) ? 32 : 64;
            constexpr int kChunks = kWarpCols / kChunkCols;
#pragma unroll 1
            for (int chunk = 0; chunk < kChunks; ++chunk) {
                const int c0 = ch * kWarpCols + chunk * kChunkCols;  // column inside the tile
                const bool chunk_ok = n0 + c0 < p.N;  // N % 64 == 0: a chunk is all in or all out
                uint32_t outw[32];  // one 128-byte output row segment

                if (!chunk_ok) {
                    // columns past N: nothing to compute or store
                } else if constexpr (EPI == FLUKE_SM100_EPI_RAW) {
                    tmem_ld_32x32(t_row + c0, outw);
                    tmem_ld_wait();
                } else if constexpr (EPI == FLUKE_SM100_EPI_SILU) {
#pragma unroll
                    for (int half = 0; half < 2; ++half) {
                        uint32_t g[32], u[32];
                        tmem_ld_32x32(t_row + c0 + half * 32, g);
                        tmem_ld_32x32(t_row + BN_OUT + c0 + half * 32, u);
                        float sg[32], su[32];
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            // weight scales through L1 (the same address in every lane); N % 128 == 0 here
                            const float4 a4 = __ldg(reinterpret_cast<const float4 *>(p.scale_b + n0 + c0 + half * 32) + i);
                            const float4 b4 = __ldg(reinterpret_cast<const float4 *>(p.scale_b2 + n0 + c0 + half * 32) + i);
                            sg[4 * i] = a4.x; sg[4 * i + 1] = a4.y; sg[4 * i + 2] = a4.z; sg[4 * i + 3] = a4.w;
                            su[4 * i] = b4.x; su[4 * i + 1] = b4.y; su[4 * i + 2] = b4.z; su[4 * i + 3] = b4.w;
                        }
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            float o[2];
#pragma unroll
                            for (int j = 0; j < 2; ++j) {
                                const int e = 2 * i + j;
                                const float gate = (acc_to_float<KIND>(g[e]) * sa) * sg[e];
                                const float up = (acc_to_float<KIND>(u[e]) * sa) * su[e];
                                const float sig = 0.5f * tanh_approx(0.5f * gate) + 0.5f;
                                o[j] = gate * sig * up;
                            }
                            outw[half * 16 + i] = pack_half2(o[0], o[1]);
                        }
                    }
                } else if constexpr (EPI == FLUKE_SM100_EPI_ROTARY) {
                    // One head: pairs (i, i+32). Two passes of 16 pairs; every load of a pass is
                    // issued before its first use.
#pragma unroll
                    for (int sub = 0; sub < 2; ++sub) {
                        uint32_t lo[16], hi[16];
                        tmem_ld_32x16(t_row + c0 + sub * 16, lo);
                        tmem_ld_32x16(t_row + c0 + 32 + sub * 16, hi);
                        float bl[16], bh[16], sn[16], cs[16];
#pragma unroll
                        for (int i = 0; i < 4; ++i) {
                            float t4[4];
                            ld4(sbs + c0 + sub * 16 + 4 * i, t4);
                            bl[4 * i] = t4[0]; bl[4 * i + 1] = t4[1]; bl[4 * i + 2] = t4[2]; bl[4 * i + 3] = t4[3];
                            ld4(sbs + c0 + 32 + sub * 16 + 4 * i, t4);
                            bh[4 * i] = t4[0]; bh[4 * i + 1] = t4[1]; bh[4 * i + 2] = t4[2]; bh[4 * i + 3] = t4[3];
                            if (rotate) {
                                ld4(reinterpret_cast<const float *>(tables + sw128_offset(lane, sub * 4 + i)), t4);
                                sn[4 * i] = t4[0]; sn[4 * i + 1] = t4[1]; sn[4 * i + 2] = t4[2]; sn[4 * i + 3] = t4[3];
                                ld4(reinterpret_cast<const float *>(tables + 4096 + sw128_offset(lane, sub * 4 + i)), t4);
                                cs[4 * i] = t4[0]; cs[4 * i + 1] = t4[1]; cs[4 * i + 2] = t4[2]; cs[4 * i + 3] = t4[3];
                            }
                        }
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            float o_lo[2], o_hi[2];
#pragma unroll
                            for (int j = 0; j < 2; ++j) {
                                const int e = 2 * i + j;
                                const float x0 = (acc_to_float<KIND>(lo[e]) * sa) * bl[e];
                                const float x1 = (acc_to_float<KIND>(hi[e]) * sa) * bh[e];
                                if (rotate) {
                                    // fixed operation order (no compiler-chosen contraction)
                                    o_lo[j] = __fmaf_rn(x0, cs[e], -__fmul_rn(x1, sn[e]));
                                    o_hi[j] = __fmaf_rn(x0, sn[e], __fmul_rn(x1, cs[e]));
                                } else {
                                    o_lo[j] = x0;
                                    o_hi[j] = x1;
                                }
                            }
                            outw[sub * 8 + i] = pack_half2(o_lo[0], o_lo[1]);
                            outw[16 + sub * 8 + i] = pack_half2(o_hi[0], o_hi[1]);
                        }
                    }
                } else {
                    // DEQUANT / DEQUANT2: 64 columns in two passes of 32
#pragma unroll
                    for (int half = 0; half < 2; ++half) {
                        uint32_t a[32];
                        tmem_ld_32x32(t_row + c0 + half * 32, a);
                        float bv[32];
#pragma unroll
                        for (int i = 0; i < 8; ++i) {
                            float t4[4];
                            ld4(sbs + c0 + half * 32 + 4 * i, t4);
                            bv[4 * i] = t4[0]; bv[4 * i + 1] = t4[1]; bv[4 * i + 2] = t4[2]; bv[4 * i + 3] = t4[3];
                        }
                        tmem_ld_wait();
#pragma unroll
                        for (int i = 0; i < 16; ++i) {
                            float o[2];
#pragma unroll
                            for (int j = 0; j < 2; ++j) {
                                const float v = acc_to_float<KIND>(a[2 * i + j]);
                                if constexpr (EPI == FLUKE_SM100_EPI_DEQUANT) o[j] = v * (sa * bv[2 * i + j]);
                                else o[j] = (v * sa) * bv[2 * i + j];
                            }
                            outw[half * 16 + i] = pack_half2(o[0], o[1]);
                        }
                    }
                }

                if (chunk == kChunks - 1) {
                    // Every TMEM read of this accumulator is done: hand it back to the MMA warp
                    // before the slower store path.
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
            if constexpr (EPI == FLUKE_SM100_EPI_ROTARY) {
                if (rotate) {
                    // both warps of the quadrant are done with the tables of this tile
                    ok = pair_barrier(&tab_empty_bar[q], tab_phase, lane, abort_flag);
                    tab_phase ^= 1u;
                }
            }
        }
        if (lane == 0) tma_store_wait_all<0>();
        __syncwarp();
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
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
    int per_n = sms / p.num_n_tiles;
    if (per_n > p.num_m_tiles) per_n = p.num_m_tiles;
    if (per_n < 1) per_n = 1;
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
// N = 256 per K step, K up to 512 resident) for the two fused transformer kernels. The last
// number is the depth of the ring of 16 KB activation stages that fits beside the resident
// weight tile, the store staging and (rotary) the tables.
constexpr int kPlainBN = 128, kPlainStages = 4;
constexpr int kFusedBN = 256, kFusedStages = 2, kSiluStages = 4;

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
