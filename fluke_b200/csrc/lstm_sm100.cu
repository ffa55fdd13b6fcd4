// lstm_sm100.cu -- factored-LSTM kernels for sm_100a.
//
// The fused step replaces TensorOpFactoredLstmI8 (cute/ampere/factored_lstm/
// factored_lstm_i8.py:169-476): A = [hh_down | x_down] (f16, K-merged) is contracted against
// the four gate weights W_g = [up_hh_g | up_ih_g] into four f32 accumulators, then bias,
// hard-sigmoid / clamp gates, f32 cell update in place and an int8 hidden output at the
// fixed scale 1/127 (round half away from zero, :459-473).
//
// Mapping: a CTA owns 128 chunk rows (TMEM lanes) and UNITS hidden units. The four gate
// slices of W (UNITS rows each) are TMA-loaded back to back into one shared-memory operand,
// so ONE tcgen05.mma of shape 128 x (4*UNITS) x 16 per K step fills all four gate
// accumulators: gate g of unit u is TMEM column g*UNITS + u, and the epilogue thread that
// owns a row finds i, f, g, o of a unit in its own registers.
//
// The layer driver runs x_down for all timesteps as one int8 GEMM, then per timestep the
// int8 down-projection of h_{t-1} and the fused step, with every tensor map built once per
// layer (the timestep is a TMA plane coordinate).
#include <fluke/fluke.h>

#include "fluke_sm100.h"
#include "sm100_ptx.cuh"
#include "tma_host.cuh"

#include <cuda_fp16.h>

namespace fluke_sm100 {
namespace {

constexpr int kLstmThreads = 192;
constexpr int kLstmMaxKB = 4;  // K blocks of 64 f16 kept resident: Kc <= 256

struct LstmDev {
    int B, H;
    int nkb, nkb_lo;        // K blocks in total / taken from a_lo
    int plane_lo, plane_hi; // planes of the two A tensor maps read by this launch
    const float *bias[4];
    float *c;
    int8_t *h_out;
};

template <int UNITS>
struct LstmSmem {
    static constexpr int kABytes = 128 * 128;
    static constexpr int kWBytes = 4 * UNITS * 128;
    static constexpr int kOffA = 0;
    static constexpr int kOffW = kLstmMaxKB * kABytes;
    static constexpr int kOffBars = kOffW + kLstmMaxKB * kWBytes;
    static constexpr int kOffMisc = kOffBars + (kLstmMaxKB + 1) * 8;
    static constexpr int kDynamic = kOffMisc + 16 + 1024;
};

__device__ __forceinline__ float hard_sigmoid(float x) {
    return fmaxf(0.f, fminf(1.f, __fmaf_rn(x, 0.2f, 0.5f)));
}

// h in [-1, 1] -> int8 code at scale 1/127, rounding half away from zero.
__device__ __forceinline__ int quant_h(float h) {
    const float hs = __fmul_rn(h, 127.0f);
    const float half = fmaxf(-0.5f, fminf(0.5f, hs * 1e30f));
    return __float2int_rz(hs + half);
}

template <int UNITS>
__global__ void __launch_bounds__(kLstmThreads, 1)
lstm_step_kernel(const __grid_constant__ CUtensorMap tm_a_lo,
                 const __grid_constant__ CUtensorMap tm_a_hi,
                 const __grid_constant__ CUtensorMap tm_w0, const __grid_constant__ CUtensorMap tm_w1,
                 const __grid_constant__ CUtensorMap tm_w2, const __grid_constant__ CUtensorMap tm_w3,
                 const LstmDev p) {
    using L = LstmSmem<UNITS>;
    constexpr int N_MMA = 4 * UNITS;
    constexpr uint32_t kTmemCols = N_MMA <= 64 ? 64 : (N_MMA <= 128 ? 128 : 256);
    constexpr uint32_t kIdesc = make_idesc<kKindF16>(128, N_MMA);

    extern __shared__ uint8_t smem_raw[];
    uint8_t *smem = reinterpret_cast<uint8_t *>(
        (reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    uint64_t *full_bar = reinterpret_cast<uint64_t *>(smem + L::kOffBars);
    uint64_t *tfull_bar = full_bar + kLstmMaxKB;
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(smem + L::kOffMisc);
    volatile int *abort_flag = reinterpret_cast<volatile int *>(smem + L::kOffMisc + 4);

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int m0 = blockIdx.x * 128;
    const int n0 = blockIdx.y * UNITS;

    if (threadIdx.x == 0) {
        for (int s = 0; s < kLstmMaxKB; ++s) mbar_init(&full_bar[s], 1);
        mbar_init(tfull_bar, 1);
        *abort_flag = 0;
        fence_barrier_init();
    }
    if (warp == 1) tmem_alloc(tmem_slot, kTmemCols);
    tc_fence_before_sync();
    __syncthreads();
    tc_fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            for (int kb = 0; kb < p.nkb; ++kb) {
                mbar_arrive_expect_tx(&full_bar[kb], L::kABytes + L::kWBytes);
                uint8_t *sa = smem + L::kOffA + kb * L::kABytes;
                uint8_t *sw = smem + L::kOffW + kb * L::kWBytes;
                if (kb < p.nkb_lo) tma_load_3d(sa, &tm_a_lo, &full_bar[kb], kb * 64, m0, p.plane_lo);
                else tma_load_3d(sa, &tm_a_hi, &full_bar[kb], (kb - p.nkb_lo) * 64, m0, p.plane_hi);
                tma_load_2d(sw + 0 * UNITS * 128, &tm_w0, &full_bar[kb], kb * 64, n0);
                tma_load_2d(sw + 1 * UNITS * 128, &tm_w1, &full_bar[kb], kb * 64, n0);
                tma_load_2d(sw + 2 * UNITS * 128, &tm_w2, &full_bar[kb], kb * 64, n0);
                tma_load_2d(sw + 3 * UNITS * 128, &tm_w3, &full_bar[kb], kb * 64, n0);
            }
        }
        __syncwarp();
    } else if (warp == 1) {
        bool ok = true;
        for (int kb = 0; kb < p.nkb && ok; ++kb) {
            ok = mbar_wait(&full_bar[kb], 0, abort_flag, 16);
            if (!ok) break;
            tc_fence_after_sync();
            if (lane == 0) {
                const uint64_t adesc = make_smem_desc_sw128(smem_u32(smem + L::kOffA + kb * L::kABytes));
                const uint64_t bdesc = make_smem_desc_sw128(smem_u32(smem + L::kOffW + kb * L::kWBytes));
#pragma unroll
                for (int k = 0; k < 4; ++k)
                    tc_mma<kKindF16>(tmem_base, adesc + uint64_t(2 * k), bdesc + uint64_t(2 * k),
                                     kIdesc, (kb | k) != 0 ? 1u : 0u);
                if (kb == p.nkb - 1) tc_commit(tfull_bar);
            }
            __syncwarp();
        }
    } else {
        const int q = warp & 3;
        const int row = m0 + q * 32 + lane;
        const bool row_ok = row < p.B;
        if (mbar_wait(tfull_bar, 0, abort_flag, 17)) {
            tc_fence_after_sync();
            const uint32_t t_row = tmem_base + (uint32_t(q * 32) << 16);
#pragma unroll 1
            for (int u0 = 0; u0 < UNITS; u0 += 16) {
                uint32_t gi[16], gf[16], gg[16], go[16];
                tmem_ld_32x16(t_row + 0 * UNITS + u0, gi);
                tmem_ld_32x16(t_row + 1 * UNITS + u0, gf);
                tmem_ld_32x16(t_row + 2 * UNITS + u0, gg);
                tmem_ld_32x16(t_row + 3 * UNITS + u0, go);
                tmem_ld_wait();
                if (row_ok) {
                    const int64_t off = int64_t(row) * p.H + n0 + u0;
                    float cv[16];
#pragma unroll
                    for (int v = 0; v < 4; ++v) {
                        const float4 c4 = *reinterpret_cast<const float4 *>(p.c + off + 4 * v);
                        cv[4 * v] = c4.x; cv[4 * v + 1] = c4.y; cv[4 * v + 2] = c4.z; cv[4 * v + 3] = c4.w;
                    }
                    uint32_t hq[4];
#pragma unroll
                    for (int v = 0; v < 4; ++v) {
                        const float4 bi = __ldg(reinterpret_cast<const float4 *>(p.bias[0] + n0 + u0) + v);
                        const float4 bf = __ldg(reinterpret_cast<const float4 *>(p.bias[1] + n0 + u0) + v);
                        const float4 bg = __ldg(reinterpret_cast<const float4 *>(p.bias[2] + n0 + u0) + v);
                        const float4 bo = __ldg(reinterpret_cast<const float4 *>(p.bias[3] + n0 + u0) + v);
                        const float bis[4] = {bi.x, bi.y, bi.z, bi.w}, bfs[4] = {bf.x, bf.y, bf.z, bf.w};
                        const float bgs[4] = {bg.x, bg.y, bg.z, bg.w}, bos[4] = {bo.x, bo.y, bo.z, bo.w};
                        uint32_t packed = 0;
#pragma unroll
                        for (int j = 0; j < 4; ++j) {
                            const int e = 4 * v + j;
                            const float i_a = hard_sigmoid(__uint_as_float(gi[e]) + bis[j]);
                            const float f_a = hard_sigmoid(__uint_as_float(gf[e]) + bfs[j]);
                            const float o_a = hard_sigmoid(__uint_as_float(go[e]) + bos[j]);
                            const float g_a = fmaxf(-1.f, fminf(1.f, __uint_as_float(gg[e]) + bgs[j]));
                            const float c_new = __fmaf_rn(f_a, cv[e], __fmul_rn(i_a, g_a));
                            cv[e] = c_new;
                            const float h_new = o_a * tanhf(c_new);
                            packed |= (uint32_t(quant_h(h_new)) & 0xFFu) << (8 * j);
                        }
                        hq[v] = packed;
                    }
#pragma unroll
                    for (int v = 0; v < 4; ++v)
                        *reinterpret_cast<float4 *>(p.c + off + 4 * v) =
                            make_float4(cv[4 * v], cv[4 * v + 1], cv[4 * v + 2], cv[4 * v + 3]);
                    *reinterpret_cast<uint4 *>(p.h_out + off) = make_uint4(hq[0], hq[1], hq[2], hq[3]);
                }
            }
        }
    }

    tc_fence_before_sync();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after_sync();
        tmem_dealloc(tmem_base, kTmemCols);
    }
}

// ---- host side ---------------------------------------------------------------------------------

struct LstmPlan {
    CUtensorMap tm_a_lo, tm_a_hi, tm_w[4];
    LstmDev p;
    int units;
    dim3 grid;
};

inline int pick_units(int B, int H) {
    const int row_tiles = (B + 127) / 128;
    const int cand[4] = {64, 48, 32, 16};
    int best = 0;
    for (int i = 0; i < 4; ++i) {
        if (H % cand[i]) continue;
        best = cand[i];
        if (row_tiles * (H / cand[i]) >= 128) break;  // enough CTAs to fill the GPU
    }
    return best;
}

// planes_lo / planes_hi: number of [B, k] planes behind a_lo / a_hi (plane stride B*ld).
int lstm_plan_build(const fluke_sm100_lstm_step_t *s, int planes_lo, int planes_hi, LstmPlan *plan) {
    if (s->B <= 0 || s->H <= 0 || s->H % 16 || s->Kc % 64 || s->Kc > 64 * kLstmMaxKB ||
        s->k_lo % 64 || s->k_lo < 0 || s->k_lo > s->Kc)
        return (int)cudaErrorInvalidValue;
    plan->units = pick_units(s->B, s->H);
    if (!plan->units) return (int)cudaErrorInvalidValue;
    int rc;
    const int k_lo = s->k_lo, k_hi = s->Kc - s->k_lo;
    if (k_lo > 0) {
        rc = make_tmap_3d(&plan->tm_a_lo, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, s->a_lo, planes_lo, s->B,
                          k_lo, uint64_t(s->ld_a_lo) * 2, uint64_t(s->B) * s->ld_a_lo * 2, 128, 64, true);
        if (rc) return rc;
    }
    if (k_hi > 0) {
        rc = make_tmap_3d(&plan->tm_a_hi, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, s->a_hi, planes_hi, s->B,
                          k_hi, uint64_t(s->ld_a_hi) * 2, uint64_t(s->B) * s->ld_a_hi * 2, 128, 64, true);
        if (rc) return rc;
    } else {
        plan->tm_a_hi = plan->tm_a_lo;
    }
    if (k_lo == 0) plan->tm_a_lo = plan->tm_a_hi;
    for (int g = 0; g < 4; ++g) {
        rc = make_tmap_2d(&plan->tm_w[g], CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, s->w[g], s->H, s->Kc,
                          uint64_t(s->ld_w) * 2, plan->units, 64, true);
        if (rc) return rc;
    }
    LstmDev &p = plan->p;
    p.B = s->B; p.H = s->H;
    p.nkb = s->Kc / 64; p.nkb_lo = k_lo / 64;
    p.plane_lo = 0; p.plane_hi = 0;
    for (int g = 0; g < 4; ++g) p.bias[g] = s->bias[g];
    p.c = s->c; p.h_out = s->h_out;
    plan->grid = dim3((s->B + 127) / 128, s->H / plan->units, 1);
    return 0;
}

template <int UNITS>
int lstm_launch_units(const LstmPlan &plan, const LstmDev &p, cudaStream_t stream) {
    auto kernel = lstm_step_kernel<UNITS>;
    static bool done[64] = {false};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) dev = 0;
    if (!done[dev]) {
        cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             LstmSmem<UNITS>::kDynamic);
        if (e != cudaSuccess) return (int)e;
        done[dev] = true;
    }
    kernel<<<plan.grid, kLstmThreads, LstmSmem<UNITS>::kDynamic, stream>>>(
        plan.tm_a_lo, plan.tm_a_hi, plan.tm_w[0], plan.tm_w[1], plan.tm_w[2], plan.tm_w[3], p);
    return (int)cudaGetLastError();
}

int lstm_plan_launch(const LstmPlan &plan, int plane_lo, int plane_hi, int8_t *h_out,
                     cudaStream_t stream) {
    LstmDev p = plan.p;
    p.plane_lo = plane_lo; p.plane_hi = plane_hi; p.h_out = h_out;
    switch (plan.units) {
        case 64: return lstm_launch_units<64>(plan, p, stream);
        case 48: return lstm_launch_units<48>(plan, p, stream);
        case 32: return lstm_launch_units<32>(plan, p, stream);
        case 16: return lstm_launch_units<16>(plan, p, stream);
        default: return (int)cudaErrorInvalidValue;
    }
}

}  // namespace
}  // namespace fluke_sm100

extern "C" int fluke_sm100_lstm_step(const fluke_sm100_lstm_step_t *s, void *stream) {
    using namespace fluke_sm100;
    if (!s) return (int)cudaErrorInvalidValue;
    LstmPlan plan;
    int rc = lstm_plan_build(s, 1, 1, &plan);
    if (rc) return rc;
    return lstm_plan_launch(plan, 0, 0, s->h_out, static_cast<cudaStream_t>(stream));
}

// ---- whole layer --------------------------------------------------------------------------------

extern "C" int fluke_sm100_lstm_layer_persistent(const void *layer, const void *x_down, void *hh_down,
                                                 void *flags, void *stream);
extern "C" int fluke_sm100_lstm_layer_cluster(const void *layer, const void *x_down, int allow_waves,
                                              void *stream);
// Form selection (see fluke_sm100_set_lstm_persistent in fluke_sm100.h) and the form the last
// whole-layer call used: 0 per step, 1 cluster, 2 L2 exchange. Both are kept per host thread: a
// process that drives several GPUs from several threads sets and reads its own.
static thread_local int g_lstm_last_form = -1;
extern "C" int fluke_sm100_lstm_last_form(void) { return g_lstm_last_form; }
static thread_local int g_lstm_persistent = 1;
extern "C" void fluke_sm100_set_lstm_persistent(int mode) { g_lstm_persistent = (mode == 0 || mode == 2 || mode == 4) ? mode : 1; }

static size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Workspace layout: hh_down f16 [B,R] | x_down f16 [T,B,R] | 1 KB of exchange counters.
static size_t lstm_ws_off_flags(int T, int B, int R) {
    return align_up(size_t(B) * R * 2, 1024) + align_up(size_t(T) * B * R * 2, 1024);
}

extern "C" size_t fluke_sm100_lstm_layer_workspace(int T, int B, int H, int R) {
    (void)H;
    if (T <= 0 || B <= 0 || R <= 0) return 0;
    return lstm_ws_off_flags(T, B, R) + 1024;
}

// phase_mask selects which kernel classes are launched: 1 = x_down GEMM, 2 = per-step
// down-projection, 4 = per-step fused step. 7 is the layer; other masks exist so a benchmark
// can time one kernel class alone (their outputs are not a valid layer result).
extern "C" int fluke_sm100_lstm_layer_phases(const void *layer, int phase_mask, void *stream_) {
    using namespace fluke_sm100;
    const fluke_flstm_layer_t *l = static_cast<const fluke_flstm_layer_t *>(layer);
    cudaStream_t stream = static_cast<cudaStream_t>(stream_);
    if (!l || l->T <= 0 || l->B <= 0 || l->H <= 0 || l->R <= 0) return (int)cudaErrorInvalidValue;
    const int T = l->T, B = l->B, H = l->H, R = l->R;
    if (H % 64 || R % 64 || 2 * R > 64 * kLstmMaxKB) return (int)cudaErrorInvalidValue;
    if (!l->x_i8 || !l->dn_ih_i8 || !l->dn_ih_scale || !l->dn_hh_i8 || !l->dn_hh_scale ||
        !l->w_up_f16 || !l->bias_f32 || !l->c_f32 || !l->h_i8 || !l->h_out_i8 || !l->workspace)
        return (int)cudaErrorInvalidValue;
    if (l->workspace_bytes < fluke_sm100_lstm_layer_workspace(T, B, H, R))
        return (int)cudaErrorInvalidValue;

    uint8_t *ws = static_cast<uint8_t *>(l->workspace);
    __half *hh_down = reinterpret_cast<__half *>(ws);
    __half *x_down = reinterpret_cast<__half *>(ws + align_up(size_t(B) * R * 2, 1024));
    const float kHScale = 1.0f / 127.0f;
    int rc;

    // 1. x_down[t] = down_proj(x[t], dn_ih) for every timestep, as one GEMM with M = T*B.
    if (phase_mask & 1) {
        fluke_sm100_gemm_t g = {};
        g.kind = FLUKE_SM100_KIND_I8; g.epilogue = FLUKE_SM100_EPI_DEQUANT;
        g.M = T * B; g.N = R; g.K = H;
        g.a = l->x_i8; g.b = l->dn_ih_i8; g.out = x_down; g.ld_out = R;
        g.scale_a = static_cast<const float *>(l->x_scale); g.const_scale_a = kHScale;
        g.scale_b = static_cast<const float *>(l->dn_ih_scale);
        rc = launch<kKindI8, FLUKE_SM100_EPI_DEQUANT, kPlainBN, kPlainStages>(&g, stream);
        if (rc) return rc;
    }

    // 2. the recurrence in one launch where a single-launch form covers the shape. Order of
    //    preference per mode; a form answers -2 when it does not cover the shape.
    if (phase_mask == 7 && g_lstm_persistent) {
        uint8_t *flags = ws + lstm_ws_off_flags(T, B, R);
        auto run_form = [&](int form) -> int {
            switch (form) {
                case 1: return fluke_sm100_lstm_layer_cluster(l, x_down, 0, stream);   // all tiles at once only
                case 5: return fluke_sm100_lstm_layer_cluster(l, x_down, 1, stream);   // in rounds if need be
                case 2: return fluke_sm100_lstm_layer_persistent(l, x_down, hh_down, flags, stream);
                default: return -2;
            }
        };
        int order[4] = {0, 0, 0, 0};
        switch (g_lstm_persistent) {
            case 2: order[0] = 2; break;
            case 4: order[0] = 5; order[1] = 2; break;
            default: order[0] = 1; order[1] = 2; order[2] = 5; break;
        }
        rc = -2;
        for (int i = 0; i < 4 && rc == -2 && order[i]; ++i) {
            rc = run_form(order[i]);
            g_lstm_last_form = order[i] == 5 ? 1 : order[i];
        }
        if (rc == 0) {
            const int t_last = l->reverse ? 0 : T - 1;
            return (int)cudaMemcpyAsync(l->h_i8, static_cast<int8_t *>(l->h_out_i8) + size_t(t_last) * B * H,
                                        size_t(B) * H, cudaMemcpyDeviceToDevice, stream);
        }
        if (rc != -2) return rc;
    }

    if (phase_mask == 7) g_lstm_last_form = 0;
    // 3. otherwise: plans of the per-step kernels (tensor maps built once; t is a plane coordinate)
    GemmPlan dp_first, dp_rest;
    {
        fluke_sm100_gemm_t g = {};
        g.kind = FLUKE_SM100_KIND_I8; g.epilogue = FLUKE_SM100_EPI_DEQUANT;
        g.M = B; g.N = R; g.K = H;
        g.b = l->dn_hh_i8; g.out = hh_down; g.ld_out = R;
        g.scale_a = nullptr; g.const_scale_a = kHScale;
        g.scale_b = static_cast<const float *>(l->dn_hh_scale);
        g.a = l->h_i8;
        rc = plan_build<kKindI8, FLUKE_SM100_EPI_DEQUANT, kPlainBN, kPlainStages>(&g, 1, &dp_first);
        if (rc) return rc;
        g.a = l->h_out_i8;
        rc = plan_build<kKindI8, FLUKE_SM100_EPI_DEQUANT, kPlainBN, kPlainStages>(&g, T, &dp_rest);
        if (rc) return rc;
    }
    LstmPlan step;
    {
        fluke_sm100_lstm_step_t s = {};
        s.B = B; s.H = H; s.Kc = 2 * R;
        s.a_lo = hh_down; s.ld_a_lo = R; s.k_lo = R;
        s.a_hi = x_down; s.ld_a_hi = R;
        for (int g = 0; g < 4; ++g) {
            s.w[g] = static_cast<const __half *>(l->w_up_f16) + size_t(g) * H * 2 * R;
            s.bias[g] = static_cast<const float *>(l->bias_f32) + size_t(g) * H;
        }
        s.ld_w = 2 * R;
        s.c = static_cast<float *>(l->c_f32);
        s.h_out = static_cast<int8_t *>(l->h_out_i8);
        rc = lstm_plan_build(&s, 1, T, &step);
        if (rc) return rc;
    }

    // 4. the recurrence, two launches per timestep
    int8_t *h_out = static_cast<int8_t *>(l->h_out_i8);
    int t_prev = -1;
    for (int i = 0; i < T; ++i) {
        const int t = l->reverse ? T - 1 - i : i;
        rc = 0;
        if (!(phase_mask & 2)) {
        } else if (i == 0) {
            rc = plan_launch<kKindI8, FLUKE_SM100_EPI_DEQUANT, kPlainBN, kPlainStages>(dp_first, 0, stream);
        } else {
            rc = plan_launch<kKindI8, FLUKE_SM100_EPI_DEQUANT, kPlainBN, kPlainStages>(dp_rest, t_prev, stream);
        }
        if (rc) return rc;
        if (phase_mask & 4) rc = lstm_plan_launch(step, 0, t, h_out + size_t(t) * B * H, stream);
        if (rc) return rc;
        t_prev = t;
    }
    // 5. final hidden state
    return (int)cudaMemcpyAsync(l->h_i8, h_out + size_t(t_prev) * B * H, size_t(B) * H,
                                cudaMemcpyDeviceToDevice, stream);
}

extern "C" int fluke_sm100_lstm_layer(const void *layer, void *stream) {
    return fluke_sm100_lstm_layer_phases(layer, 7, stream);
}
