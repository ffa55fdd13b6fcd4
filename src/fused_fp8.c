/* fused_fp8.c -- the fp8 (E4M3, scale amax/448) twins of the fused transformer kernels
 * (reference ABI: include/fluke/fluke.h:251-275; a stub on the reference's CUDA build,
 * src/fused_hip.c:128-147). Here they are real: tcgen05 kind::f8f6f4 with f32 accumulation.
 *
 * The ABI passes weights PRESHUFFLED as [N/16, K/16, 2, 16, 8] bytes, which neither TMA nor a
 * UMMA shared-memory descriptor can address as a K-major operand, so the first call that sees
 * a weight pointer re-orders it once into a private row-major [N, K] device copy; later calls
 * find it in a small pointer-keyed table. The *_plain_gpu variants take row-major weights and
 * allocate nothing. */
#include <fluke/fluke.h>

#include <stddef.h>
#include <stdio.h>

#include "fused_dims.h"
#include "gpu_common.h"

int fluke_dims_supported(fluke_dims_t d); /* fused_i8.c */

/* device allocation helpers implemented next to the kernels */


struct fluke_fp8_backend {
    fluke_dims_t dims;
    int cc;
};

#define FLUKE_MAX_DEVICES 64
static struct fluke_fp8_backend g_backends[FLUKE_MAX_DEVICES];
static int g_announced[FLUKE_MAX_DEVICES];

fluke_fp8_backend_t *fluke_fp8_select(int device_index, fluke_dims_t dims) {
    int cc;
    if (device_index < 0 || device_index >= FLUKE_MAX_DEVICES) return NULL;
    cc = fluke_sm100_compute_capability(device_index);
    if (cc != 100) {
        if (cc >= 0)
            fprintf(stderr, "[fluke] no fp8 backend for compute capability %d.%d — using fp16\n",
                    cc / 10, cc % 10);
        return NULL;
    }
    if (!fluke_dims_supported(dims)) {
        fprintf(stderr,
                "[fluke] model dims do not match precompiled kernels "
                "(need d_model=%d, dim_feedforward=%d, nhead=%d, head_dim=%d) — using fp16\n",
                FLUKE_SUP_D_MODEL, FLUKE_SUP_DIM_FF, FLUKE_SUP_NHEAD, FLUKE_SUP_HEAD_DIM);
        return NULL;
    }
    if (!g_announced[device_index]) {
        g_announced[device_index] = 1;
        fprintf(stderr, "[fluke] fp8 kernel backend active on device %d (sm_%d)\n", device_index, cc);
    }
    g_backends[device_index].dims = dims;
    g_backends[device_index].cc = cc;
    return &g_backends[device_index];
}

/* ---- re-ordered weight cache -------------------------------------------------------------- */

#define FLUKE_FP8_CACHE_SLOTS 64
static struct { const void *src; int N, K; void *plain; } g_wcache[FLUKE_FP8_CACHE_SLOTS];
static int g_wcache_used = 0;

static const void *plain_weight(const void *preshuffled, int N, int K) {
    int i;
    void *dst = NULL;
    for (i = 0; i < g_wcache_used; ++i)
        if (g_wcache[i].src == preshuffled && g_wcache[i].N == N && g_wcache[i].K == K)
            return g_wcache[i].plain;
    if (g_wcache_used == FLUKE_FP8_CACHE_SLOTS) return NULL;
    if (fluke_host_note_error(fluke_sm100_malloc(&dst, (size_t)N * K)) != 0) return NULL;
    if (fluke_host_note_error(fluke_sm100_fp8_unshuffle(dst, preshuffled, N, K, fluke_host_stream())) != 0)
        return NULL;
    g_wcache[g_wcache_used].src = preshuffled;
    g_wcache[g_wcache_used].N = N;
    g_wcache[g_wcache_used].K = K;
    g_wcache[g_wcache_used].plain = dst;
    ++g_wcache_used;
    return dst;
}

int fluke_fp8_unshuffle_gpu(void *dst_nk, const void *src_preshuffled, int N, int K) {
    return fluke_host_note_error(
        fluke_sm100_fp8_unshuffle(dst_nk, src_preshuffled, N, K, fluke_host_stream()));
}

/* ---- launches ----------------------------------------------------------------------------- */

int fluke_qkv_rotary_fp8_plain_gpu(const fluke_fp8_backend_t *b, void *out, const void *a_fp8,
                                   const void *wqkv_fp8_nk, const void *scale_a,
                                   const void *scale_b, const void *sin, const void *cos, int M,
                                   int seqlen) {
    fluke_sm100_gemm_t g = {0};
    if (!b) return -1;
    g.kind = FLUKE_SM100_KIND_F8;
    g.epilogue = FLUKE_SM100_EPI_ROTARY;
    g.M = M; g.N = 3 * FLUKE_SUP_D_MODEL; g.K = FLUKE_SUP_D_MODEL;
    g.a = a_fp8; g.b = wqkv_fp8_nk; g.out = out; g.ld_out = g.N;
    g.scale_a = (const float *)scale_a; g.scale_b = (const float *)scale_b;
    g.sin_tab = (const float *)sin; g.cos_tab = (const float *)cos;
    g.seqlen = seqlen;
    g.qk_cols = 2 * FLUKE_SUP_NHEAD * FLUKE_SUP_HEAD_DIM;
    return fluke_host_note_error(fluke_sm100_gemm(&g, fluke_host_stream()));
}

int fluke_gated_mlp_fp8_plain_gpu(const fluke_fp8_backend_t *b, void *out, const void *a_fp8,
                                  const void *gate_fp8_nk, const void *up_fp8_nk,
                                  const void *scale_a, const void *scale_gate,
                                  const void *scale_up, int M) {
    fluke_sm100_gemm_t g = {0};
    if (!b) return -1;
    g.kind = FLUKE_SM100_KIND_F8;
    g.epilogue = FLUKE_SM100_EPI_SILU;
    g.M = M; g.N = FLUKE_SUP_DIM_FF; g.K = FLUKE_SUP_D_MODEL;
    g.a = a_fp8; g.b = gate_fp8_nk; g.b2 = up_fp8_nk; g.out = out; g.ld_out = g.N;
    g.scale_a = (const float *)scale_a;
    g.scale_b = (const float *)scale_gate; g.scale_b2 = (const float *)scale_up;
    return fluke_host_note_error(fluke_sm100_gemm(&g, fluke_host_stream()));
}

int fluke_qkv_rotary_fp8_gpu(const fluke_fp8_backend_t *b, void *out, const void *a_fp8,
                             const void *wqkv_fp8, const void *scale_a, const void *scale_b,
                             const void *sin, const void *cos, int M, int seqlen) {
    const void *w;
    if (!b) return -1;
    w = plain_weight(wqkv_fp8, 3 * FLUKE_SUP_D_MODEL, FLUKE_SUP_D_MODEL);
    if (!w) return -1;
    return fluke_qkv_rotary_fp8_plain_gpu(b, out, a_fp8, w, scale_a, scale_b, sin, cos, M, seqlen);
}

int fluke_gated_mlp_fp8_gpu(const fluke_fp8_backend_t *b, void *out, const void *a_fp8,
                            const void *gate_fp8, const void *up_fp8, const void *scale_a,
                            const void *scale_gate, const void *scale_up, int M) {
    const void *wg, *wu;
    if (!b) return -1;
    wg = plain_weight(gate_fp8, FLUKE_SUP_DIM_FF, FLUKE_SUP_D_MODEL);
    wu = plain_weight(up_fp8, FLUKE_SUP_DIM_FF, FLUKE_SUP_D_MODEL);
    if (!wg || !wu) return -1;
    return fluke_gated_mlp_fp8_plain_gpu(b, out, a_fp8, wg, wu, scale_a, scale_gate, scale_up, M);
}

int fluke_gemm_fp8_gpu(void *out_f16, const void *a_fp8, const void *b_fp8, const void *scale_a,
                       const void *scale_b, int M, int N, int K) {
    fluke_sm100_gemm_t g = {0};
    g.kind = FLUKE_SM100_KIND_F8;
    g.epilogue = FLUKE_SM100_EPI_DEQUANT2;
    g.M = M; g.N = N; g.K = K;
    g.a = a_fp8; g.b = b_fp8; g.out = out_f16; g.ld_out = N;
    g.scale_a = (const float *)scale_a; g.scale_b = (const float *)scale_b;
    return fluke_host_note_error(fluke_sm100_gemm(&g, fluke_host_stream()));
}
