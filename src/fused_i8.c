/* fused_i8.c -- selection and dispatch of the fused int8 transformer kernels (reference:
 * src/fused_cuda.c:31-111 with its per-arch vtable src/i8_ops.h:23-30 and src/i8_arch.c).
 * The compute-capability table has one row, 10.0 -> the tcgen05 kernels; there is no module
 * to load, so select only checks the device and the dims. One backend object per device. */
#include <fluke/fluke.h>

#include <stddef.h>
#include <stdio.h>

#include "fused_dims.h"
#include "gpu_common.h"

struct fluke_i8_ops {
    int (*qkv_rotary)(void *out, const void *a_i8, const void *wqkv_i8, const void *scale_a,
                      const void *scale_b, const void *sin, const void *cos, int M, int seqlen);
    int (*gated_mlp)(void *out, const void *a_i8, const void *gate_i8, const void *up_i8,
                     const void *scale_a, const void *scale_gate, const void *scale_up, int M);
};

static int sm100_qkv_rotary(void *out, const void *a_i8, const void *wqkv_i8, const void *scale_a,
                            const void *scale_b, const void *sin, const void *cos, int M,
                            int seqlen) {
    fluke_sm100_gemm_t g = {0};
    g.kind = FLUKE_SM100_KIND_I8;
    g.epilogue = FLUKE_SM100_EPI_ROTARY;
    g.M = M; g.N = 3 * FLUKE_SUP_D_MODEL; g.K = FLUKE_SUP_D_MODEL;
    g.a = a_i8; g.b = wqkv_i8; g.out = out; g.ld_out = g.N;
    g.scale_a = (const float *)scale_a; g.scale_b = (const float *)scale_b;
    g.sin_tab = (const float *)sin; g.cos_tab = (const float *)cos;
    g.seqlen = seqlen;
    g.qk_cols = 2 * FLUKE_SUP_NHEAD * FLUKE_SUP_HEAD_DIM;
    return fluke_host_note_error(fluke_sm100_gemm(&g, fluke_host_stream()));
}

static int sm100_gated_mlp(void *out, const void *a_i8, const void *gate_i8, const void *up_i8,
                           const void *scale_a, const void *scale_gate, const void *scale_up,
                           int M) {
    fluke_sm100_gemm_t g = {0};
    g.kind = FLUKE_SM100_KIND_I8;
    g.epilogue = FLUKE_SM100_EPI_SILU;
    g.M = M; g.N = FLUKE_SUP_DIM_FF; g.K = FLUKE_SUP_D_MODEL;
    g.a = a_i8; g.b = gate_i8; g.b2 = up_i8; g.out = out; g.ld_out = g.N;
    g.scale_a = (const float *)scale_a;
    g.scale_b = (const float *)scale_gate; g.scale_b2 = (const float *)scale_up;
    return fluke_host_note_error(fluke_sm100_gemm(&g, fluke_host_stream()));
}

static const struct fluke_i8_ops g_ops_sm100 = {sm100_qkv_rotary, sm100_gated_mlp};

static const struct { int cc; const struct fluke_i8_ops *ops; } g_archs[] = {
    {100, &g_ops_sm100},
};

struct fluke_int8_backend {
    fluke_dims_t dims;
    int cc;
    const struct fluke_i8_ops *ops;
};

#define FLUKE_MAX_DEVICES 64
static struct fluke_int8_backend g_backends[FLUKE_MAX_DEVICES];
static int g_announced[FLUKE_MAX_DEVICES];

int fluke_dims_supported(fluke_dims_t d) {
    return d.d_model == FLUKE_SUP_D_MODEL && d.dim_feedforward == FLUKE_SUP_DIM_FF &&
           d.nhead == FLUKE_SUP_NHEAD && d.head_dim == FLUKE_SUP_HEAD_DIM;
}

fluke_int8_backend_t *fluke_int8_select(int device_index, fluke_dims_t dims) {
    const struct fluke_i8_ops *ops = NULL;
    size_t i;
    int cc;
    if (device_index < 0 || device_index >= FLUKE_MAX_DEVICES) return NULL;
    cc = fluke_sm100_compute_capability(device_index);
    if (cc < 0) return NULL;
    for (i = 0; i < sizeof(g_archs) / sizeof(g_archs[0]); ++i)
        if (g_archs[i].cc == cc) ops = g_archs[i].ops;
    if (!ops) {
        fprintf(stderr, "[fluke] no int8 backend for compute capability %d.%d — using fp16\n",
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
        fprintf(stderr, "[fluke] int8 kernel backend active on device %d (sm_%d)\n", device_index, cc);
    }
    g_backends[device_index].dims = dims;
    g_backends[device_index].cc = cc;
    g_backends[device_index].ops = ops;
    return &g_backends[device_index];
}

fluke_dims_t fluke_int8_dims(const fluke_int8_backend_t *b) { return b->dims; }

int fluke_qkv_rotary_i8_gpu(const fluke_int8_backend_t *b, void *out, const void *a_i8,
                            const void *wqkv_i8, const void *scale_a, const void *scale_b,
                            const void *sin, const void *cos, int M, int seqlen) {
    if (!b || !b->ops) return -1;
    return b->ops->qkv_rotary(out, a_i8, wqkv_i8, scale_a, scale_b, sin, cos, M, seqlen);
}

int fluke_gated_mlp_i8_gpu(const fluke_int8_backend_t *b, void *out, const void *a_i8,
                           const void *gate_i8, const void *up_i8, const void *scale_a,
                           const void *scale_gate, const void *scale_up, int M) {
    if (!b || !b->ops) return -1;
    return b->ops->gated_mlp(out, a_i8, gate_i8, up_i8, scale_a, scale_gate, scale_up, M);
}

/* ---- additive base GEMMs -------------------------------------------------------------- */

int fluke_gemm_i8_gpu(void *out_f16, const void *a_i8, const void *b_i8, const void *scale_a,
                      float const_scale_a, const void *scale_b, int M, int N, int K) {
    fluke_sm100_gemm_t g = {0};
    g.kind = FLUKE_SM100_KIND_I8;
    g.epilogue = FLUKE_SM100_EPI_DEQUANT;
    g.M = M; g.N = N; g.K = K;
    g.a = a_i8; g.b = b_i8; g.out = out_f16; g.ld_out = N;
    g.scale_a = (const float *)scale_a; g.const_scale_a = const_scale_a;
    g.scale_b = (const float *)scale_b;
    return fluke_host_note_error(fluke_sm100_gemm(&g, fluke_host_stream()));
}

int fluke_gemm_i8_s32_gpu(void *out_s32, const void *a_i8, const void *b_i8, int M, int N, int K) {
    fluke_sm100_gemm_t g = {0};
    g.kind = FLUKE_SM100_KIND_I8;
    g.epilogue = FLUKE_SM100_EPI_RAW;
    g.M = M; g.N = N; g.K = K;
    g.a = a_i8; g.b = b_i8; g.out = out_s32; g.ld_out = N;
    return fluke_host_note_error(fluke_sm100_gemm(&g, fluke_host_stream()));
}
