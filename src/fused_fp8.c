/* fused_fp8.c -- the fp8 (E4M3, scale amax/448) twins of the fused transformer kernels
 * (reference ABI: include/fluke/fluke.h:251-275; a stub on the reference's CUDA build,
 * src/fused_hip.c:128-147). Here they are real: tcgen05 kind::f8f6f4 with f32 accumulation.
 *
 * The ABI passes weights PRESHUFFLED as [N/16, K/16, 2, 16, 8] bytes, which neither TMA nor a
 * UMMA shared-memory descriptor can address as a K-major operand, so the first call that sees
 * a weight pointer re-orders it once into a private row-major [N, K] device copy; later calls
 * find it in a small pointer-keyed table (fluke_fp8_prepare_weight does that step ahead of time,
 * fluke_fp8_release_weight drops it). The *_plain_gpu variants take row-major weights and
 * allocate nothing. */
#include <fluke/fluke.h>

#include <stddef.h>
#include <stdio.h>

#include "fused_dims.h"
#include "gpu_common.h"

int fluke_dims_supported(fluke_dims_t d); /* fused_i8.c */

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
/* Keyed by (device, pointer, N, K). The library cannot see a caller free or overwrite a weight, so
 * the contract is pointer identity: a caller that re-uses a weight address for other contents
 * calls fluke_fp8_release_weight first. The table is guarded by a mutex; when it is full the
 * oldest entry is dropped (its copy is freed after the device has finished with it; a process
 * that keeps more than 64 fp8 weights live and calls from several threads should use the
 * *_plain_gpu entry points, since a copy handed to one thread's call can then be dropped by
 * another thread's). */

#include <pthread.h>

#define FLUKE_FP8_CACHE_SLOTS 64
static struct { const void *src; int dev, N, K; void *plain; unsigned long age; } g_wcache[FLUKE_FP8_CACHE_SLOTS];
static unsigned long g_wcache_clock = 0;
static pthread_mutex_t g_wcache_lock = PTHREAD_MUTEX_INITIALIZER;

/* Hooks the CPU tests replace to exercise the table without a GPU. */
static int (*g_hook_malloc)(void **, size_t) = fluke_sm100_malloc;
static int (*g_hook_free)(void *) = fluke_sm100_free;
static int (*g_hook_unshuffle)(void *, const void *, int, int, void *) = fluke_sm100_fp8_unshuffle;
static int (*g_hook_device)(void) = fluke_sm100_current_device;
void fluke_fp8_cache_test_hooks(int (*m)(void **, size_t), int (*f)(void *),
                                int (*u)(void *, const void *, int, int, void *), int (*d)(void)) {
    g_hook_malloc = m ? m : fluke_sm100_malloc;
    g_hook_free = f ? f : fluke_sm100_free;
    g_hook_unshuffle = u ? u : fluke_sm100_fp8_unshuffle;
    g_hook_device = d ? d : fluke_sm100_current_device;
}

static const void *plain_weight(const void *preshuffled, int N, int K) {
    int i, slot = -1, dev;
    void *dst = NULL;
    const void *found = NULL;
    if (!preshuffled) return NULL;
    dev = g_hook_device();
    pthread_mutex_lock(&g_wcache_lock);
    for (i = 0; i < FLUKE_FP8_CACHE_SLOTS; ++i)
        if (g_wcache[i].plain && g_wcache[i].src == preshuffled && g_wcache[i].dev == dev &&
            g_wcache[i].N == N && g_wcache[i].K == K) {
            found = g_wcache[i].plain;
            break;
        }
    if (!found) {
        /* a free slot, else the oldest entry */
        for (i = 0; i < FLUKE_FP8_CACHE_SLOTS; ++i) {
            if (!g_wcache[i].plain) { slot = i; break; }
            if (slot < 0 || g_wcache[i].age < g_wcache[slot].age) slot = i;
        }
        if (fluke_host_note_error(g_hook_malloc(&dst, (size_t)N * K)) == 0) {
            if (fluke_host_note_error(g_hook_unshuffle(dst, preshuffled, N, K, fluke_host_stream())) == 0) {
                if (g_wcache[slot].plain) g_hook_free(g_wcache[slot].plain);
                g_wcache[slot].src = preshuffled;
                g_wcache[slot].dev = dev;
                g_wcache[slot].N = N;
                g_wcache[slot].K = K;
                g_wcache[slot].plain = dst;
                g_wcache[slot].age = ++g_wcache_clock;
                found = dst;
            } else {
                g_hook_free(dst);
            }
        }
    }
    pthread_mutex_unlock(&g_wcache_lock);
    return found;
}

int fluke_fp8_prepare_weight(const void *preshuffled, int N, int K) {
    if (N <= 0 || K <= 0 || N % 16 || K % 16) return -1;
    return plain_weight(preshuffled, N, K) ? 0 : -1;
}

int fluke_fp8_release_weight(const void *preshuffled) {
    int i, n = 0;
    pthread_mutex_lock(&g_wcache_lock);
    for (i = 0; i < FLUKE_FP8_CACHE_SLOTS; ++i)
        if (g_wcache[i].plain && (!preshuffled || g_wcache[i].src == preshuffled)) {
            g_hook_free(g_wcache[i].plain);
            g_wcache[i].plain = NULL;
            g_wcache[i].src = NULL;
            ++n;
        }
    pthread_mutex_unlock(&g_wcache_lock);
    return n;
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
