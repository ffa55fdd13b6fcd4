/* nn_cpu.c -- fp32 CPU implementations of the three always-exported layer functions.
 *
 * Same results, element for element, as the reference's src/nn_cpu.c (rotary :10-39 and
 * :80-131, rmsnorm :145-208, flstm step :210-285): identical scalar expressions and, for
 * the RMSNorm sum of squares, the identical left-to-right accumulation order. Work is cut
 * into contiguous slices of the outermost index (batch / token / chunk) across at most
 * n_threads pthreads, as in the reference; the rotary loop nest here walks memory in
 * address order (seq, head, pair innermost) instead of striding by stride_seq.
 * Built with -ffp-contract=off so no product is fused into an FMA.
 */
#include "error.h"

#include <fluke/fluke.h>

#include <math.h>
#include <pthread.h>
#include <stdint.h>

/* ---- slice-parallel driver ---------------------------------------------------------- */

typedef void (*slice_fn)(const void *op, int64_t begin, int64_t end);

typedef struct {
    slice_fn fn;
    const void *op;
    int64_t begin, end;
} slice_job_t;

static void *slice_trampoline(void *p) {
    const slice_job_t *job = (const slice_job_t *)p;
    job->fn(job->op, job->begin, job->end);
    return NULL;
}

/* Runs fn over [0, n) split into min(n, n_threads) contiguous slices whose lengths differ
 * by at most one (the first n % workers slices are the longer ones). */
static void run_sliced(slice_fn fn, const void *op, int64_t n, int n_threads) {
    if (n <= 0) return;
    int workers = n_threads < 1 ? 1 : n_threads;
    if ((int64_t)workers > n) workers = (int)n;

    pthread_t tid[workers];
    slice_job_t job[workers];
    const int64_t base = n / workers, extra = n % workers;
    int64_t at = 0;
    for (int w = 0; w < workers; ++w) {
        const int64_t len = base + (w < extra ? 1 : 0);
        job[w].fn = fn;
        job[w].op = op;
        job[w].begin = at;
        job[w].end = at + len;
        at += len;
    }
    FLUKE_LOG_TRACE("dispatching %d threads", workers);
    for (int w = 0; w < workers; ++w) {
        int rc = pthread_create(&tid[w], NULL, slice_trampoline, &job[w]);
        NEG_CHK(-rc);
    }
    for (int w = 0; w < workers; ++w) {
        int rc = pthread_join(tid[w], NULL);
        NEG_CHK(-rc);
    }
}

/* ---- rotary embedding ---------------------------------------------------------------- */

typedef struct {
    float *x;
    const float *sin_tab, *cos_tab;
    int64_t seq_len, n_heads, width;
    int64_t stride_batch, stride_seq, stride_head;
} rotary_op_t;

static void rotary_slice(const void *p, int64_t b0, int64_t b1) {
    const rotary_op_t *op = (const rotary_op_t *)p;
    const int64_t W = op->width;
    for (int64_t b = b0; b < b1; ++b) {
        for (int64_t s = 0; s < op->seq_len; ++s) {
            const float *cs = op->cos_tab + s * W;
            const float *sn = op->sin_tab + s * W;
            float *row = op->x + b * op->stride_batch + s * op->stride_seq;
            for (int64_t h = 0; h < op->n_heads; ++h) {
                float *lo = row + h * op->stride_head;
                float *hi = lo + W;
                for (int64_t i = 0; i < W; ++i) {
                    const float x0 = lo[i], x1 = hi[i];
                    lo[i] = x0 * cs[i] - x1 * sn[i];
                    hi[i] = x0 * sn[i] + x1 * cs[i];
                }
            }
        }
    }
}

void fluke_rotary_emb_cpu(void *x, const void *sin_buf, const void *cos_buf, int batch_size,
                          int seq_len, int n_heads, int head_dim, int sincos_width,
                          int stride_batch, int stride_seq, int stride_head, int n_threads) {
    (void)head_dim;
    rotary_op_t op = {(float *)x,   (const float *)sin_buf, (const float *)cos_buf,
                      seq_len,      n_heads,                sincos_width,
                      stride_batch, stride_seq,             stride_head};
    run_sliced(rotary_slice, &op, batch_size, n_threads);
}

/* ---- RMSNorm --------------------------------------------------------------------------- */

typedef struct {
    const float *in, *residual, *weight;
    float *out;
    int hidden;
    float alpha, eps;
} rmsnorm_op_t;

static void rmsnorm_slice(const void *p, int64_t r0, int64_t r1) {
    const rmsnorm_op_t *op = (const rmsnorm_op_t *)p;
    const int H = op->hidden;
    for (int64_t r = r0; r < r1; ++r) {
        const float *in = op->in + r * H, *res = op->residual + r * H;
        float *out = op->out + r * H;
        float sum_sq = 0.0f;
        for (int j = 0; j < H; ++j) {
            const float v = in[j] + op->alpha * res[j];
            sum_sq += v * v;
        }
        const float rms_inv = 1.0f / sqrtf(sum_sq / H + op->eps);
        for (int j = 0; j < H; ++j) {
            const float v = in[j] + op->alpha * res[j];
            out[j] = v * rms_inv * op->weight[j];
        }
    }
}

void fluke_rmsnorm_cpu(void *in, const void *residual, const void *weight, void *out,
                       int n_tokens, int hidden_dim, float alpha, float eps, int n_threads) {
    rmsnorm_op_t op = {(const float *)in, (const float *)residual, (const float *)weight,
                       (float *)out,      hidden_dim,              alpha,
                       eps};
    run_sliced(rmsnorm_slice, &op, n_tokens, n_threads);
}

/* ---- LSTM gate epilogue ------------------------------------------------------------------ */

typedef struct {
    const float *scratch, *ih_t;
    float *cell, *hh_next;
    int hidden;
} flstm_op_t;

static inline float clampf(float v, float lo, float hi) { return v < lo ? lo : (v > hi ? hi : v); }

static void flstm_slice(const void *p, int64_t n0, int64_t n1) {
    const flstm_op_t *op = (const flstm_op_t *)p;
    const int H = op->hidden;
    for (int64_t n = n0; n < n1; ++n) {
        const float *a = op->scratch + n * 4 * H, *b = op->ih_t + n * 4 * H;
        float *cell = op->cell + n * H, *hh = op->hh_next + n * H;
        for (int ch = 0; ch < H; ++ch) {
            const float gi = a[ch] + b[ch];
            const float gf = a[H + ch] + b[H + ch];
            const float gg = a[2 * H + ch] + b[2 * H + ch];
            const float go = a[3 * H + ch] + b[3 * H + ch];
            const float i_g = clampf(gi * 0.2f + 0.5f, 0.f, 1.f);
            const float f_g = clampf(gf * 0.2f + 0.5f, 0.f, 1.f);
            const float g_g = clampf(gg, -1.f, 1.f);
            const float o_g = clampf(go * 0.2f + 0.5f, 0.f, 1.f);
            const float c_new = f_g * cell[ch] + i_g * g_g;
            cell[ch] = c_new;
            hh[ch] = o_g * tanhf(c_new);
        }
    }
}

void fluke_flstm_step_cpu(const void *scratch, const void *ih_t, void *cell, void *hh_next,
                          int batch_size, int hidden_dim, int n_threads) {
    flstm_op_t op = {(const float *)scratch, (const float *)ih_t, (float *)cell, (float *)hh_next,
                     hidden_dim};
    run_sliced(flstm_slice, &op, batch_size, n_threads);
}
