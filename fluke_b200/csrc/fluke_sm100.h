/* fluke_sm100.h -- thin internal C ABI between the pure-C host code in src/ and the
 * sm_100a CUDA translation units in this directory.
 *
 * Every launcher takes raw device pointers, sizes and a stream (cudaStream_t as void*;
 * NULL = legacy default stream), enqueues work without synchronising, and returns 0 or
 * a cudaError_t value (as int). Argument checking that the public ABI promises
 * (exit on bad dims, NULL/-1 on unsupported dims) is done by the callers in src/.
 */
#ifndef FLUKE_SM100_H
#define FLUKE_SM100_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- device / status ------------------------------------------------------------------ */

/* major*10+minor of the device, or -1 when it cannot be queried. */
int fluke_sm100_compute_capability(int device_index);
const char *fluke_sm100_error_string(int code);

/* Device-side status word. Kernels never spin forever: a wait that exceeds its cycle limit
 * records FLUKE_SM100_STATUS_TIMEOUT | (site << 8) here and the kernel drains and returns.
 * Reading synchronises the device; `reset` != 0 clears the word after reading. */
#define FLUKE_SM100_STATUS_OK 0u
#define FLUKE_SM100_STATUS_TIMEOUT 1u
int fluke_sm100_read_status(unsigned int *status_out, int reset);

/* Device allocation for the one place the library keeps private memory (the re-ordered fp8
 * weight copies). */
int fluke_sm100_malloc(void **ptr, size_t bytes);
int fluke_sm100_free(void *ptr);
/* Index of the calling thread's current device, -1 when it cannot be queried. */
int fluke_sm100_current_device(void);

/* ---- memory-bound row kernels (bit-compatible with the reference's pure-CUDA kernels) --- */

int fluke_sm100_rmsnorm(const void *in, const void *residual, const void *weight, void *out,
                        int n_tokens, int hidden_dim, float alpha, float eps, void *stream);
int fluke_sm100_rmsnorm_quant_int8(const void *in, const void *weight, void *residual,
                                   void *residual_scale, int n_tokens, int hidden_dim,
                                   float alpha, float eps, void *stream);
int fluke_sm100_rmsnorm_quant_fp8(const void *in, const void *weight, void *residual,
                                  void *residual_scale, int n_tokens, int hidden_dim,
                                  float alpha, float eps, void *stream);
int fluke_sm100_quant_int8(const void *in, void *out, void *scale, int n_tokens, int hidden_dim,
                           void *stream);
int fluke_sm100_quant_fp8(const void *in, void *out, void *scale, int n_tokens, int hidden_dim,
                          void *stream);
int fluke_sm100_dequant_transpose(const void *in, void *out, int n_timesteps, int batch_size,
                                  int n_channels, float scale, int is_fp8, void *stream);
int fluke_sm100_rotary_emb(void *x, const void *sin_tab, const void *cos_tab, int batch_size,
                           int seq_len, int n_heads, int head_dim, int sincos_width,
                           long long stride_batch, long long stride_seq, long long stride_head,
                           void *stream);
int fluke_sm100_silu_mul(const void *in, void *out, int n_tokens, int hidden_dim, void *stream);
int fluke_sm100_flstm_step(const void *scratch, const void *ih_t, void *cell, void *hh_next,
                           int batch_size, int hidden_dim, void *stream);
int fluke_sm100_fp8_unshuffle(void *dst_nk, const void *src, int N, int K, void *stream);

/* tcgen05.mma issue-rate probe (lib/libfluke_probe.so, not libfluke): n_ctas CTAs each time
 * `iters` back-to-back MMAs of shape 128 x n x 32 bytes (kind 0 int8, 1 e4m3, 2 f16) on
 * shared-memory-resident operands (pattern 0: zeros, 1: pseudo-random bytes) and write, per CTA,
 * their SM-clock cycles and nanoseconds to cycles_dev[0 .. 2 n_ctas) (device, int64). */
int fluke_sm100_mma_peak(int kind, int n, int iters, int pattern, void *cycles_dev, int n_ctas, void *stream);
/* Same library: one thread records n pairs (SM cycle counter, nanosecond timer) gap_ns apart into
 * out_dev (device, int64), so that the clock of kernels running beside it can be read. */
int fluke_sm100_clock_samples(void *out_dev, int n, int gap_ns, void *stream);
/* Strided copy between pinned host memory and the device by the copy engine alone (no staging
 * buffer, no kernel): `height` rows of `width` bytes, pitches in bytes. to_device != 0: host ->
 * device, else device -> host. For drivers that place a batch beside another one in a wider
 * device tensor. */
int fluke_sm100_copy_rows_async(void *dst, size_t dst_pitch, const void *src, size_t src_pitch,
                                size_t width, size_t height, int to_device, void *stream);

/* ---- tcgen05 GEMM family ---------------------------------------------------------------- */

enum fluke_sm100_kind {
    FLUKE_SM100_KIND_I8 = 0,  /* int8 x int8 -> int32  (tcgen05 kind::i8)      */
    FLUKE_SM100_KIND_F8 = 1   /* e4m3 x e4m3 -> f32    (tcgen05 kind::f8f6f4)  */
};

enum fluke_sm100_epilogue {
    FLUKE_SM100_EPI_RAW = 0,      /* out 32-bit accumulators (int32 or f32)                    */
    FLUKE_SM100_EPI_DEQUANT = 1,  /* out f16 = acc * (sa[m]*sb[n])                             */
    FLUKE_SM100_EPI_DEQUANT2 = 2, /* out f16 = (acc * sa[m]) * sb[n]                           */
    FLUKE_SM100_EPI_ROTARY = 3,   /* DEQUANT2, then rotate-half on the Q and K heads           */
    FLUKE_SM100_EPI_SILU = 4      /* two weights: out f16 = g*sigmoid(g)*u, both DEQUANT2      */
};

typedef struct {
    int kind;               /* enum fluke_sm100_kind     */
    int epilogue;           /* enum fluke_sm100_epilogue */
    int M, N, K;            /* out [M,N]; a [M,K]; b (and b2) [N,K]; all row-major          */
    const void *a;
    const void *b;
    const void *b2;         /* second weight (SILU only)                                     */
    void *out;
    int ld_out;             /* row stride of out in elements                                 */
    const float *scale_a;   /* f32 [M] or NULL -> const_scale_a                              */
    float const_scale_a;
    const float *scale_b;   /* f32 [N]                                                       */
    const float *scale_b2;  /* f32 [N] (SILU only)                                           */
    const float *sin_tab;   /* ROTARY: f32 [seqlen, head_dim/2]                              */
    const float *cos_tab;
    int seqlen;             /* ROTARY: position = m % seqlen                                 */
    int qk_cols;            /* ROTARY: columns [0, qk_cols) are rotated, in heads of 64      */
} fluke_sm100_gemm_t;

int fluke_sm100_gemm(const fluke_sm100_gemm_t *g, void *stream);

/* ---- factored LSTM ------------------------------------------------------------------------ */

typedef struct {
    int B, H, Kc;                   /* chunks, hidden size, merged contraction length         */
    const void *a_lo;               /* f16 [B, k_lo] first K columns of A (hh_down)           */
    int ld_a_lo;                    /* row stride of a_lo in elements                         */
    const void *a_hi;               /* f16 [B, Kc-k_lo] remaining K columns (x_down)          */
    int ld_a_hi;
    int k_lo;                       /* multiple of 64; Kc when A is one tensor                */
    const void *w[4];               /* f16 [H, Kc] per gate i,f,g,o, row stride ld_w          */
    int ld_w;
    const float *bias[4];           /* f32 [H] per gate                                       */
    float *c;                       /* f32 [B,H] in/out                                       */
    int8_t *h_out;                  /* int8 [B,H]                                             */
} fluke_sm100_lstm_step_t;

int fluke_sm100_lstm_step(const fluke_sm100_lstm_step_t *s, void *stream);

/* Whole layer (x_down GEMM, then per timestep down-projection + fused step). The argument is
 * the public fluke_flstm_layer_t of <fluke/fluke.h>. */
size_t fluke_sm100_lstm_layer_workspace(int T, int B, int H, int R);
int fluke_sm100_lstm_layer(const void *layer /* const fluke_flstm_layer_t* */, void *stream);
/* Launch only some kernel classes of the layer: 1 = x_down GEMM, 2 = per-step down-projection,
 * 4 = per-step fused step (7 = the layer). For timing one class alone. */
int fluke_sm100_lstm_layer_phases(const void *layer, int phase_mask, void *stream);
/* How the recurrence of a layer is run (a per-host-thread setting).
 * 1 (default): one launch, the fastest single-launch form the shape and the device allow: the
 *    cluster form while all row tiles of the layer run at once, else the L2-exchange form, else the
 *    cluster form in rounds;
 * 2: the L2-exchange form only (separate projection CTAs; R = 128, H a multiple of 128 up to 1024);
 * 4: the cluster form only, in rounds when the layer has more row tiles than clusters fit
 *    (exchange inside thread-block clusters; R = 128, H a multiple of 64 up to 768);
 * 0: two launches per timestep.
 * A form that does not cover the shape falls back to the next one that does. */
void fluke_sm100_set_lstm_persistent(int mode);
/* Configuration of the L2-exchange form. Narrow: 24 or 32 hidden units per gate CTA, two workers
 * per row tile (8 row tiles per launch on 148 SMs at H = 768). Wide: 48 units per gate CTA, one
 * worker per row tile, for H = 384 or 768: 16 row tiles per launch, a step about 15 % longer.
 * -1 (default): wide when the layer has more row tiles than a narrow launch holds; 0: never;
 * 1: whenever the shape allows it. */
void fluke_sm100_set_lstm_wide(int mode);
/* Which form the last whole-layer call used: 1 cluster exchange, 2 L2 exchange, 0 per step. */
int fluke_sm100_lstm_last_form(void);
/* Row tiles (clusters) of the cluster form that run at once for hidden size H; 0 = unavailable. */
int fluke_sm100_lstm_cluster_capacity(int H);

#ifdef __cplusplus
}
#endif

#endif /* FLUKE_SM100_H */
