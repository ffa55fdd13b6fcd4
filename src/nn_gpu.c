/* nn_gpu.c -- the ten `void fluke_*_gpu` entry points of the C ABI (reference launch
 * wrappers: src/nn_cuda.c:11-204). Pure C: each checks the dimension limits the reference
 * asserts, forwards raw pointers to the sm_100a launcher and exits on a launch error. */
#include <fluke/fluke.h>

#include "error.h"
#include "gpu_common.h"

/* Per host thread: a process that drives several GPUs from one thread each gives every thread
 * its own stream (and reads back its own last error) without racing on shared state. */
static _Thread_local void *g_stream = NULL;
static _Thread_local int g_last_error = 0;

void fluke_set_stream(void *cuda_stream) { g_stream = cuda_stream; }
void *fluke_get_stream(void) { return g_stream; }
void *fluke_host_stream(void) { return g_stream; }

int fluke_host_note_error(int code) {
    if (code != 0) g_last_error = code;
    return code;
}

const char *fluke_last_error(void) {
    return g_last_error ? fluke_sm100_error_string(g_last_error) : "";
}

/* reference src/nn_cuda.c:11-39 */
void fluke_rotary_emb_gpu(void *x, const void *sin_gpu, const void *cos_gpu, int batch_size,
                          int seq_len, int n_heads, int head_dim, int sincos_width,
                          int stride_batch, int stride_seq, int stride_head) {
    FLUKE_CHECK_LAUNCH(fluke_sm100_rotary_emb(x, sin_gpu, cos_gpu, batch_size, seq_len, n_heads,
                                              head_dim, sincos_width, stride_batch, stride_seq,
                                              stride_head, g_stream));
}

/* reference src/nn_cuda.c:41-57 */
void fluke_silu_mul_gpu(const void *in, void *out, int n_tokens, int hidden_dim) {
    FLUKE_CHECK_LAUNCH(fluke_sm100_silu_mul(in, out, n_tokens, hidden_dim, g_stream));
}

/* reference src/nn_cuda.c:59-79 */
void fluke_rmsnorm_gpu(const void *in, const void *residual, const void *weight, void *out,
                       int n_tokens, int hidden_dim, float alpha, float eps) {
    ASSERT(hidden_dim <= 1024);
    ASSERT(hidden_dim % 2 == 0);
    FLUKE_CHECK_LAUNCH(fluke_sm100_rmsnorm(in, residual, weight, out, n_tokens, hidden_dim, alpha,
                                           eps, g_stream));
}

/* reference src/nn_cuda.c:81-101 */
void fluke_rmsnorm_quant_int8_gpu(const void *in, const void *weight, void *residual,
                                  void *residual_scale, int n_tokens, int hidden_dim, float alpha,
                                  float eps) {
    ASSERT(hidden_dim <= 1024);
    ASSERT(hidden_dim % 2 == 0);
    FLUKE_CHECK_LAUNCH(fluke_sm100_rmsnorm_quant_int8(in, weight, residual, residual_scale,
                                                      n_tokens, hidden_dim, alpha, eps, g_stream));
}

/* reference src/nn_cuda.c:103-118 */
void fluke_flstm_step_gpu(const void *scratch, const void *ih_t, void *cell, void *hh_next,
                          int batch_size, int hidden_dim) {
    FLUKE_CHECK_LAUNCH(
        fluke_sm100_flstm_step(scratch, ih_t, cell, hh_next, batch_size, hidden_dim, g_stream));
}

/* reference src/nn_cuda.c:120-140 */
void fluke_rmsnorm_quant_fp8_gpu(const void *in, const void *weight, void *residual,
                                 void *residual_scale, int n_tokens, int hidden_dim, float alpha,
                                 float eps) {
    ASSERT(hidden_dim <= 1024);
    ASSERT(hidden_dim % 2 == 0);
    FLUKE_CHECK_LAUNCH(fluke_sm100_rmsnorm_quant_fp8(in, weight, residual, residual_scale,
                                                     n_tokens, hidden_dim, alpha, eps, g_stream));
}

/* reference src/nn_cuda.c:142-156 */
void fluke_dequant_fp8_transpose_gpu(const void *in, void *out, int n_timesteps, int batch_size,
                                     int n_channels, float scale) {
    ASSERT(n_channels <= 1024);
    FLUKE_CHECK_LAUNCH(fluke_sm100_dequant_transpose(in, out, n_timesteps, batch_size, n_channels,
                                                     scale, 1, g_stream));
}

/* reference src/nn_cuda.c:158-172 */
void fluke_dequant_int8_transpose_gpu(const void *in, void *out, int n_timesteps, int batch_size,
                                      int n_channels, float scale) {
    ASSERT(n_channels <= 1024);
    FLUKE_CHECK_LAUNCH(fluke_sm100_dequant_transpose(in, out, n_timesteps, batch_size, n_channels,
                                                     scale, 0, g_stream));
}

/* reference src/nn_cuda.c:174-188 */
void fluke_quant_int8_gpu(const void *in, void *out, void *scale, int n_tokens, int hidden_dim) {
    ASSERT(hidden_dim <= 2048);
    ASSERT(hidden_dim % 2 == 0);
    FLUKE_CHECK_LAUNCH(fluke_sm100_quant_int8(in, out, scale, n_tokens, hidden_dim, g_stream));
}

/* reference src/nn_cuda.c:190-204 */
void fluke_quant_fp8_gpu(const void *in, void *out, void *scale, int n_tokens, int hidden_dim) {
    ASSERT(hidden_dim <= 2048);
    ASSERT(hidden_dim % 2 == 0);
    FLUKE_CHECK_LAUNCH(fluke_sm100_quant_fp8(in, out, scale, n_tokens, hidden_dim, g_stream));
}
