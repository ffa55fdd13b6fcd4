/* lstm_host.c -- additive factored-LSTM entry points of the C ABI. The reference has no C
 * prototype for them: its two kernels are CuTe exports driven by slorado
 * (cute/ampere/factored_lstm/export_factored_lstm_i8.py:1-9, README.md:82-92). */
#include <fluke/fluke.h>

#include <stddef.h>

#include "gpu_common.h"

int fluke_down_proj_i8_stream_gpu(void *out_f16, int ld_out, const void *a_i8, const void *w_i8,
                                  const void *scale_a, const void *scale_b, int M, int N, int K,
                                  void *stream) {
    fluke_sm100_gemm_t g = {0};
    g.kind = FLUKE_SM100_KIND_I8;
    g.epilogue = FLUKE_SM100_EPI_DEQUANT;
    g.M = M; g.N = N; g.K = K;
    g.a = a_i8; g.b = w_i8; g.out = out_f16; g.ld_out = ld_out;
    g.scale_a = (const float *)scale_a;
    g.const_scale_a = 1.0f / 127.0f;
    g.scale_b = (const float *)scale_b;
    return fluke_host_note_error(fluke_sm100_gemm(&g, stream));
}

int fluke_down_proj_i8_gpu(void *out_f16, int ld_out, const void *a_i8, const void *w_i8,
                           const void *scale_a, const void *scale_b, int M, int N, int K) {
    return fluke_down_proj_i8_stream_gpu(out_f16, ld_out, a_i8, w_i8, scale_a, scale_b, M, N, K, fluke_host_stream());
}

int fluke_factored_lstm_step_i8_stream_gpu(const void *A, const void *W_i, const void *W_f,
                                           const void *W_g, const void *W_o, const void *bias_i,
                                           const void *bias_f, const void *bias_g, const void *bias_o,
                                           void *c, void *h_out, int B, int H, int Kc, void *stream) {
    fluke_sm100_lstm_step_t s = {0};
    s.B = B; s.H = H; s.Kc = Kc;
    s.a_lo = A; s.ld_a_lo = Kc; s.k_lo = Kc;
    s.a_hi = A; s.ld_a_hi = Kc;
    s.w[0] = W_i; s.w[1] = W_f; s.w[2] = W_g; s.w[3] = W_o;
    s.ld_w = Kc;
    s.bias[0] = (const float *)bias_i; s.bias[1] = (const float *)bias_f;
    s.bias[2] = (const float *)bias_g; s.bias[3] = (const float *)bias_o;
    s.c = (float *)c;
    s.h_out = (int8_t *)h_out;
    return fluke_host_note_error(fluke_sm100_lstm_step(&s, stream));
}

int fluke_factored_lstm_step_i8_gpu(const void *A, const void *W_i, const void *W_f,
                                    const void *W_g, const void *W_o, const void *bias_i,
                                    const void *bias_f, const void *bias_g, const void *bias_o,
                                    void *c, void *h_out, int B, int H, int Kc) {
    return fluke_factored_lstm_step_i8_stream_gpu(A, W_i, W_f, W_g, W_o, bias_i, bias_f, bias_g, bias_o, c, h_out, B, H,
                                                  Kc, fluke_host_stream());
}

/* fp8 export's down-projection and step (fly/rdna4/factored_lstm/export_fp8_factored_lstm.py:113-181) */
int fluke_down_proj_fp8_gpu(void *out_f16, int ld_out, const void *a_fp8, const void *w_fp8_nk,
                            const void *scale_a, const void *scale_b, int M, int N, int K) {
    fluke_sm100_gemm_t g = {0};
    g.kind = FLUKE_SM100_KIND_F8;
    g.epilogue = FLUKE_SM100_EPI_DEQUANT2;
    g.M = M; g.N = N; g.K = K;
    g.a = a_fp8; g.b = w_fp8_nk; g.out = out_f16; g.ld_out = ld_out;
    g.scale_a = (const float *)scale_a;
    g.scale_b = (const float *)scale_b;
    if (!scale_a) return fluke_host_note_error(1 /* cudaErrorInvalidValue */);
    return fluke_host_note_error(fluke_sm100_gemm(&g, fluke_host_stream()));
}

int fluke_factored_lstm_step_fp8_gpu(const void *A, const void *W_i, const void *W_f,
                                     const void *W_g, const void *W_o, const void *bias_i,
                                     const void *bias_f, const void *bias_g, const void *bias_o,
                                     void *c, void *h_out, int B, int H, int Kc) {
    return fluke_factored_lstm_step_i8_gpu(A, W_i, W_f, W_g, W_o, bias_i, bias_f, bias_g, bias_o, c, h_out, B, H, Kc);
}

size_t fluke_factored_lstm_layer_workspace(int T, int B, int H, int R) {
    return fluke_sm100_lstm_layer_workspace(T, B, H, R);
}

int fluke_factored_lstm_layer_i8_gpu(const fluke_flstm_layer_t *layer) {
    if (!layer) return -1;
    return fluke_host_note_error(fluke_sm100_lstm_layer(layer, fluke_host_stream()));
}

/* Measurement aid of the benchmark, not part of the public header: launches only some kernel
 * classes of the layer (1 = x_down GEMM, 2 = per-step down-projection, 4 = per-step fused step). */
int fluke_factored_lstm_layer_phases_gpu(const fluke_flstm_layer_t *layer, int phase_mask);
int fluke_factored_lstm_layer_phases_gpu(const fluke_flstm_layer_t *layer, int phase_mask) {
    if (!layer) return -1;
    return fluke_host_note_error(fluke_sm100_lstm_layer_phases(layer, phase_mask, fluke_host_stream()));
}

void fluke_set_lstm_persistent(int mode) { fluke_sm100_set_lstm_persistent(mode); }
