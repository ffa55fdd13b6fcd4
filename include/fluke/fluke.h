/* fluke.h -- public C ABI of the sm_100a (B200) implementation of fluke's quantized
 * basecaller layer path.
 *
 * Every prototype in parts 1-4 has the same name, argument order, argument types and
 * return type as the reference header include/fluke/fluke.h (cited per function), so
 * slorado (static link of lib/libfluke.a) and the ctypes loader (fluke_lib.py) bind to
 * it unchanged. Part 5 is additive: entry points the reference only has as CuTe-DSL
 * exports (base int8 GEMM, factored-LSTM kernels), plus stream control.
 *
 * Conventions: all `_gpu` pointers are caller-owned DEVICE pointers; nothing is
 * synchronised internally; launches go to the stream set with fluke_set_stream()
 * (default: the legacy default stream, as in the reference). `void` GPU functions
 * print a message and exit(1) on a bad dimension or a launch error (reference:
 * src/cuda_utils.h:5-23, src/error.h:74-81); `int` functions return 0 on success.
 */
#ifndef FLUKE_H
#define FLUKE_H

#include <stdbool.h>
#include <stdlib.h>
#include <stdint.h>
#include <stddef.h>

#include "fluke_error.h"

#ifdef __cplusplus
extern "C" {
#endif

/* ------------------------------------------------------------------------------------
 * Part 1 -- CPU functions (fp32, pthreads). Reference: include/fluke/fluke.h:26-68,
 * implemented in src/nn_cpu.c.
 * ---------------------------------------------------------------------------------- */

/* In-place rotate-half rotary embedding on fp32 data (reference fluke.h:26-39).
 * x is addressed as x[b*stride_batch + s*stride_seq + h*stride_head + i] (strides in
 * elements). sin_buf/cos_buf are [seq_len, sincos_width]. For i < sincos_width:
 *     x[i]              <- x[i]*cos[s,i] - x[i+sincos_width]*sin[s,i]
 *     x[i+sincos_width] <- x[i]*sin[s,i] + x[i+sincos_width]*cos[s,i]
 * so 2*sincos_width <= head_dim elements of each head are rotated. */
void fluke_rotary_emb_cpu(
    void *x,
    const void *sin_buf,
    const void *cos_buf,
    int batch_size,
    int seq_len,
    int n_heads,
    int head_dim,
    int sincos_width,
    int stride_batch,
    int stride_seq,
    int stride_head,
    int n_threads
);

/* out = (in + alpha*residual) * rsqrt(mean((in + alpha*residual)^2) + eps) * weight,
 * per row of [n_tokens, hidden_dim]; fp32 (reference fluke.h:45-55). */
void fluke_rmsnorm_cpu(
    void *in,
    const void *residual,
    const void *weight,
    void *out,
    int n_tokens,
    int hidden_dim,
    float alpha,
    float eps,
    int n_threads
);

/* One LSTM timestep's gate epilogue in fp32 (reference fluke.h:60-68). scratch and ih_t
 * are [batch_size, 4*hidden_dim] pre-activations in gate order i,f,g,o; their sum g is
 * activated as i,f,o = clamp(0.2*g+0.5, 0, 1), g = clamp(g, -1, 1); cell
 * [batch_size, hidden_dim] becomes f*cell + i*g in place; hh_next = o*tanh(cell). */
void fluke_flstm_step_cpu(
    const void* scratch,
    const void* ih_t,
    void* cell,
    void* hh_next,
    int batch_size,
    int hidden_dim,
    int n_threads
);

/* Model dimensions a fused backend is selected for (reference fluke.h:72). */
typedef struct { int d_model, dim_feedforward, nhead, head_dim, max_seq; } fluke_dims_t;

#if defined(HAVE_CUDA) || defined(HAVE_ROCM)

/* ------------------------------------------------------------------------------------
 * Part 2 -- memory-bound GPU kernels. Reference: fluke.h:78-197, kernels in
 * src/nn_kernel_cuda.h, launchers in src/nn_cuda.c.
 * ---------------------------------------------------------------------------------- */

/* f16 RMSNorm over a residual add, fp32 math (reference fluke.h:78-87).
 * hidden_dim even and <= 1024. */
void fluke_rmsnorm_gpu(
    const void* in,
    const void* residual,
    const void* weight,
    void* out,
    int n_tokens,
    int hidden_dim,
    float alpha,
    float eps
);

/* Per-token symmetric int8 quantisation of f16 rows (reference fluke.h:92-98):
 * scale[row] = max(amax,1e-12)/128 (the dequant multiplier), out = clamp(rn(in/scale),
 * -127, 127). hidden_dim even and <= 2048. */
void fluke_quant_int8_gpu(
    const void* in,
    void*       out,
    void*       scale,
    int         n_tokens,
    int         hidden_dim
);

/* Per-token fp8 E4M3FN quantisation of f16 rows (reference fluke.h:103-109):
 * scale[row] = max(amax,1e-12)/448, out = e4m3(clamp(in/scale, -448, 448)) with the
 * reference's software conversion (round half up in magnitude, saturating, no NaN).
 * hidden_dim even and <= 2048. */
void fluke_quant_fp8_gpu(
    const void* in,
    void*       out,
    void*       scale,
    int         n_tokens,
    int         hidden_dim
);

/* RMSNorm fused with per-token int8 quantisation, in place (reference fluke.h:114-123).
 * On entry `residual` (int8) / `residual_scale` (f32 per token) hold the previous
 * quantised residual; on return they hold the quantised
 * rmsnorm(in + alpha*dequant(residual))*weight with scale amax/127.
 * hidden_dim even and <= 1024. */
void fluke_rmsnorm_quant_int8_gpu(
    const void* in,
    const void* weight,
    void* residual,
    void* residual_scale,
    int n_tokens,
    int hidden_dim,
    float alpha,
    float eps
);

/* fp8 E4M3FN twin of fluke_rmsnorm_quant_int8_gpu, scale amax/448
 * (reference fluke.h:128-137). */
void fluke_rmsnorm_quant_fp8_gpu(
    const void* in,
    const void* weight,
    void* residual,
    void* residual_scale,
    int n_tokens,
    int hidden_dim,
    float alpha,
    float eps
);

/* out[n,t,c] (f16) = e4m3(in[t,n,c]) * scale: dequantise and swap the two leading
 * dimensions in one pass (reference fluke.h:141-148). n_channels <= 1024. */
void fluke_dequant_fp8_transpose_gpu(
    const void* in,
    void*       out,
    int         n_timesteps,
    int         batch_size,
    int         n_channels,
    float       scale
);

/* int8 twin of fluke_dequant_fp8_transpose_gpu (reference fluke.h:152-159). */
void fluke_dequant_int8_transpose_gpu(
    const void* in,
    void*       out,
    int         n_timesteps,
    int         batch_size,
    int         n_channels,
    float       scale
);

/* f16 in-place rotary embedding, fp32 math; same addressing and table layout as
 * fluke_rotary_emb_cpu (reference fluke.h:163-175). */
void fluke_rotary_emb_gpu(
    void *x,
    const void *sin_gpu,
    const void *cos_gpu,
    int batch_size,
    int seq_len,
    int n_heads,
    int head_dim,
    int sincos_width,
    int stride_batch,
    int stride_seq,
    int stride_head
);

/* out[t,k] = silu(in[t,hidden_dim+k]) * in[t,k] for f16 in [n_tokens, 2*hidden_dim]
 * (reference fluke.h:180-185). */
void fluke_silu_mul_gpu(
    const void *in,
    void *out,
    int n_tokens,
    int hidden_dim
);

/* f16 twin of fluke_flstm_step_cpu; the cell state is stored in f16
 * (reference fluke.h:190-197). */
void fluke_flstm_step_gpu(
    const void* scratch,
    const void* ih_t,
    void* cell,
    void* hh_next,
    int batch_size,
    int hidden_dim
);

/* ------------------------------------------------------------------------------------
 * Part 3 -- fused int8 transformer kernels (reference fluke.h:209-236; dispatch in
 * src/fused_cuda.c, CuTe kernels cute/ampere/rotary/gemm_i8_rotary.py and
 * cute/ampere/dual_gemm_silu/dual_gemm_i8_silu.py). Here they run as tcgen05 kind::i8
 * MMA with int32 accumulators in tensor memory.
 * ---------------------------------------------------------------------------------- */

/* Process-lifetime backend handle; NULL when the device is not compute capability 10.0
 * or `dims` is not (512, 2048, 8, 64). Never free it. */
typedef struct fluke_int8_backend fluke_int8_backend_t;
fluke_int8_backend_t *fluke_int8_select(int device_index, fluke_dims_t dims);

/* The dims a backend was selected with. */
fluke_dims_t fluke_int8_dims(const fluke_int8_backend_t *b);

/* out f16 [M, 3*d_model] = rotary(qkv) with qkv = (int32(a_i8 @ wqkv_i8^T) * scale_a[m])
 * * scale_b[n]. a_i8 [M, d_model], wqkv_i8 [3*d_model, d_model] (row-major int8),
 * sin/cos f32 [seqlen, head_dim/2]; rotate-half on every head of Q and K at position
 * m % seqlen, V copied through. Returns 0 on success. */
int fluke_qkv_rotary_i8_gpu(
    const fluke_int8_backend_t *b, void *out,
    const void *a_i8, const void *wqkv_i8,
    const void *scale_a, const void *scale_b,
    const void *sin, const void *cos,
    int M, int seqlen
);

/* out f16 [M, dim_feedforward] = silu(g) * u with g = (int32(a @ gate^T)*scale_a)*scale_gate,
 * u likewise with up/scale_up. Returns 0 on success. */
int fluke_gated_mlp_i8_gpu(
    const fluke_int8_backend_t *b, void *out,
    const void *a_i8, const void *gate_i8, const void *up_i8,
    const void *scale_a, const void *scale_gate, const void *scale_up,
    int M
);

/* ------------------------------------------------------------------------------------
 * Part 4 -- fused fp8 (E4M3, scale amax/448, f32 accumulate) twins (reference
 * fluke.h:251-275; stubs on the reference's CUDA build, src/fused_hip.c:128-147).
 * Here they run as tcgen05 kind::f8f6f4 MMA. Weights arrive PRESHUFFLED as
 * [N/16, K/16, 2, 16, 8] bytes; the first call with a given weight pointer re-orders
 * it once into a private row-major [N, K] copy (one device allocation per weight,
 * kept for the life of the process).
 * ---------------------------------------------------------------------------------- */

typedef struct fluke_fp8_backend fluke_fp8_backend_t;
fluke_fp8_backend_t *fluke_fp8_select(int device_index, fluke_dims_t dims);

int fluke_qkv_rotary_fp8_gpu(
    const fluke_fp8_backend_t *b, void *out,
    const void *a_fp8, const void *wqkv_fp8,
    const void *scale_a, const void *scale_b,
    const void *sin, const void *cos,
    int M, int seqlen
);

int fluke_gated_mlp_fp8_gpu(
    const fluke_fp8_backend_t *b, void *out,
    const void *a_fp8, const void *gate_fp8, const void *up_fp8,
    const void *scale_a, const void *scale_gate, const void *scale_up,
    int M
);

/* ------------------------------------------------------------------------------------
 * Part 5 -- additive entry points (no prototype in the reference header).
 * ---------------------------------------------------------------------------------- */

/* Stream used by every later launch this library makes FROM THE CALLING HOST THREAD (a
 * cudaStream_t passed as void*; the setting is thread-local, so threads that each drive their own
 * GPU or stream do not disturb one another). NULL, the initial value in every thread, selects the
 * legacy default stream, which is what the reference always uses (src/nn_cuda.c launches with
 * <<<grid, block>>>). Launches go to the calling thread's current CUDA device. */
void  fluke_set_stream(void *cuda_stream);
void *fluke_get_stream(void);

/* Last CUDA error string recorded by an `int`-returning entry point ("" if none). */
const char *fluke_last_error(void);

/* Base int8 GEMM: out f16 [M,N] = f16( float(int32(a @ b^T)) * (sa[m]*scale_b[n]) ) with
 * a [M,K], b [N,K] row-major int8; sa[m] = scale_a[m], or const_scale_a when scale_a is
 * NULL. Replaces TensorOpGemmI8 (cute/ampere/gemm/gemm_i8_quant.py:182-809, scale
 * arithmetic :617 and :750). K % 16 == 0, K <= 1024, N % 64 == 0. */
int fluke_gemm_i8_gpu(
    void *out_f16, const void *a_i8, const void *b_i8,
    const void *scale_a, float const_scale_a, const void *scale_b,
    int M, int N, int K
);

/* The same contraction with the raw int32 accumulators written out (out_s32 [M,N]);
 * the integer-exact check of cute/ampere/gemm/gemm_i8_quant.py:1060-1071. */
int fluke_gemm_i8_s32_gpu(void *out_s32, const void *a_i8, const void *b_i8, int M, int N, int K);

/* fp8 E4M3 base GEMM with a plain row-major [N,K] weight: out = f16((acc*sa[m])*sb[n]). */
int fluke_gemm_fp8_gpu(
    void *out_f16, const void *a_fp8, const void *b_fp8,
    const void *scale_a, const void *scale_b, int M, int N, int K
);

/* Re-order a PRESHUFFLED fp8 weight [N/16, K/16, 2, 16, 8] (the layout
 * preshuffle_b_fp8 produces, fly/rdna4/gemm/rdna_fp8_preshuffle_gemm.py:40-54) into
 * row-major [N, K]. */
int fluke_fp8_unshuffle_gpu(void *dst_nk, const void *src_preshuffled, int N, int K);

/* The reference-ABI fp8 entry points (fluke_qkv_rotary_fp8_gpu, fluke_gated_mlp_fp8_gpu) keep a
 * private row-major copy of every PRESHUFFLED weight they are given, made on the first call that
 * sees the weight's (device, address, N, K) -- one cudaMalloc and one re-ordering kernel, so that
 * first call must not sit inside a stream capture. The copy is found again by the weight's
 * ADDRESS: a caller that frees a weight, or writes new contents to the same address, must call
 * fluke_fp8_release_weight before using that address again, or the stale copy is used.
 *   fluke_fp8_prepare_weight   makes the copy now (at model load). 0 on success.
 *   fluke_fp8_release_weight   drops the copy of one weight, or of all when passed NULL (it waits
 *                              for the device before freeing). Returns the number dropped.
 * The table holds 64 weights per process; beyond that the oldest copy is dropped to make room.
 * Thread-safe. */
int fluke_fp8_prepare_weight(const void *preshuffled, int N, int K);
int fluke_fp8_release_weight(const void *preshuffled);

/* fp8 fused ops taking plain row-major [N, K] weights (no private copy is made). */
int fluke_qkv_rotary_fp8_plain_gpu(
    const fluke_fp8_backend_t *b, void *out,
    const void *a_fp8, const void *wqkv_fp8_nk,
    const void *scale_a, const void *scale_b,
    const void *sin, const void *cos,
    int M, int seqlen
);
int fluke_gated_mlp_fp8_plain_gpu(
    const fluke_fp8_backend_t *b, void *out,
    const void *a_fp8, const void *gate_fp8_nk, const void *up_fp8_nk,
    const void *scale_a, const void *scale_gate, const void *scale_up,
    int M
);

/* int8 down-projection of the factored LSTM: out f16 [M,N] (row stride ld_out elements)
 * = f16( float(int32(a @ w^T)) * (sa*scale_b[n]) ), sa = scale_a[m] or 1/127 when
 * scale_a is NULL (the fixed scale of an int8 hidden state). Replaces the
 * down_proj_i8_R{R}_K{H} export (cute/ampere/factored_lstm/export_factored_lstm_i8.py:65-77). */
int fluke_down_proj_i8_gpu(
    void *out_f16, int ld_out, const void *a_i8, const void *w_i8,
    const void *scale_a, const void *scale_b, int M, int N, int K
);

/* One fused factored-LSTM timestep. Argument order follows TensorOpFactoredLstmI8.__call__
 * (cute/ampere/factored_lstm/factored_lstm_i8.py:85-99): A f16 [B,Kc] = [hh_down | x_down];
 * W_g f16 [H,Kc] = [up_hh_g | up_ih_g] and bias_g f32 [H] for g in i,f,g,o; c f32 [B,H]
 * updated in place; h int8 [B,H] = round-half-away(127 * o*tanh(c)). Gate math as in
 * fluke_flstm_step_cpu. H % 16 == 0, Kc % 64 == 0, Kc <= 512. */
int fluke_factored_lstm_step_i8_gpu(
    const void *A,
    const void *W_i, const void *W_f, const void *W_g, const void *W_o,
    const void *bias_i, const void *bias_f, const void *bias_g, const void *bias_o,
    void *c, void *h_out,
    int B, int H, int Kc
);

/* The two per-step entry points again with the stream as a trailing argument, as the reference's
 * exports take it (cute/ampere/gemm/gemm_i8_quant.py:237-239,
 * cute/ampere/factored_lstm/factored_lstm_i8.py:98-99: a CUstream, so that a caller can capture its
 * own per-timestep loop); NULL = the legacy default stream. The forms without it use the calling
 * thread's fluke_set_stream setting. */
int fluke_down_proj_i8_stream_gpu(
    void *out_f16, int ld_out, const void *a_i8, const void *w_i8,
    const void *scale_a, const void *scale_b, int M, int N, int K, void *stream
);
int fluke_factored_lstm_step_i8_stream_gpu(
    const void *A,
    const void *W_i, const void *W_f, const void *W_g, const void *W_o,
    const void *bias_i, const void *bias_f, const void *bias_g, const void *bias_o,
    void *c, void *h_out,
    int B, int H, int Kc, void *stream
);

/* The two kernels of the reference's fp8 factored-LSTM export
 * (fly/rdna4/factored_lstm/export_fp8_factored_lstm.py).
 *   fluke_down_proj_fp8_gpu          its down-projection (:161-181, `down_proj_fp8_R{R}_K{H}`): the fp8
 *                                    base GEMM with N = R, K = H: out f16 [M,N] (row stride ld_out) =
 *                                    f16((f32(a @ w^T) * scale_a[m]) * scale_b[n]), a e4m3 [M,K] with
 *                                    per-row scales, w e4m3 [N,K] ROW-MAJOR with per-channel scales
 *                                    (a PRESHUFFLED weight goes through fluke_fp8_unshuffle_gpu once).
 *                                    K % 16 == 0, K <= 1024, N % 64 == 0.
 *   fluke_factored_lstm_step_fp8_gpu its fused step (rdna_fp8_factored_lstm.py:113-294). In that export
 *                                    only the down-projection is fp8: the step contracts f16
 *                                    [hh_down | x_down] with f16 up-projections and writes int8 h at
 *                                    1/127, i.e. it IS fluke_factored_lstm_step_i8_gpu; the name exists so
 *                                    that a caller of the fp8 export finds its two symbols.
 * How h (int8 at 1/127) becomes the e4m3 operand of the next down-projection is the caller's
 * step (slorado; not part of the reference checkout). */
int fluke_down_proj_fp8_gpu(
    void *out_f16, int ld_out, const void *a_fp8, const void *w_fp8_nk,
    const void *scale_a, const void *scale_b, int M, int N, int K
);
int fluke_factored_lstm_step_fp8_gpu(
    const void *A,
    const void *W_i, const void *W_f, const void *W_g, const void *W_o,
    const void *bias_i, const void *bias_f, const void *bias_g, const void *bias_o,
    void *c, void *h_out,
    int B, int H, int Kc
);

/* One whole factored-LSTM layer over T timesteps (the loop slorado's CRFModel drives,
 * README.md:82-92): x_down = down_proj(x, dn_ih) for all t, then per step
 * hh_down = down_proj(h_{t-1}, dn_hh), gates on [hh_down | x_down_t], cell update,
 * h_t int8. `reverse` != 0 walks t from T-1 down to 0 (h_out keeps x's time order). */
typedef struct {
    int T, B, H, R;             /* timesteps, chunks, hidden size, factor rank          */
    int reverse;                /* 0: t = 0..T-1, else t = T-1..0                       */
    const void *x_i8;           /* [T,B,H] int8 layer input                             */
    const void *x_scale;        /* f32 [T*B] per-row dequant scales, or NULL = 1/127    */
    const void *dn_ih_i8;       /* [R,H] int8 input down-projection                     */
    const void *dn_ih_scale;    /* f32 [R]                                              */
    const void *dn_hh_i8;       /* [R,H] int8 recurrent down-projection                 */
    const void *dn_hh_scale;    /* f32 [R]                                              */
    const void *w_up_f16;       /* [4*H, 2*R] f16, row g*H+n = [up_hh_g[n] | up_ih_g[n]] */
    const void *bias_f32;       /* [4*H] f32, gate order i,f,g,o                        */
    void *c_f32;                /* [B,H] f32 cell state, in/out                         */
    void *h_i8;                 /* [B,H] int8 hidden state @1/127, in (h_0) / out (h_T) */
    void *h_out_i8;             /* [T,B,H] int8 hidden outputs @1/127                   */
    void *workspace;            /* fluke_factored_lstm_layer_workspace() bytes          */
    size_t workspace_bytes;
} fluke_flstm_layer_t;

size_t fluke_factored_lstm_layer_workspace(int T, int B, int H, int R);
int fluke_factored_lstm_layer_i8_gpu(const fluke_flstm_layer_t *layer);

/* How fluke_factored_lstm_layer_i8_gpu runs the recurrence (a per-thread setting).
 *   1 (default): one launch per layer -- gate weights in shared memory and the cell state in
 *      registers for all T timesteps -- in the fastest form the shape and the device allow.
 *   2: exchange through L2 with separate projection thread blocks (R = 128, H a multiple of 128
 *      up to 1024).
 *   4: exchange inside thread-block clusters through distributed shared memory (R = 128, H a
 *      multiple of 64 up to 768; 7 row tiles of 128 chunks at a time on a B200).
 *   0: two launches per timestep.
 * A form that does not cover the shape falls back to one that does. The single-launch forms give
 * identical bytes; the per-step kernels the same int8 outputs within one code (the two K halves
 * are accumulated in the other order, tanh by the library routine). */
void fluke_set_lstm_persistent(int mode);

/* ---- whole stack ---------------------------------------------------------------------------
 * The loop around the layer that slorado's CRFModel runs (README.md:82-92; the loop itself is
 * not part of the reference checkout): layers applied in order, layer 0 on per-row quantised
 * input (x_scale), every later layer on the previous layer's int8 hidden output at the fixed
 * scale 1/127, each walking time forwards or backwards as its `reverse` says. */
typedef struct {
    const void *dn_ih_i8;       /* [R,H] int8   */
    const void *dn_ih_scale;    /* f32 [R]      */
    const void *dn_hh_i8;       /* [R,H] int8   */
    const void *dn_hh_scale;    /* f32 [R]      */
    const void *w_up_f16;       /* [4*H, 2*R] f16, as in fluke_flstm_layer_t */
    const void *bias_f32;       /* [4*H] f32    */
    int reverse;
} fluke_flstm_weights_t;

/* One pass of the stack over device buffers, on the calling thread's stream; allocates nothing.
 * x_i8 [T,B,H] with x_scale f32 [T*B] (or NULL = 1/127); out_i8 [T,B,H] receives the last
 * layer's hidden outputs; scratch_i8 [T,B,H] is a second buffer the layers alternate with (may
 * be NULL for a single layer; x_i8 is not written). c_f32 [n_layers,B,H] and h_i8 [n_layers,B,H]
 * hold every layer's state, in (initial) and out (final). workspace as for one layer. */
int fluke_factored_lstm_stack_i8_gpu(
    const fluke_flstm_weights_t *layers, int n_layers, int T, int B, int H, int R,
    const void *x_i8, const void *x_scale, void *out_i8, void *scratch_i8,
    void *c_f32, void *h_i8, void *workspace, size_t workspace_bytes
);

/* Host-to-host streaming of many passes of a stack. The handle owns its device buffers (two input
 * sets, two output buffers, two layer buffers, state and workspace: about 6 x T*P*B*H bytes) and
 * three streams: while one group of passes runs the layers, the inputs of the next are copied in
 * and the outputs of the one before copied out.
 *   create   passes_per_launch = P >= 1 puts P consecutive passes side by side in one batch of
 *            P*B chunks and runs each layer once over it (chunks are independent: the same
 *            bytes); time_chunks = C >= 1 runs the first and the last layer in C calls over
 *            consecutive blocks of timesteps so that a group's copies overlap its own layers.
 *            Allocates on the calling thread's current device. NULL on failure.
 *   submit   x_host_i8 [T,B,H], x_scale_host f32 [T*B] and out_host_i8 [T,B,H] are PINNED host
 *            buffers that stay valid until drain. zero_state != 0: the pass starts from c = 0,
 *            h = 0. Only enqueues work. A group is launched when it is full (P passes).
 *   flush    launches a group that is only partly filled (a caller whose next pass is not at
 *            hand yet calls it instead of leaving the GPU idle).
 *   drain    flush, then blocks until every submitted pass's output is in its host buffer.
 *   destroy  waits for outstanding work and frees everything.
 * One host thread per handle. int functions return 0 or a CUDA error code. */
typedef struct fluke_flstm_stream fluke_flstm_stream_t;
fluke_flstm_stream_t *fluke_flstm_stream_create(
    const fluke_flstm_weights_t *layers, int n_layers, int T, int B, int H, int R,
    int passes_per_launch, int time_chunks
);
int  fluke_flstm_stream_submit(fluke_flstm_stream_t *s, const void *x_host_i8, const void *x_scale_host,
                               void *out_host_i8, int zero_state);
int  fluke_flstm_stream_flush(fluke_flstm_stream_t *s);
int  fluke_flstm_stream_drain(fluke_flstm_stream_t *s);
void fluke_flstm_stream_destroy(fluke_flstm_stream_t *s);

/* No counterpart in the reference. The same layer as fluke_factored_lstm_layer_i8_gpu for
 * callers that cannot allocate device memory (plug-ins without an allocator, fixed memory
 * budgets, regions where the CUDA allocator must not be called): layer->workspace /
 * workspace_bytes are ignored and the
 * intermediates live in a FLUKE_LSTM_NOALLOC_SCRATCH_BYTES array built into the library, held
 * by every GPU that loads it. Nothing is allocated. The layer must satisfy
 * fluke_factored_lstm_layer_workspace(T,B,H,R) <= FLUKE_LSTM_NOALLOC_SCRATCH_BYTES, otherwise
 * a message is printed and non-zero returned (at rank 128: 1024 chunks x 14 timesteps fit, 15
 * do not). The first call on a device resolves the array's device address and configures the
 * kernels of its shape and mode: make it before any stream capture begins. All calls share the array, so calls
 * whose kernels overlap on the GPU race; run one such layer at a time per device. */
#define FLUKE_LSTM_NOALLOC_SCRATCH_BYTES (4u << 20)
int fluke_factored_lstm_layer_i8_noalloc_gpu(const fluke_flstm_layer_t *layer);

#endif /* HAVE_CUDA || HAVE_ROCM */

#ifdef __cplusplus
}
#endif

#endif /* FLUKE_H */
