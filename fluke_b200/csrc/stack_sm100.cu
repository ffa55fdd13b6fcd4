// stack_sm100.cu -- host-side drivers for a whole factored-LSTM stack (the loop slorado's CRFModel
// runs around the two LSTM kernels, reference README.md:82-92): layers applied in order, each
// consuming the previous layer's int8 hidden output at the fixed scale 1/127, odd or even layers
// walking time backwards as their `reverse` flag says.
//
//   fluke_factored_lstm_stack_i8_gpu   one pass over device-resident buffers, launched on the
//                                      calling thread's stream; nothing is allocated.
//   fluke_flstm_stream_*               host-to-host streaming of many passes: while one group of
//                                      passes runs its layers on a compute stream, the inputs of
//                                      the next are copied in and the outputs of the one before
//                                      copied out on two copy streams (the two directions of the
//                                      link are independent), so a pass costs max(compute,
//                                      copy-in, copy-out) in steady state instead of their sum.
//
// No kernels here: everything below is CUDA runtime calls around fluke_sm100_lstm_layer.
#include <fluke/fluke.h>

#include "fluke_sm100.h"

#include <cuda_runtime.h>

#include <new>
#include <utility>
#include <vector>

extern "C" int fluke_host_note_error(int code);  // src/nn_gpu.c: records the last error text
extern "C" void *fluke_host_stream(void);        // src/nn_gpu.c: the calling thread's stream

namespace {

int stack_args_ok(const fluke_flstm_weights_t *layers, int n_layers, int T, int B, int H, int R) {
    if (!layers || n_layers < 1 || T < 1 || B < 1 || H < 1 || R < 1) return 0;
    for (int i = 0; i < n_layers; ++i)
        if (!layers[i].dn_ih_i8 || !layers[i].dn_ih_scale || !layers[i].dn_hh_i8 || !layers[i].dn_hh_scale ||
            !layers[i].w_up_f16 || !layers[i].bias_f32)
            return 0;
    return 1;
}

void fill_layer(fluke_flstm_layer_t *l, const fluke_flstm_weights_t &w, int T, int B, int H, int R) {
    *l = fluke_flstm_layer_t{};
    l->T = T; l->B = B; l->H = H; l->R = R; l->reverse = w.reverse;
    l->dn_ih_i8 = w.dn_ih_i8; l->dn_ih_scale = w.dn_ih_scale;
    l->dn_hh_i8 = w.dn_hh_i8; l->dn_hh_scale = w.dn_hh_scale;
    l->w_up_f16 = w.w_up_f16; l->bias_f32 = w.bias_f32;
}

}  // namespace

extern "C" int fluke_factored_lstm_stack_i8_gpu(const fluke_flstm_weights_t *layers, int n_layers, int T, int B,
                                                int H, int R, const void *x_i8, const void *x_scale,
                                                void *out_i8, void *scratch_i8, void *c_f32, void *h_i8,
                                                void *workspace, size_t workspace_bytes) {
    if (!stack_args_ok(layers, n_layers, T, B, H, R) || !x_i8 || !out_i8 || !c_f32 || !h_i8 || !workspace ||
        (n_layers > 1 && !scratch_i8))
        return fluke_host_note_error((int)cudaErrorInvalidValue);
    void *stream = fluke_host_stream();
    const void *cur = x_i8, *cur_scale = x_scale;
    for (int i = 0; i < n_layers; ++i) {
        // alternate between the two buffers so that the last layer writes `out_i8`
        void *dst = ((n_layers - 1 - i) % 2 == 0) ? out_i8 : scratch_i8;
        fluke_flstm_layer_t l;
        fill_layer(&l, layers[i], T, B, H, R);
        l.x_i8 = cur; l.x_scale = cur_scale;
        l.c_f32 = static_cast<float *>(c_f32) + size_t(i) * B * H;
        l.h_i8 = static_cast<int8_t *>(h_i8) + size_t(i) * B * H;
        l.h_out_i8 = dst;
        l.workspace = workspace; l.workspace_bytes = workspace_bytes;
        const int rc = fluke_sm100_lstm_layer(&l, stream);
        if (rc) return fluke_host_note_error(rc);
        cur = dst; cur_scale = nullptr;
    }
    return 0;
}

// ---- streaming driver ----------------------------------------------------------------------------

struct fluke_flstm_stream {
    int n_layers = 0, T = 0, B = 0, H = 0, R = 0, P = 1, device = 0;
    std::vector<fluke_flstm_weights_t> layers;
    std::vector<std::pair<int, int>> blocks;  // blocks of timesteps of the first and the last layer
    // per slot (groups alternate between two): inputs, outputs, state, events
    int8_t *x[2] = {nullptr, nullptr};
    float *xs[2] = {nullptr, nullptr};
    int8_t *out[2] = {nullptr, nullptr};
    float *c[2] = {nullptr, nullptr};
    int8_t *h[2] = {nullptr, nullptr};
    cudaEvent_t ev_run[2] = {nullptr, nullptr}, ev_out[2] = {nullptr, nullptr};
    std::vector<cudaEvent_t> ev_blk_in[2], ev_blk_run[2];
    int8_t *bufs[2] = {nullptr, nullptr};  // layer ping-pong, shared by the slots (one group computes at a time)
    void *ws = nullptr;
    size_t ws_bytes = 0;
    cudaStream_t s_in = nullptr, s_run = nullptr, s_out = nullptr;
    long groups = 0;
    struct Pass { const int8_t *x; const float *xs; int8_t *out; };
    std::vector<Pass> pending;
    int zero_state = 1;
};

namespace {

#define STACK_TRY(call)                                   \
    do {                                                  \
        const int rc_ = (int)(call);                      \
        if (rc_ != 0) return fluke_host_note_error(rc_);  \
    } while (0)

int block_index(const fluke_flstm_stream *s, int t0) {
    for (size_t i = 0; i < s->blocks.size(); ++i)
        if (s->blocks[i].first == t0) return (int)i;
    return 0;
}

// The blocks of timesteps in the order a layer walks them.
std::vector<std::pair<int, int>> blocks_for(const fluke_flstm_stream *s, int layer) {
    std::vector<std::pair<int, int>> b = s->blocks;
    if (s->layers[layer].reverse) b = std::vector<std::pair<int, int>>(b.rbegin(), b.rend());
    return b;
}

int launch_group(fluke_flstm_stream *s) {
    const int slot = int(s->groups % 2);
    const long g = s->groups++;
    const int T = s->T, B = s->B, H = s->H, n = s->n_layers;
    const int filled = (int)s->pending.size();
    const int Bf = filled * B;  // a partly filled group runs over its own chunks only
    const size_t row = size_t(B) * H;
    // copy-in, block by block in the order the first layer needs them; the group that last used
    // this slot (g - 2) must have finished reading the buffers
    if (g >= 2) STACK_TRY(cudaStreamWaitEvent(s->s_in, s->ev_run[slot], 0));
    for (const auto &blk : blocks_for(s, 0)) {
        const int t0 = blk.first, nt = blk.second - blk.first;
        for (int j = 0; j < filled; ++j) {
            const fluke_flstm_stream::Pass &p = s->pending[j];
            if (filled == 1) {
                STACK_TRY(cudaMemcpyAsync(s->x[slot] + size_t(t0) * row, p.x + size_t(t0) * row, size_t(nt) * row,
                                          cudaMemcpyHostToDevice, s->s_in));
                STACK_TRY(cudaMemcpyAsync(s->xs[slot] + size_t(t0) * B, p.xs + size_t(t0) * B, size_t(nt) * B * 4,
                                          cudaMemcpyHostToDevice, s->s_in));
            } else {
                // pass j's columns of every timestep plane: a strided copy by the copy engine itself
                STACK_TRY(cudaMemcpy2DAsync(s->x[slot] + (size_t(t0) * Bf + size_t(j) * B) * H, size_t(Bf) * H,
                                            p.x + size_t(t0) * row, row, row, nt, cudaMemcpyHostToDevice, s->s_in));
                STACK_TRY(cudaMemcpy2DAsync(s->xs[slot] + size_t(t0) * Bf + size_t(j) * B, size_t(Bf) * 4,
                                            p.xs + size_t(t0) * B, size_t(B) * 4, size_t(B) * 4, nt,
                                            cudaMemcpyHostToDevice, s->s_in));
            }
        }
        STACK_TRY(cudaEventRecord(s->ev_blk_in[slot][block_index(s, t0)], s->s_in));
    }
    // compute: after the copy-out that last read this slot's output buffer
    if (g >= 2) STACK_TRY(cudaStreamWaitEvent(s->s_run, s->ev_out[slot], 0));
    if (s->zero_state) {
        STACK_TRY(cudaMemsetAsync(s->c[slot], 0, size_t(n) * s->P * row * 4, s->s_run));
        STACK_TRY(cudaMemsetAsync(s->h[slot], 0, size_t(n) * s->P * row, s->s_run));
    }
    const int8_t *cur = s->x[slot];
    const float *cur_scale = s->xs[slot];
    for (int i = 0; i < n; ++i) {
        int8_t *dst = (i == n - 1) ? s->out[slot] : s->bufs[i % 2];
        // first and last layer: one call per block of timesteps, state carried from call to call
        std::vector<std::pair<int, int>> blocks;
        if (i == 0 || i == n - 1) blocks = blocks_for(s, i);
        else blocks.push_back(std::make_pair(0, T));
        for (const auto &blk : blocks) {
            const int t0 = blk.first, nt = blk.second - blk.first;
            if (i == 0) STACK_TRY(cudaStreamWaitEvent(s->s_run, s->ev_blk_in[slot][block_index(s, t0)], 0));
            fluke_flstm_layer_t l;
            fill_layer(&l, s->layers[i], nt, Bf, H, s->R);
            l.x_i8 = cur + size_t(t0) * Bf * H;
            l.x_scale = cur_scale ? cur_scale + size_t(t0) * Bf : nullptr;
            l.c_f32 = s->c[slot] + size_t(i) * s->P * row;
            l.h_i8 = s->h[slot] + size_t(i) * s->P * row;
            l.h_out_i8 = dst + size_t(t0) * Bf * H;
            l.workspace = s->ws; l.workspace_bytes = s->ws_bytes;
            STACK_TRY(fluke_sm100_lstm_layer(&l, s->s_run));
            if (i == n - 1) STACK_TRY(cudaEventRecord(s->ev_blk_run[slot][block_index(s, t0)], s->s_run));
        }
        cur = dst; cur_scale = nullptr;
    }
    STACK_TRY(cudaEventRecord(s->ev_run[slot], s->s_run));
    // copy-out, block by block as the last layer writes them
    for (const auto &blk : blocks_for(s, n - 1)) {
        const int t0 = blk.first, nt = blk.second - blk.first;
        STACK_TRY(cudaStreamWaitEvent(s->s_out, s->ev_blk_run[slot][block_index(s, t0)], 0));
        for (int j = 0; j < filled; ++j) {
            const fluke_flstm_stream::Pass &p = s->pending[j];
            if (filled == 1)
                STACK_TRY(cudaMemcpyAsync(p.out + size_t(t0) * row, s->out[slot] + size_t(t0) * row, size_t(nt) * row,
                                          cudaMemcpyDeviceToHost, s->s_out));
            else
                STACK_TRY(cudaMemcpy2DAsync(p.out + size_t(t0) * row, row,
                                            s->out[slot] + (size_t(t0) * Bf + size_t(j) * B) * H, size_t(Bf) * H, row, nt,
                                            cudaMemcpyDeviceToHost, s->s_out));
        }
    }
    STACK_TRY(cudaEventRecord(s->ev_out[slot], s->s_out));
    s->pending.clear();
    return 0;
}

}  // namespace

extern "C" void fluke_flstm_stream_destroy(fluke_flstm_stream_t *s) {
    if (!s) return;
    cudaSetDevice(s->device);
    if (s->s_in) cudaStreamSynchronize(s->s_in);
    if (s->s_run) cudaStreamSynchronize(s->s_run);
    if (s->s_out) cudaStreamSynchronize(s->s_out);
    for (int k = 0; k < 2; ++k) {
        cudaFree(s->x[k]); cudaFree(s->xs[k]); cudaFree(s->out[k]); cudaFree(s->c[k]); cudaFree(s->h[k]);
        cudaFree(s->bufs[k]);
        if (s->ev_run[k]) cudaEventDestroy(s->ev_run[k]);
        if (s->ev_out[k]) cudaEventDestroy(s->ev_out[k]);
        for (cudaEvent_t e : s->ev_blk_in[k]) cudaEventDestroy(e);
        for (cudaEvent_t e : s->ev_blk_run[k]) cudaEventDestroy(e);
    }
    cudaFree(s->ws);
    if (s->s_in) cudaStreamDestroy(s->s_in);
    if (s->s_run) cudaStreamDestroy(s->s_run);
    if (s->s_out) cudaStreamDestroy(s->s_out);
    delete s;
}

extern "C" fluke_flstm_stream_t *fluke_flstm_stream_create(const fluke_flstm_weights_t *layers, int n_layers, int T,
                                                           int B, int H, int R, int passes_per_launch,
                                                           int time_chunks) {
    if (!stack_args_ok(layers, n_layers, T, B, H, R) || passes_per_launch < 1) {
        fluke_host_note_error((int)cudaErrorInvalidValue);
        return nullptr;
    }
    fluke_flstm_stream *s = new (std::nothrow) fluke_flstm_stream;
    if (!s) return nullptr;
    s->n_layers = n_layers; s->T = T; s->B = B; s->H = H; s->R = R; s->P = passes_per_launch;
    s->layers.assign(layers, layers + n_layers);
    int C = time_chunks < 1 ? 1 : (time_chunks > T ? T : time_chunks);
    for (int i = 0; i < C; ++i) {
        // edges at round(i * T / C)
        const int e0 = int((2LL * i * T + C) / (2 * C)), e1 = int((2LL * (i + 1) * T + C) / (2 * C));
        if (e1 > e0) s->blocks.push_back(std::make_pair(e0, e1));
    }
    const size_t plane = size_t(T) * s->P * B * H;
    const size_t state = size_t(n_layers) * s->P * B * H;
    s->ws_bytes = fluke_sm100_lstm_layer_workspace(T, s->P * B, H, R);
    bool ok = cudaGetDevice(&s->device) == cudaSuccess;
    for (int k = 0; k < 2 && ok; ++k) {
        ok = ok && cudaMalloc(&s->x[k], plane) == cudaSuccess;
        ok = ok && cudaMalloc(&s->xs[k], size_t(T) * s->P * B * 4) == cudaSuccess;
        ok = ok && cudaMalloc(&s->out[k], plane) == cudaSuccess;
        ok = ok && cudaMalloc(&s->c[k], state * 4) == cudaSuccess;
        ok = ok && cudaMalloc(&s->h[k], state) == cudaSuccess;
        ok = ok && cudaMalloc(&s->bufs[k], plane) == cudaSuccess;
        ok = ok && cudaEventCreateWithFlags(&s->ev_run[k], cudaEventDisableTiming) == cudaSuccess;
        ok = ok && cudaEventCreateWithFlags(&s->ev_out[k], cudaEventDisableTiming) == cudaSuccess;
        for (size_t b = 0; b < s->blocks.size() && ok; ++b) {
            cudaEvent_t e1 = nullptr, e2 = nullptr;
            ok = cudaEventCreateWithFlags(&e1, cudaEventDisableTiming) == cudaSuccess &&
                 cudaEventCreateWithFlags(&e2, cudaEventDisableTiming) == cudaSuccess;
            if (e1) s->ev_blk_in[k].push_back(e1);
            if (e2) s->ev_blk_run[k].push_back(e2);
        }
    }
    ok = ok && cudaMalloc(&s->ws, s->ws_bytes) == cudaSuccess;
    ok = ok && cudaStreamCreateWithFlags(&s->s_in, cudaStreamNonBlocking) == cudaSuccess;
    ok = ok && cudaStreamCreateWithFlags(&s->s_run, cudaStreamNonBlocking) == cudaSuccess;
    ok = ok && cudaStreamCreateWithFlags(&s->s_out, cudaStreamNonBlocking) == cudaSuccess;
    if (!ok) {
        fluke_host_note_error((int)cudaGetLastError());
        fluke_flstm_stream_destroy(s);
        return nullptr;
    }
    return s;
}

extern "C" int fluke_flstm_stream_submit(fluke_flstm_stream_t *s, const void *x_host_i8, const void *x_scale_host,
                                         void *out_host_i8, int zero_state) {
    if (!s || !x_host_i8 || !x_scale_host || !out_host_i8) return fluke_host_note_error((int)cudaErrorInvalidValue);
    fluke_flstm_stream::Pass p = {static_cast<const int8_t *>(x_host_i8), static_cast<const float *>(x_scale_host),
                                  static_cast<int8_t *>(out_host_i8)};
    s->pending.push_back(p);
    s->zero_state = zero_state;
    // Only a full group is launched here; flush and drain launch a partly filled one. (Starting
    // a lone pass whenever the GPU is idle halves the fill time of a job, but that pass and the
    // odd one it leaves at the end then run at the single-batch step time: 2 x 38.8 ms instead
    // of one 46.1 ms group at the benchmark's shape.)
    if ((int)s->pending.size() == s->P) return launch_group(s);
    return 0;
}

extern "C" int fluke_flstm_stream_flush(fluke_flstm_stream_t *s) {
    if (!s) return fluke_host_note_error((int)cudaErrorInvalidValue);
    if (!s->pending.empty()) return launch_group(s);
    return 0;
}

extern "C" int fluke_flstm_stream_drain(fluke_flstm_stream_t *s) {
    if (!s) return fluke_host_note_error((int)cudaErrorInvalidValue);
    if (!s->pending.empty()) {
        const int rc = launch_group(s);
        if (rc) return rc;
    }
    STACK_TRY(cudaStreamSynchronize(s->s_in));
    STACK_TRY(cudaStreamSynchronize(s->s_run));
    STACK_TRY(cudaStreamSynchronize(s->s_out));
    return 0;
}

// Strided copy between pinned host memory and the device by the copy engine alone (no staging
// buffer, no kernel): `height` rows of `width` bytes, pitches in bytes.
extern "C" int fluke_sm100_copy_rows_async(void *dst, size_t dst_pitch, const void *src, size_t src_pitch,
                                           size_t width, size_t height, int to_device, void *stream) {
    return (int)cudaMemcpy2DAsync(dst, dst_pitch, src, src_pitch, width, height,
                                  to_device ? cudaMemcpyHostToDevice : cudaMemcpyDeviceToHost,
                                  static_cast<cudaStream_t>(stream));
}
