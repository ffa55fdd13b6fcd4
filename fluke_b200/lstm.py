"""Factored-LSTM stack driver: the per-layer loop that slorado's CRFModel runs around the two
LSTM kernels (reference README.md:82-92). A stack is a list of layers applied in order, odd
layers walking time backwards; layer 0 takes per-row quantised input (amax/127 scales), later
layers take the previous layer's int8 hidden output at the fixed scale 1/127.

The stack definition (number of layers, direction pattern, input quantisation) is not part of
the reference checkout; it follows the benchmark configuration this library is measured on.
"""
import math

import torch

from . import lib as _lib, ops, prep


class FactoredLstmLayer:
    """Weights of one layer (device tensors): dn_ih/dn_hh int8 [R,H] + f32 [R] scales,
    w_up f16 [4H, 2R] = [up_hh | up_ih] gate-major (i,f,g,o), bias f32 [4H]."""

    def __init__(self, dn_ih, dn_ih_scale, dn_hh, dn_hh_scale, w_up, bias, reverse=False):
        self.dn_ih, self.dn_ih_scale = dn_ih, dn_ih_scale
        self.dn_hh, self.dn_hh_scale = dn_hh, dn_hh_scale
        self.w_up, self.bias, self.reverse = w_up, bias, reverse

    @property
    def hidden(self):
        return self.dn_ih.size(1)

    @property
    def rank(self):
        return self.dn_ih.size(0)

    @staticmethod
    def random(hidden, rank, reverse, generator, device):
        """Synthetic weights: N(0, 1/sqrt(fan_in)), per-output-channel int8 down-projections,
        bias N(0, 0.05). Generated on the CPU from `generator`, then moved."""
        def rn(*s):
            return torch.randn(*s, generator=generator)
        dn_ih, s_ih = prep.quantize_int8_rows(rn(rank, hidden) / math.sqrt(hidden))
        dn_hh, s_hh = prep.quantize_int8_rows(rn(rank, hidden) / math.sqrt(hidden))
        w_up = (rn(4 * hidden, 2 * rank) / math.sqrt(2 * rank)).to(torch.float16)
        bias = (rn(4 * hidden) * 0.05).to(torch.float32)
        mv = lambda t: t.contiguous().to(device)
        return FactoredLstmLayer(mv(dn_ih), mv(s_ih), mv(dn_hh), mv(s_hh), mv(w_up), mv(bias), reverse)


def run_stack(layers, x_i8, x_scale, state=None, workspace=None, buffers=None):
    """x_i8 [T,B,H] int8 with per-row scales x_scale [T*B]. Returns (h_out of the last layer
    [T,B,H] int8 @1/127, state) where state is a list of (c f32 [B,H], h int8 [B,H]) per layer.
    `buffers` may hold two reusable [T,B,H] int8 outputs."""
    t, b, h = x_i8.shape
    dev = x_i8.device
    if state is None:
        state = [(torch.zeros(b, h, dtype=torch.float32, device=dev),
                  torch.zeros(b, h, dtype=torch.int8, device=dev)) for _ in layers]
    if buffers is None:
        buffers = [torch.empty(t, b, h, dtype=torch.int8, device=dev) for _ in range(2)]
    cur, cur_scale = x_i8, x_scale
    for i, layer in enumerate(layers):
        c, hs = state[i]
        out = buffers[i % 2]
        ops.factored_lstm_layer_i8(cur, cur_scale, layer.dn_ih, layer.dn_ih_scale, layer.dn_hh,
                                   layer.dn_hh_scale, layer.w_up, layer.bias, c, hs,
                                   reverse=layer.reverse, h_out=out, workspace=workspace)
        cur, cur_scale = out, None
    return cur, state


def _weights_array(layers):
    """ctypes array of fluke_flstm_weights_t for a list of FactoredLstmLayer (the tensors must stay alive)."""
    arr = (_lib.fluke_flstm_weights_t * len(layers))()
    for i, l in enumerate(layers):
        arr[i] = _lib.fluke_flstm_weights_t(l.dn_ih.data_ptr(), l.dn_ih_scale.data_ptr(), l.dn_hh.data_ptr(),
                                            l.dn_hh_scale.data_ptr(), l.w_up.data_ptr(), l.bias.data_ptr(),
                                            1 if l.reverse else 0)
    return arr


def run_stack_c(layers, x_i8, x_scale, state=None, workspace=None):
    """One pass through fluke_factored_lstm_stack_i8_gpu (the C entry point a C caller uses).
    Returns (h_out of the last layer, (c [L,B,H] f32, h [L,B,H] int8))."""
    t, b, h = x_i8.shape
    dev = x_i8.device
    n = len(layers)
    if state is None:
        state = (torch.zeros(n, b, h, dtype=torch.float32, device=dev), torch.zeros(n, b, h, dtype=torch.int8, device=dev))
    need = ops._L().fluke_factored_lstm_layer_workspace(t, b, h, layers[0].rank)
    if workspace is None or workspace.numel() < need:
        workspace = torch.empty(need, dtype=torch.uint8, device=dev)
    out = torch.empty(t, b, h, dtype=torch.int8, device=dev)
    scratch = torch.empty(t, b, h, dtype=torch.int8, device=dev)
    rc = ops._L().fluke_factored_lstm_stack_i8_gpu(_weights_array(layers), n, t, b, h, layers[0].rank, x_i8.data_ptr(),
                                                   0 if x_scale is None else x_scale.data_ptr(), out.data_ptr(),
                                                   scratch.data_ptr(), state[0].data_ptr(), state[1].data_ptr(),
                                                   workspace.data_ptr(), workspace.numel())
    if rc:
        raise RuntimeError(f"fluke_factored_lstm_stack_i8_gpu failed: rc={rc} {ops._L().fluke_last_error().decode()}")
    return out, state


class StackPipeline:
    """Host-to-host streaming of whole stack passes: a thin binding of the C handle
    fluke_flstm_stream_* (fluke_b200/csrc/stack_sm100.cu), which owns the device buffers and the
    three streams. While one group of passes runs the layers, the inputs of the next are copied
    in and the outputs of the one before copied out, so in steady state a pass costs
    max(compute, copy-in, copy-out) instead of their sum.

    `passes_per_launch` = P > 1 puts P consecutive passes side by side in one batch of P*B chunks
    and runs each layer once over it (chunks are independent, so the results are those of the
    separate passes). `time_chunks` = C > 1 runs the first and the last layer in C calls over
    consecutive blocks of timesteps, each as soon as its block has been copied in / copied out as
    soon as it is written. A group is launched when it is full, or by `drain()`. Inputs and
    outputs are pinned host tensors; `submit` only enqueues."""

    def __init__(self, layers, T, B, device, passes_per_launch=1, time_chunks=1):
        self.layers = layers  # keeps the weight tensors alive
        self.shape = (T, B, layers[0].hidden)
        self.device = torch.device(device)
        self._keep = []
        with torch.cuda.device(self.device):
            self._h = ops._L().fluke_flstm_stream_create(_weights_array(layers), len(layers), T, B, layers[0].hidden,
                                                         layers[0].rank, int(passes_per_launch), int(time_chunks))
        if not self._h:
            raise RuntimeError(f"fluke_flstm_stream_create failed: {ops._L().fluke_last_error().decode()}")

    def submit(self, x_host, xs_host, out_host, zero_state=True):
        """Enqueue one pass: x_host int8 [T,B,H] and xs_host f32 [T*B] (pinned) in, the last layer's
        int8 output into out_host (pinned). The buffers must stay valid until `drain`."""
        assert x_host.is_pinned() and xs_host.is_pinned() and out_host.is_pinned()
        assert tuple(x_host.shape) == self.shape and x_host.is_contiguous() and out_host.is_contiguous()
        self._keep.append((x_host, xs_host, out_host))
        rc = ops._L().fluke_flstm_stream_submit(self._h, x_host.data_ptr(), xs_host.data_ptr(), out_host.data_ptr(),
                                                1 if zero_state else 0)
        if rc:
            raise RuntimeError(f"fluke_flstm_stream_submit failed: CUDA error {rc}")

    def flush(self):
        """Launch a group that is only partly filled (without waiting for anything)."""
        rc = ops._L().fluke_flstm_stream_flush(self._h)
        if rc:
            raise RuntimeError(f"fluke_flstm_stream_flush failed: CUDA error {rc}")

    def drain(self):
        """Run a group that is only partly filled, then wait until every output has arrived."""
        rc = ops._L().fluke_flstm_stream_drain(self._h)
        self._keep = []
        if rc:
            raise RuntimeError(f"fluke_flstm_stream_drain failed: CUDA error {rc}")

    def close(self):
        if self._h:
            ops._L().fluke_flstm_stream_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
