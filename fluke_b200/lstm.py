"""Factored-LSTM stack driver: the per-layer loop that slorado's CRFModel runs around the two
LSTM kernels (reference README.md:82-92). A stack is a list of layers applied in order, odd
layers walking time backwards; layer 0 takes per-row quantised input (amax/127 scales), later
layers take the previous layer's int8 hidden output at the fixed scale 1/127.

The stack definition (number of layers, direction pattern, input quantisation) is not part of
the reference checkout; it follows the benchmark configuration this library is measured on.
"""
import math

import torch

from . import ops, prep


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
