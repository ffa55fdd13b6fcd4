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


class StackPipeline:
    """Host-to-host streaming of whole stack passes: while one group of passes runs the layers on
    the compute stream, the inputs of the next are copied in and the outputs of the one before are
    copied out on two copy streams (the two PCIe directions are independent), so in steady state a
    pass costs max(compute, copy-in, copy-out) instead of their sum.

    `passes_per_launch` = P > 1 puts P consecutive passes side by side in one batch of P*B chunks
    and runs each layer once over it (chunks are independent, so the results are those of the
    separate passes). The recurrence is a latency-bound chain, and a layer call over twice the
    chunks costs far less than two calls (the wide single-launch configuration holds 16 row tiles).
    The results of a pass are then complete when its group has run: after the P-th `submit` of
    the group, or after `drain()`, which also runs a group that is only partly filled.

    Device memory: two input sets, the two ping-pong layer buffers and two output buffers of
    [T,P*B,H] int8. Inputs and outputs are pinned host tensors; `submit` only enqueues work."""

    def __init__(self, layers, T, B, device, passes_per_launch=1):
        self.layers = layers
        h = layers[0].hidden
        P = int(passes_per_launch)
        assert P >= 1
        self.P = P
        self.shape = (T, B, h)
        dev = torch.device(device)
        self.device = dev
        mk = lambda: torch.zeros(T, P * B, h, dtype=torch.int8, device=dev)
        self.x = [mk(), mk()]
        self.xs = [torch.zeros(T * P * B, dtype=torch.float32, device=dev) for _ in range(2)]
        self.bufs = [mk(), mk()]
        self.out = [mk(), mk()]
        self.state = [[(torch.zeros(P * B, h, dtype=torch.float32, device=dev),
                        torch.zeros(P * B, h, dtype=torch.int8, device=dev)) for _ in layers] for _ in range(2)]
        need = ops._L().fluke_factored_lstm_layer_workspace(T, P * B, h, layers[0].rank)
        self.ws = torch.empty(need, dtype=torch.uint8, device=dev)
        self.s_in, self.s_run, self.s_out = (torch.cuda.Stream(dev) for _ in range(3))
        self.ev_in = [torch.cuda.Event() for _ in range(2)]     # inputs of the group in slot g%2 copied in
        self.ev_run = [torch.cuda.Event() for _ in range(2)]    # group that used slot g%2 finished computing
        self.ev_out = [torch.cuda.Event() for _ in range(2)]    # output buffer g%2 copied out
        self.k = 0
        self.pending = []   # host output tensors of the group being filled

    def _block(self, t, j):
        """Pass j's columns of a [T, P*B, ...] device tensor."""
        T, B, _ = self.shape
        return t.view(T, self.P, B, *t.shape[2:])[:, j]

    def submit(self, x_host, xs_host, out_host, zero_state=True):
        """Enqueue one pass: x_host int8 [T,B,H] and xs_host f32 [T*B] (pinned) in, the last layer's
        int8 output into out_host (pinned). Every pass starts from a zero state unless
        zero_state=False (then the group continues from the state its slot last held). Returns the
        event that marks the outputs of the pass's group complete, or None while the group is
        still being filled."""
        T, B, _ = self.shape
        k, g = self.k, self.k // self.P
        j, slot = k % self.P, g % 2
        self.k += 1
        cur = torch.cuda.current_stream(self.device)
        # copy-in: the slot's previous group (g-2) must have finished reading it
        if j == 0:
            self.s_in.wait_stream(cur)
            if g >= 2:
                self.s_in.wait_event(self.ev_run[slot])
        with torch.cuda.stream(self.s_in):
            if self.P == 1:
                self.x[slot].copy_(x_host, non_blocking=True)
                self.xs[slot].copy_(xs_host, non_blocking=True)
            else:
                self._block(self.x[slot], j).copy_(x_host, non_blocking=True)
                self.xs[slot].view(T, self.P, B)[:, j].copy_(xs_host.view(T, B), non_blocking=True)
            self.ev_in[slot].record()
        self.pending.append(out_host)
        if j == self.P - 1:
            return self._launch(slot, g, zero_state)
        self._zero_state = zero_state
        return None

    def _launch(self, slot, g, zero_state):
        # compute: after the group's inputs are in, and after the copy-out that last read this output buffer
        T, B, H = self.shape
        filled = len(self.pending)
        Bf = filled * B
        self.s_run.wait_event(self.ev_in[slot])
        if g >= 2:
            self.s_run.wait_event(self.ev_out[slot])
        lib = ops._L()
        prev_stream = lib.fluke_get_stream()
        lib.fluke_set_stream(self.s_run.cuda_stream)
        # a partly filled group runs over its own chunks only: the buffers are used as flat
        # memory holding [T, filled*B, H]
        flat = lambda t: t.view(-1)[:T * Bf * H].view(T, Bf, H)
        try:
            with torch.cuda.stream(self.s_run):
                state = [(c[:Bf], hs[:Bf]) for c, hs in self.state[slot]]
                if zero_state:
                    for c, hs in state:
                        c.zero_()
                        hs.zero_()
                if filled == self.P:
                    cur_x, cur_s = self.x[slot], self.xs[slot]
                else:
                    cur_x = flat(self.bufs[1])   # free until the second layer writes it
                    cur_x.view(T, filled, B, H).copy_(self.x[slot].view(T, self.P, B, H)[:, :filled])
                    cur_s = self.xs[slot].view(T, self.P, B)[:, :filled].reshape(T * Bf)
                out = flat(self.out[slot])
                n = len(self.layers)
                for i, layer in enumerate(self.layers):
                    c, hs = state[i]
                    dst = out if i == n - 1 else flat(self.bufs[i % 2])
                    ops.factored_lstm_layer_i8(cur_x, cur_s, layer.dn_ih, layer.dn_ih_scale, layer.dn_hh,
                                               layer.dn_hh_scale, layer.w_up, layer.bias, c, hs,
                                               reverse=layer.reverse, h_out=dst, workspace=self.ws)
                    cur_x, cur_s = dst, None
                self.ev_run[slot].record()
        finally:
            lib.fluke_set_stream(prev_stream)
        # copy-out
        self.s_out.wait_event(self.ev_run[slot])
        with torch.cuda.stream(self.s_out):
            for j, out_host in enumerate(self.pending):
                out_host.copy_(out if filled == 1 else out.view(T, filled, B, H)[:, j], non_blocking=True)
            self.ev_out[slot].record()
        self.pending = []
        return self.ev_out[slot]

    def drain(self):
        """Run a group that is only partly filled (over its own chunks only), then make the current
        stream wait for everything submitted so far."""
        if self.pending:
            g = (self.k - 1) // self.P
            self.k = (g + 1) * self.P   # the next pass starts a new group
            self._launch(g % 2, g, getattr(self, "_zero_state", True))
        cur = torch.cuda.current_stream(self.device)
        cur.wait_stream(self.s_in)
        cur.wait_stream(self.s_run)
        cur.wait_stream(self.s_out)
