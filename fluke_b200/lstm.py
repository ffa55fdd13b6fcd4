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
    A group is launched when it is full, or earlier when nothing is running (a job therefore
    starts with a single pass, which halves the fill time), or by `drain()`, which runs a group
    that is only partly filled; the results of a pass are complete when its group has run.

    Device memory: two input sets, the two ping-pong layer buffers and two output buffers of
    [T,P*B,H] int8. Inputs and outputs are pinned host tensors; `submit` only enqueues work."""

    def __init__(self, layers, T, B, device, passes_per_launch=1, time_chunks=1):
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
        self.ev_run = [torch.cuda.Event() for _ in range(2)]    # group that used slot g%2 finished computing
        self.ev_out = [torch.cuda.Event() for _ in range(2)]    # output buffer g%2 copied out
        self.k = 0          # passes submitted
        self.g = 0          # groups launched
        self._last_run = None
        self._zero_state = True
        self.pending = []   # (x_host, xs_host, out_host) of the group being filled
        # time_chunks = C > 1: the first layer runs in C calls over consecutive blocks of timesteps
        # (state carried from call to call: the same bytes), each as soon as its block has been
        # copied in, and the last layer likewise, each block copied out as soon as it is written.
        # That overlaps the copies of a group with its OWN layers: it shortens the fill and the
        # drain of the pipeline (copies of other groups are overlapped in any case).
        C = max(1, min(int(time_chunks), T))
        edges = [round(i * T / C) for i in range(C + 1)]
        self.t_blocks = [(edges[i], edges[i + 1]) for i in range(C) if edges[i + 1] > edges[i]]
        self.ev_blk_in = [[torch.cuda.Event() for _ in self.t_blocks] for _ in range(2)]
        self.ev_blk_run = [[torch.cuda.Event() for _ in self.t_blocks] for _ in range(2)]

    def submit(self, x_host, xs_host, out_host, zero_state=True):
        """Enqueue one pass: x_host int8 [T,B,H] and xs_host f32 [T*B] (pinned) in, the last layer's
        int8 output into out_host (pinned). Every pass starts from a zero state unless
        zero_state=False (then the group continues from the state its slot last held). The work
        of a group (copies included) is enqueued when the group is full, when nothing is running
        (so a job starts with a group of one pass), or by `drain`.
        Returns the event that marks the outputs of the pass's group complete, or None while the
        group is still being filled."""
        self.k += 1
        self.pending.append((x_host, xs_host, out_host))
        self._zero_state = zero_state
        # a full group, or nothing running: waiting for more passes would only leave the GPU idle
        # (this is what starts a job with a single pass, and halves the pipeline's fill time)
        if len(self.pending) == self.P or self._idle():
            return self._launch_pending()
        return None

    def _idle(self):
        return self._last_run is None or self._last_run.query()

    def _launch_pending(self):
        g = self.g
        self.g += 1
        ev = self._launch(g % 2, g, self._zero_state)
        self._last_run = self.ev_run[g % 2]
        return ev

    @staticmethod
    def _copy_rows(dst, src, stream, to_device):
        """dst, src: tensors of equal shape [rows, ...] whose rows are contiguous; one of them may
        have a row pitch larger than the row (a column block of a wider tensor)."""
        rows = dst.shape[0]
        width = dst[0].numel() * dst.element_size()
        rc = ops._L().fluke_sm100_copy_rows_async(dst.data_ptr(), dst.stride(0) * dst.element_size(), src.data_ptr(),
                                                  src.stride(0) * src.element_size(), width, rows, 1 if to_device else 0,
                                                  stream.cuda_stream)
        if rc:
            raise RuntimeError(f"strided copy failed: CUDA error {rc}")

    def _blocks_for(self, layer):
        """The layer's blocks of timesteps in the order it walks them."""
        return list(reversed(self.t_blocks)) if layer.reverse else self.t_blocks

    def _launch(self, slot, g, zero_state):
        T, B, H = self.shape
        filled = len(self.pending)
        Bf = filled * B
        n = len(self.layers)
        # a partly filled group runs over its own chunks only: the buffers are used as flat
        # memory holding [T, filled*B, ...]
        flat = lambda t: t.view(-1)[:T * Bf * H].view(T, Bf, H)
        x_dev, out_dev = flat(self.x[slot]), flat(self.out[slot])
        xs_dev = self.xs[slot][:T * Bf]
        first_blocks, last_blocks = self._blocks_for(self.layers[0]), self._blocks_for(self.layers[n - 1])
        cur = torch.cuda.current_stream(self.device)
        # copy-in, block by block in the order the first layer needs them; the slot's previous
        # group (g-2) must have finished reading the buffers
        self.s_in.wait_stream(cur)
        if g >= 2:
            self.s_in.wait_event(self.ev_run[slot])
        with torch.cuda.stream(self.s_in):
            for (t0, t1) in first_blocks:
                for j, (x_host, xs_host, _) in enumerate(self.pending):
                    if filled == 1:
                        x_dev[t0:t1].copy_(x_host[t0:t1], non_blocking=True)
                        xs_dev[t0 * B:t1 * B].copy_(xs_host[t0 * B:t1 * B], non_blocking=True)
                    else:
                        # pass j's columns of every timestep plane: a strided copy by the copy
                        # engine itself (torch would stage it and run a kernel beside the layers)
                        self._copy_rows(x_dev[t0:t1].view(t1 - t0, filled, B, H)[:, j], x_host[t0:t1], self.s_in, True)
                        self._copy_rows(xs_dev[t0 * Bf:t1 * Bf].view(t1 - t0, filled, B)[:, j],
                                        xs_host[t0 * B:t1 * B].view(t1 - t0, B), self.s_in, True)
                self.ev_blk_in[slot][self.t_blocks.index((t0, t1))].record()
        # compute: after the copy-out that last read this output buffer
        if g >= 2:
            self.s_run.wait_event(self.ev_out[slot])
        lib = ops._L()
        prev_stream = lib.fluke_get_stream()
        lib.fluke_set_stream(self.s_run.cuda_stream)
        try:
            with torch.cuda.stream(self.s_run):
                state = [(c[:Bf], hs[:Bf]) for c, hs in self.state[slot]]
                if zero_state:
                    for c, hs in state:
                        c.zero_()
                        hs.zero_()
                cur_x, cur_s = x_dev, xs_dev
                for i, layer in enumerate(self.layers):
                    c, hs = state[i]
                    dst = out_dev if i == n - 1 else flat(self.bufs[i % 2])
                    # first and last layer: one call per block of timesteps, state carried over
                    blocks = self._blocks_for(layer) if (i == 0 or i == n - 1) else [(0, T)]
                    for (t0, t1) in blocks:
                        if i == 0:
                            self.s_run.wait_event(self.ev_blk_in[slot][self.t_blocks.index((t0, t1))])
                        ops.factored_lstm_layer_i8(cur_x[t0:t1], None if cur_s is None else cur_s[t0 * Bf:t1 * Bf],
                                                   layer.dn_ih, layer.dn_ih_scale, layer.dn_hh, layer.dn_hh_scale,
                                                   layer.w_up, layer.bias, c, hs, reverse=layer.reverse,
                                                   h_out=dst[t0:t1], workspace=self.ws)
                        if i == n - 1:
                            self.ev_blk_run[slot][self.t_blocks.index((t0, t1))].record()
                    cur_x, cur_s = dst, None
                self.ev_run[slot].record()
        finally:
            lib.fluke_set_stream(prev_stream)
        # copy-out, block by block as the last layer writes them
        with torch.cuda.stream(self.s_out):
            for (t0, t1) in last_blocks:
                self.s_out.wait_event(self.ev_blk_run[slot][self.t_blocks.index((t0, t1))])
                for j, (_, _, out_host) in enumerate(self.pending):
                    if filled == 1:
                        out_host[t0:t1].copy_(out_dev[t0:t1], non_blocking=True)
                    else:
                        self._copy_rows(out_host[t0:t1], out_dev[t0:t1].view(t1 - t0, filled, B, H)[:, j], self.s_out, False)
            self.ev_out[slot].record()
        self.pending = []
        return self.ev_out[slot]

    def drain(self):
        """Run a group that is only partly filled (over its own chunks only), then make the current
        stream wait for everything submitted so far."""
        if self.pending:
            self._launch_pending()
        cur = torch.cuda.current_stream(self.device)
        cur.wait_stream(self.s_in)
        cur.wait_stream(self.s_run)
        cur.wait_stream(self.s_out)
