"""fluke_factored_lstm_layer_i8_noalloc_gpu: the LSTM layer for callers that cannot allocate
device memory (plug-ins that are given device pointers but have no allocator, services with a
memory budget fixed at start-up, code in regions where the CUDA allocator must not be called).
It keeps its intermediates in an array built into the library instead of a caller workspace.

Called through the C ABI and compared with the workspace-taking entry point on the same inputs,
twice in a row with different shapes, so the second call starts with the first call's leftovers
in the shared array. Collected last so that a failure here cannot hide other tests.
"""
import ctypes

import numpy as np
import pytest
import torch

from fluke_b200 import lib as L, ops, prep
from fluke_b200.lstm import FactoredLstmLayer

pytestmark = pytest.mark.gpu
DEV = "cuda"
SCRATCH_BYTES = 4 << 20  # FLUKE_LSTM_NOALLOC_SCRATCH_BYTES


def _call_noalloc(layer, x, xs, c, h, reverse):
    t, b, hd = x.shape
    out = torch.empty(t, b, hd, dtype=torch.int8, device=DEV)
    desc = L.fluke_flstm_layer_t(t, b, hd, layer.rank, int(reverse), x.data_ptr(), 0 if xs is None else xs.data_ptr(),
                                 layer.dn_ih.data_ptr(), layer.dn_ih_scale.data_ptr(), layer.dn_hh.data_ptr(),
                                 layer.dn_hh_scale.data_ptr(), layer.w_up.data_ptr(), layer.bias.data_ptr(),
                                 c.data_ptr(), h.data_ptr(), out.data_ptr(), 0, 0)  # no workspace passed
    rc = L.load().fluke_factored_lstm_layer_i8_noalloc_gpu(ctypes.byref(desc))
    return rc, out


@pytest.fixture(params=[1, 4, 2, 0], ids=["default", "cluster", "l2_exchange", "per_step"])
def form(request):
    """Every way the layer can run keeps different intermediates in the shared array: the cluster
    form only x_down, the L2-exchange form also hh_down and its exchange counters, the per-step
    kernels hh_down. The leftovers of the previous call must be harmless in each."""
    L.load().fluke_set_lstm_persistent(request.param)
    yield request.param
    L.load().fluke_set_lstm_persistent(1)


@pytest.mark.parametrize("first,second", [((5, 300, False), (3, 130, True))])
def test_noalloc_layer_matches_workspace_layer_on_two_calls_in_a_row(first, second, form):
    H, R = 768, 128
    g = torch.Generator().manual_seed(2024)
    layer = FactoredLstmLayer.random(H, R, False, g, DEV)
    for (T, B, reverse) in (first, second):
        assert L.load().fluke_factored_lstm_layer_workspace(T, B, H, R) <= SCRATCH_BYTES
        x, xs = prep.quantize_int8_rows(torch.randn(T * B, H, generator=g))
        x, xs = x.view(T, B, H).to(DEV), xs.to(DEV)
        c0 = (torch.randn(B, H, generator=g) * 0.1).to(DEV)
        h0 = torch.randint(-127, 128, (B, H), generator=g, dtype=torch.int8).to(DEV)
        c_ref, h_ref = c0.clone(), h0.clone()
        want = ops.factored_lstm_layer_i8(x, xs, layer.dn_ih, layer.dn_ih_scale, layer.dn_hh, layer.dn_hh_scale,
                                          layer.w_up, layer.bias, c_ref, h_ref, reverse=reverse)
        c_got, h_got = c0.clone(), h0.clone()
        rc, got = _call_noalloc(layer, x, xs, c_got, h_got, reverse)
        torch.cuda.synchronize()
        assert rc == 0
        d = (got.int() - want.int()).abs()
        assert int(d.max()) <= 1 and float((d != 0).float().mean()) < 5e-3   # the LSTM tests' tolerance
        assert float((c_got - c_ref).abs().max()) < 1e-2
        # same kernels on the same inputs: in fact identical
        assert torch.equal(got, want) and torch.equal(c_got, c_ref) and torch.equal(h_got, h_ref)


def test_noalloc_layer_size_limit_is_exact(capfd):
    """At 1024 chunks and rank 128 the intermediates of 14 timesteps fit the 4 MiB array and those
    of 15 do not: the first runs (and equals the workspace entry point), the second is refused."""
    H, R, B = 768, 128, 1024
    lib = L.load()
    assert lib.fluke_factored_lstm_layer_workspace(14, B, H, R) <= SCRATCH_BYTES < lib.fluke_factored_lstm_layer_workspace(15, B, H, R)
    g = torch.Generator().manual_seed(3)
    layer = FactoredLstmLayer.random(H, R, False, g, DEV)
    x, xs = prep.quantize_int8_rows(torch.randn(15 * B, H, generator=g))
    x, xs = x.view(15, B, H).to(DEV), xs.to(DEV)
    c = torch.zeros(B, H, device=DEV); h = torch.zeros(B, H, dtype=torch.int8, device=DEV)
    rc, got = _call_noalloc(layer, x[:14].contiguous(), xs[:14 * B].contiguous(), c, h, False)
    torch.cuda.synchronize()
    assert rc == 0
    c2 = torch.zeros(B, H, device=DEV); h2 = torch.zeros(B, H, dtype=torch.int8, device=DEV)
    want = ops.factored_lstm_layer_i8(x[:14].contiguous(), xs[:14 * B].contiguous(), layer.dn_ih, layer.dn_ih_scale, layer.dn_hh,
                                      layer.dn_hh_scale, layer.w_up, layer.bias, c2, h2)
    assert torch.equal(got, want) and torch.equal(c, c2)
    c.zero_()
    rc, _ = _call_noalloc(layer, x, xs, c, h, False)
    torch.cuda.synchronize()
    assert rc != 0 and "built-in buffer" in capfd.readouterr().err and not bool(c.any())


def test_noalloc_layer_refuses_layers_beyond_its_buffer(capfd):
    H, R, T, B = 768, 128, 64, 1024
    assert L.load().fluke_factored_lstm_layer_workspace(T, B, H, R) > SCRATCH_BYTES
    layer = FactoredLstmLayer.random(H, R, False, torch.Generator().manual_seed(1), DEV)
    x = torch.zeros(T, B, H, dtype=torch.int8, device=DEV)
    c = torch.zeros(B, H, device=DEV)
    h = torch.zeros(B, H, dtype=torch.int8, device=DEV)
    rc, _ = _call_noalloc(layer, x, None, c, h, False)
    torch.cuda.synchronize()
    assert rc != 0
    assert "built-in buffer" in capfd.readouterr().err
    assert not bool(c.any())  # nothing ran
