"""GPU parity of the factored-LSTM kernels, called through the C ABI.

Bar (f16 tensor-core contraction, f32 accumulate in an unspecified order): cell state within
1e-2 of the oracle, no int8 hidden code off by more than 1; across a recurrent layer the same
bar holds per step while the fraction of differing codes stays small. Batch shards reproduce
the unsharded result bit for bit.
"""
import numpy as np
import pytest
import torch

from fluke_b200 import lib as L, ops, prep
from fluke_b200.lstm import FactoredLstmLayer, StackPipeline, run_stack, run_stack_c
from fluke_b200.shard import shard_range
from oracle import port

pytestmark = pytest.mark.gpu
DEV = "cuda"


# name -> (mode for fluke_set_lstm_persistent, form fluke_sm100_lstm_last_form then reports)
LSTM_MODES = {"cluster": (4, 1), "persistent_l2": (2, 2), "per_step": (0, 0)}


@pytest.fixture(params=list(LSTM_MODES))
def lstm_mode(request, flib):
    """Runs a test with each form of the layer recurrence: one launch with the exchange inside
    thread-block clusters, one launch with the exchange through L2, and two launches per step."""
    flib.fluke_set_lstm_persistent(LSTM_MODES[request.param][0])
    yield request.param
    flib.fluke_set_lstm_persistent(1)


@pytest.mark.parametrize("B,H,Kc", [(256, 1024, 256), (128, 768, 256), (100, 768, 256), (200, 96, 128), (1, 64, 64), (1024, 768, 256)])
def test_step_vs_oracle(B, H, Kc):
    g = torch.Generator().manual_seed(B + H)
    A = (torch.randn(B, Kc, generator=g) * 0.3).half(); W = (torch.randn(4 * H, Kc, generator=g) * 0.1).half()
    bias = torch.randn(4 * H, generator=g) * 0.1; c = torch.randn(B, H, generator=g) * 0.1
    cg = c.clone().to(DEV)
    hg = ops.factored_lstm_step_i8(A.to(DEV), W.to(DEV), bias.to(DEV), cg)
    ce, he = port.lstm_step(A.numpy(), W.numpy(), bias.numpy(), c.numpy())
    assert np.abs(cg.cpu().numpy() - ce).max() < 1e-4
    d = np.abs(hg.cpu().numpy().astype(np.int32) - he.astype(np.int32))
    assert d.max() <= 1 and (d != 0).mean() < 1e-3


def test_step_golden_from_reference_test(golden_tests):
    g = golden_tests
    H = g["lstm_c"].shape[1]
    A = np.concatenate([g["lstm_hh_down"], g["lstm_x_down"]], 1).astype(np.float16)
    W = np.concatenate([np.concatenate([g["lstm_up_hh"][k * H:(k + 1) * H], g["lstm_up_ih"][k * H:(k + 1) * H]], 1) for k in range(4)], 0).astype(np.float16)
    bias = (g["lstm_bhh"] + g["lstm_bih"]).astype(np.float32)
    T = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(DEV)
    c = T(g["lstm_c"])
    h = ops.factored_lstm_step_i8(T(A), T(W), T(bias), c)
    assert (c.cpu() - torch.from_numpy(g["lstm_c_ref"])).abs().max() < 0.08   # ABS_TOL of cute/test_factored_lstm.py
    assert (h.float().cpu() / 127.0 - torch.from_numpy(g["lstm_h_ref"])).abs().max() < 0.08


def test_fp8_export_step_golden_from_fly_reference_test(golden_tests):
    """The fused step of the reference's fp8 export (fly/rdna4/factored_lstm/rdna_fp8_factored_lstm.py)
    against the torch reference of fly/test_factored_lstm.py on inputs drawn as that test draws
    them; its bar (:66-72): cell < 1e-2, every int8 code within one level."""
    g = golden_tests
    T = lambda k: torch.from_numpy(np.ascontiguousarray(g[k])).to(DEV)
    c = T("flstm8_c0")
    h = ops.factored_lstm_step_i8(T("flstm8_A"), T("flstm8_W"), T("flstm8_bias"), c, fp8_export_name=True)
    assert (c.cpu() - torch.from_numpy(g["flstm8_c_ref"])).abs().max() < 1e-2
    d = (h.cpu().int() - torch.from_numpy(g["flstm8_h_ref"]).int()).abs()
    assert int(d.max()) <= 1
    # and the oracle on the same inputs: same bar against the reference, tighter against the kernel
    ce, he = port.lstm_step(g["flstm8_A"], g["flstm8_W"], g["flstm8_bias"], g["flstm8_c0"])
    assert np.abs(ce - g["flstm8_c_ref"]).max() < 1e-2 and np.abs(he.astype(np.int32) - g["flstm8_h_ref"].astype(np.int32)).max() <= 1
    assert np.abs(c.cpu().numpy() - ce).max() < 1e-4


@pytest.mark.parametrize("M", [48, 128, 1024, 300])
def test_fp8_down_projection_vs_oracle_and_fly_reference(golden_tests, M):
    """fluke_down_proj_fp8_gpu (N = R = 128, K = H = 768): against the oracle within 1e-2 of the
    output RMS (f32 accumulation order), against the reference construction of the fly tests
    within their 5e-2, and into a wider buffer (row stride)."""
    gt = golden_tests
    if M == 48:   # the fixture built with the reference's own fp8 quantisers
        a8, sa = torch.from_numpy(gt["dp8_A"]), torch.from_numpy(gt["dp8_sa"])
        w8 = torch.from_numpy(np.ascontiguousarray(gt["dp8_B_kn"].T)); sb = torch.from_numpy(gt["dp8_sb"])
    else:
        g = torch.Generator().manual_seed(M)
        a, sa = prep.quantize_fp8_rows(torch.randn(M, 768, generator=g) * 0.3)
        w, sb = prep.quantize_fp8_rows(torch.randn(128, 768, generator=g) / 768 ** 0.5)
        a8, w8 = a.view(torch.uint8), w.view(torch.uint8)
    buf = torch.full((M, 256), 3.0, dtype=torch.float16, device=DEV)
    ops.down_proj_fp8(a8.to(DEV), w8.to(DEV), sa.to(DEV), sb.to(DEV), out=buf[:, :128])
    got = buf[:, :128].float().cpu().numpy()
    assert bool((buf[:, 128:] == 3.0).all())
    exp = port.down_proj_fp8(a8.numpy(), w8.numpy(), sa.numpy(), sb.numpy()).astype(np.float32)
    assert np.abs(got - exp).max() <= 1e-2 * np.sqrt((exp ** 2).mean())
    if M == 48:
        assert np.abs(got - gt["dp8_expected"].astype(np.float32)).max() < 5e-2
    # a preshuffled weight, as the fp8 ABI passes it, goes through the re-ordering kernel once
    wsh = prep.preshuffle_fp8_weight(w8)
    plain = ops.fp8_unshuffle(wsh.to(DEV), 128, 768)
    again = ops.down_proj_fp8(a8.to(DEV), plain, sa.to(DEV), sb.to(DEV))
    assert torch.equal(again, buf[:, :128])


def test_per_step_entry_points_with_an_explicit_stream(flib):
    """The `_stream` forms of the two per-step kernels launch on the stream they are given (here a
    side stream while the thread's own setting stays the default stream) and give the bytes of the
    forms without it; a step loop driven this way equals the layer entry point's per-step mode."""
    T, B, H, R = 4, 200, 768, 128
    layer, x, xs = _layer_case(T, B, H, R, 21, False)
    X, XS = x.to(DEV), xs.to(DEV)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    c = torch.zeros(B, H, device=DEV); h = torch.zeros(B, H, dtype=torch.int8, device=DEV)
    A = torch.empty(B, 2 * R, dtype=torch.float16, device=DEV)
    outs = []
    w = [layer.w_up.data_ptr() + g * H * 2 * R * 2 for g in range(4)]
    bs = [layer.bias.data_ptr() + g * H * 4 for g in range(4)]
    assert flib.fluke_get_stream() is None
    with torch.cuda.stream(side):
        for t in range(T):
            assert flib.fluke_down_proj_i8_stream_gpu(A.data_ptr(), 2 * R, h.data_ptr(), layer.dn_hh.data_ptr(), 0,
                                                      layer.dn_hh_scale.data_ptr(), B, R, H, side.cuda_stream) == 0
            assert flib.fluke_down_proj_i8_stream_gpu(A.data_ptr() + 2 * R, 2 * R, X[t].data_ptr(), layer.dn_ih.data_ptr(),
                                                      XS[t * B:(t + 1) * B].data_ptr(), layer.dn_ih_scale.data_ptr(), B, R, H,
                                                      side.cuda_stream) == 0
            hn = torch.empty(B, H, dtype=torch.int8, device=DEV)
            assert flib.fluke_factored_lstm_step_i8_stream_gpu(A.data_ptr(), w[0], w[1], w[2], w[3], bs[0], bs[1], bs[2], bs[3],
                                                               c.data_ptr(), hn.data_ptr(), B, H, 2 * R, side.cuda_stream) == 0
            h = hn
            outs.append(hn)
    side.synchronize()
    flib.fluke_set_lstm_persistent(0)
    c2 = torch.zeros(B, H, device=DEV); h2 = torch.zeros(B, H, dtype=torch.int8, device=DEV)
    want = ops.factored_lstm_layer_i8(X, XS, layer.dn_ih, layer.dn_ih_scale, layer.dn_hh, layer.dn_hh_scale, layer.w_up, layer.bias, c2, h2)
    flib.fluke_set_lstm_persistent(1)
    assert torch.equal(torch.stack(outs), want) and torch.equal(c, c2)


def test_hidden_quantiser_rounds_half_away_from_zero():
    """Gates forced open (large o bias, zero weights): h = tanh(c); codes at +-k.5/127 round away."""
    B, H, Kc = 128, 64, 64
    ks = torch.arange(0, 64).float()
    target = (ks + 0.5) / 127.0
    c_prev = torch.atanh(target.clamp(max=0.999)).repeat(B, 1)
    c_prev[::2] *= -1
    A = torch.zeros(B, Kc, dtype=torch.float16); W = torch.zeros(4 * H, Kc, dtype=torch.float16)
    bias = torch.zeros(4 * H); bias[H:2 * H] = 10.0; bias[3 * H:] = 10.0   # f = 1, o = 1, i*g = 0.5*0
    cg = c_prev.clone().to(DEV)
    h = ops.factored_lstm_step_i8(A.to(DEV), W.to(DEV), bias.to(DEV), cg).cpu()
    _, he = port.lstm_step(A.numpy(), W.numpy(), bias.numpy(), c_prev.numpy())
    assert np.abs(h.numpy().astype(np.int32) - he.astype(np.int32)).max() <= 1
    assert torch.equal(h[0], -h[1])  # symmetric rounding


def _layer_case(T, B, H, R, seed, reverse):
    g = torch.Generator().manual_seed(seed)
    layer = FactoredLstmLayer.random(H, R, reverse, g, DEV)
    x, xs = prep.quantize_int8_rows(torch.randn(T * B, H, generator=g))
    return layer, x.view(T, B, H), xs


def _run_oracle_layer(layer, x, xs, reverse, c0=None, h0=None):
    B, H = x.shape[1], x.shape[2]
    c0 = np.zeros((B, H), np.float32) if c0 is None else c0
    h0 = np.zeros((B, H), np.int8) if h0 is None else h0
    n = lambda t: t.cpu().numpy()
    return port.lstm_layer(x.numpy(), None if xs is None else xs.numpy(), n(layer.dn_ih), n(layer.dn_ih_scale), n(layer.dn_hh),
                           n(layer.dn_hh_scale), n(layer.w_up), n(layer.bias), c0, h0, reverse)


@pytest.mark.parametrize("T,B,reverse", [(12, 200, False), (12, 200, True), (40, 128, False), (3, 1, True),
                                         (6, 330, True), (5, 60, False)])
def test_layer_vs_oracle(T, B, reverse, lstm_mode):
    H, R = 768, 128
    layer, x, xs = _layer_case(T, B, H, R, 42 + T, reverse)
    c = torch.zeros(B, H, device=DEV); h = torch.zeros(B, H, dtype=torch.int8, device=DEV)
    ho = ops.factored_lstm_layer_i8(x.to(DEV), xs.to(DEV), layer.dn_ih, layer.dn_ih_scale, layer.dn_hh, layer.dn_hh_scale,
                                    layer.w_up, layer.bias, c, h, reverse=reverse)
    assert L.load().fluke_sm100_lstm_last_form() == LSTM_MODES[lstm_mode][1]  # each form covers this shape
    he, ce, hf = _run_oracle_layer(layer, x, xs, reverse)
    d = np.abs(ho.cpu().numpy().astype(np.int32) - he.astype(np.int32))
    assert d.max() <= 1 and (d != 0).mean() < 5e-3
    assert np.abs(c.cpu().numpy() - ce).max() < 1e-2
    last = 0 if reverse else T - 1
    assert torch.equal(h, ho[last])  # final hidden state = last written step


def test_layer_resumes_from_state_and_fixed_scale_input(lstm_mode):
    """Two halves run back to back (state carried in c/h) equal one run; input at the fixed
    1/127 scale (x_scale NULL) as for layers fed by a previous layer."""
    T, B, H, R = 10, 130, 768, 128
    layer, x, _ = _layer_case(T, B, H, R, 7, False)
    run = lambda xx, c, h: ops.factored_lstm_layer_i8(xx.to(DEV), None, layer.dn_ih, layer.dn_ih_scale, layer.dn_hh, layer.dn_hh_scale,
                                                      layer.w_up, layer.bias, c, h)
    c1 = torch.zeros(B, H, device=DEV); h1 = torch.zeros(B, H, dtype=torch.int8, device=DEV)
    whole = run(x, c1, h1)
    c2 = torch.zeros(B, H, device=DEV); h2 = torch.zeros(B, H, dtype=torch.int8, device=DEV)
    first = run(x[:5].contiguous(), c2, h2); second = run(x[5:].contiguous(), c2, h2)
    assert torch.equal(whole, torch.cat([first, second])) and torch.equal(c1, c2) and torch.equal(h1, h2)
    he, _, _ = _run_oracle_layer(layer, x, None, False)
    assert np.abs(whole.cpu().numpy().astype(np.int32) - he.astype(np.int32)).max() <= 1


def test_stack_alternating_directions_and_batch_shards(lstm_mode):
    """3-layer stack (odd layer reversed): sharding the chunk axis over 2 'ranks' reproduces
    the unsharded output bit for bit; the stack agrees with the oracle stack within one code
    per layer input."""
    T, B, H, R = 8, 192, 768, 128
    g = torch.Generator().manual_seed(1)
    layers = [FactoredLstmLayer.random(H, R, bool(i % 2), g, DEV) for i in range(3)]
    x, xs = prep.quantize_int8_rows(torch.randn(T * B, H, generator=g))
    x = x.view(T, B, H); xs2 = xs.view(T, B)
    full, _ = run_stack(layers, x.to(DEV), xs.to(DEV))
    full = full.clone()
    parts = []
    for rank in range(2):
        b0, b1 = shard_range(B, rank, 2)
        out, _ = run_stack(layers, x[:, b0:b1].contiguous().to(DEV), xs2[:, b0:b1].contiguous().view(-1).to(DEV))
        parts.append(out.clone())
    assert torch.equal(full, torch.cat(parts, dim=1))
    # oracle stack, feeding each layer the ORACLE's own previous output
    cur, cur_s = x, xs
    for layer in layers:
        he, _, _ = _run_oracle_layer(layer, cur, cur_s, layer.reverse)
        cur, cur_s = torch.from_numpy(he), None
    d = np.abs(full.cpu().numpy().astype(np.int32) - cur.numpy().astype(np.int32))
    assert d.max() <= 2 and (d > 1).mean() < 1e-3 and (d != 0).mean() < 2e-2


def test_stack_entry_point_equals_layer_by_layer(flib):
    """fluke_factored_lstm_stack_i8_gpu (one C call per pass) gives the bytes and the final state
    of the layer-by-layer loop; 4 layers (even count: the first layer writes the scratch buffer)
    and a single layer (no scratch buffer needed)."""
    T, B, H, R = 6, 200, 768, 128
    g = torch.Generator().manual_seed(5)
    x, xs = prep.quantize_int8_rows(torch.randn(T * B, H, generator=g))
    X, XS = x.view(T, B, H).to(DEV), xs.to(DEV)
    for n_layers in (4, 1, 3):
        layers = [FactoredLstmLayer.random(H, R, bool(i % 2), g, DEV) for i in range(n_layers)]
        want, state = run_stack(layers, X, XS)
        got, (c, h) = run_stack_c(layers, X, XS)
        assert torch.equal(got, want)
        for i in range(n_layers):
            assert torch.equal(c[i], state[i][0]) and torch.equal(h[i], state[i][1])
    assert flib.fluke_factored_lstm_stack_i8_gpu(None, 0, T, B, H, R, 0, 0, 0, 0, 0, 0, 0, 0) != 0  # bad arguments: refused


def test_persistent_and_per_step_layers_agree(flib):
    """Same layer through all three drivers: the only difference is the accumulation order of the two
    K halves, so codes differ by at most one, rarely. Also other hidden sizes (1024, 384 with an odd
    number of 128-byte K blocks, 512), batches that are not a multiple of the 128-row tile and one
    with more row tiles than one single-launch kernel holds."""
    for (T, B, H) in [(16, 300, 768), (6, 130, 1024), (5, 1024, 768), (4, 140, 384), (4, 70, 512), (3, 1100, 768)]:
        layer, x, xs = _layer_case(T, B, H, 128, 11 + B, False)
        outs = []
        for mode in (4, 2, 0):
            flib.fluke_set_lstm_persistent(mode)
            c = torch.zeros(B, H, device=DEV); h = torch.zeros(B, H, dtype=torch.int8, device=DEV)
            outs.append((ops.factored_lstm_layer_i8(x.to(DEV), xs.to(DEV), layer.dn_ih, layer.dn_ih_scale, layer.dn_hh,
                                                    layer.dn_hh_scale, layer.w_up, layer.bias, c, h).clone(), c, h))
        flib.fluke_set_lstm_persistent(1)
        for other in (outs[1], outs[2]):
            d = (outs[0][0].int() - other[0].int()).abs()
            assert int(d.max()) <= 1 and float((d != 0).float().mean()) < 5e-3
            assert float((outs[0][1] - other[1]).abs().max()) < 1e-2
            assert torch.equal(outs[0][2], outs[0][0][-1]) and torch.equal(other[2], other[0][-1])
        he, ce, _ = _run_oracle_layer(layer, x, xs, False)
        d = np.abs(outs[0][0].cpu().numpy().astype(np.int32) - he.astype(np.int32))
        assert d.max() <= 1 and (d != 0).mean() < 5e-3


def test_cluster_form_runs_in_rounds_when_nothing_else_covers_the_shape(flib):
    """H = 192 is outside the L2-exchange form (H % 128) and 17 row tiles are more clusters than
    fit at once, so the cluster form runs them in rounds; a ragged last tile as well."""
    T, B, H, R = 4, 2100, 192, 128
    layer, x, xs = _layer_case(T, B, H, R, 5, True)
    c = torch.zeros(B, H, device=DEV); h = torch.zeros(B, H, dtype=torch.int8, device=DEV)
    flib.fluke_set_lstm_persistent(4)
    ho = ops.factored_lstm_layer_i8(x.to(DEV), xs.to(DEV), layer.dn_ih, layer.dn_ih_scale, layer.dn_hh, layer.dn_hh_scale,
                                    layer.w_up, layer.bias, c, h, reverse=True)
    flib.fluke_set_lstm_persistent(1)
    assert flib.fluke_sm100_lstm_last_form() == 1
    he, ce, _ = _run_oracle_layer(layer, x, xs, True)
    d = np.abs(ho.cpu().numpy().astype(np.int32) - he.astype(np.int32))
    assert d.max() <= 1 and (d != 0).mean() < 5e-3
    assert np.abs(c.cpu().numpy() - ce).max() < 1e-2


def test_layer_config_size_properties(lstm_mode):
    """H = 768, R = 128, B = 1024 (T cut to 24): codes stay in [-127, 127], the first step of a
    zero state matches the single-step kernel on [0 | x_down], and the reversed layer on
    time-flipped input equals the flipped forward output."""
    T, B, H, R = 24, 1024, 768, 128
    layer, x, xs = _layer_case(T, B, H, R, 3, False)
    X, XS = x.to(DEV), xs.to(DEV)
    args = (layer.dn_ih, layer.dn_ih_scale, layer.dn_hh, layer.dn_hh_scale, layer.w_up, layer.bias)
    c = torch.zeros(B, H, device=DEV); h = torch.zeros(B, H, dtype=torch.int8, device=DEV)
    fwd = ops.factored_lstm_layer_i8(X, XS, *args, c, h, reverse=False).clone()
    form = L.load().fluke_sm100_lstm_last_form()
    assert form == LSTM_MODES[lstm_mode][1]
    assert int(fwd.min()) >= -127
    c2 = torch.zeros(B, H, device=DEV); h2 = torch.zeros(B, H, dtype=torch.int8, device=DEV)
    rev = ops.factored_lstm_layer_i8(X.flip(0).contiguous(), XS.view(T, B).flip(0).contiguous().view(-1), *args, c2, h2, reverse=True)
    assert torch.equal(rev.flip(0), fwd) and torch.equal(c, c2)
    xd = ops.down_proj_i8(X[0], layer.dn_ih, XS[:B].contiguous(), layer.dn_ih_scale)
    A = torch.cat([torch.zeros(B, R, dtype=torch.float16, device=DEV), xd], dim=1).contiguous()
    c3 = torch.zeros(B, H, device=DEV)
    h3 = ops.factored_lstm_step_i8(A, layer.w_up, layer.bias, c3)
    d = (h3.int() - fwd[0].int()).abs()   # the persistent kernel uses the fast-exp tanh: rare one-code ties
    assert int(d.max()) <= 1 and float((d != 0).float().mean()) < 1e-3
    if lstm_mode == "per_step":
        assert torch.equal(h3, fwd[0])


def test_two_batches_side_by_side_config_size(flib):
    """Two benchmark-size batches (2 x 1024 chunks, H = 768, R = 128; T cut to 24) in one layer
    call, which the wide L2-exchange configuration runs in a single launch of 16 row tiles, give
    the bytes of the two batches run on their own (narrow configuration, 8 row tiles each)."""
    T, B, H, R = 24, 1024, 768, 128
    flib.fluke_set_lstm_persistent(2)
    layer, x, xs = _layer_case(T, 2 * B, H, R, 9, True)
    X, XS = x.to(DEV), xs.to(DEV)
    args = (layer.dn_ih, layer.dn_ih_scale, layer.dn_hh, layer.dn_hh_scale, layer.w_up, layer.bias)
    c = torch.zeros(2 * B, H, device=DEV); h = torch.zeros(2 * B, H, dtype=torch.int8, device=DEV)
    both = ops.factored_lstm_layer_i8(X, XS, *args, c, h, reverse=True).clone()
    assert flib.fluke_sm100_lstm_last_form() == 2
    for j in range(2):
        xj = X[:, j * B:(j + 1) * B].contiguous()
        xsj = XS.view(T, 2 * B)[:, j * B:(j + 1) * B].contiguous().view(-1)
        cj = torch.zeros(B, H, device=DEV); hj = torch.zeros(B, H, dtype=torch.int8, device=DEV)
        one = ops.factored_lstm_layer_i8(xj, xsj, *args, cj, hj, reverse=True)
        assert torch.equal(one, both[:, j * B:(j + 1) * B])
        assert torch.equal(cj, c[j * B:(j + 1) * B]) and torch.equal(hj, h[j * B:(j + 1) * B])
    flib.fluke_set_lstm_persistent(1)


@pytest.mark.parametrize("passes_per_launch,time_chunks", [(1, 1), (2, 1), (2, 3), (1, 4)])
def test_streaming_pipeline_equals_pass_by_pass(passes_per_launch, time_chunks):
    """Five passes with different inputs through the three-stream driver (copy-in, layers,
    copy-out overlapped across groups of passes) give the bytes of run_stack on each input alone;
    with two passes per launch the fifth is a group of its own that `drain` runs; with time chunks
    the first and the last layer run block by block between their copies."""
    T, B, H, R, NL = 6, 200, 768, 128, 3
    g = torch.Generator().manual_seed(77)
    layers = [FactoredLstmLayer.random(H, R, bool(i % 2), g, DEV) for i in range(NL)]
    pipe = StackPipeline(layers, T, B, DEV, passes_per_launch=passes_per_launch, time_chunks=time_chunks)
    ins, outs = [], []
    for k in range(5):
        x, xs = prep.quantize_int8_rows(torch.randn(T * B, H, generator=g))
        ins.append((x.view(T, B, H).contiguous().pin_memory(), xs.contiguous().pin_memory()))
        outs.append(torch.empty(T, B, H, dtype=torch.int8).pin_memory())
    for k in range(5):
        pipe.submit(ins[k][0], ins[k][1], outs[k])
    pipe.drain()
    torch.cuda.synchronize()
    for k in range(5):
        ref, _ = run_stack(layers, ins[k][0].to(DEV), ins[k][1].to(DEV))
        assert torch.equal(outs[k], ref.cpu())


def test_streaming_pipeline_launches_full_groups_and_flush_launches_a_partial_one():
    """With two passes per launch, `submit` of a lone pass only queues it (its output buffer stays
    untouched however long one waits); `flush` launches it without blocking, and the bytes are
    those of the pass alone."""
    T, B, H, R, NL = 4, 130, 768, 128, 2
    g = torch.Generator().manual_seed(78)
    layers = [FactoredLstmLayer.random(H, R, bool(i % 2), g, DEV) for i in range(NL)]
    pipe = StackPipeline(layers, T, B, DEV, passes_per_launch=2, time_chunks=2)
    x, xs = prep.quantize_int8_rows(torch.randn(T * B, H, generator=g))
    x, xs = x.view(T, B, H).contiguous().pin_memory(), xs.contiguous().pin_memory()
    out = torch.full((T, B, H), 77, dtype=torch.int8).pin_memory()
    pipe.submit(x, xs, out)
    torch.cuda.synchronize()
    assert bool((out == 77).all())          # nothing was launched
    pipe.flush()
    pipe.drain()
    ref, _ = run_stack(layers, x.to(DEV), xs.to(DEV))
    assert torch.equal(out, ref.cpu())
    pipe.close()


def test_wide_l2_configuration_matches_the_narrow_one(flib):
    """The L2-exchange form with 48 units per gate CTA and one worker per row tile (chosen by itself
    when a layer has more row tiles than a narrow launch holds) computes every element in the same
    order as the narrow configuration: identical bytes. Shapes: ragged tiles, H = 384, and a batch
    of 2100 chunks (17 row tiles: one full wide launch and a second one)."""
    for (T, B, H) in [(6, 300, 768), (5, 130, 384), (3, 2100, 768), (4, 1, 768)]:
        layer, x, xs = _layer_case(T, B, H, 128, 3 + B, False)
        res = []
        for wide in (0, 1, -1):
            flib.fluke_set_lstm_persistent(2)
            flib.fluke_sm100_set_lstm_wide(wide)
            c = torch.zeros(B, H, device=DEV); h = torch.zeros(B, H, dtype=torch.int8, device=DEV)
            out = ops.factored_lstm_layer_i8(x.to(DEV), xs.to(DEV), layer.dn_ih, layer.dn_ih_scale, layer.dn_hh,
                                             layer.dn_hh_scale, layer.w_up, layer.bias, c, h)
            assert flib.fluke_sm100_lstm_last_form() == 2
            res.append((out.clone(), c.clone(), h.clone()))
        flib.fluke_sm100_set_lstm_wide(-1)
        flib.fluke_set_lstm_persistent(1)
        for other in res[1:]:
            assert torch.equal(res[0][0], other[0]) and torch.equal(res[0][1], other[1]) and torch.equal(res[0][2], other[2])
        he, ce, _ = _run_oracle_layer(layer, x, xs, False)
        d = np.abs(res[1][0].cpu().numpy().astype(np.int32) - he.astype(np.int32))
        assert d.max() <= 1 and (d != 0).mean() < 5e-3
