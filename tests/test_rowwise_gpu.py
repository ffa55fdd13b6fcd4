"""GPU parity of the memory-bound kernels, called through the C ABI (ctypes on lib/libfluke.so).

Bar: bit-exact against the reference's own CUDA kernels -- both the committed B200 capture
(tests/golden/reference_cuda_kernels.npz) and, when oracle/_ref is present, the reference
library run side by side on larger seeded inputs; plus the CPU oracle at the benchmark sizes
and size-independent properties.
"""
import numpy as np
import pytest
import torch

import cases
from fluke_b200 import ops, prep
from oracle import port, ref

pytestmark = pytest.mark.gpu
DEV = "cuda"


def D(a):
    return torch.from_numpy(np.ascontiguousarray(a)).to(DEV)


def bits(t):
    return t.contiguous().view(torch.int16 if t.element_size() == 2 else torch.int32 if t.element_size() == 4 else torch.uint8)


def same_bits(a, b):
    return torch.equal(bits(a), bits(b))


# ---- against the committed capture of the reference's kernels ------------------------------------

@pytest.mark.parametrize("n,h", cases.RMS_SHAPES)
def test_rmsnorm_family_matches_reference_capture(golden_cuda, n, h):
    c = cases.rmsnorm_case(n, h)
    out = ops.rmsnorm(D(c["x"]), D(c["res"]), D(c["w"]), cases.ALPHA, cases.EPS)
    assert np.array_equal(out.cpu().numpy().view(np.uint16), golden_cuda[f"rmsnorm_{n}x{h}"].view(np.uint16))
    c = cases.rmsnorm_quant_case(n, h)
    r8, s8 = D(c["res_i8"]), D(c["scale"])
    ops.rmsnorm_quant_int8(D(c["x"]), D(c["w"]), r8, s8, cases.ALPHA, cases.EPS)
    assert np.array_equal(r8.cpu().numpy(), golden_cuda[f"rmsq_i8_{n}x{h}"])
    assert np.array_equal(s8.cpu().numpy(), golden_cuda[f"rmsq_i8_scale_{n}x{h}"])
    rf, sf = D(c["res_f8"]), D(c["scale"])
    ops.rmsnorm_quant_fp8(D(c["x"]), D(c["w"]), rf, sf, cases.ALPHA, cases.EPS)
    assert np.array_equal(rf.cpu().numpy(), golden_cuda[f"rmsq_f8_{n}x{h}"])
    assert np.array_equal(sf.cpu().numpy(), golden_cuda[f"rmsq_f8_scale_{n}x{h}"])


@pytest.mark.parametrize("n,h", cases.QUANT_SHAPES)
def test_quantisers_match_reference_capture(golden_cuda, n, h):
    x = D(cases.quant_case(n, h)["x"])
    q, s = ops.quant_int8(x)
    f, fs = ops.quant_fp8(x)
    assert np.array_equal(q.cpu().numpy(), golden_cuda[f"quant_i8_{n}x{h}"])
    assert np.array_equal(s.cpu().numpy(), golden_cuda[f"quant_i8_scale_{n}x{h}"])
    assert np.array_equal(f.cpu().numpy(), golden_cuda[f"quant_f8_{n}x{h}"])
    assert np.array_equal(fs.cpu().numpy(), golden_cuda[f"quant_f8_scale_{n}x{h}"])


def test_rotary_silu_flstm_dequant_match_reference_capture(golden_cuda):
    c = cases.rotary_case()
    qkv = ops.rotary_qkv_(D(c["qkv"]), D(c["sin"]), D(c["cos"]), 32)
    assert np.array_equal(qkv.cpu().numpy().view(np.uint16), golden_cuda["rotary"].view(np.uint16))
    out = ops.silu_mul(D(cases.silu_case()["x"]))
    assert np.array_equal(out.cpu().numpy().view(np.uint16), golden_cuda["silu"].view(np.uint16))
    c = cases.flstm_case()
    cell = D(c["cell"])
    hh = ops.flstm_step(D(c["scratch"]), D(c["ih"]), cell)
    assert np.array_equal(cell.cpu().numpy().view(np.uint16), golden_cuda["flstm_cell"].view(np.uint16))
    assert np.array_equal(hh.cpu().numpy().view(np.uint16), golden_cuda["flstm_hh"].view(np.uint16))
    c = cases.dequant_case()
    assert np.array_equal(ops.dequant_transpose(D(c["i8"]), c["scale"]).cpu().numpy().view(np.uint16), golden_cuda["dequant_i8"].view(np.uint16))
    assert np.array_equal(ops.dequant_transpose(D(c["f8"]), c["scale"], fp8=True).cpu().numpy().view(np.uint16), golden_cuda["dequant_f8"].view(np.uint16))


# ---- side by side with the reference library, larger and ragged shapes -------------------------------

def _ref():
    r = ref.cuda()
    if r is None:
        pytest.skip("oracle/_ref/libfluke_ref_cuda.so not built")
    return r


@pytest.mark.parametrize("n,h", [(32000, 512), (4096, 768), (8192, 1024), (1, 256), (7, 512), (333, 640), (50, 2)])
def test_rmsnorm_family_side_by_side(n, h):
    R = _ref()
    g = torch.Generator().manual_seed(n + h)
    x = torch.randn(n, h, generator=g).half().to(DEV); res = torch.randn(n, h, generator=g).half().to(DEV)
    w = (1 + 0.1 * torch.randn(h, generator=g)).half().to(DEV)
    mine = ops.rmsnorm(x, res, w, 2.0, 1e-5)
    theirs = torch.empty_like(x)
    R.fluke_rmsnorm_gpu(x.data_ptr(), res.data_ptr(), w.data_ptr(), theirs.data_ptr(), n, h, 2.0, 1e-5)
    assert same_bits(mine, theirs)
    r8 = torch.randint(-127, 128, (n, h), generator=g, dtype=torch.int8).to(DEV)
    rs = (torch.rand(n, generator=g) * 0.02 + 0.001).to(DEV)
    for alpha in (2.0, 0.0):
        a8, as_, b8, bs = r8.clone(), rs.clone(), r8.clone(), rs.clone()
        ops.rmsnorm_quant_int8(x, w, a8, as_, alpha, 1e-5)
        R.fluke_rmsnorm_quant_int8_gpu(x.data_ptr(), w.data_ptr(), b8.data_ptr(), bs.data_ptr(), n, h, alpha, 1e-5)
        assert torch.equal(a8, b8) and same_bits(as_, bs)
    u8 = torch.randint(0, 256, (n, h), generator=g, dtype=torch.uint8).to(DEV)
    a8, as_, b8, bs = u8.clone(), rs.clone(), u8.clone(), rs.clone()
    ops.rmsnorm_quant_fp8(x, w, a8, as_, 2.0, 1e-5)
    R.fluke_rmsnorm_quant_fp8_gpu(x.data_ptr(), w.data_ptr(), b8.data_ptr(), bs.data_ptr(), n, h, 2.0, 1e-5)
    assert torch.equal(a8, b8) and same_bits(as_, bs)


def test_fp8_quantiser_rounds_ties_like_the_reference_encoder():
    """The reference's e4m3 encoder rounds a value half-way between two codes away from zero; the
    conversion instruction the row kernel uses rounds such ties to even and is therefore fed with
    the lowest mantissa bit set. Rows whose maximum is 448 have scale 1, so the inputs below reach
    the encoder unchanged: every f16 value that lies exactly between two e4m3 codes (normal and
    subnormal range, both signs), its f16 neighbours, and the saturating end."""
    codes = port.e4m3_decode_table()[:0x7F].astype(np.float64)          # positive finite codes, ascending
    mids = (codes[:-1] + codes[1:]) / 2
    mids = mids[mids.astype(np.float16).astype(np.float64) == mids]      # exactly representable in f16
    near = np.concatenate([np.nextafter(mids.astype(np.float16), np.float16(0)).astype(np.float64),
                           np.nextafter(mids.astype(np.float16), np.float16(1000)).astype(np.float64)])
    vals = np.concatenate([mids, near, codes, [2.0 ** -10, 2.0 ** -11, 3 * 2.0 ** -11, 447.0, 440.0, 432.0]])
    vals = np.concatenate([vals, -vals]).astype(np.float16)
    for h in (512, 384):                                                  # register path and generic path
        n = (vals.size + h - 2) // (h - 1)
        x = np.zeros((n, h), dtype=np.float16)
        x[:, 0] = 448.0
        flat = np.zeros(n * (h - 1), dtype=np.float16)
        flat[:vals.size] = vals
        x[:, 1:] = flat.reshape(n, h - 1)
        f, fs = ops.quant_fp8(torch.from_numpy(x).to(DEV))
        assert np.all(fs.cpu().numpy() == 1.0)
        assert np.array_equal(f.cpu().numpy(), port.e4m3_encode(x.astype(np.float32)))


@pytest.mark.parametrize("n,h", [(300, 512), (128, 1024), (64, 2048), (512, 512), (9, 6), (1000, 1000), (32000, 512), (77, 768), (5, 256)])
def test_quantisers_side_by_side(n, h):
    R = _ref()
    x = (torch.randn(n, h, generator=torch.Generator().manual_seed(n * h)) * 3).half().to(DEV)
    q, s = ops.quant_int8(x); f, fs = ops.quant_fp8(x)
    q2, s2, f2, fs2 = torch.empty_like(q), torch.empty_like(s), torch.empty_like(f), torch.empty_like(fs)
    R.fluke_quant_int8_gpu(x.data_ptr(), q2.data_ptr(), s2.data_ptr(), n, h)
    R.fluke_quant_fp8_gpu(x.data_ptr(), f2.data_ptr(), fs2.data_ptr(), n, h)
    assert torch.equal(q, q2) and same_bits(s, s2) and torch.equal(f, f2) and same_bits(fs, fs2)


@pytest.mark.parametrize("b,s,h,w,hd", [(32, 1000, 8, 32, 64), (4, 128, 8, 32, 64), (3, 77, 8, 16, 64), (2, 5, 3, 5, 16), (2, 50, 6, 32, 64), (5, 33, 4, 24, 64)])
def test_rotary_side_by_side(b, s, h, w, hd):
    R = _ref()
    g = torch.Generator().manual_seed(b * s)
    qkv = torch.randn(b, s, 3, h, hd, generator=g).half().to(DEV)
    fr = torch.outer(torch.arange(s, dtype=torch.float64), 1.0 / 10000 ** (torch.arange(w, dtype=torch.float64) / w))
    sin, cos = fr.sin().float().to(DEV), fr.cos().float().to(DEV)
    mine = ops.rotary_qkv_(qkv.clone(), sin, cos, w)
    theirs = qkv.clone()
    for ch in (0, 1):
        R.fluke_rotary_emb_gpu(theirs.data_ptr() + ch * theirs.stride(2) * 2, sin.data_ptr(), cos.data_ptr(),
                               b, s, h, hd, w, theirs.stride(0), theirs.stride(1), theirs.stride(3))
    assert same_bits(mine, theirs)
    assert torch.equal(mine[:, :, 2], qkv[:, :, 2])  # v untouched


@pytest.mark.parametrize("n,h", [(300, 512), (32000, 2048), (7, 10)])
def test_silu_mul_side_by_side(n, h):
    R = _ref()
    x = (torch.randn(n, 2 * h, generator=torch.Generator().manual_seed(h)) * 2).half().to(DEV)
    mine, theirs = ops.silu_mul(x), torch.empty(n, h, dtype=torch.float16, device=DEV)
    R.fluke_silu_mul_gpu(x.data_ptr(), theirs.data_ptr(), n, h)
    assert same_bits(mine, theirs)


@pytest.mark.parametrize("n,h", [(200, 96), (1024, 768), (5, 3)])
def test_flstm_step_side_by_side(n, h):
    R = _ref()
    g = torch.Generator().manual_seed(n)
    sc, ih = torch.randn(n, 4 * h, generator=g).half().to(DEV), torch.randn(n, 4 * h, generator=g).half().to(DEV)
    c = torch.randn(n, h, generator=g).half().to(DEV)
    c1, c2 = c.clone(), c.clone()
    h1, h2 = ops.flstm_step(sc, ih, c1), torch.empty_like(c)
    R.fluke_flstm_step_gpu(sc.data_ptr(), ih.data_ptr(), c2.data_ptr(), h2.data_ptr(), n, h)
    assert same_bits(c1, c2) and same_bits(h1, h2)


@pytest.mark.parametrize("t,n,c", [(33, 20, 512), (1000, 8, 768), (3, 2, 5)])
def test_dequant_transpose_side_by_side(t, n, c):
    R = _ref()
    g = torch.Generator().manual_seed(t)
    i8 = torch.randint(-127, 128, (t, n, c), generator=g, dtype=torch.int8).to(DEV)
    u8 = torch.randint(0, 256, (t, n, c), generator=g, dtype=torch.uint8).to(DEV)
    a, a2 = ops.dequant_transpose(i8, 0.0131), ops.dequant_transpose(u8, 0.0131, fp8=True)
    b, b2 = torch.empty_like(a), torch.empty_like(a2)
    R.fluke_dequant_int8_transpose_gpu(i8.data_ptr(), b.data_ptr(), t, n, c, 0.0131)
    R.fluke_dequant_fp8_transpose_gpu(u8.data_ptr(), b2.data_ptr(), t, n, c, 0.0131)
    assert same_bits(a, b) and same_bits(a2, b2)


# ---- against the CPU oracle and size-independent properties at the benchmark sizes ----------------

def test_rmsnorm_quant_config_size_vs_oracle_and_properties():
    n, h = 32000, 512
    g = torch.Generator().manual_seed(0)
    x = torch.randn(n, h, generator=g).half(); w = (1 + 0.1 * torch.randn(h, generator=g)).half()
    r8, rs = torch.zeros(n, h, dtype=torch.int8), torch.ones(n)
    q, s = r8.to(DEV), rs.to(DEV)
    ops.rmsnorm_quant_int8(x.to(DEV), w.to(DEV), q, s, 0.0, 1e-5)
    rows = slice(0, 512)
    oq, os_ = port.rmsnorm_quant(x[rows].numpy(), w.numpy(), r8[rows].numpy(), rs[rows].numpy(), 0.0, 1e-5)
    assert np.abs(q[rows].cpu().numpy().astype(np.int32) - oq.astype(np.int32)).max() <= 1  # rsqrtf vs 1/sqrtf
    assert np.allclose(s[rows].cpu().numpy(), os_, rtol=1e-6)
    # properties over all rows: every row uses the full int8 range and dequantises to unit RMS * w
    assert bool((q.abs().amax(dim=1) == 127).all())
    deq = q.float() * s[:, None]
    assert torch.allclose((deq / w.float().to(DEV)).pow(2).mean(dim=1), torch.ones(n, device=DEV), atol=2e-2)
    # idempotence of re-quantising the dequantised row with unit weight and alpha = 0
    y = deq.half()
    q2, s2 = torch.zeros_like(q), torch.ones_like(s)
    ops.rmsnorm_quant_int8(y, torch.ones(h, dtype=torch.float16, device=DEV), q2, s2, 0.0, 0.0)
    assert (q2.int() - torch.round(y.float() / y.float().abs().amax(dim=1, keepdim=True) * 127).int()).abs().max() <= 1


def test_rotary_config_size_round_trip():
    b, s = 32, 1000
    sin, cos = prep.rotary_tables(s, 64, device=DEV)
    qkv = torch.randn(b, s, 3, 8, 64, generator=torch.Generator().manual_seed(0)).half().to(DEV)
    fwd = ops.rotary_qkv_(qkv.clone(), sin, cos, 32)
    # rotation preserves the norm of every (i, i+32) pair and is undone by the opposite angle
    n0 = qkv[:, :, :2].float().view(b, s, 2, 8, 2, 32).pow(2).sum(dim=4)
    n1 = fwd[:, :, :2].float().view(b, s, 2, 8, 2, 32).pow(2).sum(dim=4)
    assert torch.allclose(n0, n1, rtol=2e-3, atol=2e-3)
    back = ops.rotary_qkv_(fwd.clone(), -sin, cos, 32)
    assert (back.float() - qkv.float()).abs().max() < 6e-3
    assert torch.equal(fwd[:, :, 2], qkv[:, :, 2])
    sub = qkv[:2].cpu().numpy().ravel()
    for ch in (0, 1):
        off = ch * 512
        sub = np.concatenate([sub[:off], port.rotary_f16(sub[off:], sin.cpu().numpy(), cos.cpu().numpy(), 2, s, 8, 32, s * 1536, 1536, 64)])
    assert np.array_equal(sub.view(np.uint16), fwd[:2].cpu().numpy().ravel().view(np.uint16))


def test_empty_inputs_are_noops():
    z = torch.zeros(0, 512, dtype=torch.float16, device=DEV)
    assert ops.quant_int8(z)[0].shape == (0, 512)
    assert ops.rmsnorm(z, z, torch.ones(512, dtype=torch.float16, device=DEV), 1.0, 1e-5).shape == (0, 512)
    assert ops.silu_mul(torch.zeros(0, 64, dtype=torch.float16, device=DEV)).shape == (0, 32)
