"""GPU parity of the tcgen05 GEMM family, called through the C ABI.

Bar: int32 accumulators bit-exact; f16 outputs of the base GEMM and of the QKV rotary kernel
bit-exact against the CPU oracle (their epilogues are IEEE-only with a fixed operation order);
the SiLU and fp8 kernels within max-abs <= 1e-2 x output RMS (tanh.approx / f32 accumulation
order); all within the reference tests' own 0.05 against their torch references.
"""
import numpy as np
import pytest
import torch

from fluke_b200 import lib as L, ops, prep
from oracle import port

pytestmark = pytest.mark.gpu
DEV = "cuda"
TOL_REL_RMS = 1e-2


def i8(g, *shape):
    return torch.randint(-127, 128, shape, generator=g, dtype=torch.int8)


@pytest.fixture(scope="module")
def be():
    b = ops.int8_select(0)
    assert b, "fluke_int8_select returned NULL on a B200"
    return b


@pytest.fixture(scope="module")
def be8():
    b = ops.fp8_select(0)
    assert b
    return b


@pytest.fixture(autouse=True)
def _fp8_weight_copies_dropped(flib):
    """The reference-ABI fp8 entry points find their re-ordered copy of a weight by the weight's
    ADDRESS; these tests create and free weights all the time and torch hands the same addresses
    out again, so every test ends by dropping the copies, as the contract asks of a caller that
    frees a weight."""
    yield
    flib.fluke_fp8_release_weight(None)


def test_select_rejects_other_dims_and_reports_dims(flib, be):
    assert flib.fluke_int8_select(0, L.fluke_dims_t(768, 2048, 8, 64, 2048)) is None
    assert flib.fluke_fp8_select(0, L.fluke_dims_t(512, 2048, 16, 64, 2048)) is None
    d = flib.fluke_int8_dims(be)
    assert (d.d_model, d.dim_feedforward, d.nhead, d.head_dim) == (512, 2048, 8, 64)


@pytest.mark.parametrize("m,n,k", [(128, 128, 128), (256, 768, 512), (1000, 128, 768), (77, 192, 256),
                                   (1, 64, 16), (129, 64, 48), (4097, 1536, 512), (300, 2048, 1024)])
def test_int32_accumulators_bit_exact(m, n, k):
    g = torch.Generator().manual_seed(m * 7 + n)
    a, b = i8(g, m, k), i8(g, n, k)
    got = ops.gemm_i8_s32(a.to(DEV), b.to(DEV)).cpu()
    assert torch.equal(got, a.int() @ b.int().T)


def test_int32_extremes_do_not_saturate():
    a = torch.full((128, 1024), -127, dtype=torch.int8); b = torch.full((64, 1024), 127, dtype=torch.int8)
    assert torch.equal(ops.gemm_i8_s32(a.to(DEV), b.to(DEV)).cpu(), torch.full((128, 64), -127 * 127 * 1024, dtype=torch.int32))


def test_int32_full_size_checksum():
    """M = 32000: row sums of C equal A @ (column sums of B), exactly, in int64."""
    g = torch.Generator().manual_seed(1)
    a, b = i8(g, 32000, 512), i8(g, 1536, 512)
    c = ops.gemm_i8_s32(a.to(DEV), b.to(DEV))
    assert torch.equal(c.sum(dim=1, dtype=torch.int64).cpu(), a.long() @ b.long().sum(dim=0))
    assert torch.equal(c.sum(dim=0, dtype=torch.int64).cpu(), b.long() @ a.long().sum(dim=0))


@pytest.mark.parametrize("m,n,k", [(256, 768, 512), (1000, 128, 768), (33, 64, 512)])
def test_base_gemm_f16_bit_exact_vs_oracle(m, n, k):
    g = torch.Generator().manual_seed(m)
    a, sa = prep.quantize_int8_rows(torch.randn(m, k, generator=g) * 0.1)
    b, sb = prep.quantize_int8_rows(torch.randn(n, k, generator=g) * 0.1)
    got = ops.gemm_i8(a.to(DEV), b.to(DEV), sa.to(DEV), sb.to(DEV)).cpu().numpy()
    assert np.array_equal(got.view(np.uint16), port.gemm_i8(a.numpy(), b.numpy(), sa.numpy(), sb.numpy()).view(np.uint16))
    dp = ops.down_proj_i8(a.to(DEV), b.to(DEV), None, sb.to(DEV)).cpu().numpy()
    assert np.array_equal(dp.view(np.uint16), port.down_proj(a.numpy(), b.numpy(), None, sb.numpy()).view(np.uint16))
    # reference test bar: within 0.05 of the fp16-dequantised torch GEMM (cute/test_gemm.py:85-93)
    ref = (a.float() * sa[:, None]).half().float() @ (b.float() * sb[:, None]).half().float().T
    assert (torch.from_numpy(got.astype(np.float32)) - ref).abs().max() < 0.05


def test_accumulators_beyond_2_pow_22_stay_bit_exact(be):
    """The epilogues convert int32 -> f32 with an integer-add trick that is exact below 2^22 and
    must fall back to the plain conversion above it: rows and weight rows of +-127/-128 drive
    |acc| up to 512 * 128 * 128 = 2^23 in some output positions and leave others ordinary."""
    g = torch.Generator().manual_seed(22)
    m = 300
    a = i8(g, m, 512)
    a[5] = 127; a[70] = -128; a[131] = -127; a[299] = 127
    sa = torch.rand(m, generator=g) * 0.02 + 0.001
    w = i8(g, 1536, 512)
    w[3] = 127; w[40] = -128; w[1000] = 127; w[1535] = -127; w[1030] = -128
    sb = torch.rand(1536, generator=g) * 0.001 + 0.0001
    A, W, SA, SB = a.to(DEV), w.to(DEV), sa.to(DEV), sb.to(DEV)
    assert int(ops.gemm_i8_s32(A, W).abs().max()) >= 1 << 22
    got = ops.gemm_i8(A, W, SA, SB).cpu().numpy()
    assert np.array_equal(got.view(np.uint16), port.gemm_i8(a.numpy(), w.numpy(), sa.numpy(), sb.numpy()).view(np.uint16))
    sin, cos = prep.rotary_tables(150, 64)
    got = ops.qkv_rotary_i8(be, A, W, SA, SB, sin.to(DEV), cos.to(DEV), 150).cpu().numpy()
    exp = port.qkv_rotary_i8(a.numpy(), w.numpy(), sa.numpy(), sb.numpy(), sin.numpy(), cos.numpy(), 150)
    assert np.array_equal(got.view(np.uint16), exp.view(np.uint16))
    wg, wu = i8(g, 2048, 512), i8(g, 2048, 512)
    wg[7] = 127; wu[7] = -128; wg[2047] = -127; wu[100] = 127
    sg, su = torch.rand(2048, generator=g) * 1e-4 + 1e-5, torch.rand(2048, generator=g) * 1e-4 + 1e-5
    got = ops.gated_mlp_i8(be, A, wg.to(DEV), wu.to(DEV), SA, sg.to(DEV), su.to(DEV)).cpu().numpy().astype(np.float32)
    exp = port.gated_mlp_i8(a.numpy(), wg.numpy(), wu.numpy(), sa.numpy(), sg.numpy(), su.numpy()).astype(np.float32)
    assert np.isfinite(got).all() == np.isfinite(exp).all()
    fin = np.isfinite(exp) & np.isfinite(got)
    assert np.abs(got - exp)[fin].max() <= TOL_REL_RMS * np.sqrt((exp[fin] ** 2).mean())


def test_down_proj_writes_into_a_wider_buffer():
    g = torch.Generator().manual_seed(3)
    a, b = i8(g, 200, 768), i8(g, 128, 768)
    sb = torch.rand(128, generator=g) * 0.01
    buf = torch.full((200, 256), 7.0, dtype=torch.float16, device=DEV)
    ops.down_proj_i8(a.to(DEV), b.to(DEV), None, sb.to(DEV), out=buf[:, :128])
    exp = port.down_proj(a.numpy(), b.numpy(), None, sb.numpy())
    assert np.array_equal(buf[:, :128].cpu().numpy().view(np.uint16), exp.view(np.uint16))
    assert bool((buf[:, 128:] == 7.0).all())


def _qkv_inputs(m, g):
    a, sa = prep.quantize_int8_rows(torch.randn(m, 512, generator=g))
    w, sb = prep.quantize_int8_rows(torch.randn(1536, 512, generator=g) * 0.02)
    return a, sa, w, sb


@pytest.mark.parametrize("batch,seqlen", [(4, 16), (1, 256), (3, 100), (5, 1000), (1, 1), (2, 77), (3, 130), (2, 128), (40, 300)])
def test_qkv_rotary_bit_exact_vs_oracle(be, batch, seqlen):
    m = batch * seqlen
    a, sa, w, sb = _qkv_inputs(m, torch.Generator().manual_seed(m))
    sin, cos = prep.rotary_tables(seqlen, 64)
    got = ops.qkv_rotary_i8(be, a.to(DEV), w.to(DEV), sa.to(DEV), sb.to(DEV), sin.to(DEV), cos.to(DEV), seqlen).cpu().numpy()
    exp = port.qkv_rotary_i8(a.numpy(), w.numpy(), sa.numpy(), sb.numpy(), sin.numpy(), cos.numpy(), seqlen)
    assert np.array_equal(got.view(np.uint16), exp.view(np.uint16))


def test_qkv_rotary_golden_from_reference_test(be, golden_tests):
    g = golden_tests
    T = lambda k: torch.from_numpy(g[k]).to(DEV)
    got = ops.qkv_rotary_i8(be, T("rot_A"), T("rot_B"), T("rot_sa"), T("rot_sb"), T("rot_sin"), T("rot_cos"), 16)
    assert (got.float().cpu() - torch.from_numpy(g["rot_expected"].astype(np.float32))).abs().max() < 0.05  # cute/test_rotary.py ABS_TOL


def test_qkv_rotary_full_size_sampled_rows_and_v_passthrough(be):
    m, seqlen = 32000, 1000
    a, sa, w, sb = _qkv_inputs(m, torch.Generator().manual_seed(0))
    sin, cos = prep.rotary_tables(seqlen, 64)
    out = ops.qkv_rotary_i8(be, a.to(DEV), w.to(DEV), sa.to(DEV), sb.to(DEV), sin.to(DEV), cos.to(DEV), seqlen)
    rows = torch.cat([torch.arange(0, 64), torch.arange(999, 1063), torch.randint(0, m, (256,), generator=torch.Generator().manual_seed(5)),
                      torch.arange(m - 64, m)])
    pos = rows % seqlen
    exp = port.epi_rotary(port.gemm_i8_s32(a[rows].numpy(), w.numpy()), sa[rows].numpy(), sb.numpy(),
                          sin[pos].numpy(), cos[pos].numpy(), len(rows), 1024)
    assert np.array_equal(out[rows.to(DEV)].cpu().numpy().view(np.uint16), exp.view(np.uint16))
    # V columns are the plain dequantised GEMM for every row
    v = ops.gemm_i8(a.to(DEV), w[1024:].contiguous().to(DEV), sa.to(DEV), sb[1024:].contiguous().to(DEV))
    # base GEMM multiplies acc*(sa*sb), the fused kernel (acc*sa)*sb: equal up to one f16 ulp
    assert (out[:, 1024:].float() - v.float()).abs().max() <= 2e-3 * out[:, 1024:].float().abs().max()
    # rotation preserves pair norms: |q|^2 per head equals that of the unrotated projection
    plain = ops.gemm_i8(a.to(DEV), w[:1024].contiguous().to(DEV), sa.to(DEV), sb[:1024].contiguous().to(DEV))
    n_rot = out[:, :1024].float().view(m, 16, 64).pow(2).sum(-1)
    n_pl = plain.float().view(m, 16, 64).pow(2).sum(-1)
    assert torch.allclose(n_rot, n_pl, rtol=5e-3, atol=1e-3)


@pytest.mark.parametrize("m", [64, 1000, 4096, 129])
def test_gated_mlp_vs_oracle(be, m):
    g = torch.Generator().manual_seed(m)
    a, sa = prep.quantize_int8_rows(torch.randn(m, 512, generator=g))
    wg, sg = prep.quantize_int8_rows(torch.randn(2048, 512, generator=g) * 0.02)
    wu, su = prep.quantize_int8_rows(torch.randn(2048, 512, generator=g) * 0.02)
    got = ops.gated_mlp_i8(be, a.to(DEV), wg.to(DEV), wu.to(DEV), sa.to(DEV), sg.to(DEV), su.to(DEV)).cpu().numpy().astype(np.float32)
    exp = port.gated_mlp_i8(a.numpy(), wg.numpy(), wu.numpy(), sa.numpy(), sg.numpy(), su.numpy()).astype(np.float32)
    rms = np.sqrt((exp ** 2).mean())
    assert np.abs(got - exp).max() <= TOL_REL_RMS * rms


def test_gated_mlp_against_silu_mul_kernel_and_full_size(be):
    """The CUDA-C epilogue oracle of the reference test (cute/test_dual_gemm_silu.py:99-112):
    plain GEMMs to f16, then fluke_silu_mul_gpu on [up | gate]; M = 32000."""
    m = 32000
    g = torch.Generator().manual_seed(4)
    a, sa = prep.quantize_int8_rows(torch.randn(m, 512, generator=g))
    wg, sg = prep.quantize_int8_rows(torch.randn(2048, 512, generator=g) * 0.02)
    wu, su = prep.quantize_int8_rows(torch.randn(2048, 512, generator=g) * 0.02)
    A, SA = a.to(DEV), sa.to(DEV)
    out = ops.gated_mlp_i8(be, A, wg.to(DEV), wu.to(DEV), SA, sg.to(DEV), su.to(DEV))
    gate = ops.gemm_i8(A, wg.to(DEV), SA, sg.to(DEV)); up = ops.gemm_i8(A, wu.to(DEV), SA, su.to(DEV))
    two = ops.silu_mul(torch.cat([up, gate], dim=1).contiguous())
    rms = out.float().pow(2).mean().sqrt()
    assert (out.float() - two.float()).abs().max() <= 2 * TOL_REL_RMS * rms  # the two-kernel path rounds gate/up to f16 first
    assert (out.float() - two.float()).abs().max() < 0.05


def _sample_rows(m, seqlen, seed):
    """First and last tiles, the rows around a sequence boundary and a 128-row tile edge, 256 random rows."""
    return torch.cat([torch.arange(0, 64), torch.arange(seqlen - 1, seqlen + 63), torch.arange(128 * 100 - 8, 128 * 100 + 8),
                      torch.randint(0, m, (256,), generator=torch.Generator().manual_seed(seed)), torch.arange(m - 64, m)])


def test_gated_mlp_full_size_sampled_rows_vs_oracle(be):
    """M = 32000 (the benchmark shape) through the fused kernel, sampled rows against the oracle
    (reference: cute/test_dual_gemm_silu.py:90-96)."""
    m = 32000
    g = torch.Generator().manual_seed(40)
    a, sa = prep.quantize_int8_rows(torch.randn(m, 512, generator=g))
    wg, sg = prep.quantize_int8_rows(torch.randn(2048, 512, generator=g) * 0.02)
    wu, su = prep.quantize_int8_rows(torch.randn(2048, 512, generator=g) * 0.02)
    out = ops.gated_mlp_i8(be, a.to(DEV), wg.to(DEV), wu.to(DEV), sa.to(DEV), sg.to(DEV), su.to(DEV))
    rows = _sample_rows(m, 1000, 6)
    exp = port.gated_mlp_i8(a[rows].numpy(), wg.numpy(), wu.numpy(), sa[rows].numpy(), sg.numpy(), su.numpy()).astype(np.float32)
    got = out[rows.to(DEV)].float().cpu().numpy()
    assert np.abs(got - exp).max() <= TOL_REL_RMS * np.sqrt((exp ** 2).mean())


def test_gated_mlp_golden_from_reference_test(be, golden_tests):
    """The fixture of the reference's own test (cute/test_dual_gemm_silu.py, N cut to 256) through
    the FUSED kernel: its 256 gate/up rows are the first rows of 2048-row weights padded with zero
    rows (output columns are independent), so columns [0, 256) must meet the test's 0.05."""
    g = golden_tests
    pad = lambda w: np.concatenate([w, np.zeros((2048 - w.shape[0],) + w.shape[1:], w.dtype)], 0)
    T = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(DEV)
    got = ops.gated_mlp_i8(be, T(g["silu_A"]), T(pad(g["silu_Bg"])), T(pad(g["silu_Bu"])), T(g["silu_sa"]),
                           T(pad(g["silu_sbg"])), T(pad(g["silu_sbu"])))
    got = got.float().cpu().numpy()
    assert np.abs(got[:, :256] - g["silu_expected"].astype(np.float32)).max() < 0.05  # ABS_TOL of the reference test
    assert not got[:, 256:].any()
    # and the oracle's epilogue on the same accumulators, against the same fixture
    acc_g, acc_u = ops.gemm_i8_s32(T(g["silu_A"]), T(g["silu_Bg"])).cpu().numpy(), ops.gemm_i8_s32(T(g["silu_A"]), T(g["silu_Bu"])).cpu().numpy()
    ora = port.epi_silu(acc_g, acc_u, g["silu_sa"], g["silu_sbg"], g["silu_sbu"]).astype(np.float32)
    assert np.abs(ora - g["silu_expected"].astype(np.float32)).max() < 0.05
    assert np.abs(got[:, :256] - ora).max() <= TOL_REL_RMS * np.sqrt((ora ** 2).mean())


# ---- fp8 (E4M3, amax/448) ---------------------------------------------------------------------------------

def test_fp8_unshuffle_and_fused_ops(be8, golden_tests):
    gt = golden_tests
    g = torch.Generator().manual_seed(11)
    m, seqlen = 600, 200
    a, sa = prep.quantize_fp8_rows(torch.randn(m, 512, generator=g) * 0.1)
    w, sb = prep.quantize_fp8_rows(torch.randn(1536, 512, generator=g) * 0.1)
    sin, cos = prep.rotary_tables(seqlen, 64)
    a8, w8 = a.view(torch.uint8), w.view(torch.uint8)
    wsh = prep.preshuffle_fp8_weight(w)
    assert torch.equal(ops.fp8_unshuffle(wsh.to(DEV), 1536, 512).cpu(), w8)
    out_sh = ops.qkv_rotary_fp8(be8, a8.to(DEV), wsh.to(DEV), sa.to(DEV), sb.to(DEV), sin.to(DEV), cos.to(DEV), seqlen)
    out_pl = ops.qkv_rotary_fp8(be8, a8.to(DEV), w8.to(DEV), sa.to(DEV), sb.to(DEV), sin.to(DEV), cos.to(DEV), seqlen, plain=True)
    assert torch.equal(out_sh.view(torch.int16), out_pl.view(torch.int16))  # both ABI forms, same bits
    exp = port.epi_rotary(port.gemm_fp8_f32(a8.numpy(), w8.numpy()), sa.numpy(), sb.numpy(), sin.numpy(), cos.numpy(), seqlen, 1024).astype(np.float32)
    err = np.abs(out_sh.float().cpu().numpy() - exp).max()
    assert err <= TOL_REL_RMS * np.sqrt((exp ** 2).mean()) and err < 5e-2
    wg, sg = prep.quantize_fp8_rows(torch.randn(2048, 512, generator=g) * 0.1)
    wu, su = prep.quantize_fp8_rows(torch.randn(2048, 512, generator=g) * 0.1)
    out = ops.gated_mlp_fp8(be8, a8.to(DEV), prep.preshuffle_fp8_weight(wg).to(DEV), prep.preshuffle_fp8_weight(wu).to(DEV),
                            sa.to(DEV), sg.to(DEV), su.to(DEV))
    exp = port.epi_silu(port.gemm_fp8_f32(a8.numpy(), wg.view(torch.uint8).numpy()), port.gemm_fp8_f32(a8.numpy(), wu.view(torch.uint8).numpy()),
                        sa.numpy(), sg.numpy(), su.numpy()).astype(np.float32)
    err = np.abs(out.float().cpu().numpy() - exp).max()
    assert err <= TOL_REL_RMS * np.sqrt((exp ** 2).mean()) and err < 5e-2
    # golden from the reference's fly/test_rotary.py reference, through the preshuffled ABI
    T = lambda k: torch.from_numpy(gt[k]).to(DEV)
    w_nk = torch.from_numpy(np.ascontiguousarray(gt["fp8_B_kn"].T))
    got = ops.qkv_rotary_fp8(be8, T("fp8_A"), prep.preshuffle_fp8_weight(w_nk).to(DEV), T("fp8_sa"), T("fp8_sb"), T("fp8_sin"), T("fp8_cos"), 16)
    assert (got.float().cpu() - torch.from_numpy(gt["fp8_rot_expected"].astype(np.float32))).abs().max() < 5e-2


def test_fp8_fused_ops_full_size_sampled_rows(be8):
    """M = 32000, seqlen 1000 (the benchmark shape: the sequence-aligned tiling of the rotary
    epilogue) for both fused fp8 entry points, sampled rows against the oracle; tolerance of the
    reference's fp8 tests (fly/test_rotary.py:103: 5e-2) and 1e-2 of the output RMS."""
    m, seqlen = 32000, 1000
    g = torch.Generator().manual_seed(41)
    a, sa = prep.quantize_fp8_rows(torch.randn(m, 512, generator=g))
    w, sb = prep.quantize_fp8_rows(torch.randn(1536, 512, generator=g) * 0.02)
    sin, cos = prep.rotary_tables(seqlen, 64)
    a8, w8 = a.view(torch.uint8), w.view(torch.uint8)
    A, SA = a8.to(DEV), sa.to(DEV)
    rows = _sample_rows(m, seqlen, 8)
    pos = rows % seqlen
    out = ops.qkv_rotary_fp8(be8, A, prep.preshuffle_fp8_weight(w).to(DEV), SA, sb.to(DEV), sin.to(DEV), cos.to(DEV), seqlen)
    exp = port.epi_rotary(port.gemm_fp8_f32(a8[rows].numpy(), w8.numpy()), sa[rows].numpy(), sb.numpy(),
                          sin[pos].numpy(), cos[pos].numpy(), len(rows), 1024).astype(np.float32)
    err = np.abs(out[rows.to(DEV)].float().cpu().numpy() - exp).max()
    assert err <= TOL_REL_RMS * np.sqrt((exp ** 2).mean()) and err < 5e-2
    wg, sg = prep.quantize_fp8_rows(torch.randn(2048, 512, generator=g) * 0.02)
    wu, su = prep.quantize_fp8_rows(torch.randn(2048, 512, generator=g) * 0.02)
    out = ops.gated_mlp_fp8(be8, A, prep.preshuffle_fp8_weight(wg).to(DEV), prep.preshuffle_fp8_weight(wu).to(DEV),
                            SA, sg.to(DEV), su.to(DEV))
    exp = port.epi_silu(port.gemm_fp8_f32(a8[rows].numpy(), wg.view(torch.uint8).numpy()),
                        port.gemm_fp8_f32(a8[rows].numpy(), wu.view(torch.uint8).numpy()),
                        sa[rows].numpy(), sg.numpy(), su.numpy()).astype(np.float32)
    err = np.abs(out[rows.to(DEV)].float().cpu().numpy() - exp).max()
    assert err <= TOL_REL_RMS * np.sqrt((exp ** 2).mean()) and err < 5e-2


def test_fp8_weight_copy_follows_the_address_until_released(be8, flib):
    """New weight bytes written to an address the library has seen: the kept copy (the old weight)
    is used until fluke_fp8_release_weight is called for that address, the new one afterwards."""
    g = torch.Generator().manual_seed(14)
    m = 256
    a, sa = prep.quantize_fp8_rows(torch.randn(m, 512, generator=g))
    w1, s1 = prep.quantize_fp8_rows(torch.randn(2048, 512, generator=g) * 0.02)
    w2, _ = prep.quantize_fp8_rows(torch.randn(2048, 512, generator=g) * 0.02)
    up, su = prep.quantize_fp8_rows(torch.randn(2048, 512, generator=g) * 0.02)
    A, SA, S1, SU = a.view(torch.uint8).to(DEV), sa.to(DEV), s1.to(DEV), su.to(DEV)
    UP = prep.preshuffle_fp8_weight(up).to(DEV)
    gate = prep.preshuffle_fp8_weight(w1).to(DEV)
    run = lambda: ops.gated_mlp_fp8(be8, A, gate, UP, SA, S1, SU).clone()
    first = run()
    gate.copy_(prep.preshuffle_fp8_weight(w2).to(DEV))     # same address, other contents
    assert torch.equal(run(), first)                        # the kept copy still answers
    assert flib.fluke_fp8_release_weight(gate.data_ptr()) == 1
    second = run()
    want = ops.gated_mlp_fp8(be8, A, w2.view(torch.uint8).to(DEV), up.view(torch.uint8).to(DEV), SA, S1, SU, plain=True)
    assert torch.equal(second, want) and not torch.equal(second, first)
    assert flib.fluke_fp8_prepare_weight(gate.data_ptr(), 2048, 512) == 0    # already there: nothing to do


def test_fp8_base_gemm_vs_oracle():
    g = torch.Generator().manual_seed(12)
    a, sa = prep.quantize_fp8_rows(torch.randn(300, 768, generator=g)); b, sb = prep.quantize_fp8_rows(torch.randn(128, 768, generator=g))
    got = ops.gemm_fp8(a.view(torch.uint8).to(DEV), b.view(torch.uint8).to(DEV), sa.to(DEV), sb.to(DEV)).float().cpu().numpy()
    exp = port.epi_dequant2(port.gemm_fp8_f32(a.view(torch.uint8).numpy(), b.view(torch.uint8).numpy()), sa.numpy(), sb.numpy()).astype(np.float32)
    assert np.abs(got - exp).max() <= TOL_REL_RMS * np.sqrt((exp ** 2).mean())


def test_rmsnorm_quant_then_qkv_back_to_back_at_config_size(be):
    """The chain a transformer block runs: fluke_rmsnorm_quant_int8_gpu writes the int8 activations
    and their row scales, fluke_qkv_rotary_i8_gpu consumes them, on four buffer sets one after the
    other ([32000, 512] each, more than L2 in total). Sampled rows of every set against the oracle
    chain; the f16 output is bit-exact because both kernels are."""
    n, h, sets = 32000, 512, 4
    g = torch.Generator().manual_seed(31)
    w = (1 + 0.1 * torch.randn(h, generator=g)).half()
    wq, sq = prep.quantize_int8_rows(torch.randn(1536, 512, generator=g) * 0.02)
    sin, cos = prep.rotary_tables(1000, 64)
    xs = [torch.randn(n, h, generator=g).half() for _ in range(sets)]
    W, WQ, SQ, SIN, COS = w.to(DEV), wq.to(DEV), sq.to(DEV), sin.to(DEV), cos.to(DEV)
    X = [x.to(DEV) for x in xs]
    q8 = [torch.zeros(n, h, dtype=torch.int8, device=DEV) for _ in range(sets)]
    s8 = [torch.ones(n, device=DEV) for _ in range(sets)]
    outs = []
    for i in range(sets):
        ops.rmsnorm_quant_int8(X[i], W, q8[i], s8[i], 0.0, 1e-5)
        outs.append(ops.qkv_rotary_i8(be, q8[i], WQ, s8[i], SQ, SIN, COS, 1000))
    rows = _sample_rows(n, 1000, 3)[::4]
    pos = rows % 1000
    for i in range(sets):
        oq, osc = port.rmsnorm_quant(xs[i][rows].numpy(), w.numpy(), np.zeros((len(rows), h), np.int8), np.ones(len(rows), np.float32), 0.0, 1e-5)
        gq = q8[i][rows.to(DEV)].cpu().numpy()
        assert np.abs(gq.astype(np.int32) - oq.astype(np.int32)).max() <= 1      # rsqrt: within one code of the CPU oracle
        exp = port.epi_rotary(port.gemm_i8_s32(gq, wq.numpy()), s8[i][rows.to(DEV)].cpu().numpy(), sq.numpy(),
                              sin[pos].numpy(), cos[pos].numpy(), len(rows), 1024)
        assert np.array_equal(outs[i][rows.to(DEV)].cpu().numpy().view(np.uint16), exp.view(np.uint16))


def test_quant_kernel_feeds_the_gemm(be):
    """fluke_quant_int8_gpu output (amax/128 convention) straight into the fused kernel."""
    g = torch.Generator().manual_seed(13)
    x = torch.randn(512, 512, generator=g).half().to(DEV)
    q, s = ops.quant_int8(x)
    w, sb = prep.quantize_int8_rows(torch.randn(1536, 512, generator=g) * 0.02)
    sin, cos = prep.rotary_tables(128, 64)
    out = ops.qkv_rotary_i8(be, q, w.to(DEV), s, sb.to(DEV), sin.to(DEV), cos.to(DEV), 128)
    exp = port.qkv_rotary_i8(q.cpu().numpy(), w.numpy(), s.cpu().numpy(), sb.numpy(), sin.numpy(), cos.numpy(), 128)
    assert np.array_equal(out.cpu().numpy().view(np.uint16), exp.view(np.uint16))


def test_transformer_ops_are_shard_invariant(be, be8):
    """Replicas-only multi-GPU: a rank takes whole sequences of the token axis and runs the same
    kernels on its rows. Whatever the split, the concatenated shard outputs are the single-call
    output bit for bit (no result depends on which tile or CTA a row falls into): RMSNorm+quant,
    QKV+rotary and the gated MLP, int8 and fp8, 7 sequences of 300 tokens cut 3 + 4 and 1 + 6."""
    seqlen, n_seq = 300, 7
    m = seqlen * n_seq
    g = torch.Generator().manual_seed(11)
    x = torch.randn(m, 512, generator=g).half().to(DEV)
    w = (torch.randn(512, generator=g) * 0.1 + 1).half().to(DEV)
    res = torch.randint(-127, 128, (m, 512), generator=g, dtype=torch.int8).to(DEV)
    rs = (torch.rand(m, generator=g) * 0.02 + 0.001).to(DEV)
    sin, cos = prep.rotary_tables(seqlen, 64, device=DEV)
    wq, sq = prep.quantize_int8_rows(torch.randn(1536, 512, generator=g) * 0.02)
    wg, sg = prep.quantize_int8_rows(torch.randn(2048, 512, generator=g) * 0.02)
    wu, su = prep.quantize_int8_rows(torch.randn(2048, 512, generator=g) * 0.02)
    wq, sq, wg, sg, wu, su = (t.to(DEV) for t in (wq, sq, wg, sg, wu, su))
    a8, s8 = prep.quantize_fp8_rows(torch.randn(m, 512, generator=g))
    wq8, sq8 = prep.quantize_fp8_rows(torch.randn(1536, 512, generator=g) * 0.02)
    wg8, sg8 = prep.quantize_fp8_rows(torch.randn(2048, 512, generator=g) * 0.02)
    wu8, su8 = prep.quantize_fp8_rows(torch.randn(2048, 512, generator=g) * 0.02)
    a8, s8, wq8, sq8, wg8, sg8, wu8, su8 = (t.to(DEV) for t in (a8, s8, wq8, sq8, wg8, sg8, wu8, su8))

    def run(lo, hi):
        r, sc = res[lo:hi].clone(), rs[lo:hi].clone()
        q, qs = ops.rmsnorm_quant_int8(x[lo:hi].contiguous(), w, r, sc, 2.0, 1e-5)
        qkv = ops.qkv_rotary_i8(be, q, wq, qs, sq, sin, cos, seqlen)
        mlp = ops.gated_mlp_i8(be, q, wg, wu, qs, sg, su)
        qkv8 = ops.qkv_rotary_fp8(be8, a8[lo:hi].contiguous(), wq8, s8[lo:hi].contiguous(), sq8, sin, cos, seqlen, plain=True)
        mlp8 = ops.gated_mlp_fp8(be8, a8[lo:hi].contiguous(), wg8, wu8, s8[lo:hi].contiguous(), sg8, su8, plain=True)
        torch.cuda.synchronize()
        return [q, qs, qkv, mlp, qkv8, mlp8]

    whole = run(0, m)
    for cut in (3, 1):
        a, b = run(0, cut * seqlen), run(cut * seqlen, m)
        for full, pa, pb in zip(whole, a, b):
            assert torch.equal(full, torch.cat([pa, pb], dim=0))
    assert L.read_status() == 0
