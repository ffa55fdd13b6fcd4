"""Pins the CPU oracle (oracle/fluke_oracle.c):
  * against tests/golden/reference_cuda_kernels.npz -- outputs of the REFERENCE's own CUDA
    kernels run on a B200 -- bit for bit where the kernel is IEEE-only (quantisers, e4m3,
    dequant-transpose, rotary, the f16 LSTM cell), and within one int8 code / f16 ulp where the
    GPU uses MUFU approximations (rsqrtf, __expf, tanhf);
  * against tests/golden/reference_tests.npz -- outputs of the torch reference functions of the
    reference's own test files -- within each test's own tolerance.
"""
import numpy as np
import pytest

import cases
from oracle import port


def ulp_diff_f16(a, b):
    """Distance in f16 representable steps (sign-magnitude ordered)."""
    def key(x):
        u = x.view(np.uint16).astype(np.int32)
        return np.where(u & 0x8000, -(u & 0x7FFF), u & 0x7FFF)
    return np.abs(key(np.ascontiguousarray(a)) - key(np.ascontiguousarray(b)))


# ---- vs the reference's CUDA kernels (captured on a B200) --------------------------------------

@pytest.mark.parametrize("n,h", cases.QUANT_SHAPES)
def test_quant_bit_exact(golden_cuda, n, h):
    x = cases.quant_case(n, h)["x"]
    q, s = port.quant(x, fp8=False)
    assert np.array_equal(q, golden_cuda[f"quant_i8_{n}x{h}"])
    assert np.array_equal(s, golden_cuda[f"quant_i8_scale_{n}x{h}"])
    f, fs = port.quant(x, fp8=True)
    assert np.array_equal(f, golden_cuda[f"quant_f8_{n}x{h}"])
    assert np.array_equal(fs, golden_cuda[f"quant_f8_scale_{n}x{h}"])


def test_dequant_transpose_bit_exact(golden_cuda):
    c = cases.dequant_case()
    assert np.array_equal(port.dequant_transpose(c["i8"], c["scale"]).view(np.uint16), golden_cuda["dequant_i8"].view(np.uint16))
    assert np.array_equal(port.dequant_transpose(c["f8"], c["scale"], fp8=True).view(np.uint16), golden_cuda["dequant_f8"].view(np.uint16))


def test_rotary_bit_exact(golden_cuda):
    c = cases.rotary_case()
    x = c["qkv"].ravel()
    for ch in (0, 1):
        off = ch * 512
        x = np.concatenate([x[:off], port.rotary_f16(x[off:], c["sin"], c["cos"], 2, 24, 8, 32, 24 * 1536, 1536, 64)])
    assert np.array_equal(x.view(np.uint16), golden_cuda["rotary"].ravel().view(np.uint16))


def test_flstm_step_f16(golden_cuda):
    c = cases.flstm_case()
    cell, hh = port.flstm_step_f16(c["scratch"], c["ih"], c["cell"])
    assert np.array_equal(cell.view(np.uint16), golden_cuda["flstm_cell"].view(np.uint16))  # IEEE only
    assert ulp_diff_f16(hh, golden_cuda["flstm_hh"]).max() <= 1                            # tanhf


def test_silu_mul_f16(golden_cuda):
    got = port.silu_mul_f16(cases.silu_case()["x"])
    assert ulp_diff_f16(got, golden_cuda["silu"]).max() <= 1  # __expf on the GPU


@pytest.mark.parametrize("n,h", cases.RMS_SHAPES)
def test_rmsnorm_family_within_one_step(golden_cuda, n, h):
    c = cases.rmsnorm_case(n, h)
    got = port.rmsnorm_f16(c["x"], c["res"], c["w"], cases.ALPHA, cases.EPS)
    assert ulp_diff_f16(got, golden_cuda[f"rmsnorm_{n}x{h}"]).max() <= 1  # rsqrtf on the GPU
    c = cases.rmsnorm_quant_case(n, h)
    q, s = port.rmsnorm_quant(c["x"], c["w"], c["res_i8"], c["scale"], cases.ALPHA, cases.EPS)
    gq, gs = golden_cuda[f"rmsq_i8_{n}x{h}"], golden_cuda[f"rmsq_i8_scale_{n}x{h}"]
    assert np.abs(q.astype(np.int32) - gq.astype(np.int32)).max() <= 1
    assert np.abs(s - gs).max() <= 1e-6 * np.abs(gs).max() + 1e-9
    f, fs = port.rmsnorm_quant(c["x"], c["w"], c["res_f8"], c["scale"], cases.ALPHA, cases.EPS, fp8=True)
    gf, gfs = golden_cuda[f"rmsq_f8_{n}x{h}"], golden_cuda[f"rmsq_f8_scale_{n}x{h}"]
    lut = port.e4m3_decode_table()
    step = np.maximum(np.abs(lut[gf]) / 8.0, 2.0 ** -9)
    assert (np.abs(lut[f] - lut[gf]) <= step * 1.001).all()
    assert np.abs(fs - gfs).max() <= 1e-6 * np.abs(gfs).max() + 1e-12


def test_e4m3_codec_properties():
    lut = port.e4m3_decode_table()
    codes = np.arange(256, dtype=np.uint8)
    finite = (codes & 0x7F) != 0x7F
    assert np.array_equal(port.e4m3_encode(lut[finite]), np.where((codes[finite] & 0x7F) == 0, 0, codes[finite]))
    assert port.e4m3_encode([1e9, -1e9]).tolist() == [0x7E, 0xFE]          # saturation, never NaN
    assert port.e4m3_encode([17.0]).tolist() == port.e4m3_encode([18.0]).tolist()  # tie rounds up (away)
    assert port.e4m3_encode([2.0 ** -11]).tolist() == [0]                  # flush below half the smallest subnormal


# ---- vs the torch references of the reference's test files -------------------------------------

def test_base_gemm_accumulators_exact(golden_tests):
    g = golden_tests
    assert np.array_equal(port.gemm_i8_s32(g["gemm_A"], g["gemm_B"]), g["gemm_acc"])


def test_qkv_rotary_vs_cute_torch_reference(golden_tests):
    g = golden_tests
    got = port.qkv_rotary_i8(g["rot_A"], g["rot_B"], g["rot_sa"], g["rot_sb"], g["rot_sin"], g["rot_cos"], 16)
    err = np.abs(got.astype(np.float32) - g["rot_expected"].astype(np.float32)).max()
    assert err < 0.05  # ABS_TOL of cute/test_rotary.py
    assert err < 2e-3  # and in fact within f16 rounding of it


def test_gated_mlp_vs_cute_torch_reference(golden_tests):
    g = golden_tests
    got = port.gated_mlp_i8(g["silu_A"], g["silu_Bg"], g["silu_Bu"], g["silu_sa"], g["silu_sbg"], g["silu_sbu"])
    err = np.abs(got.astype(np.float32) - g["silu_expected"].astype(np.float32)).max()
    assert err < 0.05 and err < 2e-3


def test_lstm_step_vs_cute_torch_reference(golden_tests):
    g = golden_tests
    H = g["lstm_c"].shape[1]
    A = np.concatenate([g["lstm_hh_down"], g["lstm_x_down"]], 1).astype(np.float16)
    W = np.concatenate([np.concatenate([g["lstm_up_hh"][k * H:(k + 1) * H], g["lstm_up_ih"][k * H:(k + 1) * H]], 1)
                        for k in range(4)], 0).astype(np.float16)
    bias = (g["lstm_bhh"] + g["lstm_bih"]).astype(np.float32)
    c_new, h = port.lstm_step(A, W, bias, g["lstm_c"])
    assert np.abs(c_new - g["lstm_c_ref"]).max() < 0.08      # ABS_TOL of cute/test_factored_lstm.py
    assert np.abs(h.astype(np.float32) / 127.0 - g["lstm_h_ref"]).max() < 0.08
    assert np.abs(c_new - g["lstm_c_ref"]).max() < 5e-3      # f16 operand rounding only


def test_rmsnorm_and_quant_vs_test_references(golden_tests):
    g = golden_tests
    got = port.rmsnorm_f16(g["rms_x"], g["rms_res"], g["rms_w"], 2.0, 1e-5)
    assert np.abs(got.astype(np.float32) - g["rms_expected"].astype(np.float32)).max() < 5e-3  # test_rmsnorm_gpu.py:85
    q, s = port.rmsnorm_quant(g["rmsq_x"], g["rmsq_w"], g["rmsq_res"], g["rmsq_scale"], 2.0, 1e-5)
    assert np.abs(s - g["rmsq_new_scale"]).max() < 1e-4                                        # :111
    assert np.abs(q.astype(np.int32) - g["rmsq_q"].astype(np.int32)).max() <= 1                # :104-112
    q, s = port.quant(g["quant_x"])
    d = np.abs(q.astype(np.int32) - g["quant_q"].astype(np.int32))
    assert d.max() <= 1 and (d != 0).sum() <= 2 and np.abs(s - g["quant_scale"]).max() < 1e-6  # test_quant_gpu.py:58


def test_rotary_vs_test_reference(golden_tests):
    g = golden_tests
    x = g["rope_qkv"].ravel()
    for ch in (0, 1):
        off = ch * 512
        x = np.concatenate([x[:off], port.rotary_f16(x[off:], g["rope_sin"], g["rope_cos"], 2, 24, 8, 32, 24 * 1536, 1536, 64)])
    got = x.reshape(g["rope_qkv"].shape)
    assert np.array_equal(got[:, :, 2], g["rope_qkv"][:, :, 2])  # v untouched
    assert np.abs(got.astype(np.float32) - g["rope_expected"].astype(np.float32)).max() < 5e-3  # test_rotary_gpu.py:100


def test_fp8_path_vs_fly_references(golden_tests):
    import torch
    from fluke_b200 import prep
    g = golden_tests
    w_nk = np.ascontiguousarray(g["fp8_B_kn"].T)
    acc = port.gemm_fp8_f32(g["fp8_A"], w_nk)
    got = port.epi_rotary(acc, g["fp8_sa"], g["fp8_sb"], g["fp8_sin"], g["fp8_cos"], 16, 1024)
    assert np.abs(got.astype(np.float32) - g["fp8_rot_expected"].astype(np.float32)).max() < 5e-2  # fly/test_rotary.py:103
    small_nk = torch.from_numpy(np.ascontiguousarray(g["fp8_small_kn"].T))
    assert np.array_equal(prep.preshuffle_fp8_weight(small_nk).numpy(), g["fp8_small_shuffled"])
