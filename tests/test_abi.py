"""The C-ABI boundary: lib/libfluke.so loads, exports every symbol include/fluke/fluke.h
declares, keeps the reference loader's contract, and its CPU functions agree bit for bit with
the oracle and with the reference's own nn_cpu.c (when oracle/_ref is built)."""
import ctypes
import os
import re

import numpy as np
import pytest

from conftest import ROOT
from oracle import port, ref


def _declared_functions():
    text = open(os.path.join(ROOT, "include", "fluke", "fluke.h")).read()
    text += open(os.path.join(ROOT, "include", "fluke", "fluke_error.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    text = re.sub(r"#define[^\n]*(\\\n[^\n]*)*", "", text)
    names = set(re.findall(r"\b((?:fluke|get_fluke|set_fluke)_\w+)\s*\(", text))
    return sorted(n for n in names if not n.endswith("_t"))


def test_every_declared_symbol_is_exported(flib):
    names = _declared_functions()
    assert len(names) >= 35
    for n in names:
        assert hasattr(flib, n), f"{n} declared in include/fluke/*.h but not exported"


def test_reference_loader_contract():
    import fluke_lib
    lib = fluke_lib.load()
    assert set(fluke_lib._SIGNATURES) == {
        "fluke_rotary_emb_gpu", "fluke_silu_mul_gpu", "fluke_rmsnorm_gpu", "fluke_quant_int8_gpu",
        "fluke_quant_fp8_gpu", "fluke_rmsnorm_quant_int8_gpu", "fluke_rmsnorm_quant_fp8_gpu",
        "fluke_dequant_fp8_transpose_gpu", "fluke_dequant_int8_transpose_gpu", "fluke_flstm_step_gpu"}
    for name, argtypes in fluke_lib._SIGNATURES.items():
        fn = getattr(lib, name)
        assert fn.restype is None and list(fn.argtypes) == list(argtypes)
    assert os.path.samefile(fluke_lib._SO, os.path.join(ROOT, "lib", "libfluke.so"))


def test_log_level_roundtrip(flib):
    assert flib.get_fluke_log_level() == 4  # FLUKE_LOG_VERB, the reference default
    flib.set_fluke_log_level(1)
    assert flib.get_fluke_log_level() == 1
    flib.set_fluke_log_level(4)


def test_select_without_supported_device_returns_null(flib):
    import torch
    from fluke_b200 import lib as L
    if torch.cuda.is_available():
        pytest.skip("covered by the gpu tests")
    dims = L.fluke_dims_t(512, 2048, 8, 64, 2048)
    assert flib.fluke_int8_select(0, dims) is None
    assert flib.fluke_fp8_select(0, dims) is None
    assert flib.fluke_qkv_rotary_i8_gpu(None, 0, 0, 0, 0, 0, 0, 0, 4, 2) != 0
    assert flib.fluke_gated_mlp_fp8_gpu(None, 0, 0, 0, 0, 0, 0, 0, 4) != 0


def test_ops_refuse_cpu_tensors():
    import torch
    from fluke_b200 import ops
    with pytest.raises(RuntimeError):
        ops.quant_int8(torch.zeros(4, 8, dtype=torch.float16))


def _tables(seq, w):
    fr = np.outer(np.arange(seq), 1.0 / 10000 ** (np.arange(0, 2 * w, 2) / (2 * w)))
    return np.sin(fr).astype(np.float32), np.cos(fr).astype(np.float32)


@pytest.mark.parametrize("batch,seq,heads,hd,w,threads", [
    (4, 50, 8, 64, 32, 3), (1, 7, 2, 16, 4, 8), (5, 3, 1, 64, 32, 1), (32, 100, 8, 64, 32, 8), (3, 9, 4, 32, 8, 64)])
def test_rotary_cpu_matches_oracle_and_reference(flib, batch, seq, heads, hd, w, threads):
    rng = np.random.default_rng(batch * 1000 + seq)
    x = rng.standard_normal((batch, seq, 3, heads, hd)).astype(np.float32)
    sin, cos = _tables(seq, w)
    sb, ss, sh = seq * 3 * heads * hd, 3 * heads * hd, hd
    got = x.copy()
    flib.fluke_rotary_emb_cpu(got.ctypes.data, sin.ctypes.data, cos.ctypes.data, batch, seq, heads, hd, w, sb, ss, sh, threads)
    exp = port.rotary_f32(x.ravel(), sin, cos, batch, seq, heads, w, sb, ss, sh).reshape(x.shape)
    assert np.array_equal(got, exp)
    assert np.array_equal(got[:, :, 1:], x[:, :, 1:])  # only the first chunk (q) was addressed
    r = ref.cpu()
    if r is not None:
        theirs = x.copy()
        r.fluke_rotary_emb_cpu(theirs.ctypes.data, sin.ctypes.data, cos.ctypes.data, batch, seq, heads, hd, w, sb, ss, sh, threads)
        assert np.array_equal(got, theirs)


@pytest.mark.parametrize("n,h,threads", [(77, 512, 4), (1, 768, 8), (9, 10, 3), (300, 1024, 8)])
def test_rmsnorm_cpu_matches_oracle_and_reference(flib, n, h, threads):
    rng = np.random.default_rng(n + h)
    x, res = rng.standard_normal((n, h)).astype(np.float32), rng.standard_normal((n, h)).astype(np.float32)
    w = rng.standard_normal(h).astype(np.float32)
    got = np.empty_like(x)
    flib.fluke_rmsnorm_cpu(x.ctypes.data, res.ctypes.data, w.ctypes.data, got.ctypes.data, n, h, 2.0, 1e-5, threads)
    assert np.array_equal(got, port.rmsnorm_f32(x, res, w, 2.0, 1e-5))
    r = ref.cpu()
    if r is not None:
        theirs = np.empty_like(x)
        r.fluke_rmsnorm_cpu(x.ctypes.data, res.ctypes.data, w.ctypes.data, theirs.ctypes.data, n, h, 2.0, 1e-5, threads)
        assert np.array_equal(got, theirs)


@pytest.mark.parametrize("n,h,threads", [(33, 96, 2), (1, 768, 8), (128, 64, 5)])
def test_flstm_step_cpu_matches_oracle_and_reference(flib, n, h, threads):
    rng = np.random.default_rng(n * h)
    s, ih = rng.standard_normal((n, 4 * h)).astype(np.float32), rng.standard_normal((n, 4 * h)).astype(np.float32)
    cell = rng.standard_normal((n, h)).astype(np.float32)
    c1, h1 = cell.copy(), np.empty_like(cell)
    flib.fluke_flstm_step_cpu(s.ctypes.data, ih.ctypes.data, c1.ctypes.data, h1.ctypes.data, n, h, threads)
    c2, h2 = port.flstm_step_f32(s, ih, cell)
    assert np.array_equal(c1, c2) and np.array_equal(h1, h2)
    r = ref.cpu()
    if r is not None:
        c3, h3 = cell.copy(), np.empty_like(cell)
        r.fluke_flstm_step_cpu(s.ctypes.data, ih.ctypes.data, c3.ctypes.data, h3.ctypes.data, n, h, threads)
        assert np.array_equal(c1, c3) and np.array_equal(h1, h3)


def test_cpu_functions_accept_empty_batches(flib):
    z = np.zeros(8, dtype=np.float32)
    flib.fluke_rmsnorm_cpu(z.ctypes.data, z.ctypes.data, z.ctypes.data, z.ctypes.data, 0, 8, 1.0, 1e-5, 4)
    flib.fluke_flstm_step_cpu(z.ctypes.data, z.ctypes.data, z.ctypes.data, z.ctypes.data, 0, 2, 4)
    flib.fluke_rotary_emb_cpu(z.ctypes.data, z.ctypes.data, z.ctypes.data, 0, 1, 1, 8, 4, 8, 8, 8, 4)
    assert not z.any()


def test_workspace_size_formula(flib):
    assert flib.fluke_factored_lstm_layer_workspace(1000, 1024, 768, 128) >= (1000 * 1024 + 1024) * 128 * 2
    assert flib.fluke_factored_lstm_layer_workspace(0, 4, 64, 64) == 0
