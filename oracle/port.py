"""numpy front end of oracle/liboracle.so (built from oracle/fluke_oracle.c by
oracle/build_oracle.py). Arrays are numpy; f16 data is passed as float16 arrays (viewed as
uint16 bit patterns), e4m3 data as uint8. TEST INFRASTRUCTURE ONLY.
"""
import ctypes
import os
import subprocess
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(HERE, "liboracle.so")
_LIB = None
P, I, F, L = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_long


def lib():
    global _LIB
    if _LIB is None:
        src = os.path.join(HERE, "fluke_oracle.c")
        if not os.path.isfile(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
            subprocess.run([sys.executable, os.path.join(HERE, "build_oracle.py")], check=True, stdout=subprocess.DEVNULL)
        _LIB = ctypes.CDLL(_SO)
        _LIB.orc_e4m3_decode.restype = F
        _LIB.orc_e4m3_decode.argtypes = [ctypes.c_uint8]
        _LIB.orc_e4m3_encode.restype = ctypes.c_uint8
        _LIB.orc_e4m3_encode.argtypes = [F]
    return _LIB


def _c(a, dtype):
    a = np.ascontiguousarray(a)
    if dtype == np.float16:
        assert a.dtype == np.float16, a.dtype
    else:
        assert a.dtype == dtype, (a.dtype, dtype)
    return a


def _ptr(a):
    return None if a is None else a.ctypes.data_as(P)


def _call(name, *args):
    fn = getattr(lib(), name)
    conv = []
    for a in args:
        if isinstance(a, np.ndarray) or a is None:
            conv.append(_ptr(a))
        elif isinstance(a, float):
            conv.append(F(a))
        elif isinstance(a, tuple) and a[0] == "long":
            conv.append(L(a[1]))
        else:
            conv.append(I(int(a)))
    fn.restype = None
    fn(*conv)


def set_threads(n):
    """OpenMP threads used by the parallel oracle loops; returns the count in effect."""
    fn = lib().orc_set_threads
    fn.restype = I
    fn.argtypes = [I]
    return fn(int(n))


def set_fma_modes(sumsq=1, resadd=1, rot_lo=1, rot_hi=1, gate=1, cell=2):
    _call("orc_set_fma_modes", sumsq, resadd, rot_lo, rot_hi, gate, cell)


# ---- fp32 CPU trio ---------------------------------------------------------------------------
def rotary_f32(x, sin, cos, batch, seq_len, n_heads, width, sb, ss, sh):
    x = _c(x, np.float32).copy()
    _call("orc_rotary_f32", x, _c(sin, np.float32), _c(cos, np.float32), batch, seq_len, n_heads, width,
          ("long", sb), ("long", ss), ("long", sh))
    return x


def rmsnorm_f32(x, res, w, alpha, eps):
    x = _c(x, np.float32)
    out = np.empty_like(x)
    _call("orc_rmsnorm_f32", x, _c(res, np.float32), _c(w, np.float32), out, x.shape[0], x.shape[1],
          float(alpha), float(eps))
    return out


def flstm_step_f32(scratch, ih, cell):
    cell = _c(cell, np.float32).copy()
    hh = np.empty_like(cell)
    _call("orc_flstm_step_f32", _c(scratch, np.float32), _c(ih, np.float32), cell, hh, cell.shape[0], cell.shape[1])
    return cell, hh


# ---- pure-CUDA kernel restatements -------------------------------------------------------------
def e4m3_decode_table():
    return np.array([lib().orc_e4m3_decode(i) for i in range(256)], dtype=np.float32)


def e4m3_encode(values):
    v = np.asarray(values, dtype=np.float32).ravel()
    return np.array([lib().orc_e4m3_encode(float(x)) for x in v], dtype=np.uint8).reshape(np.shape(values))


def rmsnorm_f16(x, res, w, alpha, eps):
    x = _c(x, np.float16)
    out = np.empty_like(x)
    _call("orc_rmsnorm_f16", x, _c(res, np.float16), _c(w, np.float16), out, x.shape[0], x.shape[1],
          float(alpha), float(eps))
    return out


def rmsnorm_quant(x, w, res, res_scale, alpha, eps, fp8=False):
    """Returns (new residual bytes as int8/uint8, new scales)."""
    x = _c(x, np.float16)
    res = np.ascontiguousarray(res).copy()
    scale = _c(res_scale, np.float32).copy()
    _call("orc_rmsnorm_quant", x, _c(w, np.float16), res.view(np.uint8), scale, x.shape[0], x.shape[1],
          float(alpha), float(eps), 1 if fp8 else 0)
    return res, scale


def quant(x, fp8=False):
    x = _c(x, np.float16)
    out = np.empty(x.shape, dtype=np.uint8)
    scale = np.empty(x.shape[0], dtype=np.float32)
    _call("orc_quant", x, out, scale, x.shape[0], x.shape[1], 1 if fp8 else 0)
    return (out if fp8 else out.view(np.int8)), scale


def dequant_transpose(x, scale, fp8=False):
    x = np.ascontiguousarray(x)
    t, n, c = x.shape
    out = np.empty((n, t, c), dtype=np.float16)
    _call("orc_dequant_transpose", x.view(np.uint8), out, t, n, c, float(scale), 1 if fp8 else 0)
    return out


def rotary_f16(x, sin, cos, batch, seq_len, n_heads, width, sb, ss, sh):
    """x: flat float16 buffer (copied); strides in elements."""
    x = _c(x, np.float16).copy()
    _call("orc_rotary_f16", x, _c(sin, np.float32), _c(cos, np.float32), batch, seq_len, n_heads, width,
          ("long", sb), ("long", ss), ("long", sh))
    return x


def silu_mul_f16(x):
    x = _c(x, np.float16)
    h = x.shape[1] // 2
    out = np.empty((x.shape[0], h), dtype=np.float16)
    _call("orc_silu_mul_f16", x, out, x.shape[0], h)
    return out


def flstm_step_f16(scratch, ih, cell):
    cell = _c(cell, np.float16).copy()
    hh = np.empty_like(cell)
    _call("orc_flstm_step_f16", _c(scratch, np.float16), _c(ih, np.float16), cell, hh, cell.shape[0], cell.shape[1])
    return cell, hh


# ---- GEMM class ----------------------------------------------------------------------------------
def gemm_i8_s32(a, b):
    a, b = _c(a, np.int8), _c(b, np.int8)
    out = np.empty((a.shape[0], b.shape[0]), dtype=np.int32)
    _call("orc_gemm_i8_s32", a, b, out, a.shape[0], b.shape[0], a.shape[1])
    return out


def gemm_fp8_f32(a, b):
    a, b = _c(a, np.uint8), _c(b, np.uint8)
    out = np.empty((a.shape[0], b.shape[0]), dtype=np.float32)
    _call("orc_gemm_fp8_f32", a, b, out, a.shape[0], b.shape[0], a.shape[1])
    return out


def epi_dequant(acc, sa, sb, const_sa=0.0):
    acc = _c(np.asarray(acc, dtype=np.float32), np.float32)
    out = np.empty(acc.shape, dtype=np.float16)
    _call("orc_epi_dequant", acc, None if sa is None else _c(sa, np.float32), float(const_sa),
          _c(sb, np.float32), out, acc.shape[0], acc.shape[1])
    return out


def epi_dequant2(acc, sa, sb):
    acc = _c(np.asarray(acc, dtype=np.float32), np.float32)
    out = np.empty(acc.shape, dtype=np.float16)
    _call("orc_epi_dequant2", acc, _c(sa, np.float32), _c(sb, np.float32), out, acc.shape[0], acc.shape[1])
    return out


def epi_rotary(acc, sa, sb, sin, cos, seqlen, qk_cols):
    acc = _c(np.asarray(acc, dtype=np.float32), np.float32)
    out = np.empty(acc.shape, dtype=np.float16)
    _call("orc_epi_rotary", acc, _c(sa, np.float32), _c(sb, np.float32), _c(sin, np.float32),
          _c(cos, np.float32), seqlen, qk_cols, out, acc.shape[0], acc.shape[1])
    return out


def epi_silu(acc_g, acc_u, sa, sbg, sbu):
    acc_g = _c(np.asarray(acc_g, dtype=np.float32), np.float32)
    acc_u = _c(np.asarray(acc_u, dtype=np.float32), np.float32)
    out = np.empty(acc_g.shape, dtype=np.float16)
    _call("orc_epi_silu", acc_g, acc_u, _c(sa, np.float32), _c(sbg, np.float32), _c(sbu, np.float32), out,
          acc_g.shape[0], acc_g.shape[1])
    return out


def qkv_rotary_i8(a, w, sa, sb, sin, cos, seqlen, qk_cols=1024):
    return epi_rotary(gemm_i8_s32(a, w), sa, sb, sin, cos, seqlen, qk_cols)


def gated_mlp_i8(a, wg, wu, sa, sbg, sbu):
    return epi_silu(gemm_i8_s32(a, wg), gemm_i8_s32(a, wu), sa, sbg, sbu)


def gemm_i8(a, w, sa, sb, const_sa=0.0):
    return epi_dequant(gemm_i8_s32(a, w), sa, sb, const_sa)


# ---- factored LSTM ---------------------------------------------------------------------------------
def down_proj(a, w, sa, sb, const_sa=1.0 / 127.0):
    a, w = _c(a, np.int8), _c(w, np.int8)
    out = np.empty((a.shape[0], w.shape[0]), dtype=np.float16)
    _call("orc_down_proj", a, w, None if sa is None else _c(sa, np.float32), float(np.float32(const_sa)),
          _c(sb, np.float32), out, a.shape[0], w.shape[0], a.shape[1])
    return out


def down_proj_fp8(a, w_nk, sa, sb):
    """fp8 down-projection of the fp8 stack: the base fp8 GEMM with N = R, K = H, out f16 =
    (acc * sa[m]) * sb[n] (fly/rdna4/factored_lstm/export_fp8_factored_lstm.py:161-181; epilogue
    fly/rdna4/gemm/rdna_fp8_preshuffle_gemm.py:379-393). a [M,K] and w_nk [N,K] are e4m3 bytes."""
    return epi_dequant2(gemm_fp8_f32(a, w_nk), sa, sb)


def lstm_step(A, W4, bias4, c):
    """Returns (c_new f32 [B,H], h int8 [B,H])."""
    A, W4 = _c(A, np.float16), _c(W4, np.float16)
    c = _c(c, np.float32).copy()
    h = np.empty(c.shape, dtype=np.int8)
    _call("orc_lstm_step", A, W4, _c(bias4, np.float32), c, h, c.shape[0], c.shape[1], A.shape[1])
    return c, h


def lstm_layer(x, x_scale, dn_ih, dn_ih_s, dn_hh, dn_hh_s, w_up, bias, c, h, reverse=False):
    """Returns (h_out int8 [T,B,H], c_final, h_final)."""
    x = _c(x, np.int8)
    t, b, hd = x.shape
    r = dn_ih.shape[0]
    c = _c(c, np.float32).copy()
    h = _c(h, np.int8).copy()
    h_out = np.empty((t, b, hd), dtype=np.int8)
    _call("orc_lstm_layer", x, None if x_scale is None else _c(x_scale, np.float32), _c(dn_ih, np.int8),
          _c(dn_ih_s, np.float32), _c(dn_hh, np.int8), _c(dn_hh_s, np.float32), _c(w_up, np.float16),
          _c(bias, np.float32), c, h, h_out, t, b, hd, r, 1 if reverse else 0)
    return h_out, c, h
