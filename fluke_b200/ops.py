"""Tensor-level operator interface: one function per C entry point, same name without the
`fluke_` prefix, same argument meaning and the same error behaviour (void functions exit the
process on a bad dimension, int functions raise on a non-zero return). Inputs must be
contiguous CUDA tensors; nothing here computes on the host.
"""
import ctypes

import torch

from . import lib as _lib

TX_DIMS = dict(d_model=512, dim_feedforward=2048, nhead=8, head_dim=64)


def _L():
    return _lib.load()


def _dev(*ts):
    for t in ts:
        if t is None:
            continue
        if not t.is_cuda:
            raise RuntimeError("fluke_b200.ops needs CUDA tensors (there is no CPU fallback)")
        if not t.is_contiguous():
            raise RuntimeError("fluke_b200.ops needs contiguous tensors")


def _p(t):
    return 0 if t is None else t.data_ptr()


def _check(rc, what):
    if rc != 0:
        raise RuntimeError(f"{what} failed: rc={rc} {_L().fluke_last_error().decode()}")


def set_stream(stream=None):
    """Route later launches to `stream` (torch.cuda.Stream) or back to the legacy default stream."""
    _L().fluke_set_stream(0 if stream is None else stream.cuda_stream)


# ---- memory-bound kernels -----------------------------------------------------------------

def rmsnorm(x, residual, weight, alpha, eps, out=None):
    _dev(x, residual, weight)
    out = torch.empty_like(x) if out is None else out
    _L().fluke_rmsnorm_gpu(_p(x), _p(residual), _p(weight), _p(out), x.size(0), x.size(1), float(alpha), float(eps))
    return out


def rmsnorm_quant_int8(x, weight, residual_i8, residual_scale, alpha, eps):
    """In place on (residual_i8, residual_scale)."""
    _dev(x, weight, residual_i8, residual_scale)
    _L().fluke_rmsnorm_quant_int8_gpu(_p(x), _p(weight), _p(residual_i8), _p(residual_scale),
                                      x.size(0), x.size(1), float(alpha), float(eps))
    return residual_i8, residual_scale


def rmsnorm_quant_fp8(x, weight, residual_u8, residual_scale, alpha, eps):
    _dev(x, weight, residual_u8, residual_scale)
    _L().fluke_rmsnorm_quant_fp8_gpu(_p(x), _p(weight), _p(residual_u8), _p(residual_scale),
                                     x.size(0), x.size(1), float(alpha), float(eps))
    return residual_u8, residual_scale


def quant_int8(x, out=None, scale=None):
    _dev(x)
    if out is None:
        out = torch.empty(x.shape, dtype=torch.int8, device=x.device)
    if scale is None:
        scale = torch.empty(x.size(0), dtype=torch.float32, device=x.device)
    _L().fluke_quant_int8_gpu(_p(x), _p(out), _p(scale), x.size(0), x.size(1))
    return out, scale


def quant_fp8(x, out=None, scale=None):
    _dev(x)
    if out is None:
        out = torch.empty(x.shape, dtype=torch.uint8, device=x.device)
    if scale is None:
        scale = torch.empty(x.size(0), dtype=torch.float32, device=x.device)
    _L().fluke_quant_fp8_gpu(_p(x), _p(out), _p(scale), x.size(0), x.size(1))
    return out, scale


def dequant_transpose(x, scale, fp8=False):
    """[T,N,C] int8 / e4m3 bytes -> f16 [N,T,C]."""
    _dev(x)
    t, n, c = x.shape
    out = torch.empty(n, t, c, dtype=torch.float16, device=x.device)
    fn = _L().fluke_dequant_fp8_transpose_gpu if fp8 else _L().fluke_dequant_int8_transpose_gpu
    fn(_p(x), _p(out), t, n, c, float(scale))
    return out


def rotary_emb_(x_ptr, sin, cos, batch, seq_len, n_heads, head_dim, width, sb, ss, sh):
    """In place on the f16 tensor starting at device address x_ptr (strides in elements)."""
    _dev(sin, cos)
    _L().fluke_rotary_emb_gpu(x_ptr, _p(sin), _p(cos), batch, seq_len, n_heads, head_dim, width, sb, ss, sh)


def rotary_qkv_(qkv, sin, cos, width):
    """Rotate the q and k chunks of qkv [N, seq, 3, heads, head_dim] in place, passing the full
    qkv strides (the call pattern of test/test_rotary_gpu.py:26-38)."""
    _dev(qkv)
    n, s, _, h, d = qkv.shape
    for chunk in (0, 1):
        rotary_emb_(qkv.data_ptr() + chunk * qkv.stride(2) * qkv.element_size(), sin, cos,
                    n, s, h, d, width, qkv.stride(0), qkv.stride(1), qkv.stride(3))
    return qkv


def silu_mul(x):
    _dev(x)
    h = x.size(1) // 2
    out = torch.empty(x.size(0), h, dtype=x.dtype, device=x.device)
    _L().fluke_silu_mul_gpu(_p(x), _p(out), x.size(0), h)
    return out


def flstm_step(scratch, ih_t, cell, hh_next=None):
    _dev(scratch, ih_t, cell)
    hh_next = torch.empty_like(cell) if hh_next is None else hh_next
    _L().fluke_flstm_step_gpu(_p(scratch), _p(ih_t), _p(cell), _p(hh_next), cell.size(0), cell.size(1))
    return hh_next


# ---- fused transformer kernels ------------------------------------------------------------

def int8_select(device_index=0, max_seq=2048, **dims):
    d = dict(TX_DIMS, **dims)
    b = _L().fluke_int8_select(device_index, _lib.fluke_dims_t(d["d_model"], d["dim_feedforward"],
                                                               d["nhead"], d["head_dim"], max_seq))
    return b  # None when unsupported (the caller keeps fp16, as with the reference)


def fp8_select(device_index=0, max_seq=2048, **dims):
    d = dict(TX_DIMS, **dims)
    return _L().fluke_fp8_select(device_index, _lib.fluke_dims_t(d["d_model"], d["dim_feedforward"],
                                                                d["nhead"], d["head_dim"], max_seq))


def qkv_rotary_i8(backend, a_i8, wqkv_i8, scale_a, scale_b, sin, cos, seqlen, out=None):
    _dev(a_i8, wqkv_i8, scale_a, scale_b, sin, cos)
    m = a_i8.size(0)
    out = torch.empty(m, wqkv_i8.size(0), dtype=torch.float16, device=a_i8.device) if out is None else out
    _check(_L().fluke_qkv_rotary_i8_gpu(backend, _p(out), _p(a_i8), _p(wqkv_i8), _p(scale_a), _p(scale_b),
                                        _p(sin), _p(cos), m, seqlen), "fluke_qkv_rotary_i8_gpu")
    return out


def gated_mlp_i8(backend, a_i8, gate_i8, up_i8, scale_a, scale_gate, scale_up, out=None):
    _dev(a_i8, gate_i8, up_i8, scale_a, scale_gate, scale_up)
    m = a_i8.size(0)
    out = torch.empty(m, gate_i8.size(0), dtype=torch.float16, device=a_i8.device) if out is None else out
    _check(_L().fluke_gated_mlp_i8_gpu(backend, _p(out), _p(a_i8), _p(gate_i8), _p(up_i8), _p(scale_a),
                                       _p(scale_gate), _p(scale_up), m), "fluke_gated_mlp_i8_gpu")
    return out


def qkv_rotary_fp8(backend, a_fp8, w_fp8, scale_a, scale_b, sin, cos, seqlen, plain=False, out=None):
    """w_fp8: PRESHUFFLED bytes (plain=False, the reference ABI) or row-major [N,K] (plain=True)."""
    _dev(a_fp8, w_fp8, scale_a, scale_b, sin, cos)
    m = a_fp8.size(0)
    out = torch.empty(m, 3 * TX_DIMS["d_model"], dtype=torch.float16, device=a_fp8.device) if out is None else out
    fn = _L().fluke_qkv_rotary_fp8_plain_gpu if plain else _L().fluke_qkv_rotary_fp8_gpu
    _check(fn(backend, _p(out), _p(a_fp8), _p(w_fp8), _p(scale_a), _p(scale_b), _p(sin), _p(cos), m, seqlen),
           "fluke_qkv_rotary_fp8_gpu")
    return out


def gated_mlp_fp8(backend, a_fp8, gate_fp8, up_fp8, scale_a, scale_gate, scale_up, plain=False, out=None):
    _dev(a_fp8, gate_fp8, up_fp8, scale_a, scale_gate, scale_up)
    m = a_fp8.size(0)
    out = torch.empty(m, TX_DIMS["dim_feedforward"], dtype=torch.float16, device=a_fp8.device) if out is None else out
    fn = _L().fluke_gated_mlp_fp8_plain_gpu if plain else _L().fluke_gated_mlp_fp8_gpu
    _check(fn(backend, _p(out), _p(a_fp8), _p(gate_fp8), _p(up_fp8), _p(scale_a), _p(scale_gate), _p(scale_up), m),
           "fluke_gated_mlp_fp8_gpu")
    return out


# ---- base GEMMs (additive) ----------------------------------------------------------------

def gemm_i8(a_i8, b_i8, scale_a, scale_b, const_scale_a=0.0):
    _dev(a_i8, b_i8, scale_a, scale_b)
    m, k = a_i8.shape
    n = b_i8.size(0)
    out = torch.empty(m, n, dtype=torch.float16, device=a_i8.device)
    _check(_L().fluke_gemm_i8_gpu(_p(out), _p(a_i8), _p(b_i8), _p(scale_a), float(const_scale_a), _p(scale_b),
                                  m, n, k), "fluke_gemm_i8_gpu")
    return out


def gemm_i8_s32(a_i8, b_i8):
    _dev(a_i8, b_i8)
    m, k = a_i8.shape
    n = b_i8.size(0)
    out = torch.empty(m, n, dtype=torch.int32, device=a_i8.device)
    _check(_L().fluke_gemm_i8_s32_gpu(_p(out), _p(a_i8), _p(b_i8), m, n, k), "fluke_gemm_i8_s32_gpu")
    return out


def gemm_fp8(a_fp8, b_fp8_nk, scale_a, scale_b):
    _dev(a_fp8, b_fp8_nk, scale_a, scale_b)
    m, k = a_fp8.shape
    n = b_fp8_nk.size(0)
    out = torch.empty(m, n, dtype=torch.float16, device=a_fp8.device)
    _check(_L().fluke_gemm_fp8_gpu(_p(out), _p(a_fp8), _p(b_fp8_nk), _p(scale_a), _p(scale_b), m, n, k),
           "fluke_gemm_fp8_gpu")
    return out


def fp8_unshuffle(w_preshuffled, n, k):
    _dev(w_preshuffled)
    out = torch.empty(n, k, dtype=torch.uint8, device=w_preshuffled.device)
    _check(_L().fluke_fp8_unshuffle_gpu(_p(out), _p(w_preshuffled), n, k), "fluke_fp8_unshuffle_gpu")
    return out


# ---- factored LSTM (additive) ---------------------------------------------------------------

def down_proj_i8(a_i8, w_i8, scale_a, scale_b, out=None):
    """f16 [M,N] = int8 GEMM * (sa*sb); scale_a None = the fixed 1/127 of an int8 hidden state."""
    _dev(a_i8, w_i8, scale_a, scale_b)
    m, k = a_i8.shape
    n = w_i8.size(0)
    out = torch.empty(m, n, dtype=torch.float16, device=a_i8.device) if out is None else out
    _check(_L().fluke_down_proj_i8_gpu(_p(out), out.stride(0), _p(a_i8), _p(w_i8), _p(scale_a), _p(scale_b),
                                       m, n, k), "fluke_down_proj_i8_gpu")
    return out


def down_proj_fp8(a_fp8, w_fp8_nk, scale_a, scale_b, out=None):
    """f16 [M,N] = (e4m3 GEMM * sa[m]) * sb[n]; a_fp8 [M,K], w_fp8_nk [N,K] as uint8 e4m3 bytes."""
    _dev(a_fp8, w_fp8_nk, scale_a, scale_b)
    m, k = a_fp8.shape
    n = w_fp8_nk.size(0)
    out = torch.empty(m, n, dtype=torch.float16, device=a_fp8.device) if out is None else out
    _check(_L().fluke_down_proj_fp8_gpu(_p(out), out.stride(0), _p(a_fp8), _p(w_fp8_nk), _p(scale_a), _p(scale_b),
                                        m, n, k), "fluke_down_proj_fp8_gpu")
    return out


def factored_lstm_step_i8(A, W4, bias4, c, h_out=None, fp8_export_name=False):
    """A f16 [B,Kc]; W4 f16 [4H,Kc] (gate-major i,f,g,o); bias4 f32 [4H]; c f32 [B,H] in place."""
    _dev(A, W4, bias4, c)
    b, kc = A.shape
    h = c.size(1)
    h_out = torch.empty(b, h, dtype=torch.int8, device=A.device) if h_out is None else h_out
    w = [W4.data_ptr() + g * h * kc * 2 for g in range(4)]
    bs = [bias4.data_ptr() + g * h * 4 for g in range(4)]
    fn = _L().fluke_factored_lstm_step_fp8_gpu if fp8_export_name else _L().fluke_factored_lstm_step_i8_gpu
    _check(fn(_p(A), w[0], w[1], w[2], w[3], bs[0], bs[1], bs[2], bs[3], _p(c), _p(h_out), b, h, kc),
           "fluke_factored_lstm_step_i8_gpu")
    return h_out


def factored_lstm_layer_i8(x_i8, x_scale, dn_ih, dn_ih_scale, dn_hh, dn_hh_scale, w_up, bias, c, h,
                           reverse=False, h_out=None, workspace=None, phase_mask=7):
    """One layer over x_i8 [T,B,H]; c (f32 [B,H]) and h (int8 [B,H]) are state, updated in place.
    phase_mask != 7 launches only some kernel classes (timing aid, see fluke.h)."""
    _dev(x_i8, x_scale, dn_ih, dn_ih_scale, dn_hh, dn_hh_scale, w_up, bias, c, h)
    t, b, hd = x_i8.shape
    r = dn_ih.size(0)
    need = _L().fluke_factored_lstm_layer_workspace(t, b, hd, r)
    if workspace is None or workspace.numel() < need:
        workspace = torch.empty(need, dtype=torch.uint8, device=x_i8.device)
    h_out = torch.empty(t, b, hd, dtype=torch.int8, device=x_i8.device) if h_out is None else h_out
    layer = _lib.fluke_flstm_layer_t(t, b, hd, r, 1 if reverse else 0, _p(x_i8), _p(x_scale),
                                     _p(dn_ih), _p(dn_ih_scale), _p(dn_hh), _p(dn_hh_scale),
                                     _p(w_up), _p(bias), _p(c), _p(h), _p(h_out),
                                     _p(workspace), workspace.numel())
    if phase_mask == 7:
        _check(_L().fluke_factored_lstm_layer_i8_gpu(ctypes.byref(layer)), "fluke_factored_lstm_layer_i8_gpu")
    else:
        _check(_L().fluke_factored_lstm_layer_phases_gpu(ctypes.byref(layer), phase_mask),
               "fluke_factored_lstm_layer_phases_gpu")
    return h_out
