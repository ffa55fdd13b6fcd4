"""Input and weight preparation that the reference does in torch, outside the hot path:
symmetric quantisers, rotary tables, fp8 weight pre-shuffle. These run on whatever device the
tensors are on; none of them is a GPU kernel of the library.
"""
import torch

E4M3_MAX = 448.0


def quantize_int8_rows(t, dim=-1):
    """Symmetric per-row int8 (amax/127): returns (int8, f32 dequant scale).
    Restates cute/common.py:63-69 of the reference (scale = 1/(127/amax))."""
    qm = 127
    fr = t.abs().amax(dim=dim).clamp_min(1e-8)
    qs = qm / fr
    ti = (t * qs.unsqueeze(dim)).round().clamp(-qm, qm).to(torch.int8)
    return ti, qs.to(torch.float32).reciprocal()


def quantize_fp8_rows(t):
    """Per-row e4m3 (amax/448): returns (float8_e4m3fn, f32 scale [rows]).
    Restates fp8_quantize_per_token, fly/rdna4/gemm/rdna_fp8_preshuffle_gemm.py:57-70."""
    amax = t.abs().amax(dim=-1, keepdim=True).clamp(min=1e-12)
    scale = amax / E4M3_MAX
    q = (t / scale).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn)
    return q, scale.squeeze(-1).to(torch.float32)


def preshuffle_fp8_weight(w_nk):
    """Row-major [N, K] e4m3 weight -> the [N/16, K/16, 2, 16, 8] byte layout the fp8 ABI takes
    (preshuffle_b_fp8 of fly/rdna4/gemm/rdna_fp8_preshuffle_gemm.py:40-54 applied to w^T)."""
    n, k = w_nk.shape
    assert n % 16 == 0 and k % 16 == 0
    b = w_nk.view(torch.uint8).reshape(n // 16, 16, k // 16, 2, 8)  # n0, nl, k0, kl, kp
    return b.permute(0, 2, 3, 1, 4).contiguous()


def rotary_tables(seq_len, head_dim=64, theta=10000.0, device="cpu"):
    """(sin, cos) f32 [seq_len, head_dim/2] built in f64 like test/test_rotary_gpu.py:53-58."""
    inv_freq = torch.pow(theta, torch.arange(0, head_dim, 2, dtype=torch.float64) / head_dim).reciprocal()
    freqs = torch.outer(torch.arange(seq_len, dtype=torch.float64), inv_freq)
    return (torch.sin(freqs).to(torch.float32).contiguous().to(device),
            torch.cos(freqs).to(torch.float32).contiguous().to(device))
