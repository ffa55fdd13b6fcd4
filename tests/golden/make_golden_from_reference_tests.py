"""Generate tests/golden/reference_tests.npz by IMPORTING the reference's own Python test
modules and calling their reference functions on the CPU.

    python tests/golden/make_golden_from_reference_tests.py --ref-dir <reference checkout>

Runs only where the reference checkout is mounted (the build machine); the resulting fixture
is committed and is what the test-suite reads. `.cuda()` is patched to the identity so the
torch references run on CPU tensors; `flydsl` (AMD-only, absent) is stubbed so the pure-torch
helpers of the fp8 modules import. Inputs are drawn exactly as each reference test draws them
(same seeds, same call order).
"""
import argparse
import importlib
import importlib.util
import os
import sys
import types
from unittest import mock

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--ref-dir", default=os.environ.get("FLUKE_REFERENCE_DIR"), required=os.environ.get("FLUKE_REFERENCE_DIR") is None,
                    help="checkout of the reference project (or set FLUKE_REFERENCE_DIR)")
    ref = ap.parse_args().ref_dir
    for sub in ("fly/rdna4/gemm", "fly/rdna4/rotary", "test", "", "cute"):  # cute/ first: its common.py
        sys.path.insert(0, os.path.join(ref, sub))
    torch.Tensor.cuda = lambda self, *a, **k: self
    for name in ("flydsl", "flydsl.compiler", "flydsl.expr", "flydsl._mlir", "flydsl._mlir.dialects",
                 "flydsl.runtime", "flydsl.runtime.device", "flydsl.compiler.kernel_function",
                 "flydsl._mlir.ir", "flydsl.expr.typing", "flydsl.utils", "flydsl.utils.smem_allocator"):
        sys.modules.setdefault(name, mock.MagicMock())
    out = {}
    T = lambda t: t.detach().cpu().numpy()

    # ---- cute/test_rotary.py (jit dims: batch 4 x seq 16, :145-167) --------------------------
    cute_common = importlib.import_module("common")
    tr = importlib.import_module("test_rotary")
    d = types.SimpleNamespace(nhead=8, head_dim=64, rotary_dim=64, K=512, L=1, batch_size=4, sequence_len=16)
    d.M = 64; d.N = 1536; d.seqlen = 16; d.sincos_width = 32
    torch.manual_seed(0)
    A, sa = cute_common.quantize_tensor(torch.randn(d.M, d.K) * 0.1, dim=-1)
    B, sb = cute_common.quantize_tensor(torch.randn(d.N, d.K) * 0.1, dim=-1)
    inv_freq = 1.0 / (10000.0 ** (torch.arange(0, d.sincos_width).float() / d.head_dim * 2))
    freqs = torch.outer(torch.arange(d.seqlen).float(), inv_freq)
    sin, cos = freqs.sin().contiguous(), freqs.cos().contiguous()
    C_gemm = (A.float() * sa[:, None]) @ (B.float() * sb[:, None]).T
    exp = tr.torch_reference(C_gemm, sin, cos, d)
    out.update(rot_A=T(A), rot_sa=T(sa), rot_B=T(B), rot_sb=T(sb), rot_sin=T(sin), rot_cos=T(cos),
               rot_expected=T(exp).astype(np.float16))

    # ---- cute/test_dual_gemm_silu.py (jit dims M=64, K=512, :139-151; N cut to 256 to keep the fixture small) -------------------------
    td = importlib.import_module("test_dual_gemm_silu")
    torch.manual_seed(0)
    A, sa = cute_common.quantize_tensor(torch.randn(64, 512) * 0.1, dim=-1)
    Bg, sbg = cute_common.quantize_tensor(torch.randn(256, 512) * 0.1, dim=-1)
    Bu, sbu = cute_common.quantize_tensor(torch.randn(256, 512) * 0.1, dim=-1)
    exp = td.torch_reference(A, Bg, Bu, sa, sbg, sbu)
    out.update(silu_A=T(A), silu_sa=T(sa), silu_Bg=T(Bg), silu_sbg=T(sbg), silu_Bu=T(Bu), silu_sbu=T(sbu),
               silu_expected=T(exp).astype(np.float16))

    # ---- cute/test_gemm.py: int8 GEMM vs fp16-dequantised torch GEMM (:70-90) ------------------
    torch.manual_seed(0)
    A, sa = cute_common.quantize_tensor(torch.randn(64, 512) * 0.1, dim=-1)
    B, sb = cute_common.quantize_tensor(torch.randn(256, 512) * 0.1, dim=-1)
    acc = (A.int() @ B.int().T)
    out.update(gemm_A=T(A), gemm_sa=T(sa), gemm_B=T(B), gemm_sb=T(sb), gemm_acc=T(acc).astype(np.int32))

    # ---- cute/test_factored_lstm.py (make_inputs :40-51, torch_reference :54-65) ----------------
    tl = importlib.import_module("test_factored_lstm")
    B_, H, Khh, R = 64, 64, 128, 128
    inp = tl.make_inputs(B_, H, Khh, R, "cpu")
    h_ref, c_ref = tl.torch_reference(inp, H)
    out.update({f"lstm_{k}": T(v) for k, v in inp.items()})
    out.update(lstm_h_ref=T(h_ref), lstm_c_ref=T(c_ref))

    # ---- test/test_rmsnorm_gpu.py (ref_rmsnorm :46-49, ref_rmsnorm_quant_int8 :52-60) -------------
    tn = importlib.import_module("test_rmsnorm_gpu")
    torch.manual_seed(0)
    n, hd = 64, 512
    x = torch.randn(n, hd).to(torch.float16); res = torch.randn(n, hd).to(torch.float16)
    w = torch.randn(hd).to(torch.float16)
    out.update(rms_x=T(x), rms_res=T(res), rms_w=T(w), rms_expected=T(tn.ref_rmsnorm(x, res, w, 2.0, 1e-5)))
    x8 = torch.randn(n, hd).to(torch.float16); w8 = torch.randn(hd).to(torch.float16)
    r8 = torch.randint(-127, 128, (n, hd), dtype=torch.int8); rs = torch.rand(n) * 0.02 + 0.001
    q, s, norm = tn.ref_rmsnorm_quant_int8(x8, w8, r8.clone(), rs.clone(), 2.0, 1e-5)
    out.update(rmsq_x=T(x8), rmsq_w=T(w8), rmsq_res=T(r8), rmsq_scale=T(rs), rmsq_q=T(q), rmsq_new_scale=T(s))

    # ---- test/test_quant_gpu.py (quantize_tensor_ref :30-37) --------------------------------------
    tq = importlib.import_module("test_quant_gpu")
    torch.manual_seed(0)
    x = (torch.randn(48, 512).to(torch.float16) * 3.0)
    q, s = tq.quantize_tensor_ref(x.float())
    out.update(quant_x=T(x), quant_q=T(q), quant_scale=T(s))

    # ---- test/test_rotary_gpu.py (build_cos_sin :53-58, reference :61-73) ---------------------------
    tg = importlib.import_module("test_rotary_gpu")
    cos_t, sin_t = tg.build_cos_sin(64, "cpu")
    torch.manual_seed(0)
    qkv = torch.randn(2, 24, 3, 8, 64).to(torch.float16).contiguous()
    exp = tg.reference(qkv, cos_t, sin_t, 32)
    out.update(rope_qkv=T(qkv), rope_cos=T(cos_t[:24]), rope_sin=T(sin_t[:24]), rope_expected=T(exp))

    # ---- fly fp8 helpers (rdna_fp8_preshuffle_gemm.py:40-86) and fly/test_rotary.py reference -------
    fg = importlib.import_module("rdna_fp8_preshuffle_gemm")
    torch.manual_seed(42)
    A = torch.randn(32, 512) * 0.1
    Bkn = torch.randn(512, 1536) * 0.1
    A8, sa = fg.fp8_quantize_per_token(A)
    B8, sb = fg.fp8_quantize_per_channel(Bkn)
    seqlen = 16
    theta = torch.arange(seqlen).float().unsqueeze(1) * 0.01
    rot = torch.arange(32).float().unsqueeze(0)
    sin_b, cos_b = torch.sin(theta + rot).contiguous(), torch.cos(theta + rot).contiguous()
    C = ((A8.float() * sa[:, None]) @ (B8.float() * sb[None, :])).clone()
    rows = torch.arange(32)
    cr, sr = cos_b[rows % seqlen], sin_b[rows % seqlen]
    for chunk_start in (0, 512):  # fly/test_rotary.py:56-68
        for h in range(8):
            h0 = chunk_start + h * 64
            x0 = C[:, h0:h0 + 32].clone(); x1 = C[:, h0 + 32:h0 + 64].clone()
            C[:, h0:h0 + 32] = x0 * cr - x1 * sr
            C[:, h0 + 32:h0 + 64] = x0 * sr + x1 * cr
    out.update(fp8_A=T(A8.view(torch.uint8)), fp8_sa=T(sa), fp8_B_kn=T(B8.view(torch.uint8)), fp8_sb=T(sb),
               fp8_sin=T(sin_b), fp8_cos=T(cos_b), fp8_rot_expected=T(C).astype(np.float16))
    # the pre-shuffled layout itself, on a small weight
    small = B8[:64, :48].contiguous()
    out.update(fp8_small_kn=T(small.view(torch.uint8)), fp8_small_shuffled=T(fg.preshuffle_b_fp8(small).contiguous()))

    # ---- fly/test_factored_lstm.py: torch reference of the fp8 stack's fused step (:38-47), inputs
    # drawn as the test draws them (:60-66) at a smaller hidden size to keep the fixture small -----
    spec = importlib.util.spec_from_file_location("fly_test_factored_lstm", os.path.join(ref, "fly", "test_factored_lstm.py"))
    fl = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(fl)
    torch.manual_seed(0)
    M, Hs, Kc = 64, 128, fl.Kc
    A = (torch.randn(M, Kc) * 0.3).to(torch.float16)
    Bs = [(torch.randn(Hs, Kc) * 0.3).to(torch.float16) for _ in range(4)]
    biases = [torch.randn(Hs) * 0.1 for _ in range(4)]
    cell0 = torch.randn(M, Hs) * 0.5
    c_ref, h_ref = fl.reference(A, Bs, biases, cell0)
    out.update(flstm8_A=T(A), flstm8_W=T(torch.cat(Bs, 0)), flstm8_bias=T(torch.cat(biases, 0)), flstm8_c0=T(cell0),
               flstm8_c_ref=T(c_ref), flstm8_h_ref=T(h_ref))
    # ---- fp8 down-projection: the base fp8 GEMM of rdna_fp8_preshuffle_gemm.py with N = R, K = H
    # (export_fp8_factored_lstm.py:161-181); reference as fly/test_rotary.py builds its GEMM (:88-90) --
    torch.manual_seed(7)
    hx = torch.randn(48, 768) * 0.3
    dn = torch.randn(768, 128) / 768 ** 0.5            # [K, N] as the fly helpers take it
    h8, sh = fg.fp8_quantize_per_token(hx)
    d8, sd = fg.fp8_quantize_per_channel(dn)
    dp = (h8.float() * sh[:, None]) @ (d8.float() * sd[None, :])
    out.update(dp8_A=T(h8.view(torch.uint8)), dp8_sa=T(sh), dp8_B_kn=T(d8.view(torch.uint8)), dp8_sb=T(sd),
               dp8_expected=T(dp).astype(np.float16))

    path = os.path.join(HERE, "reference_tests.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, os.path.getsize(path), "bytes;", len(out), "arrays")


if __name__ == "__main__":
    main()
