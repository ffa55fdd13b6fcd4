"""Run the REFERENCE's own pure-CUDA kernels (oracle/_ref/libfluke_ref_cuda.so: the reference's
src/nn_cuda.c + src/nn_kernel_cuda.h compiled unmodified for sm_100a by oracle/build_oracle.py)
on the seeded cases of tests/golden/cases.py and store their outputs.

    python tests/golden/capture_reference_cuda_kernels.py [out.npz]     # needs a GPU

The committed result, tests/golden/reference_cuda_kernels.npz, was produced by this script on
a B200. It pins the CPU oracle (exact where the kernel is IEEE-only) and this library's kernels
(bit-for-bit) without needing the reference at test time.
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, HERE)
import cases  # noqa: E402
from oracle import ref  # noqa: E402


def main():
    out_path = sys.argv[1] if len(sys.argv) > 1 else os.path.join(HERE, "reference_cuda_kernels.npz")
    R = ref.cuda()
    assert R is not None, "oracle/_ref/libfluke_ref_cuda.so missing: run oracle/build_oracle.py where the reference is mounted"
    dev = "cuda"
    D = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    out = {}
    for (n, h) in cases.RMS_SHAPES:
        c = cases.rmsnorm_case(n, h)
        x, res, w = D(c["x"]), D(c["res"]), D(c["w"])
        o = torch.empty_like(x)
        R.fluke_rmsnorm_gpu(x.data_ptr(), res.data_ptr(), w.data_ptr(), o.data_ptr(), n, h, cases.ALPHA, cases.EPS)
        out[f"rmsnorm_{n}x{h}"] = o.cpu().numpy()
        c = cases.rmsnorm_quant_case(n, h)
        x, w = D(c["x"]), D(c["w"])
        r8, s8 = D(c["res_i8"]), D(c["scale"])
        R.fluke_rmsnorm_quant_int8_gpu(x.data_ptr(), w.data_ptr(), r8.data_ptr(), s8.data_ptr(), n, h, cases.ALPHA, cases.EPS)
        out[f"rmsq_i8_{n}x{h}"], out[f"rmsq_i8_scale_{n}x{h}"] = r8.cpu().numpy(), s8.cpu().numpy()
        rf, sf = D(c["res_f8"]), D(c["scale"])
        R.fluke_rmsnorm_quant_fp8_gpu(x.data_ptr(), w.data_ptr(), rf.data_ptr(), sf.data_ptr(), n, h, cases.ALPHA, cases.EPS)
        out[f"rmsq_f8_{n}x{h}"], out[f"rmsq_f8_scale_{n}x{h}"] = rf.cpu().numpy(), sf.cpu().numpy()
    for (n, h) in cases.QUANT_SHAPES:
        x = D(cases.quant_case(n, h)["x"])
        q = torch.empty(n, h, dtype=torch.int8, device=dev); s = torch.empty(n, dtype=torch.float32, device=dev)
        R.fluke_quant_int8_gpu(x.data_ptr(), q.data_ptr(), s.data_ptr(), n, h)
        f = torch.empty(n, h, dtype=torch.uint8, device=dev); fs = torch.empty(n, dtype=torch.float32, device=dev)
        R.fluke_quant_fp8_gpu(x.data_ptr(), f.data_ptr(), fs.data_ptr(), n, h)
        out[f"quant_i8_{n}x{h}"], out[f"quant_i8_scale_{n}x{h}"] = q.cpu().numpy(), s.cpu().numpy()
        out[f"quant_f8_{n}x{h}"], out[f"quant_f8_scale_{n}x{h}"] = f.cpu().numpy(), fs.cpu().numpy()
    c = cases.rotary_case()
    qkv, sin, cos = D(c["qkv"]), D(c["sin"]), D(c["cos"])
    for ch in (0, 1):
        R.fluke_rotary_emb_gpu(qkv.data_ptr() + ch * qkv.stride(2) * 2, sin.data_ptr(), cos.data_ptr(),
                               2, 24, 8, 64, 32, qkv.stride(0), qkv.stride(1), qkv.stride(3))
    out["rotary"] = qkv.cpu().numpy()
    x = D(cases.silu_case()["x"])
    o = torch.empty(32, 128, dtype=torch.float16, device=dev)
    R.fluke_silu_mul_gpu(x.data_ptr(), o.data_ptr(), 32, 128)
    out["silu"] = o.cpu().numpy()
    c = cases.flstm_case()
    sc, ih, cell = D(c["scratch"]), D(c["ih"]), D(c["cell"])
    hh = torch.empty_like(cell)
    R.fluke_flstm_step_gpu(sc.data_ptr(), ih.data_ptr(), cell.data_ptr(), hh.data_ptr(), 32, 96)
    out["flstm_cell"], out["flstm_hh"] = cell.cpu().numpy(), hh.cpu().numpy()
    c = cases.dequant_case()
    i8, f8 = D(c["i8"]), D(c["f8"])
    o1 = torch.empty(6, 5, 64, dtype=torch.float16, device=dev); o2 = torch.empty_like(o1)
    R.fluke_dequant_int8_transpose_gpu(i8.data_ptr(), o1.data_ptr(), 5, 6, 64, c["scale"])
    R.fluke_dequant_fp8_transpose_gpu(f8.data_ptr(), o2.data_ptr(), 5, 6, 64, c["scale"])
    torch.cuda.synchronize()
    out["dequant_i8"], out["dequant_f8"] = o1.cpu().numpy(), o2.cpu().numpy()
    np.savez_compressed(out_path, **out)
    print("wrote", out_path, os.path.getsize(out_path), "bytes")


if __name__ == "__main__":
    main()
