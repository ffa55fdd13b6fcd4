"""Seeded inputs of the pure-CUDA-kernel parity cases, shared by the capture script (which
runs the reference's kernels on a GPU) and by the tests (which run this library and the CPU
oracle on the same inputs). numpy's PCG64 stream is stable across versions and platforms.
"""
import numpy as np


def _rng(tag):
    return np.random.default_rng(abs(hash_str(tag)) % (2 ** 32))


def hash_str(s):
    h = 2166136261
    for ch in s.encode():
        h = ((h ^ ch) * 16777619) & 0xFFFFFFFF
    return h


def f16(rng, *shape, scale=1.0):
    return (rng.standard_normal(shape) * scale).astype(np.float32).astype(np.float16)


def rotary_tables(seq_len, width=32, head_dim=64, theta=10000.0):
    inv = 1.0 / theta ** (np.arange(0, head_dim, 2, dtype=np.float64)[:width] / head_dim)
    fr = np.outer(np.arange(seq_len, dtype=np.float64), inv)
    return np.sin(fr).astype(np.float32), np.cos(fr).astype(np.float32)


ALPHA, EPS = 2.0, 1e-5
RMS_SHAPES = [(48, 512), (16, 768), (8, 1024), (12, 256), (10, 320)]
QUANT_SHAPES = [(32, 512), (8, 2048), (5, 100)]


def rmsnorm_case(n, h):
    r = _rng(f"rmsnorm{n}x{h}")
    return dict(x=f16(r, n, h), res=f16(r, n, h), w=f16(r, h))


def rmsnorm_quant_case(n, h):
    r = _rng(f"rmsq{n}x{h}")
    return dict(x=f16(r, n, h), w=f16(r, h),
                res_i8=r.integers(-127, 128, (n, h), dtype=np.int8),
                res_f8=r.integers(0, 256, (n, h), dtype=np.uint8),
                scale=(r.random(n) * 0.02 + 0.001).astype(np.float32))


def quant_case(n, h):
    return dict(x=f16(_rng(f"quant{n}x{h}"), n, h, scale=3.0))


def rotary_case():
    r = _rng("rotary")
    sin, cos = rotary_tables(24)
    return dict(qkv=f16(r, 2, 24, 3, 8, 64), sin=sin, cos=cos)


def silu_case():
    return dict(x=f16(_rng("silu"), 32, 2 * 128, scale=2.0))


def flstm_case():
    r = _rng("flstm")
    return dict(scratch=f16(r, 32, 4 * 96), ih=f16(r, 32, 4 * 96), cell=f16(r, 32, 96))


def dequant_case():
    r = _rng("dequant")
    return dict(i8=r.integers(-127, 128, (5, 6, 64), dtype=np.int8),
                f8=r.integers(0, 256, (5, 6, 64), dtype=np.uint8), scale=0.013)
