"""Loaders of oracle/_ref/*.so: the reference's own sources compiled unmodified by
oracle/build_oracle.py (src/nn_cpu.c with gcc; src/nn_cuda.c + src/nn_kernel_cuda.h with nvcc
for sm_100a). They return None when the library was not built (the reference checkout only
exists on the build machine; the built .so files travel with the repository snapshot).
TEST INFRASTRUCTURE ONLY.
"""
import ctypes
import os

HERE = os.path.dirname(os.path.abspath(__file__))
P, I, F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float

_CPU_SIGS = {
    "fluke_rotary_emb_cpu": [P, P, P, I, I, I, I, I, I, I, I, I],
    "fluke_rmsnorm_cpu": [P, P, P, P, I, I, F, F, I],
    "fluke_flstm_step_cpu": [P, P, P, P, I, I, I],
}
_GPU_SIGS = {
    "fluke_rotary_emb_gpu": [P, P, P, I, I, I, I, I, I, I, I],
    "fluke_silu_mul_gpu": [P, P, I, I],
    "fluke_rmsnorm_gpu": [P, P, P, P, I, I, F, F],
    "fluke_quant_int8_gpu": [P, P, P, I, I],
    "fluke_quant_fp8_gpu": [P, P, P, I, I],
    "fluke_rmsnorm_quant_int8_gpu": [P, P, P, P, I, I, F, F],
    "fluke_rmsnorm_quant_fp8_gpu": [P, P, P, P, I, I, F, F],
    "fluke_dequant_fp8_transpose_gpu": [P, P, I, I, I, F],
    "fluke_dequant_int8_transpose_gpu": [P, P, I, I, I, F],
    "fluke_flstm_step_gpu": [P, P, P, P, I, I],
}


def _load(name, sigs):
    path = os.path.join(HERE, "_ref", name)
    if not os.path.isfile(path):
        return None
    lib = ctypes.CDLL(path)
    for fn, args in sigs.items():
        f = getattr(lib, fn)
        f.restype = None
        f.argtypes = args
    lib.set_fluke_log_level.argtypes = [I]
    lib.set_fluke_log_level(1)
    return lib


_cache = {}


def cpu():
    """The reference's CPU library (fluke_*_cpu), or None."""
    if "cpu" not in _cache:
        _cache["cpu"] = _load("libfluke_ref_cpu.so", _CPU_SIGS)
    return _cache["cpu"]


def cuda():
    """The reference's CUDA library (its ten fluke_*_gpu kernels, sm_100a build), or None."""
    if "cuda" not in _cache:
        _cache["cuda"] = _load("libfluke_ref_cuda.so", dict(_CPU_SIGS, **_GPU_SIGS))
    return _cache["cuda"]
