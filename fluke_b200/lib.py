"""ctypes binding of lib/libfluke.so -- the same C ABI slorado links and the reference's
fluke_lib.py loads (reference: fluke_lib.py:19-62 for the ten void functions,
fly/common.py:96-107 for the fused fp8 signatures, include/fluke/fluke.h for the rest).

There is no fallback: if the library cannot be built or loaded, `load()` raises.
"""
import ctypes
import os
import subprocess

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
SO_PATH = os.path.join(ROOT, "lib", "libfluke.so")

P, I, F, Z = ctypes.c_void_p, ctypes.c_int, ctypes.c_float, ctypes.c_size_t


class fluke_dims_t(ctypes.Structure):
    _fields_ = [("d_model", I), ("dim_feedforward", I), ("nhead", I), ("head_dim", I), ("max_seq", I)]


class fluke_flstm_layer_t(ctypes.Structure):
    _fields_ = [
        ("T", I), ("B", I), ("H", I), ("R", I), ("reverse", I),
        ("x_i8", P), ("x_scale", P),
        ("dn_ih_i8", P), ("dn_ih_scale", P), ("dn_hh_i8", P), ("dn_hh_scale", P),
        ("w_up_f16", P), ("bias_f32", P),
        ("c_f32", P), ("h_i8", P), ("h_out_i8", P),
        ("workspace", P), ("workspace_bytes", Z),
    ]


class fluke_flstm_weights_t(ctypes.Structure):
    _fields_ = [("dn_ih_i8", P), ("dn_ih_scale", P), ("dn_hh_i8", P), ("dn_hh_scale", P),
                ("w_up_f16", P), ("bias_f32", P), ("reverse", I)]


# name -> (restype, argtypes). The first ten are exactly fluke_lib._SIGNATURES of the reference.
VOID_SIGNATURES = {
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

SIGNATURES = {
    # CPU trio
    "fluke_rotary_emb_cpu": (None, [P, P, P, I, I, I, I, I, I, I, I, I]),
    "fluke_rmsnorm_cpu": (None, [P, P, P, P, I, I, F, F, I]),
    "fluke_flstm_step_cpu": (None, [P, P, P, P, I, I, I]),
    "get_fluke_log_level": (I, []),
    "set_fluke_log_level": (None, [I]),
    # fused int8
    "fluke_int8_select": (P, [I, fluke_dims_t]),
    "fluke_int8_dims": (fluke_dims_t, [P]),
    "fluke_qkv_rotary_i8_gpu": (I, [P, P, P, P, P, P, P, P, I, I]),
    "fluke_gated_mlp_i8_gpu": (I, [P, P, P, P, P, P, P, P, I]),
    # fused fp8
    "fluke_fp8_select": (P, [I, fluke_dims_t]),
    "fluke_qkv_rotary_fp8_gpu": (I, [P, P, P, P, P, P, P, P, I, I]),
    "fluke_gated_mlp_fp8_gpu": (I, [P, P, P, P, P, P, P, P, I]),
    # additive
    "fluke_set_stream": (None, [P]),
    "fluke_set_lstm_persistent": (None, [I]),
    "fluke_get_stream": (P, []),
    "fluke_last_error": (ctypes.c_char_p, []),
    "fluke_gemm_i8_gpu": (I, [P, P, P, P, F, P, I, I, I]),
    "fluke_gemm_i8_s32_gpu": (I, [P, P, P, I, I, I]),
    "fluke_gemm_fp8_gpu": (I, [P, P, P, P, P, I, I, I]),
    "fluke_fp8_unshuffle_gpu": (I, [P, P, I, I]),
    "fluke_qkv_rotary_fp8_plain_gpu": (I, [P, P, P, P, P, P, P, P, I, I]),
    "fluke_gated_mlp_fp8_plain_gpu": (I, [P, P, P, P, P, P, P, P, I]),
    "fluke_down_proj_i8_gpu": (I, [P, I, P, P, P, P, I, I, I]),
    "fluke_factored_lstm_step_i8_gpu": (I, [P, P, P, P, P, P, P, P, P, P, P, I, I, I]),
    "fluke_down_proj_fp8_gpu": (I, [P, I, P, P, P, P, I, I, I]),
    "fluke_down_proj_i8_stream_gpu": (I, [P, I, P, P, P, P, I, I, I, P]),
    "fluke_factored_lstm_step_i8_stream_gpu": (I, [P, P, P, P, P, P, P, P, P, P, P, I, I, I, P]),
    "fluke_factored_lstm_step_fp8_gpu": (I, [P, P, P, P, P, P, P, P, P, P, P, I, I, I]),
    "fluke_factored_lstm_layer_workspace": (Z, [I, I, I, I]),
    "fluke_factored_lstm_layer_i8_gpu": (I, [ctypes.POINTER(fluke_flstm_layer_t)]),
    "fluke_factored_lstm_layer_phases_gpu": (I, [ctypes.POINTER(fluke_flstm_layer_t), I]),
    "fluke_factored_lstm_layer_i8_noalloc_gpu": (I, [ctypes.POINTER(fluke_flstm_layer_t)]),
    "fluke_factored_lstm_stack_i8_gpu": (I, [ctypes.POINTER(fluke_flstm_weights_t), I, I, I, I, I, P, P, P, P, P, P, P, Z]),
    "fluke_flstm_stream_create": (P, [ctypes.POINTER(fluke_flstm_weights_t), I, I, I, I, I, I, I]),
    "fluke_flstm_stream_submit": (I, [P, P, P, P, I]),
    "fluke_flstm_stream_flush": (I, [P]),
    "fluke_flstm_stream_drain": (I, [P]),
    "fluke_flstm_stream_destroy": (None, [P]),
    "fluke_fp8_prepare_weight": (I, [P, I, I]),
    "fluke_fp8_release_weight": (I, [P]),
    # internal status word (bounded device waits)
    "fluke_sm100_read_status": (I, [ctypes.POINTER(ctypes.c_uint), I]),
    "fluke_sm100_copy_rows_async": (I, [P, ctypes.c_size_t, P, ctypes.c_size_t, ctypes.c_size_t, ctypes.c_size_t, I, P]),
    "fluke_sm100_lstm_last_form": (I, []),
    "fluke_sm100_set_lstm_wide": (None, [I]),
    "fluke_sm100_lstm_cluster_capacity": (I, [I]),
}
for _n, _a in VOID_SIGNATURES.items():
    SIGNATURES[_n] = (None, _a)


PROBE_PATH = os.path.join(ROOT, "lib", "libfluke_probe.so")


def build(verbose=False):
    """`make shared probe waitprobe cuda=1` at the repository root (nvcc cross-compiles sm_100a
    without a GPU): the library, the benchmark's issue-rate probe and the tests' wait probe."""
    cmd = ["make", "shared", "probe", "waitprobe", "cuda=1"]
    res = subprocess.run(cmd, cwd=ROOT, stdout=subprocess.PIPE, stderr=subprocess.STDOUT, text=True)
    if verbose or res.returncode != 0:
        print(res.stdout)
    if res.returncode != 0:
        raise RuntimeError("building lib/libfluke.so failed (see output above)")
    return SO_PATH


_LIB = None


def load(rebuild=False):
    """Return the CDLL with restype/argtypes set for every exported entry point."""
    global _LIB
    if _LIB is not None and not rebuild:
        return _LIB
    if rebuild or not os.path.isfile(SO_PATH):
        build()
    lib = ctypes.CDLL(SO_PATH)
    for name, (restype, argtypes) in SIGNATURES.items():
        fn = getattr(lib, name)  # AttributeError = a symbol the header declares is missing
        fn.restype = restype
        fn.argtypes = argtypes
    _LIB = lib
    return lib


_PROBE = None


def load_probe():
    """The tcgen05 issue-rate probe and the in-GPU clock sampler the benchmark uses
    (lib/libfluke_probe.so; not part of libfluke)."""
    global _PROBE
    if _PROBE is None:
        if not os.path.isfile(PROBE_PATH):
            build()
        _PROBE = ctypes.CDLL(PROBE_PATH)
        _PROBE.fluke_sm100_mma_peak.restype = I
        _PROBE.fluke_sm100_mma_peak.argtypes = [I, I, I, I, P, I, P]
        _PROBE.fluke_sm100_clock_samples.restype = I
        _PROBE.fluke_sm100_clock_samples.argtypes = [P, I, I, P]
    return _PROBE


def read_status(reset=True):
    """Device status word: 0, or 1 | (site << 8) after a device-side wait gave up."""
    v = ctypes.c_uint(0)
    rc = load().fluke_sm100_read_status(ctypes.byref(v), 1 if reset else 0)
    if rc != 0:
        raise RuntimeError(f"fluke_sm100_read_status failed with CUDA error {rc}")
    return v.value
