"""fluke_b200 -- host-side Python mirror of the fluke C ABI on sm_100a.

The product is lib/libfluke.so (C host code in src/ + one CUDA translation unit in
fluke_b200/csrc/). This package only loads it and wraps its entry points for torch tensors:
`fluke_b200.lib` is the ctypes binding, `fluke_b200.ops` the tensor-level operator interface
(same names and argument meaning as the C functions), `fluke_b200.lstm` the factored-LSTM
layer/stack driver and `fluke_b200.prep` the weight/input preparation the reference's tests
do in torch (quantisers, rotary tables).
"""
from . import lib  # noqa: F401

__all__ = ["lib", "ops", "lstm", "prep"]
