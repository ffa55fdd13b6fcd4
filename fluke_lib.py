"""Loader with the contract of the reference's fluke_lib.py (:53-62): `load()` returns the
ctypes handle of <root>/lib/libfluke.so with argtypes set for the ten `void fluke_*_gpu`
functions, building the library with `make shared cuda=1` when it is missing. The reference's
own fluke_lib.py also works unchanged at this repository root (same Makefile target and
variables, same output path); this one additionally types the fused and additive entry points.
"""
from fluke_b200.lib import SO_PATH as _SO, VOID_SIGNATURES as _SIGNATURES, build as _build, load  # noqa: F401
