"""beantensor_b200 — sm_100a matmul subsystem behind BeanTensor's GPU operator boundary.

The implementation is libbtm.so (hand-written CUDA, C ABI in include/btm.h). This package is
the host-side mirror of the reference's operator interface for that path plus the in-tree
build recipe. Importing it does not load the library; the first operator call does, and fails
loudly if the library or a GPU is missing.
"""
from . import _lib, errors, synth  # noqa: F401

__all__ = ["_lib", "errors", "synth"]
