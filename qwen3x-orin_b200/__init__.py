"""q3x-b200: the fused per-layer elementwise / normalisation operators of Qwen3.6-27B for B200.

The product is the native library ``libq3x_b200.so`` (hand-written sm_100a CUDA behind the C ABI of
``include/q3x_b200.h``) and ``libq3x_b200_host.so`` (the C++17 mirror of the reference operator API).
This Python package only loads them for the tests and the bench: ``capi`` binds every C entry point
with ctypes and passes raw device pointers (torch is used for device memory and streams only).

There is no CPU fallback: loading fails loudly when the CUDA library has not been built.
The directory name contains a dash, so import it with
``importlib.import_module("qwen3x-orin_b200")``.
"""
from . import capi  # noqa: F401
from .capi import lib, load  # noqa: F401

__all__ = ["capi", "lib", "load"]
