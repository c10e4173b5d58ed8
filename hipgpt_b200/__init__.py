"""B200 (sm_100a) attention-forward path of HipGPT behind the reference's launcher API.

The product is libhipgpt_attn.so (hipgpt_b200/csrc, C ABI in include/hipgpt_attn.h); this
package builds it, binds it with ctypes and mirrors the reference's launcher names for tests
and benchmarks.  Import of the launchers needs torch; the library itself does not.
"""
from . import build as build_lib  # noqa: F401
from . import _capi  # noqa: F401

__all__ = ["build_lib", "_capi"]
