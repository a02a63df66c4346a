"""B200-native FlashAttention-3 backward behind the shaobo_fa3_bwd_v2 C ABI.

The product is the shared library ``libfa3bwd_b200.so`` (CUDA, sm_100a) built
from ``csrc/``.  This package only binds it (``capi``) and offers a thin
tensor-level helper (``ops``) that owns no math: it allocates outputs and the
workspace with torch and calls the C entry points.  Nothing here falls back to
a CPU or PyTorch implementation; if the library is missing or no CUDA device is
present the calls raise.
"""
from . import capi  # noqa: F401

__all__ = ["capi"]
