"""B200 (sm_100a) kernels for RapidLLM's qwen3_5 hybrid-attention hot path.

The product is librl_b200.so (C ABI in include/rl_b200.h).  This package is the
thin host-side mirror used by tests and the bench: `ops` has the reference's
operator names (attn_decode, delta_recurrent_step, conv1d_update, ...) over
torch CUDA tensors; `cache.HybridCache` is the device-side DualCache with the
layer_types[] dispatch.
"""
from . import _lib  # noqa: F401
from ._lib import RlError  # noqa: F401

__all__ = ["ops", "cache", "RlError"]
