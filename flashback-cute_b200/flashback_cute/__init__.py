"""B200 (sm_100a) drop-in for the `flashback_cute` package: twice-differentiable softmax
attention whose second-order step runs as hand-written CUDA kernels behind a C ABI."""

from .interface import (  # noqa: F401
    flashback_attn_func,
    flashback_attn_varlen_func,
    flashback_attn_jvp,
    flashback_attn_hvp,
)

__all__ = ["flashback_attn_func", "flashback_attn_varlen_func", "flashback_attn_jvp", "flashback_attn_hvp"]
