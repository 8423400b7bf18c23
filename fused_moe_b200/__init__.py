"""B200-native FP8 block-scale fused MoE layer (DeepSeek-V3 shape).

``from fused_moe_b200 import run`` gives the reference's ten-argument entry point
(``fused_moe_b200.kernel`` mirrors the reference's ``kernel.py``: ``run``, ``kernel``,
``custom_kernel``).  The CUDA library is loaded on first use and its absence is an error,
never a fallback.
"""
from .kernel import run, custom_kernel, route, MoEError  # noqa: F401

__all__ = ["run", "custom_kernel", "route", "MoEError"]
