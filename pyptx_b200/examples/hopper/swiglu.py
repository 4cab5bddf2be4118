"""``examples.hopper.swiglu`` import path of the reference (examples/hopper/swiglu.py), kept so that
callers written against it resolve; the kernel behind it is the sm_100a one and any
other ``arch`` is rejected."""
from ..blackwell.swiglu import build_fused_silu_mul  # noqa: F401

__all__ = ["build_fused_silu_mul"]
