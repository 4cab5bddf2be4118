"""``examples.hopper.rms_norm`` import path of the reference (examples/hopper/rms_norm.py), kept so that
callers written against it resolve; the kernel behind it is the sm_100a one and any
other ``arch`` is rejected."""
from ..blackwell.rms_norm import build_rms_norm  # noqa: F401

__all__ = ["build_rms_norm"]
