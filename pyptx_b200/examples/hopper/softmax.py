"""``examples.hopper.softmax`` import path of the reference (examples/hopper/softmax.py), kept so that
callers written against it resolve; the kernel behind it is the sm_100a one and any
other ``arch`` is rejected."""
from ..blackwell.softmax import build_softmax  # noqa: F401

__all__ = ["build_softmax"]
