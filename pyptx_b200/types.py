"""Scalar type tags used in :class:`pyptx_b200.specs.Tile` specs.

API-compatible with the reference's ``pyptx.types`` (pyptx/types.py:27-105):
the same singleton names (``bf16``, ``f32``, ``u32`` ...), the same ``name`` /
``bits`` / ``ptx`` attributes, equality by name, and ``from_name``.  Here the
tags only describe tensor element types at the kernel boundary; no PTX text is
generated from them.
"""
from __future__ import annotations


class PtxType:
    """An element type tag: ``name`` as PTX spells it, and its width in bits."""

    __slots__ = ("name", "bits")

    def __init__(self, name: str, bits: int) -> None:
        self.name = name
        self.bits = bits

    @property
    def ptx(self) -> str:
        return "." + self.name

    @property
    def bytes(self) -> int:
        return max(self.bits // 8, 1)

    def __repr__(self) -> str:
        return self.name

    def __hash__(self) -> int:
        return hash(self.name)

    def __eq__(self, other: object) -> bool:
        if isinstance(other, PtxType):
            return other.name == self.name
        return NotImplemented


_TABLE = (
    ("b8", 8), ("b16", 16), ("b32", 32), ("b64", 64), ("b128", 128),
    ("u8", 8), ("u16", 16), ("u32", 32), ("u64", 64),
    ("s8", 8), ("s16", 16), ("s32", 32), ("s64", 64),
    ("f16", 16), ("f16x2", 32), ("bf16", 16), ("bf16x2", 32),
    ("tf32", 32), ("f32", 32), ("f64", 64),
    ("e4m3", 8), ("e5m2", 8),
    ("pred", 1),
)
_BY_NAME: dict[str, PtxType] = {n: PtxType(n, w) for n, w in _TABLE}
globals().update(_BY_NAME)

# Names listed for static tooling; the objects are created from _TABLE above.
b8: PtxType; b16: PtxType; b32: PtxType; b64: PtxType; b128: PtxType
u8: PtxType; u16: PtxType; u32: PtxType; u64: PtxType
s8: PtxType; s16: PtxType; s32: PtxType; s64: PtxType
f16: PtxType; f16x2: PtxType; bf16: PtxType; bf16x2: PtxType
tf32: PtxType; f32: PtxType; f64: PtxType
e4m3: PtxType; e5m2: PtxType; pred: PtxType


def from_name(name: str) -> PtxType:
    """Look a type up by PTX name, with or without the leading dot."""
    t = _BY_NAME.get(name.lstrip("."))
    if t is None:
        raise ValueError(f"Unknown PTX type: {name!r}")
    return t
