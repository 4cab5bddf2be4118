"""Tensor boundary specs: ``Tile`` and ``Layout``.

API-compatible with the reference's ``pyptx.specs`` (pyptx/specs.py:46-62 for
``Layout``, :69-209 for ``Tile``, :363-378 for ``unify_envs``).  A ``Tile``
states the shape (concrete ints or symbolic names), element type, memory layout
and optional TMA box of one kernel argument; the launch path uses it to
validate inputs, bind symbolic dims and size outputs.
"""
from __future__ import annotations

from enum import Enum
from typing import Iterable, Union

from .types import PtxType


class Layout(Enum):
    """How a tile is laid out / fetched.  ``TMA_*`` name the TMA swizzle width."""

    ROW = "row"
    COL = "col"
    TMA_128B = "tma_128b"
    TMA_64B = "tma_64b"
    TMA_32B = "tma_32b"
    INTERLEAVED = "interleaved"


Dim = Union[int, str]

_TORCH_NAMES = {
    "f16": "float16", "bf16": "bfloat16", "f32": "float32", "f64": "float64",
    "s8": "int8", "s16": "int16", "s32": "int32", "s64": "int64",
    "u8": "uint8", "u16": "uint16", "u32": "uint32", "u64": "uint64",
    "b8": "uint8", "b16": "uint16", "b32": "uint32", "b64": "uint64",
    "pred": "bool_",
}


class Tile:
    """Spec of one tensor argument: ``Tile("M", 64, bf16, Layout.ROW)``.

    Positional arguments are dims (``int`` or ``str``), at most one dtype and at
    most one layout, in any order after the dims; ``dtype`` / ``layout`` /
    ``tma_box`` / ``tma_rank`` / ``tma_padding`` may also be keywords.
    Instances are immutable and hashable.
    """

    __slots__ = ("shape", "dtype", "layout", "tma_box", "tma_rank", "tma_padding")

    def __init__(self, *dims_and_dtype, dtype: PtxType | None = None,
                 layout: Layout = Layout.ROW, tma_box: tuple | None = None,
                 tma_rank: int = 2, tma_padding: bool = False) -> None:
        shape: list[Dim] = []
        for a in dims_and_dtype:
            if isinstance(a, PtxType):
                if dtype is not None and dtype is not a:
                    raise ValueError(f"Tile got two dtypes: {dtype} and {a}")
                dtype = a
            elif isinstance(a, Layout):
                layout = a
            elif isinstance(a, bool) or not isinstance(a, (int, str)):
                raise TypeError(
                    f"Tile arg must be int, str, PtxType, or Layout; got {type(a).__name__}: {a!r}")
            else:
                shape.append(a)
        if dtype is None:
            raise ValueError("Tile requires a dtype (e.g. bf16, f32)")
        if not shape:
            raise ValueError("Tile requires at least one dimension")
        set_ = object.__setattr__
        set_(self, "shape", tuple(shape))
        set_(self, "dtype", dtype)
        set_(self, "layout", layout)
        set_(self, "tma_box", None if tma_box is None else tuple(tma_box))
        set_(self, "tma_rank", tma_rank)
        set_(self, "tma_padding", tma_padding)

    def __setattr__(self, key, value):
        raise AttributeError("Tile is immutable")

    def _key(self):
        return (self.shape, self.dtype, self.layout, self.tma_box, self.tma_rank, self.tma_padding)

    def __eq__(self, other):
        return isinstance(other, Tile) and other._key() == self._key()

    def __hash__(self):
        return hash(self._key())

    def __repr__(self) -> str:
        dims = ", ".join(repr(d) for d in self.shape)
        return f"Tile({dims}, {self.dtype}, {self.layout.name})"

    @property
    def rank(self) -> int:
        return len(self.shape)

    @property
    def symbolic_dims(self) -> tuple[str, ...]:
        return tuple(d for d in self.shape if isinstance(d, str))

    def resolve_shape(self, env: dict[str, int]) -> tuple[int, ...]:
        """Concrete shape with symbolic dims replaced from ``env``."""
        out = []
        for d in self.shape:
            if isinstance(d, str):
                if d not in env:
                    raise KeyError(
                        f"Tile shape variable {d!r} not bound in env. Available: {sorted(env)}")
                d = env[d]
            out.append(int(d))
        return tuple(out)

    def matches(self, array_shape: tuple[int, ...], array_dtype_name: str) -> bool:
        """Rank, dtype name (PTX or numpy/torch spelling) and static dims agree."""
        if len(array_shape) != self.rank:
            return False
        if array_dtype_name not in (self.dtype.name, _TORCH_NAMES.get(self.dtype.name, self.dtype.name)):
            return False
        return all(isinstance(s, str) or s == a for s, a in zip(self.shape, array_shape))

    def extract_env(self, array_shape: tuple[int, ...]) -> dict[str, int]:
        """Bind symbolic dims from a concrete shape; static dims must agree."""
        if len(array_shape) != self.rank:
            raise ValueError(
                f"Tile rank mismatch: tile has {self.rank} dims, array has {len(array_shape)} dims")
        env: dict[str, int] = {}
        for s, a in zip(self.shape, array_shape):
            if isinstance(s, str):
                env[s] = int(a)
            elif s != a:
                raise ValueError(f"Tile dim mismatch: expected {s}, got {a}")
        return env

    def nbytes(self, env: dict[str, int] | None = None) -> int:
        n = self.dtype.bytes
        for d in self.resolve_shape(env or {}):
            n *= d
        return n


def unify_envs(envs: Iterable[dict[str, int]]) -> dict[str, int]:
    """Merge per-tensor dim bindings; the same name must bind to one value."""
    merged: dict[str, int] = {}
    for env in envs:
        for k, v in env.items():
            if merged.setdefault(k, v) != v:
                raise ValueError(f"Tile dim {k!r} has conflicting values: {merged[k]} vs {v}")
    return merged
