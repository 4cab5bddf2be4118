"""Row softmax for B200 in f32.

Drop-in for ``build_softmax(B, N, *, arch)`` (examples/hopper/softmax.py:49-182);
the reference has no Blackwell wrapper module for it, only the ``arch=`` parameter.
"""
from __future__ import annotations

from ..._ids import K_SOFTMAX
from ...kernel import NativeKernel
from ...specs import Tile
from ...types import PtxType, f32
from .rms_norm import _check_row_shape, _out_flags


def build_softmax(B: int, N: int, *, arch: str = "sm_100a", out_dtype: PtxType = f32) -> NativeKernel:
    """Kernel ``k(x[B,N] f32) -> y[B,N] f32`` with ``y = softmax(x, -1)``."""
    _check_row_shape(B, N, "softmax")
    return NativeKernel(
        "softmax", K_SOFTMAX, (B, N),
        in_specs=(Tile(B, N, f32),),
        out_specs=(Tile(B, N, out_dtype),),
        flags=_out_flags(out_dtype), arch=arch,
    )


def softmax_bytes(B: int, N: int) -> int:
    """benchmarks/bench_final.py:108."""
    return 2 * B * N * 4
