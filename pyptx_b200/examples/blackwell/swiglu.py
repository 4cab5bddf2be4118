"""SwiGLU gate for B200: ``out = silu(gate) * up`` in f32.

Drop-in for ``build_fused_silu_mul(M, F, *, rows_per_cta=None)``
(examples/blackwell/swiglu.py:24-35; body examples/hopper/swiglu.py:48-156).
"""
from __future__ import annotations

from ..._ids import K_SWIGLU
from ...kernel import NativeKernel
from ...specs import Tile
from ...types import PtxType, f32
from .layer_norm import _pick_rows_per_cta
from .rms_norm import _check_row_shape, _out_flags


def build_fused_silu_mul(M: int, F: int, *, rows_per_cta: int | None = None,
                         arch: str = "sm_100a", out_dtype: PtxType = f32) -> NativeKernel:
    """Kernel ``k(gate[M,F], up[M,F]) -> out[M,F]`` (all f32).

    ``rows_per_cta`` is accepted for compatibility; the native kernel treats the
    operands as one flat array.
    """
    _check_row_shape(M, F, "fused_silu_mul")
    if rows_per_cta is None:
        rows_per_cta = _pick_rows_per_cta(M)
    assert rows_per_cta >= 1, "rows_per_cta must be at least 1"
    return NativeKernel(
        "fused_silu_mul", K_SWIGLU, (M, F),
        in_specs=(Tile(M, F, f32), Tile(M, F, f32)),
        out_specs=(Tile(M, F, out_dtype),),
        flags=_out_flags(out_dtype), arch=arch, meta={"rows_per_cta": rows_per_cta},
    )


def swiglu_bytes(M: int, F: int) -> int:
    """benchmarks/bench_blackwell_kernels.py:114."""
    return 3 * M * F * 4
