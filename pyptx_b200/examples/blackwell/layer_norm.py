"""LayerNorm for B200: ``y = (x - mean) * rsqrt(var + eps) * w + b`` in f32.

Drop-in for ``build_layer_norm(B, N, *, eps=1e-5, rows_per_cta=None)``
(examples/blackwell/layer_norm.py:24-35; body examples/hopper/layer_norm.py:57-225).
"""
from __future__ import annotations

from ..._ids import K_LAYER_NORM
from ...kernel import NativeKernel
from ...specs import Tile
from ...types import PtxType, f32
from .rms_norm import _check_row_shape, _out_flags


def _pick_rows_per_cta(B: int) -> int:
    """The reference's heuristic (examples/blackwell/layer_norm.py:24-29); advisory here."""
    if B <= 64:
        return 8
    if B <= 256:
        return 4
    return 1


def build_layer_norm(B: int, N: int, *, eps: float = 1e-5, rows_per_cta: int | None = None,
                     arch: str = "sm_100a", out_dtype: PtxType = f32) -> NativeKernel:
    """Kernel ``k(x[B,N], w[N], b[N]) -> y[B,N]`` (all f32).

    ``rows_per_cta`` is accepted for compatibility and validated, but the native
    kernel always maps one CTA to one row at a time.
    """
    _check_row_shape(B, N, "layer_norm")
    if rows_per_cta is None:
        rows_per_cta = _pick_rows_per_cta(B)
    assert rows_per_cta >= 1, "rows_per_cta must be at least 1"
    return NativeKernel(
        "layer_norm", K_LAYER_NORM, (B, N),
        in_specs=(Tile(B, N, f32), Tile(N, f32), Tile(N, f32)),
        out_specs=(Tile(B, N, out_dtype),),
        fparams=(eps,), flags=_out_flags(out_dtype), arch=arch, meta={"eps": eps, "rows_per_cta": rows_per_cta},
    )


def layer_norm_bytes(B: int, N: int) -> int:
    """benchmarks/bench_blackwell_kernels.py:91."""
    return 2 * B * N * 4 + 2 * N * 4
