"""Backward kernels of the row ops for B200, for use with ``differentiable_kernel``.

The reference has the autograd hook (pyptx/torch_support.py:446-519) but no backward kernels;
these are the halves that pair with ``build_rms_norm`` / ``build_layer_norm`` /
``build_fused_silu_mul``::

    fwd, bwd = build_rms_norm(B, N), build_rms_norm_bwd(B, N)
    rms_norm = differentiable_kernel(fwd, bwd)      # backward gets (x, w, dy) and returns (dx, dw)

The two norm kernels keep per-CTA partial column sums in device scratch memory
(``kernel.scratch_bytes``), which the launch path allocates per call and discards.
"""
from __future__ import annotations

from ..._ids import K_LAYER_NORM_BWD, K_RMS_NORM_BWD, K_SWIGLU_BWD
from ...kernel import NativeKernel
from ...specs import Tile
from ...types import f32
from .rms_norm import _check_row_shape

MAX_NORM_BWD_COLS = 16384


def build_rms_norm_bwd(B: int, N: int, *, eps: float = 1e-6, arch: str = "sm_100a") -> NativeKernel:
    """Kernel ``k(x[B,N], w[N], dy[B,N]) -> (dx[B,N], dw[N])`` (all f32) for ``y = x*rsqrt(mean(x^2)+eps)*w``."""
    _check_row_shape(B, N, "rms_norm_bwd")
    assert N <= MAX_NORM_BWD_COLS, f"N={N} exceeds {MAX_NORM_BWD_COLS}"
    return NativeKernel(
        "rms_norm_bwd", K_RMS_NORM_BWD, (B, N),
        in_specs=(Tile(B, N, f32), Tile(N, f32), Tile(B, N, f32)),
        out_specs=(Tile(B, N, f32), Tile(N, f32)),
        fparams=(eps,), arch=arch, meta={"eps": eps},
    )


def build_layer_norm_bwd(B: int, N: int, *, eps: float = 1e-5, arch: str = "sm_100a") -> NativeKernel:
    """Kernel ``k(x[B,N], w[N], dy[B,N]) -> (dx[B,N], dw[N], db[N])`` (all f32)."""
    _check_row_shape(B, N, "layer_norm_bwd")
    assert N <= MAX_NORM_BWD_COLS, f"N={N} exceeds {MAX_NORM_BWD_COLS}"
    return NativeKernel(
        "layer_norm_bwd", K_LAYER_NORM_BWD, (B, N),
        in_specs=(Tile(B, N, f32), Tile(N, f32), Tile(B, N, f32)),
        out_specs=(Tile(B, N, f32), Tile(N, f32), Tile(N, f32)),
        fparams=(eps,), arch=arch, meta={"eps": eps},
    )


def build_fused_silu_mul_bwd(M: int, F: int, *, arch: str = "sm_100a") -> NativeKernel:
    """Kernel ``k(gate[M,F], up[M,F], dout[M,F]) -> (dgate[M,F], dup[M,F])`` (all f32)."""
    _check_row_shape(M, F, "fused_silu_mul_bwd")
    return NativeKernel(
        "fused_silu_mul_bwd", K_SWIGLU_BWD, (M, F),
        in_specs=(Tile(M, F, f32), Tile(M, F, f32), Tile(M, F, f32)),
        out_specs=(Tile(M, F, f32), Tile(M, F, f32)),
        arch=arch,
    )


def norm_bwd_bytes(B: int, N: int) -> int:
    """Algorithmic HBM bytes of one norm backward call: x and dy read, dx written, w once, dw (db) once."""
    return 3 * B * N * 4 + 3 * N * 4
