"""RMSNorm for B200: ``y = x * rsqrt(mean(x^2, -1) + eps) * w`` in f32.

Drop-in for the reference entry point ``build_rms_norm(B, N, *, eps=1e-6)``
(examples/blackwell/rms_norm.py:26-27; kernel body examples/hopper/rms_norm.py:63-182).
"""
from __future__ import annotations

from ..._ids import K_RMS_NORM
from ...kernel import NativeKernel
from ...specs import Tile
from ...types import f32


def _check_row_shape(rows: int, cols: int, what: str) -> None:
    assert rows >= 1 and cols >= 1, f"{what}: shape ({rows}, {cols}) must be positive"
    assert cols % 4 == 0, f"{what}: N={cols} must be divisible by 4 (128-bit vector access)"


def build_rms_norm(B: int, N: int, *, eps: float = 1e-6, arch: str = "sm_100a") -> NativeKernel:
    """Kernel ``k(x[B,N] f32, w[N] f32) -> y[B,N] f32`` specialised for (B, N)."""
    _check_row_shape(B, N, "rms_norm")
    return NativeKernel(
        "rms_norm", K_RMS_NORM, (B, N),
        in_specs=(Tile(B, N, f32), Tile(N, f32)),
        out_specs=(Tile(B, N, f32),),
        fparams=(eps,), arch=arch, meta={"eps": eps},
    )


def rms_norm_bytes(B: int, N: int) -> int:
    """Algorithmic HBM bytes of one call, as the reference's benchmark counts them
    (benchmarks/bench_blackwell_kernels.py:67): x read + y written + w once."""
    return 2 * B * N * 4 + N * 4
