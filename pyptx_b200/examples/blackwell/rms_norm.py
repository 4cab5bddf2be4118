"""RMSNorm for B200: ``y = x * rsqrt(mean(x^2, -1) + eps) * w`` in f32.

Drop-in for the reference entry point ``build_rms_norm(B, N, *, eps=1e-6)``
(examples/blackwell/rms_norm.py:26-27; kernel body examples/hopper/rms_norm.py:63-182).
"""
from __future__ import annotations

from ..._ids import F_OUT_BF16, K_RMS_NORM
from ...kernel import NativeKernel
from ...specs import Tile
from ...types import PtxType, bf16, f32


def _check_row_shape(rows: int, cols: int, what: str) -> None:
    assert rows >= 1 and cols >= 1, f"{what}: shape ({rows}, {cols}) must be positive"
    assert cols % 4 == 0, f"{what}: N={cols} must be divisible by 4 (128-bit vector access)"


def _out_flags(out_dtype: PtxType) -> int:
    assert out_dtype in (f32, bf16), f"out_dtype must be f32 or bf16, got {out_dtype}"
    return F_OUT_BF16 if out_dtype == bf16 else 0


def build_rms_norm(B: int, N: int, *, eps: float = 1e-6, arch: str = "sm_100a",
                   out_dtype: PtxType = f32) -> NativeKernel:
    """Kernel ``k(x[B,N] f32, w[N] f32) -> y[B,N]`` specialised for (B, N).

    ``out_dtype=bf16`` (an extension) rounds the result in the kernel, which fuses the cast that
    usually follows a normalisation and halves the bytes written."""
    _check_row_shape(B, N, "rms_norm")
    return NativeKernel(
        "rms_norm", K_RMS_NORM, (B, N),
        in_specs=(Tile(B, N, f32), Tile(N, f32)),
        out_specs=(Tile(B, N, out_dtype),),
        fparams=(eps,), flags=_out_flags(out_dtype), arch=arch, meta={"eps": eps},
    )


def rms_norm_bytes(B: int, N: int) -> int:
    """Algorithmic HBM bytes of one call, as the reference's benchmark counts them
    (benchmarks/bench_blackwell_kernels.py:67): x read + y written + w once."""
    return 2 * B * N * 4 + N * 4
