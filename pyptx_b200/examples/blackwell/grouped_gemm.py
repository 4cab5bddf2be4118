"""Grouped (MoE) bf16 GEMM for B200: ``C[g] = A[g] @ B[g]`` for ``g < G``.

Drop-in for ``build_grouped_gemm(G, M, N, K, *, arch="sm_100a")``
(examples/blackwell/grouped_gemm.py:61-289).  Operands are stacked along the
row axis: ``A[G*M, K]`` bf16, ``B_T[G*N, K]`` bf16 (each expert's weight
transposed to K-major, :302-303), result ``C[G*M, N]`` f32.
"""
from __future__ import annotations

from ..._ids import F_OUT_BF16, K_GROUPED_GEMM, K_GROUPED_GEMM_SWIGLU, K_GROUPED_GEMM_VARLEN
from ...kernel import NativeKernel
from ...specs import Layout, Tile
from ...types import PtxType, bf16, f32, s32

BM = 128
BK = 64


def _pick_bn(N: int) -> int:
    """Widest supported N tile that divides N (the reference uses min(N, 256), :51-58)."""
    for bn in (256, 128, 64):
        if N % bn == 0:
            return bn
    raise AssertionError(f"N={N} must be divisible by 64")


def build_grouped_gemm(G: int, M: int, N: int, K: int, *, arch: str = "sm_100a",
                       out_dtype: PtxType = f32) -> NativeKernel:
    """Kernel ``k(A[G*M,K] bf16, B_T[G*N,K] bf16) -> C[G*M,N]``."""
    assert arch.startswith("sm_100"), "Blackwell grouped GEMM is only implemented for sm_100*"
    assert G >= 1, "G must be at least 1"
    assert M % BM == 0, f"M={M} must be divisible by {BM}"
    assert K % BK == 0, f"K={K} must be divisible by {BK}"
    bn = _pick_bn(N)
    assert out_dtype in (f32, bf16), f"out_dtype must be f32 or bf16, got {out_dtype}"
    return NativeKernel(
        "grouped_gemm_bw", K_GROUPED_GEMM, (G, M, N, K),
        in_specs=(Tile(G * M, K, bf16, Layout.TMA_128B, tma_box=(BM, BK)),
                  Tile(G * N, K, bf16, Layout.TMA_128B, tma_box=(bn, BK))),
        out_specs=(Tile(G * M, N, out_dtype, Layout.ROW),),
        flags=F_OUT_BF16 if out_dtype == bf16 else 0, arch=arch,
        meta={"block_n": bn},
    )


def build_grouped_gemm_swiglu(G: int, M: int, F: int, K: int, *, arch: str = "sm_100a",
                              out_dtype: PtxType = f32) -> NativeKernel:
    """MoE up-projection with its activation fused into the GEMM epilogue (an extension; the
    reference runs ``build_grouped_gemm`` and then ``build_fused_silu_mul`` as two kernels).

    Kernel ``k(A[G*M,K] bf16, W_T[G*2F,K] bf16) -> out[G*M,F]`` with, per expert ``g``,
    ``out = silu(A[g] @ W_gate[g].T) * (A[g] @ W_up[g].T)``; ``W_T`` stacks each expert's ``F`` gate
    rows followed by its ``F`` up rows.  The ``[G*M, 2F]`` intermediate never reaches HBM.
    """
    assert arch.startswith("sm_100"), "Blackwell grouped GEMM is only implemented for sm_100*"
    assert G >= 1, "G must be at least 1"
    assert M % BM == 0, f"M={M} must be divisible by {BM}"
    assert F % 128 == 0, f"F={F} must be divisible by 128"
    assert K % BK == 0, f"K={K} must be divisible by {BK}"
    assert out_dtype in (f32, bf16), f"out_dtype must be f32 or bf16, got {out_dtype}"
    return NativeKernel(
        "grouped_gemm_swiglu_bw", K_GROUPED_GEMM_SWIGLU, (G, M, F, K),
        in_specs=(Tile(G * M, K, bf16, Layout.TMA_128B, tma_box=(BM, BK)),
                  Tile(G * 2 * F, K, bf16, Layout.TMA_128B, tma_box=(128, BK))),
        out_specs=(Tile(G * M, F, out_dtype, Layout.ROW),),
        flags=F_OUT_BF16 if out_dtype == bf16 else 0, arch=arch,
        meta={"block_f": 128},
    )


def build_grouped_gemm_varlen(G: int, M_total: int, N: int, K: int, *, arch: str = "sm_100a",
                              out_dtype: PtxType = f32) -> NativeKernel:
    """Grouped GEMM with a different row count per expert -- the follow-up the reference names
    (examples/hopper/grouped_gemm.py:15-17) but does not ship.

    Kernel ``k(A[M_total,K] bf16, B_T[G*N,K] bf16, offsets[G+1] int32) -> C[M_total,N]``: expert ``e``
    owns rows ``[offsets[e], offsets[e+1])`` of ``A`` and ``C`` and multiplies them by its own
    ``B_T[e*N:(e+1)*N]``.  ``offsets`` lives on the device (it usually comes out of the router's
    scan), starts at 0, is non-decreasing in multiples of 128 and ends at or below ``M_total``;
    rows at or beyond ``offsets[G]`` are left unwritten.  ``M_total`` is the static capacity, so
    one kernel object (and one CUDA graph) serves every routing outcome.
    """
    assert arch.startswith("sm_100"), "Blackwell grouped GEMM is only implemented for sm_100*"
    assert G >= 1, "G must be at least 1"
    assert M_total % BM == 0, f"M_total={M_total} must be divisible by {BM}"
    assert K % BK == 0, f"K={K} must be divisible by {BK}"
    bn = _pick_bn(N)
    assert out_dtype in (f32, bf16), f"out_dtype must be f32 or bf16, got {out_dtype}"
    return NativeKernel(
        "grouped_gemm_varlen_bw", K_GROUPED_GEMM_VARLEN, (G, M_total, N, K),
        in_specs=(Tile(M_total, K, bf16, Layout.TMA_128B, tma_box=(BM, BK)),
                  Tile(G * N, K, bf16, Layout.TMA_128B, tma_box=(bn, BK)),
                  Tile(G + 1, s32)),
        out_specs=(Tile(M_total, N, out_dtype, Layout.ROW),),
        flags=F_OUT_BF16 if out_dtype == bf16 else 0, arch=arch,
        meta={"block_n": bn},
    )


def grouped_gemm_flops(G: int, M: int, N: int, K: int) -> int:
    """benchmarks/bench_blackwell_kernels.py:141."""
    return 2 * G * M * N * K
