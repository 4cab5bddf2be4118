"""bf16 GEMM for B200 on tcgen05 tensor cores: ``D = A @ B_T.T`` with fp32 accumulation.

Drop-in for the reference entry points (examples/blackwell/gemm_highperf_blackwell.py):

* ``build_gemm(M, N, K, *, arch, stages, grid_minor_dim, grid_tile_width)`` (:69-313):
  1-SM MMA, one 128x256 output tile per CTA at a time;
* ``build_gemm_2sm(M, N, K, *, arch, stages, grid_minor_dim, grid_tile_width)`` (:902-1246):
  ``cta_group::2`` MMA, one 256x256 tile per 2-CTA cluster.

Both take ``A[M,K]`` bf16 and ``B_T[N,K]`` bf16 (the caller passes
``b.t().contiguous()``, as in the reference, :1264) and return ``D[M,N]`` f32.
``out_dtype=bf16`` is an extension that rounds the result in the epilogue.
"""
from __future__ import annotations

from ..._ids import F_ACT_GELU, F_ACT_RELU, F_ACT_SILU, F_BIAS, F_OUT_BF16, K_GEMM_1SM, K_GEMM_2SM
from ...kernel import NativeKernel
from ...specs import Layout, Tile
from ...types import PtxType, bf16, f32

BM = 128
BN = 256
BK = 64
STAGES = 4
STAGES_2SM = 5
GRID_MINOR_DIM = "n"
GRID_TILE_WIDTH = 16


_TILE_FLAGS = {"auto": 0, "narrow": 1 << 18, "wide": 1 << 19}
_ACT_FLAGS = {None: 0, "relu": F_ACT_RELU, "gelu": F_ACT_GELU, "silu": F_ACT_SILU}


def _epilogue(N: int, bias: bool, activation):
    """Flags and extra input spec of the fused epilogue ``D = act(A @ B_T.T + bias)``."""
    assert activation in _ACT_FLAGS, f"activation must be one of {list(_ACT_FLAGS)}, got {activation!r}"
    flags = _ACT_FLAGS[activation] | (F_BIAS if bias else 0)
    extra = (Tile(N, f32, Layout.ROW),) if bias else ()
    return flags, extra


def _out_flags(out_dtype: PtxType) -> int:
    assert out_dtype in (f32, bf16), f"out_dtype must be f32 or bf16, got {out_dtype}"
    return F_OUT_BF16 if out_dtype == bf16 else 0


def build_gemm(M: int, N: int, K: int, *, arch: str = "sm_100a", stages: int = STAGES,
               grid_minor_dim: str = GRID_MINOR_DIM, grid_tile_width: int = GRID_TILE_WIDTH,
               out_dtype: PtxType = f32, tile: str = "auto", bias: bool = False,
               activation: str | None = None, _name: str = "blackwell_gemm",
               _meta: dict | None = None) -> NativeKernel:
    """Kernel ``k(A[M,K] bf16, B_T[N,K] bf16) -> D[M,N]``.

    ``stages`` and ``grid_minor_dim`` are accepted and validated as in the
    reference; the native kernel sizes its own shared-memory ring and always
    rasterises M-fastest inside a band.  ``grid_tile_width`` is the number of
    M-tiles per raster band (with the default the kernel picks the band itself).
    ``tile`` (an addition): ``"auto"`` runs large problems on double-height tiles
    (256 x 256 per CTA), ``"narrow"`` / ``"wide"`` force one.
    ``bias`` / ``activation`` (additions): with ``bias=True`` the kernel takes a third
    input ``bias[N]`` (f32) and computes ``act(A @ B_T.T + bias)`` in its epilogue;
    ``activation`` is ``None``, ``"relu"``, ``"gelu"`` (erf form) or ``"silu"``.
    """
    assert arch.startswith("sm_100"), "Blackwell GEMM is only implemented for sm_100*"
    assert M % BM == 0, f"M={M} must be divisible by {BM}"
    assert N % BN == 0, f"N={N} must be divisible by {BN}"
    assert K % BK == 0, f"K={K} must be divisible by {BK}"
    assert stages >= 2, "Blackwell GEMM requires at least two stages"
    assert grid_tile_width >= 1, "grid_tile_width must be at least 1"
    assert grid_minor_dim.lower() in {"m", "n"}, "grid_minor_dim must be 'm' or 'n'"
    assert tile in _TILE_FLAGS, f"tile must be one of {sorted(_TILE_FLAGS)}, got {tile!r}"
    dims = (M, N, K) if grid_tile_width == GRID_TILE_WIDTH else (M, N, K, grid_tile_width)
    epi_flags, epi_inputs = _epilogue(N, bias, activation)
    return NativeKernel(
        _name, K_GEMM_1SM, dims,
        in_specs=(Tile(M, K, bf16, Layout.TMA_128B, tma_box=(BM, BK)),
                  Tile(N, K, bf16, Layout.TMA_128B, tma_box=(BN, BK))) + epi_inputs,
        out_specs=(Tile(M, N, out_dtype, Layout.ROW),),
        flags=_out_flags(out_dtype) | _TILE_FLAGS[tile] | epi_flags, arch=arch,
        meta=dict({"stages": stages, "grid_minor_dim": grid_minor_dim, "grid_tile_width": grid_tile_width,
                   "tile": tile}, **(_meta or {})),
    )


def build_gemm_2sm(M: int, N: int, K: int, *, arch: str = "sm_100a", stages: int = STAGES_2SM,
                   grid_minor_dim: str = GRID_MINOR_DIM, grid_tile_width: int = GRID_TILE_WIDTH,
                   out_dtype: PtxType = f32, tile: str = "auto", bias: bool = False,
                   activation: str | None = None) -> NativeKernel:
    """2-SM variant: same call convention (``bias`` / ``activation`` as for :func:`build_gemm`),
    ``M`` must divide by 256.

    ``tile`` (an addition): ``"auto"`` lets the kernel run large problems on 512 x 256 tiles
    per CTA pair (``M % 512 == 0`` and enough tiles to fill the last wave) and the rest on
    256 x 256; ``"narrow"`` / ``"wide"`` force one.  With the default ``grid_tile_width`` the
    kernel picks the raster band itself."""
    assert arch.startswith("sm_100")
    assert M % (2 * BM) == 0, f"M={M} must be divisible by {2 * BM} for 2SM"
    assert N % BN == 0, f"N={N} must be divisible by {BN}"
    assert K % BK == 0, f"K={K} must be divisible by {BK}"
    assert stages >= 2, "2SM Blackwell GEMM requires at least two stages"
    assert grid_tile_width >= 1, "grid_tile_width must be at least 1"
    assert grid_minor_dim.lower() in {"m", "n"}, "grid_minor_dim must be 'm' or 'n'"
    assert tile in _TILE_FLAGS, f"tile must be one of {sorted(_TILE_FLAGS)}, got {tile!r}"
    dims = (M, N, K) if grid_tile_width == GRID_TILE_WIDTH else (M, N, K, grid_tile_width)
    epi_flags, epi_inputs = _epilogue(N, bias, activation)
    return NativeKernel(
        "blackwell_gemm_2sm", K_GEMM_2SM, dims,
        in_specs=(Tile(M, K, bf16, Layout.TMA_128B, tma_box=(BM, BK)),
                  Tile(N, K, bf16, Layout.TMA_128B, tma_box=(BN // 2, BK))) + epi_inputs,
        out_specs=(Tile(M, N, out_dtype, Layout.ROW),),
        flags=_out_flags(out_dtype) | _TILE_FLAGS[tile] | epi_flags, arch=arch,
        meta={"stages": stages, "grid_minor_dim": grid_minor_dim, "grid_tile_width": grid_tile_width, "tile": tile},
    )


def build_gemm_persistent(M: int, N: int, K: int, *, arch: str = "sm_100a", stages: int = STAGES,
                          grid_minor_dim: str = "n", grid_tile_width: int = 8, num_ctas: int | None = None,
                          out_dtype: PtxType = f32) -> NativeKernel:
    """The reference's persistent 1-SM entry point (gemm_highperf_blackwell.py:316-326), same call
    convention as :func:`build_gemm`.  Every kernel of this library is persistent (one CTA per SM
    walks a static tile list), so this is an alias of :func:`build_gemm` with the reference's default
    band of 8 and the reference's kernel name (``blackwell_gemm_persistent``, :370).  ``num_ctas`` and
    ``stages`` are validated and recorded in ``meta`` but do not shape the launch: the grid is always
    one CTA per SM (or per tile if fewer) and the ring depth follows from the tile shape."""
    assert num_ctas is None or num_ctas >= 1, "num_ctas must be positive"
    return build_gemm(M, N, K, arch=arch, stages=stages, grid_minor_dim=grid_minor_dim,
                      grid_tile_width=grid_tile_width, out_dtype=out_dtype,
                      _name="blackwell_gemm_persistent", _meta={"num_ctas": num_ctas})


def gemm_flops(M: int, N: int, K: int) -> int:
    """benchmarks/bench_blackwell_gemm.py:56."""
    return 2 * M * N * K
