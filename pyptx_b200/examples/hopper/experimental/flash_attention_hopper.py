"""The reference's single-head attention entry point, served by the sm_100a kernel.

``build_flash_attention_hopper(M_q, N_seq, head_dim=64, *, sm_scale=None)`` keeps the call
convention of examples/hopper/experimental/flash_attention_hopper.py:44-50: inputs
``Q[M_q, HD]``, ``K_t[HD, N_seq]`` (K transposed by the caller) and ``V[N_seq, HD]`` in
bf16, output ``O[M_q, HD]`` in f32.  Differences: ``head_dim`` is any multiple of 8 up to 128 (the
reference takes 16, 32 or 64); ``M_q`` is any positive length (the reference wants multiples of 128) and ``N_seq``
any multiple of 8 (the reference: multiples of 64; 8 keeps the rows of ``K_t`` 16-byte aligned).
"""
from __future__ import annotations

import math

from ...._ids import F_K_TRANSPOSED, K_FLASH_ATTN
from ....kernel import NativeKernel
from ....specs import Layout, Tile
from ....types import bf16, f32
from ...blackwell.flash_attention import BLOCK_M, BLOCK_N, _check


def build_flash_attention_hopper(M_q: int, N_seq: int, head_dim: int = 64, *,
                                 sm_scale: float | None = None, arch: str = "sm_100a") -> NativeKernel:
    _check(M_q, N_seq, head_dim, False)
    assert N_seq % 8 == 0, f"N_seq={N_seq} must be divisible by 8 (16-byte aligned rows of K_t)"
    scale = 1.0 / math.sqrt(head_dim) if sm_scale is None else float(sm_scale)
    return NativeKernel(
        "flash_attn", K_FLASH_ATTN, (1, M_q, N_seq, head_dim),
        in_specs=(Tile(M_q, head_dim, bf16, Layout.TMA_128B, tma_box=(BLOCK_M, 64)),
                  Tile(head_dim, N_seq, bf16, Layout.TMA_128B, tma_box=(head_dim, 64)),
                  Tile(N_seq, head_dim, bf16, Layout.TMA_128B, tma_box=(BLOCK_N, 64))),
        out_specs=(Tile(M_q, head_dim, f32, Layout.ROW),),
        fparams=(scale,), flags=F_K_TRANSPOSED, arch=arch,
        meta={"sm_scale": scale},
    )
