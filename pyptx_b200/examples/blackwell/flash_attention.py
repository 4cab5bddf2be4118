"""Flash-attention forward for B200 (tcgen05), batched over batch x heads.

``O = softmax(Q K^T * sm_scale [+ causal mask]) V`` with bf16 operands, fp32 scores and
statistics.  The algorithm is the reference's
(examples/hopper/experimental/flash_attention_hopper.py:44-465: online softmax over K/V
tiles, P rounded to bf16 before the second product); that kernel is sm_90a-only, single
head, non-causal and limited to head_dim <= 64, so this entry point adds the batch and head
dimensions, head dimensions up to 128 (any multiple of 8) and the causal mask.  ``build_flash_attention_hopper`` in
``pyptx_b200.examples.hopper.experimental.flash_attention_hopper`` keeps the reference's
single-head call signature on top of the same kernel.
"""
from __future__ import annotations

import math

from ..._ids import (F_CAUSAL, F_DETERMINISTIC, F_K_TRANSPOSED, F_OUT_BF16, F_RETURN_LSE, K_FLASH_ATTN,
                      K_FLASH_ATTN_BWD)
from ...kernel import NativeKernel
from ...specs import Layout, Tile
from ...types import PtxType, bf16, f32

BLOCK_M = 128   # query rows per tile (two tiles per CTA)
BLOCK_N = 128   # keys per K/V tile
HEAD_DIMS = tuple(range(8, 129, 8))   # tiles are 64 or 128 wide; narrower heads are zero-filled by TMA


def _check(seq_q: int, seq_kv: int, head_dim: int, causal: bool) -> None:
    assert head_dim in HEAD_DIMS, f"head_dim={head_dim} must be a multiple of 8 in [8, 128]"
    assert seq_q >= 1, f"M_q={seq_q} must be positive"
    assert seq_kv >= 1, f"N_seq={seq_kv} must be positive"
    assert not causal or seq_kv >= seq_q, "causal attention needs N_seq >= M_q"


def build_flash_attention(batch: int, heads: int, seq_q: int, seq_kv: int | None = None,
                          head_dim: int = 64, *, causal: bool = False, sm_scale: float | None = None,
                          out_dtype: PtxType = bf16, arch: str = "sm_100a", return_lse: bool = False,
                          _debug_flags: int = 0) -> NativeKernel:
    """Kernel ``k(Q[B,H,Sq,d], K[B,H,Skv,d], V[B,H,Skv,d]) -> O[B,H,Sq,d]`` (bf16 in).

    ``causal`` lets query ``i`` see keys ``j <= i + (Skv - Sq)``.  ``sm_scale`` defaults to
    ``1/sqrt(head_dim)``.  ``out_dtype`` is bf16 (default) or f32.  Sequence lengths need not be
    multiples of the 128-wide tiles: partial tiles are zero-filled by TMA and masked.  The kernel's
    tiles are 64 (``head_dim <= 64``) or 128 columns wide; narrower heads are zero-filled the same way.
    With ``return_lse`` the kernel returns ``(O, lse)``, ``lse[B,H,Sq]`` (f32) being the natural-log
    sum-exp of the scaled, masked scores of each query row.
    """
    assert arch.startswith("sm_100"), "Blackwell attention is only implemented for sm_100*"
    seq_kv = seq_q if seq_kv is None else seq_kv
    _check(seq_q, seq_kv, head_dim, causal)
    assert batch >= 1 and heads >= 1 and batch * heads <= 65535, "batch*heads must be in [1, 65535]"
    assert out_dtype in (f32, bf16), f"out_dtype must be f32 or bf16, got {out_dtype}"
    scale = 1.0 / math.sqrt(head_dim) if sm_scale is None else float(sm_scale)
    flags = ((F_CAUSAL if causal else 0) | (F_OUT_BF16 if out_dtype == bf16 else 0) |
             (F_RETURN_LSE if return_lse else 0) | _debug_flags)
    lse_spec = (Tile(batch, heads, seq_q, f32, Layout.ROW),) if return_lse else ()
    return NativeKernel(
        "flash_attn_fwd", K_FLASH_ATTN, (batch * heads, seq_q, seq_kv, head_dim),
        in_specs=(Tile(batch, heads, seq_q, head_dim, bf16, Layout.TMA_128B, tma_box=(BLOCK_M, 64)),
                  Tile(batch, heads, seq_kv, head_dim, bf16, Layout.TMA_128B, tma_box=(BLOCK_N, 64)),
                  Tile(batch, heads, seq_kv, head_dim, bf16, Layout.TMA_128B, tma_box=(BLOCK_N, 64))),
        out_specs=(Tile(batch, heads, seq_q, head_dim, out_dtype, Layout.ROW),) + lse_spec,
        fparams=(scale,), flags=flags, arch=arch,
        meta={"causal": causal, "sm_scale": scale, "block_m": BLOCK_M, "block_n": BLOCK_N},
    )


def build_flash_attention_bwd(batch: int, heads: int, seq_q: int, seq_kv: int | None = None,
                              head_dim: int = 64, *, causal: bool = False, sm_scale: float | None = None,
                              out_dtype: PtxType = bf16, deterministic: bool = False,
                              arch: str = "sm_100a") -> NativeKernel:
    """Kernel ``k(Q, K, V, O, lse, dO) -> (dQ, dK, dV)``: the backward half of
    ``build_flash_attention(..., return_lse=True)`` (same ``causal`` / ``sm_scale``).

    ``Q``, ``K``, ``V``, ``O`` and ``dO`` are bf16 in the forward's layouts, ``lse[B,H,Sq]`` is the
    forward's second output (the argument order is the one ``differentiable_kernel`` uses: saved
    inputs, saved outputs, incoming gradient); the gradients come back as ``out_dtype`` (bf16 or f32).  The reference
    has the autograd hook for such a pair (pyptx/torch_support.py:446-519) but no backward kernel.
    P and dS are recomputed from ``lse`` tile by tile.  By default one pass over key tiles produces
    dK, dV and each tile pair's share of dQ, which is added into an fp32 buffer with atomics (five
    products per tile pair; dQ may differ in the last bits from run to run).  ``deterministic=True``
    takes dQ from a second pass over query tiles instead (seven products, no atomics,
    bit-reproducible).
    """
    assert arch.startswith("sm_100"), "Blackwell attention is only implemented for sm_100*"
    seq_kv = seq_q if seq_kv is None else seq_kv
    _check(seq_q, seq_kv, head_dim, causal)
    assert batch >= 1 and heads >= 1 and batch * heads <= 65535, "batch*heads must be in [1, 65535]"
    assert out_dtype in (f32, bf16), f"out_dtype must be f32 or bf16, got {out_dtype}"
    scale = 1.0 / math.sqrt(head_dim) if sm_scale is None else float(sm_scale)
    flags = (F_CAUSAL if causal else 0) | (F_OUT_BF16 if out_dtype == bf16 else 0) | \
            (F_DETERMINISTIC if deterministic else 0)
    q_tile = Tile(batch, heads, seq_q, head_dim, bf16, Layout.TMA_128B, tma_box=(BLOCK_M, 64))
    kv_tile = Tile(batch, heads, seq_kv, head_dim, bf16, Layout.TMA_128B, tma_box=(BLOCK_N, 64))
    return NativeKernel(
        "flash_attn_bwd", K_FLASH_ATTN_BWD, (batch * heads, seq_q, seq_kv, head_dim),
        in_specs=(q_tile, kv_tile, kv_tile, Tile(batch, heads, seq_q, head_dim, bf16, Layout.ROW),
                  Tile(batch, heads, seq_q, f32, Layout.ROW), q_tile),
        out_specs=(Tile(batch, heads, seq_q, head_dim, out_dtype, Layout.ROW),
                   Tile(batch, heads, seq_kv, head_dim, out_dtype, Layout.ROW),
                   Tile(batch, heads, seq_kv, head_dim, out_dtype, Layout.ROW)),
        fparams=(scale,), flags=flags, arch=arch,
        meta={"causal": causal, "sm_scale": scale, "block_m": BLOCK_M, "block_n": BLOCK_N,
              "deterministic": deterministic},
    )


def build_differentiable_flash_attention(batch: int, heads: int, seq_q: int, seq_kv: int | None = None,
                                         head_dim: int = 64, *, causal: bool = False,
                                         sm_scale: float | None = None, deterministic: bool = False):
    """``attn(Q, K, V) -> O`` (bf16) that takes part in autograd: the forward kernel with its
    log-sum-exp output, and the backward kernel, joined by ``differentiable_kernel``
    (the reference's hook, pyptx/torch_support.py:446-519)."""
    from ...torch_support import differentiable_kernel

    fwd = build_flash_attention(batch, heads, seq_q, seq_kv, head_dim, causal=causal, sm_scale=sm_scale,
                                out_dtype=bf16, return_lse=True)
    bwd = build_flash_attention_bwd(batch, heads, seq_q, seq_kv, head_dim, causal=causal, sm_scale=sm_scale,
                                    out_dtype=bf16, deterministic=deterministic)
    return differentiable_kernel(fwd, bwd, save_outputs=(0, 1), visible_outputs=(0,))


def attention_bwd_flops(batch: int, heads: int, seq_q: int, seq_kv: int, head_dim: int, causal: bool = False) -> float:
    """Five products per tile pair (S, dP, dV, dK, dQ): 2.5x the forward."""
    return 2.5 * attention_flops(batch, heads, seq_q, seq_kv, head_dim, causal)


def attention_flops(batch: int, heads: int, seq_q: int, seq_kv: int, head_dim: int, causal: bool = False) -> float:
    """4*B*H*Sq*Skv*d for the two products; half of it under the causal mask."""
    f = 4.0 * batch * heads * seq_q * seq_kv * head_dim
    return f / 2 if causal else f


__all__ = ["build_flash_attention", "build_flash_attention_bwd", "build_differentiable_flash_attention",
           "attention_flops", "attention_bwd_flops", "F_K_TRANSPOSED"]
