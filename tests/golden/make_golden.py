"""Generates the golden fixtures in this folder from the reference tree.

Run in a container that has the reference checked out (read-only is enough):

    python tests/golden/make_golden.py /path/to/reference   (or set PYPTX_REFERENCE_DIR)

What it records:

* ``encodings.json`` -- outputs of the reference's own descriptor helpers
  (``ptx.tcgen05.make_instr_desc_f16bf16_f32`` over a grid of arguments), the
  shared-memory descriptor constant its Blackwell GEMMs use, the 128/64/32-byte
  swizzle images implied by ``pyptx.smem._SWIZZLE_PARAMS``, and the launch
  heuristics ``_pick_block`` / ``_pick_rows_per_cta`` of the row kernels;
* ``row_refs.npz`` -- the reference's ``rms_norm_ref`` / ``layer_norm_ref`` /
  ``fused_silu_mul_ref`` / ``softmax_ref`` evaluated on the seeded inputs of its
  example self-tests.  Those functions are written against ``jax.numpy``; jax is
  not installed here, so they run on a stand-in module that maps the handful of
  calls they make onto numpy float32 (same expressions, CPU arithmetic);
* ``matmul_refs.npz`` -- the torch expressions the GEMM / grouped-GEMM /
  attention examples compare against, on small seeded cases with the examples'
  seeds and scales (those expressions are inline in the examples' ``main()``
  helpers, so they are restated here verbatim rather than imported).

The fixtures are small (a few hundred KB) and committed; tests never read the
reference tree.
"""
from __future__ import annotations

import json
import math
import os
import sys
import types

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def install_jax_stand_in() -> None:
    """A numpy-backed module tree that satisfies ``import jax`` / ``jax.numpy``."""
    jnp = types.ModuleType("jax.numpy")
    for name in dir(np):
        if not name.startswith("_"):
            setattr(jnp, name, getattr(np, name))
    jnp.ndarray = np.ndarray
    lax = types.ModuleType("jax.lax")
    lax.rsqrt = lambda v: (np.float32(1.0) / np.sqrt(v)).astype(np.float32)
    nn = types.ModuleType("jax.nn")
    nn.silu = lambda v: (v / (np.float32(1.0) + np.exp(-v))).astype(np.float32)
    jax = types.ModuleType("jax")
    jax.numpy, jax.lax, jax.nn = jnp, lax, nn
    jax.jit = lambda f=None, **kw: f if f is not None else (lambda g: g)
    jax.default_backend = lambda: "cpu"
    jax.Array = np.ndarray
    for n, m in (("jax", jax), ("jax.numpy", jnp), ("jax.lax", lax), ("jax.nn", nn)):
        sys.modules[n] = m


def encodings(ref_root: str) -> dict:
    from pyptx import ptx  # noqa: PLC0415 - reference import
    from pyptx import smem as ref_smem  # noqa: PLC0415
    import examples.blackwell.gemm_highperf_blackwell as ref_gemm  # noqa: PLC0415
    import examples.blackwell.grouped_gemm as ref_grouped  # noqa: PLC0415
    import examples.hopper.rms_norm as ref_rms  # noqa: PLC0415
    import examples.hopper.softmax as ref_softmax  # noqa: PLC0415
    import examples.blackwell.layer_norm as ref_ln  # noqa: PLC0415

    out: dict = {}
    idesc = []
    for m in (64, 128, 256):
        for n in (8, 64, 128, 256):
            for ab in ("f16", "bf16", "tf32"):
                for a_major in ("K", "MN"):
                    for b_major in ("K", "MN"):
                        for scale_a in (1, -1):
                            kw = dict(m=m, n=n, ab_dtype=ab, a_major=a_major, b_major=b_major, scale_a=scale_a)
                            idesc.append({"kw": kw, "value": int(ptx.tcgen05.make_instr_desc_f16bf16_f32(**kw))})
    out["idesc"] = idesc
    out["mma_desc_b128"] = int(ref_gemm.MMA_DESC_B128)
    out["grouped_mma_desc"] = int(getattr(ref_grouped, "MMA_DESC_B128", ref_gemm.MMA_DESC_B128))
    out["gemm_consts"] = {k: int(getattr(ref_gemm, k)) for k in
                          ("BM", "BN", "BK", "STAGES", "STAGES_2SM", "A_STAGE", "B_STAGE", "SMEM_BYTES")}
    sw = {}
    for kind, (mask, shift) in ref_smem._SWIZZLE_PARAMS.items():
        sw[kind] = [int(o ^ ((o & mask) >> shift)) for o in range(0, 2048, 16)]
    out["swizzle"] = sw
    out["pick_block_rms"] = {str(n): int(ref_rms._pick_block(n)) for n in (64, 512, 1024, 2048, 4096, 8192, 16384)}
    out["pick_block_softmax"] = {str(n): int(ref_softmax._pick_block(n)) for n in (64, 512, 1024, 2048, 4096, 8192)}
    out["rows_per_cta"] = {str(b): int(ref_ln._pick_rows_per_cta(b)) for b in (4, 64, 65, 256, 257, 2048)}
    return out


def row_refs() -> dict:
    from examples.hopper.rms_norm import rms_norm_ref  # noqa: PLC0415
    from examples.hopper.layer_norm import layer_norm_ref  # noqa: PLC0415
    from examples.hopper.swiglu import fused_silu_mul_ref  # noqa: PLC0415
    from examples.hopper.softmax import softmax_ref  # noqa: PLC0415

    out = {}
    for B, N in [(4, 64), (16, 512)]:
        # examples/blackwell/rms_norm.py:54-56
        np.random.seed(B * 7919 + N)
        x = np.random.randn(B, N).astype(np.float32) * 0.3
        w = (np.random.randn(N) * 0.1 + 1.0).astype(np.float32)
        out[f"rms_{B}_{N}_x"], out[f"rms_{B}_{N}_w"] = x, w
        out[f"rms_{B}_{N}_y"] = np.asarray(rms_norm_ref(x, w), dtype=np.float32)
        # examples/blackwell/layer_norm.py:64-67
        np.random.seed(B * 65537 + N)
        x = np.random.randn(B, N).astype(np.float32) * 2.0 - 1.0
        w = (np.random.randn(N) * 0.1 + 1.0).astype(np.float32)
        b = (np.random.randn(N) * 0.1).astype(np.float32)
        out[f"ln_{B}_{N}_x"], out[f"ln_{B}_{N}_w"], out[f"ln_{B}_{N}_b"] = x, w, b
        out[f"ln_{B}_{N}_y"] = np.asarray(layer_norm_ref(x, w, b), dtype=np.float32)
        # examples/blackwell/swiglu.py:60-62
        np.random.seed(B * 65537 + N)
        g = np.random.randn(B, N).astype(np.float32) * 0.5
        u = np.random.randn(B, N).astype(np.float32) * 0.5
        out[f"swiglu_{B}_{N}_g"], out[f"swiglu_{B}_{N}_u"] = g, u
        out[f"swiglu_{B}_{N}_y"] = np.asarray(fused_silu_mul_ref(g, u), dtype=np.float32)
        # examples/hopper/softmax.py:218-220
        np.random.seed(B * 7919 + N)
        x = np.random.randn(B, N).astype(np.float32)
        out[f"softmax_{B}_{N}_x"] = x
        out[f"softmax_{B}_{N}_y"] = np.asarray(softmax_ref(x), dtype=np.float32)
    return out


def matmul_refs() -> dict:
    import torch  # noqa: PLC0415

    out = {}
    # examples/blackwell/gemm_highperf_blackwell.py:1257-1268 (seed, scale 0.1, a.float() @ b.float())
    for M, N, K in [(128, 256, 64), (128, 256, 128)]:
        torch.manual_seed(M * 10007 + N * 313 + K)
        a = (torch.randn(M, K) * 0.1).to(torch.bfloat16)
        b = (torch.randn(K, N) * 0.1).to(torch.bfloat16)
        out[f"gemm_{M}_{N}_{K}_a"] = a.view(torch.int16).numpy()
        out[f"gemm_{M}_{N}_{K}_bt"] = b.t().contiguous().view(torch.int16).numpy()
        out[f"gemm_{M}_{N}_{K}_d"] = (a.float() @ b.float()).numpy()
    # examples/blackwell/grouped_gemm.py:296-306
    for G, M, N, K in [(2, 128, 64, 64), (2, 128, 128, 128)]:
        torch.manual_seed(G * 1009 + M * 997 + N * 17 + K)
        a3 = (torch.randn(G, M, K) * 0.1).to(torch.bfloat16)
        b3 = (torch.randn(G, K, N) * 0.1).to(torch.bfloat16)
        out[f"grouped_{G}_{M}_{N}_{K}_a"] = a3.reshape(G * M, K).view(torch.int16).numpy()
        out[f"grouped_{G}_{M}_{N}_{K}_bt"] = b3.transpose(1, 2).contiguous().reshape(G * N, K).view(torch.int16).numpy()
        out[f"grouped_{G}_{M}_{N}_{K}_c"] = torch.einsum("gmk,gkn->gmn", a3.float(), b3.float()).reshape(G * M, N).numpy()
    # examples/hopper/experimental/flash_attention_hopper.py:472-479
    for M_q, N_seq, HD in [(128, 128, 64), (128, 256, 64), (128, 128, 128)]:
        torch.manual_seed(M_q * 131 + N_seq + HD * 7)
        q = (torch.randn(M_q, HD) * 0.3).to(torch.bfloat16)
        k = (torch.randn(N_seq, HD) * 0.3).to(torch.bfloat16)
        v = (torch.randn(N_seq, HD) * 0.3).to(torch.bfloat16)
        ref = torch.softmax(q.float() @ k.float().T / math.sqrt(HD), dim=-1) @ v.float()
        for name, t in (("q", q), ("k", k), ("v", v)):
            out[f"fa_{M_q}_{N_seq}_{HD}_{name}"] = t.view(torch.int16).numpy()
        out[f"fa_{M_q}_{N_seq}_{HD}_o"] = ref.numpy()
    return out


def main() -> None:
    ref_root = sys.argv[1] if len(sys.argv) > 1 else os.environ.get("PYPTX_REFERENCE_DIR", "")
    if not os.path.isdir(os.path.join(ref_root, "pyptx")):
        raise SystemExit("usage: make_golden.py <reference tree>  (or set PYPTX_REFERENCE_DIR)")
    install_jax_stand_in()
    sys.path.insert(0, ref_root)
    with open(os.path.join(HERE, "encodings.json"), "w") as f:
        json.dump(encodings(ref_root), f, indent=1, sort_keys=True)
    np.savez_compressed(os.path.join(HERE, "row_refs.npz"), **row_refs())
    np.savez_compressed(os.path.join(HERE, "matmul_refs.npz"), **matmul_refs())
    for name in ("encodings.json", "row_refs.npz", "matmul_refs.npz"):
        print(name, os.path.getsize(os.path.join(HERE, name)), "bytes")


if __name__ == "__main__":
    main()
