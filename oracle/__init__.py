"""CPU oracle for the kernel library -- TEST INFRASTRUCTURE, NOT PRODUCT CODE.

This package restates, on the CPU, what the reference project itself uses as
ground truth for the kernels this library implements: the torch / jax.numpy
reference formulas written next to each example kernel, and the integer
encodings (tcgen05 instruction descriptor, shared-memory matrix descriptor,
128-byte swizzle) that its tests pin as known answers.

Only ``tests/``, ``__graft_entry__.smoke()`` and ``bench.py``'s CPU-baseline /
reference legs may import it.  Nothing under ``pyptx_b200/`` imports it, and
the product path has no CPU fallback.

Parity pin: ``tests/golden/make_golden.py`` runs the reference's own
``*_ref`` functions and descriptor helpers (imported from the reference tree
with a numpy-backed stand-in for the absent ``jax`` package) and commits their
outputs under ``tests/golden/``; ``tests/test_oracle.py`` checks every function
here against those vectors and against the reference tests' known answers.
"""
from .formulas import (  # noqa: F401
    attention_ref, gemm_ref, grouped_gemm_ref, grouped_gemm_swiglu_ref, grouped_gemm_varlen_ref, layer_norm_ref, rms_norm_ref,
    softmax_ref, swiglu_ref,
)
from .encodings import (  # noqa: F401
    instr_desc_f16bf16_f32, smem_desc, swizzle_128b, SMEM_DESC_SW128_KMAJOR,
)
