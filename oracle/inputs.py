"""Seeded synthetic inputs for every benchmark configuration.  TEST INFRASTRUCTURE.

Inputs are drawn on the CPU from a seeded ``torch.Generator`` so that the
oracle and the CUDA kernels see identical bits; the reference's own benchmarks
use unseeded ``torch.randn`` of the same shapes
(benchmarks/bench_blackwell_kernels.py:55-56, 78-80, 102-103, 125-126).
Seeds follow the reference's example self-tests
(examples/blackwell/rms_norm.py:54, layer_norm.py:64, swiglu.py:60,
gemm_highperf_blackwell.py:1257, grouped_gemm.py:296,
examples/hopper/experimental/flash_attention_hopper.py:472).
"""
from __future__ import annotations

import math

import torch


def _gen(seed: int) -> torch.Generator:
    g = torch.Generator(device="cpu")
    g.manual_seed(int(seed))
    return g


def rms_norm_inputs(B: int = 2048, N: int = 8192):
    """x ~ N(0,1), w ~ N(1, 0.02); seed B*7919+N."""
    g = _gen(B * 7919 + N)
    x = torch.randn(B, N, generator=g, dtype=torch.float32)
    w = 1.0 + 0.02 * torch.randn(N, generator=g, dtype=torch.float32)
    return x, w


def layer_norm_inputs(B: int = 2048, N: int = 8192):
    """x ~ N(0,1), gamma ~ N(1,0.02), beta ~ N(0,0.02); seed B*65537+N."""
    g = _gen(B * 65537 + N)
    x = torch.randn(B, N, generator=g, dtype=torch.float32)
    w = 1.0 + 0.02 * torch.randn(N, generator=g, dtype=torch.float32)
    b = 0.02 * torch.randn(N, generator=g, dtype=torch.float32)
    return x, w, b


def swiglu_inputs(M: int = 2048, F: int = 8192):
    """gate, up ~ N(0,1); seed M*65537+F."""
    g = _gen(M * 65537 + F)
    gate = torch.randn(M, F, generator=g, dtype=torch.float32)
    up = torch.randn(M, F, generator=g, dtype=torch.float32)
    return gate, up


def softmax_inputs(B: int = 2048, N: int = 8192):
    """x ~ N(0, 2^2); seed B*7919+N."""
    g = _gen(B * 7919 + N)
    return (2.0 * torch.randn(B, N, generator=g, dtype=torch.float32),)


def gemm_inputs(M: int, N: int, K: int):
    """A[M,K], B[K,N] ~ N(0,1)/sqrt(K) rounded to bf16; returns (A, B_T) with
    B_T = B.t().contiguous(); seed M*10007+N*313+K."""
    g = _gen(M * 10007 + N * 313 + K)
    s = 1.0 / math.sqrt(K)
    a = (torch.randn(M, K, generator=g, dtype=torch.float32) * s).to(torch.bfloat16)
    b = (torch.randn(K, N, generator=g, dtype=torch.float32) * s).to(torch.bfloat16)
    return a, b.t().contiguous()


def grouped_gemm_inputs(G: int, M: int, N: int, K: int):
    """A[G,M,K], W[G,K,N] ~ N(0,1)/sqrt(K) -> bf16; returns (A2[G*M,K], B_T2[G*N,K]);
    seed G*1009+M*997+N*17+K."""
    g = _gen(G * 1009 + M * 997 + N * 17 + K)
    s = 1.0 / math.sqrt(K)
    a = (torch.randn(G, M, K, generator=g, dtype=torch.float32) * s).to(torch.bfloat16)
    w = (torch.randn(G, K, N, generator=g, dtype=torch.float32) * s).to(torch.bfloat16)
    return a.reshape(G * M, K), w.transpose(1, 2).contiguous().reshape(G * N, K)


def attention_inputs(BH: int, S_q: int, S_kv: int, d: int):
    """Q[BH,S_q,d], K[BH,S_kv,d], V[BH,S_kv,d] ~ N(0,1) -> bf16; seed S_q*131+S_kv+d*7."""
    g = _gen(S_q * 131 + S_kv + d * 7)
    q = torch.randn(BH, S_q, d, generator=g, dtype=torch.float32).to(torch.bfloat16)
    k = torch.randn(BH, S_kv, d, generator=g, dtype=torch.float32).to(torch.bfloat16)
    v = torch.randn(BH, S_kv, d, generator=g, dtype=torch.float32).to(torch.bfloat16)
    return q, k, v
