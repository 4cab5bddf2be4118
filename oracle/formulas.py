"""fp32 CPU formulas -- the numerical oracle.  TEST INFRASTRUCTURE, NOT PRODUCT CODE.

Each function restates the torch expression the reference compares its kernel
against (file:line given per function) and runs it with torch on the host in
float32.  bf16 inputs are widened to float32 first, so matrix products are
fp32-accumulated results of the bf16-rounded operands.
"""
from __future__ import annotations

import math

import torch


def rms_norm_ref(x: torch.Tensor, w: torch.Tensor, eps: float = 1e-6) -> torch.Tensor:
    """examples/blackwell/rms_norm.py:62-63 (torch case); examples/hopper/rms_norm.py:189-192."""
    x = x.float()
    ms = (x * x).mean(dim=-1, keepdim=True)
    return x * torch.rsqrt(ms + eps) * w.float()


def layer_norm_ref(x: torch.Tensor, w: torch.Tensor, b: torch.Tensor, eps: float = 1e-5) -> torch.Tensor:
    """examples/hopper/layer_norm.py:232-236; tests/test_torch_dispatch.py:65-67
    (equivalent to F.layer_norm, examples/blackwell/layer_norm.py:74)."""
    x = x.float()
    mean = x.mean(dim=-1, keepdim=True)
    var = ((x - mean) ** 2).mean(dim=-1, keepdim=True)
    return (x - mean) * torch.rsqrt(var + eps) * w.float() + b.float()


def swiglu_ref(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """examples/blackwell/swiglu.py:66; examples/hopper/swiglu.py:163-164."""
    return torch.nn.functional.silu(gate.float()) * up.float()


def softmax_ref(x: torch.Tensor) -> torch.Tensor:
    """examples/hopper/softmax.py:189-193 and :224."""
    return torch.softmax(x.float(), dim=-1)


def gemm_ref(a: torch.Tensor, b_t: torch.Tensor) -> torch.Tensor:
    """``a.float() @ b.float()`` (examples/blackwell/gemm_highperf_blackwell.py:1268) with
    the kernel's operand convention: ``b_t`` is ``b.t().contiguous()`` (:1264)."""
    return a.float() @ b_t.float().t()


def gemm_bias_act_ref(a: torch.Tensor, b_t: torch.Tensor, bias: torch.Tensor | None = None,
                      activation: str | None = None) -> torch.Tensor:
    """``act(a.float() @ b.float() + bias)``: the reference's GEMM formula
    (examples/blackwell/gemm_highperf_blackwell.py:1268) followed by the torch ops a caller
    would apply to its result (``F.relu`` / ``F.gelu`` (erf form) / ``F.silu``, the last as
    in examples/blackwell/swiglu.py:66).  The reference has no fused form."""
    d = gemm_ref(a, b_t)
    if bias is not None:
        d = d + bias.float()
    if activation is None:
        return d
    fn = torch.nn.functional
    return {"relu": fn.relu, "gelu": fn.gelu, "silu": fn.silu}[activation](d)


def grouped_gemm_ref(a2: torch.Tensor, b_t2: torch.Tensor, G: int) -> torch.Tensor:
    """``einsum("gmk,gkn->gmn")`` in fp32 (examples/blackwell/grouped_gemm.py:306) on the
    stacked operands ``a2[G*M,K]`` and ``b_t2[G*N,K]`` (:302-303); returns ``[G*M, N]``."""
    gm, k = a2.shape
    gn = b_t2.shape[0]
    m, n = gm // G, gn // G
    a3 = a2.float().reshape(G, m, k)
    b3 = b_t2.float().reshape(G, n, k).transpose(1, 2)
    return torch.einsum("gmk,gkn->gmn", a3, b3).reshape(G * m, n)


def grouped_gemm_varlen_ref(a: torch.Tensor, b_t2: torch.Tensor, offsets, n: int) -> torch.Tensor:
    """Per-expert ``a[o_e:o_{e+1}].float() @ b_t2[e*n:(e+1)*n].float().T`` -- the grouped formula
    (examples/blackwell/grouped_gemm.py:306) with the row ranges given by ``offsets``; rows at or
    beyond ``offsets[-1]`` come back as NaN so that a test notices anything written there."""
    out = torch.full((a.shape[0], n), float("nan"), dtype=torch.float32)
    offs = [int(o) for o in offsets]
    for e in range(len(offs) - 1):
        lo, hi = offs[e], offs[e + 1]
        if hi > lo:
            out[lo:hi] = a[lo:hi].float() @ b_t2[e * n:(e + 1) * n].float().t()
    return out


def grouped_gemm_swiglu_ref(a2: torch.Tensor, w_t2: torch.Tensor, G: int) -> torch.Tensor:
    """The two reference ops composed: grouped GEMM (examples/blackwell/grouped_gemm.py:306) then
    ``F.silu(gate) * up`` (examples/blackwell/swiglu.py:66).  ``w_t2[G*2F, K]`` holds, per expert,
    F gate rows followed by F up rows; returns ``[G*M, F]`` in fp32."""
    c = grouped_gemm_ref(a2, w_t2, G)                 # [G*M, 2F]
    f = c.shape[1] // 2
    return torch.nn.functional.silu(c[:, :f]) * c[:, f:]


def attention_ref(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, *, causal: bool = False,
                  sm_scale: float | None = None) -> torch.Tensor:
    """``softmax(q k^T * scale) v`` in fp32 per leading index
    (examples/hopper/experimental/flash_attention_hopper.py:479).  ``q[..., M, d]``,
    ``k[..., N, d]``, ``v[..., N, d]``.  ``causal`` adds the lower-triangular mask
    before the softmax (query i sees keys j <= i + N - M); the reference has no
    causal case."""
    q, k, v = q.float(), k.float(), v.float()
    d = q.shape[-1]
    scale = (1.0 / math.sqrt(d)) if sm_scale is None else sm_scale
    s = q @ k.transpose(-1, -2) * scale
    if causal:
        m, n = s.shape[-2], s.shape[-1]
        mask = torch.ones(m, n, dtype=torch.bool).tril(diagonal=n - m)
        s = s.masked_fill(~mask, float("-inf"))
    return torch.softmax(s, dim=-1) @ v


def attention_lse_ref(q: torch.Tensor, k: torch.Tensor, *, causal: bool = False,
                      sm_scale: float | None = None) -> torch.Tensor:
    """Row-wise ``logsumexp`` of the scaled (and causally masked) scores of :func:`attention_ref`:
    the statistic the reference's kernel keeps per row as running max and sum
    (examples/hopper/experimental/flash_attention_hopper.py:213-256)."""
    q, k = q.float(), k.float()
    scale = (1.0 / math.sqrt(q.shape[-1])) if sm_scale is None else sm_scale
    s = q @ k.transpose(-1, -2) * scale
    if causal:
        m, n = s.shape[-2], s.shape[-1]
        s = s.masked_fill(~torch.ones(m, n, dtype=torch.bool).tril(diagonal=n - m), float("-inf"))
    return torch.logsumexp(s, dim=-1)


def attention_bwd_ref(q, k, v, d_out, *, causal: bool = False, sm_scale: float | None = None):
    """(dq, dk, dv) by autograd through :func:`attention_ref`'s formula in float64 (returned as
    float32), the way the row-kernel backward references are formed."""
    q64, k64, v64 = (t.double().requires_grad_() for t in (q, k, v))
    d = q.shape[-1]
    scale = (1.0 / math.sqrt(d)) if sm_scale is None else sm_scale
    s = q64 @ k64.transpose(-1, -2) * scale
    if causal:
        m, n = s.shape[-2], s.shape[-1]
        s = s.masked_fill(~torch.ones(m, n, dtype=torch.bool).tril(diagonal=n - m), float("-inf"))
    o = torch.softmax(s, dim=-1) @ v64
    dq, dk, dv = torch.autograd.grad(o, (q64, k64, v64), d_out.double())
    return dq.float(), dk.float(), dv.float()


def rms_norm_bwd_ref(x, w, dy, eps: float = 1e-6):
    """(dx, dw) by autograd through the forward formula (float64 internally, returned as float32)."""
    x64, w64 = x.double().requires_grad_(), w.double().requires_grad_()
    y = x64 * torch.rsqrt((x64 * x64).mean(-1, keepdim=True) + eps) * w64
    dx, dw = torch.autograd.grad(y, (x64, w64), dy.double())
    return dx.float(), dw.float()


def layer_norm_bwd_ref(x, w, dy, eps: float = 1e-5):
    """(dx, dw, db) by autograd through the forward formula (float64 internally)."""
    x64, w64 = x.double().requires_grad_(), w.double().requires_grad_()
    b64 = torch.zeros_like(w64).requires_grad_()
    mean = x64.mean(-1, keepdim=True)
    var = ((x64 - mean) ** 2).mean(-1, keepdim=True)
    y = (x64 - mean) * torch.rsqrt(var + eps) * w64 + b64
    dx, dw, db = torch.autograd.grad(y, (x64, w64, b64), dy.double())
    return dx.float(), dw.float(), db.float()


def swiglu_bwd_ref(gate, up, dout):
    """(dgate, dup) by autograd through ``F.silu(gate) * up`` (float64 internally)."""
    g64, u64 = gate.double().requires_grad_(), up.double().requires_grad_()
    y = torch.nn.functional.silu(g64) * u64
    dg, du = torch.autograd.grad(y, (g64, u64), dout.double())
    return dg.float(), du.float()


def rel_fro(out: torch.Tensor, ref: torch.Tensor) -> float:
    """Relative Frobenius error ``|out-ref|_F / |ref|_F`` in float64."""
    o, r = out.double().cpu(), ref.double().cpu()
    return float((o - r).norm() / r.norm().clamp_min(1e-300))


def max_scaled_err(out: torch.Tensor, ref: torch.Tensor) -> float:
    """``max |out-ref| / max(|ref|, 1)``, the elementwise companion of ``rel_fro``."""
    o, r = out.double().cpu(), ref.double().cpu()
    return float(((o - r).abs() / r.abs().clamp_min(1.0)).max())
