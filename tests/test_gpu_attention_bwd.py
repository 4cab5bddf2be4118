"""GPU parity of the flash-attention backward kernel: dQ, dK, dV against float64 autograd through
the oracle's attention formula, on the forward's shape list (both head dims, causal and not,
ragged lengths, narrow heads), through ``differentiable_kernel``, and on the benchmark
configuration with sampled heads."""
import pytest
import torch

from oracle import formulas, inputs
from pyptx_b200.examples.blackwell.flash_attention import (build_differentiable_flash_attention,
                                                           build_flash_attention, build_flash_attention_bwd)
from pyptx_b200.types import bf16, f32

pytestmark = pytest.mark.gpu

TOL = 1e-2      # relative Frobenius error per gradient (bf16 operands, P and dS rounded to bf16)


def _inputs(B, H, Sq, Skv, d, seed=11):
    q, k, v = inputs.attention_inputs(B * H, Sq, Skv, d)
    g = torch.Generator().manual_seed(seed + Sq + 7 * Skv + d)
    do = torch.randn(B, H, Sq, d, generator=g).to(torch.bfloat16)
    return q.view(B, H, Sq, d), k.view(B, H, Skv, d), v.view(B, H, Skv, d), do


def _run(q, k, v, do, *, causal, out_dtype=f32, sm_scale=None, deterministic=False):
    B, H, Sq, d = q.shape
    Skv = k.shape[2]
    fwd = build_flash_attention(B, H, Sq, Skv, d, causal=causal, sm_scale=sm_scale, out_dtype=bf16, return_lse=True)
    bwd = build_flash_attention_bwd(B, H, Sq, Skv, d, causal=causal, sm_scale=sm_scale, out_dtype=out_dtype,
                                    deterministic=deterministic)
    qc, kc, vc = q.cuda(), k.cuda(), v.cuda()
    o, lse = fwd(qc, kc, vc)
    dq, dk, dv = bwd(qc, kc, vc, o, lse, do.cuda())
    return dq.cpu(), dk.cpu(), dv.cpu()


def _check(got, ref, tol=TOL):
    # A gradient that is exactly zero in the reference (one visible key: P = 1, dS = 0) is measured
    # against the largest of the three reference norms instead of its own.
    floor = 1e-2 * max(float(r.norm()) for r in ref)
    for name, g, r in zip(("dq", "dk", "dv"), got, ref):
        assert g.shape == r.shape, (name, g.shape, r.shape)
        assert torch.isfinite(g.float()).all(), name
        err = float((g.float() - r).norm()) / max(float(r.norm()), floor, 1e-30)
        assert err < tol, f"{name}: rel_fro {err:.3e}"


DETERMINISTIC = pytest.mark.parametrize("deterministic", [False, True], ids=["fused", "two_pass"])


@DETERMINISTIC
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("B,H,Sq,Skv", [(1, 1, 128, 128), (2, 3, 256, 256), (1, 2, 384, 384), (2, 2, 512, 1024),
                                        (1, 4, 1024, 1024), (1, 1, 128, 640)])
def test_batched(B, H, Sq, Skv, d, causal, deterministic):
    q, k, v, do = _inputs(B, H, Sq, Skv, d)
    _check(_run(q, k, v, do, causal=causal, deterministic=deterministic),
           formulas.attention_bwd_ref(q, k, v, do, causal=causal))


@DETERMINISTIC
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("Sq,Skv", [(1, 1), (5, 40), (100, 100), (129, 300), (200, 513), (257, 257), (383, 1000)])
def test_ragged_sequence_lengths(Sq, Skv, d, causal, deterministic):
    """Lengths that are not multiples of the 128-wide tiles: zero-filled partial tiles; padding
    queries carry lse = +inf (P = 0), padding keys multiply zero rows of K and V."""
    q, k, v, do = _inputs(1, 3, Sq, Skv, d)
    _check(_run(q, k, v, do, causal=causal, deterministic=deterministic), formulas.attention_bwd_ref(q, k, v, do, causal=causal))


@DETERMINISTIC
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("d", [8, 32, 72, 120])
def test_head_dims_narrower_than_the_tile(d, causal, deterministic):
    q, k, v, do = _inputs(2, 2, 200, 328, d)
    _check(_run(q, k, v, do, causal=causal, deterministic=deterministic), formulas.attention_bwd_ref(q, k, v, do, causal=causal))


@DETERMINISTIC
@pytest.mark.parametrize("d", [64, 128])
def test_causal_head_groups_with_a_partial_last_group(d, deterministic):
    """Causal launches deal the stationary tiles out heaviest-first across groups of 16 heads; 21
    heads leave a last group of 5, and 600 rows a partial last tile."""
    q, k, v, do = _inputs(3, 7, 600, 600, d)
    _check(_run(q, k, v, do, causal=True, deterministic=deterministic),
           formulas.attention_bwd_ref(q, k, v, do, causal=True))


@DETERMINISTIC
def test_bf16_gradients_and_scale(deterministic):
    q, k, v, do = _inputs(2, 2, 256, 256, 128)
    got = _run(q, k, v, do, causal=True, out_dtype=bf16, sm_scale=0.05, deterministic=deterministic)
    assert all(g.dtype == torch.bfloat16 for g in got)
    _check(got, formulas.attention_bwd_ref(q, k, v, do, causal=True, sm_scale=0.05))


@DETERMINISTIC
def test_one_hot_attention_gradients(deterministic):
    """Sharp scores (each query attends to one key): dV is a permutation of dO and dQ, dK vanish
    up to the softmax's saturation, which pins the pairing of queries and keys in both passes."""
    B, H, S, d = 1, 1, 256, 64
    g = torch.Generator().manual_seed(3)
    k = torch.randn(B, H, S, d, generator=g)
    k = (k / k.norm(dim=-1, keepdim=True)).to(torch.bfloat16)
    perm = torch.randperm(S, generator=g)
    q = (k.float()[:, :, perm] * 200.0).to(torch.bfloat16)
    v = torch.randn(B, H, S, d, generator=g).to(torch.bfloat16)
    do = torch.randn(B, H, S, d, generator=g).to(torch.bfloat16)
    dq, dk, dv = _run(q, k, v, do, causal=False, sm_scale=1.0, deterministic=deterministic)
    ref = formulas.attention_bwd_ref(q, k, v, do, sm_scale=1.0)
    assert formulas.rel_fro(dv, ref[2]) < TOL
    inv = torch.empty_like(perm)
    inv[perm] = torch.arange(S)
    assert formulas.rel_fro(dv, do.float()[:, :, inv]) < 2e-2
    assert dq.abs().max() < 1e-2 * do.float().abs().max() and dk.abs().max() < 1e-2 * 200.0 * do.float().abs().max()


def test_differentiable_attention_through_autograd():
    """``build_differentiable_flash_attention``: forward + backward kernels joined by
    ``differentiable_kernel``; gradients land in ``.grad`` with the inputs' dtype."""
    B, H, S, d = 2, 2, 384, 64
    q, k, v, do = _inputs(B, H, S, S, d)
    attn = build_differentiable_flash_attention(B, H, S, S, d, causal=True)
    qc, kc, vc = (t.cuda().requires_grad_() for t in (q, k, v))
    o = attn(qc, kc, vc)
    assert o.dtype == torch.bfloat16 and o.requires_grad
    (o.float() * do.cuda().float()).sum().backward()
    ref = formulas.attention_bwd_ref(q, k, v, do, causal=True)
    for name, t, r in zip(("dq", "dk", "dv"), (qc, kc, vc), ref):
        assert t.grad is not None and t.grad.dtype == torch.bfloat16, name
        assert formulas.rel_fro(t.grad.float().cpu(), r) < TOL, name


@DETERMINISTIC
@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("d", [64, 128])
def test_benchmark_configuration(d, causal, deterministic):
    """B=4, H=16, S=4096 on all 64 heads; float64 autograd on a sample of them."""
    B, H, S = 4, 16, 4096
    q, k, v, do = _inputs(B, H, S, S, d)
    dq, dk, dv = _run(q, k, v, do, causal=causal, out_dtype=bf16, deterministic=deterministic)
    for t in (dq, dk, dv):
        assert torch.isfinite(t.float()).all()
    for b, h in [(0, 0), (3, 15)]:
        ref = formulas.attention_bwd_ref(q[b, h], k[b, h], v[b, h], do[b, h], causal=causal)
        _check((dq[b, h], dk[b, h], dv[b, h]), ref)


def test_two_pass_form_is_bit_reproducible_and_fused_dk_dv_too():
    """The two-pass form uses no atomics: two runs agree bit for bit.  In the fused form only dQ is
    accumulated with atomics; dK and dV come from the same MMAs in the same order."""
    q, k, v, do = _inputs(2, 2, 640, 640, 128)
    a = _run(q, k, v, do, causal=True, deterministic=True)
    b = _run(q, k, v, do, causal=True, deterministic=True)
    assert all(torch.equal(x, y) for x, y in zip(a, b))
    c = _run(q, k, v, do, causal=True)
    d = _run(q, k, v, do, causal=True)
    assert torch.equal(c[1], d[1]) and torch.equal(c[2], d[2])
    assert formulas.rel_fro(c[0], a[0]) < 1e-3


@pytest.mark.parametrize("d", [64, 128])
def test_fused_backward_replays_from_a_cuda_graph(d):
    """The fused form clears its fp32 dQ accumulator inside the call (a memset node in the graph), so a
    replay must give the gradients of the inputs as they are at replay time, every time."""
    B, H, S = 1, 3, 384
    q, k, v, do = _inputs(B, H, S, S, d)
    fwd = build_flash_attention(B, H, S, S, d, causal=True, return_lse=True)
    bwd = build_flash_attention_bwd(B, H, S, S, d, causal=True, out_dtype=f32)
    qc, kc, vc, dc = q.cuda(), k.cuda(), v.cuda(), do.cuda()
    o, lse = fwd(qc, kc, vc)
    bwd(qc, kc, vc, o, lse, dc)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        dq, dk, dv = bwd(qc, kc, vc, o, lse, dc)
    for scale in (2.0, -0.5):
        dc.copy_(do.cuda() * scale)
        g.replay()
        torch.cuda.synchronize()
        # delta = rowsum(O o dO) scales with dO, so all three gradients are linear in dO
        ref = formulas.attention_bwd_ref(q, k, v, (do.float() * scale).to(torch.bfloat16), causal=True)
        _check((dq.cpu(), dk.cpu(), dv.cpu()), ref)


def test_no_device_wait_gave_up():
    from pyptx_b200 import _native
    _native.device_status()
