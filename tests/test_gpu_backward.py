"""GPU parity of the backward row kernels against autograd through the oracle's forward formulas,
and the forward/backward pairs under torch.autograd via differentiable_kernel."""
import pytest
import torch

from oracle import formulas, inputs
from pyptx_b200 import differentiable_kernel
from pyptx_b200.examples.blackwell.backward import (build_fused_silu_mul_bwd, build_layer_norm_bwd,
                                                    build_rms_norm_bwd)
from pyptx_b200.examples.blackwell.layer_norm import build_layer_norm
from pyptx_b200.examples.blackwell.rms_norm import build_rms_norm
from pyptx_b200.examples.blackwell.swiglu import build_fused_silu_mul

pytestmark = pytest.mark.gpu

SHAPES = [(1, 4), (4, 64), (16, 512), (33, 1000), (128, 2048), (256, 4096), (700, 8192), (5, 16384)]
TOL = 2e-5      # f32 kernels against a float64 evaluation; dw sums up to thousands of rows


def _dy(B, N, seed=5):
    g = torch.Generator().manual_seed(seed * 7919 + B * 31 + N)
    return torch.randn(B, N, generator=g)


@pytest.mark.parametrize("B,N", SHAPES)
def test_rms_norm_backward(B, N):
    x, w = inputs.rms_norm_inputs(B, N)
    dy = _dy(B, N)
    k = build_rms_norm_bwd(B, N)
    assert k.scratch_bytes > 0
    dx, dw = k(x.cuda(), w.cuda(), dy.cuda())
    rdx, rdw = formulas.rms_norm_bwd_ref(x, w, dy)
    assert formulas.rel_fro(dx.cpu(), rdx) < TOL and formulas.rel_fro(dw.cpu(), rdw) < TOL


@pytest.mark.parametrize("B,N", SHAPES)
def test_layer_norm_backward(B, N):
    x, w, _ = inputs.layer_norm_inputs(B, N)
    x = x * 2.0 - 1.0
    dy = _dy(B, N, 6)
    dx, dw, db = build_layer_norm_bwd(B, N)(x.cuda(), w.cuda(), dy.cuda())
    rdx, rdw, rdb = formulas.layer_norm_bwd_ref(x, w, dy)
    if N > 4:
        assert formulas.rel_fro(dx.cpu(), rdx) < 2e-4      # dx of a near-degenerate row amplifies rounding
    assert formulas.rel_fro(dw.cpu(), rdw) < TOL and formulas.rel_fro(db.cpu(), rdb) < TOL


@pytest.mark.parametrize("M,F", SHAPES + [(3, 70000)])
def test_swiglu_backward(M, F):
    g, u = inputs.swiglu_inputs(M, F)
    do = _dy(M, F, 7)
    k = build_fused_silu_mul_bwd(M, F)
    assert k.scratch_bytes == 0
    dg, du = k(g.cuda(), u.cuda(), do.cuda())
    rdg, rdu = formulas.swiglu_bwd_ref(g, u, do)
    assert formulas.rel_fro(dg.cpu(), rdg) < 1e-5 and formulas.rel_fro(du.cpu(), rdu) < 1e-5


def test_full_size_backward_is_deterministic():
    B, N = 2048, 8192
    x, w = inputs.rms_norm_inputs(B, N)
    dy = _dy(B, N)
    k = build_rms_norm_bwd(B, N)
    xc, wc, dc = x.cuda(), w.cuda(), dy.cuda()
    dx1, dw1 = k(xc, wc, dc)
    dx2, dw2 = k(xc, wc, dc)
    assert torch.equal(dx1, dx2) and torch.equal(dw1, dw2)       # no atomics: bit-identical runs
    rdx, rdw = formulas.rms_norm_bwd_ref(x, w, dy)
    assert formulas.rel_fro(dx1.cpu(), rdx) < TOL and formulas.rel_fro(dw1.cpu(), rdw) < TOL


def test_autograd_pairs():
    B, N = 64, 1024
    x, w, b = inputs.layer_norm_inputs(B, N)
    rms = differentiable_kernel(build_rms_norm(B, N), build_rms_norm_bwd(B, N))
    xg, wg = x.cuda().requires_grad_(), w.cuda().requires_grad_()
    rms(xg, wg).square().sum().backward()
    x2, w2 = x.cuda().requires_grad_(), w.cuda().requires_grad_()
    (x2 * torch.rsqrt((x2 * x2).mean(-1, keepdim=True) + 1e-6) * w2).square().sum().backward()
    torch.testing.assert_close(xg.grad, x2.grad, rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(wg.grad, w2.grad, rtol=1e-4, atol=1e-4)

    ln_fwd, ln_bwd = build_layer_norm(B, N), build_layer_norm_bwd(B, N)
    # forward takes (x, w, b); backward takes (x, w, dy) and yields (dx, dw, db)
    ln = differentiable_kernel(ln_fwd, lambda xs, ws, dy: ln_bwd(xs, ws, dy), save_for_backward=[0, 1])
    xg, wg, bg = (t.cuda().requires_grad_() for t in (x, w, b))
    ln(xg, wg, bg).sin().sum().backward()
    x2, w2, b2 = (t.cuda().requires_grad_() for t in (x, w, b))
    torch.nn.functional.layer_norm(x2, (N,), w2, b2, 1e-5).sin().sum().backward()
    torch.testing.assert_close(xg.grad, x2.grad, rtol=1e-3, atol=1e-5)
    torch.testing.assert_close(wg.grad, w2.grad, rtol=1e-4, atol=1e-4)
    torch.testing.assert_close(bg.grad, b2.grad, rtol=1e-4, atol=1e-4)

    sw = differentiable_kernel(build_fused_silu_mul(B, N), build_fused_silu_mul_bwd(B, N))
    g, u = (t.cuda().requires_grad_() for t in inputs.swiglu_inputs(B, N))
    sw(g, u).sum().backward()
    g2, u2 = (t.detach().clone().requires_grad_() for t in (g, u))
    (torch.nn.functional.silu(g2) * u2).sum().backward()
    torch.testing.assert_close(g.grad, g2.grad, rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(u.grad, u2.grad, rtol=1e-4, atol=1e-5)


def test_backward_under_cuda_graph():
    """The per-call scratch comes from the caching allocator, so capture and replay work."""
    B, N = 128, 2048
    x, w = inputs.rms_norm_inputs(B, N)
    dy = _dy(B, N)
    k = build_rms_norm_bwd(B, N)
    xc, wc, dc = x.cuda(), w.cuda(), dy.cuda()
    k(xc, wc, dc)
    torch.cuda.synchronize()
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        dx, dw = k(xc, wc, dc)
    dc.mul_(2.0)
    g.replay()
    torch.cuda.synchronize()
    rdx, rdw = formulas.rms_norm_bwd_ref(x, w, dy * 2.0)
    assert formulas.rel_fro(dx.cpu(), rdx) < TOL and formulas.rel_fro(dw.cpu(), rdw) < TOL
