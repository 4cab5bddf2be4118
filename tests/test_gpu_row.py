"""GPU parity of the f32 row kernels (RMSNorm, LayerNorm, SwiGLU, softmax) against the CPU
oracle: the golden vectors, the reference's example shape lists and seeds
(examples/blackwell/rms_norm.py:73, swiglu.py:76-83), ragged / edge shapes, and the
full-size benchmark configurations, all through the public build_* entry points."""
import os

import numpy as np
import pytest
import torch

from oracle import formulas, inputs
from pyptx_b200.examples.blackwell.layer_norm import build_layer_norm
from pyptx_b200.examples.blackwell.rms_norm import build_rms_norm
from pyptx_b200.examples.blackwell.softmax import build_softmax
from pyptx_b200.examples.blackwell.swiglu import build_fused_silu_mul
from tests.gpu_util import check_f32

pytestmark = pytest.mark.gpu

REF_SHAPES = [(4, 64), (16, 512), (32, 1024), (128, 2048), (256, 4096)]
EDGE_SHAPES = [(1, 4), (3, 36), (5, 132), (7, 1000), (2, 8192), (3, 12288), (2, 32768), (1, 65536), (2, 70000)]


@pytest.fixture(scope="module")
def rows(golden_dir):
    return np.load(os.path.join(golden_dir, "row_refs.npz"))


def _cuda(*ts):
    return [t.cuda() for t in ts]


@pytest.mark.parametrize("B,N", [(4, 64), (16, 512)])
def test_golden_vectors(rows, B, N):
    x, w = _cuda(torch.from_numpy(rows[f"rms_{B}_{N}_x"]), torch.from_numpy(rows[f"rms_{B}_{N}_w"]))
    check_f32(build_rms_norm(B, N)(x, w).cpu(), torch.from_numpy(rows[f"rms_{B}_{N}_y"]))
    x, w, b = _cuda(*(torch.from_numpy(rows[f"ln_{B}_{N}_{k}"]) for k in "xwb"))
    check_f32(build_layer_norm(B, N)(x, w, b).cpu(), torch.from_numpy(rows[f"ln_{B}_{N}_y"]))
    g, u = _cuda(torch.from_numpy(rows[f"swiglu_{B}_{N}_g"]), torch.from_numpy(rows[f"swiglu_{B}_{N}_u"]))
    check_f32(build_fused_silu_mul(B, N)(g, u).cpu(), torch.from_numpy(rows[f"swiglu_{B}_{N}_y"]))
    (x,) = _cuda(torch.from_numpy(rows[f"softmax_{B}_{N}_x"]))
    check_f32(build_softmax(B, N)(x).cpu(), torch.from_numpy(rows[f"softmax_{B}_{N}_y"]))


@pytest.mark.parametrize("B,N", REF_SHAPES + EDGE_SHAPES)
def test_rms_norm(B, N):
    x, w = inputs.rms_norm_inputs(B, N)
    out = build_rms_norm(B, N)(*_cuda(x, w))
    check_f32(out.cpu(), formulas.rms_norm_ref(x, w))


@pytest.mark.parametrize("B,N", REF_SHAPES + EDGE_SHAPES)
def test_layer_norm(B, N):
    x, w, b = inputs.layer_norm_inputs(B, N)
    x = x * 2.0 - 1.0  # non-zero mean, as the reference's self-test (examples/blackwell/layer_norm.py:65)
    out = build_layer_norm(B, N)(*_cuda(x, w, b))
    check_f32(out.cpu(), formulas.layer_norm_ref(x, w, b))


def test_layer_norm_large_offset():
    """mean >> std: the case where E[x^2]-mean^2 loses digits; the kernel must not."""
    x, w, b = inputs.layer_norm_inputs(8, 4096)
    x = x * 0.01 + 100.0
    out = build_layer_norm(8, 4096)(*_cuda(x, w, b))
    ref = formulas.layer_norm_ref(x.double(), w.double(), b.double()) if False else formulas.layer_norm_ref(x, w, b)
    assert formulas.rel_fro(out.cpu(), ref) < 1e-3


@pytest.mark.parametrize("M,F", REF_SHAPES + [(512, 8192)] + EDGE_SHAPES)
def test_swiglu(M, F):
    g, u = inputs.swiglu_inputs(M, F)
    out = build_fused_silu_mul(M, F)(*_cuda(g, u))
    check_f32(out.cpu(), formulas.swiglu_ref(g, u))


def test_swiglu_extreme_gates():
    g = torch.tensor([[-100.0, -30.0, -1.0, 0.0, 1.0, 30.0, 100.0, 88.0]]).repeat(4, 1)
    u = torch.full_like(g, 2.0)
    out = build_fused_silu_mul(4, 8)(*_cuda(g, u)).cpu()
    assert torch.isfinite(out).all()
    check_f32(out, formulas.swiglu_ref(g, u))


@pytest.mark.parametrize("B,N", REF_SHAPES + EDGE_SHAPES)
def test_softmax(B, N):
    (x,) = inputs.softmax_inputs(B, N)
    out = build_softmax(B, N)(x.cuda()).cpu()
    check_f32(out, formulas.softmax_ref(x))
    torch.testing.assert_close(out.sum(-1), torch.ones(B), rtol=2e-5, atol=2e-5)


def test_softmax_shift_invariance_and_large_values():
    (x,) = inputs.softmax_inputs(16, 2048)
    k = build_softmax(16, 2048)
    a = k(x.cuda()).cpu()
    b = k((x + 1000.0).cuda()).cpu()
    assert torch.isfinite(b).all()
    torch.testing.assert_close(a, b, rtol=1e-3, atol=1e-6)


# ---- full-size benchmark configurations (2048 x 8192 f32) ----------------------

def test_full_size_rms_norm():
    x, w = inputs.rms_norm_inputs()
    out = build_rms_norm(2048, 8192)(*_cuda(x, w))
    check_f32(out.cpu(), formulas.rms_norm_ref(x, w))


def test_full_size_layer_norm():
    x, w, b = inputs.layer_norm_inputs()
    out = build_layer_norm(2048, 8192)(*_cuda(x, w, b))
    check_f32(out.cpu(), formulas.layer_norm_ref(x, w, b))


def test_full_size_swiglu():
    g, u = inputs.swiglu_inputs()
    out = build_fused_silu_mul(2048, 8192)(*_cuda(g, u))
    check_f32(out.cpu(), formulas.swiglu_ref(g, u))


def test_full_size_softmax():
    (x,) = inputs.softmax_inputs()
    out = build_softmax(2048, 8192)(x.cuda())
    check_f32(out.cpu(), formulas.softmax_ref(x))


# ---- fused bf16 output (extension) --------------------------------------------------

@pytest.mark.parametrize("B,N", [(16, 512), (5, 132), (64, 8192), (2, 70000)])
def test_bf16_output_is_the_rounded_f32_result(B, N):
    """out_dtype=bf16 gives exactly the round-to-nearest bf16 of the kernel's own f32 result."""
    from pyptx_b200.types import bf16
    x, w, b = inputs.layer_norm_inputs(B, N)
    g, u = inputs.swiglu_inputs(B, N)
    xc, wc, bc, gc, uc = _cuda(x, w, b, g, u)
    pairs = [
        (build_rms_norm(B, N), build_rms_norm(B, N, out_dtype=bf16), (xc, wc)),
        (build_layer_norm(B, N), build_layer_norm(B, N, out_dtype=bf16), (xc, wc, bc)),
        (build_fused_silu_mul(B, N), build_fused_silu_mul(B, N, out_dtype=bf16), (gc, uc)),
        (build_softmax(B, N), build_softmax(B, N, out_dtype=bf16), (xc,)),
    ]
    for k32, k16, args in pairs:
        y32, y16 = k32(*args), k16(*args)
        assert y16.dtype == torch.bfloat16 and y16.shape == y32.shape
        assert torch.equal(y16, y32.to(torch.bfloat16)), k32.__name__


# ---- size-independent properties -------------------------------------------------

def test_rms_norm_scale_invariance():
    """rms_norm(c*x) == rms_norm(x) up to eps effects; output RMS per row equals RMS of w-scaled unit rows."""
    x, w = inputs.rms_norm_inputs(64, 4096)
    k = build_rms_norm(64, 4096, eps=0.0)
    a = k(*_cuda(x, w)).cpu()
    b = k(*_cuda(x * 8.0, w)).cpu()
    torch.testing.assert_close(a, b, rtol=1e-5, atol=1e-6)
    ones = torch.ones_like(w)
    y = k(*_cuda(x, ones)).cpu()
    torch.testing.assert_close((y * y).mean(-1), torch.ones(64), rtol=1e-5, atol=1e-5)


def test_inputs_are_not_modified_and_outputs_are_fresh():
    x, w = inputs.rms_norm_inputs(32, 1024)
    xc, wc = _cuda(x, w)
    k = build_rms_norm(32, 1024)
    y1, y2 = k(xc, wc), k(xc, wc)
    assert y1.data_ptr() != y2.data_ptr() and torch.equal(y1, y2)
    assert torch.equal(xc.cpu(), x) and torch.equal(wc.cpu(), w)
