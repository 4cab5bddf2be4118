"""The allocation-free RMSNorm backward entry point (pb200_rms_norm_bwd_static).

Who needs it: hosts that may not allocate device memory where they call the library -- a serving
process whose memory plan is fixed when the model is loaded, a plugin slot of a bigger engine that
is handed its tensors and nothing else -- and so cannot provide the scratch buffer that the regular
backward kernel asks its caller for.  This entry keeps its scratch in a fixed 4 MiB array inside
the library.

The test drives the entry straight through the C ABI (raw pointers, stream as an integer), twice
in a row with different data, and compares each result with the regular entry point on the same
inputs.  The second call matters: the built-in scratch still holds the first call's partial sums,
and none of them may leak into the second result.  The file name sorts last on purpose, so that a
run that stops at the first failure has already been through every other test; the test neither
relies on nor disturbs state left by the others.
"""
import ctypes

import pytest
import torch

from oracle import formulas, inputs
from pyptx_b200 import _ids, _native
from pyptx_b200.examples.blackwell.backward import build_rms_norm_bwd

pytestmark = pytest.mark.gpu

TOL = 2e-5      # same bound as the backward parity tests: f32 kernels, sums over thousands of rows


def _call_static(lib, x, w, dy, eps=1e-6):
    rows, cols = x.shape
    dx = torch.empty_like(x)
    dw = torch.empty_like(w)
    err = ctypes.create_string_buffer(_native.ERR_LEN)
    rc = lib.pb200_rms_norm_bwd_static(rows, cols, eps, torch.cuda.current_stream().cuda_stream,
                                       x.data_ptr(), w.data_ptr(), dy.data_ptr(), dx.data_ptr(), dw.data_ptr(), err)
    assert rc == 0, err.value.decode(errors="replace")
    return dx, dw


@pytest.mark.parametrize("rows,cols", [(2048, 8192), (300, 1000), (64, 16384)])
def test_static_scratch_entry_matches_the_regular_one_twice_in_a_row(rows, cols):
    lib = _native.load()
    regular = build_rms_norm_bwd(rows, cols)
    x, w = inputs.rms_norm_inputs(rows, cols)
    g = torch.Generator().manual_seed(rows * 31 + cols)
    for call in range(2):
        dy = torch.randn(rows, cols, generator=g) * (1.0 + 3.0 * call)     # new data for the second call
        xc, wc, dc = (x * (1.0 + call)).cuda(), w.cuda(), dy.cuda()
        dx_ref, dw_ref = regular(xc, wc, dc)
        dx, dw = _call_static(lib, xc, wc, dc)
        torch.cuda.synchronize()
        assert torch.isfinite(dx).all() and torch.isfinite(dw).all()
        # dx does not touch the scratch: identical arithmetic, identical bits
        assert torch.equal(dx, dx_ref)
        # dw is folded from a different number of partial rows, so only the summation order differs
        assert formulas.rel_fro(dw.cpu(), dw_ref.cpu()) < TOL
        o_dx, o_dw = formulas.rms_norm_bwd_ref(x * (1.0 + call), w, dy)
        assert formulas.rel_fro(dx.cpu(), o_dx) < TOL and formulas.rel_fro(dw.cpu(), o_dw) < TOL


def test_static_scratch_entry_rejects_what_it_cannot_hold():
    lib = _native.load()
    err = ctypes.create_string_buffer(_native.ERR_LEN)
    t = torch.zeros(64, device="cuda")
    p = t.data_ptr()
    stream = torch.cuda.current_stream().cuda_stream
    rc = lib.pb200_rms_norm_bwd_static(4, 16384 + 4, 1e-6, stream, p, p, p, p, p, err)
    assert rc == _ids.ERR_BAD_SHAPE and b"exceeds" in err.value and b"16384" in err.value
    rc = lib.pb200_rms_norm_bwd_static(4, 6, 1e-6, stream, p, p, p, p, p, err)
    assert rc == _ids.ERR_BAD_SHAPE
    rc = lib.pb200_rms_norm_bwd_static(4, 8, 1e-6, stream, p, p + 4, p, p, p, err)
    assert rc == _ids.ERR_MISALIGNED
    rc = lib.pb200_rms_norm_bwd_static(4, 8, 1e-6, stream, p, p, p, None, p, err)
    assert rc == _ids.ERR_MISALIGNED
