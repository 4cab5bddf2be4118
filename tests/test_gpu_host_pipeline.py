"""HostPipeline: pinned host operands through upload / kernel / download streams.  Every call's
result must equal the direct call's, whatever the depth and however the slots are reused."""
import pytest
import torch

from oracle import formulas, inputs
from pyptx_b200.examples.blackwell.gemm_highperf_blackwell import build_gemm
from pyptx_b200.examples.blackwell.layer_norm import build_layer_norm
from pyptx_b200.host_pipeline import HostPipeline

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("depth", [1, 2, 3])
def test_pipelined_calls_equal_direct_calls(depth):
    M, N, K = 256, 512, 128
    kernel = build_gemm(M, N, K)
    pipe = HostPipeline(kernel, depth=depth)
    a0, bt = inputs.gemm_inputs(M, N, K)
    steps = 7
    a_host = [(a0.float() * (i + 1)).to(torch.bfloat16).pin_memory() for i in range(steps)]
    bt_pin = bt.pin_memory()
    outs = [torch.empty(M, N, dtype=torch.float32).pin_memory() for _ in range(steps)]
    tickets = [pipe.submit(a_host[i], bt_pin, out=outs[i]) for i in range(steps)]
    assert tickets == list(range(1, steps + 1))
    pipe.wait(tickets[2])
    assert formulas.rel_fro(outs[2], formulas.gemm_ref(a_host[2], bt)) < 1e-4
    pipe.wait()
    for i in range(steps):
        direct = kernel(a_host[i].cuda(), bt.cuda()).cpu()
        assert torch.equal(outs[i], direct)


def test_multiple_outputs_and_validation():
    B, N = 64, 1024
    kernel = build_layer_norm(B, N)
    x, w, b = inputs.layer_norm_inputs(B, N)
    pipe = HostPipeline(kernel)
    y = torch.empty(B, N).pin_memory()
    pipe.submit(x.pin_memory(), w.pin_memory(), b.pin_memory(), out=[y])
    pipe.join()
    torch.cuda.current_stream().synchronize()
    assert formulas.rel_fro(y, formulas.layer_norm_ref(x, w, b)) < 1e-5
    with pytest.raises(ValueError, match="pinned"):
        pipe.submit(x, w.pin_memory(), b.pin_memory(), out=y)
    with pytest.raises(ValueError, match="outputs"):
        pipe.submit(x.pin_memory(), w.pin_memory(), b.pin_memory(), out=[y, y.clone().pin_memory()])
    with pytest.raises(ValueError, match="depth"):
        HostPipeline(kernel, depth=0)
    with pytest.raises(ValueError, match="ticket"):
        pipe.wait(99)
