"""The PyTorch launch path on a GPU: eager (pybind11 extension and ctypes), torch.compile through
the registered custom op, CUDA-graph capture and replay, the autograd wrapper, stream ordering
and call-time validation.  Mirrors the reference's tests/test_torch_dispatch.py:38-204."""
import ctypes

import pytest
import torch

from oracle import formulas, inputs
from pyptx_b200 import _ids, _native, differentiable_kernel, torch_support
from pyptx_b200.examples.blackwell.gemm_highperf_blackwell import build_gemm
from pyptx_b200.examples.blackwell.layer_norm import build_layer_norm
from pyptx_b200.examples.blackwell.rms_norm import build_rms_norm
from pyptx_b200.examples.blackwell.softmax import build_softmax
from pyptx_b200.examples.blackwell.swiglu import build_fused_silu_mul
from tests.gpu_util import check_f32

pytestmark = pytest.mark.gpu


def test_native_library_is_the_loaded_path():
    lib = _native.load()
    assert lib.pb200_arch() == b"sm_100a"
    assert _native.load_torch_ext() is not None, "the in-tree pybind11 extension should be built and loadable"


def test_eager_ext_and_ctypes_paths_agree():
    x, w = inputs.rms_norm_inputs(16, 512)
    xc, wc = x.cuda(), w.cuda()
    k = build_rms_norm(16, 512)
    y_ext = k(xc, wc)
    launcher = k._launcher
    assert launcher.ext is not None
    launcher.ext = None               # force the ctypes path on the same kernel object
    try:
        y_ct = k(xc, wc)
    finally:
        launcher.ext = _native.load_torch_ext()
    assert torch.equal(y_ext, y_ct)
    check_f32(y_ext.cpu(), formulas.rms_norm_ref(x, w))


def test_raw_c_abi_call():
    """pb200_launch_raw with raw pointers and the stream as an integer, as a non-Python host would call it."""
    lib = _native.load()
    x, w = inputs.rms_norm_inputs(8, 256)
    xc, wc = x.cuda(), w.cuda()
    y = torch.empty_like(xc)
    h = _native.create_handle(_ids.K_RMS_NORM, (8, 256), (1e-6,))
    ptrs = (ctypes.c_void_p * 3)(xc.data_ptr(), wc.data_ptr(), y.data_ptr())
    err = ctypes.create_string_buffer(_native.ERR_LEN)
    rc = lib.pb200_launch_raw(h, torch.cuda.current_stream().cuda_stream, ptrs, 3, err)
    assert rc == 0, err.value
    torch.cuda.synchronize()
    check_f32(y.cpu(), formulas.rms_norm_ref(x, w))
    assert lib.pb200_device_status(err) == 0
    lib.pb200_destroy(h)


def test_raw_c_abi_call_rejects_memory_the_gpu_cannot_reach():
    """The first launch of a handle looks at where its buffers live: pageable host memory is
    refused with a code and a message, before any kernel could fault on it."""
    import numpy as np

    lib = _native.load()
    x, w = inputs.rms_norm_inputs(8, 256)
    xc, wc = x.cuda(), w.cuda()
    host = np.zeros(8 * 256 + 8, dtype=np.float32)
    addr = (host.ctypes.data + 15) & ~15            # the entry point also wants 16-byte alignment
    h = _native.create_handle(_ids.K_RMS_NORM, (8, 256), (1e-6,))
    ptrs = (ctypes.c_void_p * 3)(xc.data_ptr(), wc.data_ptr(), addr)
    err = ctypes.create_string_buffer(_native.ERR_LEN)
    rc = lib.pb200_launch_raw(h, torch.cuda.current_stream().cuda_stream, ptrs, 3, err)
    assert rc == _ids.ERR_WRONG_DEVICE and b"not device-accessible" in err.value
    # the same handle with proper buffers still works
    y = torch.empty_like(xc)
    ptrs = (ctypes.c_void_p * 3)(xc.data_ptr(), wc.data_ptr(), y.data_ptr())
    assert lib.pb200_launch_raw(h, torch.cuda.current_stream().cuda_stream, ptrs, 3, err) == 0, err.value
    torch.cuda.synchronize()
    check_f32(y.cpu(), formulas.rms_norm_ref(x, w))
    lib.pb200_destroy(h)


def test_torch_compile_through_custom_op():
    x, w = inputs.rms_norm_inputs(16, 512)
    k = build_rms_norm(16, 512)

    @torch.compile(fullgraph=True)
    def f(a, b):
        return k(a * 2.0, b) + 1.0

    out = f(x.cuda(), w.cuda())
    ref = formulas.rms_norm_ref(x * 2.0, w) + 1.0
    check_f32(out.cpu(), ref)
    assert k.handle in torch_support._REGISTERED_OPS


def test_torch_compile_matrix_kernels():
    """GEMM, grouped GEMM and attention inside ``torch.compile(fullgraph=True)`` graphs, next to
    ordinary torch ops (the reference compiles a grouped GEMM and an attention call the same way,
    tests/test_torch_dispatch.py:161-204)."""
    from pyptx_b200.examples.blackwell.flash_attention import build_flash_attention
    from pyptx_b200.examples.blackwell.grouped_gemm import build_grouped_gemm
    from pyptx_b200.types import f32

    a, bt = inputs.gemm_inputs(256, 256, 128)
    kg = build_gemm(256, 256, 128)

    @torch.compile(fullgraph=True)
    def f_gemm(x, y):
        return torch.relu(kg(x, y)) * 0.5

    ref = torch.relu(formulas.gemm_ref(a, bt)) * 0.5
    assert formulas.rel_fro(f_gemm(a.cuda(), bt.cuda()).cpu(), ref) < 1e-4

    G, M, N, K = 2, 128, 256, 128
    ga, gb = inputs.grouped_gemm_inputs(G, M, N, K)
    kgg = build_grouped_gemm(G, M, N, K)

    @torch.compile(fullgraph=True)
    def f_grouped(x, y):
        return kgg(x, y) + 1.0

    assert formulas.rel_fro(f_grouped(ga.cuda(), gb.cuda()).cpu(), formulas.grouped_gemm_ref(ga, gb, G) + 1.0) < 1e-4

    q, k, v = (t.view(1, 2, 256, 64) for t in inputs.attention_inputs(2, 256, 256, 64))
    ka = build_flash_attention(1, 2, 256, 256, 64, causal=True, out_dtype=f32)

    @torch.compile(fullgraph=True)
    def f_attn(qq, kk, vv):
        return ka(qq, kk, vv) * 2.0

    ref = formulas.attention_ref(q, k, v, causal=True) * 2.0
    assert formulas.rel_fro(f_attn(q.cuda(), k.cuda(), v.cuda()).cpu(), ref) < 1e-2
    for kern in (kg, kgg, ka):
        assert kern.handle in torch_support._REGISTERED_OPS


def test_custom_op_fake_shapes():
    k = build_gemm(256, 256, 128)
    op = torch_support.get_or_register_torch_op(k)
    from torch._subclasses.fake_tensor import FakeTensorMode
    with FakeTensorMode():
        a = torch.empty(256, 128, dtype=torch.bfloat16, device="cuda")
        b = torch.empty(256, 128, dtype=torch.bfloat16, device="cuda")
        (d,) = op([a, b])
        assert d.shape == (256, 256) and d.dtype == torch.float32 and d.device.type == "cuda"


def test_compile_swiglu_layernorm_softmax():
    g, u = inputs.swiglu_inputs(32, 1024)
    x, w, b = inputs.layer_norm_inputs(32, 1024)
    ks, kl, km = build_fused_silu_mul(32, 1024), build_layer_norm(32, 1024), build_softmax(32, 1024)

    @torch.compile
    def f(g, u, x, w, b):
        return km(kl(ks(g, u) + x, w, b))

    out = f(*(t.cuda() for t in (g, u, x, w, b))).cpu()
    ref = formulas.softmax_ref(formulas.layer_norm_ref(formulas.swiglu_ref(g, u) + x, w, b))
    check_f32(out, ref, tol=2e-5)


def test_cuda_graph_capture_and_replay():
    x, w = inputs.rms_norm_inputs(64, 2048)
    a, bt = inputs.gemm_inputs(256, 256, 256)
    k_rms, k_gemm = build_rms_norm(64, 2048), build_gemm(256, 256, 256)
    xs, ws, as_, bts = x.cuda(), w.cuda(), a.cuda(), bt.cuda()
    k_rms(xs, ws); k_gemm(as_, bts)            # warm-up outside capture (first-call set-up)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        y = k_rms(xs, ws)
        d = k_gemm(as_, bts)
    for scale in (1.0, 3.0):
        xs.copy_((x * scale).cuda())
        as_.copy_((a.float() * scale).to(torch.bfloat16).cuda())
        graph.replay()
        torch.cuda.synchronize()
        check_f32(y.cpu(), formulas.rms_norm_ref(x * scale, w))
        ref = formulas.gemm_ref((a.float() * scale).to(torch.bfloat16), bt)
        assert formulas.rel_fro(d.cpu(), ref) < 1e-4
    _native.device_status()


def test_stream_ordering():
    """The launch is enqueued on the caller's current stream: work queued before it on that
    stream is visible, and no other stream is touched."""
    k = build_rms_norm(64, 4096)
    x, w = inputs.rms_norm_inputs(64, 4096)
    s = torch.cuda.Stream()
    wc = w.cuda()
    torch.cuda.synchronize()
    with torch.cuda.stream(s):
        xs = torch.empty(64, 4096, device="cuda")
        for _ in range(20):
            xs.zero_()
        xs.copy_(x.cuda(), non_blocking=True)
        y = k(xs, wc)
    s.synchronize()
    check_f32(y.cpu(), formulas.rms_norm_ref(x, w))


def test_differentiable_kernel_wrapper():
    """Forward kernel + a backward callable through torch.autograd (the backward here is the
    analytic SwiGLU gradient in torch; backward kernels are outside this library's scope)."""
    M, F = 16, 256
    fwd = build_fused_silu_mul(M, F)

    def bwd(g, u, grad_out):
        sig = torch.sigmoid(g)
        return grad_out * u * (sig * (1 + g * (1 - sig))), grad_out * g * sig

    op = differentiable_kernel(fwd, bwd)
    g, u = (t.cuda().requires_grad_() for t in inputs.swiglu_inputs(M, F))
    out = op(g, u)
    out.sum().backward()
    g2, u2 = (t.detach().clone().requires_grad_() for t in (g, u))
    (torch.nn.functional.silu(g2) * u2).sum().backward()
    torch.testing.assert_close(g.grad, g2.grad, rtol=1e-4, atol=1e-5)
    torch.testing.assert_close(u.grad, u2.grad, rtol=1e-4, atol=1e-5)
    assert op.forward_kernel is fwd


def test_call_time_validation():
    k = build_rms_norm(16, 512)
    x, w = (t.cuda() for t in inputs.rms_norm_inputs(16, 512))
    with pytest.raises(TypeError, match="expected 2 input arrays, got 1"):
        k(x)
    with pytest.raises(ValueError, match="dim mismatch"):
        k(x[:8].contiguous(), w)
    with pytest.raises(TypeError, match="dtype"):
        k(x.double(), w)
    with pytest.raises(ValueError, match="not contiguous"):
        k(x.t().contiguous().t(), w)
    with pytest.raises(ValueError, match="CUDA tensors"):
        k(x.cpu(), w.cpu())
    with pytest.raises(TypeError):
        k([1, 2], w)
    kg = build_gemm(128, 256, 64)
    with pytest.raises(TypeError, match="dtype"):
        kg(torch.zeros(128, 64, device="cuda"), torch.zeros(256, 64, device="cuda"))


def test_misaligned_view_is_rejected_by_the_c_abi():
    k = build_rms_norm(4, 64)
    base = torch.zeros(4 * 64 + 1, device="cuda")
    x = base[1:].view(4, 64)                      # 4-byte offset: not 16-byte aligned
    with pytest.raises(RuntimeError, match="code -10"):
        k(x, torch.ones(64, device="cuda"))


def test_dispatch_overhead_is_reported(capsys):
    """Host-side cost of one eager call (not asserted tightly; the figure is printed for the log)."""
    import time
    k = build_rms_norm(4, 64)
    x, w = torch.zeros(4, 64, device="cuda"), torch.ones(64, device="cuda")
    for _ in range(200):
        k(x, w)
    torch.cuda.synchronize()
    t0 = time.perf_counter()
    n = 2000
    for _ in range(n):
        k(x, w)
    host_us = (time.perf_counter() - t0) / n * 1e6
    torch.cuda.synchronize()
    print(f"eager dispatch: {host_us:.1f} us per call (ext={'yes' if k._launcher.ext else 'no'})")
    assert host_us < 200


@pytest.mark.parametrize("path", ["pybind11", "ctypes"])
def test_concurrent_launches_from_threads_on_their_own_streams(path):
    """Host threads launch kernels at once (two threads per kernel), each on its own stream: the
    launch path (handle lookup under a shared lock, per-launch tensor maps, per-thread pointer
    arrays and error buffers, one-time function attributes) must give every thread its own correct
    results, through the pybind11 extension and through plain ctypes."""
    import threading

    from oracle import formulas, inputs
    from pyptx_b200.examples.blackwell.flash_attention import build_flash_attention
    from pyptx_b200.examples.blackwell.gemm_highperf_blackwell import build_gemm, build_gemm_2sm
    from pyptx_b200.examples.blackwell.rms_norm import build_rms_norm
    from pyptx_b200.examples.blackwell.softmax import build_softmax
    from pyptx_b200.types import f32

    a, bt = inputs.gemm_inputs(512, 512, 256)
    x, w = inputs.rms_norm_inputs(256, 2048)
    q, k, v = (t.view(1, 2, 256, 64) for t in inputs.attention_inputs(2, 256, 256, 64))
    jobs = {
        "gemm_1sm": (build_gemm(512, 512, 256), (a.cuda(), bt.cuda()), formulas.gemm_ref(a, bt), 1e-4),
        "gemm_2sm": (build_gemm_2sm(512, 512, 256), (a.cuda(), bt.cuda()), formulas.gemm_ref(a, bt), 1e-4),
        "rms_norm": (build_rms_norm(256, 2048), (x.cuda(), w.cuda()), formulas.rms_norm_ref(x, w), 1e-5),
        "softmax": (build_softmax(256, 2048), (x.cuda(),), torch.softmax(x, -1), 1e-5),
        "attention": (build_flash_attention(1, 2, 256, 256, 64, out_dtype=f32), (q.cuda(), k.cuda(), v.cuda()),
                      formulas.attention_ref(q, k, v), 1e-2),
    }
    for kernel, args, _, _ in jobs.values():
        kernel(*args)                      # builds the per-kernel launcher
        if path == "ctypes":
            kernel._launcher.ext = None    # the same C-ABI call, made through ctypes
        else:
            assert kernel._launcher.ext is not None, "the pybind11 extension was not built"
    torch.cuda.synchronize()
    errors: list[str] = []

    def worker(name):
        kernel, args, ref, tol = jobs[name]
        try:
            stream = torch.cuda.Stream()
            with torch.cuda.stream(stream):
                outs = [kernel(*args) for _ in range(25)]
            stream.synchronize()
            for o in outs:
                err = formulas.rel_fro(o.float().cpu(), ref)
                if not err <= tol:
                    errors.append(f"{name}: rel_fro {err:.3e}")
                    return
        except Exception as exc:  # noqa: BLE001
            errors.append(f"{name}: {exc!r}")

    threads = [threading.Thread(target=worker, args=(n,)) for n in jobs for _ in range(2)]
    for t in threads:
        t.start()
    for t in threads:
        t.join()
    assert not errors, errors[:3]
