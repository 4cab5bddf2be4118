"""PyTorch launch path for :class:`pyptx_b200.kernel.NativeKernel`.

Mirrors the reference's torch integration (pyptx/torch_support.py):

* eager launch -- ``call_kernel_via_torch`` (:171-271): outputs from
  ``torch.empty`` on the first input's device, a ``void*[]`` of inputs then
  outputs, the current CUDA stream as an integer, one call into the C ABI;
* ``torch.compile`` -- one ``torch.library.custom_op`` per handle with schema
  ``(Tensor[] inputs) -> Tensor[]`` and a ``register_fake`` that only sizes the
  outputs (:347-438);
* CUDA graphs -- the launch is stream-ordered, never synchronises and only
  allocates through torch's caching allocator, so it can be captured;
* autograd -- ``differentiable_kernel`` pairs a forward and a backward kernel
  (:446-519).

Unlike the reference, the inputs are checked at call time (device, dtype,
contiguity, alignment) and a ``TypeError`` / ``ValueError`` is raised before
anything is enqueued.
"""
from __future__ import annotations

import ctypes
import threading
from typing import Any, Sequence

from . import _native

_TORCH = None


def _torch():
    global _TORCH
    if _TORCH is None:
        import torch
        _TORCH = torch
    return _TORCH


def is_torch_tensor(obj: Any) -> bool:
    try:
        return isinstance(obj, _torch().Tensor)
    except ImportError:
        return False


def any_torch_tensors(inputs: Sequence[Any]) -> bool:
    return any(is_torch_tensor(x) for x in inputs)


_PTX_TO_TORCH_NAME = {
    "f16": "float16", "bf16": "bfloat16", "f32": "float32", "f64": "float64",
    "s8": "int8", "s16": "int16", "s32": "int32", "s64": "int64",
    "u8": "uint8", "b8": "uint8", "b16": "uint16", "b32": "uint32", "b64": "uint64",
    "pred": "bool",
}


def _ptx_type_to_torch_dtype(dtype):
    """Map a ``PtxType`` to a ``torch.dtype`` (pyptx/torch_support.py:278-301)."""
    name = _PTX_TO_TORCH_NAME.get(dtype.name)
    if name is None or not hasattr(_torch(), name):
        raise TypeError(f"Cannot map PtxType {dtype.name} to a torch.dtype")
    return getattr(_torch(), name)


def _torch_dtype_to_ptx_type_name(torch_dtype) -> str:
    """Inverse mapping, used to check input dtypes (pyptx/torch_support.py:304-323)."""
    torch = _torch()
    table = {
        torch.float16: "f16", torch.bfloat16: "bf16", torch.float32: "f32", torch.float64: "f64",
        torch.int8: "s8", torch.int16: "s16", torch.int32: "s32", torch.int64: "s64",
        torch.uint8: "u8", torch.bool: "pred",
    }
    if torch_dtype not in table:
        raise TypeError(f"Cannot map torch dtype {torch_dtype} to a pyptx type")
    return table[torch_dtype]


def extract_input_shapes(inputs) -> list[tuple[int, ...]]:
    return [tuple(t.shape) for t in inputs]


# ---------------------------------------------------------------------------
# Eager launch
# ---------------------------------------------------------------------------

class _Launcher:
    """Per-kernel cached state for the eager path.  The ctypes pointer array and error buffer
    are reused between calls, but each host thread has its own pair: ctypes releases the GIL
    around the call, so a shared array could be refilled by another thread mid-launch."""

    def __init__(self, kernel) -> None:
        self.lib = _native.load()
        self.handle = ctypes.c_int64(kernel.handle)
        self.n_in = len(kernel.in_specs)
        self.scratch_bytes = kernel.scratch_bytes
        self.n = self.n_in + len(kernel.out_specs) + (1 if self.scratch_bytes else 0)
        self._tls = threading.local()
        self.in_dtypes = [_ptx_type_to_torch_dtype(s.dtype) for s in kernel.in_specs]
        self.out_dtypes = [_ptx_type_to_torch_dtype(s.dtype) for s in kernel.out_specs]
        self.static_out_shapes = None
        if not any(s.symbolic_dims for s in kernel.out_specs):
            self.static_out_shapes = kernel.out_shapes({})
        self.in_shapes = [s.shape if not s.symbolic_dims else None for s in kernel.in_specs]
        self.ext = _native.load_torch_ext()
        # c10::ScalarType integers, as the reference passes them (pyptx/torch_support.py:209-214)
        torch = _torch()
        codes = {torch.uint8: 0, torch.int8: 1, torch.int16: 2, torch.int32: 3, torch.int64: 4,
                 torch.float16: 5, torch.float32: 6, torch.float64: 7, torch.bool: 11, torch.bfloat16: 15}
        self.out_dtype_codes = [codes[d] for d in self.out_dtypes]
        self.handle_int = int(kernel.handle)


    def call_buffers(self):
        """This thread's (pointer array, its address, error buffer)."""
        tls = self._tls
        if not hasattr(tls, "ptrs"):
            tls.ptrs = (ctypes.c_void_p * self.n)()
            tls.ptrs_ref = ctypes.cast(tls.ptrs, ctypes.c_void_p)
            tls.err = ctypes.create_string_buffer(_native.ERR_LEN)
        return tls.ptrs, tls.ptrs_ref, tls.err


def _check_inputs(kernel, launcher: _Launcher, inputs) -> dict[str, int]:
    torch = _torch()
    dev = inputs[0].device
    if dev.type != "cuda":
        raise ValueError(
            f"Kernel {kernel.__name__}: inputs must be CUDA tensors, got device {dev} "
            f"(there is no CPU path)")
    needs_env = False
    for i, (t, want_dt, want_shape) in enumerate(zip(inputs, launcher.in_dtypes, launcher.in_shapes)):
        if not isinstance(t, torch.Tensor):
            raise TypeError(f"Kernel {kernel.__name__}: input {i} is {type(t).__name__}, not a torch.Tensor")
        if t.device != dev:
            raise ValueError(f"Kernel {kernel.__name__}: input {i} is on {t.device}, input 0 on {dev}")
        if t.dtype != want_dt:
            raise TypeError(f"Kernel {kernel.__name__}: input {i} has dtype {t.dtype}, spec wants {want_dt}")
        if not t.is_contiguous():
            raise ValueError(f"Kernel {kernel.__name__}: input {i} is not contiguous")
        if want_shape is None:
            needs_env = True
        elif tuple(t.shape) != want_shape:
            # Same wording as Tile.extract_env so messages match the reference's.
            kernel.in_specs[i].extract_env(tuple(t.shape))
    if needs_env:
        return kernel.bind_shapes([tuple(t.shape) for t in inputs])
    return {}


def call_kernel_via_torch(kernel, inputs: Sequence[Any]):
    """Enqueue ``kernel`` on the current stream of the inputs' device; returns a list of outputs."""
    torch = _torch()
    if not inputs:
        raise ValueError("pyptx_b200: a kernel call requires at least one input")
    if not isinstance(inputs[0], torch.Tensor):
        raise TypeError(f"Kernel {kernel.__name__} takes torch.Tensor inputs (the JAX path is not built)")
    launcher = kernel._launcher
    if launcher is None:
        launcher = kernel._launcher = _Launcher(kernel)
    env = _check_inputs(kernel, launcher, inputs)
    dev = inputs[0].device
    shapes = launcher.static_out_shapes or kernel.out_shapes(env)
    if launcher.scratch_bytes:
        # Scratch rides along as one more buffer after the outputs; it comes from torch's caching
        # allocator like the outputs (so capture in a CUDA graph works) and is dropped on return.
        shapes = list(shapes) + [(launcher.scratch_bytes,)]
    if launcher.ext is not None:
        # pybind11 fast path: output allocation and the C-ABI call happen in C++.
        codes = launcher.out_dtype_codes + ([0] if launcher.scratch_bytes else [])      # scratch: uint8
        if torch.cuda.current_device() != dev.index:
            with torch.cuda.device(dev):
                res = launcher.ext.launch_kernel(launcher.handle_int, torch.cuda.current_stream(dev).cuda_stream,
                                                 list(inputs), [list(s) for s in shapes], codes)
        else:
            res = launcher.ext.launch_kernel(launcher.handle_int, torch.cuda.current_stream(dev).cuda_stream,
                                             list(inputs), [list(s) for s in shapes], codes)
        return res[:-1] if launcher.scratch_bytes else res
    dtypes = launcher.out_dtypes + ([torch.uint8] if launcher.scratch_bytes else [])
    outs = [torch.empty(shp, dtype=dt, device=dev) for shp, dt in zip(shapes, dtypes)]
    ptrs, ptrs_ref, err = launcher.call_buffers()
    for i, t in enumerate(inputs):
        ptrs[i] = t.data_ptr()
    for i, t in enumerate(outs):
        ptrs[launcher.n_in + i] = t.data_ptr()
    if torch.cuda.current_device() != dev.index:
        with torch.cuda.device(dev):
            stream = torch.cuda.current_stream(dev).cuda_stream
            rc = launcher.lib.pb200_launch_raw(launcher.handle, stream, ptrs_ref, launcher.n, err)
    else:
        stream = torch.cuda.current_stream(dev).cuda_stream
        rc = launcher.lib.pb200_launch_raw(launcher.handle, stream, ptrs_ref, launcher.n, err)
    if rc != 0:
        msg = err.value.decode("utf-8", errors="replace")
        raise RuntimeError(f"pyptx_b200: pb200_launch_raw failed (code {rc}): {msg}")
    return outs[:-1] if launcher.scratch_bytes else outs


# ---------------------------------------------------------------------------
# torch.compile: one custom_op per handle
# ---------------------------------------------------------------------------

_REGISTERED_OPS: dict[int, Any] = {}


def get_or_register_torch_op(kernel):
    """Return the ``torch.library.custom_op`` wrapping ``kernel`` (registered once per handle)."""
    op = _REGISTERED_OPS.get(kernel.handle)
    if op is not None:
        return op
    torch = _torch()
    op_name = f"pyptx_b200::kernel_{kernel.handle}"

    @torch.library.custom_op(op_name, mutates_args=(), schema="(Tensor[] inputs) -> Tensor[]")
    def native_op(inputs):
        return call_kernel_via_torch(kernel, list(inputs))

    @native_op.register_fake
    def _fake(inputs):
        dev = inputs[0].device if inputs else torch.device("cuda")
        env = kernel.bind_shapes([tuple(t.shape) for t in inputs])
        return [torch.empty(spec.resolve_shape(env), dtype=_ptx_type_to_torch_dtype(spec.dtype), device=dev)
                for spec in kernel.out_specs]

    _REGISTERED_OPS[kernel.handle] = native_op
    kernel._op = native_op
    return native_op


def call_kernel(kernel, inputs: Sequence[Any]):
    """Dispatch used by ``NativeKernel.__call__``: the registered op while Dynamo
    is tracing, the direct launch otherwise; one output -> tensor, several -> tuple."""
    torch = _torch()
    if torch.compiler.is_compiling():
        op = kernel._op
        if op is None:
            raise RuntimeError(
                f"Kernel {kernel.__name__} was built before torch was imported; call "
                "pyptx_b200.torch_support.get_or_register_torch_op(kernel) once before torch.compile traces it")
        outs = op(list(inputs))
    else:
        outs = call_kernel_via_torch(kernel, inputs)
    return outs[0] if len(outs) == 1 else tuple(outs)


def call_kernel_via_torch_compile(kernel, inputs: Sequence[Any]):
    """Always go through the registered custom op (what ``torch.compile`` sees)."""
    outs = get_or_register_torch_op(kernel)(list(inputs))
    return outs[0] if len(outs) == 1 else tuple(outs)


# ---------------------------------------------------------------------------
# Autograd
# ---------------------------------------------------------------------------

def differentiable_kernel(forward_kernel, backward_kernel, *,
                          save_for_backward: Sequence[int] | None = None,
                          num_grad_inputs: int | None = None,
                          save_outputs: Sequence[int] | None = None,
                          visible_outputs: Sequence[int] | None = None):
    """Wrap a forward / backward kernel pair in a ``torch.autograd.Function``.

    ``backward_kernel`` is called with ``(*saved_inputs, *grad_outputs)`` and
    returns one gradient per differentiable input; missing trailing gradients
    are filled with ``None`` (pyptx/torch_support.py:446-519).

    Two additions for forwards that emit statistics next to their result (attention's
    log-sum-exp): ``save_outputs`` lists forward outputs to keep for the backward pass, which then
    receives ``(*saved_inputs, *saved_outputs, *grad_outputs)``; ``visible_outputs`` lists the
    forward outputs the caller gets back (default: all), and gradients arrive for those only.
    """
    torch = _torch()
    saved_idx = None if save_for_backward is None else list(save_for_backward)
    out_keep = [] if save_outputs is None else list(save_outputs)
    out_show = None if visible_outputs is None else list(visible_outputs)

    class _Fn(torch.autograd.Function):
        @staticmethod
        def forward(ctx, *inputs):
            keep = inputs if saved_idx is None else tuple(inputs[i] for i in saved_idx)
            ctx.n_inputs = len(inputs)
            with torch.no_grad():
                outs = forward_kernel(*inputs)
            all_outs = outs if isinstance(outs, tuple) else (outs,)
            ctx.save_for_backward(*keep, *(all_outs[i] for i in out_keep))
            if out_show is None:
                return outs
            shown = tuple(all_outs[i] for i in out_show)
            return shown[0] if len(shown) == 1 else shown

        @staticmethod
        def backward(ctx, *grad_outputs):
            # Autograd hands out expanded (stride-0) gradients for reductions such as sum(); the
            # kernels take contiguous buffers.
            grad_outputs = tuple(g.contiguous() if g is not None else None for g in grad_outputs)
            with torch.no_grad():
                grads = backward_kernel(*ctx.saved_tensors, *grad_outputs)
            if not isinstance(grads, tuple):
                grads = (grads,)
            n = ctx.n_inputs if num_grad_inputs is None else num_grad_inputs
            grads = tuple(grads) + (None,) * max(0, n - len(grads))
            return grads[:n] + (None,) * max(0, ctx.n_inputs - n)

    def wrapper(*inputs):
        return _Fn.apply(*inputs)

    wrapper.__name__ = getattr(forward_kernel, "__name__", "kernel")
    wrapper.__doc__ = f"Differentiable kernel ({wrapper.__name__})"
    wrapper.forward_kernel = forward_kernel
    wrapper.backward_kernel = backward_kernel
    return wrapper
