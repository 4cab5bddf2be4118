"""``NativeKernel``: the callable object every ``build_*`` entry point returns.

It exposes the same attribute surface as the reference's ``Kernel``
(pyptx/kernel.py:402-447: ``in_specs``, ``out_specs``, ``grid``, ``block``,
``cluster``, ``smem``, ``arch``) and the same call convention
(pyptx/kernel.py:875-916): positional tensors in ``in_specs`` order, outputs
freshly allocated and returned (one tensor, or a tuple).  Behind it sits a
handle of the C-ABI library instead of a traced-and-JIT-compiled PTX module.
"""
from __future__ import annotations

import sys
from typing import Any, Sequence

from . import _native
from .specs import Tile, unify_envs


class NativeKernel:
    """A compiled sm_100a kernel bound to one static shape."""

    def __init__(self, name: str, kernel_id: int, dims: Sequence[int], *,
                 in_specs: Sequence[Tile], out_specs: Sequence[Tile],
                 fparams: Sequence[float] = (), flags: int = 0,
                 arch: str = "sm_100a", meta: dict | None = None) -> None:
        if not arch.startswith("sm_100"):
            raise AssertionError(f"{name} is only implemented for sm_100*, got arch={arch!r}")
        self.__name__ = name
        self._name = name
        self._kernel_id = int(kernel_id)
        self._dims = tuple(int(d) for d in dims)
        self._fparams = tuple(float(f) for f in fparams)
        self._flags = int(flags)
        self._in_specs = tuple(in_specs)
        self._out_specs = tuple(out_specs)
        self._arch = arch
        self.meta = dict(meta or {})
        self._handle = _native.create_handle(self._kernel_id, self._dims, self._fparams, self._flags)
        g = _native.geometry_of(self._handle)
        self._grid = tuple(int(v) for v in g.grid)
        self._block = tuple(int(v) for v in g.block)
        self._cluster = tuple(int(v) for v in g.cluster)
        self._smem = int(g.smem_bytes)
        self._scratch_bytes = int(g.scratch_bytes)
        if (int(g.n_inputs), int(g.n_outputs)) != (len(self._in_specs), len(self._out_specs)):
            raise RuntimeError(
                f"{name}: spec count ({len(self._in_specs)} in, {len(self._out_specs)} out) disagrees "
                f"with the native kernel ({g.n_inputs} in, {g.n_outputs} out)")
        self._launcher = None  # built on first call (imports torch)
        # The torch.compile route needs its custom op to exist before Dynamo starts tracing a
        # call, so it is registered here whenever torch is already imported.
        self._op = None
        if "torch" in sys.modules:
            from . import torch_support
            self._op = torch_support.get_or_register_torch_op(self)

    # -- attribute surface of the reference's Kernel -------------------------
    @property
    def in_specs(self) -> tuple[Tile, ...]:
        return self._in_specs

    @property
    def out_specs(self) -> tuple[Tile, ...]:
        return self._out_specs

    @property
    def grid(self) -> tuple[int, int, int]:
        return self._grid

    @property
    def block(self) -> tuple[int, int, int]:
        return self._block

    @property
    def cluster(self) -> tuple[int, int, int]:
        return self._cluster

    @property
    def smem(self) -> int:
        return self._smem

    @property
    def scratch_bytes(self) -> int:
        """Device scratch the kernel needs per launch (allocated by the launch path, never kept)."""
        return self._scratch_bytes

    @property
    def arch(self) -> str:
        return self._arch

    @property
    def handle(self) -> int:
        """Handle of this kernel in the C-ABI registry."""
        return self._handle

    @property
    def template_params(self) -> dict[str, Any]:
        return dict(self.meta)

    def __repr__(self) -> str:
        return (f"<NativeKernel {self._name} dims={self._dims} grid={self._grid} block={self._block} "
                f"cluster={self._cluster} smem={self._smem} arch={self._arch}>")

    # -- calling --------------------------------------------------------------
    def bind_shapes(self, shapes: Sequence[tuple[int, ...]]) -> dict[str, int]:
        """Validate input shapes against ``in_specs`` and return the dim bindings."""
        if len(shapes) != len(self._in_specs):
            raise TypeError(
                f"Kernel {self._name} expected {len(self._in_specs)} input arrays, got {len(shapes)}")
        return unify_envs(spec.extract_env(tuple(int(d) for d in shp))
                          for spec, shp in zip(self._in_specs, shapes))

    def out_shapes(self, env: dict[str, int] | None = None) -> list[tuple[int, ...]]:
        return [spec.resolve_shape(env or {}) for spec in self._out_specs]

    def __call__(self, *args: Any) -> Any:
        from . import torch_support

        inputs = args[: len(self._in_specs)]
        if len(inputs) != len(self._in_specs):
            raise TypeError(
                f"Kernel {self._name} expected {len(self._in_specs)} input arrays, got {len(inputs)}")
        return torch_support.call_kernel(self, inputs)
