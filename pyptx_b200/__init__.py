"""pyptx_b200: hand-written sm_100a kernels behind the pyptx operator surface.

Public names follow the reference package (pyptx/__init__.py:38-57) where they
exist on the kernel launch path: ``Tile``, ``Layout``, the dtype tags under
``types``, ``differentiable_kernel`` and ``detect_arch``.  The tracing DSL
(``kernel``, ``reg``, ``smem``, ``ptx``, ``intrinsic``) is not part of this
library: kernels are compiled CUDA, reached through ``build_*`` entry points in
``pyptx_b200.examples``.
"""
from . import types
from ._arch import detect_arch
from .kernel import NativeKernel
from .specs import Layout, Tile, unify_envs
from .torch_support import differentiable_kernel

__version__ = "0.1.0"

__all__ = ["Tile", "Layout", "NativeKernel", "types", "unify_envs",
           "differentiable_kernel", "detect_arch", "__version__"]
