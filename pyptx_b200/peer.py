"""Peer-memory path over NVLink: a GEMM whose epilogue is the all-gather of its result.

``shard_gemm(..., gather=True)`` runs the local GEMM and then an NCCL all-gather.  Here the
two are one kernel: rank ``r`` computes its row block ``D[r*M_local:(r+1)*M_local]`` and the
epilogue stores every finished 32-row box to the same place of the gathered buffer on
**every** rank (plain TMA stores into peer-mapped memory, no multicast), so the transfer of
tile ``i`` runs under the main loop of tile ``i+1`` and the result never makes a second trip
through HBM.  A stream-ordered flag barrier (``PB200_K_PEER_BARRIER``, bounded wait) on
both sides of the kernel replaces the collective's synchronisation:

* before: no rank may overwrite a gathered buffer that another rank is still reading from
  the previous call;
* after: every rank's block has landed everywhere.

Buffers come from torch's symmetric memory (one allocation per rank, mapped on all ranks of
the group).  One process per GPU; all ranks must make the same calls in the same order.
The reference is single-GPU; nothing here has a counterpart there.
"""
from __future__ import annotations

import ctypes
import os
from typing import Any

from . import _ids, _native


def _torch():
    import torch
    return torch


class SymmetricBuffer:
    """A tensor with the same shape on every rank, each rank's copy addressable from all ranks.

    ``tensor`` is this rank's copy, ``ptrs[p]`` the device address of rank ``p``'s copy in this
    process.  Without an initialised process group (or with ``world == 1``) it is an ordinary
    tensor and ``ptrs == [tensor.data_ptr()]``.
    """

    def __init__(self, shape, dtype, *, group=None, device=None) -> None:
        torch = _torch()
        import torch.distributed as dist

        if device is None:
            device = torch.device("cuda", torch.cuda.current_device())
        self.world, self.rank = 1, 0
        if dist.is_available() and dist.is_initialized():
            self.world = dist.get_world_size(group)
            self.rank = dist.get_rank(group)
        if self.world == 1:
            self.tensor = torch.empty(shape, dtype=dtype, device=device)
            self.ptrs = [self.tensor.data_ptr()]
            self._handle = None
            return
        # This library stores to peers with plain stores only; keep the allocation out of
        # NVLink multicast objects, which it would never use.
        os.environ.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
        import torch.distributed._symmetric_memory as symm_mem

        self.tensor = symm_mem.empty(shape, dtype=dtype, device=device)
        self._handle = symm_mem.rendezvous(self.tensor, group if group is not None else dist.group.WORLD)
        self.ptrs = [int(p) for p in self._handle.buffer_ptrs]
        if len(self.ptrs) != self.world or self.ptrs[self.rank] != self.tensor.data_ptr():
            raise RuntimeError("pyptx_b200: symmetric memory rendezvous returned unexpected addresses")


class PeerBarrier:
    """Stream-ordered barrier across the ranks of a node (kernel ``PB200_K_PEER_BARRIER``).

    ``barrier()`` enqueues one tiny kernel on the current stream; the host does not wait.  A
    rank that waits longer than ``timeout_s`` gives up and records it:
    ``pyptx_b200.device_status()`` then raises.
    """

    def __init__(self, *, group=None, device=None, timeout_s: float = 10.0) -> None:
        torch = _torch()
        import torch.distributed as dist

        self.flags = SymmetricBuffer((16,), torch.int32, group=group, device=device)
        self.world, self.rank = self.flags.world, self.flags.rank
        self.flags.tensor.zero_()
        torch.cuda.synchronize(self.flags.tensor.device)
        if self.world > 1:
            dist.barrier(group)          # every rank's flags are zero before anyone signals
        self.handle = _native.create_handle(_ids.K_PEER_BARRIER, (self.world, self.rank), (float(timeout_s),))
        self._ptrs = (ctypes.c_void_p * self.world)(*self.flags.ptrs)

    def __call__(self, stream: int | None = None) -> None:
        if stream is None:
            stream = _torch().cuda.current_stream(self.flags.tensor.device).cuda_stream
        _native.launch_raw(self.handle, stream, self._ptrs)

    barrier = __call__


class PushGatherGemm:
    """``D = A @ B_T.T`` sharded by rows of A, with the gathered ``D`` on every rank.

    ``gemm = PushGatherGemm(M_local, N, K)``; ``full = gemm(a_local, b_t)`` returns this rank's
    ``[world * M_local, N]`` buffer, complete once the call's work on the current stream has
    run.  The buffer is reused by the next call: consume (or copy) it before calling again.
    ``two_sm`` selects the 256-row ``cta_group::2`` tile (``M_local % 256 == 0``), else the
    128-row tile; ``N % 256 == 0`` and ``K % 64 == 0`` as for ``build_gemm``.
    """

    def __init__(self, M_local: int, N: int, K: int, *, group=None, device=None, out_dtype=None,
                 two_sm: bool = True, timeout_s: float = 10.0) -> None:
        torch = _torch()
        out_dtype = torch.float32 if out_dtype is None else out_dtype
        if out_dtype not in (torch.float32, torch.bfloat16):
            raise TypeError(f"out_dtype must be torch.float32 or torch.bfloat16, got {out_dtype}")
        self.M_local, self.N, self.K = int(M_local), int(N), int(K)
        self.barrier = PeerBarrier(group=group, device=device, timeout_s=timeout_s)
        self.world, self.rank = self.barrier.world, self.barrier.rank
        self.out = SymmetricBuffer((self.world * self.M_local, self.N), out_dtype, group=group, device=device)
        flags = _ids.F_OUT_BF16 if out_dtype == torch.bfloat16 else 0
        self.handle = _native.create_handle(
            _ids.K_GEMM_PUSH, (self.world, 2 if two_sm else 1, self.M_local, self.N, self.K), (), flags)
        g = _native.geometry_of(self.handle)
        self.grid, self.block, self.cluster, self.smem = tuple(g.grid), tuple(g.block), tuple(g.cluster), int(g.smem_bytes)
        block_bytes = self.M_local * self.N * self.out.tensor.element_size()
        # Own copy first, then the peers in ring order starting after this rank, so that at any
        # moment the ranks address different peers.
        order = [(self.rank + i) % self.world for i in range(self.world)]
        self._dests = [self.out.ptrs[p] + self.rank * block_bytes for p in order]
        self._ptrs = (ctypes.c_void_p * (2 + self.world))()
        for i, d in enumerate(self._dests):
            self._ptrs[2 + i] = d

    def _check(self, a: Any, b_t: Any) -> None:
        torch = _torch()
        dev = self.out.tensor.device
        for name, t, shape in (("A", a, (self.M_local, self.K)), ("B_T", b_t, (self.N, self.K))):
            if not isinstance(t, torch.Tensor):
                raise TypeError(f"PushGatherGemm: {name} is {type(t).__name__}, not a torch.Tensor")
            if t.device != dev:
                raise ValueError(f"PushGatherGemm: {name} is on {t.device}, the gathered buffer on {dev}")
            if t.dtype != torch.bfloat16:
                raise TypeError(f"PushGatherGemm: {name} has dtype {t.dtype}, wants torch.bfloat16")
            if tuple(t.shape) != shape:
                raise ValueError(f"PushGatherGemm: {name} has shape {tuple(t.shape)}, wants {shape}")
            if not t.is_contiguous():
                raise ValueError(f"PushGatherGemm: {name} is not contiguous")

    def __call__(self, a_local: Any, b_t: Any):
        self._check(a_local, b_t)
        stream = _torch().cuda.current_stream(self.out.tensor.device).cuda_stream
        self._ptrs[0] = a_local.data_ptr()
        self._ptrs[1] = b_t.data_ptr()
        if self.world > 1:
            self.barrier(stream)
        _native.launch_raw(self.handle, stream, self._ptrs)
        if self.world > 1:
            self.barrier(stream)
        return self.out.tensor
