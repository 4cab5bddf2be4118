"""Sharding over the GPUs of one node: one process per GPU, ``torch.distributed`` for plumbing.

Every kernel of the library splits along an axis whose slices are independent, so no
kernel reads another GPU's memory and the data path has no collective:

===================  =============================  =====================================
kernel               sharded axis                   replicated
===================  =============================  =====================================
row kernels          rows                           weight / bias vectors
GEMM (1-SM / 2-SM)   M (row blocks of A and D)      B_T
grouped GEMM         experts                        nothing
flash attention      batch x head                   nothing
===================  =============================  =====================================

A collective (NCCL all-gather over NVLink) runs only when the caller asks for the
gathered output (``gather=True``).  The reference is single-GPU; this layer is new and
specified by the benchmark configuration only.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Callable, Sequence


def partition(total: int, world: int, rank: int, multiple: int = 1) -> tuple[int, int]:
    """Half-open range ``[start, stop)`` of ``total`` items owned by ``rank``.

    Items are handed out in units of ``multiple`` (a kernel's tile height); the first
    ``units % world`` ranks get one unit more.  Ranges are contiguous, ordered by rank,
    and cover ``[0, total)`` exactly.  A rank may get an empty range.
    """
    if world < 1 or not 0 <= rank < world:
        raise ValueError(f"bad rank {rank} for world size {world}")
    if multiple < 1 or total % multiple:
        raise ValueError(f"total={total} must be a multiple of {multiple}")
    units = total // multiple
    base, extra = divmod(units, world)
    start = rank * base + min(rank, extra)
    stop = start + base + (1 if rank < extra else 0)
    return start * multiple, stop * multiple


def counts(total: int, world: int, multiple: int = 1) -> list[int]:
    """Items per rank under :func:`partition`."""
    return [b - a for a, b in (partition(total, world, r, multiple) for r in range(world))]


@dataclass
class Shard:
    """One rank's share of a sharded call: the local kernel plus what gathering needs.

    ``out_tail`` / ``out_dtype`` / ``gather_dim`` describe the kernel's (first) output: the shape
    without the sharded axis, its element type (a ``PtxType`` or a torch dtype) and the axis the
    shares are laid along.  They come from the builder's arguments, not from a local tensor, so a
    rank that owns nothing enters the collective with the same byte count as the others.
    """

    kernel: Callable[..., Any] | None      # None when this rank owns nothing
    start: int
    stop: int
    total: int
    world: int
    rank: int
    multiple: int = 1
    gather: bool = False
    group: Any = None
    out_tail: tuple[int, ...] | None = None
    out_dtype: Any = None
    gather_dim: int = 0

    @property
    def local(self) -> int:
        return self.stop - self.start

    def slice(self, tensor, dim: int = 0):
        """This rank's slice of a full (unsharded) tensor along ``dim``."""
        return tensor.narrow(dim, self.start, self.local)

    def _torch_dtype(self, fallback):
        import torch

        dt = self.out_dtype
        if dt is None:
            return fallback
        if isinstance(dt, torch.dtype):
            return dt
        from .torch_support import _ptx_type_to_torch_dtype
        return _ptx_type_to_torch_dtype(dt)

    def __call__(self, *local_inputs):
        """Run the local kernel on this rank's operands; all-gather the (first) output along the
        sharded axis on request.  Kernels with several outputs return the first one gathered and
        the others local."""
        out = self.kernel(*local_inputs) if self.kernel is not None else None
        if not self.gather or self.world == 1:
            return out
        first, rest = (out[0], tuple(out[1:])) if isinstance(out, tuple) else (out, ())
        if first is not None and self.gather_dim == 1:
            # attention: the local output is [1, local, S, d]; the shares lie along the head axis
            if first.shape[0] != 1:
                raise ValueError(f"expected a [1, local, ...] output, got {tuple(first.shape)}")
            first = first[0]
        like = local_inputs[0] if local_inputs else None
        tail = self.out_tail if self.out_tail is not None else tuple((first if first is not None else like).shape[1:])
        dtype = self._torch_dtype((first if first is not None else like).dtype)
        device = (first if first is not None else like).device
        full = all_gather_rows(first, counts(self.total, self.world, self.multiple), self.rank,
                               group=self.group, tail=tail, dtype=dtype, device=device)
        if self.gather_dim == 1:
            full = full.unsqueeze(0)        # [1, batch*heads, ...], the layout the local kernels use
        return (full, *rest) if rest else full


def all_gather_rows(local, rows_per_rank: Sequence[int], rank: int, *, group=None, like=None,
                    tail: tuple[int, ...] | None = None, dtype=None, device=None):
    """All-gather tensors that differ only in dim 0.  Equal shares use one
    ``all_gather_into_tensor``; unequal shares are padded to the largest share and trimmed.
    ``local`` may be ``None`` (or have no rows) on a rank whose share is empty; the trailing shape,
    dtype and device then come from ``tail`` / ``dtype`` / ``device`` (or from ``like``)."""
    import torch
    import torch.distributed as dist

    world = len(rows_per_rank)
    ref = local if local is not None else like
    tail = tuple(tail) if tail is not None else tuple(ref.shape[1:])
    dtype = dtype if dtype is not None else ref.dtype
    device = device if device is not None else ref.device
    have = 0 if local is None else local.shape[0]
    if have != rows_per_rank[rank]:
        raise ValueError(f"rank {rank} holds {have} rows, expected {rows_per_rank[rank]}")
    if local is not None and (tuple(local.shape[1:]) != tail or local.dtype != dtype):
        raise ValueError(f"rank {rank} holds {tuple(local.shape[1:])} {local.dtype}, expected {tail} {dtype}")
    biggest = max(rows_per_rank)
    if biggest == 0:
        return torch.empty((0, *tail), dtype=dtype, device=device)
    if all(c == biggest for c in rows_per_rank):
        out = torch.empty((biggest * world, *tail), dtype=dtype, device=device)
        dist.all_gather_into_tensor(out, local.contiguous(), group=group)
        return out
    padded = torch.zeros((biggest, *tail), dtype=dtype, device=device)
    if have:
        padded[:have] = local
    buf = torch.empty((biggest * world, *tail), dtype=dtype, device=device)
    dist.all_gather_into_tensor(buf, padded, group=group)
    return torch.cat([buf[r * biggest: r * biggest + c] for r, c in enumerate(rows_per_rank)], dim=0)


def _out_dtype(kw: dict, default: str):
    """Element type of a builder's output: its ``out_dtype`` argument, else the builder's default."""
    from . import types
    return kw.get("out_dtype") or types.from_name(default)


def _world_rank(world: int | None, rank: int | None) -> tuple[int, int]:
    if world is not None and rank is not None:
        return world, rank
    import torch.distributed as dist
    if dist.is_available() and dist.is_initialized():
        return dist.get_world_size(), dist.get_rank()
    return 1, 0


def shard_rows(builder: Callable[..., Any], rows: int, cols: int, *, world: int | None = None,
               rank: int | None = None, gather: bool = False, group=None, **kw) -> Shard:
    """Row kernels (``build_rms_norm`` / ``build_layer_norm`` / ``build_fused_silu_mul`` /
    ``build_softmax``): rank ``r`` normalises rows ``partition(rows, world, r)``."""
    world, rank = _world_rank(world, rank)
    a, b = partition(rows, world, rank)
    kernel = builder(b - a, cols, **kw) if b > a else None
    return Shard(kernel, a, b, rows, world, rank, 1, gather, group, (cols,), _out_dtype(kw, "f32"))


def shard_gemm(builder: Callable[..., Any], M: int, N: int, K: int, *, world: int | None = None,
               rank: int | None = None, gather: bool = False, group=None, **kw) -> Shard:
    """GEMM: A and D are split in row blocks of the kernel's tile height (128 rows for
    ``build_gemm``, 256 for ``build_gemm_2sm``); every rank holds the whole B_T."""
    world, rank = _world_rank(world, rank)
    multiple = 256 if getattr(builder, "__name__", "").endswith("2sm") else 128
    a, b = partition(M, world, rank, multiple)
    kernel = builder(b - a, N, K, **kw) if b > a else None
    return Shard(kernel, a, b, M, world, rank, multiple, gather, group, (N,), _out_dtype(kw, "f32"))


def shard_grouped_gemm(builder: Callable[..., Any], G: int, M: int, N: int, K: int, *,
                       world: int | None = None, rank: int | None = None, gather: bool = False,
                       group=None, **kw) -> Shard:
    """Grouped GEMM: whole experts per rank (contiguous expert ranges).  The returned shard
    counts rows of the stacked operand A[G*M, K]; ranks beyond G own nothing."""
    world, rank = _world_rank(world, rank)
    g0, g1 = partition(G, world, rank)
    kernel = builder(g1 - g0, M, N, K, **kw) if g1 > g0 else None
    return Shard(kernel, g0 * M, g1 * M, G * M, world, rank, M, gather, group, (N,), _out_dtype(kw, "f32"))


def shard_attention(builder: Callable[..., Any], batch: int, heads: int, seq_q: int, seq_kv: int | None = None,
                    head_dim: int = 64, *, world: int | None = None, rank: int | None = None,
                    gather: bool = False, group=None, **kw) -> Shard:
    """Attention: the ``batch*heads`` independent problems are split contiguously; a rank's
    operands are ``[1, local, S, d]`` views of the flattened ``[batch*heads, S, d]`` tensors."""
    world, rank = _world_rank(world, rank)
    a, b = partition(batch * heads, world, rank)
    kernel = builder(1, b - a, seq_q, seq_kv, head_dim, **kw) if b > a else None
    return Shard(kernel, a, b, batch * heads, world, rank, 1, gather, group, (seq_q, head_dim),
                 _out_dtype(kw, "bf16"), gather_dim=1)
