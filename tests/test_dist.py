"""Sharding arithmetic and the gather-on-request path, with world_size-2 gloo processes on CPU.
The compute kernel is replaced by a CPU stand-in here: this file tests the host logic around it."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from pyptx_b200 import dist as pdist


def test_partition_covers_everything_in_order():
    for total, world, mult in [(2048, 8, 1), (8192, 8, 128), (2048, 8, 256), (8, 8, 1), (4, 8, 1), (64, 3, 1),
                               (1280, 4, 128), (7, 2, 1)]:
        prev = 0
        for r in range(world):
            a, b = pdist.partition(total, world, r, mult)
            assert a == prev and b >= a and (b - a) % mult == 0
            prev = b
        assert prev == total
        c = pdist.counts(total, world, mult)
        assert sum(c) == total and max(c) - min(c) <= mult


def test_partition_rejects_bad_arguments():
    with pytest.raises(ValueError):
        pdist.partition(100, 4, 4)
    with pytest.raises(ValueError):
        pdist.partition(100, 4, 0, multiple=128)
    with pytest.raises(ValueError):
        pdist.partition(100, 0, 0)


def test_benchmark_partitions():
    # GEMM 8192^3 over 8 GPUs: 1024 rows each, a multiple of both tile heights
    assert pdist.counts(8192, 8, 256) == [1024] * 8
    # 2048^3 over 8 GPUs with the 2-SM tile: 256 rows each
    assert pdist.counts(2048, 8, 256) == [256] * 8
    # G=4 experts over 8 GPUs: four ranks idle
    assert pdist.counts(4, 8) == [1, 1, 1, 1, 0, 0, 0, 0]
    # 64 (batch, head) problems over 8 GPUs
    assert pdist.counts(64, 8) == [8] * 8


def test_shard_builders_use_local_shapes():
    seen = []

    def build_gemm_2sm(M, N, K, **kw):
        seen.append((M, N, K))
        return lambda a, b: a.float() @ b.float().t()

    s = pdist.shard_gemm(build_gemm_2sm, 2048, 256, 64, world=4, rank=3)
    assert (s.start, s.stop, s.multiple) == (1536, 2048, 256) and seen[-1] == (512, 256, 64)
    full = torch.arange(2048 * 4).reshape(2048, 4)
    assert torch.equal(s.slice(full), full[1536:2048])

    def build_grouped(G, M, N, K):
        seen.append((G, M, N, K))
        return None

    s = pdist.shard_grouped_gemm(build_grouped, 4, 128, 64, 64, world=8, rank=5)
    assert s.kernel is None and s.local == 0
    s = pdist.shard_grouped_gemm(build_grouped, 8, 128, 64, 64, world=2, rank=1)
    assert (s.start, s.stop) == (512, 1024) and seen[-1] == (4, 128, 64, 64)

    def build_attn(batch, heads, sq, skv, d, **kw):
        seen.append((batch, heads, sq, skv, d, kw))
        return None

    s = pdist.shard_attention(build_attn, 4, 16, 4096, None, 128, world=8, rank=2, causal=True)
    assert (s.start, s.stop) == (16, 24) and seen[-1] == (1, 8, 4096, None, 128, {"causal": True})


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank: int, world: int, port: int, rows: int, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.manual_seed(0)
        x = torch.randn(rows, 64)
        w = torch.randn(64)

        def fake_builder(b, n, eps=1e-6):
            return lambda xs, ws: xs * torch.rsqrt((xs * xs).mean(-1, keepdim=True) + eps) * ws

        ref = fake_builder(rows, 64)(x, w)
        # no collective unless asked: each rank gets only its rows
        shard = pdist.shard_rows(fake_builder, rows, 64)
        local = shard(shard.slice(x), w)
        ok_local = torch.allclose(local, ref[shard.start:shard.stop])
        # gather=True: every rank ends with the full result
        shard_g = pdist.shard_rows(fake_builder, rows, 64, gather=True)
        full = shard_g(shard_g.slice(x), w)
        ok_full = full.shape == ref.shape and torch.allclose(full, ref)
        # max-over-ranks reduction used for timing
        t = torch.tensor([float(rank + 1)])
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        results[rank] = (ok_local, ok_full, float(t.item()), shard.local)
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("rows", [64, 7])
def test_two_rank_gloo_shard_and_gather(rows):
    world = 2
    port = _free_port()
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        results = mgr.dict()
        procs = [ctx.Process(target=_worker, args=(r, world, port, rows, results)) for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(timeout=120)
            assert p.exitcode == 0
        got = dict(results)
    assert set(got) == {0, 1}
    for r in range(world):
        ok_local, ok_full, tmax, local = got[r]
        assert ok_local and ok_full and tmax == 2.0
    assert got[0][3] + got[1][3] == rows


def _worker_empty_rank_and_attention(rank: int, world: int, port: int, results):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from pyptx_b200.types import bf16, f32
        torch.manual_seed(0)
        # GEMM whose M holds one 256-row unit: rank 1 owns nothing and must still enter the
        # collective with D's trailing shape and dtype (f32 [., N]), not A's (bf16 [., K]).
        M, N, K = 256, 48, 32
        a = torch.randn(M, K).to(torch.bfloat16)
        bt = torch.randn(N, K).to(torch.bfloat16)

        def build_gemm_2sm(m, n, k, **kw):
            return lambda x, y: x.float() @ y.float().t()

        sh = pdist.shard_gemm(build_gemm_2sm, M, N, K, gather=True)
        full = sh(sh.slice(a), bt)
        ok_gemm = (sh.local == (256 if rank == 0 else 0) and full.dtype == torch.float32
                   and torch.equal(full, a.float() @ bt.float().t()))
        # zero rows everywhere: nothing to gather, no collective, an empty result
        none = pdist.Shard(None, 0, 0, 0, world, rank, 1, True, None, (5,), f32)(torch.empty(0, 3))
        ok_none = tuple(none.shape) == (0, 5)
        # attention: local outputs are [1, local, S, d]; the gathered one is [1, B*H, S, d]
        B, H, S, d = 1, 3, 4, 8
        q = torch.randn(B * H, S, d).to(torch.bfloat16)

        def build_attn(batch, heads, sq, skv, hd, **kw):
            return lambda qq: (qq.float() * 2).to(torch.bfloat16)

        sa = pdist.shard_attention(build_attn, B, H, S, None, d, gather=True, out_dtype=bf16)
        o = sa(sa.slice(q).unsqueeze(0))
        ok_attn = tuple(o.shape) == (1, B * H, S, d) and torch.equal(o[0], (q.float() * 2).to(torch.bfloat16))

        # a kernel with two outputs (O, lse): the first is gathered, the second stays local
        def build_attn_lse(batch, heads, sq, skv, hd, **kw):
            return lambda qq: ((qq.float() * 2).to(torch.bfloat16), qq.float().sum(-1))

        sl = pdist.shard_attention(build_attn_lse, B, H, S, None, d, gather=True)
        o2, lse = sl(sl.slice(q).unsqueeze(0))
        ok_lse = tuple(o2.shape) == (1, B * H, S, d) and tuple(lse.shape) == (1, sl.local, S)
        results[rank] = (ok_gemm, ok_none, ok_attn, ok_lse)
    finally:
        dist.destroy_process_group()


def test_two_rank_gloo_empty_rank_and_attention_gather():
    world = 2
    port = _free_port()
    ctx = mp.get_context("spawn")
    with ctx.Manager() as mgr:
        results = mgr.dict()
        procs = [ctx.Process(target=_worker_empty_rank_and_attention, args=(r, world, port, results))
                 for r in range(world)]
        for p in procs:
            p.start()
        for p in procs:
            p.join(timeout=120)
            assert p.exitcode == 0
        got = dict(results)
    assert set(got) == {0, 1}
    for r in range(world):
        assert got[r] == (True, True, True, True), got[r]
