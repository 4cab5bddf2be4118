"""Sharded calls on real GPUs, one process per GPU (run under ``torch.distributed.run``; with a
single process the same code paths run with world size 1).  Each rank computes its shard with
the CUDA kernels; the gathered result must equal the CPU oracle on the unsharded problem."""
import os

import pytest
import torch
import torch.distributed as dist

from oracle import formulas, inputs
from pyptx_b200 import dist as pdist
from pyptx_b200.examples.blackwell.flash_attention import build_flash_attention
from pyptx_b200.examples.blackwell.gemm_highperf_blackwell import build_gemm, build_gemm_2sm
from pyptx_b200.examples.blackwell.grouped_gemm import build_grouped_gemm
from pyptx_b200.examples.blackwell.rms_norm import build_rms_norm
from pyptx_b200.types import f32

pytestmark = pytest.mark.gpu


@pytest.fixture(scope="module", autouse=True)
def process_group():
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local)
    if world > 1 and not dist.is_initialized():
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    yield
    if dist.is_initialized():
        dist.barrier()
        dist.destroy_process_group()


def _wr():
    return (dist.get_world_size(), dist.get_rank()) if dist.is_initialized() else (1, 0)


def test_rows_sharded_and_gathered():
    world, rank = _wr()
    x, w = inputs.rms_norm_inputs(512, 2048)
    ref = formulas.rms_norm_ref(x, w)
    shard = pdist.shard_rows(build_rms_norm, 512, 2048, world=world, rank=rank)
    y = shard(shard.slice(x).cuda().contiguous(), w.cuda())
    assert formulas.rel_fro(y.cpu(), ref[shard.start:shard.stop]) < 1e-5
    full = pdist.shard_rows(build_rms_norm, 512, 2048, world=world, rank=rank, gather=True)
    yg = full(full.slice(x).cuda().contiguous(), w.cuda())
    assert yg.shape == ref.shape and formulas.rel_fro(yg.cpu(), ref) < 1e-5


@pytest.mark.parametrize("builder", [build_gemm, build_gemm_2sm])
def test_gemm_m_sharded_b_replicated(builder):
    world, rank = _wr()
    M, N, K = 2048, 512, 256
    a, bt = inputs.gemm_inputs(M, N, K)
    ref = formulas.gemm_ref(a, bt)
    shard = pdist.shard_gemm(builder, M, N, K, world=world, rank=rank, gather=True)
    d = shard(shard.slice(a).cuda().contiguous(), bt.cuda())
    assert d.shape == ref.shape and formulas.rel_fro(d.cpu(), ref) < 1e-4


def test_grouped_experts_partitioned():
    world, rank = _wr()
    G, M, N, K = 8, 256, 256, 128
    a, bt = inputs.grouped_gemm_inputs(G, M, N, K)
    ref = formulas.grouped_gemm_ref(a, bt, G)
    shard = pdist.shard_grouped_gemm(build_grouped_gemm, G, M, N, K, world=world, rank=rank, gather=True)
    g0, g1 = shard.start // M, shard.stop // M
    local_a = a[shard.start:shard.stop].cuda().contiguous()
    local_b = bt[g0 * N:g1 * N].cuda().contiguous()
    c = shard(local_a, local_b)
    assert c.shape == ref.shape and formulas.rel_fro(c.cpu(), ref) < 1e-4


def test_attention_batch_head_sharded():
    world, rank = _wr()
    B, H, S, d = 2, 8, 256, 64
    q, k, v = inputs.attention_inputs(B * H, S, S, d)
    ref = formulas.attention_ref(q, k, v, causal=True)
    shard = pdist.shard_attention(build_flash_attention, B, H, S, S, d, world=world, rank=rank, gather=True,
                                  causal=True, out_dtype=f32)
    sl = slice(shard.start, shard.stop)
    og = shard(q[sl][None].cuda().contiguous(), k[sl][None].cuda().contiguous(), v[sl][None].cuda().contiguous())
    assert og.shape == (1, *ref.shape) and formulas.rel_fro(og[0].cpu(), ref) < 1e-2


@pytest.mark.parametrize("two_sm", [False, True])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_push_gather_gemm_equals_oracle_on_every_rank(two_sm, out_dtype):
    """The GEMM whose epilogue stores each tile into every rank's gathered buffer: all ranks
    end up with the full product; repeated calls reuse the buffer safely."""
    from pyptx_b200 import _native
    from pyptx_b200.peer import PushGatherGemm

    world, rank = _wr()
    M_local, N, K = 512, 512, 256
    a, bt = inputs.gemm_inputs(world * M_local, N, K)
    ref = formulas.gemm_ref(a, bt)
    gemm = PushGatherGemm(M_local, N, K, two_sm=two_sm, out_dtype=out_dtype)
    assert (gemm.world, gemm.rank) == (world, rank)
    a_local = a[rank * M_local:(rank + 1) * M_local].cuda().contiguous()
    b_dev = bt.cuda()
    for _ in range(3):
        out = gemm(a_local, b_dev)
        torch.cuda.synchronize()
        assert out.shape == ref.shape
        assert formulas.rel_fro(out.float().cpu(), ref) < (1e-2 if out_dtype == torch.bfloat16 else 1e-4)
        out.zero_()          # the next call's entry barrier orders this before any peer's store
    _native.device_status()


def test_push_gather_is_bit_identical_to_nccl_gather():
    from pyptx_b200.peer import PushGatherGemm

    world, rank = _wr()
    M_local, N, K = 1024, 1024, 512
    a, bt = inputs.gemm_inputs(world * M_local, N, K)
    a_local = a[rank * M_local:(rank + 1) * M_local].cuda().contiguous()
    b_dev = bt.cuda()
    shard = pdist.shard_gemm(build_gemm_2sm, world * M_local, N, K, world=world, rank=rank, gather=True)
    via_nccl = shard(a_local, b_dev)
    via_push = PushGatherGemm(M_local, N, K)(a_local, b_dev)
    torch.cuda.synchronize()
    assert torch.equal(via_push, via_nccl)


def test_push_gather_replays_from_a_cuda_graph():
    """The barrier keeps its call counter on the device, so a captured call (barrier, GEMM with
    peer stores, barrier) can be replayed: every replay must leave the full product on every rank."""
    from pyptx_b200 import _native
    from pyptx_b200.peer import PushGatherGemm

    world, rank = _wr()
    M_local, N, K = 512, 512, 256
    a, bt = inputs.gemm_inputs(world * M_local, N, K)
    ref = formulas.gemm_ref(a, bt)
    gemm = PushGatherGemm(M_local, N, K)
    a_local = a[rank * M_local:(rank + 1) * M_local].cuda().contiguous()
    b_dev = bt.cuda()
    gemm(a_local, b_dev)                       # warm-up outside the capture
    torch.cuda.synchronize()
    stream = torch.cuda.Stream()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(stream):
        with torch.cuda.graph(graph, stream=stream):
            out = gemm(a_local, b_dev)
    for _ in range(3):
        out.zero_()
        torch.cuda.synchronize()
        if dist.is_initialized():
            dist.barrier()                     # nobody replays while a peer is still clearing its buffer
        graph.replay()
        torch.cuda.synchronize()
        assert formulas.rel_fro(out.cpu(), ref) < 1e-4
    _native.device_status()
