"""The push variant of the GEMM and the flag barrier on one GPU: several destinations in local
memory stand in for the peers' buffers (the store path is the same; only the addresses differ),
and the barrier's bounded wait is made to run out on a flag that nothing sets.  The multi-GPU
use of both is covered by tests/test_gpu_dist.py under ``torch.distributed.run``."""
import ctypes

import pytest
import torch

from oracle import formulas, inputs
from pyptx_b200 import _ids, _native
from pyptx_b200.peer import PeerBarrier, PushGatherGemm
from tests.gpu_util import check_bf16_matmul

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("cta_group", [1, 2])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("n_dest", [1, 3, 8])
@pytest.mark.parametrize("tile_flag", [1 << 18, 1 << 19], ids=["single_height", "double_height"])
def test_push_gemm_writes_every_destination(cta_group, out_dtype, n_dest, tile_flag):
    M, N, K = 512, 512, 256
    a, bt = inputs.gemm_inputs(M, N, K)
    ref = formulas.gemm_ref(a, bt)
    flags = (_ids.F_OUT_BF16 if out_dtype == torch.bfloat16 else 0) | tile_flag
    h = _native.create_handle(_ids.K_GEMM_PUSH, (n_dest, cta_group, M, N, K), (), flags)
    ad, bd = a.cuda(), bt.cuda()
    # destinations: disjoint [M, N] blocks of one tall buffer, filled with a sentinel first
    tall = torch.full((n_dest * M + 8, N), -7.0, dtype=out_dtype, device="cuda")
    dests = [tall[i * M:(i + 1) * M] for i in range(n_dest)]
    _native.launch_raw(h, torch.cuda.current_stream().cuda_stream,
                       [ad.data_ptr(), bd.data_ptr()] + [d.data_ptr() for d in dests])
    torch.cuda.synchronize()
    _native.device_status()
    check_bf16_matmul(dests[0].cpu(), ref, 1e-2 if out_dtype == torch.bfloat16 else 1e-4)
    for d in dests[1:]:
        assert torch.equal(d, dests[0])
    assert (tall[n_dest * M:] == -7.0).all()          # nothing written past the last block
    _native.load().pb200_destroy(h)


def test_push_gather_gemm_single_rank_matches_plain_gemm():
    M, N, K = 1024, 768, 512
    a, bt = inputs.gemm_inputs(M, N, K)
    gemm = PushGatherGemm(M, N, K)
    assert gemm.world == 1
    out = gemm(a.cuda(), bt.cuda())
    check_bf16_matmul(out.cpu(), formulas.gemm_ref(a, bt), 1e-4)
    with pytest.raises(TypeError, match="bfloat16"):
        gemm(a.cuda().float(), bt.cuda())
    with pytest.raises(ValueError, match="shape"):
        gemm(a.cuda()[:512], bt.cuda())


def test_barrier_single_rank_counts_calls():
    bar = PeerBarrier()
    for _ in range(5):
        bar()
    torch.cuda.synchronize()
    _native.device_status()
    words = bar.flags.tensor.cpu().tolist()
    assert words[0] == 5 and words[8] == 5            # own arrival word and own call counter


def test_barrier_wait_is_bounded_and_reported():
    # Two-rank barrier of which only rank 0 exists: rank 1's arrival word is never written.
    mine = torch.zeros(16, dtype=torch.int32, device="cuda")
    absent = torch.zeros(16, dtype=torch.int32, device="cuda")
    h = _native.create_handle(_ids.K_PEER_BARRIER, (2, 0), (0.25,))
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    _native.launch_raw(h, torch.cuda.current_stream().cuda_stream, [mine.data_ptr(), absent.data_ptr()])
    stop.record()
    torch.cuda.synchronize()
    assert 200.0 < start.elapsed_time(stop) < 2000.0
    with pytest.raises(RuntimeError, match=r"code -11"):
        _native.device_status()
    _native.device_status()                            # the status word is cleared by the read
    assert absent.cpu().tolist()[0] == 1               # rank 0 did signal the (absent) peer
    # the context is still usable
    assert float((mine.float() + 1).sum()) > 0
    _native.load().pb200_destroy(h)
