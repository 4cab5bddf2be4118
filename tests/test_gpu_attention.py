"""GPU parity of the flash-attention forward kernel against the fp32 CPU oracle: known-answer
patterns that pin the operand layouts (uniform attention, one-hot attention), the golden
vectors and shape list of the reference's single-head form
(examples/hopper/experimental/flash_attention_hopper.py:472-505), causal masking, both
head dims, both K layouts, the shared-memory-P cross-check and the benchmark configuration."""
import math
import os

import numpy as np
import pytest
import torch

from oracle import formulas, inputs
from pyptx_b200.examples.blackwell.flash_attention import build_flash_attention
from pyptx_b200.examples.hopper.experimental.flash_attention_hopper import build_flash_attention_hopper
from pyptx_b200.types import bf16, f32
from tests.gpu_util import check_bf16_matmul

pytestmark = pytest.mark.gpu


def _bf16(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(a.copy()).view(torch.bfloat16)


@pytest.fixture(scope="module")
def mats(golden_dir):
    return np.load(os.path.join(golden_dir, "matmul_refs.npz"))


def _run(q, k, v, *, causal=False, out_dtype=f32, flags=0, sm_scale=None):
    B, H, Sq, d = q.shape
    kern = build_flash_attention(B, H, Sq, k.shape[2], d, causal=causal, out_dtype=out_dtype,
                                 sm_scale=sm_scale, _debug_flags=flags)
    return kern(q.cuda(), k.cuda(), v.cuda()).cpu()


def _inputs(B, H, Sq, Skv, d):
    q, k, v = inputs.attention_inputs(B * H, Sq, Skv, d)
    return q.view(B, H, Sq, d), k.view(B, H, Skv, d), v.view(B, H, Skv, d)


# ---- known answers ------------------------------------------------------------------

@pytest.mark.parametrize("d", [64, 128])
def test_uniform_attention_averages_v(d):
    """Q = 0 -> every row attends uniformly -> O = column means of V (pins V's layout)."""
    B, H, S = 1, 2, 256
    q = torch.zeros(B, H, S, d, dtype=torch.bfloat16)
    k = torch.randn(B, H, S, d).to(torch.bfloat16)
    v = (torch.arange(d, dtype=torch.float32)[None, None, None, :] + torch.zeros(B, H, S, 1)).to(torch.bfloat16)
    v[:, :, ::2] *= 2          # rows differ, mean = 1.5 * column index
    o = _run(q, k, v)
    ref = formulas.attention_ref(q, k, v)
    torch.testing.assert_close(o, ref, rtol=1e-2, atol=1e-2)
    torch.testing.assert_close(o[0, 0, 17], 1.5 * torch.arange(d, dtype=torch.float32), rtol=1e-2, atol=1e-2)


@pytest.mark.parametrize("d", [64, 128])
def test_one_hot_attention_selects_rows_of_v(d):
    """Sharp scores: query i matches key perm(i) only -> O[i] = V[perm(i)] (pins the key order
    of P against the row order of V)."""
    B, H, S = 1, 1, 256
    g = torch.Generator().manual_seed(3)
    k = torch.randn(B, H, S, d, generator=g)
    k = (k / k.norm(dim=-1, keepdim=True)).to(torch.bfloat16)
    perm = torch.randperm(S, generator=g)
    q = (k.float()[:, :, perm] * 200.0).to(torch.bfloat16)
    v = torch.randn(B, H, S, d, generator=g).to(torch.bfloat16)
    o = _run(q, k, v, sm_scale=1.0)
    ref = formulas.attention_ref(q, k, v, sm_scale=1.0)
    check_bf16_matmul(o, ref)
    assert formulas.rel_fro(o, v.float()[:, :, perm]) < 2e-2


# ---- the reference's single-head form ---------------------------------------------------

@pytest.mark.parametrize("M_q,N_seq,HD", [(128, 128, 64), (128, 256, 64), (128, 128, 128)])
def test_golden_single_head(mats, M_q, N_seq, HD):
    q, k, v = (_bf16(mats[f"fa_{M_q}_{N_seq}_{HD}_{n}"]) for n in "qkv")
    kern = build_flash_attention_hopper(M_q, N_seq, HD)
    o = kern(q.cuda(), k.t().contiguous().cuda(), v.cuda()).cpu()
    ref = torch.from_numpy(mats[f"fa_{M_q}_{N_seq}_{HD}_o"])
    assert o.dtype == torch.float32 and o.shape == (M_q, HD)
    check_bf16_matmul(o, ref)
    assert torch.allclose(o, ref, atol=5e-2, rtol=1e-2)     # the reference's own criterion (:481)


@pytest.mark.parametrize("HD", [16, 32, 64, 128])       # the reference's list is (16, 32, 64), :502-505
@pytest.mark.parametrize("M_q,N_seq", [(128, 128), (128, 512), (256, 256), (512, 1024), (1024, 2048), (2048, 2048),
                                       (384, 640)])
def test_single_head_shapes(M_q, N_seq, HD):
    torch.manual_seed(M_q * 131 + N_seq + HD * 7)
    q = (torch.randn(M_q, HD) * 0.3).to(torch.bfloat16)
    k = (torch.randn(N_seq, HD) * 0.3).to(torch.bfloat16)
    v = (torch.randn(N_seq, HD) * 0.3).to(torch.bfloat16)
    o = build_flash_attention_hopper(M_q, N_seq, HD)(q.cuda(), k.t().contiguous().cuda(), v.cuda()).cpu()
    check_bf16_matmul(o, formulas.attention_ref(q, k, v))


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("out_dtype", [f32, bf16])
@pytest.mark.parametrize("d", [8, 16, 24, 32, 40, 72, 96, 120])
def test_head_dims_narrower_than_the_tile(d, out_dtype, causal):
    """Head dimensions below the 64- or 128-column tile: TMA zero-fills the missing columns of Q,
    K and V, and only ``d`` columns of O are stored."""
    B, H, Sq, Skv = 2, 2, 200, 328
    q, k, v = _inputs(B, H, Sq, Skv, d)
    kern = build_flash_attention(B, H, Sq, Skv, d, causal=causal, out_dtype=out_dtype)
    o = kern(q.cuda(), k.cuda(), v.cuda())
    check_bf16_matmul(o.cpu(), formulas.attention_ref(q, k, v, causal=causal))
    # same arithmetic as the full-width kernel on explicitly zero-padded operands
    full = 64 if d <= 64 else 128
    pad = lambda t: torch.nn.functional.pad(t, (0, full - d)).contiguous()
    wide = build_flash_attention(B, H, Sq, Skv, full, causal=causal, out_dtype=out_dtype, sm_scale=d ** -0.5)
    ow = wide(pad(q).cuda(), pad(k).cuda(), pad(v).cuda())
    assert torch.equal(ow[..., :d], o) and (ow[..., d:] == 0).all()


# ---- batched form ------------------------------------------------------------------------

@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("B,H,Sq,Skv", [(1, 1, 128, 128), (2, 3, 256, 256), (1, 2, 384, 384), (2, 2, 512, 1024),
                                        (1, 4, 1024, 1024), (1, 1, 128, 640)])
def test_batched(B, H, Sq, Skv, d, causal):
    q, k, v = _inputs(B, H, Sq, Skv, d)
    o = _run(q, k, v, causal=causal)
    check_bf16_matmul(o, formulas.attention_ref(q, k, v, causal=causal))


@pytest.mark.parametrize("d", [64, 128])
def test_causal_head_groups_with_a_partial_last_group(d):
    """Causal launches deal query blocks out heaviest-first across groups of 16 heads; 21 heads
    leave a last group of 5, and 600 rows a partial last query block."""
    q, k, v = _inputs(3, 7, 600, 600, d)
    o = _run(q, k, v, causal=True)
    check_bf16_matmul(o, formulas.attention_ref(q, k, v, causal=True))


@pytest.mark.parametrize("causal", [False, True])
def test_large_scores_rescale_path(causal):
    """Unnormalised Q.K with growing magnitude along the keys forces the running maximum to move
    by more than the lazy-rescale threshold several times."""
    B, H, S, d = 1, 2, 1024, 64
    q, k, v = _inputs(B, H, S, S, d)
    ramp = torch.linspace(0.2, 3.0, S)[None, None, :, None]
    k = (k.float() * ramp).to(torch.bfloat16)
    o = _run(q, k, v, causal=causal, sm_scale=1.0)
    check_bf16_matmul(o, formulas.attention_ref(q, k, v, causal=causal, sm_scale=1.0))


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("first_tile", [False, True])
@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("jump", [12.0, 60.0, 140.0, 400.0])
def test_late_dominant_key_at_every_chunk_position(d, jump, first_tile, causal):
    """Interior K/V tiles are exponentiated against the maximum already in use and accepted only if
    the row sums stay small.  A key far above everything seen so far, placed in a later tile at each
    position of a 32-key chunk in turn (positions differ in whether the MUFU unit or the FMA-pipe
    polynomial, whose argument is clamped, evaluates them), must send the rows to the exact path.
    ``jump`` is the score gap in natural units: around the 2^8 acceptance bound, far above it, and
    beyond what fp32 can exponentiate.  For the large gaps the output is that key's V row.
    ``first_tile`` puts the key into the second half of the FIRST tile instead, where the reference
    maximum is an estimate from the tile's first 64 scores; ``causal`` makes the key's tile the
    masked (diagonal) one for a third of the queries, which has a speculative path of its own."""
    B, H, S = 1, 1, 384
    g = torch.Generator().manual_seed(17)
    q = torch.zeros(B, H, S, d)
    q[..., 0] = 1.0                                  # score of any query against key j is k[j, 0]
    qb = q.to(torch.bfloat16)
    v = torch.randn(B, H, S, d, generator=g).to(torch.bfloat16)
    for pos in range(32):
        hot = (64 if first_tile else 128) + 32 + pos     # a key of the first tile's second half / of the second tile
        k = torch.zeros(B, H, S, d)
        k[0, 0, hot, 0] = jump
        kb = k.to(torch.bfloat16)
        o = _run(qb, kb, v, sm_scale=1.0, causal=causal)
        check_bf16_matmul(o, formulas.attention_ref(qb, kb, v, sm_scale=1.0, causal=causal))
        if jump >= 60.0:
            seen = slice(hot, S) if causal else slice(0, S)      # queries that see the key
            assert formulas.rel_fro(o[0, 0, seen], v[0, 0, hot].float().expand(S, d)[seen]) < 1e-2, pos


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("d", [64, 128])
@pytest.mark.parametrize("Sq,Skv", [(1, 1), (5, 40), (100, 100), (129, 300), (200, 513), (257, 257), (383, 1000)])
def test_ragged_sequence_lengths(Sq, Skv, d, causal):
    """Lengths that are not multiples of the 128-wide tiles: zero-filled partial tiles + masks."""
    q, k, v = _inputs(1, 3, Sq, Skv, d)
    o = _run(q, k, v, causal=causal)
    check_bf16_matmul(o, formulas.attention_ref(q, k, v, causal=causal))


def test_ragged_single_head_reference_layout():
    """The reference's call form with K transposed; N_seq a multiple of 8 but not of 64 or 128."""
    M_q, N_seq, HD = 192, 200, 64
    torch.manual_seed(1)
    q = (torch.randn(M_q, HD) * 0.3).to(torch.bfloat16)
    k = (torch.randn(N_seq, HD) * 0.3).to(torch.bfloat16)
    v = (torch.randn(N_seq, HD) * 0.3).to(torch.bfloat16)
    o = build_flash_attention_hopper(M_q, N_seq, HD)(q.cuda(), k.t().contiguous().cuda(), v.cuda()).cpu()
    check_bf16_matmul(o, formulas.attention_ref(q, k, v))
    with pytest.raises(AssertionError, match="divisible by 8"):
        build_flash_attention_hopper(128, 100, 64)


def test_bf16_output_and_scale():
    q, k, v = _inputs(2, 2, 256, 256, 128)
    o = _run(q, k, v, out_dtype=bf16, sm_scale=0.05)
    assert o.dtype == torch.bfloat16
    check_bf16_matmul(o, formulas.attention_ref(q, k, v, sm_scale=0.05))


@pytest.mark.parametrize("causal", [False, True])
def test_shared_memory_p_variant_agrees(causal):
    """P through shared memory (SS MMA) and P through TMEM (TS MMA) are the same arithmetic."""
    q, k, v = _inputs(1, 3, 512, 512, 64)
    a = _run(q, k, v, causal=causal)
    b = _run(q, k, v, causal=causal, flags=1 << 17)
    ref = formulas.attention_ref(q, k, v, causal=causal)
    check_bf16_matmul(a, ref)
    check_bf16_matmul(b, ref)
    assert formulas.rel_fro(a, b) < 1e-5


def test_causal_first_row_and_independence_of_future_keys():
    q, k, v = _inputs(1, 2, 512, 512, 64)
    o = _run(q, k, v, causal=True)
    torch.testing.assert_close(o[:, :, 0], v[:, :, 0].float(), rtol=1e-2, atol=1e-2)
    k2, v2 = k.clone(), v.clone()
    k2[:, :, 300:] = 0
    v2[:, :, 300:] = 7
    o2 = _run(q, k2, v2, causal=True)
    assert torch.equal(o[:, :, :300], o2[:, :, :300])


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("d", [64, 128])
def test_benchmark_configuration(d, causal):
    """B=4, H=16, S=4096: the kernel runs on all 64 heads; the oracle is evaluated on a
    sample of them (each head is an independent problem)."""
    B, H, S = 4, 16, 4096
    q, k, v = _inputs(B, H, S, S, d)
    o = _run(q, k, v, causal=causal, out_dtype=bf16)
    assert torch.isfinite(o.float()).all()
    for b, h in [(0, 0), (1, 7), (3, 15)]:
        ref = formulas.attention_ref(q[b, h], k[b, h], v[b, h], causal=causal)
        check_bf16_matmul(o[b, h], ref)


def test_no_device_wait_gave_up():
    from pyptx_b200 import _native
    _native.device_status()


@pytest.mark.parametrize("causal", [False, True])
@pytest.mark.parametrize("d", [32, 64, 128])
def test_log_sum_exp_output(d, causal):
    B, H, Sq, Skv = 2, 2, 300, 456
    q, k, v = _inputs(B, H, Sq, Skv, d)
    kern = build_flash_attention(B, H, Sq, Skv, d, causal=causal, out_dtype=f32, return_lse=True)
    o, lse = kern(q.cuda(), k.cuda(), v.cuda())
    plain = build_flash_attention(B, H, Sq, Skv, d, causal=causal, out_dtype=f32)(q.cuda(), k.cuda(), v.cuda())
    assert torch.equal(o, plain)
    ref = formulas.attention_lse_ref(q, k, causal=causal)
    assert lse.shape == ref.shape and lse.dtype == torch.float32
    assert torch.allclose(lse.cpu(), ref, atol=2e-3, rtol=0)      # ex2.approx / cubic exp2 in the row sum
    # softmax rebuilt from lse reproduces the output: exp(s - lse) @ v
    s = (q.float() @ k.float().transpose(-1, -2)) * d ** -0.5
    if causal:
        s = s.masked_fill(~torch.ones(Sq, Skv, dtype=torch.bool).tril(diagonal=Skv - Sq), float("-inf"))
    check_bf16_matmul(o.cpu(), torch.exp(s - lse.cpu()[..., None]) @ v.float())
