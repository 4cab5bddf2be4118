"""GPU parity of the tcgen05 GEMMs (1-SM, 2-SM, grouped) against the fp32-accumulated CPU
oracle: known-answer patterns that pin the tensor-core operand layout (the ideas of the
reference's examples/blackwell/tcgen05_suite.py:55-241), the golden vectors, the
reference's shape lists (gemm_highperf_blackwell.py:1337-1354, grouped_gemm.py:343-352)
and the benchmark configurations."""
import os

import numpy as np
import pytest
import torch

from oracle import formulas, inputs
from pyptx_b200 import _ids
from pyptx_b200.examples.blackwell.gemm_highperf_blackwell import build_gemm, build_gemm_2sm
from pyptx_b200.examples.blackwell.grouped_gemm import (build_grouped_gemm, build_grouped_gemm_swiglu,
                                                         build_grouped_gemm_varlen)
from pyptx_b200.kernel import NativeKernel
from pyptx_b200.types import bf16
from tests.gpu_util import check_bf16_matmul

pytestmark = pytest.mark.gpu

BUILDERS = {"1sm": build_gemm, "2sm": build_gemm_2sm}


def _bf16(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(a.copy()).view(torch.bfloat16)


def _min_m(kind):
    return 256 if kind == "2sm" else 128


@pytest.fixture(scope="module")
def mats(golden_dir):
    return np.load(os.path.join(golden_dir, "matmul_refs.npz"))


# ---- known answers ---------------------------------------------------------------

@pytest.mark.parametrize("kind", ["1sm", "2sm"])
@pytest.mark.parametrize("K", [64, 128, 256, 320, 1024])
def test_ones_gives_k(kind, K):
    """ones x ones = K in every element: exact in bf16 inputs / fp32 accumulate."""
    M, N = _min_m(kind), 256
    a = torch.ones(M, K, dtype=torch.bfloat16, device="cuda")
    bt = torch.ones(N, K, dtype=torch.bfloat16, device="cuda")
    d = BUILDERS[kind](M, N, K)(a, bt)
    assert d.dtype == torch.float32 and d.shape == (M, N)
    assert torch.equal(d.cpu(), torch.full((M, N), float(K)))


@pytest.mark.parametrize("kind", ["1sm", "2sm"])
def test_row_and_column_coded_operands(kind):
    """A[i,:] = i+1 on one k, B = e_k  ->  D[i,j] pins row/column/k placement exactly."""
    M, N, K = 2 * _min_m(kind), 512, 128
    a = torch.zeros(M, K)
    bt = torch.zeros(N, K)
    a[:, 3] = torch.arange(1, M + 1, dtype=torch.float32) % 251      # exactly representable in bf16
    bt[:, 3] = torch.arange(1, N + 1, dtype=torch.float32) % 127
    a[:, 77] = 1.0
    bt[:, 77] = 2.0
    ref = a @ bt.t()
    d = BUILDERS[kind](M, N, K)(a.to(torch.bfloat16).cuda(), bt.to(torch.bfloat16).cuda())
    assert torch.equal(d.cpu(), ref)


@pytest.mark.parametrize("kind", ["1sm", "2sm"])
def test_k_lane_map(kind):
    """Each k contributes with its own weight: D = sum_k 2^-(k%8) * (k//8+1) pattern, exact."""
    M, N, K = _min_m(kind), 256, 64
    a = torch.zeros(M, K)
    bt = torch.zeros(N, K)
    for k in range(K):
        a[:, k] = 2.0 ** -(k % 8)
        bt[:, k] = float(k // 8 + 1)
    ref = a @ bt.t()
    d = BUILDERS[kind](M, N, K)(a.to(torch.bfloat16).cuda(), bt.to(torch.bfloat16).cuda())
    assert torch.equal(d.cpu(), ref)


@pytest.mark.parametrize("kind", ["1sm", "2sm"])
def test_identity_selects_rows(kind):
    """A = I (K = M): D = B, bit-exact; exercises every 128-byte swizzle row of both operands."""
    M = K = 256
    N = 256
    g = torch.Generator().manual_seed(7)
    b = torch.randn(K, N, generator=g).to(torch.bfloat16)
    a = torch.eye(M, K).to(torch.bfloat16)
    d = BUILDERS[kind](M, N, K)(a.cuda(), b.t().contiguous().cuda())
    assert torch.equal(d.cpu(), b.float())


# ---- golden vectors and the reference's shape lists ----------------------------------

@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (128, 256, 128)])
def test_golden_gemm(mats, M, N, K):
    a, bt = _bf16(mats[f"gemm_{M}_{N}_{K}_a"]), _bf16(mats[f"gemm_{M}_{N}_{K}_bt"])
    d = build_gemm(M, N, K)(a.cuda(), bt.cuda()).cpu()
    ref = torch.from_numpy(mats[f"gemm_{M}_{N}_{K}_d"])
    check_bf16_matmul(d, ref, 1e-5)   # same bf16 inputs, fp32 accumulate: only summation order differs
    assert torch.allclose(d, ref, atol=5e-2, rtol=5e-2)  # the reference's own criterion (:1270)


REF_GEMM_SHAPES = [(128, 256, 64), (128, 256, 128), (256, 256, 256), (256, 512, 256), (512, 512, 512),
                   (1024, 1024, 512), (384, 768, 192), (2048, 2048, 2048)]


@pytest.mark.parametrize("kind", ["1sm", "2sm"])
@pytest.mark.parametrize("M,N,K", REF_GEMM_SHAPES)
def test_gemm_shapes(kind, M, N, K):
    if M % _min_m(kind):
        pytest.skip("M not divisible by the 2-SM tile")
    a, bt = inputs.gemm_inputs(M, N, K)
    d = BUILDERS[kind](M, N, K)(a.cuda(), bt.cuda()).cpu()
    check_bf16_matmul(d, formulas.gemm_ref(a, bt), 1e-4)


@pytest.mark.parametrize("kind", ["1sm", "2sm"])
def test_pipeline_wraparound_and_many_tiles(kind):
    """K-tiles = stages-1, stages, stages+1, 2*stages+1 and more tiles than SMs: phase bits of the
    shared-memory ring and of the double-buffered accumulator must stay consistent."""
    for K in (192, 256, 320, 384, 448, 576, 832):
        a, bt = inputs.gemm_inputs(256, 256, K)
        d = BUILDERS[kind](256, 256, K)(a.cuda(), bt.cuda()).cpu()
        check_bf16_matmul(d, formulas.gemm_ref(a, bt), 1e-4)
    M, N, K = 4096, 4096 + 256, 128          # 544 / 272 tiles: > 3 per SM, odd count per SM
    a, bt = inputs.gemm_inputs(M, N, K)
    d = BUILDERS[kind](M, N, K)(a.cuda(), bt.cuda()).cpu()
    check_bf16_matmul(d, formulas.gemm_ref(a, bt), 1e-4)


@pytest.mark.parametrize("kind", ["1sm", "2sm"])
@pytest.mark.parametrize("width", [1, 3, 16, 64])
def test_raster_band_width(kind, width):
    M, N, K = 1280, 768, 128
    a, bt = inputs.gemm_inputs(M, N, K)
    d = BUILDERS[kind](M, N, K, grid_tile_width=width)(a.cuda(), bt.cuda()).cpu()
    check_bf16_matmul(d, formulas.gemm_ref(a, bt), 1e-4)


@pytest.mark.parametrize("kind", ["1sm", "2sm"])
def test_bf16_output(kind):
    M, N, K = 512, 512, 256
    a, bt = inputs.gemm_inputs(M, N, K)
    d = BUILDERS[kind](M, N, K, out_dtype=bf16)(a.cuda(), bt.cuda())
    assert d.dtype == torch.bfloat16
    ref = formulas.gemm_ref(a, bt)
    assert torch.equal(d.cpu(), ref.to(torch.bfloat16)) or formulas.rel_fro(d.float().cpu(), ref) < 4e-3
    check_bf16_matmul(d.cpu(), ref)


@pytest.mark.parametrize("kind_id", [_ids.K_GEMM_1SM, _ids.K_GEMM_2SM])
def test_direct_store_epilogue_agrees(kind_id):
    """The register-to-global epilogue (a debugging variant) and the TMA-store epilogue give
    identical bits."""
    from pyptx_b200.specs import Tile
    from pyptx_b200.types import f32
    M, N, K = 512, 768, 256
    a, bt = inputs.gemm_inputs(M, N, K)
    specs = dict(in_specs=(Tile(M, K, bf16), Tile(N, K, bf16)), out_specs=(Tile(M, N, f32),))
    tma = NativeKernel("gemm_tma", kind_id, (M, N, K), **specs)(a.cuda(), bt.cuda())
    direct = NativeKernel("gemm_direct", kind_id, (M, N, K), flags=1 << 16, **specs)(a.cuda(), bt.cuda())
    assert torch.equal(tma, direct)


@pytest.mark.parametrize("kind", ["1sm", "2sm"])
@pytest.mark.parametrize("S", [2048, 4096])
def test_benchmark_sizes(kind, S):
    a, bt = inputs.gemm_inputs(S, S, S)
    d = BUILDERS[kind](S, S, S)(a.cuda(), bt.cuda()).cpu()
    check_bf16_matmul(d, formulas.gemm_ref(a, bt))


@pytest.mark.parametrize("kind", ["1sm", "2sm"])
def test_8192_cubed_properties(kind):
    """Full benchmark size.  The fp32 CPU product of 8192^3 takes too long for a unit test, so
    the oracle is evaluated on sampled row and column blocks, and linearity D(A1+A2) = D(A1)+D(A2)
    (exact for operands chosen so that no bf16 rounding occurs) covers the whole output."""
    S = 8192
    a, bt = inputs.gemm_inputs(S, S, S)
    k = BUILDERS[kind](S, S, S)
    d = k(a.cuda(), bt.cuda())
    for r0 in (0, 3968, 8064):
        ref = formulas.gemm_ref(a[r0:r0 + 128], bt)
        check_bf16_matmul(d[r0:r0 + 128].cpu(), ref, 1e-4)
    for c0 in (256, 7936):
        ref = formulas.gemm_ref(a, bt[c0:c0 + 64])
        check_bf16_matmul(d[:, c0:c0 + 64].cpu(), ref, 1e-4)
    ones = torch.ones(S, S, dtype=torch.bfloat16, device="cuda")
    dk = k(ones, ones)
    assert bool((dk == float(S)).all())
    del d, dk


# ---- grouped ---------------------------------------------------------------------

@pytest.mark.parametrize("G,M,N,K", [(2, 128, 64, 64), (2, 128, 128, 128)])
def test_golden_grouped(mats, G, M, N, K):
    a, bt = _bf16(mats[f"grouped_{G}_{M}_{N}_{K}_a"]), _bf16(mats[f"grouped_{G}_{M}_{N}_{K}_bt"])
    c = build_grouped_gemm(G, M, N, K)(a.cuda(), bt.cuda()).cpu()
    ref = torch.from_numpy(mats[f"grouped_{G}_{M}_{N}_{K}_c"])
    check_bf16_matmul(c, ref, 1e-5)
    assert torch.allclose(c, ref, atol=5e-3, rtol=5e-3)   # the reference's own criterion (:308)


@pytest.mark.parametrize("G,M,N,K", [(1, 128, 64, 64), (4, 128, 128, 128), (8, 512, 128, 512), (8, 1024, 128, 1024),
                                     (3, 256, 192, 320), (4, 2048, 256, 2048), (8, 2048, 256, 2048),
                                     (16, 128, 512, 64)])
def test_grouped_shapes(G, M, N, K):
    a, bt = inputs.grouped_gemm_inputs(G, M, N, K)
    c = build_grouped_gemm(G, M, N, K)(a.cuda(), bt.cuda()).cpu()
    check_bf16_matmul(c, formulas.grouped_gemm_ref(a, bt, G), 1e-4)


def test_grouped_experts_do_not_mix():
    """Expert g's output depends only on expert g's operands."""
    G, M, N, K = 4, 256, 256, 128
    a, bt = inputs.grouped_gemm_inputs(G, M, N, K)
    k = build_grouped_gemm(G, M, N, K)
    base = k(a.cuda(), bt.cuda()).cpu()
    a2 = a.clone()
    a2[2 * M:3 * M] = 0
    out = k(a2.cuda(), bt.cuda()).cpu()
    assert torch.equal(out[:2 * M], base[:2 * M]) and torch.equal(out[3 * M:], base[3 * M:])
    assert torch.count_nonzero(out[2 * M:3 * M]) == 0


@pytest.mark.parametrize("out", ["f32", "bf16"])
@pytest.mark.parametrize("G,M,F,K", [(1, 128, 128, 64), (2, 256, 256, 128), (4, 512, 384, 320), (8, 2048, 128, 2048),
                                     (3, 128, 1024, 64)])
def test_grouped_gemm_with_fused_swiglu(G, M, F, K, out):
    """silu(A Wg^T) * (A Wu^T) from one kernel equals the two reference ops composed."""
    from pyptx_b200.types import f32
    a, w = inputs.grouped_gemm_inputs(G, M, 2 * F, K)        # w: [G*2F, K], per expert gate rows then up rows
    w = (w.float() * 4.0).to(torch.bfloat16)                  # spread the gate values over the sigmoid's bend
    ref = formulas.grouped_gemm_swiglu_ref(a, w, G)
    k = build_grouped_gemm_swiglu(G, M, F, K, out_dtype=bf16 if out == "bf16" else f32)
    got = k(a.cuda(), w.cuda())
    assert got.shape == (G * M, F) and got.dtype == (torch.bfloat16 if out == "bf16" else torch.float32)
    check_bf16_matmul(got.cpu(), ref, 5e-3 if out == "bf16" else 1e-4)
    # and against this library's own two-kernel path
    from pyptx_b200.examples.blackwell.swiglu import build_fused_silu_mul
    c = build_grouped_gemm(G, M, 2 * F, K)(a.cuda(), w.cuda())
    two = build_fused_silu_mul(G * M, F)(c[:, :F].contiguous(), c[:, F:].contiguous())
    check_bf16_matmul(got.float().cpu(), two.cpu(), 5e-3 if out == "bf16" else 1e-5)


@pytest.mark.parametrize("counts,N,K", [
    ([128], 64, 64),
    ([256, 0, 384, 128], 256, 128),            # an expert with no tokens
    ([0, 0, 512], 128, 320),
    ([1024, 128, 2048, 256, 0, 640, 128, 896], 256, 512),
    ([128] * 40, 512, 64),
])
@pytest.mark.parametrize("slack", [0, 384])
def test_variable_size_grouped_gemm(counts, N, K, slack):
    """Per-expert row counts from a device-side offsets array; capacity above the routed rows stays untouched."""
    G = len(counts)
    offs = [0]
    for c in counts:
        offs.append(offs[-1] + c)
    M_total = offs[-1] + slack
    g = torch.Generator().manual_seed(G * 1009 + M_total * 997 + N * 17 + K)
    a = (torch.randn(M_total, K, generator=g) / K ** 0.5).to(torch.bfloat16)
    bt = (torch.randn(G * N, K, generator=g) / K ** 0.5).to(torch.bfloat16)
    ref = formulas.grouped_gemm_varlen_ref(a, bt, offs, N)
    k = build_grouped_gemm_varlen(G, M_total, N, K)
    offsets = torch.tensor(offs, dtype=torch.int32, device="cuda")
    # pre-fill the output allocation pattern: run once, then check the untouched tail through a sentinel run
    out = k(a.cuda(), bt.cuda(), offsets).cpu()
    used = offs[-1]
    check_bf16_matmul(out[:used], ref[:used], 1e-4)
    # same kernel object, another routing outcome with the same capacity
    if G >= 2 and counts[0] >= 256:
        offs2 = list(offs)
        offs2[1] -= 128                      # move one row block from expert 0 to expert 1
        out2 = k(a.cuda(), bt.cuda(), torch.tensor(offs2, dtype=torch.int32, device="cuda")).cpu()
        ref2 = formulas.grouped_gemm_varlen_ref(a, bt, offs2, N)
        check_bf16_matmul(out2[:used], ref2[:used], 1e-4)


def test_variable_size_grouped_gemm_leaves_capacity_rows_alone():
    G, N, K = 2, 256, 64
    offs = [0, 128, 256]
    M_total = 512
    a = torch.ones(M_total, K, dtype=torch.bfloat16)
    bt = torch.ones(G * N, K, dtype=torch.bfloat16)
    k = build_grouped_gemm_varlen(G, M_total, N, K)
    offsets = torch.tensor(offs, dtype=torch.int32, device="cuda")
    # torch.empty reuses the block freed by the sentinel tensor, so unwritten rows keep the sentinel
    sentinel = torch.full((M_total, N), -7.0, device="cuda")
    ptr = sentinel.data_ptr()
    del sentinel
    out = k(a.cuda(), bt.cuda(), offsets)
    assert bool((out[:256] == float(K)).all())
    if out.data_ptr() == ptr:
        assert bool((out[256:] == -7.0).all())


def test_no_device_wait_gave_up():
    from pyptx_b200 import _native
    _native.device_status()


# ---- tile shapes --------------------------------------------------------------------

@pytest.mark.parametrize("kind", ["1sm", "2sm"])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("shape", [(512, 256, 64), (1024, 768, 576), (2560, 512, 1024)])
def test_double_height_tile_equals_single_height(kind, out_dtype, shape):
    """The double-height tile (two A blocks per B block, no second accumulator buffer) must give
    the single-height kernel's bits: same MMAs, same accumulation order along K."""
    from pyptx_b200.types import f32
    M, N, K = shape
    a, bt = inputs.gemm_inputs(M, N, K)
    spec = bf16 if out_dtype == torch.bfloat16 else f32
    wide = BUILDERS[kind](M, N, K, tile="wide", out_dtype=spec)
    narrow = BUILDERS[kind](M, N, K, tile="narrow", out_dtype=spec)
    ad, bd = a.cuda(), bt.cuda()
    dw, dn = wide(ad, bd), narrow(ad, bd)
    check_bf16_matmul(dw.cpu(), formulas.gemm_ref(a, bt), 1e-2 if out_dtype == torch.bfloat16 else 1e-4)
    assert torch.equal(dw, dn)


@pytest.mark.parametrize("kind", ["1sm", "2sm"])
def test_double_height_tile_many_tiles_per_cta(kind):
    """Three to four double-height tiles per CTA (pair): both accumulators are reused and their
    barrier phases wrap."""
    M, N, K = 4096, 8192, 128
    a, bt = inputs.gemm_inputs(M, N, K)
    ad, bd = a.cuda(), bt.cuda()
    dw = BUILDERS[kind](M, N, K, tile="wide")(ad, bd)
    dn = BUILDERS[kind](M, N, K, tile="narrow")(ad, bd)
    assert torch.equal(dw, dn)
    rows = slice(1024, 1024 + 256)
    check_bf16_matmul(dw[rows].cpu(), formulas.gemm_ref(a[rows], bt), 1e-4)


def test_tile_choice_is_validated():
    with pytest.raises(AssertionError, match="tile must be one of"):
        build_gemm_2sm(512, 256, 64, tile="tall")


# ---- fused bias / activation epilogue -------------------------------------------------

@pytest.mark.parametrize("kind", ["1sm", "2sm"])
@pytest.mark.parametrize("bias", [False, True])
@pytest.mark.parametrize("activation", [None, "relu", "gelu", "silu"])
@pytest.mark.parametrize("out_dtype", [torch.float32, torch.bfloat16])
def test_bias_activation_epilogue(kind, bias, activation, out_dtype):
    from pyptx_b200.types import f32
    if not bias and activation is None:
        pytest.skip("plain epilogue is covered above")
    M, N, K = 512, 768, 256
    a, bt = inputs.gemm_inputs(M, N, K)
    g = torch.Generator().manual_seed(M * 31 + N)
    b = torch.randn(N, generator=g) * 0.5
    ref = formulas.gemm_bias_act_ref(a, bt, b if bias else None, activation)
    spec = bf16 if out_dtype == torch.bfloat16 else f32
    for tile in ("narrow", "wide"):
        k = BUILDERS[kind](M, N, K, out_dtype=spec, bias=bias, activation=activation, tile=tile)
        assert len(k.in_specs) == (3 if bias else 2)
        args = (a.cuda(), bt.cuda()) + ((b.cuda(),) if bias else ())
        d = k(*args)
        check_bf16_matmul(d.cpu(), ref, 1e-2 if out_dtype == torch.bfloat16 else 2e-5)


def test_bias_epilogue_rejects_wrong_inputs():
    k = build_gemm(256, 256, 64, bias=True)
    a, bt = inputs.gemm_inputs(256, 256, 64)
    with pytest.raises((TypeError, ValueError)):
        k(a.cuda(), bt.cuda())                                   # bias missing
    with pytest.raises(TypeError):
        k(a.cuda(), bt.cuda(), torch.zeros(256, dtype=torch.bfloat16, device="cuda"))
    with pytest.raises(AssertionError, match="activation must be one of"):
        build_gemm(256, 256, 64, activation="tanh")


def test_2sm_entry_on_a_single_wave_problem_keeps_its_bits():
    """2048^3 has 128 tiles of 128 x 256: the 2-SM entry point runs it on the 1-SM shape (one CTA
    per tile, no cluster); tile="narrow" keeps the CTA pairs.  Same sums in the same order."""
    S = 2048
    a, bt = inputs.gemm_inputs(S, S, S)
    auto = build_gemm_2sm(S, S, S)
    pairs = build_gemm_2sm(S, S, S, tile="narrow")
    assert auto.cluster == (1, 1, 1) and pairs.cluster == (2, 1, 1)
    d0, d1, d2 = auto(a.cuda(), bt.cuda()), pairs(a.cuda(), bt.cuda()), build_gemm(S, S, S)(a.cuda(), bt.cuda())
    assert torch.equal(d0, d1) and torch.equal(d0, d2)
    # small problems (and anything with more than one wave) stay on CTA pairs
    assert build_gemm_2sm(512, 512, 256).cluster == (2, 1, 1) and build_gemm_2sm(4096, 4096, 256).cluster == (2, 1, 1)
