"""The CPU oracle against the golden vectors generated from the reference tree
(tests/golden/make_golden.py) and against the known answers in the reference's
own tests (tests/test_typed_wrappers.py:407-438)."""
import json
import os

import numpy as np
import pytest
import torch

import oracle
from oracle import encodings, formulas, inputs


@pytest.fixture(scope="module")
def enc(golden_dir):
    with open(os.path.join(golden_dir, "encodings.json")) as f:
        return json.load(f)


@pytest.fixture(scope="module")
def rows(golden_dir):
    return np.load(os.path.join(golden_dir, "row_refs.npz"))


@pytest.fixture(scope="module")
def mats(golden_dir):
    return np.load(os.path.join(golden_dir, "matmul_refs.npz"))


def _bf16(a: np.ndarray) -> torch.Tensor:
    return torch.from_numpy(a.copy()).view(torch.bfloat16)


# ---- integer encodings: bit-exact --------------------------------------------

def test_idesc_known_answers():
    # tests/test_typed_wrappers.py:407-425 of the reference
    assert encodings.instr_desc_f16bf16_f32(m=128, n=256, ab_dtype="bf16") == 0x08400490
    assert encodings.instr_desc_f16bf16_f32(m=128, n=256, ab_dtype="f16") == 0x08400010
    assert encodings.instr_desc_f16bf16_f32(m=128, n=256, ab_dtype="f16", scale_a=-1) == 0x08402010
    assert encodings.instr_desc_f16bf16_f32(m=128, n=256, ab_dtype="tf32") == 0x08400910
    assert encodings.instr_desc_f16bf16_f32(m=256, n=256) == 0x10400490


def test_idesc_matches_reference_grid(enc):
    assert len(enc["idesc"]) == 288
    for case in enc["idesc"]:
        assert encodings.instr_desc_f16bf16_f32(**case["kw"]) == case["value"], case["kw"]


def test_smem_desc_constant(enc):
    # tests/test_typed_wrappers.py:427-438 of the reference; gemm_highperf_blackwell.py:50
    assert enc["mma_desc_b128"] == 0x4000404000010000
    assert encodings.SMEM_DESC_SW128_KMAJOR == enc["mma_desc_b128"] == enc["grouped_mma_desc"]
    assert encodings.smem_desc(0, stride_bytes=1024, leading_bytes=16, swizzle="128B") == enc["mma_desc_b128"]
    assert encodings.smem_desc(0x12340, stride_bytes=1024) == enc["mma_desc_b128"] | ((0x12340 >> 4) & 0x3FFF)


def test_swizzle_tables(enc):
    for kind, table in enc["swizzle"].items():
        got = [encodings.swizzle(o, kind) for o in range(0, 2048, 16)]
        assert got == table, kind
    assert [encodings.swizzle_128b(o) for o in range(0, 2048, 16)] == enc["swizzle"]["128B"]
    # a permutation of 16-byte chunks inside every 1024-byte atom
    assert sorted(enc["swizzle"]["128B"][:64]) == list(range(0, 1024, 16))


# ---- floating-point formulas vs the reference's own *_ref outputs --------------
# The golden values were produced by the reference's functions in numpy float32;
# torch float32 on the same inputs differs only by summation order.
ROW_TOL = dict(rtol=2e-6, atol=2e-6)


@pytest.mark.parametrize("B,N", [(4, 64), (16, 512)])
def test_rms_norm_vs_reference(rows, B, N):
    x, w = torch.from_numpy(rows[f"rms_{B}_{N}_x"]), torch.from_numpy(rows[f"rms_{B}_{N}_w"])
    torch.testing.assert_close(formulas.rms_norm_ref(x, w), torch.from_numpy(rows[f"rms_{B}_{N}_y"]), **ROW_TOL)


@pytest.mark.parametrize("B,N", [(4, 64), (16, 512)])
def test_layer_norm_vs_reference(rows, B, N):
    x, w, b = (torch.from_numpy(rows[f"ln_{B}_{N}_{k}"]) for k in "xwb")
    torch.testing.assert_close(formulas.layer_norm_ref(x, w, b), torch.from_numpy(rows[f"ln_{B}_{N}_y"]), **ROW_TOL)
    torch.testing.assert_close(torch.nn.functional.layer_norm(x, (N,), w, b, 1e-5),
                               torch.from_numpy(rows[f"ln_{B}_{N}_y"]), **ROW_TOL)


@pytest.mark.parametrize("B,N", [(4, 64), (16, 512)])
def test_swiglu_vs_reference(rows, B, N):
    g, u = torch.from_numpy(rows[f"swiglu_{B}_{N}_g"]), torch.from_numpy(rows[f"swiglu_{B}_{N}_u"])
    torch.testing.assert_close(formulas.swiglu_ref(g, u), torch.from_numpy(rows[f"swiglu_{B}_{N}_y"]), **ROW_TOL)


@pytest.mark.parametrize("B,N", [(4, 64), (16, 512)])
def test_softmax_vs_reference(rows, B, N):
    x = torch.from_numpy(rows[f"softmax_{B}_{N}_x"])
    y = formulas.softmax_ref(x)
    torch.testing.assert_close(y, torch.from_numpy(rows[f"softmax_{B}_{N}_y"]), **ROW_TOL)
    torch.testing.assert_close(y.sum(-1), torch.ones(B), rtol=1e-5, atol=1e-5)


@pytest.mark.parametrize("M,N,K", [(128, 256, 64), (128, 256, 128)])
def test_gemm_vs_reference(mats, M, N, K):
    a, bt = _bf16(mats[f"gemm_{M}_{N}_{K}_a"]), _bf16(mats[f"gemm_{M}_{N}_{K}_bt"])
    torch.testing.assert_close(formulas.gemm_ref(a, bt), torch.from_numpy(mats[f"gemm_{M}_{N}_{K}_d"]),
                               rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("G,M,N,K", [(2, 128, 64, 64), (2, 128, 128, 128)])
def test_grouped_vs_reference(mats, G, M, N, K):
    a, bt = _bf16(mats[f"grouped_{G}_{M}_{N}_{K}_a"]), _bf16(mats[f"grouped_{G}_{M}_{N}_{K}_bt"])
    torch.testing.assert_close(formulas.grouped_gemm_ref(a, bt, G),
                               torch.from_numpy(mats[f"grouped_{G}_{M}_{N}_{K}_c"]), rtol=1e-5, atol=1e-6)


@pytest.mark.parametrize("M_q,N_seq,HD", [(128, 128, 64), (128, 256, 64), (128, 128, 128)])
def test_attention_vs_reference(mats, M_q, N_seq, HD):
    q, k, v = (_bf16(mats[f"fa_{M_q}_{N_seq}_{HD}_{n}"]) for n in "qkv")
    o = formulas.attention_ref(q, k, v)
    torch.testing.assert_close(o, torch.from_numpy(mats[f"fa_{M_q}_{N_seq}_{HD}_o"]), rtol=1e-5, atol=1e-6)
    # batched form agrees with the per-head form
    ob = formulas.attention_ref(q[None].repeat(3, 1, 1), k[None].repeat(3, 1, 1), v[None].repeat(3, 1, 1))
    torch.testing.assert_close(ob[2], o, rtol=1e-5, atol=1e-6)


def test_causal_attention_properties():
    q, k, v = inputs.attention_inputs(2, 64, 64, 32)
    o = formulas.attention_ref(q, k, v, causal=True)
    # row 0 sees only key 0 -> output row 0 equals v[0]
    torch.testing.assert_close(o[:, 0], v[:, 0].float(), rtol=1e-6, atol=1e-6)
    # last row sees everything -> equals the non-causal last row
    torch.testing.assert_close(o[:, -1], formulas.attention_ref(q, k, v)[:, -1], rtol=1e-5, atol=1e-6)


def test_inputs_are_seeded_and_shaped():
    a1, b1 = inputs.gemm_inputs(128, 256, 64)
    a2, b2 = inputs.gemm_inputs(128, 256, 64)
    assert torch.equal(a1, a2) and torch.equal(b1, b2)
    assert a1.shape == (128, 64) and b1.shape == (256, 64) and a1.dtype == torch.bfloat16
    x, w = inputs.rms_norm_inputs(8, 64)
    assert x.shape == (8, 64) and w.shape == (64,) and abs(float(w.mean()) - 1.0) < 0.05
    a, bt = inputs.grouped_gemm_inputs(2, 128, 64, 64)
    assert a.shape == (256, 64) and bt.shape == (128, 64)
    (sx,) = inputs.softmax_inputs(64, 256)
    assert 1.8 < float(sx.std()) < 2.2


def test_error_metrics():
    r = torch.ones(4, 4)
    assert formulas.rel_fro(r, r) == 0.0
    assert abs(formulas.rel_fro(r * 1.01, r) - 0.01) < 1e-6
    assert abs(formulas.max_scaled_err(r + 0.5, r) - 0.5) < 1e-12
    assert oracle.rms_norm_ref is formulas.rms_norm_ref


def test_gemm_bias_act_ref_composes_the_reference_formulas():
    a, bt = inputs.gemm_inputs(128, 256, 64)
    bias = torch.linspace(-1, 1, 256)
    base = formulas.gemm_ref(a, bt)
    assert torch.equal(formulas.gemm_bias_act_ref(a, bt), base)
    assert torch.equal(formulas.gemm_bias_act_ref(a, bt, bias, "relu"), torch.relu(base + bias))
    assert torch.allclose(formulas.gemm_bias_act_ref(a, bt, None, "silu"), base * torch.sigmoid(base), atol=1e-6)
    x = base + bias
    assert torch.allclose(formulas.gemm_bias_act_ref(a, bt, bias, "gelu"), 0.5 * x * (1 + torch.erf(x / 2 ** 0.5)), atol=1e-6)
