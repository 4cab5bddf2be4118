"""Helpers shared by the GPU parity tests."""
import torch

from oracle import formulas


def check_f32(out: torch.Tensor, ref: torch.Tensor, tol: float = 1e-5) -> None:
    """f32 row kernels: relative Frobenius error and the elementwise scaled error both within
    ``tol`` (1e-5, the tolerance the benchmark specification states for f32 row kernels)."""
    assert out.dtype == torch.float32 and out.shape == ref.shape
    assert torch.isfinite(out).all()
    fro = formulas.rel_fro(out, ref)
    mx = formulas.max_scaled_err(out, ref)
    assert fro <= tol and mx <= tol, f"rel_fro={fro:.3e} max_scaled={mx:.3e} (tol {tol:g})"


def check_bf16_matmul(out: torch.Tensor, ref: torch.Tensor, tol: float = 1e-2) -> float:
    """bf16 GEMM / attention: relative Frobenius error against the fp32-accumulated oracle
    within 1e-2 (the tolerance the benchmark specification states)."""
    assert out.shape == ref.shape, (out.shape, ref.shape)
    assert torch.isfinite(out.float()).all()
    fro = formulas.rel_fro(out.float(), ref)
    assert fro <= tol, f"rel_fro={fro:.3e} (tol {tol:g})"
    return fro
