"""Runs the reference's OWN sm_100a kernels (staged by prepare_ref.py under baseline/_ref) on
the GPU, through the reference's public ``build_*`` entry points and its PyTorch launch path,
and prints one JSON object with their throughput and their error against the torch formula.

    python baseline/run_pyptx.py            # every family, each in a child process with a time limit
    python baseline/run_pyptx.py gemm       # one family in this process

This is a comparison baseline only; nothing of this library is on that path.  Launches are
captured in a CUDA graph (the reference documents graph capture, docs/runtime/torch.md:78-104)
so that the figures are device time rather than Python dispatch time; if capture fails the
eager loop is timed instead and the entry says so.  The reference has no attention kernel for
sm_100a (its flash attention is wgmma / sm_90a only), so there is no attention row.
"""
from __future__ import annotations

import json
import os
import subprocess
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")
FAMILIES = ("rows", "gemm", "grouped")
CHILD_TIMEOUT_S = 120


def _setup_paths() -> None:
    sys.path.insert(0, REF)
    sys.path.insert(0, os.path.join(HERE, "jax_stub"))


def _time(fn, torch, iters: int):
    """(ms per call, how): CUDA-graph replay when the launches can be captured, else eager."""
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    how = "cuda-graph replay"
    try:
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        g = torch.cuda.CUDAGraph()
        with torch.cuda.stream(side):
            fn()
            side.synchronize()
            with torch.cuda.graph(g, stream=side):
                for _ in range(iters):
                    fn()
        run, n = g.replay, 1
    except Exception as exc:  # noqa: BLE001
        how = f"eager loop (capture failed: {str(exc)[:80]})"
        torch.cuda.synchronize()

        def run():
            for _ in range(iters):
                fn()
        n = 1
    run()
    torch.cuda.synchronize()
    best = float("inf")
    for _ in range(3):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(n):
            run()
        e1.record()
        torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1) / (n * iters))
    return best, how


def family_rows(torch) -> dict:
    from examples.blackwell.layer_norm import build_layer_norm
    from examples.blackwell.rms_norm import build_rms_norm
    from examples.blackwell.swiglu import build_fused_silu_mul
    from examples.hopper.softmax import build_softmax
    B, N = 2048, 8192
    SETS = 6   # rotate over 6 buffer sets (384 MiB per operand) so launches stream from HBM
    xs = [torch.randn(B, N, device="cuda") for _ in range(SETS)]
    us = [torch.randn(B, N, device="cuda") for _ in range(SETS)]
    w = torch.randn(N, device="cuda") * 0.02 + 1.0
    b = torch.randn(N, device="cuda") * 0.02
    out = {}
    F = torch.nn.functional
    cases = {
        "rms_norm": (build_rms_norm(B, N), lambda k, i: k(xs[i], w),
                     lambda: xs[0] * torch.rsqrt((xs[0] * xs[0]).mean(-1, keepdim=True) + 1e-6) * w, 2 * B * N * 4 + N * 4),
        "layer_norm": (build_layer_norm(B, N), lambda k, i: k(xs[i], w, b),
                       lambda: F.layer_norm(xs[0], (N,), w, b, 1e-5), 2 * B * N * 4 + 2 * N * 4),
        "swiglu": (build_fused_silu_mul(B, N), lambda k, i: k(xs[i], us[i]), lambda: F.silu(xs[0]) * us[0], 3 * B * N * 4),
        "softmax": (build_softmax(B, N, arch="sm_100a"), lambda k, i: k(xs[i]), lambda: torch.softmax(xs[0], -1), 2 * B * N * 4),
    }
    for name, (k, call, ref, nbytes) in cases.items():
        try:
            y = call(k, 0)
            torch.cuda.synchronize()
            err = float((y - ref()).abs().max())
            counter = [0]

            outs = [None] * SETS     # rotating output slots, so that writes go to HBM too

            def fn():
                i = counter[0] % SETS
                outs[i] = call(k, i)
                counter[0] += 1

            ms, how = _time(fn, torch, 24)
            out[name] = {"ms": ms, "GB/s": nbytes / (ms * 1e-3) / 1e9, "max_abs_err": err, "timing": how}
        except Exception as exc:  # noqa: BLE001
            out[name] = {"error": str(exc)[:300]}
    return out


def family_gemm(torch) -> dict:
    from examples.blackwell.gemm_highperf_blackwell import build_gemm, build_gemm_2sm
    out = {}
    for S in (2048, 4096, 8192):
        a = (torch.randn(S, S, device="cuda") / S ** 0.5).to(torch.bfloat16)
        bt = (torch.randn(S, S, device="cuda") / S ** 0.5).to(torch.bfloat16)
        ref = None
        if S <= 4096:
            ref = a.float() @ bt.float().t()
        for name, builder in (("1sm", build_gemm), ("2sm", build_gemm_2sm)):
            key = f"gemm_{name}_{S}"
            try:
                k = builder(S, S, S)
                d = k(a, bt)
                torch.cuda.synchronize()
                entry = {}
                if ref is not None:
                    entry["rel_fro"] = float((d - ref).norm() / ref.norm())
                ms, how = _time(lambda: k(a, bt), torch, 10)
                entry.update({"ms": ms, "TFLOP/s": 2.0 * S ** 3 / (ms * 1e-3) / 1e12, "timing": how})
                out[key] = entry
            except Exception as exc:  # noqa: BLE001
                out[key] = {"error": str(exc)[:300]}
        del a, bt, ref
    return out


def family_grouped(torch) -> dict:
    from examples.blackwell.grouped_gemm import build_grouped_gemm
    out = {}
    for G in (8, 4):
        M, N, K = 2048, 256, 2048
        key = f"grouped_G{G}"
        try:
            a3 = (torch.randn(G, M, K, device="cuda") / K ** 0.5).to(torch.bfloat16)
            b3 = (torch.randn(G, K, N, device="cuda") / K ** 0.5).to(torch.bfloat16)
            a2 = a3.reshape(G * M, K)
            bt2 = b3.transpose(1, 2).contiguous().reshape(G * N, K)
            k = build_grouped_gemm(G, M, N, K)
            c = k(a2, bt2)
            torch.cuda.synchronize()
            ref = torch.einsum("gmk,gkn->gmn", a3.float(), b3.float()).reshape(G * M, N)
            ms, how = _time(lambda: k(a2, bt2), torch, 20)
            out[key] = {"ms": ms, "TFLOP/s": 2.0 * G * M * N * K / (ms * 1e-3) / 1e12,
                        "rel_fro": float((c - ref).norm() / ref.norm()), "timing": how}
        except Exception as exc:  # noqa: BLE001
            out[key] = {"error": str(exc)[:300]}
    return out


def run_family(name: str) -> dict:
    _setup_paths()
    import torch
    torch.cuda.set_device(0)
    # The reference JIT-compiles a pybind11 extension with ninja on first use (about a minute);
    # its ctypes launch path is the stock fallback and is what runs here.
    import pyptx.torch_support as ts
    ts._CPP_EXT_CHECKED = True
    return {"rows": family_rows, "gemm": family_gemm, "grouped": family_grouped}[name](torch)


def main() -> None:
    if not os.path.isdir(os.path.join(REF, "pyptx")):
        print(json.dumps({"unavailable": "baseline/_ref is not staged (run baseline/prepare_ref.py where the reference tree exists)"}))
        return
    if len(sys.argv) > 1:
        print(json.dumps(run_family(sys.argv[1])))
        return
    merged: dict = {}
    for fam in FAMILIES:
        try:
            r = subprocess.run([sys.executable, os.path.abspath(__file__), fam], capture_output=True, text=True,
                               timeout=CHILD_TIMEOUT_S)
            line = r.stdout.strip().splitlines()[-1] if r.stdout.strip() else ""
            merged.update(json.loads(line) if line.startswith("{") else {fam: {"error": (r.stderr or "no output")[-300:]}})
        except subprocess.TimeoutExpired:
            merged[fam] = {"error": f"timed out after {CHILD_TIMEOUT_S} s"}
    print(json.dumps(merged))


if __name__ == "__main__":
    main()
