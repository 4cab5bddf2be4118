#!/usr/bin/env python
"""Benchmark of the hot path: bf16 GEMM TFLOPS at 8192^3 (headline) plus the row kernels' HBM GB/s.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--variant 1sm|2sm]

A step is one D = A @ B_T.T at M = N = K = 8192 (bf16 in, fp32 accumulate, f32 out) through the
public ``build_gemm`` / ``build_gemm_2sm`` entry point.  With N > 1 (one process per GPU under
``torch.distributed.run``) every rank owns one 8192-row block of A and of D with B_T replicated --
M-sharding, no collective on the data path -- so the job is a (N*8192) x 8192 x 8192 product and
scaling is weak.  One JSON line is printed by rank 0.

``--impl reference`` times the reference's CPU path for the same product (its torch formula
``a.float() @ b.float()``, the expression its GEMM example checks against) on the host cores, on a
bounded row block per step.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

S = 8192                       # headline size
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}
CPU_SAMPLE_ROWS = 8192         # rows of A per CPU step: the whole 8192^3 product (1.1 TFLOP, about a second on 16 cores)


def host_cores() -> int:
    try:
        return max(1, len(os.sched_getaffinity(0)))
    except AttributeError:
        return os.cpu_count() or 1


def load_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            p = json.load(f)
        return {k: float(p[k]) for k in FALLBACK_PEAKS}, "measured"
    except Exception:  # noqa: BLE001 - absent or malformed file -> stated fallback
        return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clock, power and throttle reasons through NVML (read-only queries) from a
    thread while the timed region runs; about one sample per millisecond."""

    REASONS = {0x4: "sw_power_cap", 0x8: "hw_slowdown", 0x20: "sw_thermal_slowdown", 0x40: "hw_thermal_slowdown"}

    def __init__(self, torch, device_index: int) -> None:
        self.samples: list[tuple[float, int, float, int]] = []
        self.stop_flag = threading.Event()
        self.thread = None
        self.error = None
        self.sm_max = None
        try:
            import pynvml
            pynvml.nvmlInit()
            uuid = str(torch.cuda.get_device_properties(device_index).uuid)
            if not uuid.startswith("GPU-"):
                uuid = "GPU-" + uuid
            try:
                self.handle = pynvml.nvmlDeviceGetHandleByUUID(uuid.encode())
            except Exception:  # noqa: BLE001 - older bindings take str
                self.handle = pynvml.nvmlDeviceGetHandleByUUID(uuid)
            self.nvml = pynvml
            self.sm_max = int(pynvml.nvmlDeviceGetMaxClockInfo(self.handle, pynvml.NVML_CLOCK_SM))
        except Exception as exc:  # noqa: BLE001 - clocks are reported as unavailable
            self.nvml = None
            self.error = f"NVML unavailable: {exc}"[:120]

    def _loop(self) -> None:
        n = self.nvml
        while not self.stop_flag.is_set():
            try:
                clk = int(n.nvmlDeviceGetClockInfo(self.handle, n.NVML_CLOCK_SM))
                pw = n.nvmlDeviceGetPowerUsage(self.handle) / 1000.0
                rs = int(n.nvmlDeviceGetCurrentClocksThrottleReasons(self.handle))
                self.samples.append((time.perf_counter(), clk, pw, rs))
            except Exception as exc:  # noqa: BLE001
                self.error = f"NVML query failed: {exc}"[:120]
                return
            time.sleep(0.0005)

    def start(self) -> None:
        if self.nvml is None:
            return
        self.thread = threading.Thread(target=self._loop, daemon=True)
        self.thread.start()

    def stop(self, t_begin: float, t_end: float) -> dict:
        """Summary of the samples taken between the two ``perf_counter`` instants."""
        if self.nvml is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [self.error or "NVML unavailable"]}
        self.stop_flag.set()
        self.thread.join(timeout=2)
        inside = [s for s in self.samples if t_begin <= s[0] <= t_end] or self.samples[-3:]
        if not inside:
            return {"sm_mhz": None, "sm_max_mhz": self.sm_max, "reasons": [self.error or "no samples"]}
        bits = 0
        for s in inside:
            bits |= s[3]
        reasons = sorted(name for bit, name in self.REASONS.items() if bits & bit)
        return {"sm_mhz": statistics.median(s[1] for s in inside), "sm_max_mhz": self.sm_max, "reasons": reasons,
                "samples": len(inside), "power_w_max": max(s[2] for s in inside)}


def time_cuda(fn, steps: int, warmup: int, torch) -> float:
    """Milliseconds per call of ``fn`` over ``steps`` back-to-back calls, CUDA events on the current stream."""
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    start.record()
    for _ in range(steps):
        fn()
    stop.record()
    torch.cuda.synchronize()
    return start.elapsed_time(stop) / steps


def time_graph(fn, iters: int, torch, repeats: int = 3) -> float:
    """Milliseconds per call of ``fn`` with ``iters`` calls captured in one CUDA graph and replayed:
    device time without per-launch host dispatch, which matters for kernels of 20-30 us."""
    for _ in range(3):
        fn()
    torch.cuda.synchronize()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.stream(side):
        fn()
        side.synchronize()
        with torch.cuda.graph(graph, stream=side):
            for _ in range(iters):
                fn()
    graph.replay()
    torch.cuda.synchronize()
    best = float("inf")
    for _ in range(repeats):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        graph.replay()
        e1.record()
        torch.cuda.synchronize()
        best = min(best, e0.elapsed_time(e1) / iters)
    return best


def pyptx_reference_kernels() -> dict:
    """The reference's own sm_100a kernels on this GPU (baseline/run_pyptx.py), when staged."""
    script = os.path.join(ROOT, "baseline", "run_pyptx.py")
    if not os.path.isdir(os.path.join(ROOT, "baseline", "_ref", "pyptx")):
        return {"unavailable": "baseline/_ref not staged"}
    import subprocess
    try:
        r = subprocess.run([sys.executable, script], capture_output=True, text=True, timeout=420)
        line = r.stdout.strip().splitlines()[-1] if r.stdout.strip() else ""
        return json.loads(line) if line.startswith("{") else {"error": (r.stderr or "no output")[-300:]}
    except Exception as exc:  # noqa: BLE001 - context only
        return {"error": str(exc)[:300]}


def cpu_gemm_tflops(torch, a_bf16, bt_bf16, rows: int, repeats: int, warmup: int = 1):
    """The oracle's GEMM formula on ``rows`` rows of A with every host thread torch uses."""
    from oracle import formulas
    a = a_bf16[:rows]
    for _ in range(warmup):
        formulas.gemm_ref(a, bt_bf16)
    times = []
    for _ in range(repeats):
        t0 = time.perf_counter()
        formulas.gemm_ref(a, bt_bf16)
        times.append(time.perf_counter() - t0)
    flops = 2.0 * rows * bt_bf16.shape[0] * bt_bf16.shape[1]
    return flops / min(times) / 1e12, sum(times), times


def run_reference(args) -> None:
    """Reference arm: the reference's CPU path for the headline product, on rank 0 only."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import torch
    from oracle import inputs, formulas
    torch.manual_seed(0)
    # torch.distributed.run exports OMP_NUM_THREADS=1; the CPU arm is meant to use every host core.
    torch.set_num_threads(host_cores())
    threads = torch.get_num_threads()
    a, bt = inputs.gemm_inputs(CPU_SAMPLE_ROWS, S, S)
    for _ in range(args.warmup):
        formulas.gemm_ref(a, bt)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        formulas.gemm_ref(a, bt)
    dt = time.perf_counter() - t0
    flops = 2.0 * CPU_SAMPLE_ROWS * S * S * args.steps
    value = flops / dt / 1e12
    sample = (f"{CPU_SAMPLE_ROWS} of {S} rows of A per step ({CPU_SAMPLE_ROWS / S:.3g} of the 8192^3 product), "
              f"torch CPU a.float() @ b.float(), {threads} threads")
    print(json.dumps({
        "impl": "reference", "metric": "bf16 GEMM TFLOPS @8192^3", "value": value, "unit": "TFLOP/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "gemm_bf16_8192x8192x8192_f32out", "cpu_sample_rows": CPU_SAMPLE_ROWS},
        "cpu_baseline": {"value": value, "unit": "TFLOP/s", "cores": threads, "kind": "port", "sample": sample,
                         "host_cpus": os.cpu_count()},
        "e2e": {"value": value, "unit": "TFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def row_kernel_table(torch, peaks, steps: int, warmup: int, errors: list) -> dict:
    """GB/s of the four row kernels at 2048 x 8192 f32, rotating over buffer sets whose total
    footprint exceeds L2 several times so that every launch streams from HBM."""
    from pyptx_b200.examples.blackwell.layer_norm import build_layer_norm, layer_norm_bytes
    from pyptx_b200.examples.blackwell.rms_norm import build_rms_norm, rms_norm_bytes
    from pyptx_b200.examples.blackwell.softmax import build_softmax, softmax_bytes
    from pyptx_b200.examples.blackwell.swiglu import build_fused_silu_mul, swiglu_bytes
    B, N, SETS = 2048, 8192, 6
    xs = [torch.randn(B, N, device="cuda") for _ in range(SETS)]
    us = [torch.randn(B, N, device="cuda") for _ in range(SETS)]
    w = torch.randn(N, device="cuda") * 0.02 + 1.0
    b = torch.randn(N, device="cuda") * 0.02
    table = {}
    cases = {
        "rms_norm": (build_rms_norm(B, N), lambda k, i: k(xs[i], w), rms_norm_bytes(B, N)),
        "layer_norm": (build_layer_norm(B, N), lambda k, i: k(xs[i], w, b), layer_norm_bytes(B, N)),
        "swiglu": (build_fused_silu_mul(B, N), lambda k, i: k(xs[i], us[i]), swiglu_bytes(B, N)),
        "softmax": (build_softmax(B, N), lambda k, i: k(xs[i]), softmax_bytes(B, N)),
    }
    for name, (k, call, nbytes) in cases.items():
        counter = [0]

        # Outputs are kept in rotating slots as well: an output that is freed at once would be
        # handed the same 64 MiB block every launch and its writes would stay in L2.
        outs = [None] * SETS

        def fn():
            i = counter[0] % SETS
            outs[i] = call(k, i)
            counter[0] += 1

        ms_eager = time_cuda(fn, steps, warmup, torch)
        counter[0] = 0
        ms = time_graph(fn, 24, torch)       # 24 launches = 4 passes over the 6 buffer sets
        gbs = nbytes / (ms * 1e-3) / 1e9
        table[name] = {"ms": ms, "GB/s": gbs, "bytes": nbytes, "frac_of_measured_hbm": gbs / peaks["hbm_gbs"],
                       "frac_of_8TBps": gbs / 8000.0, "timing": "cuda-graph replay, 6 rotating buffer sets",
                       "ms_eager_loop": ms_eager}
    # backward halves (extension): 3*B*N*4 bytes for the norms, 5*M*F*4 for SwiGLU
    try:
        from pyptx_b200.examples.blackwell.backward import (build_fused_silu_mul_bwd, build_layer_norm_bwd,
                                                            build_rms_norm_bwd, norm_bwd_bytes)
        bwd_cases = {
            "rms_norm_bwd": (build_rms_norm_bwd(B, N), lambda k, i: k(xs[i], w, us[i]), norm_bwd_bytes(B, N)),
            "layer_norm_bwd": (build_layer_norm_bwd(B, N), lambda k, i: k(xs[i], w, us[i]), norm_bwd_bytes(B, N)),
            "swiglu_bwd": (build_fused_silu_mul_bwd(B, N), lambda k, i: k(xs[i], us[i], xs[(i + 1) % SETS]), 5 * B * N * 4),
        }
        for name, (k, call, nbytes) in bwd_cases.items():
            counter = [0]
            outs = [None] * SETS

            def fn():
                i = counter[0] % SETS
                outs[i] = call(k, i)
                counter[0] += 1

            ms = time_graph(fn, 24, torch)
            gbs = nbytes / (ms * 1e-3) / 1e9
            table[name] = {"ms": ms, "GB/s": gbs, "bytes": nbytes, "frac_of_measured_hbm": gbs / peaks["hbm_gbs"],
                           "timing": "cuda-graph replay, 6 rotating buffer sets"}
            del outs
    except Exception as exc:  # noqa: BLE001 - reported in "errors"
        errors.append(f"row backward: {exc}"[:300])
    # torch's own GPU kernels for the same formulas, same buffers, same method (what the
    # reference's kernel benchmark prints next to its kernels, bench_blackwell_kernels.py:61-62, 85-86, 108-109)
    F = torch.nn.functional
    torch_refs = {
        "rms_norm": lambda i: xs[i] * torch.rsqrt((xs[i] * xs[i]).mean(-1, keepdim=True) + 1e-6) * w,
        "layer_norm": lambda i: F.layer_norm(xs[i], (N,), w, b, 1e-5),
        "swiglu": lambda i: F.silu(xs[i]) * us[i],
        "softmax": lambda i: torch.softmax(xs[i], -1),
    }
    for name, ref in torch_refs.items():
        if name not in table:
            continue
        counter = [0]
        outs = [None] * SETS

        def fn():
            i = counter[0] % SETS
            outs[i] = ref(i)
            counter[0] += 1

        try:
            ms = time_graph(fn, 24, torch)
            table[name]["torch_gpu_GB/s"] = table[name]["bytes"] / (ms * 1e-3) / 1e9
        except Exception as exc:  # noqa: BLE001 - reported in "errors"
            errors.append(f"torch {name}: {exc}"[:300])
    return table


def rotating_graph_ms(torch, call, n_sets: int, iters: int) -> float:
    """Milliseconds per launch of ``call(i)`` (``i`` = buffer set) under CUDA-graph replay, with
    every launch's result kept in a slot of its own so that neither operands nor outputs are
    served from L2 when the sets together exceed it several times."""
    outs = [None] * n_sets
    counter = [0]

    def fn():
        i = counter[0] % n_sets
        outs[i] = call(i)
        counter[0] += 1

    return time_graph(fn, iters, torch)


def grouped_table(torch, peaks) -> dict:
    """Grouped GEMM at the benchmark configurations, cold: operands and outputs rotate over buffer
    sets that together exceed L2 at least four times, so the time is an HBM time; ``torch.bmm``
    (bf16 out) is timed the same way on the same operands."""
    from oracle import inputs
    from pyptx_b200.examples.blackwell.grouped_gemm import build_grouped_gemm
    table = {}
    l2 = 126e6
    for (G, M, N, K) in ((8, 2048, 256, 2048), (4, 2048, 256, 2048), (8, 512, 128, 512), (8, 1024, 128, 1024)):
        nbytes = G * (M * K * 2 + N * K * 2 + M * N * 4)
        sets = max(4, int(4 * l2 // nbytes) + 1)
        base_a, base_b = inputs.grouped_gemm_inputs(G, M, N, K)
        ga = [base_a.cuda().roll(i, 0) for i in range(sets)]
        gb = [base_b.cuda().roll(i, 0) for i in range(sets)]
        k = build_grouped_gemm(G, M, N, K)
        flops = 2.0 * G * M * N * K
        iters = 4 * sets if sets <= 16 else sets
        ms = rotating_graph_ms(torch, lambda i: k(ga[i], gb[i]), sets, iters)
        ms_warm = time_graph(lambda: k(ga[0], gb[0]), 20, torch)
        a3 = [x.view(G, M, K) for x in ga]
        b3 = [x.view(G, N, K).transpose(1, 2) for x in gb]
        ms_bmm = rotating_graph_ms(torch, lambda i: torch.bmm(a3[i], b3[i]), sets, iters)
        roof_ms = nbytes / (peaks["hbm_gbs"] * 1e9) * 1e3
        table[f"G{G}_M{M}_N{N}_K{K}"] = {
            "tflops": flops / (ms * 1e-3) / 1e12, "ms": ms, "bytes": nbytes, "hbm_roof_ms": roof_ms,
            "frac_of_hbm_roof": roof_ms / ms, "buffer_sets": sets,
            "tflops_one_buffer_set_l2_warm": flops / (ms_warm * 1e-3) / 1e12,
            "torch_bmm_bf16_out_tflops": flops / (ms_bmm * 1e-3) / 1e12,
            "timing": "cuda-graph replay over rotating operand/output sets (> 4x L2 in total)",
        }
        del ga, gb, a3, b3
    return table


def moe_table(torch) -> dict:
    """MoE up-projection + activation: one fused kernel against grouped GEMM followed by SwiGLU."""
    from oracle import inputs
    from pyptx_b200.examples.blackwell.grouped_gemm import build_grouped_gemm, build_grouped_gemm_swiglu
    from pyptx_b200.examples.blackwell.swiglu import build_fused_silu_mul
    from pyptx_b200.types import bf16 as _bf16
    G, M, F, K = 8, 2048, 1024, 2048
    ga, gw = inputs.grouped_gemm_inputs(G, M, 2 * F, K)
    ga, gw = ga.cuda(), gw.cuda()
    fused = build_grouped_gemm_swiglu(G, M, F, K, out_dtype=_bf16)
    two_a, two_b = build_grouped_gemm(G, M, 2 * F, K), build_fused_silu_mul(G * M, F, out_dtype=_bf16)

    def two_kernels():
        c = two_a(ga, gw)
        return two_b(c[:, :F].contiguous(), c[:, F:].contiguous())

    fl = 2.0 * G * M * 2 * F * K
    ms = time_graph(lambda: fused(ga, gw), 10, torch)
    ms2 = time_graph(two_kernels, 10, torch)
    return {"moe_up_swiglu_fused_G8_M2048_F1024_K2048_tflops": fl / (ms * 1e-3) / 1e12,
            "moe_up_swiglu_two_kernels_tflops": fl / (ms2 * 1e-3) / 1e12}


def attention_table(torch) -> dict:
    """Attention forward and backward at B=4, H=16, S=4096 against torch SDPA on the same operands
    (the backward counts five products per tile pair, 2.5x the forward's flops)."""
    import torch.nn.functional as F
    from oracle import inputs
    from pyptx_b200.examples.blackwell.flash_attention import (attention_bwd_flops, attention_flops,
                                                               build_flash_attention, build_flash_attention_bwd)
    out = {}
    for d in (64, 128):
        q, kk, v = (t.view(4, 16, 4096, d).cuda() for t in inputs.attention_inputs(64, 4096, 4096, d))
        for causal in (False, True):
            k = build_flash_attention(4, 16, 4096, 4096, d, causal=causal)
            fl = attention_flops(4, 16, 4096, 4096, d, causal)
            tag = f"attention_d{d}_{'causal' if causal else 'full'}"
            ms = time_cuda(lambda: k(q, kk, v), 20, 5, torch)
            out[tag + "_tflops"] = fl / (ms * 1e-3) / 1e12
            ms = time_cuda(lambda: F.scaled_dot_product_attention(q, kk, v, is_causal=causal), 20, 5, torch)
            out[tag + "_torch_sdpa_tflops"] = fl / (ms * 1e-3) / 1e12
            # backward: (dQ, dK, dV) from (Q, K, V, O, lse, dO)
            fwd = build_flash_attention(4, 16, 4096, 4096, d, causal=causal, return_lse=True)
            bwd = build_flash_attention_bwd(4, 16, 4096, 4096, d, causal=causal)
            o, lse = fwd(q, kk, v)
            d_o = torch.randn_like(o)
            flb = attention_bwd_flops(4, 16, 4096, 4096, d, causal)
            ms = time_cuda(lambda: bwd(q, kk, v, o, lse, d_o), 10, 3, torch)
            out[tag + "_bwd_tflops"] = flb / (ms * 1e-3) / 1e12
            bwd2 = build_flash_attention_bwd(4, 16, 4096, 4096, d, causal=causal, deterministic=True)
            ms = time_cuda(lambda: bwd2(q, kk, v, o, lse, d_o), 10, 3, torch)
            out[tag + "_bwd_two_pass_tflops"] = flb / (ms * 1e-3) / 1e12
            del bwd2
            qg, kg, vg = (t.detach().clone().requires_grad_() for t in (q, kk, v))
            og = F.scaled_dot_product_attention(qg, kg, vg, is_causal=causal)
            ms = time_cuda(lambda: torch.autograd.grad(og, (qg, kg, vg), d_o, retain_graph=True), 10, 3, torch)
            out[tag + "_bwd_torch_sdpa_tflops"] = flb / (ms * 1e-3) / 1e12
            del fwd, bwd, o, lse, d_o, qg, kg, vg, og
        del q, kk, v
    return out


def gpu_host_placement(torch, local_rank: int, pinned) -> dict:
    """Where this rank's GPU and pinned buffer sit relative to the host's NUMA nodes (read-only:
    sysfs attributes of the GPU's PCI function and this process's numa_maps)."""
    info = {"cpu_affinity": len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else None}
    try:
        bdf = torch.cuda.get_device_properties(local_rank).pci_bus_id
        bdf = f"{torch.cuda.get_device_properties(local_rank).pci_domain_id:04x}:{bdf:02x}:" \
              f"{torch.cuda.get_device_properties(local_rank).pci_device_id:02x}.0"
        base = f"/sys/bus/pci/devices/{bdf}"
        with open(base + "/numa_node") as f:
            info["gpu_numa_node"] = int(f.read().strip())
        with open(base + "/local_cpulist") as f:
            info["gpu_local_cpulist"] = f.read().strip()
    except Exception as exc:  # noqa: BLE001 - containers often hide sysfs
        info["gpu_numa_node"] = f"unknown ({type(exc).__name__})"
    try:
        ptr = pinned.data_ptr()
        best = None
        with open("/proc/self/numa_maps") as f:
            for line in f:
                start = int(line.split()[0], 16)
                if start <= ptr and (best is None or start > best[0]):
                    best = (start, line)
        if best:
            info["pinned_pages_by_node"] = {tok.split("=")[0]: int(tok.split("=")[1])
                                            for tok in best[1].split() if tok[0] == "N" and "=" in tok}
    except Exception as exc:  # noqa: BLE001
        info["pinned_pages_by_node"] = f"unknown ({type(exc).__name__})"
    return info


def host_link_table(torch, dist, world: int, local_rank: int, up_pins, d_pin) -> dict:
    """Host <-> device copy rate of every rank, all ranks copying at the same time: upload only,
    download only, and both directions at once, with the end-to-end step's own buffers (A and B_T up,
    D down).  Each direction is timed with CUDA events on its own stream.  This is the ceiling of
    the end-to-end leg; at N > 1 the ranks share the host's PCIe root ports and memory controllers."""
    dev_up = [torch.empty(t.shape, dtype=t.dtype, device="cuda") for t in up_pins]
    dev_d = torch.empty(d_pin.shape, dtype=d_pin.dtype, device="cuda")
    up, down = torch.cuda.Stream(), torch.cuda.Stream()
    up_bytes = sum(t.numel() * t.element_size() for t in up_pins)
    down_bytes = d_pin.numel() * d_pin.element_size()
    reps = 3

    def run(do_up: bool, do_down: bool):
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()
        ev = {n: (torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for n in ("up", "down")}
        if do_up:
            with torch.cuda.stream(up):
                ev["up"][0].record()
                for _ in range(reps):
                    for dst, src in zip(dev_up, up_pins):
                        dst.copy_(src, non_blocking=True)
                ev["up"][1].record()
        if do_down:
            with torch.cuda.stream(down):
                ev["down"][0].record()
                for _ in range(reps):
                    d_pin.copy_(dev_d, non_blocking=True)
                ev["down"][1].record()
        up.synchronize(); down.synchronize()
        h2d = up_bytes * reps / (ev["up"][0].elapsed_time(ev["up"][1]) * 1e-3) / 1e9 if do_up else 0.0
        d2h = down_bytes * reps / (ev["down"][0].elapsed_time(ev["down"][1]) * 1e-3) / 1e9 if do_down else 0.0
        return h2d, d2h

    run(True, True)
    out = {}
    for name, (u, d) in (("h2d_only", (True, False)), ("d2h_only", (False, True)), ("both", (True, True))):
        t = torch.tensor(run(u, d), device="cuda", dtype=torch.float64)
        if world > 1:
            gathered = [torch.zeros_like(t) for _ in range(world)]
            dist.all_gather(gathered, t)
        else:
            gathered = [t]
        ups = [float(g[0]) for g in gathered]
        downs = [float(g[1]) for g in gathered]
        out[name] = {"h2d_GBs_per_rank": [round(v, 1) for v in ups], "d2h_GBs_per_rank": [round(v, 1) for v in downs],
                     "h2d_GBs_total": round(sum(ups), 1), "d2h_GBs_total": round(sum(downs), 1)}
    out["placement_rank0"] = gpu_host_placement(torch, local_rank, up_pins[0])
    out["bytes_per_step"] = {"h2d": up_bytes, "d2h": down_bytes}
    return out


def run_case(args) -> None:
    """``--case NAME``: launch one kernel of the library ``warmup + steps`` times on its benchmark
    configuration and print its device time: a small, single-kernel command to profile."""
    import torch
    from oracle import inputs
    from pyptx_b200 import _native
    from pyptx_b200.examples.blackwell.flash_attention import attention_flops, build_flash_attention
    from pyptx_b200.examples.blackwell.gemm_highperf_blackwell import build_gemm, build_gemm_2sm
    from pyptx_b200.examples.blackwell.grouped_gemm import build_grouped_gemm
    from pyptx_b200.examples.blackwell.layer_norm import build_layer_norm, layer_norm_bytes
    from pyptx_b200.examples.blackwell.rms_norm import build_rms_norm, rms_norm_bytes
    from pyptx_b200.examples.blackwell.softmax import build_softmax, softmax_bytes
    from pyptx_b200.examples.blackwell.swiglu import build_fused_silu_mul, swiglu_bytes

    torch.cuda.set_device(0)
    name, size = args.case, args.size
    B, N = 2048, 8192
    work, unit = 0.0, "GB/s"
    if name in ("gemm_1sm", "gemm_2sm"):
        a, bt = inputs.gemm_inputs(size, size, size)
        k = (build_gemm if name == "gemm_1sm" else build_gemm_2sm)(size, size, size)
        ops = (a.cuda(), bt.cuda()); work, unit = 2.0 * size ** 3, "TFLOP/s"
    elif name == "grouped":
        a, bt = inputs.grouped_gemm_inputs(8, 2048, 256, 2048)
        k = build_grouped_gemm(8, 2048, 256, 2048)
        ops = (a.cuda(), bt.cuda()); work, unit = 2.0 * 8 * 2048 * 256 * 2048, "TFLOP/s"
    elif name.startswith("attention"):
        d = 64 if "64" in name else 128
        causal = "causal" in name
        q, kk, v = inputs.attention_inputs(64, size, size, d)
        ops = tuple(t.view(4, 16, size, d).cuda() for t in (q, kk, v))
        if "bwd" in name:
            from pyptx_b200.examples.blackwell.flash_attention import attention_bwd_flops, build_flash_attention_bwd
            o, lse = build_flash_attention(4, 16, size, size, d, causal=causal, return_lse=True)(*ops)
            k = build_flash_attention_bwd(4, 16, size, size, d, causal=causal)
            ops = ops + (o, lse, torch.randn_like(o))
            work, unit = attention_bwd_flops(4, 16, size, size, d, causal), "TFLOP/s"
        else:
            k = build_flash_attention(4, 16, size, size, d, causal=causal)
            work, unit = attention_flops(4, 16, size, size, d, causal), "TFLOP/s"
    elif name in ("rms_norm_bwd", "layer_norm_bwd"):
        from pyptx_b200.examples.blackwell.backward import build_layer_norm_bwd, build_rms_norm_bwd, norm_bwd_bytes
        x, w = inputs.rms_norm_inputs(B, N)
        k = (build_rms_norm_bwd if name == "rms_norm_bwd" else build_layer_norm_bwd)(B, N)
        ops, work = (x.cuda(), w.cuda(), torch.randn(B, N, device="cuda")), norm_bwd_bytes(B, N)
    elif name == "rms_norm":
        k, ops, work = build_rms_norm(B, N), tuple(t.cuda() for t in inputs.rms_norm_inputs(B, N)), rms_norm_bytes(B, N)
    elif name == "layer_norm":
        k, ops, work = build_layer_norm(B, N), tuple(t.cuda() for t in inputs.layer_norm_inputs(B, N)), layer_norm_bytes(B, N)
    elif name == "swiglu":
        k, ops, work = build_fused_silu_mul(B, N), tuple(t.cuda() for t in inputs.swiglu_inputs(B, N)), swiglu_bytes(B, N)
    elif name == "softmax":
        k, ops, work = build_softmax(B, N), tuple(t.cuda() for t in inputs.softmax_inputs(B, N)), softmax_bytes(B, N)
    else:
        raise SystemExit(f"unknown --case {name}")
    flush = torch.empty(1 << 30, dtype=torch.uint8, device="cuda")   # 8x L2; also long enough to hide the host-side launch

    def fn():
        flush.zero_()
        k(*ops)

    for _ in range(args.warmup):
        fn()
    torch.cuda.synchronize()
    times = []
    for _ in range(args.steps):
        flush.zero_()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record(); k(*ops); e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    _native.device_status()
    ms = statistics.median(times)
    rate = work / (ms * 1e-3) / (1e12 if unit == "TFLOP/s" else 1e9)
    print(json.dumps({"case": name, "size": size, "ms": ms, "rate": rate, "unit": unit, "steps": args.steps,
                      "l2": "1 GiB buffer written between launches"}))


def gather_table(torch, dist, world: int, peak_tflops: float, iters: int = 10) -> dict:
    """Context for N > 1: one 8192^3 product split by rows of A over the ranks, with the full D
    wanted on every rank.  Three ways: the local GEMM alone (no gather), GEMM then NCCL
    all-gather, and the GEMM whose epilogue pushes its tiles into every rank's buffer.
    Times are CUDA events, max over ranks; TFLOP/s counts the whole product."""
    from pyptx_b200.examples.blackwell.gemm_highperf_blackwell import build_gemm_2sm
    from pyptx_b200.peer import PushGatherGemm
    from pyptx_b200.types import bf16, f32

    def timed(fn):
        for _ in range(3):
            fn()
        torch.cuda.synchronize()
        dist.barrier()
        torch.cuda.synchronize()
        s, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        s.record()
        for _ in range(iters):
            fn()
        e.record()
        torch.cuda.synchronize()
        t = torch.tensor([s.elapsed_time(e) / iters], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    m_local = S // world
    table = {"problem": f"M={S} split {world} ways (M_local={m_local}), N=K={S}", "nvlink_peer_copy_GBs_measured": 770}
    a = torch.randn(m_local, S, device="cuda").to(torch.bfloat16)
    bt = torch.randn(S, S, device="cuda").to(torch.bfloat16)
    flops = 2.0 * S * S * S
    for odt, tag, spec in ((torch.float32, "f32", f32), (torch.bfloat16, "bf16", bf16)):
        k = build_gemm_2sm(m_local, S, S, out_dtype=spec)
        full = torch.empty(S, S, dtype=odt, device="cuda")
        push = PushGatherGemm(m_local, S, S, out_dtype=odt)

        def with_nccl():
            dist.all_gather_into_tensor(full, k(a, bt))

        t_local, t_nccl, t_push = timed(lambda: k(a, bt)), timed(with_nccl), timed(lambda: push(a, bt))
        sent = (world - 1) * m_local * S * (4 if odt == torch.float32 else 2)
        table[tag] = {
            "local_gemm_ms": t_local, "gemm_then_nccl_all_gather_ms": t_nccl, "push_epilogue_ms": t_push,
            "gemm_then_nccl_tflops": flops / (t_nccl * 1e-3) / 1e12, "push_epilogue_tflops": flops / (t_push * 1e-3) / 1e12,
            "bytes_sent_per_rank": sent,
            # the slower of the tensor-bound time (per-rank FLOPs / measured cuBLAS bf16 peak) and
            # the link-bound time (bytes leaving this GPU / measured peer-copy bandwidth)
            "roofline_ms": max(flops / world / (peak_tflops * 1e12) * 1e3, sent / 770e9 * 1e3),
        }
        table[tag]["frac_of_roofline"] = table[tag]["roofline_ms"] / t_push
        with_nccl()
        same = torch.equal(push(a, bt), full)
        torch.cuda.synchronize()
        table[tag]["bit_identical_to_nccl_path"] = bool(same)
        del push, full, k
    return table


def sharded_table(torch, dist, world: int, rank: int) -> dict:
    """Context for N > 1: the other benchmark configurations split over the ranks the way
    ``pyptx_b200.dist`` partitions them (rows, experts, batch x head), no collective.  Each rank
    times its share under CUDA-graph replay (inputs rotate over at least 512 MiB and every launch
    of the graph writes its own output buffer, so neither side is served by L2); the figure is
    whole-problem work over the slowest rank."""
    from pyptx_b200 import dist as pdist
    from pyptx_b200.examples.blackwell.flash_attention import attention_flops, build_flash_attention
    from pyptx_b200.examples.blackwell.grouped_gemm import build_grouped_gemm
    from pyptx_b200.examples.blackwell.rms_norm import build_rms_norm
    from pyptx_b200.examples.blackwell.swiglu import build_fused_silu_mul

    def graph_ms(call, iters: int) -> float:
        for i in range(3):
            call(i)
        torch.cuda.synchronize()
        side = torch.cuda.Stream()
        side.wait_stream(torch.cuda.current_stream())
        graph = torch.cuda.CUDAGraph()
        keep = []
        with torch.cuda.stream(side):
            call(0)
            side.synchronize()
            with torch.cuda.graph(graph, stream=side):
                for i in range(iters):
                    keep.append(call(i))
        graph.replay()
        torch.cuda.synchronize()
        best = float("inf")
        for _ in range(3):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            graph.replay()
            e1.record()
            torch.cuda.synchronize()
            best = min(best, e0.elapsed_time(e1) / iters)
        del graph, keep
        return best

    def slowest(ms: float) -> float:
        t = torch.tensor([ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    table = {}
    B, N = 2048, 8192
    sh = pdist.shard_rows(build_rms_norm, B, N, world=world, rank=rank)
    ms = 0.0
    if sh.kernel is not None:
        sets = max(4, (512 << 20) // (sh.local * N * 4))
        xs = [torch.randn(sh.local, N, device="cuda") for _ in range(sets)]
        w = torch.randn(N, device="cuda")
        ms = graph_ms(lambda i: sh.kernel(xs[i % sets], w), 32)
        del xs
    ms = slowest(ms)
    table["rms_norm_2048x8192_rows_split"] = {"ms": ms, "GB/s": (2 * B * N * 4 + N * 4) / (ms * 1e-3) / 1e9}
    sh = pdist.shard_rows(build_fused_silu_mul, B, N, world=world, rank=rank)
    ms = 0.0
    if sh.kernel is not None:
        sets = max(4, (512 << 20) // (sh.local * N * 4))
        gs = [torch.randn(sh.local, N, device="cuda") for _ in range(sets)]
        ms = graph_ms(lambda i: sh.kernel(gs[i % sets], gs[(i + 1) % sets]), 32)
        del gs
    ms = slowest(ms)
    table["swiglu_2048x8192_rows_split"] = {"ms": ms, "GB/s": 3 * B * N * 4 / (ms * 1e-3) / 1e9}
    G, M, Ng, K = 8, 2048, 256, 2048
    sh = pdist.shard_grouped_gemm(build_grouped_gemm, G, M, Ng, K, world=world, rank=rank)
    ms = 0.0
    if sh.kernel is not None:
        g_local = sh.local // M
        sets = max(2, (512 << 20) // (g_local * M * K * 2))
        a = [(torch.randn(g_local * M, K, device="cuda") / K ** 0.5).to(torch.bfloat16) for _ in range(sets)]
        bw = (torch.randn(g_local * Ng, K, device="cuda") / K ** 0.5).to(torch.bfloat16)
        ms = graph_ms(lambda i: sh.kernel(a[i % sets], bw), 32)
        del a
    ms = slowest(ms)
    table["grouped_G8_experts_split"] = {"ms": ms, "TFLOP/s": 2.0 * G * M * Ng * K / (ms * 1e-3) / 1e12}
    Bq, H, Sq, d = 4, 16, 4096, 128
    sh = pdist.shard_attention(build_flash_attention, Bq, H, Sq, Sq, d, world=world, rank=rank)
    ms = 0.0
    if sh.kernel is not None:
        q, k, v = (torch.randn(1, sh.local, Sq, d, device="cuda").to(torch.bfloat16) for _ in range(3))
        ms = graph_ms(lambda i: sh.kernel(q, k, v), 10)
    ms = slowest(ms)
    table["attention_d128_S4096_batch_head_split"] = {"ms": ms, "TFLOP/s": attention_flops(Bq, H, Sq, Sq, d) / (ms * 1e-3) / 1e12}
    return table


def run_ours(args) -> None:
    import torch
    import torch.distributed as dist

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py: no CUDA device; the kernels have no CPU path")
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    from oracle import inputs
    from pyptx_b200 import _native
    from pyptx_b200.examples.blackwell.gemm_highperf_blackwell import build_gemm, build_gemm_2sm

    peaks, peak_kind = load_peaks()
    builders = {"1sm": build_gemm, "2sm": build_gemm_2sm}
    kernel = builders[args.variant](S, S, S)

    # Each rank's M-block of A; B_T replicated.  Seeded on the CPU so the oracle sees the same bits.
    a_host, bt_host = inputs.gemm_inputs(S, S, S)
    if rank:
        a_host = a_host.roll(rank * 17, 0)
    a_pin, bt_pin = a_host.pin_memory(), bt_host.pin_memory()
    a, bt = a_pin.cuda(non_blocking=True), bt_pin.cuda(non_blocking=True)
    torch.cuda.synchronize()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- device-resident timing -------------------------------------------------------------
    out_holder = [None]

    def step():
        out_holder[0] = kernel(a, bt)

    for _ in range(max(args.warmup, 3)):
        step()
    barrier()
    sampler = ClockSampler(torch, local_rank) if rank == 0 else None
    if sampler:
        sampler.start()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_begin = time.perf_counter()
    start.record()
    for _ in range(args.steps):
        step()
    stop.record()
    barrier()
    t_end = time.perf_counter()
    ms_total = start.elapsed_time(stop)
    clocks = sampler.stop(t_begin, t_end) if sampler else None
    _native.device_status()
    if world > 1:
        t = torch.tensor([ms_total], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_total = float(t.item())
    ms_per_step = ms_total / args.steps
    flops_per_rank = 2.0 * S * S * S
    value = flops_per_rank * world / (ms_per_step * 1e-3) / 1e12
    kernel_tflops = flops_per_rank / (ms_per_step * 1e-3) / 1e12

    # sanity of the timed output (sampled rows against the oracle happens in the tests; here: finite + nonzero)
    d = out_holder[0]
    checksum = float(d[::1024, ::1024].double().abs().sum().item())
    if not (checksum > 0.0 and checksum == checksum):
        raise SystemExit("bench.py: timed GEMM produced an empty or non-finite result")

    # ---- end to end: pinned host -> device, kernel, device -> pinned host -----------------------
    # Through the library's host-operand call (HostPipeline): every step uploads A and B_T from
    # pinned memory, multiplies, and downloads D into pinned memory; the upload of step i+1 runs
    # while D of step i is on its way back (PCIe is full duplex).  --e2e-depth 1 gives the serial
    # order.  The timed region runs from before the first upload to after the last download.
    from pyptx_b200.host_pipeline import HostPipeline

    depth = max(1, args.e2e_depth)
    pipe = HostPipeline(kernel, depth=depth)
    d_pins = [torch.empty(S, S, dtype=torch.float32).pin_memory() for _ in range(depth)]
    d_pin = d_pins[0]
    e2e_steps = args.steps

    def e2e_run(n):
        for i in range(n):
            pipe.submit(a_pin, bt_pin, out=d_pins[i % depth])
        pipe.join()

    e2e_run(depth + 1)
    barrier()
    start.record()
    e2e_run(e2e_steps)
    stop.record()
    barrier()
    e2e_ms = start.elapsed_time(stop) / e2e_steps
    e2e_check = float(d_pins[(e2e_steps - 1) % depth][::1024, ::1024].double().abs().sum().item())
    if abs(e2e_check - checksum) > 1e-6 * max(checksum, 1.0):
        raise SystemExit("bench.py: the end-to-end result differs from the device-resident one")
    if world > 1:
        t = torch.tensor([e2e_ms], device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e_ms = float(t.item())
    e2e_value = flops_per_rank * world / (e2e_ms * 1e-3) / 1e12
    h2d = a_pin.numel() * 2 + bt_pin.numel() * 2
    d2h = d_pin.numel() * 4
    # what the host link gives when nothing but copies runs (every rank at once)
    host_link = host_link_table(torch, dist, world, local_rank, [a_pin, bt_pin], d_pin)
    # the e2e step moves h2d + d2h bytes per rank; with both directions busy it cannot beat this
    both = host_link["both"]
    link_floor_ms = max(h2d / (min(both["h2d_GBs_per_rank"]) * 1e9), d2h / (min(both["d2h_GBs_per_rank"]) * 1e9)) * 1e3

    gather = None
    gather_error = None
    if world > 1 and not args.no_extras:
        # every rank takes part; a failure on any rank is reported, not fatal to the headline
        try:
            gather = gather_table(torch, dist, world, peaks["bf16_tflops"])
            gather["other_kernels_split_over_ranks"] = sharded_table(torch, dist, world, rank)
            _native.device_status()
        except Exception as exc:  # noqa: BLE001 - reported in "errors"
            gather, gather_error = None, f"gather: {exc}"[:300]

    extras, cpu_baseline = None, None
    errors: list[str] = []          # a context measurement that failed is named here, at the top level
    if gather_error:
        errors.append(gather_error)
    if rank == 0 and (world > 1 or args.no_extras):
        torch.set_num_threads(host_cores())
        tflops, spent, _ = cpu_gemm_tflops(torch, a_host, bt_host, CPU_SAMPLE_ROWS, repeats=1)
        cpu_baseline = {"value": tflops, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
                        "host_cpus": os.cpu_count(), "sample": f"{CPU_SAMPLE_ROWS} of {S} rows of A, one pass"}
    elif rank == 0:
        # ---- context numbers: other variant, cuBLAS, smaller sizes, grouped, row kernels ----------------
        extras = {}
        other = "2sm" if args.variant == "1sm" else "1sm"
        shapes = [(2048, 2048, 2048), (4096, 4096, 4096), (4096, 8192, 8192), (8192, 4096, 8192), (8192, 8192, 8192)]

        def shape_tag(m, n, k):
            return str(m) if m == n == k else f"{m}x{n}x{k}"

        # Shape by shape, the three implementations back to back with a short pause before each, so
        # that every figure of a row is taken in the same thermal / power state of the GPU.
        for (m, n, k_) in shapes:
            x, y = a[:m, :k_].contiguous(), bt[:n, :k_].contiguous()
            yt = y.t().contiguous()
            for name in (args.variant, other):
                k = builders[name](m, n, k_)
                time.sleep(0.3)
                ms = time_cuda(lambda: k(x, y), 20, 5, torch)
                extras[f"gemm_{name}_{shape_tag(m, n, k_)}_tflops"] = 2.0 * m * n * k_ / (ms * 1e-3) / 1e12
            time.sleep(0.3)
            ms = time_cuda(lambda: torch.matmul(x, yt), 20, 5, torch)
            extras[f"cublas_{shape_tag(m, n, k_)}_tflops"] = 2.0 * m * n * k_ / (ms * 1e-3) / 1e12
            del x, y, yt
        try:
            extras["grouped"] = grouped_table(torch, peaks)
        except Exception as exc:  # noqa: BLE001 - reported in "errors"
            errors.append(f"grouped: {exc}"[:300])
        try:
            extras.update(moe_table(torch))
        except Exception as exc:  # noqa: BLE001
            errors.append(f"moe_up_swiglu: {exc}"[:300])
        try:
            extras.update(attention_table(torch))
        except Exception as exc:  # noqa: BLE001
            errors.append(f"attention: {exc}"[:300])
        extras["row_kernels_2048x8192_f32"] = row_kernel_table(torch, peaks, 200, 20, errors)
        _native.device_status()
        # ---- CPU baseline: the oracle formula on a bounded row block -----------------------------
        torch.set_num_threads(host_cores())
        tflops, spent, _ = cpu_gemm_tflops(torch, a_host, bt_host, CPU_SAMPLE_ROWS, repeats=3)
        cpu_baseline = {
            "value": tflops, "unit": "TFLOP/s", "cores": torch.get_num_threads(), "kind": "port",
            "host_cpus": os.cpu_count(),
            "sample": (f"{CPU_SAMPLE_ROWS} of {S} rows of A ({CPU_SAMPLE_ROWS / S:.3g} of the product), best of 3, "
                       f"torch CPU a.float() @ b.float(); {spent:.1f} s of CPU work"),
        }

    if rank == 0:
        peak = peaks["bf16_tflops"]
        line = {
            "metric": "bf16 GEMM TFLOPS @8192^3", "value": value, "unit": "TFLOP/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_per_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": value / world / 1240.0,
            "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "gemm_bf16_8192x8192x8192_f32out", "variant": args.variant,
                       "per_gpu": "M=N=K=8192, A,B~N(0,1)/sqrt(K) seeded, B_T replicated, M-block per rank",
                       "l2": "operands (256 MiB) + output (256 MiB) exceed the 126 MB L2",
                       "vs_baseline_ref": "reference README.md:54: its 1-SM kernel 1240 TFLOPS at 8192^3 on B200 (per GPU)"},
            "clocks": dict(clocks or {}, note="NVML samples taken during the timed region (NVML reports the requested SM clock)"),
            "e2e": {"value": e2e_value, "unit": "TFLOP/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e_ms, "steps": e2e_steps, "calls_in_flight": depth,
                    "host_link": host_link, "copy_bound_ms_per_step": link_floor_ms,
                    "frac_of_copy_bound": link_floor_ms / e2e_ms,
                    "api": "pyptx_b200.host_pipeline.HostPipeline(build_gemm_2sm(...)).submit(pinned A, pinned B_T, out=pinned D)"},
            "gpu_launches": args.steps,
            "roofline": {"bound": "tensor", "achieved": kernel_tflops, "peak": peak, "unit": "TFLOP/s",
                         "frac": kernel_tflops / peak,
                         "traffic": 1060119808 if args.variant == "2sm" else 1121270784,
                         "traffic_source": ("dram__bytes_read.sum + dram__bytes_write.sum of one launch of this kernel at this "
                                            "size from a separate ncu capture; a constant, not measured by this run"),
                         "algorithmic_bytes": 2 * S * S * 2 + S * S * 4,
                         "peak_kind": f"{peak_kind} burst cuBLAS bf16",
                         "frac_of_nominal_2250": kernel_tflops / 2250.0},
            "cpu_baseline": cpu_baseline,
            "errors": errors,
        }
        if gather is not None:
            line["gather"] = gather
            # the same 8192^3 product split by rows over the ranks (strong scaling of the headline
            # kernel): slowest rank's local GEMM against this run's one-GPU step time
            t_local = gather.get("f32", {}).get("local_gemm_ms")
            if t_local:
                line["strong"] = {
                    "problem": f"one 8192^3 product, M split {world} ways, B_T replicated, no gather",
                    "local_gemm_ms_max_over_ranks": t_local, "one_gpu_ms": ms_per_step,
                    "tflops_total": flops_per_rank / (t_local * 1e-3) / 1e12,
                    "efficiency": ms_per_step / (world * t_local),
                    "tiles": (f"M_local={S // world}: {(S // world) // 256 * (S // 256)} tiles of 256x256 "
                              f"(or half as many of 512x256) on 74 CTA pairs"),
                }
        if extras is not None:
            line["kernels"] = extras
            if not args.no_pyptx:
                # Last, after every number of this library is in hand: the reference's own sm_100a
                # kernels in child processes (their device waits are unbounded, hence the time limits).
                del a, bt
                torch.cuda.empty_cache()
                extras["pyptx_reference_kernels"] = pyptx_reference_kernels()
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


def main() -> None:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", choices=["ours", "reference"], default="ours")
    ap.add_argument("--variant", choices=["1sm", "2sm"], default="2sm")
    ap.add_argument("--no-pyptx", action="store_true",
                    help="do not run the reference's own sm_100a kernels (baseline/_ref) for the context table")
    ap.add_argument("--e2e-depth", type=int, default=2,
                    help="calls in flight in the end-to-end leg (1 = upload, multiply, download strictly in turn)")
    ap.add_argument("--no-extras", action="store_true", help="skip the context table (other kernels, cuBLAS)")
    ap.add_argument("--case", default=None,
                    help="run ONE kernel only: gemm_1sm gemm_2sm grouped attention_d64 attention_d128[_causal][_bwd] "
                         "rms_norm layer_norm swiglu softmax rms_norm_bwd layer_norm_bwd")
    ap.add_argument("--size", type=int, default=8192, help="M=N=K (gemm cases) or sequence length (attention cases)")
    args = ap.parse_args()
    if args.case:
        run_case(args)
    elif args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
