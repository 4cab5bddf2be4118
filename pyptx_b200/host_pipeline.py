"""Host-resident operands: overlap the PCIe copies of neighbouring calls with the kernel.

A kernel of this library runs in well under a millisecond at the benchmark sizes, while moving
its operands from pinned host memory and its result back takes several: a caller whose data
lives on the host is bound by the copies.  PCIe is full duplex, so the upload of call ``i+1``
can run while the result of call ``i`` is downloaded.  :class:`HostPipeline` does that with
three streams (upload, compute, download) and ``depth`` sets of device buffers::

    pipe = HostPipeline(build_gemm_2sm(M, N, K), depth=2)
    tickets = [pipe.submit(a_pinned, bt_pinned, out=d_pinned[i % 2]) for i in range(steps)]
    pipe.wait()                      # or pipe.wait(ticket) for one call

Every call still uploads all of its inputs and downloads all of its outputs; only the order
in which the copy engines and the SMs work on neighbouring calls changes.  The reference
launches on the caller's stream with device tensors only (pyptx/torch_support.py:171-271);
this helper is an addition above that call and uses nothing but the kernel's ``__call__``.
"""
from __future__ import annotations

from typing import Any, Sequence


class HostPipeline:
    """Runs ``kernel`` on pinned host tensors, ``depth`` calls in flight."""

    def __init__(self, kernel: Any, depth: int = 2, device: Any = None) -> None:
        import torch

        if depth < 1:
            raise ValueError(f"depth must be at least 1, got {depth}")
        if not torch.cuda.is_available():
            raise RuntimeError("pyptx_b200: HostPipeline needs a CUDA device (there is no CPU path)")
        self.kernel = kernel
        self.depth = int(depth)
        self.device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
        self._up = torch.cuda.Stream(self.device)
        self._run = torch.cuda.Stream(self.device)
        self._down = torch.cuda.Stream(self.device)
        self._slots: list[dict] = [{} for _ in range(self.depth)]
        self._count = 0

    def submit(self, *host_inputs: Any, out: Any | Sequence[Any]) -> int:
        """Enqueue one call: upload ``host_inputs`` (pinned CPU tensors), run the kernel, download
        its output(s) into ``out`` (a pinned CPU tensor, or one per output).  Returns a ticket for
        :meth:`wait`.  ``out`` and the inputs must stay untouched until the ticket is waited on."""
        import torch

        outs = [out] if isinstance(out, torch.Tensor) else list(out)
        for i, t in enumerate(list(host_inputs) + outs):
            if not isinstance(t, torch.Tensor) or t.device.type != "cpu" or not t.is_pinned():
                raise ValueError(f"HostPipeline.submit: tensor {i} must be a pinned CPU tensor")
        slot = self._slots[self._count % self.depth]
        # Anything the caller enqueued on its current stream (e.g. a previous consumer) comes first.
        entry = torch.cuda.Event()
        entry.record(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(self._up):
            self._up.wait_event(entry)
            if "ran" in slot:
                self._up.wait_event(slot["ran"])          # the kernel that last read these buffers
            bufs = slot.get("inputs")
            if bufs is None or [(b.shape, b.dtype) for b in bufs] != [(t.shape, t.dtype) for t in host_inputs]:
                bufs = slot["inputs"] = [torch.empty(t.shape, dtype=t.dtype, device=self.device) for t in host_inputs]
            for b, t in zip(bufs, host_inputs):
                b.copy_(t, non_blocking=True)
            uploaded = torch.cuda.Event()
            uploaded.record(self._up)
        with torch.cuda.stream(self._run):
            self._run.wait_event(uploaded)
            result = self.kernel(*bufs)
            results = [result] if isinstance(result, torch.Tensor) else list(result)
            ran = slot["ran"] = torch.cuda.Event()
            ran.record(self._run)
        if len(results) != len(outs):
            raise ValueError(f"HostPipeline.submit: kernel returns {len(results)} outputs, got {len(outs)} host buffers")
        with torch.cuda.stream(self._down):
            self._down.wait_event(ran)
            for r, o in zip(results, outs):
                r.record_stream(self._down)               # allocated on the compute stream, read here
                o.copy_(r, non_blocking=True)
            done = slot["done"] = torch.cuda.Event()
            done.record(self._down)
        self._count += 1
        slot["ticket"] = self._count
        return self._count

    def wait(self, ticket: int | None = None) -> None:
        """Block the host until call ``ticket`` (default: every submitted call) has landed in its
        host buffer."""
        if ticket is not None:
            if not 1 <= ticket <= self._count:
                raise ValueError(f"unknown ticket {ticket}")
            # The slot's latest download is this call's or a later one on the same stream.
            self._slots[(ticket - 1) % self.depth]["done"].synchronize()
            return
        for slot in self._slots:
            if "done" in slot:
                slot["done"].synchronize()

    def join(self, stream: Any = None) -> None:
        """Make ``stream`` (default: the current one) wait for every submitted call, without
        blocking the host."""
        import torch

        stream = torch.cuda.current_stream(self.device) if stream is None else stream
        for slot in self._slots:
            if "done" in slot:
                stream.wait_event(slot["done"])
