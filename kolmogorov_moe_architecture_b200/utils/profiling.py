"""Timing and tracing helpers.

* ``PhaseTimer``  - per-phase breakdown (data / forward / backward / optimizer) measured with CUDA
  events on the compute stream, reduced as max over ranks; the host-clock ``TimingStats`` of the
  reference (train_custom.py:597-640) without the device synchronisations inside the step.
* ``nvtx_range``  - context manager adding an NVTX range (no-op when CUDA is absent).
* ``annotate_blocks`` - NVTX ranges around every transformer block's forward and backward (and around
  its sequence mixer and FFN), so a timeline shows which layer a kernel belongs to.
* ``device_timed``- run a callable K times between CUDA events with barrier + synchronize on both
  sides; returns milliseconds per call (max over ranks).
* ``roofline``    - achieved / peak against the measured peaks file.
"""
from __future__ import annotations

import contextlib
import json
import os
import time
from collections import defaultdict
from typing import Callable, Dict, Optional

import torch


@contextlib.contextmanager
def nvtx_range(name: str):
    on = torch.cuda.is_available()
    if on:
        torch.cuda.nvtx.range_push(name)
    try:
        yield
    finally:
        if on:
            torch.cuda.nvtx.range_pop()


class BlockAnnotations:
    """Handle returned by ``annotate_blocks``: ``remove()`` takes the hooks off again; ``events`` counts
    the ranges opened (forward, backward) - also without a GPU, where the ranges themselves are no-ops."""

    def __init__(self):
        self.handles = []
        self.events = {"forward": 0, "backward": 0}

    def remove(self) -> None:
        for h in self.handles:
            h.remove()
        self.handles.clear()


def annotate_blocks(model, parts=("seq_layer", "ffn")) -> BlockAnnotations:
    """Forward ranges ``L{i}`` / ``L{i}.seq_layer`` / ``L{i}.ffn`` and backward ranges ``L{i}.bwd`` on every
    block of ``model.layers``.  The backward range opens when the block's output gradient is ready and
    closes when its input gradient has been produced."""
    ann = BlockAnnotations()
    on = torch.cuda.is_available()

    def push(name, kind):
        ann.events[kind] += 1
        if on:
            torch.cuda.nvtx.range_push(name)

    def pop():
        if on:
            torch.cuda.nvtx.range_pop()

    base = getattr(model, "_orig_mod", model)
    for i, layer in enumerate(base.layers):
        mods = [(f"L{i}", layer)] + [(f"L{i}.{p}", getattr(layer, p)) for p in parts if getattr(layer, p, None) is not None]
        for name, m in mods:
            ann.handles.append(m.register_forward_pre_hook(lambda mod, a, n=name: push(n, "forward")))
            ann.handles.append(m.register_forward_hook(lambda mod, a, o: pop()))
        ann.handles.append(layer.register_full_backward_pre_hook(lambda mod, g, n=f"L{i}.bwd": push(n, "backward")))
        ann.handles.append(layer.register_full_backward_hook(lambda mod, gi, go: pop()))
    return ann


class PhaseTimer:
    def __init__(self, enabled: bool = True, device: Optional[torch.device] = None):
        self.enabled = enabled
        self.cuda = torch.cuda.is_available() and (device is None or torch.device(device).type == "cuda")
        self.pending = []
        self.totals: Dict[str, float] = defaultdict(float)
        self.counts: Dict[str, int] = defaultdict(int)

    @contextlib.contextmanager
    def phase(self, name: str):
        if not self.enabled:
            yield
            return
        if self.cuda:
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            with nvtx_range(name):
                yield
            e1.record()
            self.pending.append((name, e0, e1))
        else:
            t0 = time.perf_counter()
            yield
            self.totals[name] += (time.perf_counter() - t0) * 1e3
            self.counts[name] += 1

    def flush(self):
        """Resolve recorded events (synchronises once; call at logging time, not per step)."""
        if self.pending:
            torch.cuda.synchronize()
            for name, e0, e1 in self.pending:
                self.totals[name] += e0.elapsed_time(e1)
                self.counts[name] += 1
            self.pending.clear()

    def summary(self, reduce_max: bool = False) -> Dict[str, float]:
        self.flush()
        out = {k: self.totals[k] / max(self.counts[k], 1) for k in self.totals}
        if reduce_max:
            import torch.distributed as dist
            if dist.is_available() and dist.is_initialized():
                keys = sorted(out)
                t = torch.tensor([out[k] for k in keys], dtype=torch.float64,
                                 device="cuda" if self.cuda else "cpu")
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                out = dict(zip(keys, t.tolist()))
        return out

    def reset(self):
        self.pending.clear()
        self.totals.clear()
        self.counts.clear()


TimingStats = PhaseTimer


def device_timed(fn: Callable[[], None], iters: int = 10, warmup: int = 3) -> float:
    import torch.distributed as dist
    multi = dist.is_available() and dist.is_initialized()
    for _ in range(warmup):
        fn()
    if multi:
        dist.barrier()
    torch.cuda.synchronize()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(iters):
        fn()
    e1.record()
    if multi:
        dist.barrier()
    torch.cuda.synchronize()
    ms = e0.elapsed_time(e1) / iters
    if multi:
        t = torch.tensor([ms], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    return ms


def measured_peaks(root: Optional[str] = None) -> Dict[str, float]:
    root = root or os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    p = os.path.join(root, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return {"hbm_bytes_s": d["hbm_gbs"] * 1e9, "bf16_flops": d["bf16_tflops"] * 1e12,
                "bf16_flops_sustained": d.get("bf16_tflops_sustained", d["bf16_tflops"]) * 1e12, "kind": "measured"}
    return {"hbm_bytes_s": 6.65e12, "bf16_flops": 1.59e15, "bf16_flops_sustained": 1.4e15, "kind": "fallback"}


def roofline(seconds: float, flops: float = 0.0, hbm_bytes: float = 0.0, nvlink_bytes: float = 0.0,
             nvlink_bw: float = 770e9) -> Dict[str, float]:
    """Fraction of the roofline: target time = slowest of compute at peak, HBM bytes at copy
    bandwidth and NVLink bytes at the measured per-direction peer bandwidth."""
    pk = measured_peaks()
    target = max(flops / pk["bf16_flops"] if flops else 0.0, hbm_bytes / pk["hbm_bytes_s"] if hbm_bytes else 0.0,
                 nvlink_bytes / nvlink_bw if nvlink_bytes else 0.0)
    return {"target_s": target, "achieved_fraction": target / seconds if seconds > 0 else 0.0, "peaks": pk["kind"]}
