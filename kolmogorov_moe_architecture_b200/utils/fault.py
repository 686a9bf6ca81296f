"""Failure detection and training-health monitors.

Host side only - nothing here makes a GPU fault, trap or hang:

* ``InterruptGuard``       - SIGINT/SIGTERM handler that requests a checkpoint at the next step
  boundary (reference: train.py:211-225,391-392).
* ``StepWatchdog``         - a thread that raises the alarm (callback, default: log + flag) when
  no step completed within a deadline; steps call ``beat()``.
* ``HeartbeatMonitor``     - ranks publish a heartbeat through a ``torch.distributed`` store; a rank
  that stopped beating is reported before the next collective is entered, so the others can
  stop between steps instead of blocking in NCCL.
* ``FaultInjector``        - test helper that makes a chosen rank raise, stall or skip at a chosen
  step (host-side injection).
* ``check_router_collapse``- entropy / max-usage probe of every MoE router on random hidden
  states (reference: train.py:57-159).
* ``gradient_census``      - NaN / Inf / zero-gradient counts per parameter group
  (reference: train_distributed.py:425-510).
* ``NormWatch``            - flags norm weights that never moved from 1.0 (reference: train.py:997-1068).
"""
from __future__ import annotations

import math
import signal
import threading
import time
from typing import Callable, Dict, List, Optional, Tuple

import torch


class InterruptGuard:
    def __init__(self, signals=(signal.SIGINT, signal.SIGTERM)):
        self.requested = False
        self.signum: Optional[int] = None
        self._old = {}
        self.signals = signals

    def _handler(self, signum, frame):
        if self.requested:            # second signal: give up immediately
            raise KeyboardInterrupt
        self.requested, self.signum = True, signum

    def __enter__(self):
        for s in self.signals:
            try:
                self._old[s] = signal.signal(s, self._handler)
            except ValueError:        # not in the main thread
                pass
        return self

    def __exit__(self, *exc):
        for s, h in self._old.items():
            signal.signal(s, h)
        return False


class StepWatchdog:
    def __init__(self, deadline_s: float, on_timeout: Optional[Callable[[float], None]] = None, poll_s: float = 0.25):
        self.deadline_s, self.on_timeout, self.poll_s = deadline_s, on_timeout, poll_s
        self.last = time.monotonic()
        self.tripped = False
        self._stop = threading.Event()
        self._t = threading.Thread(target=self._run, daemon=True)

    def start(self):
        self.last = time.monotonic()
        self._t.start()
        return self

    def beat(self):
        self.last = time.monotonic()

    def _run(self):
        while not self._stop.wait(self.poll_s):
            idle = time.monotonic() - self.last
            if idle > self.deadline_s and not self.tripped:
                self.tripped = True
                if self.on_timeout is not None:
                    self.on_timeout(idle)

    def stop(self):
        self._stop.set()


class HeartbeatMonitor:
    """Each rank writes ``hb/{rank} = step`` into the store after every step; ``dead_ranks(step)``
    lists ranks that are more than ``max_lag`` steps behind or have not written for ``timeout_s``."""

    def __init__(self, store, rank: int, world: int, timeout_s: float = 30.0, max_lag: int = 2):
        self.store, self.rank, self.world, self.timeout_s, self.max_lag = store, rank, world, timeout_s, max_lag
        self._seen: Dict[int, Tuple[int, float]] = {}

    def beat(self, step: int) -> None:
        self.store.set(f"hb/{self.rank}", str(step))

    def mark_leaving(self) -> None:
        self.store.set(f"hb/{self.rank}", "-1")

    def _read(self, r: int) -> Optional[int]:
        try:
            if hasattr(self.store, "check") and not self.store.check([f"hb/{r}"]):
                return None
            return int(self.store.get(f"hb/{r}").decode())
        except Exception:
            return None

    def wait_all(self, step: int, timeout_s: Optional[float] = None, poll_s: float = 0.01) -> List[int]:
        """Host-side agreement before a step's collectives: publish ``step``, then wait until every
        other rank has published a value >= ``step`` or has marked itself as leaving.  Returns the ranks
        that left or did not show up within the timeout; an empty list means it is safe to launch."""
        self.beat(step)
        deadline = time.monotonic() + (self.timeout_s if timeout_s is None else timeout_s)
        pending = [r for r in range(self.world) if r != self.rank]
        gone: List[int] = []
        while pending:
            for r in list(pending):
                v = self._read(r)
                if v == -1:
                    gone.append(r)
                    pending.remove(r)
                elif v is not None and v >= step:
                    pending.remove(r)
            if not pending or time.monotonic() > deadline:
                break
            time.sleep(poll_s)
        return sorted(gone + pending)

    def dead_ranks(self, step: int) -> List[int]:
        now = time.monotonic()
        dead = []
        for r in range(self.world):
            if r == self.rank:
                continue
            v = self._read(r)
            if v == -1:
                dead.append(r)
                continue
            prev = self._seen.get(r)
            if v is not None and (prev is None or v != prev[0]):
                self._seen[r] = (v, now)
                prev = self._seen[r]
            if prev is None:
                self._seen[r] = (-10**9, now)
                continue
            stale = now - prev[1] > self.timeout_s
            lagging = v is not None and step - v > self.max_lag and stale
            if stale and (v is None or lagging or step - prev[0] > self.max_lag):
                dead.append(r)
        return dead


class FaultInjector:
    """``FaultInjector(rank=1, step=3, kind="raise")`` - call ``maybe_fail(rank, step)`` once per step."""

    def __init__(self, rank: int, step: int, kind: str = "raise", stall_s: float = 5.0):
        assert kind in ("raise", "stall", "exit")
        self.rank, self.step, self.kind, self.stall_s = rank, step, kind, stall_s

    def maybe_fail(self, rank: int, step: int) -> None:
        if rank != self.rank or step != self.step:
            return
        if self.kind == "raise":
            raise RuntimeError(f"injected failure on rank {rank} at step {step}")
        if self.kind == "stall":
            time.sleep(self.stall_s)
        if self.kind == "exit":
            raise SystemExit(17)


@torch.no_grad()
def check_router_collapse(model, n_samples: int = 512, entropy_threshold: float = 0.7, generator=None):
    """Returns (layer_stats, collapsed_layers, summary).  Collapsed = normalised usage entropy below
    the threshold or one expert taking more than half of the assignments."""
    base = getattr(model, "_orig_mod", model)
    was_training = base.training
    base.eval()
    stats, collapsed = {}, []
    p0 = next(base.parameters())
    hidden = torch.randn(1, n_samples, base.config.d_model, device=p0.device, dtype=p0.dtype, generator=generator)
    for i, layer in enumerate(base.layers):
        ffn = getattr(layer, "ffn", None)
        router = getattr(ffn, "router", None)
        if router is None or not hasattr(ffn, "n_experts"):
            continue
        out = router(hidden)
        E = ffn.n_experts
        if len(out) == 3:
            counts = torch.bincount(out[1].flatten(), minlength=E).float()
        else:
            counts = torch.ones(E, device=p0.device)
        usage = counts / counts.sum().clamp(min=1)
        ent = float(-(usage * torch.log(usage + 1e-10)).sum()) / (math.log(E) if E > 1 else 1.0)
        mx = float(usage.max())
        bad = ent < entropy_threshold or mx > 0.5
        stats[i] = {"entropy": ent, "max_usage": mx, "max_expert": int(usage.argmax()), "is_collapsed": bad}
        if bad:
            collapsed.append(i)
    if was_training:
        base.train()
    if not stats:
        return {}, [], "No MoE layers found"
    if collapsed:
        return stats, collapsed, f"COLLAPSE DETECTED in layers {collapsed}"
    avg = sum(s["entropy"] for s in stats.values()) / len(stats)
    return stats, collapsed, f"Routing healthy (avg entropy: {avg:.3f})"


@torch.no_grad()
def gradient_census(model) -> Dict[str, Dict[str, float]]:
    """Per top-level group: parameter count, tensors without grad, NaN/Inf grads, all-zero grads, norm."""
    groups: Dict[str, Dict[str, float]] = {}
    for name, p in model.named_parameters():
        key = "router" if "router" in name else ("experts" if "experts" in name else
                                                  ("norm" if "norm" in name else name.split(".")[0]))
        g = groups.setdefault(key, {"tensors": 0, "no_grad": 0, "nan": 0, "inf": 0, "zero": 0, "sq": 0.0})
        g["tensors"] += 1
        if p.grad is None:
            g["no_grad"] += 1
            continue
        gr = p.grad.float()
        g["nan"] += int(torch.isnan(gr).any())
        g["inf"] += int(torch.isinf(gr).any())
        g["zero"] += int((gr == 0).all())
        g["sq"] += float(gr.pow(2).sum())
    for g in groups.values():
        g["norm"] = math.sqrt(g.pop("sq"))
    return groups


_FLOW_GROUPS = ("attention", "embeddings", "expert_weights", "lm_head", "mod_router", "moe_router", "norms", "other")


def _flow_group(name: str) -> str:
    """Parameter categories of the distributed launcher's gradient-flow check
    (reference: train_distributed.py:975-996)."""
    n = name.lower()
    if "mod_router" in n:
        return "mod_router"
    if "lm_head" in n:
        return "lm_head"
    if ".ffn.router" in n or ("moe" in n and "router" in n) or ".router." in n:
        return "moe_router"
    if "grouped_experts" in n or "local_experts" in n or (".ffn." in n and any(f".{w}" in n for w in ("w1", "w2", "w3"))):
        return "expert_weights"
    if "embed" in n:
        return "embeddings"
    if "norm" in n:
        return "norms"
    if any(k in n for k in ("q_proj", "k_proj", "v_proj", "o_proj", "qkv_proj")) or ("seq_layer" in n and "ffn" not in n):
        return "attention"
    return "other"


@torch.no_grad()
def gradient_flow_report(model, group=None) -> Dict[str, Dict[str, float]]:
    """Per category: tensors, tensors that received a gradient, gradient norm; summed over the ranks of
    ``group`` with ONE all-reduce (the reference issues one all-reduce for the table and one for the
    counters, train_distributed.py:1005-1020).  Reads ``p.grad``, so it belongs between the backward pass
    and the optimizer update (``TrainEngine.before_update``)."""
    import torch.distributed as dist
    stats = {g: [0.0, 0.0, 0.0] for g in _FLOW_GROUPS}
    dev = None
    sq_terms = {g: [] for g in _FLOW_GROUPS}
    for name, p in model.named_parameters():
        if not p.requires_grad:
            continue
        dev = dev or p.device
        st = stats[_flow_group(name)]
        st[0] += 1
        if p.grad is not None:
            st[1] += 1
            sq_terms[_flow_group(name)].append(p.grad)
    vec = torch.zeros(len(_FLOW_GROUPS) * 3, dtype=torch.float64, device=dev or "cpu")
    for i, g in enumerate(_FLOW_GROUPS):
        vec[3 * i], vec[3 * i + 1] = stats[g][0], stats[g][1]
        if sq_terms[g]:
            norms = torch._foreach_norm(sq_terms[g], 2.0)
            vec[3 * i + 2] = torch.stack([x.double() for x in norms]).pow(2).sum()
    if dist.is_available() and dist.is_initialized() and dist.get_world_size(group) > 1:
        v32 = vec.float() if vec.device.type == "cuda" else vec
        dist.all_reduce(v32, group=group)
        vec = v32.double()
    out = {}
    host = vec.tolist()                              # the one host read of the report
    for i, g in enumerate(_FLOW_GROUPS):
        if host[3 * i] > 0:
            out[g] = {"tensors": int(host[3 * i]), "with_grad": int(host[3 * i + 1]),
                      "norm": math.sqrt(max(host[3 * i + 2], 0.0))}
    return out


def format_flow_report(rep: Dict[str, Dict[str, float]], world: int = 1) -> str:
    tot = sum(r["tensors"] for r in rep.values())
    got = sum(r["with_grad"] for r in rep.values())
    lines = [f"Gradient flow summary (aggregated across {world} ranks):",
             f"  Total trainable params: {tot}", f"  Params with gradients: {got}",
             f"  Params without gradients: {tot - got}", "By module:"]
    for g, r in rep.items():
        ok = "ok" if r["with_grad"] == r["tensors"] else "MISSING"
        lines.append(f"  {g:20s}: {r['with_grad']:3d}/{r['tensors']:3d} grads, norm={r['norm']:.6f} {ok}")
    lines.append("All parameters received gradients!" if got == tot
                 else f"{tot - got} parameters did not receive gradients (this can make training plateau)")
    return "\n".join(lines)


class NormWatch:
    """Reports normalisation weights that are still exactly at their initial value after training steps."""

    def __init__(self, model):
        self.init = {n: p.detach().clone() for n, p in model.named_parameters() if "norm" in n and p.dim() == 1}

    @torch.no_grad()
    def stuck(self, model, atol: float = 0.0) -> List[str]:
        cur = dict(model.named_parameters())
        return [n for n, v in self.init.items() if n in cur and torch.allclose(cur[n].detach(), v, atol=atol, rtol=0)]
