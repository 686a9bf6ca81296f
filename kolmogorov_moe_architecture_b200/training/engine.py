"""``TrainEngine``: one training step (forward, backward, clip, optimizer) as a single call.

This is the public step API used by every entrypoint and by the benchmark:

    engine = TrainEngine(model, optimizer, grad_clip=1.0, dp=DataParallelPlan(...))
    stats = engine.step(input_ids, labels)          # host or device tensors

``step`` accepts pinned host tensors (copied with ``non_blocking=True`` on the compute
stream), runs ``grad_accum`` micro-batches, reduces gradients across the data-parallel
group if one is attached, clips by global norm on the device and applies the optimizer.
Nothing in the step reads a value back to the host; ``stats`` holds device tensors and
``stats.loss_value()`` is the one explicit read.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Any, Dict, Optional

import torch


@dataclass
class StepStats:
    loss: torch.Tensor
    lm_loss: torch.Tensor
    aux_loss: Any
    grad_norm: Optional[torch.Tensor]
    tokens: int
    per_head: Optional[Dict[str, torch.Tensor]] = None

    def loss_value(self) -> float:
        return float(self.loss.item())


def clip_grad_norm_device(params, max_norm: float, extra_sq: Optional[torch.Tensor] = None,
                          group=None) -> torch.Tensor:
    """Global-norm clipping without a host round trip: the scale factor stays on the device.
    ``group``: sum the squared norm over a process group first (sharded gradients)."""
    grads = [p.grad for p in params if p.grad is not None]
    if not grads:
        return torch.zeros((), device="cpu")
    norms = torch._foreach_norm(grads, 2.0)
    sq = torch.stack([n.float() for n in norms]).pow(2).sum()
    if extra_sq is not None:
        sq = sq + extra_sq
    if group is not None:
        import torch.distributed as dist
        dist.all_reduce(sq, group=group)
    total = sq.sqrt()
    if max_norm is not None and max_norm > 0:
        coef = (max_norm / (total + 1e-6)).clamp(max=1.0)
        torch._foreach_mul_(grads, coef.to(grads[0].dtype))
    return total


class TrainEngine:
    def __init__(self, model, optimizer, lr_scheduler=None, grad_clip: Optional[float] = 1.0,
                 grad_accum: int = 1, autocast_dtype: Optional[torch.dtype] = None, dp=None,
                 device: Optional[torch.device] = None):
        self.model, self.optimizer, self.lr_scheduler = model, optimizer, lr_scheduler
        self.grad_clip, self.grad_accum, self.autocast_dtype, self.dp = grad_clip, grad_accum, autocast_dtype, dp
        self.device = device or next(model.parameters()).device
        self.global_step = 0
        self.tokens_seen = 0
        # optional instruments, all off by default:
        self.timer = None            # a utils.profiling.PhaseTimer: forward / backward / optimizer phases
        self.before_update = []      # callables(model) run after the last backward, before clipping and the update
        self.token_weights = None    # (S,) weights: the loss becomes the position-weighted next-token loss

    def _to_device(self, t: torch.Tensor) -> torch.Tensor:
        if t.device == self.device:
            return t
        return t.to(self.device, non_blocking=True)

    def _check_ids(self, input_ids: torch.Tensor) -> None:
        """Token ids that are still on the host are range-checked there (a few microseconds): an id outside
        the vocabulary would otherwise surface as a device-side assertion in the embedding lookup, which
        costs the process its CUDA context."""
        if input_ids.device.type != "cpu" or input_ids.numel() == 0:
            return
        cfg = getattr(getattr(self.model, "_orig_mod", self.model), "config", None)
        vocab = getattr(cfg, "vocab_size", None)
        if vocab is None:
            return
        lo, hi = int(input_ids.min()), int(input_ids.max())
        if lo < 0 or hi >= vocab:
            raise ValueError(f"token ids must lie in [0, {vocab}); the batch has values from {lo} to {hi}")

    def _phase(self, name: str):
        import contextlib
        return self.timer.phase(name) if self.timer is not None else contextlib.nullcontext()

    def _weighted_loss(self, out, labels):
        """Position-weighted next-token loss of the first head (reference: train_custom.py:715-752, which
        replaces the model's loss by this one when token weighting is on)."""
        import torch.nn.functional as F
        logits = out["logits"][0] if isinstance(out["logits"], (list, tuple)) else out["logits"]
        if logits.dim() == 4:
            logits = logits[..., 0, :]
        sl, tl = logits[..., :-1, :], labels[..., 1:]
        ce = F.cross_entropy(sl.reshape(-1, sl.size(-1)).float(), tl.reshape(-1), reduction="none",
                             ignore_index=-100).view(tl.shape)
        w = self.token_weights[: ce.shape[1]].to(ce.device).unsqueeze(0)
        return (ce * w).sum() / (tl != -100).sum().clamp(min=1)

    def _forward_backward(self, ids: torch.Tensor, labels: torch.Tensor, attention_mask=None):
        want_logits = self.token_weights is not None
        with self._phase("forward"):
            if self.autocast_dtype is not None and self.device.type == "cuda":
                with torch.autocast("cuda", dtype=self.autocast_dtype):
                    out = self.model(ids, attention_mask=attention_mask, labels=labels, return_logits=want_logits)
            else:
                out = self.model(ids, attention_mask=attention_mask, labels=labels, return_logits=want_logits)
            if want_logits:
                out = dict(out)
                out["loss"] = self._weighted_loss(out, labels)
                out.pop("logits", None)
            loss = out["loss"] / self.grad_accum
        with self._phase("backward"):
            loss.backward()
        return out

    def _forward_backward_scaled(self, ids, labels, attention_mask, accum: int):
        """One micro-batch whose loss is divided by ``accum`` (for callers that drive the
        accumulation themselves, like ``Trainer``)."""
        self.model.train()
        saved, self.grad_accum = self.grad_accum, accum
        try:
            am = None if attention_mask is None else self._to_device(attention_mask)
            return self._forward_backward(ids, labels, am)
        finally:
            self.grad_accum = saved

    def apply_update(self):
        """Clip, step the optimizer (through the data-parallel plan when attached) and clear gradients."""
        if self.dp is not None:
            return self.dp.reduce_clip_and_step(self.optimizer, self.grad_clip)
        gnorm = None
        if self.grad_clip:
            gnorm = clip_grad_norm_device(list(self.model.parameters()), self.grad_clip)
        self.optimizer.step()
        self.optimizer.zero_grad(set_to_none=True)
        return gnorm

    def step(self, input_ids: torch.Tensor, labels: Optional[torch.Tensor] = None,
             attention_mask: Optional[torch.Tensor] = None) -> StepStats:
        """``input_ids``: (grad_accum * micro_batch, S) or (micro_batch, S)."""
        self.model.train()
        self._check_ids(input_ids)
        ids = self._to_device(input_ids)
        lab = ids if labels is None else self._to_device(labels)
        am = None if attention_mask is None else self._to_device(attention_mask)
        chunks = ids.chunk(self.grad_accum, dim=0) if self.grad_accum > 1 else (ids,)
        lchunks = lab.chunk(self.grad_accum, dim=0) if self.grad_accum > 1 else (lab,)
        achunks = am.chunk(self.grad_accum, dim=0) if (am is not None and self.grad_accum > 1) else (am,) * len(chunks)
        loss_acc = lm_acc = None
        out = None
        for i, (c, l, a) in enumerate(zip(chunks, lchunks, achunks)):
            if self.dp is not None:
                self.dp.set_sync(i == len(chunks) - 1)
            out = self._forward_backward(c, l, a)
            ld, lm = out["loss"].detach(), out["lm_loss"].detach()
            loss_acc = ld if loss_acc is None else loss_acc + ld
            lm_acc = lm if lm_acc is None else lm_acc + lm
        for fn in self.before_update:
            fn(self.model)
        with self._phase("optimizer"):
            gnorm = self.apply_update()
        if self.lr_scheduler is not None:
            self.lr_scheduler.step()
        self.global_step += 1
        ntok = ids.numel()
        self.tokens_seen += ntok
        n = len(chunks)
        aux = out["aux_loss"].detach() if torch.is_tensor(out["aux_loss"]) else out["aux_loss"]
        return StepStats(loss_acc / n, lm_acc / n, aux, gnorm, ntok,
                         out.get("multitoken_loss_dict"))
