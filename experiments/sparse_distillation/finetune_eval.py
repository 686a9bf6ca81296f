"""Fine-tune and evaluate a converted sparse model (counterpart of the reference's
``Experiments/sparse_distillation/finetune_eval.py``): routing statistics accumulated over
batches, perplexity, MoE-only freezing, a fine-tune loop with auxiliary losses from the cached
router logits and best / latest checkpoints, optional comparison against the dense model."""
from __future__ import annotations

import math
import os
from typing import Dict, Iterable, Optional

import torch
import torch.nn.functional as F

from .convert import SparseModelWrapper


def accumulate_routing_stats(wrapper: SparseModelWrapper, batches: Iterable[torch.Tensor]) -> Dict[int, Dict[str, float]]:
    acc: Dict[int, torch.Tensor] = {}
    wrapper.model.eval()
    with torch.no_grad():
        for ids in batches:
            wrapper(ids)
            for i, m in wrapper.moe_modules().items():
                c = m._last_expert_counts.float().cpu()
                acc[i] = c if i not in acc else acc[i] + c
    out = {}
    for i, c in acc.items():
        u = c / c.sum().clamp(min=1)
        out[i] = {"entropy": float(-(u * torch.log(u + 1e-10)).sum() / math.log(max(len(u), 2))),
                  "max_usage": float(u.max()), "min_usage": float(u.min()), "dead": int((u == 0).sum())}
    return out


@torch.no_grad()
def perplexity(model, batches: Iterable[torch.Tensor], logits_of=None) -> float:
    """Next-token perplexity; ``logits_of(output)`` extracts (B, S, V) logits from the model output."""
    tot, n = 0.0, 0
    for ids in batches:
        out = model(ids)
        logits = logits_of(out) if logits_of else (out["logits"] if isinstance(out, dict) else getattr(out, "logits", out))
        loss = F.cross_entropy(logits[:, :-1].reshape(-1, logits.shape[-1]).float(), ids[:, 1:].reshape(-1))
        k = ids[:, 1:].numel()
        tot, n = tot + float(loss) * k, n + k
    return math.exp(min(tot / max(n, 1), 50.0))


def freeze_all_but_moe(wrapper: SparseModelWrapper) -> int:
    for p in wrapper.model.parameters():
        p.requires_grad_(False)
    n = 0
    for m in wrapper.moe_modules().values():
        for p in m.parameters():
            p.requires_grad_(True)
            n += p.numel()
    return n


def finetune(wrapper: SparseModelWrapper, batches: Iterable[torch.Tensor], steps: int, lr: float = 1e-5,
             lb_weight: float = 0.01, z_weight: float = 0.001, moe_only: bool = True, out_dir: Optional[str] = None,
             eval_batches=None, logits_of=None) -> Dict[str, float]:
    if moe_only:
        freeze_all_but_moe(wrapper)
    params = [p for p in wrapper.model.parameters() if p.requires_grad]
    opt = torch.optim.AdamW(params, lr=lr, weight_decay=0.0)
    best = float("inf")
    wrapper.model.train()
    it = iter(batches)
    last = 0.0
    for s in range(steps):
        try:
            ids = next(it)
        except StopIteration:
            it = iter(batches)
            ids = next(it)
        out = wrapper(ids)
        logits = logits_of(out) if logits_of else (out["logits"] if isinstance(out, dict) else getattr(out, "logits", out))
        loss = F.cross_entropy(logits[:, :-1].reshape(-1, logits.shape[-1]).float(), ids[:, 1:].reshape(-1))
        for m in wrapper.moe_modules().values():
            rl, c = m._last_router_logits, m._last_expert_counts
            if rl is not None and m.routing == "token_choice":
                E = rl.shape[-1]
                P = F.softmax(rl.reshape(-1, E).float(), -1).mean(0)
                loss = loss + lb_weight * E * ((c.float() / c.sum().clamp(min=1)) * P).sum()
            if rl is not None:
                loss = loss + z_weight * torch.logsumexp(rl.float(), -1).pow(2).mean()
        opt.zero_grad(set_to_none=True)
        loss.backward()
        torch.nn.utils.clip_grad_norm_(params, 1.0)
        opt.step()
        last = float(loss)
        if out_dir and eval_batches is not None and (s + 1) % max(steps // 4, 1) == 0:
            os.makedirs(out_dir, exist_ok=True)
            ppl = perplexity(wrapper, eval_batches, logits_of)
            wrapper.model.train()
            torch.save({"model": wrapper.model.state_dict(), "step": s + 1, "ppl": ppl}, os.path.join(out_dir, "latest_checkpoint.pt"))
            if ppl < best:
                best = ppl
                torch.save({"model": wrapper.model.state_dict(), "step": s + 1, "ppl": ppl}, os.path.join(out_dir, "best_checkpoint.pt"))
    return {"final_loss": last, "best_ppl": best}
