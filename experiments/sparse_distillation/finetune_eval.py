"""Fine-tune and evaluate a converted sparse model (counterpart of the reference's
``Experiments/sparse_distillation/finetune_eval.py``): routing statistics accumulated over
batches, perplexity, MoE-only freezing, a fine-tune loop with auxiliary losses from the cached
router logits and best / latest checkpoints, optional comparison against the dense model."""
from __future__ import annotations

import math
import os
from typing import Dict, Iterable, List, Optional

import torch
import torch.nn.functional as F

from .convert import SparseModelWrapper


def _layer_stats(counts: torch.Tensor) -> Dict[str, object]:
    """Balance figures of one layer from its per-expert assignment counts."""
    counts = counts.float().cpu()
    E = counts.numel()
    tot = float(counts.sum())
    if tot <= 0:
        return {"n_experts": E, "total_tokens": 0}
    u = counts / tot
    ent = float(-(u * torch.log(u + 1e-10)).sum())
    srt, _ = torch.sort(u)
    idx = torch.arange(1, E + 1, dtype=torch.float32)
    gini = float(((2 * idx - E - 1) * srt).sum() / E)               # 0 = uniform, 1 - 1/E = one expert
    meaningful = int((u > 0.1 / E).sum())                            # at least a tenth of the uniform share
    return {"n_experts": E, "total_tokens": int(tot), "expert_counts": counts.tolist(), "expert_fracs": u.tolist(),
            "entropy": ent, "normalized_entropy": ent / math.log(E) if E > 1 else 0.0, "gini": gini,
            "max_entropy": math.log(E), "min_frac": float(u.min()), "max_frac": float(u.max()),
            "imbalance": float(u.max() * E), "imbalance_ratio": float(u.max() / (u.min() + 1e-10)),
            "active_experts": int((counts > 0).sum()), "meaningful_experts": meaningful,
            "collapsed": meaningful < 0.5 * E}


def _summarise(per_layer: Dict[int, Dict[str, object]], verbose: bool) -> Dict[str, object]:
    live = {i: s for i, s in per_layer.items() if s.get("total_tokens", 0) > 0}
    agg: Dict[str, object] = {}
    if live:
        ne = [s["normalized_entropy"] for s in live.values()]
        agg = {"mean_normalized_entropy": sum(ne) / len(ne), "min_normalized_entropy": min(ne),
               "worst_max_frac": max(s["max_frac"] for s in live.values()),
               "worst_min_frac": min(s["min_frac"] for s in live.values()),
               "mean_active_experts": sum(s["active_experts"] for s in live.values()) / len(live),
               "mean_active_expert_frac": sum(s["active_experts"] / s["n_experts"] for s in live.values()) / len(live),
               "collapsed_layers": [i for i, s in live.items() if s["collapsed"]]}
        agg["n_collapsed"] = len(agg["collapsed_layers"])
    if verbose:
        for i, s in sorted(live.items()):
            flag = "  COLLAPSED" if s["collapsed"] else ""
            print(f"  layer {i:3d}: entropy {s['normalized_entropy']:.3f}  gini {s['gini']:.3f}  "
                  f"max {s['max_frac']:.3f}  min {s['min_frac']:.4f}  active {s['active_experts']}/{s['n_experts']}{flag}")
        if agg:
            print(f"  mean entropy {agg['mean_normalized_entropy']:.3f}, collapsed layers: {agg['collapsed_layers'] or 'none'}")
    return {"per_layer": per_layer, "aggregate": agg}


def _moe_dict(moe_layers) -> Dict[int, torch.nn.Module]:
    if isinstance(moe_layers, SparseModelWrapper):
        return moe_layers.moe_modules()
    return {int(k): v for k, v in moe_layers.items()}


def compute_routing_stats(moe_layers, verbose: bool = True) -> Dict[str, object]:
    """Load balance of every MoE layer in the LAST forward pass: entropy (normalised by log E), Gini, min /
    max share, active experts, and a collapse flag (fewer than half of the experts get a tenth of the uniform
    share).  ``moe_layers``: a ``SparseModelWrapper`` or a mapping layer index -> MoE layer
    (reference: Experiments/sparse_distillation/finetune_eval.py:67-209)."""
    per = {}
    for i, m in sorted(_moe_dict(moe_layers).items()):
        c = getattr(m, "_last_expert_counts", None)
        per[i] = _layer_stats(c) if c is not None else {"n_experts": m.n_experts, "total_tokens": 0}
    return _summarise(per, verbose)


def reset_routing_stats(moe_layers) -> None:
    for m in _moe_dict(moe_layers).values():
        m._accumulated_counts = None


def start_routing_accumulation(moe_layers) -> None:
    """From now on ``accumulate_routing_stats`` adds each forward's counts to a running total."""
    reset_routing_stats(moe_layers)
    for m in _moe_dict(moe_layers).values():
        m._accumulate_routing = True


def stop_routing_accumulation(moe_layers) -> None:
    for m in _moe_dict(moe_layers).values():
        m._accumulate_routing = False


def accumulate_routing_stats(moe_layers, batches: Optional[Iterable[torch.Tensor]] = None):
    """Without ``batches``: fold the last forward's counts into the running totals of the layers that are
    accumulating (call after each forward).  With ``batches`` (wrapper only): run them and return the
    accumulated per-layer summary - the one-call form."""
    if batches is not None:
        return _accumulate_over(moe_layers, batches)
    for m in _moe_dict(moe_layers).values():
        if getattr(m, "_accumulate_routing", False) and getattr(m, "_last_expert_counts", None) is not None:
            c = m._last_expert_counts.detach().float().cpu()
            acc = getattr(m, "_accumulated_counts", None)
            m._accumulated_counts = c if acc is None else acc + c


def compute_routing_stats_accumulated(moe_layers, verbose: bool = True) -> Dict[str, object]:
    """Same figures as ``compute_routing_stats`` over everything accumulated since
    ``start_routing_accumulation`` (reference: finetune_eval.py:251-385)."""
    per = {}
    for i, m in sorted(_moe_dict(moe_layers).items()):
        c = getattr(m, "_accumulated_counts", None)
        per[i] = _layer_stats(c) if c is not None else {"n_experts": m.n_experts, "total_tokens": 0}
    return _summarise(per, verbose)


def _accumulate_over(wrapper: SparseModelWrapper, batches: Iterable[torch.Tensor]) -> Dict[int, Dict[str, float]]:
    start_routing_accumulation(wrapper)
    wrapper.model.eval()
    with torch.no_grad():
        for ids in batches:
            wrapper(ids)
            accumulate_routing_stats(wrapper)
    stop_routing_accumulation(wrapper)
    out = {}
    for i, st in compute_routing_stats_accumulated(wrapper, verbose=False)["per_layer"].items():
        if st.get("total_tokens", 0) > 0:
            out[i] = {"entropy": st["normalized_entropy"], "max_usage": st["max_frac"], "min_usage": st["min_frac"],
                      "dead": st["n_experts"] - st["active_experts"], "gini": st["gini"]}
    return out


def _logits(out, logits_of=None):
    if logits_of is not None:
        return logits_of(out)
    return out["logits"] if isinstance(out, dict) else getattr(out, "logits", out)


def _ids_of(batch):
    if isinstance(batch, dict):
        return batch.get("input_ids", batch.get("tokens"))
    return batch[0] if isinstance(batch, (list, tuple)) else batch


@torch.no_grad()
def compute_perplexity(model, batches: Iterable = None, logits_of=None, pad_token_id: Optional[int] = None,
                       max_batches: Optional[int] = None, accumulate_routing: bool = False, dataloader=None,
                       device=None) -> float:
    """Token-weighted next-token perplexity.  Positions whose target is ``pad_token_id`` do not count;
    ``accumulate_routing`` (model = ``SparseModelWrapper``) folds every batch's expert counts into the
    layers' running totals (reference: finetune_eval.py:388-464).  The reference's call form
    ``compute_perplexity(model, dataloader, device, ...)`` works too: batches are moved to ``device``."""
    batches = dataloader if batches is None else batches
    if logits_of is not None and not callable(logits_of):        # third positional is a device
        device, logits_of = logits_of, None
    tot, n = 0.0, 0
    was_training = getattr(model, "training", False)
    model.eval()
    if accumulate_routing:
        start_routing_accumulation(model)
    for bi, batch in enumerate(batches):
        if max_batches is not None and bi >= max_batches:
            break
        ids = _ids_of(batch)
        if device is not None:
            ids = ids.to(device)
        logits = _logits(model(ids), logits_of)
        tgt = ids[:, 1:].reshape(-1)
        if pad_token_id is not None:
            tgt = tgt.masked_fill(tgt == pad_token_id, -100)
        k = int((tgt != -100).sum())
        if k == 0:
            continue
        loss = F.cross_entropy(logits[:, :-1].reshape(-1, logits.shape[-1]).float(), tgt, ignore_index=-100)
        tot, n = tot + float(loss) * k, n + k
        if accumulate_routing:
            accumulate_routing_stats(model)
    if accumulate_routing:
        stop_routing_accumulation(model)
    if was_training:
        model.train()
    return math.exp(min(tot / max(n, 1), 50.0))


def perplexity(model, batches: Iterable[torch.Tensor], logits_of=None) -> float:
    """Next-token perplexity; ``logits_of(output)`` extracts (B, S, V) logits from the model output."""
    return compute_perplexity(model, batches, logits_of)


def compare_dense(dense_model, wrapper: SparseModelWrapper, batches, logits_of=None,
                  pad_token_id: Optional[int] = None) -> Dict[str, float]:
    """Perplexity of the original dense model against the converted sparse one on the same batches."""
    batches = list(batches)
    d = compute_perplexity(dense_model, batches, logits_of, pad_token_id)
    s_ = compute_perplexity(wrapper, batches, logits_of, pad_token_id)
    return {"dense_ppl": d, "sparse_ppl": s_, "ratio": s_ / d if d > 0 else float("inf")}


def compute_load_balancing_loss(router_logits: torch.Tensor, expert_counts: torch.Tensor) -> torch.Tensor:
    """E * sum_e f_e P_e: f = share of the assignments each expert received, P = mean routing probability."""
    E = router_logits.shape[-1]
    P = F.softmax(router_logits.reshape(-1, E).float(), -1).mean(0)
    f = expert_counts.float() / expert_counts.sum().clamp(min=1)
    return E * (f * P).sum()


def compute_z_loss(router_logits: torch.Tensor) -> torch.Tensor:
    """Mean squared log-sum-exp of the router logits."""
    return torch.logsumexp(router_logits.reshape(-1, router_logits.shape[-1]).float(), -1).pow(2).mean()


def freeze_non_moe_layers(model, moe_only: bool = False):
    """The parameters to train: all of them, or with ``moe_only`` the experts, routers and norms (the rest is
    frozen) - the name rule of the reference (finetune_eval.py:467-495).  ``freeze_all_but_moe`` is the stricter
    form used by this file's ``finetune``: MoE layers only, found by module, not by name."""
    if not moe_only:
        return list(model.parameters())
    keep = []
    for name, p in model.named_parameters():
        low = name.lower()
        on = "experts" in low or "router" in low or "expert_bias" in low or "norm" in low or "ln" in low
        p.requires_grad_(on)
        if on:
            keep.append(p)
    return keep


def freeze_all_but_moe(wrapper: SparseModelWrapper) -> int:
    for p in wrapper.model.parameters():
        p.requires_grad_(False)
    n = 0
    for m in wrapper.moe_modules().values():
        for p in m.parameters():
            p.requires_grad_(True)
            n += p.numel()
    return n


def aux_losses(wrapper: SparseModelWrapper, lb_weight: float, z_weight: float) -> torch.Tensor:
    """Load-balance (E * sum_e f_e P_e) and z (mean logsumexp^2) terms from the router logits each MoE
    layer cached in the forward pass that just ran."""
    total = None
    for m in wrapper.moe_modules().values():
        rl, c = getattr(m, "_last_router_logits", None), getattr(m, "_last_expert_counts", None)
        if rl is None:
            continue
        t = 0.0
        if lb_weight > 0 and c is not None and m.routing == "token_choice":
            t = t + lb_weight * compute_load_balancing_loss(rl, c)
        if z_weight > 0:
            t = t + z_weight * compute_z_loss(rl)
        if torch.is_tensor(t):
            total = t if total is None else total + t
    return total if total is not None else torch.zeros((), device=next(wrapper.model.parameters()).device)


def _save(path: str, wrapper: SparseModelWrapper, opt, step: int, ppl: float, with_optimizer: bool) -> None:
    """``moe_layers`` (flat ``"<layer>.<key>"`` state dict), ``global_step``, ``best_ppl`` and
    ``optimizer_state_dict`` are the reference's keys (finetune_eval.py:656-681); ``model`` adds the rest of the
    model, which fine-tuning without ``moe_only`` changes too."""
    os.makedirs(os.path.dirname(path) or ".", exist_ok=True)
    ck = {"model": wrapper.model.state_dict(), "moe_layers": wrapper.moe_layers.state_dict(), "step": step,
          "global_step": step, "ppl": ppl, "best_ppl": ppl}
    if with_optimizer:
        ck["optimizer_state_dict"] = opt.state_dict()
    torch.save(ck, path)


def load_finetuned(wrapper: SparseModelWrapper, path: str, optimizer=None) -> int:
    """Load weights saved by ``finetune`` here or by the reference's (MoE layers only), and the optimizer state
    when one is passed (resume).  Returns the step the file was written at."""
    from .distill import checkpoint_layers, load_layer_state
    ck = torch.load(path, map_location="cpu", weights_only=False)
    if "model" in ck:
        wrapper.model.load_state_dict(ck["model"])
    elif ck.get("moe_layers") is not None:
        mods = wrapper.moe_modules()
        for k, sd in checkpoint_layers({"moe_layers": ck["moe_layers"]}).items():
            load_layer_state(mods[int(k)], sd)
    opt_state = ck.get("optimizer_state_dict", ck.get("optimizer"))
    if optimizer is not None and opt_state is not None:
        optimizer.load_state_dict(opt_state)
    return int(ck.get("step", ck.get("global_step", 0)))


_REF_ORDER = ("model", "train_dataloader", "eval_dataloader", "device", "epochs", "lr", "eval_every", "max_steps",
              "use_8bit_adam", "pad_token_id", "moe_only", "load_balance_weight", "z_loss_weight", "resume_checkpoint",
              "save_dir", "use_lr_schedule")
_OWN_ORDER = ("wrapper", "batches", "steps", "lr", "lb_weight", "z_weight", "moe_only", "out_dir", "eval_batches",
              "logits_of", "eval_every", "lr_schedule", "resume", "pad_token_id", "max_grad_norm", "log_every",
              "use_8bit_adam")


def finetune(*args, **kwargs) -> Dict[str, object]:
    """Fine-tune a converted model; see ``_finetune`` for the arguments.  Positional arguments are read in this
    file's order ``(wrapper, batches, steps, lr, ...)`` when the third one is a step count (or absent), and in the
    reference's order ``(model, train_dataloader, eval_dataloader, device, epochs, lr, ...)`` otherwise."""
    order = _REF_ORDER if len(args) >= 3 and not isinstance(args[2], int) else _OWN_ORDER
    for name, value in zip(order, args):
        if name in kwargs:
            raise TypeError(f"finetune() got multiple values for argument '{name}'")
        kwargs[name] = value
    return _finetune(**kwargs)


def _finetune(wrapper: SparseModelWrapper = None, batches: Iterable = None, steps=None, lr: float = 1e-5,
             lb_weight: Optional[float] = None, z_weight: Optional[float] = None, moe_only: bool = True,
             out_dir: Optional[str] = None, eval_batches=None, logits_of=None, eval_every: Optional[int] = None,
             lr_schedule: bool = False, resume: Optional[str] = None, pad_token_id: Optional[int] = None,
             max_grad_norm: float = 1.0, log_every: int = 0, use_8bit_adam: bool = False, *,
             model=None, train_dataloader=None, eval_dataloader=None, device=None, epochs: int = 1,
             max_steps: Optional[int] = None, load_balance_weight: Optional[float] = None,
             z_loss_weight: Optional[float] = None, resume_checkpoint: Optional[str] = None,
             save_dir: Optional[str] = None, use_lr_schedule: Optional[bool] = None) -> Dict[str, object]:
    """Language-model fine-tuning of the converted model: cross-entropy plus the routers' auxiliary losses,
    gradient clipping, constant LR or cosine decay to 10 %, evaluation every ``eval_every`` steps with
    ``latest_checkpoint.pt`` (with optimizer state, for ``resume``) and ``best_checkpoint.pt`` under
    ``out_dir`` (reference: finetune_eval.py:498-693).

    The keyword names of the reference are accepted as well (``model``, ``train_dataloader``, ``eval_dataloader``,
    ``device``, ``epochs``, ``max_steps``, ``load_balance_weight``, ``z_loss_weight``, ``resume_checkpoint``,
    ``save_dir``, ``use_lr_schedule``)."""
    wrapper = model if wrapper is None else wrapper
    batches = train_dataloader if batches is None else batches
    eval_batches = eval_dataloader if eval_batches is None else eval_batches
    lb_weight = (0.01 if load_balance_weight is None else load_balance_weight) if lb_weight is None else lb_weight
    z_weight = (0.001 if z_loss_weight is None else z_loss_weight) if z_weight is None else z_weight
    resume = resume_checkpoint if resume is None else resume
    out_dir = save_dir if out_dir is None else out_dir
    lr_schedule = lr_schedule if use_lr_schedule is None else use_lr_schedule
    if device is not None:
        wrapper.to(device)
        batches = [_to_device(b, device) for b in batches]
        eval_batches = [_to_device(b, device) for b in eval_batches] if eval_batches is not None else None
    if steps is None:
        n = len(batches) if hasattr(batches, "__len__") else None
        steps = max_steps if n is None else min(max_steps or epochs * n, epochs * n)
        assert steps is not None, "give steps / max_steps for a data source without a length"
    if moe_only:
        freeze_all_but_moe(wrapper)
    params = [p for p in wrapper.model.parameters() if p.requires_grad]
    opt, opt_name = None, "adamw"
    if use_8bit_adam:                            # the reference's default when bitsandbytes is importable
        try:
            import bitsandbytes as bnb
            opt, opt_name = bnb.optim.Adam8bit(params, lr=lr), "adam8bit"
        except Exception:
            opt = None
    if opt is None:
        opt = torch.optim.AdamW(params, lr=lr, weight_decay=0.0)
    start = load_finetuned(wrapper, resume, opt) if resume else 0
    eval_every = eval_every or max(steps // 4, 1)
    best, last = float("inf"), 0.0
    history: List[Dict[str, float]] = []
    wrapper.model.train()
    it = iter(batches)
    for s in range(start, steps):
        try:
            batch = next(it)
        except StopIteration:
            it = iter(batches)
            batch = next(it)
        if lr_schedule:
            for g in opt.param_groups:
                g["lr"] = lr * (0.1 + 0.9 * 0.5 * (1 + math.cos(math.pi * s / max(steps, 1))))
        ids = _ids_of(batch)
        logits = _logits(wrapper(ids), logits_of)
        tgt = ids[:, 1:].reshape(-1)
        if pad_token_id is not None:
            tgt = tgt.masked_fill(tgt == pad_token_id, -100)
        lm = F.cross_entropy(logits[:, :-1].reshape(-1, logits.shape[-1]).float(), tgt, ignore_index=-100)
        loss = lm + aux_losses(wrapper, lb_weight, z_weight)
        opt.zero_grad(set_to_none=True)
        loss.backward()
        torch.nn.utils.clip_grad_norm_(params, max_grad_norm)
        opt.step()
        last = float(loss.detach())
        if log_every and (s + 1) % log_every == 0:
            print(f"step {s + 1}/{steps}  loss {last:.4f}  lm {float(lm.detach()):.4f}", flush=True)
        if eval_batches is not None and ((s + 1) % eval_every == 0 or s + 1 == steps):
            ppl = compute_perplexity(wrapper, eval_batches, logits_of, pad_token_id)
            wrapper.model.train()
            history.append({"step": s + 1, "ppl": ppl, "loss": last})
            if out_dir:
                _save(os.path.join(out_dir, "latest_checkpoint.pt"), wrapper, opt, s + 1, ppl, True)
            if ppl < best:
                best = ppl
                if out_dir:
                    _save(os.path.join(out_dir, "best_checkpoint.pt"), wrapper, opt, s + 1, ppl, False)
    return {"final_loss": last, "best_ppl": best, "history": history, "optimizer": opt_name}


def _to_device(batch, device):
    if isinstance(batch, dict):
        return {k: (v.to(device) if torch.is_tensor(v) else v) for k, v in batch.items()}
    return batch.to(device) if torch.is_tensor(batch) else batch


def _token_batches(a, vocab: int, n: int, seed: int):
    """``n`` batches of token ids: the tokenised data set when it can be loaded, else the uint16 file ``--data``
    names, else random ids from a seed.  Returns (batches, source, pad id)."""
    from .data import load_token_batches
    return load_token_batches(a.model, vocab, dataset=a.dataset, dataset_config=a.dataset_config, data_file=a.data,
                              max_samples=a.max_samples, seq_len=a.seq_len, batch_size=a.batch_size, n_batches=n,
                              seed=seed, device=a.device)


def main(argv=None):
    """Fine-tune and/or evaluate a distilled checkpoint:

        python -m experiments.sparse_distillation.finetune_eval --model toy --checkpoint out/distilled_moe_layers.pt \\
            [--eval_only] [--compare_dense] [--random_init] [--moe_only] [--lr_schedule] [--resume latest.pt]

    Every argument of the reference's script (Experiments/sparse_distillation/finetune_eval.py:696-770) is
    accepted under the same name.
    """
    import argparse
    import copy
    import json
    from .convert import convert_to_sparse
    ap = argparse.ArgumentParser(description="fine-tune and evaluate a sparse (distilled) model")
    ap.add_argument("--model", default="toy", help="'toy' or a local Hugging Face model directory")
    ap.add_argument("--checkpoint", required=True, help="file written by SparseDistillationTrainer.save")
    ap.add_argument("--layer_config", default=None, help="layer_config.json with per-layer n_experts / d_ff_expert / top_k")
    ap.add_argument("--dtype", default="float32", choices=["float32", "float16", "bfloat16"])
    ap.add_argument("--dataset", default="wikitext")
    ap.add_argument("--dataset_config", default="wikitext-2-raw-v1")
    ap.add_argument("--max_samples", type=int, default=20000)
    ap.add_argument("--data", default=None, help="uint16 token file used when the data set cannot be loaded; "
                    "random tokens when absent as well")
    ap.add_argument("--seq_len", type=int, default=64)
    ap.add_argument("--batch_size", type=int, default=4)
    ap.add_argument("--epochs", type=int, default=1)
    ap.add_argument("--max_steps", type=int, default=100)
    ap.add_argument("--no_8bit_adam", action="store_true",
                    help="plain AdamW even where bitsandbytes' 8-bit Adam could be imported")
    ap.add_argument("--balanced-routing", "--balanced_routing", dest="balanced_routing", action="store_true",
                    help="token choice under a per-expert capacity, to keep every expert in use")
    ap.add_argument("--compile", action="store_true", help="torch.compile the model before training")
    ap.add_argument("--compile_mode", default="max-autotune",
                    choices=["default", "reduce-overhead", "max-autotune", "max-autotune-no-cudagraphs"])
    ap.add_argument("--eval_every", type=int, default=None)
    ap.add_argument("--eval_batches", type=int, default=8)
    ap.add_argument("--lr", type=float, default=1e-4)
    ap.add_argument("--moe_only", action="store_true")
    ap.add_argument("--lr_schedule", action="store_true")
    ap.add_argument("--load_balance_weight", type=float, default=0.01)
    ap.add_argument("--z_loss_weight", type=float, default=0.001)
    ap.add_argument("--resume", default=None, help="latest_checkpoint.pt of an earlier run (with optimizer state)")
    ap.add_argument("--load_finetuned", default=None, help="weights of an earlier run, no optimizer state")
    ap.add_argument("--eval_only", action="store_true")
    ap.add_argument("--compare_dense", action="store_true")
    ap.add_argument("--random_init", action="store_true", help="control: random experts instead of distilled ones")
    ap.add_argument("--output", default=None)
    ap.add_argument("--device", default="cpu")
    a = ap.parse_args(argv)
    dtype = {"float32": torch.float32, "float16": torch.float16, "bfloat16": torch.bfloat16}[a.dtype]
    if a.model == "toy":
        from .example_usage import ToyLM
        torch.manual_seed(0)
        model, vocab = ToyLM().to(dtype), 256
    else:
        from transformers import AutoModelForCausalLM
        model = AutoModelForCausalLM.from_pretrained(a.model, torch_dtype=dtype)
        vocab = model.config.vocab_size
    model.to(a.device)
    dense = copy.deepcopy(model).eval() if a.compare_dense else None
    wrapper = convert_to_sparse(model, distilled_path=a.checkpoint, random_init=a.random_init,
                                layer_config_path=a.layer_config)
    balanced = 0
    if a.balanced_routing:
        for layer in wrapper.moe_modules().values():
            if hasattr(layer, "balanced_routing") and getattr(layer, "routing", "") == "token_choice":
                layer.balanced_routing = True
                balanced += 1
    if a.load_finetuned:
        load_finetuned(wrapper, a.load_finetuned)
    if a.compile:
        try:
            wrapper.model = torch.compile(wrapper.model, mode=a.compile_mode, fullgraph=False)
        except Exception as e:
            print(f"torch.compile failed ({type(e).__name__}: {e}); continuing without it")
    train_b, source, pad = _token_batches(a, vocab, max(a.max_steps, 1), seed=1)
    eval_b, _, _ = _token_batches(a, vocab, a.eval_batches, seed=2)
    a.max_steps = min(a.max_steps, max(a.epochs, 1) * max(len(train_b), 1))
    report: Dict[str, object] = {"parameters": wrapper.count_parameters(), "data": source,
                                 "balanced_routing_layers": balanced}
    report["ppl_before"] = compute_perplexity(wrapper, eval_b, accumulate_routing=True)
    report["routing_before"] = compute_routing_stats_accumulated(wrapper, verbose=False)["aggregate"]
    if not a.eval_only:
        report["finetune"] = finetune(wrapper, train_b, a.max_steps, lr=a.lr, lb_weight=a.load_balance_weight,
                                      z_weight=a.z_loss_weight, moe_only=a.moe_only, out_dir=a.output,
                                      eval_batches=eval_b, eval_every=a.eval_every, lr_schedule=a.lr_schedule,
                                      resume=a.resume, pad_token_id=pad, use_8bit_adam=not a.no_8bit_adam)
        report["ppl_after"] = compute_perplexity(wrapper, eval_b, accumulate_routing=True)
        report["routing_after"] = compute_routing_stats_accumulated(wrapper, verbose=False)["aggregate"]
    if dense is not None:
        report["dense_ppl"] = compute_perplexity(dense, eval_b)
    print(json.dumps(report, indent=1, default=str))
    if a.output:
        os.makedirs(a.output, exist_ok=True)
        json.dump(report, open(os.path.join(a.output, "finetune_report.json"), "w"), indent=1, default=str)
    return report


if __name__ == "__main__":
    main()
