"""Training diagnosis for a checkpoint (counterpart of the reference's ``tools/diagnose_training.py``):
router collapse, parameter movement against a fresh initialisation, trainability, gradient flow,
loss on data and a greedy generation sample.

    python tools/diagnose_training.py --checkpoint ckpt.pt --config cfg.yaml [--device cpu] [--synthetic]
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def parameter_movement(model, cfg) -> dict:
    """Relative distance ||w - w_init|| / ||w_init|| per top-level component against a same-seed fresh model."""
    from kolmogorov_moe_architecture_b200 import MoETransformer
    torch.manual_seed(0)
    fresh = MoETransformer(cfg, verbose=False)
    out = {}
    cur = dict(model.named_parameters())
    for n, p0 in fresh.named_parameters():
        key = ".".join(n.split(".")[:3]) if n.startswith("layers") else n.split(".")[0]
        d = out.setdefault(key, [0.0, 0.0])
        d[0] += float((cur[n].detach().float().cpu() - p0.detach().float()).pow(2).sum())
        d[1] += float(p0.detach().float().pow(2).sum())
    return {k: (v[0] / max(v[1], 1e-12)) ** 0.5 for k, v in out.items()}


def trainability(model) -> dict:
    tot = sum(p.numel() for p in model.parameters())
    tr = sum(p.numel() for p in model.parameters() if p.requires_grad)
    frozen = [n for n, p in model.named_parameters() if not p.requires_grad]
    return {"total": tot, "trainable": tr, "frozen_tensors": frozen}


def gradient_flow(model, ids) -> dict:
    from kolmogorov_moe_architecture_b200.utils.fault import gradient_census
    model.train()
    model.zero_grad(set_to_none=True)
    model(ids, labels=ids, return_logits=False)["loss"].backward()
    return gradient_census(model)


def calculate_gini(array) -> float:
    """Gini coefficient of non-negative values (0 = all equal, -> 1 = one holds everything)."""
    values = array
    v = torch.as_tensor(values, dtype=torch.float64).flatten().clamp(min=0).sort().values
    n, tot = v.numel(), float(v.sum())
    if n == 0 or tot == 0:
        return 0.0
    idx = torch.arange(1, n + 1, dtype=torch.float64)
    return float(((2 * idx - n - 1) * v).sum() / (n * tot))


@torch.no_grad()
def analyze_router_collapse(model, n_samples: int = 8, seq_len: int = 64, device: str = "cpu", generator=None) -> dict:
    """Expert usage through the WHOLE model on token batches (``check_router_collapse`` probes each router
    alone with random hidden states): per MoE layer the usage entropy, Gini, dead experts and the share of
    the busiest expert, from the counts each layer records in its forward pass
    (reference: tools/diagnose_training.py:113-233)."""
    import math
    cfg = model.config
    was = model.training
    model.eval()
    totals = {}
    for _ in range(n_samples):
        ids = torch.randint(0, cfg.vocab_size, (1, min(seq_len, cfg.max_seq_len)), generator=generator).to(device)
        model(ids, return_logits=False)
        for i, layer in enumerate(model.layers):
            c = getattr(getattr(layer, "ffn", None), "last_expert_counts", None)
            if c is None:
                c = getattr(getattr(getattr(layer, "ffn", None), "expert_parallel_layer", None), "last_expert_counts", None)
            if c is not None:
                totals[i] = totals.get(i, 0) + c.detach().float().cpu()
    if was:
        model.train()
    out = {}
    for i, c in totals.items():
        u = c / c.sum().clamp(min=1)
        E = u.numel()
        ent = float(-(u * torch.log(u + 1e-10)).sum()) / (math.log(E) if E > 1 else 1.0)
        out[i] = {"entropy": ent, "gini": calculate_gini(c), "dead_experts": int((c == 0).sum()),
                  "max_usage": float(u.max()), "is_collapsed": ent < 0.7 or float(u.max()) > 0.5}
    return out


@torch.no_grad()
def run_evaluation(model, config=None, n_batches: int = 8, device: str = "cpu", data: str = None, batch_size: int = 2,
                   seq_len: int = None, cfg=None) -> dict:
    """Mean loss / perplexity of head 0 (next token) and of the full multi-token objective over batches from a
    uint16 token file, or over random tokens when there is none - where a trained model should sit near
    ln(vocab) and a broken one far above (reference: tools/diagnose_training.py:354-467)."""
    cfg = config if cfg is None else cfg
    import math
    import numpy as np
    S = seq_len or min(256, cfg.max_seq_len)
    g = torch.Generator().manual_seed(0)
    arr = np.memmap(data, dtype=np.uint16, mode="r") if data else None
    was = model.training
    model.eval()
    tot, lm, n = 0.0, 0.0, 0
    for _ in range(n_batches):
        if arr is not None:
            starts = torch.randint(0, len(arr) - S - 1, (batch_size,), generator=g).tolist()
            ids = torch.stack([torch.from_numpy(np.asarray(arr[s: s + S], dtype=np.int64)) for s in starts])
        else:
            ids = torch.randint(0, cfg.vocab_size, (batch_size, S), generator=g)
        ids = ids.to(device)
        out = model(ids, labels=ids, return_logits=False)
        tot += float(out["loss"])
        lm += float(out.get("lm_loss", out["loss"]))
        n += 1
    if was:
        model.train()
    mean = lm / max(n, 1)
    return {"loss": tot / max(n, 1), "lm_loss": mean, "perplexity": math.exp(min(mean, 50.0)),
            "uniform_loss": math.log(cfg.vocab_size), "batches": n, "source": data or "random tokens"}


def findings(report: dict) -> list:
    """Plain-language findings from the collected figures."""
    issues = []
    bad = [i for i, s in report.get("routing_in_model", {}).items() if s["is_collapsed"]]
    if report.get("collapsed") or bad:
        issues.append(f"router collapse in layers {sorted(set(list(report.get('collapsed', [])) + bad))}")
    still = [k for k, v in report.get("movement", {}).items() if v < 1e-4]
    if still:
        issues.append(f"{len(still)} components did not move from their initialisation: {still[:5]}")
    tr = report.get("trainability", {})
    if tr and tr["trainable"] < tr["total"]:
        issues.append(f"{tr['total'] - tr['trainable']:,} parameters are frozen")
    ev = report.get("evaluation")
    if ev and ev["lm_loss"] > ev["uniform_loss"] * 1.05 and ev["source"] != "random tokens":
        issues.append(f"loss on data {ev['lm_loss']:.3f} is above the uniform-prediction loss {ev['uniform_loss']:.3f}")
    for k, v in report.get("gradients", {}).items():
        if isinstance(v, dict) and (v.get("nan_or_inf", 0) or v.get("no_grad", 0)):
            issues.append(f"gradients of '{k}': {v.get('nan_or_inf', 0)} non-finite, {v.get('no_grad', 0)} missing")
    return issues or ["no problem found"]


@torch.no_grad()
def greedy_sample(model, prompt_ids, n: int = 20):
    model.eval()
    ids = prompt_ids
    for _ in range(n):
        h, _ = model.forward_hidden(ids[:, -model.config.max_seq_len:])
        ids = torch.cat([ids, model.lm_heads[0](h[:, -1]).argmax(-1, keepdim=True)], dim=1)
    return ids


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--checkpoint", default=None)
    ap.add_argument("--config", required=True)
    ap.add_argument("--device", default=None, help="default: cuda:<--gpu> when a GPU is present, else cpu")
    ap.add_argument("--gpu", type=int, default=0, help="GPU index (the reference's way of naming the device)")
    ap.add_argument("--synthetic", action="store_true")
    ap.add_argument("--data", default=None, help="uint16 token file for the evaluation pass")
    ap.add_argument("--eval-batches", type=int, default=8)
    ap.add_argument("--skip-eval", action="store_true", help="no evaluation pass")
    ap.add_argument("--skip-generation", action="store_true", help="no greedy sample")
    a = ap.parse_args(argv)
    if a.device is None:
        a.device = f"cuda:{a.gpu}" if torch.cuda.is_available() else "cpu"
    from eval.evaluate_perplexity import load_model
    from kolmogorov_moe_architecture_b200.utils.fault import check_router_collapse
    model, cfg = load_model(a.checkpoint, a.config, a.device, dtype=torch.float32 if a.device == "cpu" else torch.bfloat16)
    stats, collapsed, summary = check_router_collapse(model)
    print("[router]", summary)
    for i, s in stats.items():
        print(f"  layer {i}: entropy {s['entropy']:.3f} max_usage {s['max_usage']:.3f}")
    in_model = analyze_router_collapse(model, device=a.device)
    for i, s in in_model.items():
        print(f"  layer {i} (through the model): entropy {s['entropy']:.3f} gini {s['gini']:.3f} dead {s['dead_experts']}")
    mv = parameter_movement(model, cfg)
    print("[movement] least moved:", sorted(mv.items(), key=lambda kv: kv[1])[:5])
    tr = trainability(model)
    print(f"[trainable] {tr['trainable']:,} of {tr['total']:,}; frozen tensors: {len(tr['frozen_tensors'])}")
    ev = None
    if not a.skip_eval:
        ev = run_evaluation(model, cfg, a.eval_batches, a.device, None if a.synthetic else a.data)
        print(f"[eval] {ev['source']}: loss {ev['lm_loss']:.4f} (uniform {ev['uniform_loss']:.4f}) "
              f"ppl {ev['perplexity']:.1f}")
    ids = torch.randint(0, cfg.vocab_size, (2, min(64, cfg.max_seq_len)), device=a.device)
    grads = gradient_flow(model, ids)
    for k, v in grads.items():
        print(f"[grad] {k}: {v}")
    if not a.skip_generation:
        print("[sample]", greedy_sample(model, ids[:1, :8], 12)[0].tolist())
    report = {"router": stats, "collapsed": collapsed, "routing_in_model": in_model, "movement": mv,
              "trainability": tr, "gradients": grads}
    if ev is not None:
        report["evaluation"] = ev
    report["findings"] = findings(report)
    for line in report["findings"]:
        print("[finding]", line)
    return report


# ---- names of the reference's tool, for code that imports them from here
def create_model_config(config_dict):
    """``AdvancedMoEConfig`` from a YAML dict (its ``model:`` section, read with defaults)."""
    from kolmogorov_moe_architecture_b200.utils.config_io import model_config_tolerant
    return model_config_tolerant(config_dict)


def load_checkpoint(checkpoint_path, config_path, device="cpu"):
    """(model with the checkpoint's weights, model configuration)."""
    from eval.evaluate_perplexity import load_model
    return load_model(checkpoint_path, config_path, device,
                      dtype=torch.float32 if str(device) == "cpu" else torch.bfloat16)


def create_fresh_model(config, device="cpu", seed: int = 0):
    """A newly initialised model of the same configuration (seeded: the comparison is against the seed's values)."""
    from kolmogorov_moe_architecture_b200 import MoETransformer
    torch.manual_seed(seed)
    return MoETransformer(config, verbose=False).to(device)


def analyze_parameter_movement(trained_model, fresh_model=None, device="cpu") -> dict:
    """Relative distance of every component of the trained model from a fresh initialisation (the given one, or
    one built from the model's own configuration and seed 0)."""
    if fresh_model is None:
        return parameter_movement(trained_model, trained_model.config)
    fresh = dict(fresh_model.named_parameters())
    out = {}
    for name, p in trained_model.named_parameters():
        q = fresh.get(name)
        if q is not None and q.shape == p.shape:
            key = ".".join(name.split(".")[:3])
            d = float((p.detach().float() - q.detach().float().to(p.device)).norm())
            n = float(q.detach().float().norm()) + 1e-12
            prev = out.get(key, (0.0, 0.0))
            out[key] = (prev[0] + d * d, prev[1] + n * n)
    return {k: (a ** 0.5) / (b ** 0.5) for k, (a, b) in out.items()}


def analyze_trainability(model) -> dict:
    return trainability(model)


def test_generation(model, config, device="cpu", prompt_len: int = 8, new_tokens: int = 12):
    """Greedy continuation of a random prompt; returns the token ids (no tokenizer is needed to see whether the
    model repeats one token or produces a spread)."""
    ids = torch.randint(0, config.vocab_size, (1, prompt_len), device=device)
    out = greedy_sample(model, ids, new_tokens)[0].tolist()
    print("[sample]", out, "- distinct new tokens:", len(set(out[prompt_len:])))
    return out


test_generation.__test__ = False          # a tool function, not a test case


def check_gradient_flow(model, config, device="cpu", batch: int = 2) -> dict:
    """One forward-backward pass on random tokens; gradient statistics per parameter group."""
    ids = torch.randint(0, config.vocab_size, (batch, min(64, config.max_seq_len)), device=device)
    return gradient_flow(model, ids)


if __name__ == "__main__":
    main()
