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
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--synthetic", action="store_true")
    a = ap.parse_args(argv)
    from eval.evaluate_perplexity import load_model
    from kolmogorov_moe_architecture_b200.utils.fault import check_router_collapse
    model, cfg = load_model(a.checkpoint, a.config, a.device, dtype=torch.float32 if a.device == "cpu" else torch.bfloat16)
    stats, collapsed, summary = check_router_collapse(model)
    print("[router]", summary)
    for i, s in stats.items():
        print(f"  layer {i}: entropy {s['entropy']:.3f} max_usage {s['max_usage']:.3f}")
    mv = parameter_movement(model, cfg)
    print("[movement] least moved:", sorted(mv.items(), key=lambda kv: kv[1])[:5])
    tr = trainability(model)
    print(f"[trainable] {tr['trainable']:,} of {tr['total']:,}; frozen tensors: {len(tr['frozen_tensors'])}")
    ids = torch.randint(0, cfg.vocab_size, (2, min(64, cfg.max_seq_len)), device=a.device)
    for k, v in gradient_flow(model, ids).items():
        print(f"[grad] {k}: {v}")
    print("[sample]", greedy_sample(model, ids[:1, :8], 12)[0].tolist())
    return {"router": stats, "collapsed": collapsed, "movement": mv, "trainability": tr}


if __name__ == "__main__":
    main()
