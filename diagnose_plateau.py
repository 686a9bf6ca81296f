"""Loss-plateau diagnosis (counterpart of the reference's ``diagnose_plateau.py``): hooks every
router, collects selection statistics during a few forward passes, reports gradient statistics
and lints the configuration.

    python diagnose_plateau.py --config cfg.yaml [--checkpoint ckpt.pt] [--device cpu]
"""
import argparse
import os
import sys
from collections import defaultdict

import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


class RouterAnalyzer:
    """Forward hooks on every module named ``router`` recording per-expert selection counts and the
    mean max-probability of the routing distribution."""

    def __init__(self, model):
        self.stats = defaultdict(lambda: {"calls": 0, "counts": None, "max_prob": 0.0})
        self.handles = []
        for name, mod in model.named_modules():
            if name.endswith("ffn.router") or name.endswith("seq_layer.router"):
                self.handles.append(mod.register_forward_hook(self._hook(name)))

    def _hook(self, name):
        def fn(mod, inp, out):
            s = self.stats[name]
            s["calls"] += 1
            if isinstance(out, tuple) and len(out) == 3:
                w, idx, logits = out
                E = logits.shape[-1]
                c = torch.bincount(idx.flatten(), minlength=E).float().cpu()
                s["counts"] = c if s["counts"] is None else s["counts"] + c
                s["max_prob"] += float(torch.softmax(logits.detach().float(), -1).max(-1).values.mean())
        return fn

    def report(self):
        out = {}
        for n, s in self.stats.items():
            if s["counts"] is None:
                continue
            u = s["counts"] / s["counts"].sum().clamp(min=1)
            ent = float(-(u * torch.log(u + 1e-10)).sum() / torch.log(torch.tensor(float(len(u)))))
            out[n] = {"entropy": ent, "max_usage": float(u.max()), "dead_experts": int((u == 0).sum()),
                      "mean_max_prob": s["max_prob"] / max(s["calls"], 1)}
        return out

    def close(self):
        for h in self.handles:
            h.remove()


def lint_config(cfg) -> list:
    notes = []
    if cfg.mod_enabled and cfg.mod_capacity_factor < 0.5:
        notes.append("mod_capacity_factor < 0.5: more than half of the tokens skip every FFN")
    if cfg.moe_load_balance_loss_weight == 0 and cfg.moe_routing == "token_choice":
        notes.append("no load-balance loss with token-choice routing: routers can collapse")
    if cfg.n_pred_tokens > 1 and abs(sum(cfg.aux_loss_weights) - 1.0) > 1e-6:
        notes.append("aux_loss_weights do not sum to 1 (they are normalised internally)")
    if cfg.dropout > 0.2:
        notes.append("dropout > 0.2")
    return notes


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default="configs/production_training.yaml")
    ap.add_argument("--checkpoint", default=None)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--batches", type=int, default=4)
    ap.add_argument("--batch-size", type=int, default=1)
    ap.add_argument("--seq-len", type=int, default=512)
    a = ap.parse_args(argv)
    from eval.evaluate_perplexity import load_model
    from kolmogorov_moe_architecture_b200.utils.fault import gradient_census
    model, cfg = load_model(a.checkpoint, a.config, a.device, dtype=torch.float32 if a.device == "cpu" else torch.bfloat16)
    an = RouterAnalyzer(model)
    model.train()
    for _ in range(a.batches):
        ids = torch.randint(0, cfg.vocab_size, (a.batch_size, min(a.seq_len, cfg.max_seq_len)), device=a.device)
        model.zero_grad(set_to_none=True)
        model(ids, labels=ids, return_logits=False)["loss"].backward()
    rep = an.report()
    an.close()
    for n, s in rep.items():
        print(f"{n}: {s}")
    for k, v in gradient_census(model).items():
        print(f"grad[{k}]: {v}")
    for note in lint_config(cfg):
        print("config:", note)
    return rep


# ---- names of the reference's script, for code that imports them from here
def load_config(path=None, config_path=None):
    """The YAML file as a dict."""
    from kolmogorov_moe_architecture_b200.utils.config_io import load_yaml
    return load_yaml(config_path if path is None else path)


def create_model_from_config(config_dict):
    """(model, model configuration) from a configuration dict (its ``model:`` section, read with defaults)."""
    from kolmogorov_moe_architecture_b200 import MoETransformer
    from kolmogorov_moe_architecture_b200.utils.config_io import model_config_tolerant
    cfg = model_config_tolerant(config_dict)
    return MoETransformer(cfg, verbose=False), cfg


def analyze_gradients(model):
    """Gradient statistics per parameter group after a backward pass."""
    from kolmogorov_moe_architecture_b200.utils.fault import gradient_census
    return gradient_census(model)


RouterAnalyzer.register_hooks = lambda self, model=None, n_experts=None: self    # registered by the constructor
RouterAnalyzer.remove_hooks = RouterAnalyzer.close
RouterAnalyzer.get_stats = RouterAnalyzer.report


if __name__ == "__main__":
    main()
