"""Router-health analysis and expert reallocation (counterpart of the reference's
``tools/reallocate_experts.py``).

    python tools/reallocate_experts.py --checkpoint ckpt.pt --config cfg.yaml --output new.pt

``analyze_router_entropy`` runs random token sequences through the model and records, per MoE
layer, the normalised entropy of the mean router distribution, the Gini coefficient of expert
usage and the most / least used experts; a layer is collapsed when one expert takes more than
3/E of the assignments, Gini > 0.5 or entropy < 0.7.  ``reallocate_model_experts`` copies the
expert stacks (``w1``, ``w2``, ``w3``) of the healthiest layer into every collapsed layer and
re-initialises the routers of all MoE layers.  (The reference's copy looks for
``gate_proj/up_proj/down_proj`` keys, which its model does not have, so it never copies anything
- reference: tools/reallocate_experts.py:271-278; here the stacked tensors are copied.)
"""
import argparse
import os
import sys
from typing import Dict, Tuple

import torch
import torch.nn.functional as F

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def _gini(x: torch.Tensor) -> float:
    s, _ = torch.sort(x.float())
    n = s.numel()
    tot = s.sum()
    if tot <= 0:
        return 0.0
    idx = torch.arange(1, n + 1, dtype=torch.float32)
    return float((2 * (idx * s).sum() - (n + 1) * tot) / (n * tot))


@torch.no_grad()
def analyze_router_entropy(model, n_samples: int = 50, seq_len: int = 256, device=None,
                           generator=None) -> Tuple[Dict, int, int]:
    base = getattr(model, "_orig_mod", model)
    if device is not None:
        base.to(device)
    was_training = base.training
    base.eval()
    dev = next(base.parameters()).device
    V = base.token_embedding.embedding.weight.shape[0]
    counts: Dict[int, torch.Tensor] = {}
    probs: Dict[int, torch.Tensor] = {}
    E = k = 1
    for _ in range(n_samples):
        ids = torch.randint(0, V, (1, min(seq_len, base.config.max_seq_len)), generator=generator).to(dev)
        h = base.token_embedding(ids)
        for i, layer in enumerate(base.layers):
            ffn = layer.ffn
            if getattr(layer, "ffn_kind", None) == "moe" and getattr(ffn, "router", None) is not None \
                    and getattr(ffn, "routing_type", "token_choice") == "token_choice":
                E, k = ffn.n_experts, ffn.top_k
                _, sel, logits = ffn.router(layer.ffn_norm(h))
                counts[i] = counts.get(i, torch.zeros(E, device=dev)) + torch.bincount(sel.flatten(), minlength=E)
                probs[i] = probs.get(i, torch.zeros(E, device=dev)) + F.softmax(logits.float(), -1).mean((0, 1))
            h = layer(h)
    out = {}
    for i in sorted(counts):
        p = probs[i] / n_samples
        ent = float(-(p * torch.log(p + 1e-10)).sum()) / (torch.log(torch.tensor(float(E))).item() if E > 1 else 1.0)
        usage = counts[i] / counts[i].sum().clamp(min=1)
        g = _gini(counts[i].cpu())
        order = torch.argsort(counts[i], descending=True).tolist()
        out[i] = {"entropy": ent, "gini": g, "expert_usage": usage.cpu(), "most_used": order[:3],
                  "least_used": order[-3:], "probs": p.cpu(),
                  "is_collapsed": bool(usage.max() > 3.0 / E or g > 0.5 or ent < 0.7)}
    if was_training:
        base.train()
    return out, E, k


@torch.no_grad()
def reallocate_model_experts(model, entropy_threshold: float = 0.85, n_samples: int = 20, verbose: bool = True):
    base = getattr(model, "_orig_mod", model)
    stats, E, k = analyze_router_entropy(base, n_samples=n_samples, seq_len=128)
    if not stats:
        return {"collapsed": [], "healthy": [], "source": None}
    healthy = [i for i, s in stats.items() if not s["is_collapsed"] and s["entropy"] >= entropy_threshold]
    collapsed = [i for i, s in stats.items() if s["is_collapsed"]]
    source = max(healthy, key=lambda i: stats[i]["entropy"]) if healthy else None
    if source is not None:
        src = base.layers[source].ffn.grouped_experts
        for i in collapsed:
            dst = base.layers[i].ffn.grouped_experts
            for name in ("w1", "w2", "w3"):
                s_, d_ = getattr(src, name, None), getattr(dst, name, None)
                if s_ is not None and d_ is not None and s_.shape == d_.shape:
                    d_.copy_(s_)
    for i in stats:
        for m in base.layers[i].ffn.router.modules():
            if isinstance(m, torch.nn.Linear):
                torch.nn.init.normal_(m.weight, mean=0.0, std=base.config.init_std)
    if verbose:
        print(f"reallocation: collapsed layers {collapsed}, healthy {healthy}, source {source}; routers reset")
    return {"collapsed": collapsed, "healthy": healthy, "source": source, "stats": stats}


def reallocate_experts(checkpoint_path: str, config_path: str, output_path: str, device: str = "cpu",
                       entropy_threshold: float = 0.85):
    from eval.evaluate_perplexity import load_model
    model, _ = load_model(checkpoint_path, config_path, device, dtype=torch.float32)
    info = reallocate_model_experts(model, entropy_threshold)
    ck = torch.load(checkpoint_path, map_location="cpu", weights_only=False) if checkpoint_path else {}
    ck = ck if isinstance(ck, dict) else {}
    ck.update({"model_state_dict": model.state_dict(), "reallocated_from": checkpoint_path,
               "reallocated_collapsed_layers": info["collapsed"], "reallocated_healthy_layers": info["healthy"]})
    ck.pop("optimizer_state_dict", None)
    torch.save(ck, output_path)
    return info


def create_model_config(config_dict):
    """``AdvancedMoEConfig`` from a YAML dict (its ``model:`` section, read with the tolerant loader's defaults)."""
    from kolmogorov_moe_architecture_b200.utils.config_io import model_config_tolerant
    return model_config_tolerant(config_dict)


def main(argv=None):
    ap = argparse.ArgumentParser(description="copy experts from healthy to collapsed layers, reset the routers")
    ap.add_argument("--checkpoint", required=True)
    ap.add_argument("--config", required=True)
    ap.add_argument("--output", required=True)
    ap.add_argument("--device", default=None, help="default: cuda:<--gpu> when a GPU is present, else cpu")
    ap.add_argument("--gpu", type=int, default=0, help="GPU index (the reference's way of naming the device)")
    ap.add_argument("--entropy-threshold", type=float, default=0.85)
    a = ap.parse_args(argv)
    if a.device is None:
        a.device = f"cuda:{a.gpu}" if torch.cuda.is_available() else "cpu"
    return reallocate_experts(a.checkpoint, a.config, a.output, a.device, a.entropy_threshold)


if __name__ == "__main__":
    main()
