"""Parameter / memory calculator and configuration search (counterpart of the reference's
``tools/param_calculator.py``).

    python tools/param_calculator.py --config configs/training_4.5b.yaml
    python tools/param_calculator.py --d-model 1024 --n-layers 18 --n-experts 16 --top-k 2 [--all-moe]
    python tools/param_calculator.py --design --target-total 5 --target-active 1.5       # billions

``analyze`` gives exact totals by component (from an instantiated model on the meta device, so a
7B model costs no memory), the active-parameter count, and training-memory estimates for the
regimes this framework runs: replicated bf16 weights and gradients plus optimizer state sharded
over N ranks.  ``design`` brute-forces (d_model, n_layers, n_experts, d_ff_expert) grids for
configurations near a target total / active budget.
"""
import argparse
import itertools
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


def analyze(cfg, world: int = 8, micro_batch: int = 4, optimizer: str = "muon") -> dict:
    from kolmogorov_moe_architecture_b200 import MoETransformer
    with torch.device("meta"):
        m = MoETransformer(cfg, verbose=False)
    c = m.count_parameters()
    total = c["total"]
    w = g = 2 * total
    mats = sum(p.numel() for n, p in m.named_parameters() if p.dim() == 2 and "embed" not in n and "head" not in n)
    opt = (2 * mats + 8 * (total - mats)) if optimizer == "muon" else 8 * total
    tokens = micro_batch * cfg.max_seq_len
    act = tokens * cfg.d_model * 2 * 34 * cfg.n_layers
    return {"total": total, "active": c["active"], "sparsity": c["sparsity"], "analytic_estimate": cfg.count_parameters()["total"],
            "weights_gb": w / 2**30, "grads_gb": g / 2**30, "optimizer_gb_per_rank": opt / world / 2**30,
            "activations_gb_no_recompute": act / 2**30,
            "per_gpu_total_gb": (w + g + opt / world + act) / 2**30, "layers": c}


def format_params(n: float) -> str:
    for unit, div in (("B", 1e9), ("M", 1e6), ("K", 1e3)):
        if abs(n) >= div:
            return f"{n / div:.2f}{unit}"
    return str(int(n))


def breakdown(cfg) -> dict:
    """Exact parameter counts by kind of tensor (embedding, heads, attention, Mamba mixers, norms, dense FFN,
    routers, experts, MoD routers), counted on a meta-device instance so the categories follow the modules the
    model really builds (Mamba layers, RoutingMamba experts and MoD routers included)."""
    from kolmogorov_moe_architecture_b200 import MoETransformer
    with torch.device("meta"):
        m = MoETransformer(cfg, verbose=False)
    out = dict.fromkeys(("embedding", "lm_heads", "attention", "mamba", "norms", "dense_ffn", "router", "experts",
                         "mod_router"), 0)
    tied = set()
    for name, p in m.named_parameters():
        n = p.numel()
        if name.startswith("token_embedding"):
            out["embedding"] += n
        elif name.startswith("lm_heads"):
            out["lm_heads"] += n
        elif "norm" in name.split(".")[-2] or name.startswith("final_norm"):
            out["norms"] += n
        elif "mod_router" in name:
            out["mod_router"] += n
        elif ".seq_layer." in name:
            mixer = name.split(".seq_layer.")[1]
            if mixer.split(".")[0] in ("q_proj", "k_proj", "v_proj", "o_proj"):
                out["attention"] += n
            elif mixer.startswith("router"):
                out["router"] += n
            else:
                out["mamba"] += n
        elif ".ffn." in name:
            tail = name.split(".ffn.")[1]
            if "router" in tail:
                out["router"] += n
            elif "experts" in tail:
                out["experts"] += n
            else:
                out["dense_ffn"] += n
        else:
            out.setdefault("other", 0)
            out["other"] += n
    out["total"] = sum(v for k, v in out.items() if k != "total")
    return out


def print_report(cfg, world=8, micro_batch: int = 4, optimizer: str = "muon") -> dict:
    """Report of a model configuration (``print_report(cfg, world)``), or - in the reference's call form
    ``print_report(params, model_params)`` - of a ``calculate_params`` result for a ``ModelParams``."""
    if isinstance(cfg, dict) and isinstance(world, ModelParams):
        params, mp = cfg, world
        print("=" * 64)
        print(f"  vocab {mp.vocab_size:,}  d_model {mp.d_model}  layers {mp.n_layers} "
              f"({params['n_moe_layers']} MoE, {params['n_dense_layers']} dense)  experts {mp.n_experts} x "
              f"d_ff {mp.d_ff_expert}, top-{mp.moe_top_k}")
        for k in ("embedding_params", "lm_head_params", "attention_params", "norm_params", "dense_ffn_params",
                  "router_params", "expert_params"):
            print(f"  {k[:-7]:12s} {format_params(params[k]):>10s}  {100 * params[k] / max(params['total_params'], 1):5.1f} %")
        print(f"  {'total':12s} {format_params(params['total_params']):>10s}")
        print(f"  {'active':12s} {format_params(params['active_params']):>10s}  sparsity {100 * params['sparsity']:.1f} %")
        print("=" * 64)
        return params
    r, b = analyze(cfg, world, micro_batch, optimizer), breakdown(cfg)
    n_moe = len([i for i in range(cfg.n_layers) if i in set(cfg.moe_layers)]) if cfg.moe_layers is not None else cfg.n_layers
    print("=" * 64)
    print("configuration")
    print(f"  vocab {cfg.vocab_size:,}  d_model {cfg.d_model}  layers {cfg.n_layers} ({n_moe} MoE, {len(cfg.mamba_layers or ())} Mamba)")
    print(f"  heads {cfg.n_heads} / kv {cfg.n_kv_heads} x {cfg.head_dim}  d_ff {cfg.d_ff}  experts {cfg.n_experts} x d_ff {cfg.d_ff_expert}, top-{cfg.moe_top_k}")
    print("parameters by kind")
    for k in ("embedding", "lm_heads", "attention", "mamba", "norms", "dense_ffn", "router", "experts", "mod_router"):
        print(f"  {k:12s} {format_params(b[k]):>10s}  {100 * b[k] / max(b['total'], 1):5.1f} %")
    print(f"  {'total':12s} {format_params(r['total']):>10s}  ({r['total']:,}; tied head counted once)")
    print(f"  {'active':12s} {format_params(r['active']):>10s}  sparsity {100 * r['sparsity']:.1f} %")
    print(f"memory per GPU, bf16 weights and gradients replicated, optimizer state over {world} ranks ({optimizer})")
    print(f"  weights {r['weights_gb']:.2f} GB  gradients {r['grads_gb']:.2f} GB  optimizer {r['optimizer_gb_per_rank']:.2f} GB"
          f"  activations (no recompute, micro-batch {micro_batch}) {r['activations_gb_no_recompute']:.2f} GB")
    print(f"  total {r['per_gpu_total_gb']:.2f} GB of 180 GB")
    print("=" * 64)
    return {"analysis": r, "breakdown": b}


def design(target_total: float, target_active: float, tol: float = 0.1, limit: int = 10):
    from kolmogorov_moe_architecture_b200 import AdvancedMoEConfig
    out = []
    for d, L, E, ratio in itertools.product((1024, 1536, 2048, 2560, 3072), (16, 24, 32, 40), (8, 16, 32, 64),
                                            (1.0, 1.375, 2.0)):
        H = d // 128
        if H < 2:
            continue
        cfg = AdvancedMoEConfig(d_model=d, n_layers=L, n_heads=H, n_kv_heads=max(1, H // 4), head_dim=128,
                                d_ff=int(2.75 * d), d_ff_expert=int(ratio * d) // 64 * 64, n_experts=E,
                                moe_layers=tuple(i for i in range(L) if i % 4 in (2, 3)),
                                mamba_layers=tuple(i for i in range(L) if i % 4 == 1 and i >= 5))
        est = cfg.count_parameters()["total"]
        moe = len(cfg.moe_layers) * E * 3 * d * cfg.d_ff_expert
        active = est - moe * (1 - cfg.moe_top_k / E)
        if abs(est - target_total) / target_total < tol and abs(active - target_active) / target_active < tol:
            out.append({"d_model": d, "n_layers": L, "n_experts": E, "d_ff_expert": cfg.d_ff_expert,
                        "total_b": est / 1e9, "active_b": active / 1e9})
    return sorted(out, key=lambda r: abs(r["total_b"] * 1e9 - target_total))[:limit]


# ---- the reference's plain attention + MoE calculator (tools/param_calculator.py:19-236), for code that imports it
from dataclasses import dataclass                                             # noqa: E402
from typing import List, Optional                                             # noqa: E402


@dataclass
class ModelParams:
    """Sizes of an attention + SwiGLU / MoE transformer without Mamba, mixture-of-depths or extra heads."""
    vocab_size: int = 32000
    d_model: int = 1024
    n_layers: int = 18
    n_heads: int = 8
    n_kv_heads: int = 4
    head_dim: int = 128
    d_ff: int = 4096
    d_ff_expert: int = 2048
    n_experts: int = 16
    moe_top_k: int = 2
    moe_layers: Optional[List[int]] = None          # None = every layer
    tie_embeddings: bool = False


def calculate_params(cfg: ModelParams) -> dict:
    """Analytic totals of a ``ModelParams`` model: q/k/v/o projections, two norms per layer and a final one, a
    three-matrix SwiGLU in the dense layers, a d -> 128 -> E router MLP and E three-matrix experts in the MoE
    layers.  Active = everything but the experts, plus ``moe_top_k / n_experts`` of the experts.  (The reference's
    function counts one d x E matrix per router; its models, like the ones here, have the two-matrix router, so
    this count equals what an instantiated model holds - router_params and the totals differ from the
    reference's by that amount.)"""
    L, d = cfg.n_layers, cfg.d_model
    moe = set(range(L)) if cfg.moe_layers is None else set(cfg.moe_layers)
    n_moe, n_dense = len(moe), L - len(moe)
    emb = cfg.vocab_size * d
    head = 0 if cfg.tie_embeddings else cfg.vocab_size * d
    attn = 2 * d * cfg.n_heads * cfg.head_dim + 2 * d * cfg.n_kv_heads * cfg.head_dim
    norms = 2 * d * L + d
    dense = 3 * d * cfg.d_ff * n_dense
    router = (d * 128 + 128 * cfg.n_experts) * n_moe
    per_expert = 3 * d * cfg.d_ff_expert
    experts = per_expert * cfg.n_experts * n_moe
    total = emb + head + attn * L + norms + dense + router + experts
    active = total - experts + experts * cfg.moe_top_k / max(cfg.n_experts, 1)
    return {"total_params": total, "active_params": active, "sparsity": 1.0 - active / total if total else 0.0,
            "embedding_params": emb, "lm_head_params": head, "attention_params": attn * L, "norm_params": norms,
            "dense_ffn_params": dense, "router_params": router, "expert_params": experts,
            "attention_per_layer": attn, "expert_ffn_per_expert": per_expert,
            "experts_per_layer": per_expert * cfg.n_experts, "n_moe_layers": n_moe, "n_dense_layers": n_dense,
            "moe_top_k": cfg.moe_top_k, "n_experts": cfg.n_experts}


def load_config(path: str) -> ModelParams:
    """``ModelParams`` from the ``model:`` section of a YAML file (the reference's defaults for missing keys)."""
    from kolmogorov_moe_architecture_b200.utils.config_io import load_yaml
    m = load_yaml(path).get("model") or {}
    d = ModelParams()
    return ModelParams(**{k: m.get(k, getattr(d, k)) for k in d.__dataclass_fields__})


def design_model(target_total: float, target_active: float, vocab_size: int = 32000) -> Optional[ModelParams]:
    """Grid search over (d_model, n_layers, n_experts, expert width) for the plain MoE model closest to the targets
    (in billions of parameters); None when nothing comes within 15 %."""
    best, best_err = None, 0.15
    for d, L, E, f in itertools.product((512, 768, 1024, 1536, 2048, 2560, 3072, 4096), (8, 12, 16, 18, 24, 32, 40),
                                        (8, 16, 32, 64), (512, 1024, 1536, 2048, 2816, 4096)):
        cfg = ModelParams(vocab_size=vocab_size, d_model=d, n_layers=L, n_heads=max(d // 128, 1),
                          n_kv_heads=max(d // 512, 1), head_dim=128, d_ff=4 * d, d_ff_expert=f, n_experts=E)
        r = calculate_params(cfg)
        err = max(abs(r["total_params"] / 1e9 - target_total) / target_total,
                  abs(r["active_params"] / 1e9 - target_active) / target_active)
        if err < best_err:
            best, best_err = cfg, err
    if best is not None:
        r = calculate_params(best)
        print(f"closest: {best}  total {format_params(r['total_params'])}  active {format_params(r['active_params'])}")
    else:
        print("no configuration within 15 % of the targets")
    return best


def config_from_flags(a):
    """The model the manual options describe (reference: tools/param_calculator.py:343-358): attention and experts
    in every layer, no Mamba, no mixture-of-depths.  In the reference a manual configuration has experts in all
    layers with or without ``--all-moe`` (its layer list defaults to "all"); the flag is accepted and means the same
    here."""
    from kolmogorov_moe_architecture_b200 import AdvancedMoEConfig
    L = a.n_layers
    moe = tuple(range(L))
    return AdvancedMoEConfig(vocab_size=a.vocab_size, d_model=a.d_model, n_layers=L, n_heads=a.n_heads,
                             n_kv_heads=a.n_kv_heads, head_dim=a.head_dim, d_ff=a.d_ff, d_ff_expert=a.d_ff_expert,
                             n_experts=a.n_experts, moe_top_k=a.top_k, moe_layers=moe, mamba_enabled=False,
                             mamba_layers=(), mod_enabled=False)


def main(argv=None):
    ap = argparse.ArgumentParser(description="parameter and memory report of a model configuration")
    ap.add_argument("--config", default=None, help="YAML configuration")
    ap.add_argument("--world", type=int, default=8)
    manual = ap.add_argument_group("manual configuration (used when any of them is given and --config is not)")
    manual.add_argument("--vocab-size", type=int, default=None)
    manual.add_argument("--d-model", type=int, default=None)
    manual.add_argument("--n-layers", type=int, default=None)
    manual.add_argument("--n-heads", type=int, default=None)
    manual.add_argument("--n-kv-heads", type=int, default=None)
    manual.add_argument("--head-dim", type=int, default=None)
    manual.add_argument("--d-ff", type=int, default=None)
    manual.add_argument("--d-ff-expert", type=int, default=None)
    manual.add_argument("--n-experts", type=int, default=None)
    manual.add_argument("--top-k", type=int, default=None)
    manual.add_argument("--all-moe", action="store_true", help="experts in every layer (already the rule for a manual configuration)")
    ap.add_argument("--design", action="store_true", help="search configurations near the targets")
    ap.add_argument("--target-total", type=float, default=5.0,
                    help="total parameters, in billions (values above 1000 are taken as a plain count)")
    ap.add_argument("--target-active", type=float, default=1.5, help="active parameters, same unit")
    a = ap.parse_args(argv)
    if a.design:
        to_count = lambda v: v if v > 1000 else v * 1e9
        found = design(to_count(a.target_total), to_count(a.target_active))
        for r in found:
            print(r)
        return found
    from kolmogorov_moe_architecture_b200 import AdvancedMoEConfig
    from kolmogorov_moe_architecture_b200.utils.config_io import load_yaml, model_config_tolerant
    defaults = dict(vocab_size=32000, d_model=1024, n_layers=18, n_heads=8, n_kv_heads=4, head_dim=128, d_ff=4096,
                    d_ff_expert=2048, n_experts=16, top_k=2)                 # the reference's manual defaults
    given = a.all_moe or any(getattr(a, k) is not None for k in defaults)
    if a.config:
        cfg = model_config_tolerant(load_yaml(a.config))
    elif given:
        for k, v in defaults.items():
            if getattr(a, k) is None:
                setattr(a, k, v)
        cfg = config_from_flags(a)
    else:
        cfg = AdvancedMoEConfig()
    return print_report(cfg, a.world)


if __name__ == "__main__":
    main()
