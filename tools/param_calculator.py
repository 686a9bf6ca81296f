"""Parameter / memory calculator and configuration search (counterpart of the reference's
``tools/param_calculator.py``).

    python tools/param_calculator.py --config configs/training_4.5b.yaml
    python tools/param_calculator.py --design --target-total 5e9 --target-active 1.5e9

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


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", default=None)
    ap.add_argument("--world", type=int, default=8)
    ap.add_argument("--design", action="store_true")
    ap.add_argument("--target-total", type=float, default=5e9)
    ap.add_argument("--target-active", type=float, default=1.5e9)
    a = ap.parse_args()
    if a.design:
        for r in design(a.target_total, a.target_active):
            print(r)
    else:
        from kolmogorov_moe_architecture_b200 import AdvancedMoEConfig
        from kolmogorov_moe_architecture_b200.utils.config_io import load_yaml, model_config_tolerant
        cfg = model_config_tolerant(load_yaml(a.config)) if a.config else AdvancedMoEConfig()
        r = analyze(cfg, a.world)
        for k, v in r.items():
            if k != "layers":
                print(f"{k:32s} {v:,.3f}" if isinstance(v, float) else f"{k:32s} {v:,}")
