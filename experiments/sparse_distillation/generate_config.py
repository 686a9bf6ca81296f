"""Per-layer MoE configuration from cluster analysis (counterpart of the reference's
``Experiments/sparse_distillation/generate_config.py``): for every FFN layer pick the number of
experts whose k-means clustering of the layer's outputs scores best, then size the experts so
that total width = ``expansion`` x dense width and active width = ``active_ratio`` x dense width.

    python -m experiments.sparse_distillation.generate_config --analysis cluster_analysis.json --output layers.json
"""
from __future__ import annotations

import argparse
import json
from typing import Dict


def choose_layer_config(quality: Dict[str, Dict[str, float]], d_ff_dense: int, expansion: float = 2.0,
                        active_ratio: float = 0.25) -> Dict[str, int]:
    """quality: {k: {silhouette, calinski_harabasz, balance}}.  Score = silhouette x balance."""
    best_k = max(quality, key=lambda k: quality[k].get("silhouette", 0.0) * quality[k].get("balance", 0.0))
    E = int(best_k)
    d_ff_e = max(64, int(d_ff_dense * expansion / E) // 64 * 64)
    top_k = max(1, min(E, round(d_ff_dense * active_ratio / d_ff_e)))
    return {"n_experts": E, "d_ff_expert": d_ff_e, "top_k": top_k}


def generate(analysis: Dict[str, Dict], d_ff_dense: int, expansion: float = 2.0, active_ratio: float = 0.25):
    return {layer: choose_layer_config(q, d_ff_dense, expansion, active_ratio) for layer, q in analysis.items()}


if __name__ == "__main__":
    ap = argparse.ArgumentParser()
    ap.add_argument("--analysis", required=True)
    ap.add_argument("--output", required=True)
    ap.add_argument("--d-ff-dense", type=int, required=True)
    ap.add_argument("--expansion", type=float, default=2.0)
    ap.add_argument("--active-ratio", type=float, default=0.25)
    a = ap.parse_args()
    cfg = generate(json.load(open(a.analysis)), a.d_ff_dense, a.expansion, a.active_ratio)
    json.dump(cfg, open(a.output, "w"), indent=2)
    print(json.dumps(cfg, indent=2))
