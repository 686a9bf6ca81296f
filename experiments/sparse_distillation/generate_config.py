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


def compute_layer_config(analysis: Dict, target_expansion_ratio: float = 3.0, target_active_ratio: float = 0.25,
                         min_experts: int = 4, min_top_k: int = 1, max_top_k: int = 8, verbose: bool = True) -> Dict:
    """Per-layer ``n_experts / d_ff_expert / top_k`` at fixed ratios, from a cluster analysis of the form
    ``{"d_model", "d_ff", "layers": {i: {"n_experts", "balance", "silhouette"?, "all_results"?: {k: {...}}}}}``
    (reference: Experiments/sparse_distillation/generate_config.py:24-166).

    expansion = n_experts * d_ff_expert / d_ff_dense, active = top_k * d_ff_expert / d_ff_dense.  A layer whose
    best cluster count is below ``min_experts`` takes the best-balanced count >= ``min_experts`` it was
    analysed for, else ``min_experts``.  Expert widths are multiples of 64."""
    d_model, d_ff = analysis["d_model"], analysis["d_ff"]
    layers: Dict[str, Dict] = {}
    for key, ld in sorted(analysis["layers"].items(), key=lambda kv: int(kv[0])):
        E, bal = int(ld["n_experts"]), float(ld.get("balance", 0.0))
        if E < min_experts:
            alts = {int(k): v for k, v in ld.get("all_results", {}).items() if int(k) >= min_experts}
            if alts:
                E = max(alts, key=lambda k: alts[k].get("balance", 0.0))
                bal = float(alts[E].get("balance", 0.0))
            else:
                E = min_experts
        f = max(64, int(target_expansion_ratio * d_ff / E) // 64 * 64)
        k = min(E, max(min_top_k, min(max_top_k, int(round(target_active_ratio * d_ff / f)))))
        layers[str(key)] = {"n_experts": E, "d_ff_expert": f, "top_k": k, "balance": bal,
                            "silhouette": float(ld.get("silhouette", 0.0))}
    dense = len(layers) * 3 * d_model * d_ff
    moe = sum(c["n_experts"] * 3 * d_model * c["d_ff_expert"] for c in layers.values())
    act = sum(c["top_k"] * 3 * d_model * c["d_ff_expert"] for c in layers.values())
    stats = {"total_moe_params": moe, "total_dense_params": dense, "actual_expansion_ratio": moe / max(dense, 1),
             "total_active_params": act, "actual_active_ratio": act / max(dense, 1)}
    if verbose:
        print(f"{'layer':>6} | {'n_experts':>9} | {'d_ff_expert':>11} | {'top_k':>5} | {'active d_ff':>11} | balance")
        for key, c in layers.items():
            print(f"{key:>6} | {c['n_experts']:>9} | {c['d_ff_expert']:>11} | {c['top_k']:>5} | "
                  f"{c['top_k'] * c['d_ff_expert']:>11} | {c['balance']:.4f}")
        print(f"expansion {stats['actual_expansion_ratio']:.3f}x (target {target_expansion_ratio}), "
              f"active {stats['actual_active_ratio']:.3f}x (target {target_active_ratio}), "
              f"MoE FFN parameters {moe / 1e9:.3f} B against {dense / 1e9:.3f} B dense")
    return {"d_model": d_model, "d_ff_dense": d_ff, "target_expansion_ratio": target_expansion_ratio,
            "target_active_ratio": target_active_ratio, "min_experts": min_experts, "layers": layers, "stats": stats}


def main(argv=None):
    """``python -m experiments.sparse_distillation.generate_config out/cluster_analysis.json [--expansion_ratio 3]
    [--active_ratio 0.25] [--min_experts 4] [--min_top_k 1] [--max_top_k 8] [--output out/layer_config.json]``
    (the reference's arguments; the output defaults to ``layer_config.json`` beside the analysis)."""
    ap = argparse.ArgumentParser(description="per-layer MoE configuration from a cluster analysis")
    ap.add_argument("analysis_path", nargs="?", default=None, help="cluster_analysis.json of example_usage --analyze_clusters")
    ap.add_argument("--analysis", default=None, help="the same, as an option")
    ap.add_argument("--output", default=None)
    ap.add_argument("--d-ff-dense", "--d_ff_dense", dest="d_ff_dense", type=int, default=None,
                    help="needed for an analysis of the form {layer: {k: quality}}; a file with d_model / d_ff / layers brings its own")
    ap.add_argument("--expansion_ratio", "--expansion", dest="expansion", type=float, default=None,
                    help="target n_experts * d_ff_expert / d_ff_dense (default 3.0)")
    ap.add_argument("--active_ratio", "--active-ratio", dest="active_ratio", type=float, default=0.25,
                    help="target top_k * d_ff_expert / d_ff_dense")
    ap.add_argument("--min_experts", "--min-experts", dest="min_experts", type=int, default=4)
    ap.add_argument("--min_top_k", "--min-top-k", dest="min_top_k", type=int, default=1)
    ap.add_argument("--max_top_k", "--max-top-k", dest="max_top_k", type=int, default=8)
    a = ap.parse_args(argv)
    path = a.analysis_path or a.analysis
    if path is None:
        ap.error("the analysis file is required")
    out = a.output or (path.replace("cluster_analysis.json", "layer_config.json") if path.endswith("cluster_analysis.json")
                       else path + ".layer_config.json")
    data = json.load(open(path))
    if "layers" in data and "d_ff" in data:
        cfg = compute_layer_config(data, a.expansion or 3.0, a.active_ratio, a.min_experts, a.min_top_k, a.max_top_k)
    else:
        assert a.d_ff_dense, "--d-ff-dense is required for this analysis format"
        cfg = generate(data, a.d_ff_dense, a.expansion or 2.0, a.active_ratio)
        print(json.dumps(cfg, indent=2))
    json.dump(cfg, open(out, "w"), indent=2)
    print(f"saved {out}")
    return cfg


if __name__ == "__main__":
    main()
