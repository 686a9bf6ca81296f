"""Active-parameter breakdown of a preset or YAML configuration (counterpart of the reference's
``analyze_active_params.py``).

    python analyze_active_params.py [--preset 3b|5b|test|bench] [--config cfg.yaml]
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--preset", default="3b", choices=["3b", "5b", "test", "bench"])
    ap.add_argument("--config", default=None)
    a = ap.parse_args(argv)
    import kolmogorov_moe_architecture_b200 as kmoe
    if a.config:
        from kolmogorov_moe_architecture_b200.utils.config_io import load_yaml, model_config_tolerant
        cfg = model_config_tolerant(load_yaml(a.config))
    else:
        cfg = {"3b": kmoe.get_3b_config, "5b": kmoe.get_5b_config, "test": kmoe.get_test_config,
               "bench": kmoe.get_bench_5b_config}[a.preset]()
    return analyze_config(cfg, a.config or a.preset)


def analyze_config(config, name: str = ""):
    """Totals, active parameters and the per-layer-kind breakdown of one configuration (counted on a meta-device
    instance); prints the report and returns the counts."""
    cfg = config
    import kolmogorov_moe_architecture_b200 as kmoe
    if name:
        print(f"== {name}")
    with torch.device("meta"):
        m = kmoe.MoETransformer(cfg, verbose=False)
    c = m.count_parameters()
    print(f"total {c['total'] / 1e9:.3f}B | active {c['active'] / 1e9:.3f}B | sparsity {c['sparsity']:.1%}")
    print(f"layers: {c['n_attention_layers']} attention, {c['n_mamba_layers']} mamba, {c['n_moe_layers']} listed as MoE")
    rows = {}
    for i, layer in enumerate(m.layers):
        rows.setdefault((layer.mixer_kind, layer.ffn_kind), []).append(sum(p.numel() for p in layer.parameters()))
    for k, v in rows.items():
        print(f"  {k[0]:14s} + {k[1]:5s} x{len(v):2d}: {v[0] / 1e6:8.1f}M each")
    print(f"  MoD compute: {cfg.mod_capacity_factor:.0%} of tokens reach each FFN" if cfg.mod_enabled else "  MoD off")
    return c


if __name__ == "__main__":
    main()
