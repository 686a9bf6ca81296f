"""End-to-end sparse distillation (counterpart of the reference's
``Experiments/sparse_distillation/example_usage.py``):

    python -m experiments.sparse_distillation.example_usage --model <hf name or 'toy'> \
        [--analyze_clusters] [--n_experts 8] [--steps 200] [--output_dir out/]

load model -> (optional cluster analysis -> cluster_analysis.json) -> distill -> evaluate -> save ->
convert_to_sparse -> routing statistics.  ``--model toy`` builds a small random transformer so the
pipeline runs without network access.
"""
from __future__ import annotations

import argparse
import json
import os

import torch
import torch.nn as nn

from .convert import convert_to_sparse
from .distill import DistillationConfig, SparseDistillationTrainer
from .finetune_eval import accumulate_routing_stats


class ToyBlock(nn.Module):
    def __init__(self, d, f):
        super().__init__()
        self.norm = nn.LayerNorm(d)
        self.mlp = nn.Module()
        self.mlp.gate_proj, self.mlp.up_proj, self.mlp.down_proj = nn.Linear(d, f, bias=False), nn.Linear(d, f, bias=False), nn.Linear(f, d, bias=False)
        self.mlp.forward = lambda x, m=self.mlp: m.down_proj(torch.nn.functional.silu(m.gate_proj(x)) * m.up_proj(x))

    def forward(self, x):
        return x + self.mlp(self.norm(x))


class ToyLM(nn.Module):
    def __init__(self, vocab=256, d=64, f=256, layers=2):
        super().__init__()
        self.emb = nn.Embedding(vocab, d)
        self.blocks = nn.ModuleList([ToyBlock(d, f) for _ in range(layers)])
        self.head = nn.Linear(d, vocab, bias=False)

    def forward(self, ids):
        h = self.emb(ids)
        for b in self.blocks:
            h = b(h)
        return {"logits": self.head(h)}


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--model", default="toy")
    ap.add_argument("--n_experts", type=int, default=8)
    ap.add_argument("--top_k", type=int, default=2)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--analyze_clusters", action="store_true")
    ap.add_argument("--routing", default="token_choice", choices=["token_choice", "expert_choice"])
    ap.add_argument("--d_ff_expert", type=float, default=None, help="width (>4) or fraction of the dense width (<=4)")
    ap.add_argument("--layer_config", default=None, help="per-layer configuration written by generate_config")
    ap.add_argument("--mode", default="data_free",
                    choices=["data_free", "parallel", "sequential", "empirical", "dynamic"],
                    help="training mode; 'parallel' and 'sequential' train on token batches through the model")
    ap.add_argument("--router_mlp", action="store_true")
    ap.add_argument("--no_expert_bias", action="store_true")
    ap.add_argument("--lr", type=float, default=1e-3)
    ap.add_argument("--output_dir", default="sparse_distillation_output")
    ap.add_argument("--device", default="cpu")
    a = ap.parse_args(argv)
    os.makedirs(a.output_dir, exist_ok=True)
    if a.model == "toy":
        torch.manual_seed(0)
        model = ToyLM()
    else:
        from transformers import AutoModelForCausalLM
        model = AutoModelForCausalLM.from_pretrained(a.model)
    model.to(a.device).eval()
    dff = None if a.d_ff_expert is None else (int(a.d_ff_expert) if a.d_ff_expert > 4 else float(a.d_ff_expert))
    cfg = DistillationConfig(n_experts=a.n_experts, moe_top_k=a.top_k, moe_routing=a.routing, d_ff_expert=dff,
                             layer_config_path=a.layer_config, data_free=a.mode == "data_free",
                             sequential_layers=a.mode == "sequential", empirical_routing=a.mode == "empirical",
                             dynamic_experts=a.mode == "dynamic", router_mlp=a.router_mlp,
                             use_expert_bias=not a.no_expert_bias, data_free_steps=a.steps,
                             data_free_seq_len=64, cluster_samples=2048, router_train_steps=min(200, a.steps),
                             reallocate_every_n_steps=max(a.steps // 4, 1), min_d_ff=16,
                             log_interval=0, learning_rate=a.lr)
    trainer = SparseDistillationTrainer(model, cfg, device=a.device)
    if a.analyze_clusters:
        analysis = {str(i): {str(k): v for k, v in trainer.analyze_cluster_quality(i, ks=(4, 8)).items()}
                    for i in range(len(trainer.ffn))}
        json.dump(analysis, open(os.path.join(a.output_dir, "cluster_analysis.json"), "w"), indent=2)
    batches = None
    if a.mode in ("parallel", "sequential"):
        vocab = 256 if a.model == "toy" else model.config.vocab_size
        g = torch.Generator().manual_seed(0)
        batches = [torch.randint(0, vocab, (2, 64), generator=g) for _ in range(a.steps)]
    hist = trainer.distill(batches, steps=a.steps)
    ev = trainer.evaluate(2)
    trainer.save(os.path.join(a.output_dir, "distilled_moe.pt"))
    sparse = convert_to_sparse(model, trainer=trainer)
    ids = [torch.randint(0, 256, (2, 32), device=a.device) for _ in range(2)] if a.model == "toy" else []
    stats = accumulate_routing_stats(sparse, ids) if ids else {}
    print(json.dumps({"eval": {str(k): v for k, v in ev.items()}, "routing": {str(k): v for k, v in stats.items()},
                      "first_loss": hist[0][0], "last_loss": hist[0][-1]}, indent=1))
    return trainer, sparse, ev


if __name__ == "__main__":
    main()
