"""End-to-end sparse distillation (counterpart of the reference's
``Experiments/sparse_distillation/example_usage.py``):

    python -m experiments.sparse_distillation.example_usage --model <hf name or 'toy'> \
        [--analyze_clusters] [--n_experts 8] [--data_free_steps 200] [--output out/]

load model -> tokenise the data set -> (``--analyze_clusters``: cluster analysis -> cluster_analysis.json, then
stop) -> distill -> evaluate -> save ``distilled_moe_layers.pt`` -> convert_to_sparse -> save ``sparse_model.pt`` ->
routing statistics (and a short generation when a tokenizer is at hand).  Every argument of the reference's script is
accepted under the same name.  ``--model toy`` (the default here: there is no network) builds a small random
transformer so the pipeline runs anywhere; ``--mode`` and ``--steps`` are shorthands of this framework.
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import torch
import torch.nn as nn

from .convert import convert_to_sparse
from .data import load_token_batches
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


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(description="Sparse distillation: dense FFN -> MoE")
    # model
    ap.add_argument("--model", default="toy", help="Hugging Face model name or path, or 'toy'")
    ap.add_argument("--dtype", default="float32", choices=["float32", "float16", "bfloat16"])
    # data
    ap.add_argument("--dataset", default="wikitext", help="data set name (wikitext, c4, fineweb-edu, ...)")
    ap.add_argument("--dataset_config", default="wikitext-2-raw-v1")
    ap.add_argument("--data", default=None, help="uint16 token file used when the data set cannot be loaded")
    ap.add_argument("--max_samples", type=int, default=10000)
    ap.add_argument("--seq_len", type=int, default=2048)
    ap.add_argument("--batch_size", type=int, default=1)
    # mixture of experts
    ap.add_argument("--n_experts", type=int, default=8, help="experts per layer")
    ap.add_argument("--moe_top_k", "--top_k", dest="moe_top_k", type=int, default=2,
                    help="experts per token (token choice)")
    ap.add_argument("--capacity_factor", type=float, default=1.25,
                    help="expert choice: tokens per expert = seq * factor / n_experts")
    ap.add_argument("--d_ff_expert", default=None,
                    help="expert width: unset = share of the dense width, <= 1 = fraction of it, > 1 = absolute")
    ap.add_argument("--routing", default="token_choice", choices=["expert_choice", "token_choice"])
    ap.add_argument("--layer_config", default=None, help="per-layer configuration written by generate_config")
    # training
    ap.add_argument("--epochs", type=int, default=1)
    ap.add_argument("--lr", type=float, default=1e-4)
    ap.add_argument("--max_steps", type=int, default=1000)
    ap.add_argument("--sequential", action="store_true", help="one layer at a time (much lower memory)")
    ap.add_argument("--no_data_free", action="store_true", help="train on the data set instead of random inputs")
    ap.add_argument("--data_free_steps", type=int, default=20000, help="steps per layer on random inputs")
    ap.add_argument("--data_free_batch_size", type=int, default=4)
    ap.add_argument("--data_free_seq_len", type=int, default=512)
    ap.add_argument("--no_compile", action="store_true",
                    help="accepted for compatibility: this trainer never uses torch.compile")
    # auxiliary losses
    ap.add_argument("--no_load_balance", action="store_true")
    ap.add_argument("--load_balance_weight", type=float, default=0.01)
    ap.add_argument("--no_z_loss", action="store_true")
    ap.add_argument("--z_loss_weight", type=float, default=0.001)
    # supervised (cluster-based) routing
    ap.add_argument("--no_supervised_routing", action="store_true")
    ap.add_argument("--cluster_samples", type=int, default=1000000)
    ap.add_argument("--router_train_steps", type=int, default=10000)
    ap.add_argument("--analyze_clusters", action="store_true",
                    help="cluster-quality analysis of every layer -> cluster_analysis.json, then stop")
    # empirical routing and its curriculum
    ap.add_argument("--empirical_routing", action="store_true")
    ap.add_argument("--empirical_eval_interval", type=int, default=10)
    ap.add_argument("--empirical_temperature", type=float, default=0.1)
    ap.add_argument("--empirical_entropy_weight", type=float, default=0.01)
    ap.add_argument("--no_curriculum", action="store_true")
    ap.add_argument("--curriculum_warmup_steps", type=int, default=5000)
    ap.add_argument("--curriculum_initial_balance", type=float, default=0.9)
    ap.add_argument("--curriculum_final_balance", type=float, default=0.3)
    ap.add_argument("--no_gradient_routing", action="store_true", help="loss-based instead of gradient-based targets")
    ap.add_argument("--gradient_routing_exact", action="store_true")
    # router architecture
    ap.add_argument("--router_mlp", action="store_true")
    ap.add_argument("--router_hidden_dim", type=int, default=256)
    ap.add_argument("--router_n_layers", type=int, default=2)
    ap.add_argument("--no_expert_bias", action="store_true")
    # dynamic experts
    ap.add_argument("--dynamic", action="store_true", help="experts of unequal width, reallocated by tracked loss")
    ap.add_argument("--reallocate_every", type=int, default=500)
    ap.add_argument("--growth_factor", type=float, default=1.25)
    ap.add_argument("--shrink_factor", type=float, default=0.8)
    ap.add_argument("--min_d_ff", type=int, default=256)
    ap.add_argument("--max_d_ff", type=int, default=8192)
    # output, device
    ap.add_argument("--output", "--output_dir", dest="output", default="./sparse_distillation_output")
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    # shorthands of this framework
    ap.add_argument("--mode", default=None, choices=["data_free", "parallel", "sequential", "empirical", "dynamic"],
                    help="shorthand for --no_data_free / --sequential / --empirical_routing / --dynamic")
    ap.add_argument("--steps", type=int, default=None, help="sets --data_free_steps and --max_steps, and scales the "
                    "router pre-training, the cluster sample and the reallocation interval to a run of that length")
    ap.add_argument("--k_values", default=None, help="cluster counts of --analyze_clusters, comma separated "
                    "(default 4, 6, ..., 64, bounded by the sample)")
    return ap


def parse_expert_width(v):
    """None, a fraction of the dense width (<= 1) or an absolute width (> 1); unparsable text means None."""
    if v is None:
        return None
    try:
        val = float(v)
    except ValueError:
        return None
    return val if val <= 1.0 else int(val)


def config_from_args(a) -> DistillationConfig:
    if a.mode is not None:
        a.no_data_free = a.no_data_free or a.mode in ("parallel", "sequential")
        a.sequential = a.sequential or a.mode == "sequential"
        a.empirical_routing = a.empirical_routing or a.mode == "empirical"
        a.dynamic = a.dynamic or a.mode == "dynamic"
    quick = {}
    if a.steps is not None:
        a.data_free_steps = a.max_steps = a.steps
        a.router_train_steps = min(a.router_train_steps, max(a.steps, 1), 200)
        a.cluster_samples = min(a.cluster_samples, 2048)
        a.reallocate_every = min(a.reallocate_every, max(a.steps // 4, 1))
        a.data_free_seq_len = min(a.data_free_seq_len, 64)
        a.min_d_ff = min(a.min_d_ff, 16)
        quick = dict(log_interval=0)
    return DistillationConfig(
        n_experts=a.n_experts, moe_top_k=a.moe_top_k, moe_capacity_factor=a.capacity_factor, moe_routing=a.routing,
        d_ff_expert=parse_expert_width(a.d_ff_expert), layer_config_path=a.layer_config, learning_rate=a.lr,
        use_cosine_loss=True, init_from_dense=True, sequential_layers=a.sequential,
        data_free=not a.no_data_free, data_free_steps=a.data_free_steps,
        data_free_batch_size=a.data_free_batch_size, data_free_seq_len=a.data_free_seq_len, use_compile=False,
        use_load_balancing=not a.no_load_balance, load_balancing_weight=a.load_balance_weight,
        use_z_loss=not a.no_z_loss, z_loss_weight=a.z_loss_weight,
        supervised_routing=not a.no_supervised_routing and not a.empirical_routing,
        cluster_samples=a.cluster_samples, router_train_steps=a.router_train_steps,
        empirical_routing=a.empirical_routing, empirical_eval_interval=a.empirical_eval_interval,
        empirical_temperature=a.empirical_temperature, empirical_entropy_weight=a.empirical_entropy_weight,
        curriculum_routing=not a.no_curriculum, curriculum_warmup_steps=a.curriculum_warmup_steps,
        curriculum_initial_balance=a.curriculum_initial_balance, curriculum_final_balance=a.curriculum_final_balance,
        gradient_routing=not a.no_gradient_routing, gradient_routing_fast=not a.gradient_routing_exact,
        router_mlp=a.router_mlp, router_hidden_dim=a.router_hidden_dim, router_n_layers=a.router_n_layers,
        use_expert_bias=not a.no_expert_bias, dynamic_experts=a.dynamic, reallocate_every_n_steps=a.reallocate_every,
        growth_factor=a.growth_factor, shrink_factor=a.shrink_factor, min_d_ff=a.min_d_ff, max_d_ff=a.max_d_ff,
        **quick)


def analyze_all_layers(trainer: SparseDistillationTrainer, batches, k_values, max_samples: int) -> dict:
    """Cluster quality of every layer's FFN outputs for each candidate expert count; the recommended count of a
    layer is the best-balanced one.  The file layout is what ``generate_config`` reads."""
    layers = {}
    trainer.cfg.cluster_samples, keep = max_samples, trainer.cfg.cluster_samples
    try:
        for i in range(len(trainer.ffn)):
            res = trainer.analyze_cluster_quality(i, ks=tuple(k_values), batches=batches)
            best = max(res, key=lambda k: res[k]["balance"])
            layers[str(i)] = {"n_experts": int(best), "balance": res[best]["balance"],
                              "silhouette": res[best]["silhouette"],
                              "all_results": {int(k): v for k, v in res.items()}}
    finally:
        trainer.cfg.cluster_samples = keep
    return {"d_model": trainer.d_model, "d_ff": trainer.d_ff_dense, "layers": layers}


def main(argv=None):
    a = build_parser().parse_args(argv)
    os.makedirs(a.output, exist_ok=True)
    dtype = {"float32": torch.float32, "float16": torch.float16, "bfloat16": torch.bfloat16}[a.dtype]
    tokenizer = None
    if a.model == "toy":
        torch.manual_seed(0)
        model, vocab = ToyLM().to(dtype), 256
    else:
        from transformers import AutoModelForCausalLM, AutoTokenizer
        model = AutoModelForCausalLM.from_pretrained(a.model, torch_dtype=dtype)
        vocab = model.config.vocab_size
        try:
            tokenizer = AutoTokenizer.from_pretrained(a.model)
        except Exception:
            tokenizer = None
    model.to(a.device).eval()
    cfg = config_from_args(a)
    quick = a.steps is not None
    seq = min(a.seq_len, 64) if quick else a.seq_len
    n_train = a.max_steps if a.no_data_free else 0
    n_eval = 2 if quick else 100
    batches, source, _pad = load_token_batches(
        a.model, vocab, dataset=a.dataset, dataset_config=a.dataset_config, data_file=a.data,
        max_samples=a.max_samples, seq_len=seq, batch_size=max(a.batch_size, 2 if quick else 1),
        n_batches=max(n_train, n_eval, 1), seed=0, device=a.device)
    trainer = SparseDistillationTrainer(dense_model=model, config=cfg, device=a.device)
    if a.analyze_clusters:
        ks = [int(k) for k in a.k_values.split(",")] if a.k_values else ([4, 8] if quick else list(range(4, 65, 2)))
        analysis = analyze_all_layers(trainer, batches, ks, min(a.cluster_samples, 100000))
        path = os.path.join(a.output, "cluster_analysis.json")
        json.dump(analysis, open(path, "w"), indent=2)
        print(f"cluster analysis written to {path}; next: python -m experiments.sparse_distillation.generate_config "
              f"{path}")
        return trainer, None, analysis
    if cfg.data_free:
        hist = trainer.distill()
    else:
        hist = trainer.distill(dataloader=batches, epochs=a.epochs, max_steps=a.max_steps)
    ev = trainer.evaluate(batches=batches[:n_eval], max_batches=n_eval)
    ck = os.path.join(a.output, "distilled_moe_layers.pt")
    trainer.save(ck)
    sparse = convert_to_sparse(model, trainer=trainer)
    torch.save({"model_state_dict": sparse.state_dict(), "config": cfg}, os.path.join(a.output, "sparse_model.pt"))
    stats = accumulate_routing_stats(sparse, batches[:2])
    generated = None
    if tokenizer is not None and hasattr(model, "generate"):
        ids = tokenizer("The quick brown fox", return_tensors="pt").to(a.device)
        with torch.no_grad():
            generated = tokenizer.decode(model.generate(**ids, max_new_tokens=50, do_sample=True, temperature=0.7)[0],
                                         skip_special_tokens=True)
    print(json.dumps({"data": source, "eval": {str(k): v for k, v in ev.items()},
                      "routing": {str(k): v for k, v in stats.items()}, "first_loss": hist[0][0],
                      "last_loss": hist[0][-1], "generated": generated}, indent=1))
    return trainer, sparse, ev


if __name__ == "__main__":
    out = main()
    sys.exit(0)
