"""Perplexity evaluation of a checkpoint on several text corpora (counterpart of the
reference's ``eval/evaluate_perplexity.py``).

    python eval/evaluate_perplexity.py --checkpoint ckpt.pt --config configs/production_training.yaml \
        [--datasets reddit cc_news] [--tokens 2000000] [--seq-len 1024] [--stride 512] [--output eval/results.md]

Loads any supported checkpoint format, streams each corpus, cuts strided windows, and reports the
``lm_loss``-weighted perplexity per corpus and their average, as markdown and JSON.  Without network
access the corpora cannot be opened; ``--synthetic`` evaluates on uniform-random tokens instead
(perplexity then sits near the vocabulary size, which checks the pipeline end to end).
"""
import argparse
import json
import math
import os
import sys
import time
from dataclasses import dataclass
from typing import Dict, List, Optional

import torch

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))


@dataclass
class EvalDataset:
    name: str
    hf_name: str
    hf_config: Optional[str] = None
    split: str = "train"
    text_column: str = "text"
    description: str = ""


EVAL_DATASETS = [
    EvalDataset("wikipedia", "wikipedia", "20220301.en", "train", "text", "English Wikipedia (March 2022)"),
    EvalDataset("reddit", "openwebtext", None, "train", "text", "OpenWebText"),
    EvalDataset("cc_news", "cc_news", None, "train", "text", "Common Crawl News"),
    EvalDataset("arxiv", "togethercomputer/RedPajama-Data-1T-Sample", None, "train", "text", "RedPajama sample"),
    EvalDataset("stackexchange", "HuggingFaceFW/fineweb-edu", "sample-10BT", "train", "text", "FineWeb-Edu"),
    EvalDataset("books", "emozilla/pg19-test", None, "test", "text", "PG-19 books"),
]


def windows(tokens: List[int], seq_len: int, stride: int) -> List[torch.Tensor]:
    return [torch.tensor(tokens[i:i + seq_len], dtype=torch.long) for i in range(0, len(tokens) - seq_len, stride)]


def prepare_eval_data(dataset_config: EvalDataset, tokenizer, target_tokens=3_000_000, seq_len=2048, stride=512):
    ds = dataset_config
    try:
        from datasets import load_dataset
        args = (ds.hf_name, ds.hf_config) if ds.hf_config else (ds.hf_name,)
        data = load_dataset(*args, split=ds.split, streaming=True)
    except Exception as e:
        print(f"  ERROR loading {ds.name}: {type(e).__name__}: {e}")
        return []
    toks: List[int] = []
    for ex in data:
        text = ex.get(ds.text_column, "")
        if not text or len(text.strip()) < 100:
            continue
        enc = tokenizer.encode(text, truncation=False)
        toks.extend(enc["input_ids"] if isinstance(enc, dict) else enc)
        if len(toks) >= target_tokens:
            break
    if len(toks) < seq_len:
        return []
    return windows(toks[:target_tokens], seq_len, stride)


@torch.no_grad()
def compute_perplexity(model, sequences: List[torch.Tensor], batch_size: int = 1, device: str = "cuda") -> Dict[str, float]:
    if not sequences:
        return {"perplexity": float("nan"), "loss": float("nan"), "num_tokens": 0}
    tot = torch.zeros((), dtype=torch.float64, device=device)
    n = 0
    for i in range(0, len(sequences), batch_size):
        ids = torch.stack(sequences[i:i + batch_size]).to(device)
        out = model(ids, labels=ids, return_logits=False)
        k = ids.numel() - ids.shape[0]
        tot += out["lm_loss"].double() * k
        n += k
    loss = float(tot) / n
    return {"perplexity": math.exp(loss) if loss < 100 else float("inf"), "loss": loss, "num_tokens": n}


def load_model(checkpoint: Optional[str], config_path: str, device: str, dtype=torch.bfloat16):
    from kolmogorov_moe_architecture_b200 import MoETransformer
    from kolmogorov_moe_architecture_b200.training.checkpoint import load_model_state
    from kolmogorov_moe_architecture_b200.utils.config_io import load_yaml, model_config_tolerant
    cfg = model_config_tolerant(load_yaml(config_path))
    model = MoETransformer(cfg, verbose=False)
    if checkpoint:
        load_model_state(model, checkpoint, strict=False)
    return model.to(device).to(dtype if device != "cpu" else torch.float32).eval(), cfg


def write_reports(results: Dict[str, Dict], meta: Dict, out_md: str):
    """Markdown table plus a JSON file beside it, in the layout of the reference's committed results
    (eval/results.md, eval/results_2000step.json): ``{"checkpoint", "config", "settings": {"tokens_per_dataset",
    "seq_len", "stride"}, "results": {dataset: {"perplexity", "loss", "num_tokens", ...}}}`` and, in addition,
    ``"average_perplexity"`` and the full ``"meta"``.  A data set that could not be loaded is listed as N/A."""
    os.makedirs(os.path.dirname(os.path.abspath(out_md)), exist_ok=True)
    ok = lambda r: r.get("num_tokens", 0) > 0 and math.isfinite(r.get("perplexity", float("nan")))
    good = [r["perplexity"] for r in results.values() if ok(r)]
    avg = sum(good) / len(good) if good else float("nan")
    with open(out_md, "w") as f:
        f.write("# Perplexity Evaluation Results\n\n## Settings\n\n")
        labels = {"checkpoint": "Checkpoint", "config": "Config", "device": "Device",
                  "tokens_per_dataset": "Tokens per dataset", "seq_len": "Sequence length", "stride": "Stride"}
        for k, v in meta.items():
            shown = f"{v:,}" if isinstance(v, int) and k == "tokens_per_dataset" else (f"`{v}`" if isinstance(v, str) else v)
            f.write(f"- **{labels.get(k, k)}**: {shown}\n")
        f.write("\n## Results\n\n| Dataset | Perplexity | Loss | Tokens | Time (s) |\n"
                "|---------|------------|------|--------|----------|\n")
        for name, r in results.items():
            if ok(r):
                f.write(f"| {name} | {r['perplexity']:.2f} | {r['loss']:.4f} | {r['num_tokens']:,} | "
                        f"{r.get('seconds', 0):.1f} |\n")
            else:
                f.write(f"| {name} | N/A | N/A | - | - | *Could not load data* |\n")
        f.write(f"| **Average** | **{avg:.2f}** | - | - | - |\n")
    with open(os.path.splitext(out_md)[0] + ".json", "w") as f:
        json.dump({"checkpoint": meta.get("checkpoint"), "config": meta.get("config"),
                   "settings": {k: meta.get(k) for k in ("tokens_per_dataset", "seq_len", "stride")},
                   "results": results, "average_perplexity": avg, "meta": meta}, f, indent=2)
    return avg


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--checkpoint", type=str, default=None)
    ap.add_argument("--config", type=str, default="configs/production_training.yaml")
    ap.add_argument("--datasets", nargs="*", default=None)
    ap.add_argument("--tokens", type=int, default=3_000_000)
    ap.add_argument("--seq-len", type=int, default=1024)
    ap.add_argument("--stride", type=int, default=512)
    ap.add_argument("--batch-size", type=int, default=1)
    ap.add_argument("--device", type=str, default="cuda" if torch.cuda.is_available() else "cpu")
    ap.add_argument("--tokenizer", type=str, default="gpt2")
    ap.add_argument("--output", type=str, default="eval/results.md")
    ap.add_argument("--synthetic", action="store_true")
    a = ap.parse_args(argv)
    model, cfg = load_model(a.checkpoint, a.config, a.device)
    seq_len = min(a.seq_len, cfg.max_seq_len)
    results = {}
    if a.synthetic:
        g = torch.Generator().manual_seed(0)
        toks = torch.randint(0, cfg.vocab_size, (a.tokens,), generator=g).tolist()
        t0 = time.time()
        results["synthetic"] = compute_perplexity(model, windows(toks, seq_len, a.stride), a.batch_size, a.device)
        results["synthetic"]["seconds"] = time.time() - t0
    else:
        from kolmogorov_moe_architecture_b200.data import TokenizerWrapper
        tok = TokenizerWrapper(a.tokenizer)
        for ds in EVAL_DATASETS:
            if a.datasets and ds.name not in a.datasets:
                continue
            seqs = prepare_eval_data(ds, tok, a.tokens, seq_len, a.stride)
            t0 = time.time()
            results[ds.name] = compute_perplexity(model, seqs, a.batch_size, a.device)
            results[ds.name]["seconds"] = time.time() - t0
    avg = write_reports(results, {"checkpoint": a.checkpoint, "config": a.config, "device": str(a.device),
                                  "tokens_per_dataset": a.tokens, "seq_len": seq_len, "stride": a.stride}, a.output)
    print(f"average perplexity {avg:.2f} -> {a.output}")
    return results


# ---- names of the reference's script, for code that imports them from here
def load_config(path=None, config_path=None):
    """The YAML file as a dict."""
    from kolmogorov_moe_architecture_b200.utils.config_io import load_yaml
    return load_yaml(config_path if path is None else path)


def load_model_from_checkpoint(checkpoint_path, config_path, device="cuda"):
    """(model, model configuration) with the checkpoint's weights, in evaluation mode."""
    model, cfg = load_model(checkpoint_path, config_path, device,
                            dtype=torch.bfloat16 if str(device).startswith("cuda") else torch.float32)
    return model.eval(), cfg


if __name__ == "__main__":
    main()
