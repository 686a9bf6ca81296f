"""GPU memory by phase for one training step of a configuration (counterpart of the reference's
``check_memory.py``): allocated / reserved / peak after model creation,
forward, backward and the optimizer step.

    python check_memory.py --config configs/training_1.5b.yaml [--batch-size 4] [--seq-len 2048]
"""
import argparse
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))


def snapshot(tag, rows):
    if torch.cuda.is_available():
        torch.cuda.synchronize()
        rows.append((tag, torch.cuda.memory_allocated() / 2**30, torch.cuda.memory_reserved() / 2**30,
                     torch.cuda.max_memory_allocated() / 2**30))
    else:
        rows.append((tag, 0.0, 0.0, 0.0))


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("--config", required=True)
    ap.add_argument("--batch-size", type=int, default=1)
    ap.add_argument("--seq-len", type=int, default=None)
    a = ap.parse_args(argv)
    from kolmogorov_moe_architecture_b200 import MoETransformer
    from kolmogorov_moe_architecture_b200.parallel.zero import ShardedDataParallel
    from kolmogorov_moe_architecture_b200.utils.config_io import load_yaml, model_config_tolerant
    cfg = model_config_tolerant(load_yaml(a.config), seq_len=a.seq_len)
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    rows = []
    snapshot("start", rows)
    model = MoETransformer(cfg, verbose=False).to(dev).to(torch.bfloat16 if dev == "cuda" else torch.float32)
    snapshot("model", rows)
    dp = ShardedDataParallel(model, optimizer_kind="muon")
    snapshot("flat buffers + optimizer", rows)
    ids = torch.randint(0, cfg.vocab_size, (a.batch_size, cfg.max_seq_len), device=dev)
    model.train()
    out = model(ids, labels=ids, return_logits=False)
    snapshot("forward", rows)
    out["loss"].backward()
    snapshot("backward", rows)
    dp.reduce_clip_and_step(None, 1.0)
    snapshot("optimizer step", rows)
    print(f"{'phase':28s} {'alloc GB':>10s} {'reserved GB':>12s} {'peak GB':>10s}")
    for r in rows:
        print(f"{r[0]:28s} {r[1]:10.2f} {r[2]:12.2f} {r[3]:10.2f}")
    return rows


# ---- names of the reference's script, for code that imports them from here
def load_config(path=None, config_path=None):
    """The YAML file as a dict."""
    from kolmogorov_moe_architecture_b200.utils.config_io import load_yaml
    return load_yaml(config_path if path is None else path)


def print_memory(step, label):
    """One line with the allocated / reserved / peak GiB at this point; returns the row."""
    rows = []
    snapshot(f"{step}:{label}", rows)
    tag, alloc, reserved, peak = rows[0]
    print(f"[{tag}] allocated {alloc:.2f} GiB  reserved {reserved:.2f} GiB  peak {peak:.2f} GiB")
    return rows[0]


if __name__ == "__main__":
    main()
