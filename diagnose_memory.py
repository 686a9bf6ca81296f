"""Memory-leak diagnosis: device memory after every micro-batch and optimizer step of a short run.

    python diagnose_memory.py [configs/production_training.yaml] [--steps 20] [--accum 2] [--batch-size 1]

Where ``check_memory.py`` reports the footprint of one step by phase, this script looks for growth:
it runs ``--steps`` micro-batches with an optimizer step every ``--accum`` of them, records allocated /
reserved / peak memory after each, fits the growth per optimizer step, and lists module attributes that
are Python containers with contents (state that can accumulate across steps).  Counterpart of the
reference's ``diagnose_memory.py`` (reference: diagnose_memory.py:32-194).  Without a GPU it still runs
(on the host) and reports zeros, which keeps the command line testable.
"""
import argparse
import gc
import os
import sys

import torch

sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))

LEAK_MB_PER_STEP = 10.0        # growth per optimizer step above which the run is called leaking


def mem():
    if not torch.cuda.is_available():
        return 0.0, 0.0, 0.0
    torch.cuda.synchronize()
    return (torch.cuda.memory_allocated() / 1e9, torch.cuda.memory_reserved() / 1e9,
            torch.cuda.max_memory_allocated() / 1e9)


def show(label, prev=None):
    a, r, p = mem()
    delta = f" (delta {a - prev:+.3f} GB)" if prev is not None else ""
    print(f"  {label}: alloc={a:.3f} GB, reserved={r:.3f} GB, peak={p:.3f} GB{delta}")
    return a


def growing_containers(model):
    """(module path, attribute, kind, length) of list / dict attributes that hold something."""
    found = []
    for name, mod in model.named_modules():
        for attr, val in vars(mod).items():
            if attr.startswith("_") or attr in ("training",):
                continue
            if isinstance(val, (list, dict)) and len(val) > 0:
                found.append((name or "<root>", attr, type(val).__name__, len(val)))
    return found


def growth_per_step(samples):
    """Least-squares slope (GB per optimizer step) of the allocated memory after each optimizer step; the
    first sample is left out (optimizer state is created on the first step)."""
    ys = samples[1:]
    n = len(ys)
    if n < 2:
        return 0.0
    mx, my = (n - 1) / 2.0, sum(ys) / n
    den = sum((i - mx) ** 2 for i in range(n))
    return sum((i - mx) * (y - my) for i, y in enumerate(ys)) / den if den else 0.0


def main(argv=None):
    ap = argparse.ArgumentParser()
    ap.add_argument("config", nargs="?", default="configs/production_training.yaml")
    ap.add_argument("--steps", type=int, default=20, help="micro-batches to run")
    ap.add_argument("--accum", type=int, default=2, help="micro-batches per optimizer step")
    ap.add_argument("--batch-size", type=int, default=1)
    ap.add_argument("--seq-len", type=int, default=None)
    a = ap.parse_args(argv)
    from kolmogorov_moe_architecture_b200 import MoETransformer
    from kolmogorov_moe_architecture_b200.training.optim_factory import build_optimizer
    from kolmogorov_moe_architecture_b200.utils.config_io import load_yaml, model_config_tolerant

    print("=" * 70 + "\nMEMORY LEAK DIAGNOSIS\n" + "=" * 70)
    print(f"\nUsing config: {a.config}")
    cfg = model_config_tolerant(load_yaml(a.config), seq_len=a.seq_len)
    print(f"\nModel config:\n  n_layers: {cfg.n_layers}\n  n_experts: {cfg.n_experts}\n  d_model: {cfg.d_model}\n"
          f"  max_seq_len: {cfg.max_seq_len}\n  mod_enabled: {cfg.mod_enabled}")
    gc.collect()
    dev = "cuda" if torch.cuda.is_available() else "cpu"
    if dev == "cuda":
        torch.cuda.empty_cache()
        torch.cuda.reset_peak_memory_stats()
    prev = show("Initial state")
    print("\n--- Model Creation ---")
    model = MoETransformer(cfg, verbose=False).to(dev).to(torch.bfloat16 if dev == "cuda" else torch.float32)
    prev = show("After model creation", prev)
    print("\n--- Optimizer Creation ---")
    opt = build_optimizer(model)
    prev = show("After optimizer creation", prev)
    print("\n--- Training Steps ---")
    model.train()
    after_opt = []
    for step in range(a.steps):
        ids = torch.randint(0, cfg.vocab_size, (a.batch_size, cfg.max_seq_len), device=dev)
        out = model(ids, labels=ids, return_logits=False)
        (out["loss"] / a.accum).backward()
        del out
        if (step + 1) % a.accum == 0:
            torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
            opt.step()
            opt.zero_grad(set_to_none=True)
            al, re_, pk = mem()
            after_opt.append(al)
            print(f"  Step {step + 1:3d} (opt step): alloc={al:.3f} GB, reserved={re_:.3f} GB, peak={pk:.3f} GB")
        else:
            al, re_, _ = mem()
            print(f"  Step {step + 1:3d} (accum):    alloc={al:.3f} GB, reserved={re_:.3f} GB")
    print("\n--- Analysis ---")
    slope = growth_per_step(after_opt)
    leaking = slope * 1000 > LEAK_MB_PER_STEP
    if after_opt:
        print(f"Memory at first opt step: {after_opt[0]:.3f} GB")
        print(f"Memory at last opt step:  {after_opt[-1]:.3f} GB")
        print(f"Growth per opt step: {slope * 1000:.1f} MB")
    if leaking:
        print(f"\nMEMORY LEAK DETECTED: ~{slope * 1000:.0f} MB per optimizer step; this ends in an out-of-memory error."
              "\nPossible causes:\n  1. autograd graphs kept alive (a loss or output tensor stored between steps)"
              "\n  2. tensors appended to module attributes\n  3. optimizer state that keeps growing"
              "\n  4. allocator fragmentation (reserved grows while allocated does not)")
    else:
        print("\nNo significant memory leak detected"
              + (f" (memory is stable at ~{after_opt[-1]:.2f} GB)" if after_opt else ""))
    print("\n--- Checking for growing state in model ---")
    found = growing_containers(model)
    for name, attr, kind, n in found:
        print(f"  {name}.{attr}: {kind} with {n} items")
    if not found:
        print("  none")
    print("\n" + "=" * 70 + "\nDIAGNOSIS COMPLETE\n" + "=" * 70)
    return {"growth_mb_per_step": slope * 1000, "leak": leaking, "containers": found, "opt_steps": len(after_opt)}


# ---- names of the reference's script, for code that imports them from here
def load_config(path=None, config_path=None):
    """The YAML file as a dict."""
    from kolmogorov_moe_architecture_b200.utils.config_io import load_yaml
    return load_yaml(config_path if path is None else path)


def get_mem():
    """(allocated, reserved) in GB."""
    a, r, _ = mem()
    return a, r


def print_mem(label, prev_alloc=None):
    return show(label, prev_alloc)


if __name__ == "__main__":
    main()
