"""Checkpoint inspection (counterpart of the reference's ``debug_training.py``): prints the
training state stored in a checkpoint, per-tensor statistics and any NaN / Inf values.

    python debug_training.py ckpt.pt
"""
import sys

import torch


def inspect(path: str, top: int = 10):
    ck = torch.load(path, map_location="cpu", weights_only=False)
    sd = ck.get("model_state_dict", ck.get("model", ck)) if isinstance(ck, dict) else ck
    meta = {k: v for k, v in ck.items() if not isinstance(v, (dict, list)) or k == "losses"} if isinstance(ck, dict) else {}
    if "losses" in meta:
        meta["losses"] = meta["losses"][-5:]
    print("state:", meta)
    bad, rows = [], []
    for k, v in sd.items():
        if torch.is_tensor(v) and v.is_floating_point():
            f = v.float()
            if not torch.isfinite(f).all():
                bad.append(k)
            rows.append((k, tuple(v.shape), float(f.mean()), float(f.std()) if f.numel() > 1 else 0.0, float(f.abs().max())))
    for r in sorted(rows, key=lambda r: -r[4])[:top]:
        print(f"{r[0]:60s} {str(r[1]):20s} mean {r[2]:+.3e} std {r[3]:.3e} max {r[4]:.3e}")
    print("non-finite tensors:", bad)
    return {"meta": meta, "non_finite": bad, "n_tensors": len(rows)}


def analyze_checkpoint(checkpoint_path):
    """The reference's name for ``inspect``."""
    return inspect(checkpoint_path)


if __name__ == "__main__":
    inspect(sys.argv[1])
