"""Restarting launcher: runs a multi-rank training job and, when a rank dies, starts it again from the newest
checkpoint that every rank finished writing.

    python elastic_launch.py --nproc-per-node 8 --max-restarts 3 --checkpoint-dir ckpt/ -- \
        train_distributed.py --config configs/training_4.5b.yaml --async-checkpoint

Each attempt is one ``python -m torch.distributed.run`` process group (one process per GPU, rendezvous on
127.0.0.1).  ``torchrun`` tears the remaining ranks down when one exits with an error, so the survivors do
not sit in a collective nobody will join; this launcher then looks under ``--checkpoint-dir`` for the newest
directory carrying all ranks' completion markers (or written synchronously) and relaunches with
``--resume <checkpoint-dir>`` and the same ``--checkpoint-dir``.  Without a complete checkpoint the job starts
over.  The reference has no restart logic: a failed rank ends the run (reference: train_distributed.py:747-1095
has no checkpointing at all; train.py:211-225 only saves on SIGINT / SIGTERM in a single process).

The children run with ``NCCL_NVLS_ENABLE=0``, ``KMOE_MULTIMEM=0`` and ``TORCH_SYMM_MEM_DISABLE_MULTICAST=1`` unless
the caller's environment sets them: a rank that can die should not be bound to an NVLink multicast object.  The
first two keep NCCL and this library's kernels off the multicast address; the third stops torch's
symmetric-memory allocator (which backs the peer buffers of the ``p2p`` transport) from creating and binding a
multicast object at rendezvous in the first place.

``--shrink`` lets a restart use fewer processes (halving, not below ``--min-nproc``) after two failures in a
row at the same size; the replicated-parameter plan and the parameter-sharded plan both reload ``model.pt``
at any world size (optimizer shards are reused only when the layout matches).  A checkpoint written under expert
parallelism holds each rank's experts in its own file and loads only at the same size, so ``--shrink`` is
refused for such a job (the size is kept) with a message naming ``consolidate_expert_checkpoint`` as the way
to move it to another size by hand.
"""
from __future__ import annotations

import argparse
import os
import subprocess
import sys
import time
from typing import List, Optional

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)


def _strip_option(args: List[str], name: str) -> List[str]:
    out, skip = [], False
    for a in args:
        if skip:
            skip = False
            continue
        if a == name:
            skip = True
            continue
        if a.startswith(name + "="):
            continue
        out.append(a)
    return out


def build_command(nproc: int, port: int, script_args: List[str], checkpoint_dir: str, resume: Optional[str]) -> List[str]:
    args = _strip_option(_strip_option(list(script_args), "--resume"), "--checkpoint-dir")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={nproc}",
           "--master-addr", "127.0.0.1", "--master-port", str(port)] + args + ["--checkpoint-dir", checkpoint_dir]
    if resume:
        cmd += ["--resume", resume]
    return cmd


def supervise(nproc: int, script_args: List[str], checkpoint_dir: str, max_restarts: int = 3, port: int = 29500,
              shrink: bool = False, min_nproc: int = 1, backoff_s: float = 1.0, env=None, log=print) -> int:
    """Returns the exit code of the last attempt (0 = the job finished)."""
    from kolmogorov_moe_architecture_b200.training.checkpoint import latest_complete_checkpoint
    if env is None:
        env = dict(os.environ)
    # a job that may lose a rank keeps off the NVLink switch's multicast objects: a process that dies while its
    # memory is bound to one can fault the other ranks' GPUs; plain peer loads and stores have no such coupling
    env.setdefault("NCCL_NVLS_ENABLE", "0")
    env.setdefault("KMOE_MULTIMEM", "0")
    env.setdefault("TORCH_SYMM_MEM_DISABLE_MULTICAST", "1")
    attempt, fails_at_size = 0, 0
    while True:
        # completeness is judged by each directory's own manifest (its writer count), so a checkpoint written
        # by a larger job is found by a smaller one too
        found = latest_complete_checkpoint(checkpoint_dir, world=nproc) if os.path.isdir(checkpoint_dir) else None
        cmd = build_command(nproc, port + attempt, script_args, checkpoint_dir, checkpoint_dir if found else None)
        log(f"[elastic] attempt {attempt + 1}: {nproc} processes, "
            f"{'resuming from ' + os.path.basename(found) if found else 'starting fresh'}")
        t0 = time.time()
        rc = subprocess.call(cmd, env=env, cwd=ROOT)
        if rc == 0:
            log(f"[elastic] finished after {attempt} restart(s)")
            return 0
        attempt += 1
        log(f"[elastic] attempt ended with exit code {rc} after {time.time() - t0:.0f} s")
        if attempt > max_restarts:
            log(f"[elastic] giving up after {max_restarts} restart(s)")
            return rc
        fails_at_size += 1
        if shrink and fails_at_size >= 2 and nproc // 2 >= min_nproc:
            if _has_expert_shards(checkpoint_dir):
                log("[elastic] --shrink refused: the checkpoints hold per-rank expert shards (expert parallelism), "
                    "which load only at the size that wrote them; keeping "
                    f"{nproc} processes (training.checkpoint.consolidate_expert_checkpoint merges the shards "
                    "for a job of another size)")
                fails_at_size = 0
            else:
                nproc, fails_at_size = nproc // 2, 0
                log(f"[elastic] two failures in a row: continuing with {nproc} processes")
        time.sleep(backoff_s)


def _has_expert_shards(root: str) -> bool:
    import re
    if not os.path.isdir(root):
        return False
    for name in os.listdir(root):
        d = os.path.join(root, name)
        if re.fullmatch(r"checkpoint-(\d+)", name) and os.path.isdir(d):
            if any(re.fullmatch(r"experts-rank\d+\.pt", n) for n in os.listdir(d)):
                return True
    return False


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description="restart a multi-rank training job from its newest complete checkpoint")
    ap.add_argument("--nproc-per-node", type=int, required=True)
    ap.add_argument("--max-restarts", type=int, default=3)
    ap.add_argument("--checkpoint-dir", required=True)
    ap.add_argument("--master-port", type=int, default=29500)
    ap.add_argument("--shrink", action="store_true")
    ap.add_argument("--min-nproc", type=int, default=1)
    ap.add_argument("script", nargs=argparse.REMAINDER, help="-- <training script> <its arguments>")
    a = ap.parse_args(argv)
    script = a.script[1:] if a.script and a.script[0] == "--" else a.script
    assert script, "give the training script after --"
    return supervise(a.nproc_per_node, script, a.checkpoint_dir, a.max_restarts, a.master_port, a.shrink, a.min_nproc)


if __name__ == "__main__":
    sys.exit(main())
