"""Checkpoint I/O in the reference's formats, plus sharded saves.

Formats (all hold the model under the key schema of the reference, so files interchange):

* ``A`` - ``Trainer``: one ``.pt`` dict ``{model_state_dict, optimizer_state_dict,
  lr_scheduler_state_dict, global_step, epoch, tokens_seen, config[, scaler_state_dict]}``
  (reference: moe_arch/training/trainer.py:340-388).
* ``B`` - ``train.py``: ``{step, epoch, data_idx, losses[-1000:], total_tokens, config_path,
  model_state_dict, optimizer_state_dict}``; the hybrid optimizer's state is a list of two
  dicts; file ``checkpoint-{N}[-interrupted|-final].pt`` (reference: train.py:186-208).
* ``C`` - ``train_custom.py``: directory ``checkpoint-{step}/{model.pt, optimizer.pt,
  training_state.pt}``, newest three kept (reference: train_custom.py:770-847).
* ``D`` - HF ``Trainer`` directories whose model keys carry a ``model.`` prefix
  (reference: train_production.py:107-120).
* ``E`` - distillation: ``{layers: {idx: state_dict}, config}``.

``load_model_state`` accepts any of them (and a bare state dict, a ``model`` key, or keys
prefixed by ``_orig_mod.`` / ``module.`` / ``model.``).  ``save_sharded`` writes one
optimizer-state file per rank next to a single model file, all ranks taking part, so no
rank skips a collective (the reference's format-C writer returns early on non-main ranks
before a collective gather, train_custom.py:780-781).  With an ``AsyncCheckpointWriter`` the
sharded saves only copy the state to pinned host memory on the training thread; files are written
in the background and a checkpoint directory becomes valid when every rank's marker is in it.
"""
from __future__ import annotations

import copy
import os
import re
import shutil
import threading
from typing import Any, Dict, Optional

import torch

_PREFIXES = ("_orig_mod.", "module.", "model.")


def unwrap_model(model):
    for attr in ("_orig_mod", "module"):
        while hasattr(model, attr):
            model = getattr(model, attr)
    return model


def strip_prefixes(sd: Dict[str, torch.Tensor]) -> Dict[str, torch.Tensor]:
    out = {}
    for k, v in sd.items():
        changed = True
        while changed:
            changed = False
            for p in ("_orig_mod.", "module."):
                if k.startswith(p):
                    k, changed = k[len(p):], True
        out[k] = v
    if out and all(k.startswith("model.") for k in out):
        out = {k[len("model."):]: v for k, v in out.items()}
    return out


def extract_model_state(obj: Any) -> Dict[str, torch.Tensor]:
    if isinstance(obj, dict):
        for key in ("model_state_dict", "model", "state_dict"):
            if key in obj and isinstance(obj[key], dict):
                return strip_prefixes(obj[key])
        if obj and all(torch.is_tensor(v) for v in obj.values()):
            return strip_prefixes(obj)
    raise ValueError("no model state dict found in checkpoint")


def load_checkpoint_file(path: str, map_location="cpu") -> Any:
    if os.path.isdir(path):
        for name in ("model.pt", "pytorch_model.bin"):
            f = os.path.join(path, name)
            if os.path.exists(f):
                return torch.load(f, map_location=map_location, weights_only=False)
        raise FileNotFoundError(f"no model file in {path}")
    return torch.load(path, map_location=map_location, weights_only=False)


def load_model_state(model, path_or_obj, strict: bool = True, map_location="cpu"):
    obj = load_checkpoint_file(path_or_obj, map_location) if isinstance(path_or_obj, str) else path_or_obj
    sd = extract_model_state(obj)
    return unwrap_model(model).load_state_dict(sd, strict=strict), obj


# ---------------------------------------------------------------- format A
def save_format_a(path, model, optimizer, lr_scheduler, global_step, epoch, tokens_seen, config, scaler=None):
    ck = {"model_state_dict": unwrap_model(model).state_dict(), "optimizer_state_dict": optimizer.state_dict(),
          "lr_scheduler_state_dict": lr_scheduler.state_dict() if lr_scheduler is not None else None,
          "global_step": global_step, "epoch": epoch, "tokens_seen": tokens_seen, "config": config}
    if scaler is not None:
        ck["scaler_state_dict"] = scaler.state_dict()
    _atomic_save(ck, path)


# ---------------------------------------------------------------- format B
def save_format_b(path, model, optimizer, step, epoch, data_idx, losses, total_tokens, config_path, extra=None):
    ck = {"step": step, "epoch": epoch, "data_idx": data_idx, "losses": list(losses)[-1000:],
          "total_tokens": total_tokens, "config_path": config_path,
          "model_state_dict": unwrap_model(model).state_dict(), "optimizer_state_dict": optimizer.state_dict()}
    if extra:
        ck.update(extra)
    _atomic_save(ck, path)


def format_b_name(step: int, suffix: Optional[str] = None) -> str:
    return f"checkpoint-{step}{'-' + suffix if suffix else ''}.pt"


# ---------------------------------------------------------------- format C
def save_format_c(root, step, model, optimizer, training_state: Dict, keep: int = 3, is_main: bool = True):
    d = os.path.join(root, f"checkpoint-{step}")
    if is_main:
        os.makedirs(d, exist_ok=True)
        _atomic_save(unwrap_model(model).state_dict(), os.path.join(d, "model.pt"))
        _atomic_save(optimizer.state_dict(), os.path.join(d, "optimizer.pt"))
        _atomic_save(training_state, os.path.join(d, "training_state.pt"))
        prune_checkpoints(root, keep)
    return d


def prune_checkpoints(root: str, keep: int = 3, world: Optional[int] = None) -> None:
    """Keep the newest ``keep`` checkpoint directories.  With ``world`` (background saves) only complete
    directories count towards ``keep`` and incomplete ones are left alone: another rank may still be
    writing into them."""
    ds = []
    for name in os.listdir(root):
        m = re.fullmatch(r"checkpoint-(\d+)", name)
        d = os.path.join(root, name)
        if m and os.path.isdir(d) and (world is None or checkpoint_complete(d, world)):
            ds.append((int(m.group(1)), name))
    for _, name in sorted(ds)[:-keep] if keep > 0 else []:
        shutil.rmtree(os.path.join(root, name), ignore_errors=True)


def load_format_c(d: str, model, optimizer=None, map_location="cpu") -> Dict:
    unwrap_model(model).load_state_dict(torch.load(os.path.join(d, "model.pt"), map_location=map_location,
                                                   weights_only=False))
    if optimizer is not None and os.path.exists(os.path.join(d, "optimizer.pt")):
        optimizer.load_state_dict(torch.load(os.path.join(d, "optimizer.pt"), map_location=map_location,
                                             weights_only=False))
    ts = os.path.join(d, "training_state.pt")
    return torch.load(ts, map_location=map_location, weights_only=False) if os.path.exists(ts) else {}


# ---------------------------------------------------------- sharded (ZeRO) save
def _expert_parallel_names(model) -> list:
    return [n for n, p in unwrap_model(model).named_parameters() if getattr(p, "_kmoe_expert_parallel", False)]


def _pools(dp):
    """(pool of the replicated parameters, pool of the expert-parallel tensors or None)."""
    pools = getattr(dp, "pools", None)
    if pools is None:
        return dp, None
    return pools[0], (pools[1] if len(pools) > 1 else None)


def _expert_file(sd, ep_names, expert_pool, ep_rank: int, ep_size: int) -> Dict[str, Any]:
    return {"ep_rank": ep_rank, "ep_size": ep_size, "params": {n: sd[n] for n in ep_names},
            "optimizer": expert_pool.optimizer_state_dict() if expert_pool is not None else None}


def _load_expert_file(d: str, rank: int, base, expert_pool, ep_rank: int, ep_size: int, map_location="cpu") -> None:
    f = os.path.join(d, f"experts-rank{rank}.pt")
    if not os.path.exists(f):
        raise FileNotFoundError(f"{f}: this rank's experts are not in the checkpoint (written with another world size?)")
    ex = torch.load(f, map_location=map_location, weights_only=False)
    assert (ex["ep_rank"], ex["ep_size"]) == (ep_rank, ep_size), \
        f"expert file holds shard {ex['ep_rank']} of {ex['ep_size']}, this rank is {ep_rank} of {ep_size}"
    params = dict(base.named_parameters())
    with torch.no_grad():
        for n, t in ex["params"].items():
            params[n].copy_(t)
    if expert_pool is not None and ex.get("optimizer") is not None:
        expert_pool.load_optimizer_state_dict(ex["optimizer"])


MANIFEST = "manifest.json"


def _write_manifest(d: str, mode: str, world: int, files) -> None:
    """Rank 0 writes this before any other file of a multi-rank checkpoint: who writes into the
    directory and which files must exist.  ``checkpoint_complete`` trusts a directory only when
    every rank named here has dropped its marker."""
    import json
    tmp = os.path.join(d, MANIFEST + ".tmp")
    with open(tmp, "w") as f:
        json.dump({"mode": mode, "world": int(world), "files": sorted(files),
                   "markers": [f"complete-rank{r}" for r in range(int(world))]}, f)
    os.replace(tmp, os.path.join(d, MANIFEST))


def read_manifest(d: str) -> Optional[Dict[str, Any]]:
    import json
    try:
        with open(os.path.join(d, MANIFEST)) as f:
            return json.load(f)
    except (OSError, ValueError):
        return None


def _mark_complete(d: str, rank: int) -> None:
    with open(os.path.join(d, f"complete-rank{rank}"), "w") as f:
        f.write("ok")


def _expected_files(kind: str, world: int, has_experts: bool):
    names = ["model.pt", "training_state.pt"] + [f"{kind}-rank{r}.pt" for r in range(world)]
    if has_experts:
        names += [f"experts-rank{r}.pt" for r in range(world)]
    return names


def _world_size(world: Optional[int] = None) -> int:
    import torch.distributed as dist
    return world or (dist.get_world_size() if dist.is_available() and dist.is_initialized() else 1)


def save_sharded(root: str, step: int, model, dp, training_state: Dict, rank: int, keep: int = 3,
                 writer: Optional["AsyncCheckpointWriter"] = None, world: Optional[int] = None,
                 ep_rank: int = 0, ep_size: int = 1) -> str:
    """Rank 0 writes ``model.pt`` (the replicated parameters) and ``training_state.pt``; every rank writes
    ``optimizer-rank{r}.pt`` with the state of the tensors it owns.  Under expert parallelism the expert
    tensors differ from rank to rank: they are left out of ``model.pt`` and every rank writes its own
    ``experts-rank{r}.pt`` (its experts, their optimizer state, and its place ``ep_rank`` of ``ep_size``).
    ``dp``: one pool or a ``ParallelPlan``.  ``writer``: write in the background (no barrier; the directory
    is valid once all ``world`` markers exist)."""
    import torch.distributed as dist
    d = os.path.join(root, f"checkpoint-{step}")
    os.makedirs(d, exist_ok=True)
    main_pool, expert_pool = _pools(dp)
    files: Dict[str, Any] = {os.path.join(d, f"optimizer-rank{rank}.pt"): main_pool.optimizer_state_dict()}
    sd = unwrap_model(model).state_dict()
    ep_names = _expert_parallel_names(model)
    if ep_names:
        files[os.path.join(d, f"experts-rank{rank}.pt")] = _expert_file(sd, ep_names, expert_pool, ep_rank, ep_size)
    w = _world_size(world)
    if rank == 0:
        _write_manifest(d, "sharded", w, _expected_files("optimizer", w, bool(ep_names)))
        files[os.path.join(d, "model.pt")] = {k: v for k, v in sd.items() if k not in set(ep_names)}
        files[os.path.join(d, "training_state.pt")] = training_state
    if writer is not None:
        writer.submit(files, d, rank, then=(lambda: prune_checkpoints(root, keep, world=w)) if rank == 0 else None)
        return d
    for path, obj in files.items():
        _atomic_save(obj, path)
    _mark_complete(d, rank)                  # after this rank's last file; the directory counts once all are there
    if dist.is_available() and dist.is_initialized():
        dist.barrier()
    if rank == 0:
        prune_checkpoints(root, keep, world=w)
    return d


def load_sharded(d: str, model, dp, rank: int, map_location="cpu", ep_rank: int = 0, ep_size: int = 1) -> Dict:
    base = unwrap_model(model)
    main_pool, expert_pool = _pools(dp)
    ep_names = _expert_parallel_names(model)
    sd = torch.load(os.path.join(d, "model.pt"), map_location=map_location, weights_only=False)
    missing, unexpected = base.load_state_dict(sd, strict=False)
    lost = [k for k in missing if k not in set(ep_names)]
    assert not lost and not unexpected, f"model.pt does not match the model: missing {lost[:5]}, unexpected {list(unexpected)[:5]}"
    if ep_names and not all(n in sd for n in ep_names):
        _load_expert_file(d, rank, base, expert_pool, ep_rank, ep_size, map_location)
    f = os.path.join(d, f"optimizer-rank{rank}.pt")
    man = read_manifest(d)
    if not os.path.exists(f) and man is not None and man.get("world") == getattr(main_pool, "world", None):
        # same job size, so this rank's moments must be there: resuming without them would silently
        # restart the optimizer on one rank only
        raise FileNotFoundError(f"{f}: optimizer state of rank {rank} is missing from a checkpoint written by "
                                f"{man.get('world')} ranks (incomplete checkpoint?)")
    if os.path.exists(f):
        osd = torch.load(f, map_location=map_location, weights_only=False)
        same = not isinstance(osd, dict) or osd.get("world") in (None, getattr(main_pool, "world", None))
        if same:
            main_pool.load_optimizer_state_dict(osd)
        else:           # written by a job of another size: parameters carry over, optimizer moments start fresh
            print(f"[checkpoint] {os.path.basename(f)} was written by {osd.get('world')} ranks; "
                  f"optimizer state of rank {rank} starts fresh", flush=True)
    ts = os.path.join(d, "training_state.pt")
    return torch.load(ts, map_location=map_location, weights_only=False) if os.path.exists(ts) else {}


def consolidate_expert_checkpoint(d: str) -> Dict[str, torch.Tensor]:
    """One full state dict from an expert-parallel checkpoint directory: ``model.pt`` plus the expert
    tensors of shards 0..ep_size-1 concatenated along the expert dimension (what a model built with
    ``ep_size = 1`` and the same ``moe_implementation`` loads)."""
    sd = dict(torch.load(os.path.join(d, "model.pt"), map_location="cpu", weights_only=False))
    shards: Dict[int, Dict[str, torch.Tensor]] = {}
    ep_size = 1
    for name in sorted(os.listdir(d)):
        if re.fullmatch(r"experts-rank\d+\.pt", name):
            ex = torch.load(os.path.join(d, name), map_location="cpu", weights_only=False)
            ep_size = ex["ep_size"]
            shards.setdefault(ex["ep_rank"], ex["params"])      # replicas of a shard are identical
    assert sorted(shards) == list(range(ep_size)), f"expert shards present: {sorted(shards)} of {ep_size}"
    for n in shards.get(0, {}):
        sd[n] = torch.cat([shards[r][n] for r in range(ep_size)], dim=0)
    return sd


def save_param_sharded(root: str, step: int, plan, training_state: Dict, rank: int, keep: int = 3,
                       writer: Optional["AsyncCheckpointWriter"] = None, ep_rank: int = 0, ep_size: int = 1) -> str:
    """Checkpoint of the parameter-sharded plan: every rank helps gather the full parameters (rank 0
    writes them as an ordinary ``model.pt``) and writes its own shards with their AdamW moments; under
    expert parallelism also its ``experts-rank{r}.pt``.  ``plan``: the sharded plan or a ``ParallelPlan``
    of it and the expert pool.  ``writer``: files are written in the background (the gather itself stays
    collective)."""
    import torch.distributed as dist
    d = os.path.join(root, f"checkpoint-{step}")
    os.makedirs(d, exist_ok=True)
    fsdp, expert_pool = _pools(plan)
    full = fsdp.full_state_dict(to_cpu=True)
    files: Dict[str, Any] = {os.path.join(d, f"shards-rank{rank}.pt"): fsdp.shard_state_dict()}
    ep_names = _expert_parallel_names(fsdp.model)
    if ep_names:
        esd = {n: p.detach() for n, p in unwrap_model(fsdp.model).named_parameters() if n in set(ep_names)}
        files[os.path.join(d, f"experts-rank{rank}.pt")] = _expert_file(esd, ep_names, expert_pool, ep_rank, ep_size)
    if rank == 0:
        _write_manifest(d, "param_sharded", fsdp.world, _expected_files("shards", fsdp.world, bool(ep_names)))
        files[os.path.join(d, "model.pt")] = full
        files[os.path.join(d, "training_state.pt")] = training_state
    if writer is not None:
        writer.submit(files, d, rank,
                      then=(lambda: prune_checkpoints(root, keep, world=fsdp.world)) if rank == 0 else None)
        return d
    for path, obj in files.items():
        _atomic_save(obj, path)
    _mark_complete(d, rank)
    if dist.is_available() and dist.is_initialized():
        dist.barrier()
    if rank == 0:
        prune_checkpoints(root, keep, world=fsdp.world)
    return d


def load_param_sharded(d: str, plan, rank: int, ep_rank: int = 0, ep_size: int = 1) -> Dict:
    """Restores shards and moments when the file of this rank matches the current layout, otherwise the
    parameters alone from ``model.pt`` (any world size); experts from this rank's expert file."""
    fsdp, expert_pool = _pools(plan)
    f = os.path.join(d, f"shards-rank{rank}.pt")
    done = False
    if os.path.exists(f):
        sd = torch.load(f, map_location="cpu", weights_only=False)
        if sd.get("world") == fsdp.world and sd.get("rank") == fsdp.rank:
            fsdp.load_shard_state_dict(sd)
            done = True
    if not done:
        fsdp.load_full_state_dict(torch.load(os.path.join(d, "model.pt"), map_location="cpu", weights_only=False))
    if _expert_parallel_names(fsdp.model):
        _load_expert_file(d, rank, unwrap_model(fsdp.model), expert_pool, ep_rank, ep_size)
    ts = os.path.join(d, "training_state.pt")
    return torch.load(ts, map_location="cpu", weights_only=False) if os.path.exists(ts) else {}


def snapshot_to_host(obj):
    """Deep copy of a (nested) state object with every tensor on the host.  Device tensors are copied
    into pinned memory without blocking the host; the caller synchronises once before reading them."""
    if torch.is_tensor(obj):
        if obj.device.type == "cuda":
            dst = torch.empty(obj.shape, dtype=obj.dtype, device="cpu", pin_memory=True)
            dst.copy_(obj.detach(), non_blocking=True)
            return dst
        return obj.detach().clone()
    if isinstance(obj, dict):
        return type(obj)((k, snapshot_to_host(v)) for k, v in obj.items())
    if isinstance(obj, (list, tuple)):
        return type(obj)(snapshot_to_host(v) for v in obj)
    return copy.deepcopy(obj)


class AsyncCheckpointWriter:
    """Checkpoint files written off the training thread.

    ``submit`` copies the state to (pinned) host memory - the only part the training loop waits for, one
    device-to-host pass - and a background thread serialises it, each file through a temporary name, and
    finally drops a ``complete-rank{r}`` marker into the checkpoint directory.  A directory counts as a
    checkpoint only when every rank's marker is there (``checkpoint_complete``), so a job killed in the
    middle of a save resumes from the previous one.  One save is in flight at a time: a second ``submit``
    first waits for the first.  An error in the writer thread is raised by the next ``submit`` / ``wait``."""

    def __init__(self):
        self._thread: Optional[threading.Thread] = None
        self._error: Optional[BaseException] = None

    def wait(self) -> None:
        if self._thread is not None:
            self._thread.join()
            self._thread = None
        if self._error is not None:
            e, self._error = self._error, None
            raise RuntimeError(f"asynchronous checkpoint write failed: {e!r}") from e

    def submit(self, files: Dict[str, Any], directory: str, rank: int, then=None) -> None:
        """``files``: path -> state object.  ``then`` runs in the writer thread after the marker exists."""
        self.wait()
        host = {path: snapshot_to_host(obj) for path, obj in files.items()}
        if torch.cuda.is_available():
            torch.cuda.current_stream().synchronize()

        def run():
            try:
                for path, obj in host.items():
                    _atomic_save(obj, path)
                _mark_complete(directory, rank)
                if then is not None:
                    then()
            except BaseException as e:       # surfaced by wait()
                self._error = e

        self._thread = threading.Thread(target=run, daemon=False)
        self._thread.start()


def checkpoint_complete(d: str, world: int) -> bool:
    """Whether ``d`` holds a finished checkpoint.

    A multi-rank directory starts with rank 0's manifest (its writer count and expected files) and is
    complete when every rank named there has dropped its ``complete-rank{r}`` marker - each rank's
    last write - and every expected file exists.  The writer count comes from the manifest, not from
    ``world``: a job restarted on fewer ranks must still recognise what the larger job wrote.
    A directory with per-rank files or markers but no manifest is a save that rank 0 has not begun
    (or one cut off before the manifest): incomplete.  A directory without any per-rank file is the
    single-writer layout (``save_format_c``), whose last file is ``training_state.pt``."""
    if not os.path.isdir(d):
        return False
    names = set(os.listdir(d))
    man = read_manifest(d)
    if man is not None:
        return all(m in names for m in man.get("markers", [])) and all(f in names for f in man.get("files", []))
    if any(re.fullmatch(r"(complete-rank\d+|(optimizer|shards|experts)-rank\d+\.pt(\.tmp)?)", n) for n in names):
        return False
    return "training_state.pt" in names


def latest_complete_checkpoint(root: str, world: int = 1) -> Optional[str]:
    best = None
    if os.path.isdir(root):
        for name in os.listdir(root):
            m = re.fullmatch(r"checkpoint-(\d+)", name)
            d = os.path.join(root, name)
            if m and checkpoint_complete(d, world) and (best is None or int(m.group(1)) > best[0]):
                best = (int(m.group(1)), d)
    return best[1] if best else None


def _atomic_save(obj, path: str) -> None:
    os.makedirs(os.path.dirname(os.path.abspath(path)), exist_ok=True)
    tmp = path + ".tmp"
    torch.save(obj, tmp)
    os.replace(tmp, path)
