"""Process-group bootstrap: one process per GPU, ``torch.distributed`` (NCCL) for plumbing,
a gloo group for host-side control traffic, and a dp x ep mesh.

The reference only ever uses the default (world) group and creates no sub-groups
(reference: train_distributed.py:196-207, moe_arch/model/moe.py:690,709).  Here the world
is factored as ``world = dp * ep``: ranks with the same ``rank // ep`` form an
expert-parallel group (tokens are exchanged inside it), ranks with the same ``rank % ep``
form the data-parallel group of the experts they hold; all ranks form the data-parallel
group of the non-expert parameters.
"""
from __future__ import annotations

import datetime
import os
from dataclasses import dataclass
from typing import Optional

import torch
import torch.distributed as dist


@dataclass
class Mesh:
    world: int
    rank: int
    local_rank: int
    ep: int
    dp: int
    world_group: Optional[object] = None
    ep_group: Optional[object] = None          # size ep
    expert_dp_group: Optional[object] = None   # size dp: replicas of the same expert shard
    control_group: Optional[object] = None     # gloo, host tensors

    @property
    def ep_rank(self) -> int:
        return self.rank % self.ep

    @property
    def dp_rank(self) -> int:
        return self.rank // self.ep


def init_distributed(backend: Optional[str] = None, ep_size: int = 1, timeout_s: int = 600,
                     with_control_group: bool = False) -> Mesh:
    """Initialise from the torchrun environment (RANK / LOCAL_RANK / WORLD_SIZE / MASTER_*).
    Single-process runs get a trivial mesh and no process group."""
    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world == 1 and not dist.is_initialized():
        if torch.cuda.is_available():
            torch.cuda.set_device(local)
        return Mesh(1, 0, local, 1, 1)
    if backend is None:
        backend = "nccl" if torch.cuda.is_available() else "gloo"
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29500")
    if not dist.is_initialized():
        kw = {}
        if backend == "nccl":
            torch.cuda.set_device(local)
            kw["device_id"] = torch.device("cuda", local)
        dist.init_process_group(backend, timeout=datetime.timedelta(seconds=timeout_s), **kw)
    return make_mesh(ep_size, with_control_group=with_control_group)


# Expert-parallel group of the most recent mesh; expert-parallel layers built afterwards split their
# experts over it (None = the world group, the reference's only choice).
_DEFAULT_EP = [None]


def default_ep_group():
    return _DEFAULT_EP[0]


def make_mesh(ep_size: int = 1, with_control_group: bool = False) -> Mesh:
    world, rank = dist.get_world_size(), dist.get_rank()
    local = int(os.environ.get("LOCAL_RANK", str(rank)))
    assert world % ep_size == 0, f"world size {world} not divisible by ep_size {ep_size}"
    dp = world // ep_size
    ep_group = expert_dp_group = None
    if ep_size > 1:
        for d in range(dp):                       # every rank must create every group
            grp = dist.new_group(list(range(d * ep_size, (d + 1) * ep_size)))
            if d == rank // ep_size:
                ep_group = grp
        for e in range(ep_size):
            grp = dist.new_group(list(range(e, world, ep_size)))
            if e == rank % ep_size:
                expert_dp_group = grp
    control = dist.new_group(backend="gloo") if with_control_group else None
    _DEFAULT_EP[0] = ep_group
    return Mesh(world, rank, local, ep_size, dp, dist.group.WORLD, ep_group, expert_dp_group, control)


def destroy():
    if dist.is_initialized():
        dist.destroy_process_group()
