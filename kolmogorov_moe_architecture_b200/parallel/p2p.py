"""Symmetric-memory buffers and the peer-to-peer collectives built on them.

Buffers are allocated with ``torch.distributed._symmetric_memory`` (CUDA VMM allocations
whose handles are exchanged at rendezvous and mapped into every rank of the group), which
gives each rank a device pointer to every peer's copy.  The collectives themselves are this
library's kernels (``csrc/comm.cu``): plain 16-byte loads and stores through those peer
pointers over NVLink, never TMA multicast.  Cross-rank ordering uses a flag barrier whose
wait is bounded by a wall-clock limit; on expiry the kernel sets the status word that
``ops.cuda_ops.check_status`` reports, and the context stays usable.
"""
from __future__ import annotations

from typing import List, Optional

import torch
import torch.distributed as dist


def p2p_available(device) -> bool:
    if torch.device(device).type != "cuda" or not dist.is_initialized():
        return False
    try:
        import torch.distributed._symmetric_memory as symm  # noqa: F401
        return True
    except Exception:
        return False


def _group_name(group) -> str:
    g = group if group is not None else dist.group.WORLD
    return g.group_name


class SymmetricBuffers:
    """Flat parameter and gradient buffers of ``total`` elements plus a flag array, all symmetric."""

    def __init__(self, total: int, dtype, device, group=None, barrier_timeout_s: float = 30.0):
        import torch.distributed._symmetric_memory as symm
        from ..ops import cuda_ops
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        name = _group_name(group)
        if hasattr(symm, "enable_symm_mem_for_group"):
            try:
                symm.enable_symm_mem_for_group(name)
            except Exception:
                pass
        self.param = symm.empty(total, dtype=dtype, device=device)
        self.grad = symm.empty(total, dtype=dtype, device=device)
        self.flags = symm.empty(64, dtype=torch.int32, device=device)
        self.param.zero_()
        self.grad.zero_()
        self.flags.zero_()
        torch.cuda.synchronize(device)
        self._h = [symm.rendezvous(t, name) for t in (self.param, self.grad, self.flags)]
        self.param_ptrs: List[int] = [int(p) for p in self._h[0].buffer_ptrs]
        self.grad_ptrs: List[int] = [int(p) for p in self._h[1].buffer_ptrs]
        self.flag_ptrs: List[int] = [int(p) for p in self._h[2].buffer_ptrs]
        self.epoch = 0
        self.timeout_s = barrier_timeout_s
        self.status = cuda_ops.status_tensor(device)
        dist.barrier(group=group)

    def barrier(self) -> None:
        from ..ops import cuda_ops
        self.epoch += 1
        torch.ops.kmoe.p2p_barrier(self.flag_ptrs, self.rank, self.world, self.epoch, self.timeout_s, self.status)
        cuda_ops._count()

    def reduce_scatter_mean(self, off: int, n: int, sq_out: Optional[torch.Tensor]) -> None:
        from ..ops import cuda_ops
        torch.ops.kmoe.p2p_reduce_scatter(self.grad_ptrs, self.rank, self.world, off, n, sq_out)
        cuda_ops._count()

    def all_gather_range(self, off: int, n: int) -> None:
        from ..ops import cuda_ops
        torch.ops.kmoe.p2p_allgather(self.param_ptrs, self.rank, self.world, off, n)
        cuda_ops._count()
