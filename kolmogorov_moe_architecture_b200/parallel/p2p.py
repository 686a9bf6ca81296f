"""Symmetric-memory buffers and the peer-to-peer collectives built on them.

Buffers are allocated with ``torch.distributed._symmetric_memory`` (CUDA VMM allocations
whose handles are exchanged at rendezvous and mapped into every rank of the group), which
gives each rank a device pointer to every peer's copy.  The collectives themselves are this
library's kernels (``csrc/comm.cu``): plain 16-byte loads and stores through those peer
pointers over NVLink, never TMA multicast; on an NVSwitch system the reduce-scatter and the
parameter publication use the switch instead (``multimem.ld_reduce`` / ``multimem.st`` on the
buffers' multicast addresses), which moves ~1/world of the bytes through each GPU's port.  Cross-rank ordering uses a flag barrier whose
wait is bounded by a wall-clock limit; on expiry the kernel sets the status word that
``ops.cuda_ops.check_status`` reports, and the context stays usable.
"""
from __future__ import annotations

import os
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


def enable_group(name: str) -> None:
    """Older releases of the symmetric-memory module want a group registered before its first allocation;
    newer ones do it themselves and only warn about the call."""
    import warnings
    import torch.distributed._symmetric_memory as symm
    if hasattr(symm, "enable_symm_mem_for_group"):
        with warnings.catch_warnings():
            warnings.simplefilter("ignore")
            try:
                symm.enable_symm_mem_for_group(name)
            except Exception:
                pass


def _delta(handle, tensor, rank: int) -> int:
    """Byte offset of ``tensor`` inside its symmetric allocation (the allocator may sub-allocate)."""
    return int(tensor.data_ptr()) - int(handle.buffer_ptrs[rank])


def peer_ptrs(handle, tensor, rank: int) -> List[int]:
    """Device address of ``tensor``'s counterpart on every rank."""
    d = _delta(handle, tensor, rank)
    return [int(p) + d for p in handle.buffer_ptrs]


def multicast_ptr(handle, tensor, rank: int) -> int:
    """NVLink-switch multicast address of ``tensor`` (0 when the fabric offers none)."""
    try:
        base = int(handle.multicast_ptr or 0)
    except Exception:
        base = 0
    return base + _delta(handle, tensor, rank) if base else 0


class SymmetricBuffers:
    """Flat parameter and gradient buffers of ``total`` elements plus a flag array, all symmetric."""

    def __init__(self, total: int, dtype, device, group=None, barrier_timeout_s: float = 30.0):
        import torch.distributed._symmetric_memory as symm
        from ..ops import cuda_ops
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        name = _group_name(group)
        enable_group(name)
        self.param = symm.empty(total, dtype=dtype, device=device)
        self.grad = symm.empty(total, dtype=dtype, device=device)
        self.flags = symm.empty(64, dtype=torch.int32, device=device)
        self.param.zero_()
        self.grad.zero_()
        self.flags.zero_()
        torch.cuda.synchronize(device)
        self._h = [symm.rendezvous(t, name) for t in (self.param, self.grad, self.flags)]
        self.param_ptrs: List[int] = peer_ptrs(self._h[0], self.param, self.rank)
        self.grad_ptrs: List[int] = peer_ptrs(self._h[1], self.grad, self.rank)
        self.flag_ptrs: List[int] = peer_ptrs(self._h[2], self.flags, self.rank)
        # NVLink-switch multicast addresses of the two big buffers (0 = not available / switched off).
        # The switch path cuts the bytes a GPU receives and the loads it issues, not the bytes it must send.
        # Measured on the 5B step at 4 GPUs: as a stand-alone phase it is slower than plain peer loads
        # (194.9 ms against 188.2 ms per step), but under the overlapped reduce-scatter, where it takes fewer
        # issue slots from the backward pass, it is the fastest variant (186.0 ms; 188.4 ms with plain
        # loads).  Default: on from 4 ranks, where the overlap is on too.  KMOE_MULTIMEM=1/0 forces it;
        # NCCL_NVLS_ENABLE=0 also keeps every kernel on plain peer loads and stores.
        want = os.environ.get("KMOE_MULTIMEM", "auto")
        use_mc = (self.world > 1 and os.environ.get("NCCL_NVLS_ENABLE", "1") != "0"
                  and (want == "1" or (want == "auto" and self.world >= 4)))
        self.param_mc: int = multicast_ptr(self._h[0], self.param, self.rank) if use_mc else 0
        self.grad_mc: int = multicast_ptr(self._h[1], self.grad, self.rank) if use_mc else 0
        self.epoch = 0
        self.epochs = [0, 0, 0, 0]          # one counter per barrier channel (16 flag words each)
        self.timeout_s = barrier_timeout_s
        self.status = cuda_ops.status_tensor(device)
        dist.barrier(group=group)

    def barrier(self, channel: int = 0) -> None:
        """Flag barrier on the current stream.  Barriers issued on different streams must use different
        channels: each channel has its own flag words and epoch counter, so the order in which the
        streams' kernels actually run does not matter."""
        from ..ops import cuda_ops
        self.epochs[channel] += 1
        ptrs = [p + channel * 64 for p in self.flag_ptrs]
        torch.ops.kmoe.p2p_barrier(ptrs, self.rank, self.world, self.epochs[channel], self.timeout_s, self.status)
        cuda_ops._count()

    def reduce_scatter_mean(self, off: int, n: int, sq_out: Optional[torch.Tensor], max_blocks: int = 0) -> None:
        from ..ops import cuda_ops
        torch.ops.kmoe.p2p_reduce_scatter(self.grad_ptrs, self.rank, self.world, off, n, sq_out, self.grad_mc,
                                          max_blocks)
        cuda_ops._count()

    def all_gather_range(self, off: int, n: int, src: Optional[torch.Tensor] = None, max_blocks: int = 0) -> None:
        """Publish ``n`` elements at ``off`` of the parameter buffer to every rank: this rank's own copy of
        the range, or ``src`` (a bf16 vector outside the buffer, also stored into this rank's copy)."""
        from ..ops import cuda_ops
        torch.ops.kmoe.p2p_allgather(self.param_ptrs, self.rank, self.world, off, n, self.param_mc, src, max_blocks)
        cuda_ops._count()
