"""Sharded data parallelism with whole-tensor ownership.

The reference shards everything FSDP-style (FULL_SHARD per ``TransformerBlock``: bf16
all-gather of every block's parameters in forward and again in backward, bf16
reduce-scatter of gradients; reference: train_distributed.py:275-319).  On a GPU with
180 GB of HBM the bf16 weights of the 5B model (11.7 GB) are cheap to replicate, so this
runtime keeps parameters replicated and shards only what is large and rank-private:
gradients after reduction and optimizer state.  Per step that is ONE reduce-scatter of the
flat gradient buffer and ONE all-gather of the updated parameters, instead of FSDP's two
all-gathers and one reduce-scatter per block.

Ownership is per tensor, not per flat byte range: every parameter (2-D matrices and 3-D
expert stacks included) belongs to exactly one rank, so Muon's Newton-Schulz runs on whole
matrices on the owner with no gather, and each rank orthogonalises only its share of the
matrices.  Rank r's tensors are packed into segment r of two flat buffers (parameters and
gradients) whose segments have equal size, AdamW-updated tensors first and Muon-updated
matrices after them.

Three transports for the two collectives:
* ``p2p`` (CUDA ranks with peer access): the buffers live in symmetric memory and this
  library's kernels do the work over NVLink peer pointers - the reduce-scatter is fused
  with the squared-norm reduction for clipping, and the AdamW update is fused with the
  all-gather (the kernel stores each new parameter into every rank's buffer).
* ``nccl``: ``reduce_scatter_tensor`` / ``all_gather_into_tensor``.
* ``gloo`` (CPU tests): all-reduce + slice, all-gather.

Gradient accumulation needs no ``no_sync`` bookkeeping: gradients accumulate locally in the
flat buffer and are reduced once, when the step is taken.
"""
from __future__ import annotations

import os

from typing import Dict, List, Optional, Tuple

import torch
import torch.distributed as dist

from ..training.muon_optimizer import _EXCLUDE, Muon
from ..training.optim_factory import make_adamw

_ALIGN = 128   # elements; keeps every tensor 256-byte aligned inside a segment


def _round_up(x: int, m: int) -> int:
    return (x + m - 1) // m * m


def assign_owners(numels: List[int], world: int) -> List[int]:
    """Greedy balance by element count: largest tensor first onto the lightest rank.
    Deterministic, so every rank computes the same assignment."""
    load = [0] * world
    owner = [0] * len(numels)
    for i in sorted(range(len(numels)), key=lambda j: (-numels[j], j)):
        r = min(range(world), key=lambda q: (load[q], q))
        owner[i] = r
        load[r] += _round_up(numels[i], _ALIGN)
    return owner


def is_muon_param(name: str, p: torch.Tensor) -> bool:
    nl = name.lower()
    return p.dim() == 2 and ".weight" in nl and not any(t in nl for t in _EXCLUDE)


class FusedAdamW:
    """AdamW over one contiguous range of a flat bf16 buffer with fp32 moments, run by the
    ``p2p_adamw_allgather`` kernel: clip coefficient read on the device, result stored into
    every buffer in ``param_ptrs`` (all ranks under p2p, only this rank otherwise)."""

    def __init__(self, flat_param, flat_grad, start: int, n: int, lr, betas=(0.9, 0.95), eps=1e-8,
                 weight_decay=0.01):
        self.flat_param, self.flat_grad, self.start, self.n = flat_param, flat_grad, start, n
        self.m = torch.zeros(n, dtype=torch.float32, device=flat_param.device)
        self.v = torch.zeros(n, dtype=torch.float32, device=flat_param.device)
        self.param_groups = [dict(lr=lr, betas=tuple(betas), eps=eps, weight_decay=weight_decay, params=[])]
        self.step_count = 0

    def step(self, param_ptrs: List[int], rank: int, clip_coef: Optional[torch.Tensor], mc_ptr: int = 0):
        from ..ops import cuda_ops
        g = self.param_groups[0]
        self.step_count += 1
        torch.ops.kmoe.p2p_adamw_allgather(param_ptrs, self.flat_grad, self.m, self.v, rank, len(param_ptrs),
                                           self.start, self.n, g["lr"], g["betas"][0], g["betas"][1], g["eps"],
                                           g["weight_decay"], self.step_count, clip_coef, mc_ptr)
        cuda_ops._count()

    def state_dict(self):
        return {"m": self.m, "v": self.v, "step": self.step_count,
                "hyper": {k: v for k, v in self.param_groups[0].items() if k != "params"}}

    def load_state_dict(self, sd):
        self.m.copy_(sd["m"])
        self.v.copy_(sd["v"])
        self.step_count = sd["step"]


class ShardedDataParallel:
    def __init__(self, model: torch.nn.Module, optimizer_kind: str = "muon", group=None,
                 lr: float = 1e-3, adamw_lr: float = 3e-4, momentum: float = 0.95,
                 weight_decay: float = 0.01, newton_iters: int = 5, transport: Optional[str] = None,
                 broadcast_from_rank0: bool = True, expert_params: bool = False, grad_scale: float = 1.0,
                 fused_adamw: Optional[bool] = None):
        """``expert_params=False``: all parameters except expert-parallel ones (``group`` = every
        data-parallel rank).  ``expert_params=True``: only the expert-parallel tensors, with
        ``group`` the ranks that hold replicas of the same experts and ``grad_scale = 1/ep``
        (an expert's gradient already sums the losses of the ep ranks that sent it tokens).
        ``transport``: ``p2p`` | ``nccl`` | ``gloo`` | None (= p2p when available)."""
        self.model, self.group = model, group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.grad_scale = grad_scale
        self.kind = optimizer_kind
        named: List[Tuple[str, torch.nn.Parameter]] = []
        seen = set()
        for n, p in model.named_parameters():
            if p.requires_grad and id(p) not in seen and \
                    bool(getattr(p, "_kmoe_expert_parallel", False)) == expert_params:
                seen.add(id(p))
                named.append((n, p))
        assert named, "no trainable parameters"
        self.named = named
        dtype, device = named[0][1].dtype, named[0][1].device
        assert all(p.dtype == dtype for _, p in named), "parameters must share one dtype"
        self.dtype, self.device = dtype, device
        muon_flag = [optimizer_kind == "muon" and is_muon_param(n, p) for n, p in named]
        owners = assign_owners([p.numel() for _, p in named], self.world)
        # segment layout: AdamW tensors first, Muon matrices after them; inside each part the tensors
        # are placed in reverse module order, which is the order their gradients are finished by the
        # backward pass - so "everything from the output down to layer l" is a prefix of both parts
        # and can be reduced while the backward pass is still working on the earlier layers
        offsets = [0] * self.world
        self.slots: List[Optional[Tuple[int, int]]] = [None] * len(named)
        for want_muon in (False, True):
            if want_muon:
                self.adamw_end = list(offsets)
            for i in reversed(range(len(named))):
                (n, p), r = named[i], owners[i]
                if muon_flag[i] == want_muon:
                    self.slots[i] = (r, offsets[r])
                    offsets[r] += _round_up(p.numel(), _ALIGN)
        self.used = list(offsets)
        self.seg = _round_up(max(offsets), _ALIGN)
        total = self.seg * self.world

        self.transport = self._pick_transport(transport)
        self.p2p = None
        if self.transport == "p2p":
            from .p2p import SymmetricBuffers
            try:
                self.p2p = SymmetricBuffers(total, dtype, device, group)
            except Exception as e:                      # no peer mapping on this machine: use the library collectives
                if transport == "p2p":
                    raise
                print(f"[kmoe] symmetric-memory set-up failed ({type(e).__name__}: {e}); using NCCL collectives", flush=True)
                self.p2p = None
            # every rank must take the same branch
            flag = torch.tensor([1.0 if self.p2p is not None else 0.0], device=device)
            dist.all_reduce(flag, op=dist.ReduceOp.MIN, group=group)
            if flag.item() == 0.0:
                self.p2p = None
                self.transport = "nccl" if dist.get_backend(group) == "nccl" else "gloo"
        if self.transport == "p2p":
            self.flat_param, self.flat_grad = self.p2p.param, self.p2p.grad
        else:
            self.flat_param = torch.zeros(total, dtype=dtype, device=device)
            self.flat_grad = torch.zeros(total, dtype=dtype, device=device)
        with torch.no_grad():
            for (n, p), (r, off) in zip(named, self.slots):
                a = r * self.seg + off
                view = self.flat_param[a: a + p.numel()].view_as(p)
                view.copy_(p.data)
                p.data = view
                p.grad = self.flat_grad[a: a + p.numel()].view_as(p)
        self._setup_grad_landing()
        if broadcast_from_rank0 and self.world > 1:
            dist.broadcast(self.flat_param, src=dist.get_global_rank(group, 0) if group is not None else 0,
                           group=group)
        self.owned = [(n, p) for (n, p), (r, _) in zip(named, self.slots) if r == self.rank]
        self.owned_muon = [(n, p) for i, ((n, p), (r, _)) in enumerate(zip(named, self.slots))
                           if r == self.rank and muon_flag[i]]
        self.owned_adamw = [(n, p) for i, ((n, p), (r, _)) in enumerate(zip(named, self.slots))
                            if r == self.rank and not muon_flag[i]]
        if fused_adamw is None:
            fused_adamw = device.type == "cuda" and dtype == torch.bfloat16
        self.fused: Optional[FusedAdamW] = None
        self.muon: Optional[Muon] = None
        self.adamw = None
        my_adamw_n = self.adamw_end[self.rank] if optimizer_kind == "muon" else self.used[self.rank]
        if optimizer_kind == "muon" and self.owned_muon:
            self.muon = Muon([p for _, p in self.owned_muon], lr=lr, momentum=momentum, weight_decay=weight_decay,
                             newton_iters=newton_iters)
        if fused_adamw and my_adamw_n > 0:
            self.fused = FusedAdamW(self.flat_param, self.flat_grad, self.rank * self.seg, my_adamw_n, adamw_lr,
                                    weight_decay=weight_decay)
        elif self.owned_adamw:
            self.adamw = make_adamw([p for _, p in self.owned_adamw], adamw_lr, weight_decay=weight_decay)
        self.optimizer = _PoolOptimizer(self)
        self._clip: Optional[torch.Tensor] = None
        self._side_stream = None
        self._sq = torch.zeros(1, dtype=torch.float32, device=device)
        self._sync = True
        self._setup_overlap(named, muon_flag, int(os.environ.get("KMOE_RS_CHUNKS", "6")))

    # ------------------------------------------------ gradients land in the flat buffer without an add
    def _setup_grad_landing(self) -> None:
        """With ``p.grad`` pointing into the flat buffer autograd *adds* every new gradient to it, which
        costs a zero-fill of the buffer plus a read-modify-write per tensor per step.  Instead ``p.grad``
        starts each step as None: autograd then hands over the freshly computed gradient, and a
        post-accumulate hook copies it to the tensor's place in the flat buffer (one read, one write)
        and points ``p.grad`` there, so further micro-batches accumulate in place.  Ops that can write
        their weight gradient straight into the flat buffer ask ``ops.cuda_ops.grad_sink`` for the
        destination and skip even the copy."""
        self._views: Dict[int, torch.Tensor] = {}
        self._touched: set = set()
        self._landing = self.device.type == "cuda" and os.environ.get("KMOE_GRAD_LANDING", "1") != "0"
        if not self._landing:
            return
        from ..ops import cuda_ops
        # A parameter held by more than one module (tied embedding / output head) gets gradient from several nodes
        # of the graph: it must go through autograd's accumulation, which calls the hooks once with the sum.  A
        # direct write by the first op would mark it ready before the later contributions exist.
        shared = shared_parameter_ids(self.model)
        for (n, p) in self.named:
            self._views[id(p)] = p.grad
            p.grad = None
            p.register_post_accumulate_grad_hook(self._land)
            if id(p) not in shared:
                cuda_ops.register_grad_sink(p, self._views[id(p)], self._sink_commit)

    def _land(self, p) -> None:
        v = self._views[id(p)]
        if p.grad is not None and p.grad.data_ptr() != v.data_ptr():
            v.copy_(p.grad)
            p.grad = v
        self._touched.add(id(p))

    def _sink_commit(self, p) -> None:
        """An op wrote this parameter's gradient directly into the flat buffer."""
        p.grad = self._views[id(p)]
        self._touched.add(id(p))
        self._grad_ready(p)

    def _clear_grads(self) -> None:
        if self._landing:
            for (_, p) in self.named:
                p.grad = None
            self._touched.clear()
        else:
            self.flat_grad.zero_()

    def _zero_untouched(self) -> None:
        """Parameters that received no gradient this step still hold last step's values in the buffer."""
        if self._landing and len(self._touched) != len(self.named):
            for (_, p) in self.named:
                if id(p) not in self._touched:
                    self._views[id(p)].zero_()
                    p.grad = self._views[id(p)]

    # ------------------------------------------------ reduce-scatter overlapped with the backward pass
    def _setup_overlap(self, named, muon_flag, n_chunks: int) -> None:
        """Split the tensors, in the order the backward pass finishes them, into ``n_chunks`` groups of
        about equal size.  For this rank every group is one range of its AdamW part and one of its Muon
        part; a group is reduced (own kernel, side stream) as soon as its last gradient has been
        accumulated on every rank, while the backward pass continues below it."""
        self._chunks: List[List[Tuple[int, int]]] = []
        self._chunk_of: Dict[int, int] = {}
        self._pending: List[int] = []
        self._ready_seen: set = set()
        self._launched = 0
        self._rs_stream = None
        # measured at 2 GPUs the overlap costs more than the 4 ms it hides, so it is on from 4 ranks
        # (KMOE_RS_OVERLAP=1/0 forces it)
        want = os.environ.get("KMOE_RS_OVERLAP", "auto")
        if self.transport != "p2p" or n_chunks <= 1 or want == "0" or (want == "auto" and self.world < 4):
            return
        order = list(reversed(range(len(named))))                      # backward completion order
        total = sum(named[i][1].numel() for i in order)
        bounds, acc, k = [], 0, 0
        group_of = {}
        for i in order:
            group_of[i] = k
            acc += named[i][1].numel()
            if acc >= total * (k + 1) / n_chunks and k < n_chunks - 1:
                k += 1
        n_groups = max(group_of.values()) + 1
        ranges: List[List[Tuple[int, int]]] = [[] for _ in range(n_groups)]
        for want_muon in (False, True):
            lo = [None] * n_groups
            hi = [None] * n_groups
            for i in order:
                r, off = self.slots[i]
                if r != self.rank or muon_flag[i] != want_muon:
                    continue
                g = group_of[i]
                a = r * self.seg + off
                b = a + _round_up(named[i][1].numel(), _ALIGN)
                lo[g] = a if lo[g] is None else min(lo[g], a)
                hi[g] = b if hi[g] is None else max(hi[g], b)
            for g in range(n_groups):
                if lo[g] is not None:
                    ranges[g].append((lo[g], hi[g] - lo[g]))
        self._chunks = ranges
        self._group_sizes = [0] * n_groups
        for i in range(len(named)):
            self._group_sizes[group_of[i]] += 1
            self._chunk_of[id(named[i][1])] = group_of[i]
            named[i][1].register_post_accumulate_grad_hook(self._grad_ready)
        self._pending = list(self._group_sizes)
        self._rs_stream = torch.cuda.Stream(device=self.device)

    def _grad_ready(self, p) -> None:
        if not self._sync or not self._chunks:
            return
        g = self._chunk_of.get(id(p))
        if g is None:
            return
        if id(p) in self._ready_seen:
            # A group is reduced as soon as its last tensor is complete; a tensor that is completed twice (a
            # second backward pass without set_sync(False) before it, or a weight that two nodes of the graph
            # write, the first of them directly into the flat buffer) would let its group go early.
            name = next((n for n, q in self.named if q is p), "?")
            raise RuntimeError(f"gradient of {name} was marked complete twice in one step: accumulate "
                               f"micro-batches under set_sync(False), and keep weights that several modules "
                               f"use out of the direct gradient destinations")
        self._ready_seen.add(id(p))
        self._pending[g] -= 1
        while self._launched < len(self._chunks) and self._pending[self._launched] <= 0:
            self._launch_chunk(self._launched)
            self._launched += 1

    def _launch_chunk(self, g: int) -> None:
        """Side stream: wait for the gradients enqueued so far, meet the other ranks, reduce this rank's
        ranges of the group (mean over ranks, squared norm accumulated for clipping)."""
        ev = torch.cuda.Event()
        ev.record(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(self._rs_stream):
            self._rs_stream.wait_event(ev)
            self.p2p.barrier(channel=1)
            for off, n in self._chunks[g]:
                self.p2p.reduce_scatter_mean(off, n, self._sq, max_blocks=self._rs_blocks(g))

    def _rs_blocks(self, g: int) -> int:
        # while the backward pass is running the reduction gets a fraction of the SMs; the last group
        # (nothing left to overlap with) gets the whole device
        return 0 if g == len(self._chunks) - 1 else 48

    # ------------------------------------------------------------------ set-up
    def _pick_transport(self, want: Optional[str]) -> str:
        if self.world == 1:
            return "local"
        backend = dist.get_backend(self.group)
        if want in ("nccl", "gloo"):
            return want
        if self.device.type == "cuda" and want in (None, "p2p"):
            try:
                from .p2p import p2p_available
                if p2p_available(self.device):
                    return "p2p"
            except Exception:
                pass
            if want == "p2p":
                raise RuntimeError("p2p transport requested but symmetric memory is unavailable")
        return "nccl" if backend == "nccl" else "gloo"

    # -------------------------------------------------------------------- step
    def set_sync(self, flag: bool) -> None:
        """False while accumulating micro-batches: gradients are only reduced after the last one."""
        self._sync = bool(flag)

    def own_slice(self, flat: torch.Tensor) -> torch.Tensor:
        return flat[self.rank * self.seg: (self.rank + 1) * self.seg]

    def reduce(self) -> None:
        """Average gradients over the group into their owners' segments."""
        self._zero_untouched()
        self._sq_valid = False
        if self.transport == "p2p" and self._chunks:
            # groups whose last gradient arrived during the backward pass are already reduced (or in flight)
            while self._launched < len(self._chunks):
                self._launch_chunk(self._launched)
                self._launched += 1
            torch.cuda.current_stream(self.device).wait_stream(self._rs_stream)
            self._sq_valid = self.grad_scale == 1.0
        elif self.transport == "p2p":
            self.p2p.barrier()
            self._sq.zero_()
            self.p2p.reduce_scatter_mean(self.rank * self.seg, self.seg, self._sq)
            self._sq_valid = self.grad_scale == 1.0
        elif self.transport == "nccl":
            dist.reduce_scatter_tensor(self.own_slice(self.flat_grad), self.flat_grad, op=dist.ReduceOp.AVG,
                                       group=self.group)
        elif self.transport == "gloo":
            dist.all_reduce(self.flat_grad, group=self.group)
            self.flat_grad.div_(self.world)
        if self.grad_scale != 1.0:
            self.own_slice(self.flat_grad).mul_(self.grad_scale)

    def owned_sq_norm(self) -> torch.Tensor:
        if getattr(self, "_sq_valid", False):
            return self._sq[0]
        seg = self.own_slice(self.flat_grad)
        if seg.is_cuda and seg.dtype == torch.bfloat16 and seg.data_ptr() % 16 == 0 and hasattr(torch.ops, "kmoe") \
                and hasattr(torch.ops.kmoe, "sumsq"):
            return torch.ops.kmoe.sumsq(seg)[0]              # one pass, fp32 accumulation, fixed summation order
        # fused fp32-accumulating reduction: no fp32 copy of the gradient segment is materialised
        return torch.linalg.vector_norm(seg, dtype=torch.float32).pow(2)

    def scale_owned(self, coef: torch.Tensor) -> None:
        """Apply the clip coefficient: the fused AdamW kernel reads it from the device; only
        the gradients of the other optimizers are rescaled in memory."""
        self._clip = coef.reshape(1).float().contiguous()
        a0 = self.rank * self.seg
        if self.fused is not None:
            lo = a0 + self.fused.n
        else:
            lo = a0
        hi = a0 + self.used[self.rank]
        if self.fused is not None and self.muon is not None and self.adamw is None:
            # everything outside the fused AdamW range belongs to Muon, whose kernels take the coefficient as
            # they read the gradients: no pass over the gradients in memory
            self.muon.grad_coef = self._clip
        elif hi > lo:
            self.flat_grad[lo:hi].mul_(coef.to(self.flat_grad.dtype))

    def finish(self) -> None:
        # parameters are rewritten through raw pointers below: drop derived copies (quantised weights)
        from ..ops import mxfp8
        mxfp8.invalidate_weight_cache()
        a0 = self.rank * self.seg
        ptrs = self.p2p.param_ptrs if self.transport == "p2p" else [self.flat_param.data_ptr()]
        prank = self.rank if self.transport == "p2p" else 0
        mc = self.p2p.param_mc if self.transport == "p2p" else 0
        # The fused AdamW kernel is HBM-bound and Muon's Newton-Schulz is tensor-core-bound: run them
        # on two streams so they overlap (they touch disjoint ranges of the flat buffers).
        side = None
        if (self.fused is not None and self.muon is not None and self.device.type == "cuda"
                and os.environ.get("KMOE_OPT_OVERLAP", "1") != "0"):
            if self._side_stream is None:
                self._side_stream = torch.cuda.Stream(device=self.device)
            side = self._side_stream
            side.wait_stream(torch.cuda.current_stream(self.device))
            with torch.cuda.stream(side):
                self.fused.step(ptrs, prank, self._clip, mc)
        elif self.fused is not None:
            self.fused.step(ptrs, prank, self._clip, mc)
        if self.adamw is not None:
            self.adamw.step()
        if self.muon is not None:
            self.muon.step()
        if side is not None:
            torch.cuda.current_stream(self.device).wait_stream(side)
        if self.transport == "p2p":
            lo = a0 + (self.fused.n if self.fused is not None else 0)
            hi = a0 + self.used[self.rank]
            if hi > lo:
                self.p2p.all_gather_range(lo, _round_up(hi - lo, 8))
            self.p2p.barrier()
        elif self.transport == "nccl":
            dist.all_gather_into_tensor(self.flat_param, self.own_slice(self.flat_param), group=self.group)
        elif self.transport == "gloo":
            dist.all_gather_into_tensor(self.flat_param, self.own_slice(self.flat_param).clone(), group=self.group)
        self._clear_grads()
        self._clip = None
        if self._chunks:                                  # re-arm the overlapped reduction for the next backward
            self._sq.zero_()
            self._pending = list(self._group_sizes)
            self._ready_seen.clear()
            self._launched = 0

    def reduce_clip_and_step(self, optimizer=None, max_norm: Optional[float] = 1.0) -> torch.Tensor:
        """Reduce gradients to their owners, clip by the global norm, update the owned
        tensors, publish them, and clear the gradient buffer.  Returns the global gradient
        norm (device tensor)."""
        return ParallelPlan([self]).reduce_clip_and_step(optimizer, max_norm)

    # ------------------------------------------------------------- checkpoints
    def owned_names(self) -> List[str]:
        return [n for n, _ in self.owned]

    def optimizer_state_dict(self) -> Dict:
        """State of this rank's shard plus the names it covers (for sharded checkpoints)."""
        return {"rank": self.rank, "world": self.world, "owned": self.owned_names(),
                "fused_adamw": self.fused.state_dict() if self.fused is not None else None,
                "adamw": self.adamw.state_dict() if self.adamw is not None else None,
                "muon": self.muon.state_dict() if self.muon is not None else None}

    def load_optimizer_state_dict(self, sd: Dict) -> None:
        assert sd["owned"] == self.owned_names(), "optimizer shard does not match this rank's ownership"
        if self.fused is not None and sd.get("fused_adamw") is not None:
            self.fused.load_state_dict(sd["fused_adamw"])
        if self.adamw is not None and sd.get("adamw") is not None:
            self.adamw.load_state_dict(sd["adamw"])
        if self.muon is not None and sd.get("muon") is not None:
            self.muon.load_state_dict(sd["muon"])


def shared_parameter_ids(model: torch.nn.Module) -> set:
    """``id`` of every parameter that more than one module of ``model`` holds (tied weights)."""
    uses: Dict[int, int] = {}
    for m in model.modules():
        for q in m._parameters.values():
            if q is not None:
                uses[id(q)] = uses.get(id(q), 0) + 1
    return {k for k, c in uses.items() if c > 1}


class _PoolOptimizer:
    """Optimizer-shaped view of a pool (``param_groups`` for LR schedulers, state dicts)."""

    def __init__(self, pool: ShardedDataParallel):
        self.pool = pool

    @property
    def param_groups(self):
        out = []
        for o in (self.pool.muon, self.pool.adamw, self.pool.fused):
            if o is not None:
                out.extend(o.param_groups)
        return out

    def state_dict(self):
        return self.pool.optimizer_state_dict()

    def load_state_dict(self, sd):
        self.pool.load_optimizer_state_dict(sd)

    def zero_grad(self, set_to_none: bool = False):
        self.pool._clear_grads()

    def step(self):
        raise RuntimeError("step through ShardedDataParallel.reduce_clip_and_step")


class ParallelPlan:
    """One or more parameter pools (dense parameters over all ranks; expert-parallel
    parameters over their replica group) stepped together with a single global-norm clip."""

    def __init__(self, pools: List[ShardedDataParallel], norm_group=None):
        self.pools, self.norm_group = pools, norm_group
        self.optimizer = pools[0].optimizer

    def set_sync(self, flag: bool) -> None:
        for p in self.pools:
            p.set_sync(flag)

    def reduce_clip_and_step(self, optimizer=None, max_norm: Optional[float] = 1.0) -> torch.Tensor:
        for p in self.pools:
            p.reduce()
        sq = sum(p.owned_sq_norm() for p in self.pools).reshape(1).clone()
        if dist.is_initialized() and dist.get_world_size(self.norm_group) > 1:
            dist.all_reduce(sq, group=self.norm_group)
        total = sq.sqrt()[0]
        if max_norm is not None and max_norm > 0:
            coef = (max_norm / (total + 1e-6)).clamp(max=1.0)
            for p in self.pools:
                p.scale_owned(coef)
        for p in self.pools:
            p.finish()
        return total

    @property
    def param_groups(self):
        return [g for p in self.pools for g in p.optimizer.param_groups]
