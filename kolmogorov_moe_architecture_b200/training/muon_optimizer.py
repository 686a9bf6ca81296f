"""Muon optimizers and the hybrid Muon + AdamW wrappers
(reference: moe_arch/training/muon_optimizer.py:15-616, train.py:566-705).

Semantics kept from the reference, including the unusual ones:
* decoupled weight decay ``p *= 1 - lr * wd`` before the update;
* ``buf = momentum * buf + grad``; for >=2-D parameters ``buf`` is orthogonalised by
  the cubic Newton-Schulz iteration (Frobenius-normalised; 3-D = batch of matrices;
  >=4-D flattened to 2-D) and the orthogonalised matrix is **written back into the
  momentum buffer** (muon_optimizer.py:332,338,352);
* Nesterov update ``grad + momentum * buf``, then ``p -= lr * update``.
``standard_muon=True`` switches to the usual formulation (momentum buffer is not
overwritten; the update is the orthogonalised Nesterov direction).

The Newton-Schulz iteration goes through ``ops.newton_schulz`` (tcgen05 GEMM chain
on CUDA tensors); matrices of equal shape are stacked and orthogonalised in one
batched call instead of one Python-level iteration per parameter.
"""
from __future__ import annotations

import os
from typing import Optional

import torch
from torch.optim import Optimizer

from .. import ops


def _as_matrix_batch(t: torch.Tensor) -> torch.Tensor:
    if t.dim() == 2:
        return t.unsqueeze(0)
    if t.dim() == 3:
        return t
    return t.reshape(1, t.shape[0], -1)


def _qr_orthogonalize(m: torch.Tensor) -> torch.Tensor:
    if m.shape[0] <= m.shape[1]:
        q, _ = torch.linalg.qr(m.T.float())
        return q.T.to(m.dtype)
    q, _ = torch.linalg.qr(m.float())
    return q.to(m.dtype)


class Muon(Optimizer):
    def __init__(self, params, lr: float = 1e-3, momentum: float = 0.95, weight_decay: float = 0.01,
                 nesterov: bool = True, backend: str = "newton", newton_iters: int = 5,
                 standard_muon: bool = False):
        if lr < 0.0:
            raise ValueError(f"Invalid learning rate: {lr}")
        if momentum < 0.0 or momentum >= 1.0:
            raise ValueError(f"Invalid momentum: {momentum}")
        if weight_decay < 0.0:
            raise ValueError(f"Invalid weight_decay: {weight_decay}")
        super().__init__(params, dict(lr=lr, momentum=momentum, weight_decay=weight_decay,
                                      nesterov=nesterov, backend=backend, newton_iters=newton_iters,
                                      standard_muon=standard_muon))

    @staticmethod
    def _newton_schulz_orthogonalize(matrix: torch.Tensor, num_iters: int = 5) -> torch.Tensor:
        return ops.newton_schulz(matrix, num_iters)

    @staticmethod
    def _newton_schulz_orthogonalize_batched(matrices: torch.Tensor, num_iters: int = 5) -> torch.Tensor:
        return ops.newton_schulz(matrices, num_iters)

    def _bucket_state(self, group_idx: int, params):
        """Momentum of all >=2-D parameters of equal matrix shape lives in one stacked tensor
        (``state[p]['momentum_buffer']`` is a view of its slice), so momentum update, Newton-Schulz
        and write-back are a handful of launches per shape instead of several per parameter."""
        key = (group_idx, tuple(id(p) for p in params))
        cache = self.__dict__.setdefault("_buckets", {})
        if key in cache:
            return cache[key]
        buckets = {}
        for p in params:
            mb = _as_matrix_batch(p)
            buckets.setdefault((mb.shape[1], mb.shape[2], p.dtype, p.device), []).append(p)
        out = []
        for (m, n, dt, dev), ps in buckets.items():
            counts = [_as_matrix_batch(p).shape[0] for p in ps]
            stacked = torch.zeros(sum(counts), m, n, dtype=dt, device=dev)
            off = 0
            views = []
            for p, c in zip(ps, counts):
                v = stacked[off: off + c].view(p.shape)
                st = self.state[p]
                if "momentum_buffer" in st:                 # state loaded from a checkpoint
                    v.copy_(st["momentum_buffer"])
                st["momentum_buffer"] = v
                views.append(v)
                off += c
            out.append((stacked, ps, views))
        cache[key] = out
        return out

    @staticmethod
    def _fused_ok(stacked, ps, standard) -> bool:
        """The fused kernels cover the default rule on CUDA bf16 matrices whose sides are multiples of 64."""
        if standard or not stacked.is_cuda or stacked.dtype != torch.bfloat16:
            return False
        if os.environ.get("KMOE_MUON_FUSED", "1") == "0":
            return False
        if stacked.shape[1] % 64 or stacked.shape[2] % 64:
            return False
        from ..ops import ext_available
        return ext_available() and all(p.is_contiguous() and p.grad.is_contiguous() and p.grad.dtype == torch.bfloat16
                                       for p in ps)

    def _bucket_ptrs(self, stacked, ps):
        """Device arrays with the address of every matrix's gradient and parameter (rebuilt only when an
        address changes, e.g. after ``zero_grad(set_to_none=True)``)."""
        numel_b = stacked.shape[1] * stacked.shape[2] * stacked.element_size()
        sig = tuple((p.grad.data_ptr(), p.data_ptr()) for p in ps)
        cache = self.__dict__.setdefault("_ptr_cache", {})
        hit = cache.get(id(stacked))
        if hit is not None and hit[0] == sig:
            return hit[1], hit[2]
        gl, pl = [], []
        for p in ps:
            for e in range(_as_matrix_batch(p).shape[0]):
                gl.append(p.grad.data_ptr() + e * numel_b)
                pl.append(p.data_ptr() + e * numel_b)
        gp = torch.tensor(gl, dtype=torch.int64).to(stacked.device)
        pp = torch.tensor(pl, dtype=torch.int64).to(stacked.device)
        cache[id(stacked)] = (sig, gp, pp)
        return gp, pp

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for gi, group in enumerate(self.param_groups):
            lr, mu, wd = group["lr"], group["momentum"], group["weight_decay"]
            nesterov, backend, iters = group["nesterov"], group["backend"], group["newton_iters"]
            standard = group.get("standard_muon", False)
            live = [p for p in group["params"] if p.grad is not None]
            if not live:
                continue
            vecs = [p for p in live if p.dim() < 2]
            mats = [p for p in live if p.dim() >= 2]
            buckets = self._bucket_state(gi, mats) if (mats and backend != "qr") else []
            fused = [self._fused_ok(stacked, ps, standard) for stacked, ps, _ in buckets]
            in_fused = {id(p) for (b, ok) in zip(buckets, fused) if ok for p in b[1]}
            # a pending gradient coefficient (global-norm clip): the fused kernels apply it while reading the
            # gradient, everything else is scaled in memory
            coef = getattr(self, "grad_coef", None)
            if coef is not None:
                rest = [p.grad for p in live if id(p) not in in_fused]
                if rest:
                    torch._foreach_mul_(rest, coef.reshape(()).to(rest[0].dtype))
            if wd != 0:
                decay = [p for p in live if id(p) not in in_fused]      # fused buckets decay inside their kernel
                if decay:
                    torch._foreach_mul_(decay, 1 - lr * wd)
            for p in vecs:
                st = self.state[p]
                if "momentum_buffer" not in st:
                    st["momentum_buffer"] = torch.zeros_like(p.grad)
            if vecs:
                bufs = [self.state[p]["momentum_buffer"] for p in vecs]
                grads = [p.grad for p in vecs]
                torch._foreach_mul_(bufs, mu)
                torch._foreach_add_(bufs, grads)
                upd = torch._foreach_add(grads, bufs, alpha=mu) if nesterov else bufs
                torch._foreach_add_(vecs, upd, alpha=-lr)
            if not mats:
                continue
            if backend == "qr":
                for p in mats:
                    st = self.state[p]
                    if "momentum_buffer" not in st:
                        st["momentum_buffer"] = torch.zeros_like(p.grad)
                    buf, g = st["momentum_buffer"], p.grad
                    buf.mul_(mu).add_(g)
                    src = (g.add(buf, alpha=mu) if nesterov else buf) if standard else buf
                    mb = _as_matrix_batch(src)
                    o = torch.stack([_qr_orthogonalize(x) for x in mb]).reshape(buf.shape)
                    self._apply(p, g, buf, o, lr, mu, nesterov, standard)
                continue
            for (stacked, ps, views), ok in zip(buckets, fused):
                grads = [p.grad for p in ps]
                if ok:
                    # two elementwise passes in total: momentum (+ squared norms) before, parameter update after;
                    # the normalisation is folded into the first Newton-Schulz GEMMs
                    gp, pp = self._bucket_ptrs(stacked, ps)
                    sumsq = torch.zeros(stacked.shape[0], dtype=torch.float32, device=stacked.device)
                    torch.ops.kmoe.muon_momentum(stacked, gp, sumsq, mu, coef)
                    ortho = ops.newton_schulz(stacked, iters, sumsq=sumsq)
                    torch.ops.kmoe.muon_apply(stacked, ortho.contiguous(), gp, pp, lr, mu, wd, bool(nesterov), coef)
                    from ..ops import cuda_ops
                    cuda_ops._count(2)
                    continue
                stacked.mul_(mu)
                torch._foreach_add_(views, grads)
                if standard:
                    src = torch.cat([_as_matrix_batch(g.add(v, alpha=mu) if nesterov else v) for g, v in zip(grads, views)])
                    ortho = ops.newton_schulz(src, iters)
                    outs = torch.split(ortho, [_as_matrix_batch(p).shape[0] for p in ps])
                    torch._foreach_add_(ps, [o.reshape(p.shape).to(p.dtype) for o, p in zip(outs, ps)], alpha=-lr)
                    continue
                stacked.copy_(ops.newton_schulz(stacked, iters))     # the orthogonal factor replaces the momentum
                upd = torch._foreach_add(grads, views, alpha=mu) if nesterov else views
                torch._foreach_add_(ps, upd, alpha=-lr)
        self.grad_coef = None
        return loss

    @staticmethod
    def _apply(p, g, buf, ortho, lr, mu, nesterov, standard):
        if standard:
            p.add_(ortho.to(p.dtype), alpha=-lr)
            return
        buf.copy_(ortho)
        p.add_(g.add(buf, alpha=mu) if nesterov else buf, alpha=-lr)


class Muon8bit(Optimizer):
    """Muon with int8 momentum: per-``block_size`` absmax scales, values in [-127, 127]
    (reference: muon_optimizer.py:15-213).  First step seeds the buffer with the
    gradient.  1-D parameters longer than 1024 (flattened shards) are reshaped to
    their most-square factorisation before Newton-Schulz (141-155)."""

    def __init__(self, params, lr: float = 1e-3, momentum: float = 0.95, weight_decay: float = 0.01,
                 nesterov: bool = True, newton_iters: int = 5, use_8bit: bool = True, block_size: int = 2048):
        if lr < 0.0:
            raise ValueError(f"Invalid learning rate: {lr}")
        if momentum < 0.0 or momentum >= 1.0:
            raise ValueError(f"Invalid momentum: {momentum}")
        super().__init__(params, dict(lr=lr, momentum=momentum, weight_decay=weight_decay, nesterov=nesterov,
                                      newton_iters=newton_iters, use_8bit=use_8bit, block_size=block_size))
        self.use_8bit = use_8bit

    @staticmethod
    def _on_kernels(t: torch.Tensor) -> bool:
        """CUDA fp32 / bf16 tensors take the block-quantisation kernels (one pass each way) instead of the
        pad / view / amax / round chain below."""
        if not (t.is_cuda and t.dtype in (torch.float32, torch.bfloat16) and t.numel() > 0):
            return False
        from ..ops import ext_available
        return ext_available()

    @staticmethod
    def _quantize_to_8bit(t: torch.Tensor, block_size: int = 2048):
        if Muon8bit._on_kernels(t):
            q, scales = torch.ops.kmoe.q8_quant(t.contiguous(), block_size)
            return q, scales, t.shape, t.numel()
        shape, flat = t.shape, t.flatten()
        n = flat.numel()
        if n % block_size:
            flat = torch.nn.functional.pad(flat, (0, block_size - n % block_size))
        blocks = flat.view(-1, block_size)
        scales = blocks.abs().amax(dim=1, keepdim=True).clamp(min=1e-8)
        q = (blocks / scales * 127).round().to(torch.int8)
        return q, scales, shape, n

    @staticmethod
    def _dequantize_from_8bit(q, scales, shape, numel):
        return ((q.float() / 127) * scales).flatten()[:numel].view(shape)

    @staticmethod
    def _square_factor(n: int):
        r = int(n ** 0.5)
        while r > 1 and n % r:
            r -= 1
        return max(r, 1), n // max(r, 1)

    @staticmethod
    def _newton_schulz(matrix: torch.Tensor, num_iters: int = 5) -> torch.Tensor:
        return ops.newton_schulz(matrix, num_iters)

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            lr, mu, wd = group["lr"], group["momentum"], group["weight_decay"]
            for p in group["params"]:
                if p.grad is None:
                    continue
                g = p.grad
                if wd != 0:
                    p.mul_(1 - lr * wd)
                st = self.state[p]
                if group["use_8bit"]:
                    if "momentum_quantized" not in st:
                        buf = g.clone()
                    elif self._on_kernels(g) and g.is_contiguous():
                        # dequantise, decay and add the gradient in one pass
                        buf = torch.ops.kmoe.q8_momentum(st["momentum_quantized"], st["momentum_scales"], g, mu)
                    else:
                        buf = self._dequantize_from_8bit(st["momentum_quantized"], st["momentum_scales"],
                                                         st["momentum_shape"], st["momentum_numel"]).to(g)
                        buf.mul_(mu).add_(g)
                else:
                    if "momentum_buffer" not in st:
                        st["momentum_buffer"] = torch.zeros_like(g)
                    buf = st["momentum_buffer"]
                    buf.mul_(mu).add_(g)
                if p.dim() >= 2 or (p.dim() == 1 and p.numel() > 1024):
                    shape = buf.shape
                    if p.dim() == 1:
                        m2 = buf.view(*self._square_factor(buf.numel()))
                    elif p.dim() == 2:
                        m2 = buf
                    else:
                        m2 = buf.reshape(buf.shape[0], -1)
                    o = ops.newton_schulz(m2, group["newton_iters"]).reshape(shape)
                    if group["use_8bit"]:
                        buf = o
                    else:
                        buf.copy_(o)
                if group["use_8bit"]:
                    q, s, shp, n = self._quantize_to_8bit(buf, group["block_size"])
                    st["momentum_quantized"], st["momentum_scales"] = q, s
                    st["momentum_shape"], st["momentum_numel"] = shp, n
                p.add_(g.add(buf, alpha=mu) if group["nesterov"] else buf, alpha=-lr)
        return loss


_EXCLUDE = ("embedding", "embed", "lm_head", "head", "bias", "norm", "layernorm", "ln_", "scale")


class HybridOptimizer:
    """Muon on weight matrices + AdamW on the rest; ``state_dict`` is
    ``{'muon': ..., 'adamw': ...}`` (reference: muon_optimizer.py:578-614)."""

    def __init__(self, muon_opt: Optional[Optimizer], adamw_opt: Optional[Optimizer]):
        self.muon_opt, self.adamw_opt = muon_opt, adamw_opt

    def step(self, closure=None):
        for o in (self.muon_opt, self.adamw_opt):
            if o is not None:
                o.step()

    def zero_grad(self, set_to_none: bool = True):
        for o in (self.muon_opt, self.adamw_opt):
            if o is not None:
                o.zero_grad(set_to_none)

    def state_dict(self):
        return {"muon": self.muon_opt.state_dict() if self.muon_opt else None,
                "adamw": self.adamw_opt.state_dict() if self.adamw_opt else None}

    def load_state_dict(self, sd):
        if self.muon_opt and sd.get("muon"):
            self.muon_opt.load_state_dict(sd["muon"])
        if self.adamw_opt and sd.get("adamw"):
            self.adamw_opt.load_state_dict(sd["adamw"])

    @property
    def param_groups(self):
        groups = []
        for o in (self.muon_opt, self.adamw_opt):
            if o is not None:
                groups.extend(o.param_groups)
        return groups


def split_muon_params(model, fsdp_mode: Optional[bool] = None):
    """Name-based partition of the reference (muon_optimizer.py:498-537): names with
    embed/head/bias/norm/ln_/scale are excluded; Muon takes '.weight' tensors (and,
    outside sharded mode, only 2-D ones) - so stacked expert tensors ('w1' without
    '.weight') and conv kernels go to AdamW here."""
    if fsdp_mode is None:
        fsdp_mode = bool(os.environ.get("WORLD_SIZE") or os.environ.get("LOCAL_RANK"))
    muon, adamw = [], []
    for name, p in model.named_parameters():
        if not p.requires_grad:
            continue
        n = name.lower()
        is_w = ".weight" in n and not any(t in n for t in _EXCLUDE)
        (muon if (is_w and (fsdp_mode or p.dim() == 2)) else adamw).append(p)
    return muon, adamw


def get_muon_optimizer(model, lr: float = 1e-3, momentum: float = 0.95, weight_decay: float = 0.01,
                       use_8bit: bool = True, fsdp_mode: Optional[bool] = None) -> HybridOptimizer:
    muon_params, adamw_params = split_muon_params(model, fsdp_mode)
    muon_opt = Muon8bit(muon_params, lr=lr, momentum=momentum, weight_decay=weight_decay,
                        use_8bit=use_8bit) if muon_params else None
    adamw_opt = torch.optim.AdamW(adamw_params, lr=lr * 0.3, betas=(0.9, 0.95),
                                  weight_decay=weight_decay) if adamw_params else None
    return HybridOptimizer(muon_opt, adamw_opt)


class CombinedOptimizer:
    """The ndim-based hybrid of the single-GPU trainer (reference: train.py:566-705):
    Muon for every parameter with ndim >= 2 (3-D expert stacks included), AdamW with
    two groups for the rest - norm weights at ``norm_lr`` without decay, other 1-D
    parameters at ``adamw_lr``.  ``state_dict()`` is a list of the two state dicts;
    loading restores state but keeps the current hyper-parameters."""

    def __init__(self, model, muon_lr: float = 1e-3, adamw_lr: float = 3e-4, momentum: float = 0.95,
                 weight_decay: float = 0.01, nesterov: bool = True, backend: str = "newton",
                 newton_iters: int = 5, norm_lr: Optional[float] = None, betas=(0.9, 0.95)):
        mats, norms, others = [], [], []
        for name, p in model.named_parameters():
            if not p.requires_grad:
                continue
            if p.ndim >= 2:
                mats.append(p)
            elif "norm" in name.lower():
                norms.append(p)
            else:
                others.append(p)
        self.muon = Muon(mats, lr=muon_lr, momentum=momentum, weight_decay=weight_decay,
                         nesterov=nesterov, backend=backend, newton_iters=newton_iters) if mats else None
        groups = []
        if norms:
            groups.append({"params": norms, "lr": norm_lr if norm_lr is not None else adamw_lr * 10,
                           "weight_decay": 0.0})
        if others:
            groups.append({"params": others, "lr": adamw_lr, "weight_decay": weight_decay})
        self.adamw = torch.optim.AdamW(groups, lr=adamw_lr, betas=tuple(betas)) if groups else None
        self.optimizers = [o for o in (self.muon, self.adamw) if o is not None]

    @property
    def param_groups(self):
        return [g for o in self.optimizers for g in o.param_groups]

    def step(self, closure=None):
        for o in self.optimizers:
            o.step()

    def zero_grad(self, set_to_none: bool = True):
        for o in self.optimizers:
            o.zero_grad(set_to_none=set_to_none)

    def state_dict(self):
        return [o.state_dict() for o in self.optimizers]

    def load_state_dict(self, sds):
        for o, sd in zip(self.optimizers, sds):
            hyper = [{k: v for k, v in g.items() if k != "params"} for g in o.param_groups]
            o.load_state_dict(sd)
            for g, h in zip(o.param_groups, hyper):
                g.update(h)
