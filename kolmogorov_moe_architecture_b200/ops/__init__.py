"""Hot-op dispatch.

Every function here takes the CUDA kernel path for CUDA tensors and the
plain-PyTorch definition in :mod:`.eager` for CPU tensors.  On a CUDA tensor
the compiled extension is mandatory: a missing ``_C`` library raises instead
of silently falling back, unless ``KMOE_ALLOW_EAGER=1`` is set.  With ``KMOE_CHECK_INPUTS=1`` the data-dependent
inputs (expert ids, labels, kept positions, document starts) are validated before
the launch (:mod:`.checks`).
"""
from __future__ import annotations

import os

import torch

from . import checks, eager
from .loader import ext_available, load_ext, require_ext  # noqa: F401


def _use_cuda(t) -> bool:
    if not t.is_cuda:
        return False
    if ext_available():
        return True
    if os.environ.get("KMOE_ALLOW_EAGER", "0") == "1":
        return False
    require_ext()
    return True


def linear(x, weight, bias=None):
    """``F.linear``; bf16 CUDA tensors go through this library's tcgen05 GEMM (forward, dx and dW)."""
    if _use_cuda(x):
        from . import cuda_ops
        return cuda_ops.linear(x, weight, bias)
    import torch.nn.functional as F
    return F.linear(x, weight, bias)


def linear_multi(x, weights):
    """Several bias-free projections of one input: ``[F.linear(x, w) for w in weights]``.  On the GPU path they
    are one node of the autograd graph, so the input's gradient is accumulated inside the dgrad GEMMs."""
    if _use_cuda(x):
        from . import cuda_ops
        return cuda_ops.linear_multi(x, weights)
    import torch.nn.functional as F
    return [F.linear(x, w) for w in weights]


def dense_swiglu(x, w1, w2, w3):
    """``w3(silu(w1 x) * (w2 x))`` with ``nn.Linear``-layout weights (reference: moe_arch/model/ffn.py:44-64)."""
    if _use_cuda(x):
        from . import cuda_ops
        return cuda_ops.dense_swiglu(x, w1, w2, w3)
    import torch.nn.functional as F
    return F.linear(eager.swiglu(F.linear(x, w1), F.linear(x, w2)), w3)


def rmsnorm(x, weight, eps):
    if _use_cuda(x):
        from . import cuda_ops
        return cuda_ops.rmsnorm(x, weight, eps)
    return eager.rmsnorm(x, weight, eps)


def residual_rmsnorm(x, addend, weight, eps):
    """(h, y): h = x + addend (x itself when addend is None), y = rmsnorm(h); residual add and norm fused."""
    if _use_cuda(x):
        from . import cuda_ops
        return cuda_ops.residual_rmsnorm(x, addend, weight, eps)
    return eager.residual_rmsnorm(x, addend, weight, eps)


def rope_apply(x, cos, sin):
    if _use_cuda(x):
        from . import cuda_ops
        return cuda_ops.rope_apply(x, cos, sin)
    return eager.rope_apply(x, cos, sin)


def swiglu(gate, up):
    if _use_cuda(gate):
        from . import cuda_ops
        return cuda_ops.swiglu(gate, up)
    return eager.swiglu(gate, up)


def attention(q, k, v, causal=True, attn_mask=None, dropout_p=0.0, training=False, doc_start=None):
    """``doc_start`` (B, S): packed-document boundaries (see ``eager.doc_start_from_ids``); on CUDA the flash
    kernels apply them directly, elsewhere they become an additive mask."""
    if doc_start is not None and checks.enabled():
        checks.doc_start(doc_start)
    if attn_mask is None and not (dropout_p > 0.0 and training) and _use_cuda(q):
        from . import cuda_ops
        return cuda_ops.attention(q, k, v, causal, doc_start)
    if doc_start is not None:
        dm = eager.doc_start_to_mask(doc_start, q.dtype)
        attn_mask = dm if attn_mask is None else attn_mask + dm
    return eager.attention(q, k, v, causal, attn_mask, dropout_p, training)


def causal_conv1d(x, weight, bias, activation=True):
    if _use_cuda(x):
        from . import cuda_ops
        return cuda_ops.causal_conv1d(x, weight, bias, activation)
    return eager.causal_conv1d(x, weight, bias, activation)


def selective_scan(u, delta, A, Bm, Cm, D, z, delta_bias, delta_softplus=True):
    if _use_cuda(u):
        from . import cuda_ops
        return cuda_ops.selective_scan(u, delta, A, Bm, Cm, D, z, delta_bias, delta_softplus)
    return eager.selective_scan(u, delta, A, Bm, Cm, D, z, delta_bias, delta_softplus)


def grouped_swiglu(x, w1, w2, w3, idx, weights, keep=None, moe_dtype="bf16"):
    if x.shape[0] == 0:
        return x * 0
    if checks.enabled():
        checks.expert_indices(idx, w1.shape[0], top_k_distinct=False)
        checks.routing_weights(weights)
        checks.keep_mask(keep, idx)
    if _use_cuda(x):
        from . import cuda_ops
        return cuda_ops.grouped_swiglu(x, w1, w2, w3, idx, weights, keep, moe_dtype)
    return eager.grouped_swiglu(x, w1, w2, w3, idx, weights, keep)


def mtp_cross_entropy(hidden, head_weights, labels, weights, ignore_index=-100):
    if checks.enabled():
        checks.labels(labels, head_weights[0].shape[0], ignore_index)
    if _use_cuda(hidden):
        from . import cuda_ops
        return cuda_ops.mtp_cross_entropy(hidden, head_weights, labels, weights, ignore_index)
    return eager.mtp_cross_entropy(hidden, head_weights, labels, weights, ignore_index)


def newton_schulz(matrix, iters=5, sumsq=None):
    """``sumsq``: optional squared Frobenius norms already on the device (see ``cuda_ops.newton_schulz``)."""
    if _use_cuda(matrix):
        from . import cuda_ops
        return cuda_ops.newton_schulz(matrix, iters, sumsq)
    return eager.newton_schulz(matrix, iters)


def route_topk(logits, k, w_lb=0.0, w_z=0.0):
    """Router tail: (weights, indices, aux_loss, assignments per expert)."""
    if _use_cuda(logits):
        from . import cuda_ops
        return cuda_ops.route_topk(logits, k, w_lb, w_z)
    return eager.route_topk(logits, k, w_lb, w_z)


def mod_route(logits, k):
    if _use_cuda(logits):
        from . import cuda_ops
        return cuda_ops.mod_route(logits, k)
    return eager.mod_route(logits, k)


def mod_score_gather(h, w, k):
    """Mixture-of-depths scorer ``h w^T``, per-sequence top-k with softmax weights and the gather of the kept
    rows: (picked (B, k, d), ascending indices (B, k), weights (B, k), logits (B, S))."""
    if (_use_cuda(h) and h.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and h.shape[-1] % 8 == 0
            and h.shape[1] <= 16384 and h.numel() > 0):
        from . import cuda_ops
        return cuda_ops.mod_score_gather(h, w, k)
    logits = torch.nn.functional.linear(h, w).squeeze(-1)
    idx, wts, _ = mod_route(logits, k)
    return mod_gather(h, idx), idx, wts, logits


def mod_bce(aux_logits, idx):
    """Mean binary cross-entropy of (B, S) logits against "position is among the kept indices idx (B, k)"."""
    if checks.enabled():
        checks.kept_rows(idx, aux_logits.shape[1])
    if _use_cuda(aux_logits) and aux_logits.dtype == torch.bfloat16 and aux_logits.numel() > 0:
        from . import cuda_ops
        return cuda_ops.mod_bce(aux_logits, idx)
    targets = torch.zeros_like(aux_logits)
    targets.scatter_(1, idx, 1.0)
    return torch.nn.functional.binary_cross_entropy_with_logits(aux_logits, targets, reduction="mean")


def mod_gather(h, idx):
    if checks.enabled():
        checks.kept_rows(idx, h.shape[1])
    if _use_cuda(h):
        from . import cuda_ops
        return cuda_ops.mod_gather(h, idx)
    return eager.mod_gather(h, idx)


def mod_combine(res, proc, w, idx):
    if checks.enabled():
        checks.kept_rows(idx, res.shape[1])
        checks.routing_weights(w, "mixture-of-depths weights")
    if _use_cuda(res):
        from . import cuda_ops
        return cuda_ops.mod_combine(res, proc, w, idx)
    return eager.mod_combine(res, proc, w, idx)


def expert_choice_route(logits, capacity):
    if _use_cuda(logits):
        from . import cuda_ops
        return cuda_ops.expert_choice_route(logits, capacity)
    return eager.expert_choice_route(logits, capacity)


topk_softmax_route = eager.topk_softmax_route
moe_aux_loss = eager.moe_aux_loss


def capacity_keep_mask(idx, n_experts, capacity):
    """Token-choice capacity with drops: the first ``capacity`` assignments of every expert are kept."""
    if checks.enabled():
        checks.index_range(idx, n_experts, "expert index")
    if _use_cuda(idx):
        from . import cuda_ops
        return cuda_ops.capacity_keep_mask(idx, n_experts, capacity)
    return eager.capacity_keep_mask(idx, n_experts, capacity)


def balanced_assign(probs, top_k):
    """Expert indices (T, k) of the greedy capacity-balanced token-choice assignment."""
    if _use_cuda(probs):
        from . import cuda_ops
        return cuda_ops.balanced_assign(probs, top_k)
    return eager.balanced_assign(probs, top_k)


def expert_choice_swiglu(x, w1, w2, w3, wts, tok):
    """Expert-choice expert FFN (x (B, S, d); wts, tok (B, E, C))."""
    if checks.enabled():
        checks.distinct_rows(tok, x.shape[1], "expert-choice token index")
        checks.routing_weights(wts, "expert-choice weights")
    if _use_cuda(x):
        from . import cuda_ops
        return cuda_ops.expert_choice_swiglu(x, w1, w2, w3, wts, tok)
    return eager.expert_choice_swiglu(x, w1, w2, w3, wts, tok)


rope_tables = eager.rope_tables
doc_start_from_ids = eager.doc_start_from_ids
doc_start_to_mask = eager.doc_start_to_mask
