"""Plain-PyTorch definitions of every hot op.

These are the oracles: each CUDA kernel in ``csrc/`` is tested against the
function of the same name here, evaluated in fp32.  They are also the path
taken on CPU tensors, so the whole model runs (and is tested) without a GPU.
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch
import torch.nn.functional as F


# ---------------------------------------------------------------- norm / rope
def residual_rmsnorm(x, addend, weight, eps):
    """(h, rmsnorm(h)) with h = x + addend (x when addend is None)."""
    h = x if addend is None else x + addend
    return h, rmsnorm(h, weight, eps)


def rmsnorm(x: torch.Tensor, weight: torch.Tensor, eps: float) -> torch.Tensor:
    """w * x / sqrt(mean(x^2) + eps) (reference: moe_arch/model/embeddings.py:191-195)."""
    var = x.pow(2).mean(-1, keepdim=True)
    return weight * (x * torch.rsqrt(var + eps))


def rope_tables(dim: int, max_seq_len: int, theta: float, device=None) -> Tuple[torch.Tensor, torch.Tensor]:
    inv_freq = 1.0 / (theta ** (torch.arange(0, dim, 2, device=device).float() / dim))
    t = torch.arange(max_seq_len, dtype=torch.float32, device=device)
    freqs = torch.outer(t, inv_freq)
    emb = torch.cat((freqs, freqs), dim=-1)
    return emb.cos(), emb.sin()


def rope_apply(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """Rotate-half RoPE on (B, S, H, D); cos/sin are (B, S, D) or (S, D)
    (reference: embeddings.py:126-164)."""
    if cos.dim() == 2:
        cos, sin = cos.unsqueeze(0), sin.unsqueeze(0)
    cos = cos.unsqueeze(2).to(x.dtype)
    sin = sin.unsqueeze(2).to(x.dtype)
    x1, x2 = x.chunk(2, dim=-1)
    c1, c2 = cos.chunk(2, dim=-1)
    s1, s2 = sin.chunk(2, dim=-1)
    return torch.cat([x1 * c1 - x2 * s1, x2 * c2 + x1 * s2], dim=-1)


def swiglu(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    return F.silu(gate) * up


# ------------------------------------------------------------------ attention
def attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, causal: bool = True,
              attn_mask: Optional[torch.Tensor] = None, dropout_p: float = 0.0,
              training: bool = False) -> torch.Tensor:
    """GQA attention. q (B,S,H,D); k, v (B,S,Hkv,D). fp32 softmax, scale 1/sqrt(D).
    ``attn_mask`` is additive and broadcastable to (B,H,S,S)
    (reference eager path: moe_arch/model/attention.py:155-210)."""
    B, S, H, D = q.shape
    Hkv = k.shape[2]
    g = H // Hkv
    qh = q.transpose(1, 2)                                   # B,H,S,D
    kh = k.transpose(1, 2).repeat_interleave(g, dim=1)
    vh = v.transpose(1, 2).repeat_interleave(g, dim=1)
    scores = torch.matmul(qh, kh.transpose(-1, -2)) / math.sqrt(D)
    if causal:
        m = torch.triu(torch.ones(S, S, dtype=torch.bool, device=q.device), diagonal=1)
        scores = scores.masked_fill(m, float("-inf"))
    if attn_mask is not None:
        scores = scores + attn_mask
    p = F.softmax(scores, dim=-1, dtype=torch.float32).to(q.dtype)
    if dropout_p > 0.0 and training:
        p = F.dropout(p, dropout_p, training=True)
    return torch.matmul(p, vh).transpose(1, 2).contiguous()   # B,S,H,D


def doc_start_from_ids(doc_ids: torch.Tensor) -> torch.Tensor:
    """(B, S) document ids of a packed batch (constant inside a document) -> (B, S) int32 position of the first
    token of each position's document."""
    B, S = doc_ids.shape
    pos = torch.arange(S, device=doc_ids.device).expand(B, S)
    change = torch.ones(B, S, dtype=torch.bool, device=doc_ids.device)
    change[:, 1:] = doc_ids[:, 1:] != doc_ids[:, :-1]
    return torch.cummax(torch.where(change, pos, torch.zeros_like(pos)), dim=1).values.to(torch.int32)


def doc_start_to_mask(doc_start: torch.Tensor, dtype=torch.float32) -> torch.Tensor:
    """Additive (B, 1, S, S) mask equivalent to ``doc_start``: key k is hidden from query q when k < doc_start[q]."""
    B, S = doc_start.shape
    k = torch.arange(S, device=doc_start.device).view(1, 1, S)
    hidden = k < doc_start.view(B, S, 1)
    return torch.zeros(B, 1, S, S, dtype=dtype, device=doc_start.device).masked_fill(hidden.unsqueeze(1), float("-inf"))


# ---------------------------------------------------------------------- mamba
def causal_conv1d(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor],
                  activation: bool = True) -> torch.Tensor:
    """Depthwise causal conv over time. x (B, S, C) channels-last; weight (C, W), or (G, C, W) with G
    parameter sets: batch entries [g B/G, (g+1) B/G) use set g (bias (G, C) then)."""
    if weight.dim() == 3:
        G = weight.shape[0]
        parts = x.chunk(G, dim=0)
        return torch.cat([causal_conv1d(parts[g], weight[g], bias[g] if bias is not None else None, activation)
                          for g in range(G)], dim=0)
    C, W = weight.shape
    y = F.conv1d(x.transpose(1, 2), weight.unsqueeze(1), bias, padding=W - 1, groups=C)[..., : x.shape[1]]
    y = y.transpose(1, 2)
    return F.silu(y) if activation else y


def selective_scan(u: torch.Tensor, delta: torch.Tensor, A: torch.Tensor, Bm: torch.Tensor,
                   Cm: torch.Tensor, D: Optional[torch.Tensor], z: Optional[torch.Tensor],
                   delta_bias: Optional[torch.Tensor], delta_softplus: bool = True) -> torch.Tensor:
    """Mamba selective scan, channels-last.

    u, delta, z: (B, S, C); A: (C, N); Bm, Cm: (B, S, N); D, delta_bias: (C,).
    h_t = exp(delta_t A) h_{t-1} + delta_t B_t u_t ;  y_t = <C_t, h_t> + D u_t ;
    y_t *= silu(z_t).  Evaluated sequentially in fp32.  A (G, C, N) with D, delta_bias (G, C): G parameter
    sets over consecutive slices of the batch.
    """
    if A.dim() == 3:
        G = A.shape[0]
        sl = lambda t: t.chunk(G, dim=0) if t is not None else [None] * G
        us, ds, bs, cs, zs = sl(u), sl(delta), sl(Bm), sl(Cm), sl(z)
        return torch.cat([selective_scan(us[g], ds[g], A[g], bs[g], cs[g], D[g] if D is not None else None, zs[g],
                                         delta_bias[g] if delta_bias is not None else None, delta_softplus)
                          for g in range(G)], dim=0)
    dt = delta.float()
    if delta_bias is not None:
        dt = dt + delta_bias.float()
    if delta_softplus:
        dt = F.softplus(dt)
    uf = u.float()
    Bsz, S, C = u.shape
    N = A.shape[1]
    h = torch.zeros(Bsz, C, N, dtype=torch.float32, device=u.device)
    Af = A.float()
    ys = []
    for t in range(S):
        dA = torch.exp(dt[:, t, :, None] * Af)                      # B,C,N
        dBu = dt[:, t, :, None] * Bm[:, t, None, :].float() * uf[:, t, :, None]
        h = dA * h + dBu
        ys.append((h * Cm[:, t, None, :].float()).sum(-1))
    y = torch.stack(ys, dim=1)
    if D is not None:
        y = y + uf * D.float()
    if z is not None:
        y = y * F.silu(z.float())
    return y.to(u.dtype)


# -------------------------------------------------------------------- routing
def topk_softmax_route(logits: torch.Tensor, top_k: int) -> Tuple[torch.Tensor, torch.Tensor]:
    """softmax over experts -> top-k -> renormalise (reference: moe.py:441-460)."""
    probs = F.softmax(logits, dim=-1)
    w, idx = torch.topk(probs, top_k, dim=-1)
    return w / w.sum(dim=-1, keepdim=True), idx


def moe_aux_loss(logits: torch.Tensor, idx: torch.Tensor, n_experts: int,
                 w_lb: float, w_z: float) -> torch.Tensor:
    """w_lb * E * sum_i f_i P_i + w_z * mean(logsumexp^2) (reference: moe.py:840-939)."""
    flat = logits.reshape(-1, n_experts)
    P = F.softmax(flat, dim=-1).mean(0)
    counts = torch.bincount(idx.reshape(-1), minlength=n_experts).to(P.dtype)
    f = counts / idx.numel()
    lb = n_experts * (f * P).sum()
    z = (torch.logsumexp(flat, dim=-1) ** 2).mean()
    return w_lb * lb + w_z * z


def route_topk(logits: torch.Tensor, top_k: int, w_lb: float = 0.0, w_z: float = 0.0):
    """Router tail in one call: (weights, indices, aux_loss, counts_per_expert)."""
    w, idx = topk_softmax_route(logits, top_k)
    E = logits.shape[-1]
    aux = moe_aux_loss(logits.float(), idx, E, w_lb, w_z)
    counts = torch.bincount(idx.reshape(-1), minlength=E).float()
    return w, idx, aux, counts


def expert_choice_route(logits: torch.Tensor, capacity: int):
    """(B, S, E) -> softmax over tokens, per-expert top-C, renormalised (reference: moe.py:494-530)."""
    probs = F.softmax(logits.transpose(1, 2), dim=-1)
    w, tok = torch.topk(probs, capacity, dim=-1)
    return w / (w.sum(dim=-1, keepdim=True) + 1e-9), tok


def expert_choice_swiglu(x, w1, w2, w3, wts, tok):
    """Expert-choice expert FFN: expert e applies SwiGLU to the C tokens it picked from every sequence and the
    results are added back weighted (reference: moe.py:533-673).  x (B, S, d); wts, tok (B, E, C)."""
    B, S, d = x.shape
    _, E, C = tok.shape
    flat_idx = tok.reshape(B, E * C)
    xin = torch.gather(x, 1, flat_idx.unsqueeze(-1).expand(-1, -1, d)).view(B, E, C, d)
    h = swiglu(torch.matmul(xin, w1), torch.matmul(xin, w2))
    y = torch.matmul(h, w3)
    y = (y * wts.unsqueeze(-1).to(y.dtype)).view(B, E * C, d)
    return torch.zeros_like(x).scatter_add(1, flat_idx.unsqueeze(-1).expand(-1, -1, d), y)


def balanced_assign(probs: torch.Tensor, top_k: int) -> torch.Tensor:
    """Greedy per-slot assignment under a global per-expert capacity of ``(T * k) // E``: in slot j every token
    takes its best expert that was not already full at the start of the slot and that it has not used; a
    token with no such expert takes its best unused one (reference: moe.py:353-421).  Returns indices (T, k)."""
    T, E = probs.shape
    cap = max((T * top_k) // E, 1)
    counts = torch.zeros(E, dtype=torch.long, device=probs.device)
    avail = probs.detach().clone()
    sel = []
    neg = float("-inf")
    for _ in range(top_k):
        masked = avail.masked_fill((counts >= cap)[None, :], neg)
        best_p, best_e = masked.max(dim=-1)
        fb_e = avail.argmax(dim=-1)
        best_e = torch.where(best_p == neg, fb_e, best_e)
        sel.append(best_e)
        counts = counts + torch.bincount(best_e, minlength=E)
        avail = avail.scatter(1, best_e[:, None], neg)
    return torch.stack(sel, dim=1)


def capacity_keep_mask(idx: torch.Tensor, n_experts: int, capacity: int) -> torch.Tensor:
    """Drop policy for token-choice with capacity: for each expert keep the first
    ``capacity`` assignments in (token, slot) order; later ones are dropped and
    contribute zero (weights are not renormalised)."""
    flat = idx.reshape(-1)
    onehot = F.one_hot(flat, n_experts)
    rank = (onehot.cumsum(0) - 1).gather(1, flat[:, None]).squeeze(1)
    return (rank < capacity).reshape(idx.shape)


def grouped_swiglu(x: torch.Tensor, w1: torch.Tensor, w2: torch.Tensor, w3: torch.Tensor,
                   idx: torch.Tensor, weights: torch.Tensor,
                   keep: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Token-choice expert FFN: out[t] = sum_k weights[t,k] * SwiGLU_{idx[t,k]}(x[t]).

    x (T, d); w1, w2 (E, d, f); w3 (E, f, d) - the (in, out) layout of the
    reference's stacked parameters (moe.py:183-185)."""
    T, d = x.shape
    E = w1.shape[0]
    out = torch.zeros_like(x)
    for e in range(E):
        sel = idx == e
        if keep is not None:
            sel = sel & keep
        tok, slot = sel.nonzero(as_tuple=True)
        if tok.numel() == 0:
            continue
        xe = x[tok]
        h = F.silu(xe @ w1[e]) * (xe @ w2[e])
        ye = (h @ w3[e]) * weights[tok, slot].unsqueeze(1).to(x.dtype)
        out.index_add_(0, tok, ye)
    return out


def mod_route(logits: torch.Tensor, k: int) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """Per-sequence top-k of (B, S) logits; indices ascending; softmax over the kept
    logits (reference: moe_arch/model/mod.py:93-112).  Returns (sorted_idx, weights, topk_idx)."""
    topv, topi = torch.topk(logits, k, dim=-1)
    sidx, order = torch.sort(topi, dim=-1)
    w = F.softmax(torch.gather(topv, -1, order), dim=-1)
    return sidx, w, topi


def mod_gather(h: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
    """Rows of h (B, S, d) at the kept positions idx (B, k) -> (B, k, d)."""
    return torch.gather(h, 1, idx.unsqueeze(-1).expand(-1, -1, h.shape[-1]))


def mod_combine(res: torch.Tensor, proc: torch.Tensor, w: torch.Tensor, idx: torch.Tensor) -> torch.Tensor:
    """res + scatter of the weighted processed rows back to their positions
    (reference: moe_arch/model/layers.py:160-185)."""
    gi = idx.unsqueeze(-1).expand(-1, -1, res.shape[-1])
    upd = proc * w.unsqueeze(-1).to(proc.dtype)
    return res + torch.zeros_like(res).scatter_add(1, gi, upd)


# ----------------------------------------------------------------------- loss
def mtp_cross_entropy(hidden: torch.Tensor, head_weights, labels: torch.Tensor,
                      weights, ignore_index: int = -100) -> Tuple[torch.Tensor, torch.Tensor]:
    """Multi-token-prediction loss from the final hidden state.

    hidden (B, S, d); head_weights: list of (V, d); head i scores positions
    [0, S-i-1) against labels[:, i+1:] with mean CE over non-ignored targets
    (reference: moe_arch/training/losses.py:74-119).  Returns (total, per_head)."""
    B, S, _ = hidden.shape
    per = []
    for i, W in enumerate(head_weights):
        if i + 1 >= S:
            per.append(hidden.new_zeros((), dtype=torch.float32))
            continue
        logits = hidden[:, : S - i - 1] @ W.t()
        tgt = labels[:, i + 1:]
        per.append(F.cross_entropy(logits.reshape(-1, logits.size(-1)).float(), tgt.reshape(-1),
                                   ignore_index=ignore_index, reduction="mean"))
    per_t = torch.stack(per)
    total = (per_t * torch.tensor(list(weights), dtype=per_t.dtype, device=per_t.device)).sum()
    return total, per_t


# ------------------------------------------------------------------ optimiser
def newton_schulz(matrix: torch.Tensor, iters: int = 5) -> torch.Tensor:
    """Cubic Newton-Schulz iteration Y <- 1.5 Y - 0.5 (Y Y^T) Y on the Frobenius-normalised
    matrix; wide/tall branches; 3-D input is treated as a batch
    (reference: moe_arch/training/muon_optimizer.py:368-455)."""
    if matrix.dim() == 2:
        return newton_schulz(matrix.unsqueeze(0), iters).squeeze(0)
    b, m, n = matrix.shape
    norms = matrix.reshape(b, -1).norm(dim=1).view(b, 1, 1)
    Y = matrix / (norms + 1e-7)
    if m <= n:
        for _ in range(iters):
            Y = 1.5 * Y - 0.5 * torch.bmm(torch.bmm(Y, Y.transpose(-2, -1)), Y)
    else:
        for _ in range(iters):
            Y = 1.5 * Y - 0.5 * torch.bmm(Y, torch.bmm(Y.transpose(-2, -1), Y))
    return Y
