"""CUDA implementations of the hot ops: autograd wrappers over ``torch.ops.kmoe``.

Kernels work on bf16 activations with fp32 accumulation.  A call whose dtype or
shape a kernel does not cover (fp32 activations, a dimension that is not a
multiple of the kernel's vector / tile granularity) is evaluated by the PyTorch
definition in :mod:`.eager`; ``KMOE_STRICT=1`` turns that into an error, which
the GPU tests set so that a kernel path cannot be skipped unnoticed.
"""
from __future__ import annotations

import os
from typing import List, Optional, Sequence

import torch

from . import eager
from .loader import require_ext

require_ext()
K = torch.ops.kmoe

DENSE, GROUPED_M, BATCHED = 0, 1, 2
EPI_STORE, EPI_SWIGLU = 0, 1
MAJ_K, MAJ_MN = 0, 1

_STATUS = {}
LAUNCHES = {"count": 0}       # number of kernels of this library launched (bench accounting)


def _strict() -> bool:
    return os.environ.get("KMOE_STRICT", "0") == "1"


def _fallback(name: str, why: str):
    if _strict():
        raise RuntimeError(f"kmoe.{name}: no CUDA kernel for this call ({why}) and KMOE_STRICT=1")


def status_tensor(device) -> torch.Tensor:
    key = torch.device(device).index if torch.device(device).index is not None else torch.cuda.current_device()
    t = _STATUS.get(key)
    if t is None:
        t = torch.zeros(1, dtype=torch.int32, device=f"cuda:{key}")
        _STATUS[key] = t
    return t


def check_status(device=None) -> None:
    """Raise if any kernel since the last check gave up on a bounded wait.  Synchronises."""
    for key, t in list(_STATUS.items()):
        v = int(t.item())
        if v != 0:
            t.zero_()
            raise RuntimeError(f"kmoe kernel on cuda:{key} reported wait-timeout status {v}")


# Destinations for weight gradients, registered by the sharded data-parallel wrapper: parameter address ->
# (weak reference to the parameter, its slice of the flat gradient buffer, commit callback).  An op whose
# backward produces a weight gradient with a GEMM can write it straight to the destination and return None.
_GRAD_SINKS: dict = {}


def register_grad_sink(param, view, commit) -> None:
    import weakref
    _GRAD_SINKS[param.data_ptr()] = (weakref.ref(param), view, commit)


def grad_sink(w):
    """(destination, commit) when ``w`` has a registered destination and no gradient yet this step."""
    hit = _GRAD_SINKS.get(w.data_ptr())
    if hit is None:
        return None
    p = hit[0]()
    if p is None or p.grad is not None or hit[1].shape != w.shape:
        return None
    return hit[1], (lambda: hit[2](p))


def _count(n: int = 1):
    LAUNCHES["count"] += n


# ---------------------------------------------------------------------- GEMM
def gemm(A, B, C, *, M, N, Kd, mode=DENSE, epi=EPI_STORE, groups=1, a_major=MAJ_K, b_major=MAJ_K,
         lda, ldb, ldc, ldd=0, a_gs=0, b_gs=0, c_gs=0, B2=None, D=None, G=None, U=None,
         tile_group=None, num_m_tiles=None, k_begin=None, k_len=None, alpha=1.0, beta=0.0, row_scale=None,
         row_ptr=None, alpha_dev=None, beta_dev=None, sym_upper=False, diag_add=0.0, k_split=0, D2=None,
         beta2=0.0):
    """``row_ptr`` (int64, one address per output row, 0 = skip) redirects each output row, e.g. into a
    peer GPU's buffer; ``C`` then only supplies the dtype.  ``alpha_dev`` / ``beta_dev`` (fp32, one entry
    per group of a batched GEMM) multiply alpha / beta with values that live on the device.  ``sym_upper``:
    the product is symmetric (A and B are the same operand, M == N): tiles below the diagonal are mirrored
    instead of computed.  ``diag_add`` is added to the main diagonal of the (bf16) result after ``alpha``.
    ``k_split`` > 0 (with ``B2``): the reduction is split, elements [0, k_split) multiply ``B`` and the rest
    ``B2``: ``C = A[:, :k_split] B^T + A[:, k_split:] B2^T`` in one pass.  ``D2`` / ``beta2``: a second addend
    laid out like ``D`` (bf16 output): ``C = alpha A B + beta D + beta2 D2``; ``beta_dev`` scales both."""
    K.gemm(A, B, B2, C, D, G, U, mode, epi, M, N, Kd, groups, a_major, b_major, lda, ldb, ldc, ldd,
           a_gs, b_gs, c_gs, tile_group, num_m_tiles, k_begin, k_len, alpha, beta, row_scale, row_ptr,
           alpha_dev, beta_dev, sym_upper, float(diag_add), int(k_split), D2, float(beta2),
           status_tensor(A.device))
    _count()
    return C


def mm_nt(a: torch.Tensor, b: torch.Tensor, out=None, out_dtype=None, D=None, alpha=1.0, beta=0.0):
    """a [M,K] @ b[N,K]^T -> [M,N]."""
    M, Kd = a.shape
    N = b.shape[0]
    if out is None:
        out = torch.empty(M, N, dtype=out_dtype or a.dtype, device=a.device)
    return gemm(a, b, out, M=M, N=N, Kd=Kd, lda=a.stride(0), ldb=b.stride(0), ldc=out.stride(0),
                ldd=D.stride(0) if D is not None else 0, D=D, alpha=alpha, beta=beta)


def mm_nn(a: torch.Tensor, b: torch.Tensor, out=None, out_dtype=None, D=None, alpha=1.0, beta=0.0):
    """a [M,K] @ b[K,N] -> [M,N]  (b is read MN-major; N % 64 == 0)."""
    M, Kd = a.shape
    N = b.shape[1]
    if out is None:
        out = torch.empty(M, N, dtype=out_dtype or a.dtype, device=a.device)
    return gemm(a, b, out, M=M, N=N, Kd=Kd, b_major=MAJ_MN, lda=a.stride(0), ldb=b.stride(0),
                ldc=out.stride(0), ldd=D.stride(0) if D is not None else 0, D=D, alpha=alpha, beta=beta)


def mm_tn(a: torch.Tensor, b: torch.Tensor, out=None, out_dtype=None, D=None, alpha=1.0, beta=0.0):
    """a[K,M]^T @ b[K,N] -> [M,N]  (both read MN-major; M, N % 64 == 0)."""
    Kd, M = a.shape
    N = b.shape[1]
    if out is None:
        out = torch.empty(M, N, dtype=out_dtype or a.dtype, device=a.device)
    return gemm(a, b, out, M=M, N=N, Kd=Kd, a_major=MAJ_MN, b_major=MAJ_MN, lda=a.stride(0),
                ldb=b.stride(0), ldc=out.stride(0), ldd=D.stride(0) if D is not None else 0, D=D,
                alpha=alpha, beta=beta)


def _bf16(t: torch.Tensor) -> bool:
    return t.dtype == torch.bfloat16


# -------------------------------------------------------------------- Linear
def _linear_ok(x2: torch.Tensor, w: torch.Tensor) -> bool:
    """Shapes the GEMM covers for all three products of a linear layer: the input width is a whole number
    of 64-element swizzle atoms (the weight is read MN-major for dx, the activations for dW), the output
    width and the row count are multiples of 8 (16-byte rows for TMA)."""
    out_f, in_f = w.shape
    return (_bf16(x2) and _bf16(w) and w.is_contiguous() and in_f % 64 == 0 and out_f % 8 == 0
            and x2.shape[0] % 8 == 0 and x2.shape[0] > 0)


_SPLITK_RANGES: dict = {}


def split_k_parts(out_f: int, in_f: int, T: int) -> int:
    """Number of slices of the token dimension for a weight gradient whose (out_f, in_f) result is only a few
    output tiles: with T in the thousands such a GEMM would keep a handful of SMs busy for its whole length.
    Slices are at least 512 tokens long and aim at ~128 tiles in flight; 1 = no split."""
    tiles = -(-out_f // 256) * -(-in_f // 256)
    if tiles >= 48 or T < 2048 or os.environ.get("KMOE_SPLITK", "1") == "0":
        return 1
    return max(1, min(128 // tiles, T // 512, 32))


def _split_k_ranges(T: int, parts: int, device):
    key = (T, parts, device)
    hit = _SPLITK_RANGES.get(key)
    if hit is None:
        step = -(-(-(-T // parts)) // 64) * 64            # slice length: a whole number of 64-row reduction blocks
        begin = list(range(0, T, step))                   # rounding up may leave fewer slices than asked for
        length = [min(step, T - b) for b in begin]
        hit = (torch.tensor(begin, dtype=torch.int32, device=device),
               torch.tensor(length, dtype=torch.int32, device=device))
        _SPLITK_RANGES[key] = hit
    return hit


def _wgrad(dy: torch.Tensor, x2: torch.Tensor, w: torch.Tensor):
    """dW = dy^T x2 into the weight's slot of the flat gradient buffer when one is registered (returns None
    then), else into a new tensor.  Narrow results (router and projection matrices of a few output tiles) are
    computed as slices of the token dimension in one batched launch, fp32 partial results, and summed."""
    out_f, in_f = w.shape
    T = x2.shape[0]
    sink = grad_sink(w)
    dst = sink[0] if sink is not None else torch.empty_like(w)
    parts = split_k_parts(out_f, in_f, T) if (out_f * in_f) % 4 == 0 and dst.is_contiguous() else 1
    out, extra = dst, {}
    if parts > 1:
        kb, kl = _split_k_ranges(T, parts, dy.device)
        parts = kb.numel()
        out = torch.empty(parts, out_f, in_f, dtype=torch.float32, device=dy.device)
        extra = dict(mode=BATCHED, groups=parts, k_begin=kb, k_len=kl, c_gs=out_f * in_f)
    if out_f % 64 == 0:
        gemm(dy, x2, out, M=out_f, N=in_f, Kd=T, a_major=MAJ_MN, b_major=MAJ_MN, lda=dy.stride(0),
             ldb=x2.stride(0), ldc=in_f if parts > 1 else dst.stride(0), **extra)
    else:
        # dy is too narrow to be read MN-major (rows of whole 64-element atoms): use its transpose, K-major
        dyT = dy.t().contiguous()
        gemm(dyT, x2, out, M=out_f, N=in_f, Kd=T, a_major=MAJ_K, b_major=MAJ_MN, lda=T, ldb=x2.stride(0),
             ldc=in_f if parts > 1 else dst.stride(0), **extra)
    if parts > 1:
        K.sum_partials(out, dst)
        _count()
    if sink is not None:
        sink[1]()
        return None
    return dst


class _Linear(torch.autograd.Function):
    """y = x W^T on the tcgen05 GEMM; dx = dy W and dW = dy^T x read the same tensors in the other major, so
    nothing is transposed in memory."""

    @staticmethod
    def forward(ctx, x2, w):
        ctx.save_for_backward(x2, w)
        return mm_nt(x2, w)

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        if not _rows_ok(dy):
            dy = dy.contiguous()
        dx = mm_nn(dy, w) if ctx.needs_input_grad[0] else None
        dw = _wgrad(dy, x2, w) if ctx.needs_input_grad[1] else None
        return dx, dw


class _RowDot(torch.autograd.Function):
    """nn.Linear(d, 1) (a dot product per row)."""

    @staticmethod
    def forward(ctx, x2, w):
        ctx.save_for_backward(x2, w)
        _count()
        return K.rowdot_fwd(x2, w)

    @staticmethod
    def backward(ctx, dy):
        x2, w = ctx.saved_tensors
        sink = grad_sink(w)
        dst = sink[0].view(-1) if sink is not None else None
        dx, dw = K.rowdot_bwd(x2, w, dy.contiguous(), ctx.needs_input_grad[0], dst)
        _count(3)
        if sink is not None:
            sink[1]()
        return (dx if ctx.needs_input_grad[0] else None), (None if sink is not None else dw.view_as(w))


def linear(x: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None) -> torch.Tensor:
    """``F.linear`` on this library's GEMM.  Layers whose input is narrower than one 64-element swizzle atom
    (or not a multiple of it) are left to the library GEMM; none of the 5B model's layers is."""
    in_f = weight.shape[1]
    lead = x.shape[:-1]
    x2 = x.reshape(-1, in_f)
    if not _rows_ok(x2):
        x2 = x2.contiguous()
    if weight.shape[0] == 1 and _bf16(x2) and _bf16(weight) and in_f % 8 == 0 and x2.is_contiguous() and x2.shape[0] > 0:
        y = _RowDot.apply(x2, weight.contiguous()).view(*lead, 1)
    elif _linear_ok(x2, weight):
        y = _Linear.apply(x2, weight).view(*lead, weight.shape[0])
    else:
        return torch.nn.functional.linear(x, weight, bias)
    return y if bias is None else y + bias


class _LinearMulti(torch.autograd.Function):
    """Several bias-free projections of the same input as one node of the graph (the q / k / v projections of
    an attention block): the input's gradient is accumulated by the dgrad GEMMs themselves (``beta = 1`` on the
    second and later ones) instead of being formed as separate tensors that autograd then adds up."""

    @staticmethod
    def forward(ctx, x2, *ws):
        ctx.save_for_backward(x2, *ws)
        return tuple(mm_nt(x2, w) for w in ws)

    @staticmethod
    def backward(ctx, *dys):
        x2, *ws = ctx.saved_tensors
        dx = None
        dws = []
        for i, (dy, w) in enumerate(zip(dys, ws)):
            if dy is None:
                dws.append(None)
                continue
            if not _rows_ok(dy):
                dy = dy.contiguous()
            if ctx.needs_input_grad[0]:
                if dx is None:
                    dx = mm_nn(dy, w)
                else:
                    mm_nn(dy, w, out=dx, D=dx, beta=1.0)
            dws.append(_wgrad(dy, x2, w) if ctx.needs_input_grad[1 + i] else None)
        return (dx, *dws)


def linear_multi(x: torch.Tensor, weights: Sequence[torch.Tensor]):
    """``[F.linear(x, w) for w in weights]`` with one backward node (see ``_LinearMulti``)."""
    in_f = weights[0].shape[1]
    lead = x.shape[:-1]
    x2 = x.reshape(-1, in_f)
    if not _rows_ok(x2):
        x2 = x2.contiguous()
    if not all(_linear_ok(x2, w) and w.shape[0] % 64 == 0 for w in weights):
        return [linear(x, w) for w in weights]
    ys = _LinearMulti.apply(x2, *weights)
    return [y.view(*lead, w.shape[0]) for y, w in zip(ys, weights)]


class _DenseSwiGLU(torch.autograd.Function):
    """w3(silu(w1 x) * (w2 x)) with gate and up in one GEMM whose epilogue applies SwiGLU (one tile holds 128
    gate and 128 up columns), the same kernels the experts use with a single group."""

    @staticmethod
    def forward(ctx, x2, w1, w2, w3):
        T, d = x2.shape
        f = w1.shape[0]
        H = torch.empty(T, f, dtype=x2.dtype, device=x2.device)
        G, U = torch.empty_like(H), torch.empty_like(H)
        gemm(x2, w1, H, B2=w2, G=G, U=U, epi=EPI_SWIGLU, M=T, N=f, Kd=d, lda=x2.stride(0), ldb=d, ldc=f)
        y = mm_nt(H, w3)
        keep_h = os.environ.get("KMOE_MOE_KEEP_H", "1") != "0"      # else H is recomputed in the backward pass
        ctx.save_for_backward(x2, G, U, w1, w2, w3, *((H,) if keep_h else ()))
        return y

    @staticmethod
    def backward(ctx, dy):
        x2, G, U, w1, w2, w3, *kept = ctx.saved_tensors
        if not _rows_ok(dy):
            dy = dy.contiguous()
        dH = mm_nn(dy, w3)
        T, f = dH.shape
        d = w1.shape[1]
        dGU = K.swiglu_bwd_cat(G, U, dH, None)              # [dG | dU], one (T, 2f) operand
        dG, dU = dGU[:, :f], dGU[:, f:]
        _count()
        dx = None
        if ctx.needs_input_grad[0]:
            # dx = dG W1 + dU W2 as one GEMM whose reduction runs over [dG | dU] and [W1 ; W2]
            dx = torch.empty(T, d, dtype=dy.dtype, device=dy.device)
            gemm(dGU, w1, dx, B2=w2, M=T, N=d, Kd=2 * f, k_split=f, b_major=MAJ_MN, lda=2 * f, ldb=d, ldc=d)
        if kept:
            H = kept[0]
        else:
            H = K.swiglu_fwd(G, U, None)
            _count()
        dw1 = _wgrad(dG, x2, w1)
        dw2 = _wgrad(dU, x2, w2)
        dw3 = _wgrad(dy, H, w3)
        return dx, dw1, dw2, dw3


def dense_swiglu(x, w1, w2, w3):
    d, f = w1.shape[1], w1.shape[0]
    lead = x.shape[:-1]
    x2 = x.reshape(-1, d)
    if not _rows_ok(x2):
        x2 = x2.contiguous()
    ok = (_linear_ok(x2, w1) and _linear_ok(x2, w2) and _bf16(w3) and w3.is_contiguous()
          and f % 64 == 0 and d % 64 == 0)
    if not ok:
        return linear(swiglu(linear(x, w1), linear(x, w2)), w3)
    return _DenseSwiGLU.apply(x2, w1, w2, w3).view(*lead, d)


# ------------------------------------------------------------------- RMSNorm
class _RMSNorm(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, eps):
        xc = x.contiguous()
        y, rstd = K.rmsnorm_fwd(xc, w.contiguous(), eps)
        _count()
        ctx.save_for_backward(xc, w, rstd)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w, rstd = ctx.saved_tensors
        dx, dw = K.rmsnorm_bwd(x, w.contiguous(), dy.contiguous(), rstd)
        _count(2)
        return dx, dw.to(w.dtype), None


def rmsnorm(x, weight, eps):
    if not (_bf16(x) and _bf16(weight) and x.shape[-1] % 8 == 0):
        _fallback("rmsnorm", f"dtype {x.dtype}/{weight.dtype}")
        return eager.rmsnorm(x, weight, eps)
    return _RMSNorm.apply(x, weight, eps)


class _ResidualRMSNorm(torch.autograd.Function):
    """(h, y) with h = x (+ addend) the residual stream and y = rmsnorm(h): the residual add, the norm and - in
    backward - the sum of the two gradient paths that meet at h (through the norm and around it) in one kernel
    each, instead of a norm kernel plus separate add kernels in both directions."""

    @staticmethod
    def forward(ctx, x, addend, w, eps):
        xc = x.contiguous()
        ac = addend.contiguous() if addend is not None else None
        h, y, rstd = K.add_rmsnorm_fwd(xc, ac, w.contiguous(), eps)
        _count()
        ctx.save_for_backward(h, w, rstd)
        ctx.has_addend = addend is not None
        return h, y

    @staticmethod
    def backward(ctx, dh, dy):
        h, w, rstd = ctx.saved_tensors
        if dy is None:
            return dh, (dh if ctx.has_addend else None), None, None
        dres = dh.contiguous() if dh is not None else None
        dx, dw = K.rmsnorm_bwd_res(h, w.contiguous(), dy.contiguous(), rstd, dres)
        _count(2)
        return dx, (dx if ctx.has_addend else None), dw.to(w.dtype), None


def residual_rmsnorm(x, addend, weight, eps):
    """Returns (h, y): h = x + addend (x itself when ``addend`` is None), y = rmsnorm(h).  Use h as the residual
    stream from here on, so that its two gradient paths are summed inside the norm's backward kernel."""
    if not (_bf16(x) and _bf16(weight) and x.shape[-1] % 8 == 0 and (addend is None or _bf16(addend))):
        _fallback("residual_rmsnorm", f"dtype {x.dtype}/{weight.dtype}")
        return eager.residual_rmsnorm(x, addend, weight, eps)
    return _ResidualRMSNorm.apply(x, addend, weight, eps)


# ---------------------------------------------------------------------- RoPE
class _Rope(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, cos, sin):
        ctx.save_for_backward(cos, sin)
        _count()
        return K.rope(x.contiguous(), cos, sin, False)

    @staticmethod
    def backward(ctx, g):
        cos, sin = ctx.saved_tensors
        _count()
        return K.rope(g.contiguous(), cos, sin, True), None, None


def rope_apply(x, cos, sin):
    if not (_bf16(x) and x.dim() == 4 and x.shape[-1] % 16 == 0):
        _fallback("rope", f"dtype {x.dtype}")
        return eager.rope_apply(x, cos, sin)
    return _Rope.apply(x, cos.float().contiguous(), sin.float().contiguous())


# -------------------------------------------------------------------- SwiGLU
def _rows_ok(t: torch.Tensor) -> bool:
    if t.stride(-1) != 1 or t.dim() < 2:
        return False
    if t.stride(-2) % 8:
        return False
    for i in range(t.dim() - 3, -1, -1):
        if t.size(i) != 1 and t.stride(i) != t.stride(i + 1) * t.size(i + 1):
            return False
    return True


class _SwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, g, u):
        ctx.save_for_backward(g, u)
        _count()
        return K.swiglu_fwd(g, u, None)

    @staticmethod
    def backward(ctx, dh):
        g, u = ctx.saved_tensors
        _count()
        dg, du = K.swiglu_bwd(g, u, dh.contiguous(), None)
        return dg, du


def swiglu(gate, up):
    if not (_bf16(gate) and _bf16(up) and gate.shape[-1] % 8 == 0):
        _fallback("swiglu", f"dtype {gate.dtype}")
        return eager.swiglu(gate, up)
    if not _rows_ok(gate):
        gate = gate.contiguous()
    if not _rows_ok(up):
        up = up.contiguous()
    return _SwiGLU.apply(gate, up)


# --------------------------------------------------------------------- Mamba
class _Conv1d(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w, b, act):
        wf = w.float().contiguous()
        bf = b.float().contiguous() if b is not None else None
        ctx.save_for_backward(x, wf, bf)
        ctx.act, ctx.wdt, ctx.bdt = act, w.dtype, (b.dtype if b is not None else None)
        _count()
        return K.conv1d_fwd(x, wf, bf, act)

    @staticmethod
    def backward(ctx, dy):
        x, wf, bf = ctx.saved_tensors
        dx, dw, db = K.conv1d_bwd(x, wf, bf, dy.contiguous(), ctx.act)
        _count()
        return dx, dw.to(ctx.wdt), (db.to(ctx.bdt) if bf is not None else None), None


def causal_conv1d(x, weight, bias, activation=True):
    if not (_bf16(x) and weight.shape[-1] == 4 and x.dim() == 3):
        _fallback("causal_conv1d", f"dtype {x.dtype} width {weight.shape[-1]}")
        return eager.causal_conv1d(x, weight, bias, activation)
    if not _rows_ok(x):
        x = x.contiguous()
    return _Conv1d.apply(x, weight, bias, bool(activation))


class _Scan(torch.autograd.Function):
    @staticmethod
    def forward(ctx, u, delta, A, Bm, Cm, D, z, dt_bias, softplus):
        Af = A.float().contiguous()
        Bf, Cf = Bm.float().contiguous(), Cm.float().contiguous()
        Df = D.float().contiguous() if D is not None else None
        bf = dt_bias.float().contiguous() if dt_bias is not None else None
        need = any(ctx.needs_input_grad)
        out, ckpt, seg = K.scan_fwd(u, delta, z, Af, Bf, Cf, Df, bf, softplus, need)
        _count(2 if seg.numel() else 1)
        ctx.save_for_backward(u, delta, z, Af, Bf, Cf, Df, bf, ckpt, seg)
        ctx.softplus = softplus
        ctx.dtypes = (A.dtype, Bm.dtype, Cm.dtype, D.dtype if D is not None else None,
                      dt_bias.dtype if dt_bias is not None else None)
        return out

    @staticmethod
    def backward(ctx, dout):
        u, delta, z, Af, Bf, Cf, Df, bf, ckpt, seg = ctx.saved_tensors
        du, dd, dz, dA, dB, dC, dD, dbias = K.scan_bwd(u, delta, z, Af, Bf, Cf, Df, bf, dout.contiguous(),
                                                       ckpt, seg, ctx.softplus)
        _count(2 if seg.numel() else 1)
        a_dt, b_dt, c_dt, d_dt, bias_dt = ctx.dtypes
        return (du, dd, dA.to(a_dt), dB.to(b_dt), dC.to(c_dt), dD.to(d_dt) if Df is not None else None,
                dz if z is not None else None, dbias.to(bias_dt) if bf is not None else None, None)


def selective_scan(u, delta, A, Bm, Cm, D, z, delta_bias, delta_softplus=True):
    if not (_bf16(u) and _bf16(delta) and A.shape[-1] == 16 and (z is None or _bf16(z))):
        _fallback("selective_scan", f"dtype {u.dtype} d_state {A.shape[-1]}")
        return eager.selective_scan(u, delta, A, Bm, Cm, D, z, delta_bias, delta_softplus)
    u, delta = u.contiguous(), delta.contiguous()
    if z is not None and not _rows_ok(z):
        z = z.contiguous()
    return _Scan.apply(u, delta, A, Bm, Cm, D, z, delta_bias, bool(delta_softplus))


# ----------------------------------------------------------------- attention
def attention(q, k, v, causal=True, doc_start=None):
    from . import attention_cuda
    return attention_cuda.attention(q, k, v, causal, doc_start)


# ------------------------------------------------------------- MoE experts
class _GroupedSwiGLU(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w1, w2, w3, idx, weights, keep):
        T, d = x.shape
        E, _, f = w1.shape
        k = idx.shape[1]
        idx_flat = idx.reshape(-1).contiguous()
        pos, row_src, counts, offsets, tile_group, meta = K.moe_plan(idx_flat, keep.reshape(-1) if keep is not None else None, E, 0)
        max_rows = row_src.numel()
        xc = x.contiguous()
        Xp = K.moe_gather_rows(xc, row_src, None, meta, k)
        H = torch.empty(max_rows, f, dtype=x.dtype, device=x.device)
        G, U = torch.empty_like(H), torch.empty_like(H)
        nmt = meta[0:1]
        gemm(Xp, w1, H, B2=w2, G=G, U=U, mode=GROUPED_M, epi=EPI_SWIGLU, M=max_rows, N=f, Kd=d, groups=E,
             b_major=MAJ_MN, lda=d, ldb=f, ldc=f, b_gs=d * f, tile_group=tile_group, num_m_tiles=nmt)
        Y = torch.empty(max_rows, d, dtype=x.dtype, device=x.device)
        gemm(H, w3, Y, mode=GROUPED_M, M=max_rows, N=d, Kd=f, groups=E, b_major=MAJ_MN, lda=f, ldb=d, ldc=d,
             b_gs=f * d, tile_group=tile_group, num_m_tiles=nmt)
        wf = weights.reshape(-1).float().contiguous()
        out = K.moe_combine(Y, pos, wf, T, k)
        _count(3)
        # The hidden activations H are kept for the weight gradient of the down projection unless
        # KMOE_MOE_KEEP_H=0 (then they are recomputed from G and U in the backward pass: one more kernel per
        # layer, rows x f bf16 less memory held between the passes).
        keep_h = os.environ.get("KMOE_MOE_KEEP_H", "1") != "0"
        ctx.save_for_backward(Xp, G, U, Y, w1, w2, w3, wf, pos, row_src, offsets, tile_group, meta,
                              *((H,) if keep_h else ()))
        ctx.dims = (T, d, E, f, k, max_rows)
        ctx.wdtype = weights.dtype
        return out

    @staticmethod
    def backward(ctx, dout):
        Xp, G, U, Y, w1, w2, w3, wf, pos, row_src, offsets, tile_group, meta, *kept = ctx.saved_tensors
        T, d, E, f, k, max_rows = ctx.dims
        dout = dout.contiguous()
        nmt = meta[0:1]
        dYp = K.moe_gather_rows(dout, row_src, wf, meta, k)
        dwts = K.moe_combine_dw(Y, dout, pos, k).view(T, k).to(ctx.wdtype)
        dH = torch.empty(max_rows, f, dtype=dout.dtype, device=dout.device)
        gemm(dYp, w3, dH, mode=GROUPED_M, M=max_rows, N=f, Kd=d, groups=E, lda=d, ldb=d, ldc=f, b_gs=f * d,
             tile_group=tile_group, num_m_tiles=nmt)
        dGU = K.swiglu_bwd_cat(G, U, dH, meta[1:2])          # [dG | dU], one (rows, 2f) operand
        dG, dU = dGU[:, :f], dGU[:, f:]
        dXp = torch.empty(max_rows, d, dtype=dout.dtype, device=dout.device)
        # dXp = dG W1^T + dU W2^T in one grouped GEMM: the reduction runs over [dG | dU] and [W1 | W2]
        gemm(dGU, w1, dXp, B2=w2, mode=GROUPED_M, M=max_rows, N=d, Kd=2 * f, k_split=f, groups=E, lda=2 * f,
             ldb=f, ldc=d, b_gs=d * f, tile_group=tile_group, num_m_tiles=nmt)
        dx = K.moe_combine(dXp, pos, None, T, k)
        # weight gradients: per expert, reduction over that expert's (padded) row range
        kb = offsets[:E].contiguous()
        kl = (offsets[1:] - offsets[:E]).contiguous()
        H = kept[0] if kept else K.swiglu_fwd(G, U, meta[1:2])
        # weight gradients go straight to their place in the flat gradient buffer when one is registered
        sinks = [grad_sink(w) for w in (w1, w2, w3)]
        dw1, dw2, dw3 = [s[0] if s is not None else torch.empty_like(w) for s, w in zip(sinks, (w1, w2, w3))]
        common = dict(mode=BATCHED, groups=E, a_major=MAJ_MN, b_major=MAJ_MN, Kd=max_rows, k_begin=kb, k_len=kl)
        gemm(Xp, dG, dw1, M=d, N=f, lda=d, ldb=2 * f, ldc=f, c_gs=d * f, **common)
        gemm(Xp, dU, dw2, M=d, N=f, lda=d, ldb=2 * f, ldc=f, c_gs=d * f, **common)
        gemm(H, dYp, dw3, M=f, N=d, lda=f, ldb=d, ldc=d, c_gs=f * d, **common)
        _count(5)
        for s_ in sinks:
            if s_ is not None:
                s_[1]()
        dw1, dw2, dw3 = [None if s_ is not None else g for s_, g in zip(sinks, (dw1, dw2, dw3))]
        return dx, dw1, dw2, dw3, None, dwts, None


def grouped_swiglu(x, w1, w2, w3, idx, weights, keep=None, moe_dtype="bf16"):
    T, d = x.shape
    f = w1.shape[2]
    ok = _bf16(x) and _bf16(w1) and d % 64 == 0 and f % 64 == 0
    if not ok:
        _fallback("grouped_swiglu", f"dtype {x.dtype}/{w1.dtype} d={d} f={f}")
        return eager.grouped_swiglu(x, w1, w2, w3, idx, weights, keep)
    if moe_dtype == "mxfp8":
        from . import mxfp8
        return mxfp8.grouped_swiglu_mxfp8(x, w1, w2, w3, idx, weights, keep)
    return _GroupedSwiGLU.apply(x, w1.contiguous(), w2.contiguous(), w3.contiguous(), idx, weights, keep)


class _ExpertChoiceSwiGLU(torch.autograd.Function):
    """Expert-choice expert FFN on the grouped kernels.  Every expert takes the same number of rows (its ``C``
    picks from each of the ``B`` sequences), so the experts are a batched GEMM over ``E`` groups of ``B * C``
    rows.  A token can be picked by several experts; the slots are turned into the token-choice bookkeeping
    with ``k = E`` (``pos[t, e]`` = row of token t at expert e, or -1), which makes gather, the weighted
    combine and their backward the same deterministic kernels the token-choice path uses (no scatter-add,
    no atomics).  Reference: moe_arch/model/moe.py:533-673 (gather + bmm + Triton scatter)."""

    @staticmethod
    def forward(ctx, x2, w1, w2, w3, wts, tok, S):
        # x2 (B*S, d); wts, tok (B, E, C); w1, w2 (E, d, f); w3 (E, f, d)
        T, d = x2.shape
        B, E, C = tok.shape
        f = w1.shape[2]
        BC = B * C
        dev = x2.device
        t_glob = tok + (torch.arange(B, device=dev) * S).view(B, 1, 1)             # token row in x2
        a = t_glob * E + torch.arange(E, device=dev).view(1, E, 1)                 # assignment id = t * E + e
        a_rows = a.permute(1, 0, 2).reshape(-1)                                     # rows ordered (e, b, c)
        row_src = a_rows.to(torch.int32)
        pos = torch.full((T * E,), -1, dtype=torch.int32, device=dev)
        pos[a_rows] = torch.arange(E * BC, dtype=torch.int32, device=dev)
        wdense = torch.zeros(T * E, dtype=torch.float32, device=dev)
        wdense[a_rows] = wts.permute(1, 0, 2).reshape(-1).float()
        meta = torch.full((2,), E * BC, dtype=torch.int32, device=dev)          # [1] = live rows
        Xg = K.moe_gather_rows(x2.contiguous(), row_src, None, meta, E)
        H = torch.empty(E * BC, f, dtype=x2.dtype, device=dev)
        G, U = torch.empty_like(H), torch.empty_like(H)
        gemm(Xg, w1, H, B2=w2, G=G, U=U, mode=BATCHED, groups=E, epi=EPI_SWIGLU, M=BC, N=f, Kd=d, b_major=MAJ_MN,
             lda=d, ldb=f, ldc=f, a_gs=BC * d, b_gs=d * f, c_gs=BC * f)
        Y = torch.empty(E * BC, d, dtype=x2.dtype, device=dev)
        gemm(H, w3, Y, mode=BATCHED, groups=E, M=BC, N=d, Kd=f, b_major=MAJ_MN, lda=f, ldb=d, ldc=d,
             a_gs=BC * f, b_gs=f * d, c_gs=BC * d)
        out = K.moe_combine(Y, pos, wdense, T, E)
        _count(2)
        ctx.save_for_backward(Xg, G, U, Y, w1, w2, w3, wdense, pos, row_src, meta, a)
        ctx.dims = (T, d, E, f, BC)
        ctx.wdtype = wts.dtype
        return out

    @staticmethod
    def backward(ctx, dout):
        Xg, G, U, Y, w1, w2, w3, wdense, pos, row_src, meta, a = ctx.saved_tensors
        T, d, E, f, BC = ctx.dims
        dout = dout.contiguous()
        dY = K.moe_gather_rows(dout, row_src, wdense, meta, E)
        dwts = K.moe_combine_dw(Y, dout, pos, E)[a].to(ctx.wdtype)                  # (B, E, C)
        dH = torch.empty(E * BC, f, dtype=dout.dtype, device=dout.device)
        gemm(dY, w3, dH, mode=BATCHED, groups=E, M=BC, N=f, Kd=d, lda=d, ldb=d, ldc=f,
             a_gs=BC * d, b_gs=f * d, c_gs=BC * f)
        dGU = K.swiglu_bwd_cat(G, U, dH, None)
        dG, dU = dGU[:, :f], dGU[:, f:]
        dXg = torch.empty(E * BC, d, dtype=dout.dtype, device=dout.device)
        gemm(dGU, w1, dXg, B2=w2, mode=BATCHED, groups=E, M=BC, N=d, Kd=2 * f, k_split=f, lda=2 * f, ldb=f, ldc=d,
             a_gs=BC * 2 * f, b_gs=d * f, c_gs=BC * d)
        dx = K.moe_combine(dXg, pos, None, T, E)
        H = K.swiglu_fwd(G, U, None)
        sinks = [grad_sink(w) for w in (w1, w2, w3)]
        dw1, dw2, dw3 = [s_[0] if s_ is not None else torch.empty_like(w) for s_, w in zip(sinks, (w1, w2, w3))]
        common = dict(mode=BATCHED, groups=E, a_major=MAJ_MN, b_major=MAJ_MN, Kd=BC)
        gemm(Xg, dG, dw1, M=d, N=f, lda=d, ldb=2 * f, ldc=f, a_gs=BC * d, b_gs=BC * 2 * f, c_gs=d * f, **common)
        gemm(Xg, dU, dw2, M=d, N=f, lda=d, ldb=2 * f, ldc=f, a_gs=BC * d, b_gs=BC * 2 * f, c_gs=d * f, **common)
        gemm(H, dY, dw3, M=f, N=d, lda=f, ldb=d, ldc=d, a_gs=BC * f, b_gs=BC * d, c_gs=f * d, **common)
        _count(5)
        for s_ in sinks:
            if s_ is not None:
                s_[1]()
        dw1, dw2, dw3 = [None if s_ is not None else g for s_, g in zip(sinks, (dw1, dw2, dw3))]
        return dx, dw1, dw2, dw3, dwts, None, None


def expert_choice_swiglu(x, w1, w2, w3, wts, tok):
    """x (B, S, d); wts, tok (B, E, C) from ``expert_choice_route``; returns (B, S, d)."""
    B, S, d = x.shape
    f = w1.shape[2]
    ok = _bf16(x) and _bf16(w1) and d % 64 == 0 and f % 64 == 0 and tok.numel() > 0
    if not ok:
        _fallback("expert_choice_swiglu", f"dtype {x.dtype}/{w1.dtype} d={d} f={f}")
        return eager.expert_choice_swiglu(x, w1, w2, w3, wts, tok)
    out = _ExpertChoiceSwiGLU.apply(x.reshape(B * S, d), w1.contiguous(), w2.contiguous(), w3.contiguous(), wts,
                                    tok, S)
    return out.view(B, S, d)


def capacity_keep_mask(idx, n_experts: int, capacity: int):
    """First ``capacity`` assignments of each expert in (token, slot) order are kept (one kernel; no one-hot /
    cumsum tensors of size assignments x experts)."""
    if n_experts > 190:
        return eager.capacity_keep_mask(idx, n_experts, capacity)
    _count()
    return K.moe_capacity_mask(idx.contiguous(), n_experts, int(capacity))


def balanced_assign(probs, top_k: int):
    """Expert indices (T, k) of the greedy balanced assignment (see ``eager.balanced_assign``)."""
    T, E = probs.shape
    cap = max((T * top_k) // E, 1)
    _count(top_k)
    return K.moe_balanced_assign(probs.detach().float().contiguous(), top_k, cap)


# -------------------------------------------------------- routing decisions
class _RouteTopK(torch.autograd.Function):
    """softmax over experts -> top-k -> renormalise, with the auxiliary loss
    ``w_lb * E * sum_e f_e P_e + w_z * mean(lse^2)`` from the same pass."""

    @staticmethod
    def forward(ctx, logits, k, w_lb, w_z):
        shape = logits.shape
        E = shape[-1]
        lf = logits.reshape(-1, E).float().contiguous()
        T = lf.shape[0]
        w, idx, lse, acc = K.route_topk_fwd(lf, k)
        _count()
        aux = (w_lb * E / (float(T) * T * k)) * (acc[:E] * acc[E:2 * E]).sum() + (w_z / T) * acc[2 * E]
        ctx.save_for_backward(lf, lse, idx, w, acc)
        ctx.meta = (shape, logits.dtype, k, w_lb, w_z)
        ctx.mark_non_differentiable(idx)
        return w.view(*shape[:-1], k).to(logits.dtype), idx.view(*shape[:-1], k), aux, acc[E:2 * E]

    @staticmethod
    def backward(ctx, dw, _didx, daux, _dcounts):
        lf, lse, idx, w, acc = ctx.saved_tensors
        shape, dtype, k, w_lb, w_z = ctx.meta
        dwf = dw.reshape(-1, k).float().contiguous() if dw is not None else None
        da = daux.reshape(1).float().contiguous() if daux is not None else None
        dl = K.route_topk_bwd(lf, lse, idx, w, dwf, acc, da, w_lb, w_z)
        _count()
        return dl.view(shape).to(dtype), None, None, None


def route_topk(logits, k, w_lb=0.0, w_z=0.0):
    """Returns (weights, indices, aux_loss, counts_per_expert)."""
    E = logits.shape[-1]
    if E > 128 or k > 8:
        _fallback("route_topk", f"E={E} k={k}")
        return eager.route_topk(logits, k, w_lb, w_z)
    return _RouteTopK.apply(logits, k, float(w_lb), float(w_z))


class _SeqTopK(torch.autograd.Function):
    @staticmethod
    def forward(ctx, scores, k, mode):
        sf = scores.float().contiguous()
        if mode == 0:                       # (B, S): rows are contiguous
            B, S = sf.shape
            geo = (S, 1, B, 0, B, S)
        else:                               # (B, S, E): one row per (b, e), entries E apart
            B, S, E = sf.shape
            geo = (1, E, E, S * E, B * E, S)
        idx, w, stat = K.seq_topk_fwd(sf, *geo, k, mode)
        _count()
        ctx.save_for_backward(sf, idx, w, stat)
        ctx.meta = (geo, k, mode, scores.dtype)
        ctx.mark_non_differentiable(idx)
        if mode == 0:
            return idx, w.to(scores.dtype)
        return idx.view(B, E, k), w.view(B, E, k).to(scores.dtype)

    @staticmethod
    def backward(ctx, _didx, dw):
        sf, idx, w, stat = ctx.saved_tensors
        geo, k, mode, dtype = ctx.meta
        ds = K.seq_topk_bwd(sf, *geo, k, mode, idx, w, dw.reshape(-1, k).float().contiguous(), stat)
        _count()
        return ds.to(dtype), None, None


def mod_route(logits, k):
    """(B, S) logits -> (ascending indices of the k largest, softmax over them, the same indices)."""
    if logits.shape[-1] > 16384:
        _fallback("mod_route", f"S={logits.shape[-1]}")
        return eager.mod_route(logits, k)
    idx, w = _SeqTopK.apply(logits, k, 0)
    return idx, w, idx


def expert_choice_route(logits, capacity):
    """(B, S, E) logits -> (weights (B, E, C), token indices (B, E, C)): softmax over tokens,
    the C most probable tokens per expert, renormalised."""
    if logits.shape[1] > 16384:
        _fallback("expert_choice_route", f"S={logits.shape[1]}")
        return eager.expert_choice_route(logits, capacity)
    idx, w = _SeqTopK.apply(logits, capacity, 1)
    return w, idx


# -------------------------------------------------------- mixture-of-depths rows
class _ModGather(torch.autograd.Function):
    @staticmethod
    def forward(ctx, h, idx):
        ctx.save_for_backward(idx)
        ctx.S = h.shape[1]
        _count()
        return K.rows_gather(h.contiguous(), idx)

    @staticmethod
    def backward(ctx, g):
        (idx,) = ctx.saved_tensors
        _count()
        return K.rows_scatter(g.contiguous(), idx, ctx.S), None


class _ModCombine(torch.autograd.Function):
    @staticmethod
    def forward(ctx, res, proc, w, idx):
        wf = w.float().contiguous()
        procc = proc.contiguous()
        ctx.save_for_backward(procc, wf, idx)
        ctx.wdtype = w.dtype
        _count()
        return K.mod_combine_fwd(res.contiguous(), procc, wf, idx)

    @staticmethod
    def backward(ctx, g):
        proc, wf, idx = ctx.saved_tensors
        g = g.contiguous()
        dproc, dw = K.mod_combine_bwd(g, proc, wf, idx)
        _count()
        return g, dproc, dw.to(ctx.wdtype), None


class _ModScoreGather(torch.autograd.Function):
    """Mixture-of-depths scorer, top-k and row gather as one node of the graph: ``logits = h w``,
    ``idx, weights = top-k / softmax(logits)``, ``picked = h[idx]``.  The hidden states feed both the scorer and
    the gather; as one node their two gradients are formed by one kernel (scatter of the picked rows' gradient
    plus the rank-one term ``dlogits w^T``) instead of two full-size tensors and an addition."""

    @staticmethod
    def forward(ctx, h, w, k):
        B, S, d = h.shape
        hc = h.contiguous()
        h2 = hc.view(B * S, d)
        wv = w.reshape(-1).contiguous()
        logits = K.rowdot_fwd(h2, wv).view(B, S)
        sf = logits.float()
        idx, wts, stat = K.seq_topk_fwd(sf, S, 1, B, 0, B, S, k, 0)
        picked = K.rows_gather(hc, idx)
        _count(3)
        ctx.save_for_backward(h2, wv, sf, idx, wts, stat)
        ctx.w_param = w
        ctx.meta = (B, S, d, k, w.shape)
        ctx.mark_non_differentiable(idx)
        ctx.set_materialize_grads(False)
        return picked, idx, wts, logits          # weights stay fp32: the combine kernel reads them as such

    @staticmethod
    def backward(ctx, d_picked, _didx, d_wts, d_logits):
        h2, wv, sf, idx, wts, stat = ctx.saved_tensors
        B, S, d, k, wshape = ctx.meta
        dl = None
        if d_wts is not None:
            dl = K.seq_topk_bwd(sf, S, 1, B, 0, B, S, k, 0, idx, wts, d_wts.reshape(-1, k).float().contiguous(), stat)
            _count()
        if d_logits is not None:
            dl = d_logits.float() if dl is None else dl + d_logits.float()
        if d_picked is None:
            d_picked = torch.zeros(B, k, d, dtype=h2.dtype, device=h2.device)
        dw = None
        if dl is None:
            dh = K.rows_scatter(d_picked.contiguous(), idx, S)
        else:
            dlb = dl.to(h2.dtype).reshape(-1).contiguous()
            dh = K.rows_scatter_rank1(d_picked.contiguous(), idx, S, dlb, wv)
            if ctx.needs_input_grad[1]:
                sink = grad_sink(ctx.w_param) if ctx.w_param.is_contiguous() else None
                dst = sink[0].view(-1) if sink is not None else None
                _dx, dwv = K.rowdot_bwd(h2, wv, dlb, False, dst)
                _count(2)
                if sink is not None:
                    sink[1]()
                else:
                    dw = dwv.view(wshape)
        _count()
        return dh, dw, None


class _ModBCE(torch.autograd.Function):
    """Mean binary cross-entropy of the selection predictor against "this position was kept": targets are never
    materialised, the gradient is produced with the loss."""

    @staticmethod
    def forward(ctx, logits, idx):
        loss, dl = K.mod_bce(logits.contiguous(), idx)
        _count()
        ctx.save_for_backward(dl)
        return loss[0]

    @staticmethod
    def backward(ctx, g):
        (dl,) = ctx.saved_tensors
        return dl * g.to(dl.dtype), None


def mod_bce(logits, idx):
    """logits (B, S) bf16, idx (B, k) ascending kept positions -> scalar fp32 loss."""
    return _ModBCE.apply(logits, idx.contiguous())


def mod_score_gather(h, w, k):
    """h (B, S, d), scorer weight w (1, d) -> (picked rows (B, k, d), ascending indices (B, k), softmax weights
    (B, k), logits (B, S))."""
    return _ModScoreGather.apply(h, w, k)


def mod_gather(h, idx):
    """h (B, S, d), idx (B, k) ascending -> (B, k, d)."""
    if not _bf16(h) or h.shape[-1] % 8:
        _fallback("mod_gather", f"dtype {h.dtype} d={h.shape[-1]}")
        return eager.mod_gather(h, idx)
    return _ModGather.apply(h, idx.contiguous())


def mod_combine(res, proc, w, idx):
    """res + scatter(w * proc) along the sequence: (B, S, d)."""
    if not (_bf16(res) and _bf16(proc)) or res.shape[-1] % 8:
        _fallback("mod_combine", f"dtype {res.dtype}/{proc.dtype} d={res.shape[-1]}")
        return eager.mod_combine(res, proc, w, idx)
    return _ModCombine.apply(res, proc, w, idx.contiguous())


# -------------------------------------------------------- LM head + MTP loss
_HEAD_WEIGHTS: dict = {}


def _head_weight_tensor(weights: tuple, device) -> torch.Tensor:
    """The per-head loss weights on the device, created once: building a device tensor from Python numbers
    is a pageable host-to-device copy, which blocks the host until the stream has drained."""
    key = (weights, str(device))
    t = _HEAD_WEIGHTS.get(key)
    if t is None:
        t = torch.tensor(list(weights), dtype=torch.float32).to(device)
        _HEAD_WEIGHTS[key] = t
    return t


class _MTPLoss(torch.autograd.Function):
    """Per head: logits chunk = H W^T (tcgen05 GEMM) -> CE kernel writes d logits in place ->
    dH += dlogits W and dW = dlogits^T H.  Gradients are produced during forward (scaled
    for an upstream gradient of 1) and rescaled in backward."""

    @staticmethod
    def forward(ctx, hidden, labels, weights, ignore_index, chunk_rows, *head_weights):
        B, S, d = hidden.shape
        R = B * S
        h2 = hidden.reshape(R, d).contiguous()
        need_grad = ctx.needs_input_grad[0] or any(ctx.needs_input_grad[5:])
        # dH and dW are written by the first GEMM that contributes to them (beta = 0) and accumulated by the later
        # ones, so neither needs a zero fill nor an addend read on its first use
        dH = torch.empty_like(h2) if need_grad else None
        dH_started = False
        dWs: List[Optional[torch.Tensor]] = []
        per = []
        for i, W in enumerate(head_weights):
            V = W.shape[0]
            shift = i + 1
            if shift >= S:
                per.append(torch.zeros((), dtype=torch.float32, device=hidden.device))
                dWs.append(None)
                continue
            lab = torch.full((B, S), ignore_index, dtype=torch.long, device=hidden.device)
            lab[:, : S - shift] = labels[:, shift:]
            lab = lab.reshape(R)
            n_valid = (lab != ignore_index).sum().clamp(min=1).float()
            gscale = (float(weights[i]) / n_valid).reshape(1).contiguous()
            Wc = W.contiguous()
            dW = torch.empty_like(Wc) if need_grad else None
            loss_sum = torch.zeros((), dtype=torch.float32, device=hidden.device)
            for r0 in range(0, R, chunk_rows):
                r1 = min(R, r0 + chunk_rows)
                hc = h2[r0:r1]
                logits = mm_nt(hc, Wc)
                rows = K.ce_fwd_bwd(logits, lab[r0:r1].contiguous(), gscale, ignore_index, need_grad)
                _count()
                loss_sum = loss_sum + rows.sum()
                if need_grad:
                    if dH_started:
                        mm_nn(logits, Wc, out=dH[r0:r1], D=dH[r0:r1], beta=1.0)
                    else:
                        mm_nn(logits, Wc, out=dH[r0:r1])
                    if r0 > 0:
                        mm_tn(logits, hc, out=dW, D=dW, beta=1.0)
                    else:
                        mm_tn(logits, hc, out=dW)
            dH_started = dH_started or need_grad
            per.append(loss_sum / n_valid)
            dWs.append(dW)
        if need_grad and not dH_started:
            dH.zero_()
        per_t = torch.stack(per)
        total = (per_t * _head_weight_tensor(tuple(float(w) for w in weights), hidden.device)).sum()
        ctx.shape = (B, S, d)
        ctx.n_heads = len(head_weights)
        saved = [dH if dH is not None else torch.empty(0, device=hidden.device)]
        saved += [w if w is not None else torch.empty(0, device=hidden.device) for w in dWs]
        ctx.save_for_backward(*saved)
        ctx.need_grad = need_grad
        ctx.heads = head_weights
        ctx.mark_non_differentiable(per_t)
        return total, per_t

    @staticmethod
    def backward(ctx, g_total, _g_per):
        saved = ctx.saved_tensors
        dH, dWs = saved[0], saved[1:]
        B, S, d = ctx.shape
        gh = (dH * g_total.to(dH.dtype)).view(B, S, d) if dH.numel() else None
        gws = []
        for W, w in zip(ctx.heads, dWs):
            if not w.numel():
                gws.append(None)
                continue
            sink = grad_sink(W) if W.is_contiguous() else None
            if sink is not None:
                # scaled straight into the weight's slot of the flat gradient buffer: one pass instead of a
                # multiplication into a new tensor plus the copy into the buffer
                dst = sink[0]
                if dst.is_contiguous() and dst.data_ptr() % 16 == 0 and w.data_ptr() % 16 == 0:
                    K.scale_copy(w, dst, g_total.reshape(1).float())
                else:
                    torch.mul(w, g_total.to(w.dtype), out=dst)
                sink[1]()
                gws.append(None)
            else:
                gws.append(w * g_total.to(w.dtype))
        return (gh, None, None, None, None, *gws)


def mtp_cross_entropy(hidden, head_weights: Sequence[torch.Tensor], labels, weights, ignore_index=-100,
                      chunk_rows: int = 8192):
    d = hidden.shape[-1]
    V = head_weights[0].shape[0]
    ok = _bf16(hidden) and all(_bf16(w) for w in head_weights) and d % 64 == 0 and V % 64 == 0
    if not ok:
        _fallback("mtp_cross_entropy", f"dtype {hidden.dtype} d={d} V={V}")
        return eager.mtp_cross_entropy(hidden, head_weights, labels, weights, ignore_index)
    return _MTPLoss.apply(hidden, labels, tuple(weights), ignore_index, chunk_rows, *head_weights)


# ------------------------------------------------------------ Newton-Schulz
@torch.no_grad()
def _newton_schulz_small_side(Y, s1, s2, iters, wide):
    """The same five cubic steps carried out on the small side of the matrix.

    With G = Y Y^T (g x g, g = the smaller dimension) every step is ``Y <- P Y`` with ``P = 1.5 I - 0.5 G``, and
    all these factors are polynomials in the first G, so they commute: ``Y_k = Q_k Y_0`` with
    ``Q_{k+1} = P_k Q_k`` and ``G_{k+1} = P_k^2 G_k``.  Only the first Gram product and the last ``Q Y_0`` touch
    the long dimension; the steps in between are g x g products: 3 g^2 n + 12 g^3 FLOPs instead of 15 g^2 n.
    In bf16 the factors must be held as deviations from their multiples of the identity - ``1.5 - 0.5 lambda``
    rounds to 1.5 for the small eigenvalues that dominate a normalised gradient - so the stored matrices are
    ``W = P - 1.5 I`` and ``V = Q - c I`` (c = 1.5^k):

        W_0 = -0.5 s^2 Y Y^T                        V_1 = W_0
        W'  = W (W (W + 3 I) + 2.25 I)              (two products, one addend each)
        V'  = W' V + 1.5 V + c W'                   (one product, two addends)
        Y_5 = s (V Y + c Y)

    Every g x g product is symmetric: only the tiles that touch the upper triangle are computed.  Against the
    step-by-step form in bf16 this is more accurate (Y is rounded once, not five times)."""
    b, m, n = Y.shape
    g = m if wide else n
    kw = dict(mode=BATCHED, groups=b, M=g, N=g, Kd=g, lda=g, ldb=g, ldc=g, ldd=g, a_gs=g * g, b_gs=g * g,
              c_gs=g * g, sym_upper=os.environ.get("KMOE_NS_SYM", "1") != "0")
    new = lambda: torch.empty(b, g, g, dtype=torch.bfloat16, device=Y.device)
    W, Wn, T1, Vn = new(), new(), new(), new()
    ga = dict(alpha_dev=s2) if s2 is not None else {}
    if wide:
        gemm(Y, Y, W, mode=BATCHED, groups=b, M=m, N=m, Kd=n, lda=n, ldb=n, ldc=m, alpha=-0.5,
             a_gs=m * n, b_gs=m * n, c_gs=m * m, sym_upper=True, **ga)
    else:
        gemm(Y, Y, W, mode=BATCHED, groups=b, M=n, N=n, Kd=m, a_major=MAJ_MN, b_major=MAJ_MN, lda=n, ldb=n,
             ldc=n, alpha=-0.5, a_gs=m * n, b_gs=m * n, c_gs=n * n, sym_upper=True, **ga)
    V, c = W, 1.5                                                 # Q_1 = P_0: V_1 is W_0 itself
    for _ in range(iters - 1):
        gemm(W, W, T1, D=W, beta=3.0, **kw)                       # T1 = W W + 3 W
        gemm(W, T1, Wn, D=W, beta=2.25, **kw)                     # W' = W T1 + 2.25 W
        gemm(Wn, V, Vn, D=V, beta=1.5, D2=Wn, beta2=c, **kw)      # V' = W' V + 1.5 V + c W'
        old_w, old_v = W, V
        W, V = Wn, Vn
        Wn, Vn = old_w, (new() if old_v is old_w else old_v)      # the buffers just read are the next outputs
        c *= 1.5
    out = torch.empty_like(Y)
    fa = dict(alpha_dev=s1, beta_dev=s1) if s1 is not None else {}
    if wide:      # Y_out = s (V Y + c Y), Y read MN-major as the B operand
        gemm(V, Y, out, D=Y, beta=c, mode=BATCHED, groups=b, M=m, N=n, Kd=m, b_major=MAJ_MN, lda=m, ldb=n,
             ldc=n, ldd=n, a_gs=m * m, b_gs=m * n, c_gs=m * n, **fa)
    else:         # Y_out = s (Y V + c Y), V symmetric: read K-major
        gemm(Y, V, out, D=Y, beta=c, mode=BATCHED, groups=b, M=m, N=n, Kd=n, lda=n, ldb=n, ldc=n, ldd=n,
             a_gs=m * n, b_gs=n * n, c_gs=m * n, **fa)
    return out


def newton_schulz(matrix: torch.Tensor, iters: int = 5, sumsq: Optional[torch.Tensor] = None) -> torch.Tensor:
    """Batched cubic Newton-Schulz on the tcgen05 GEMM, bf16 operands, fp32 accumulation.

    Matrices whose long side is at least 1.25x the short one run the iteration on the short side
    (``_newton_schulz_small_side``); the others run it step by step: per iteration one Gram product and one
    product with the factor ``P = 1.5 I - 0.5 G`` that the Gram GEMM's epilogue emits.

    ``sumsq`` (fp32, one entry per matrix: its squared Frobenius norm, already on the device) removes the
    normalisation passes: the products run on the unnormalised bf16 input and ``s = 1 / (norm + 1e-7)`` is
    folded into the GEMM epilogues."""
    squeeze = matrix.dim() == 2
    Y = matrix.unsqueeze(0) if squeeze else matrix
    b, m, n = Y.shape
    if (m == 1 or n == 1) and matrix.is_cuda:
        # a vector: Y Y^T is the scalar |Y|^2 = 1 after the normalisation, every step multiplies by
        # 1.5 - 0.5 |Y|^2 = 1, so the result is the normalised vector itself
        Yf = Y.float()
        out = (Yf / (Yf.reshape(b, -1).norm(dim=1).view(b, 1, 1) + 1e-7)).to(matrix.dtype)
        return out.squeeze(0) if squeeze else out
    if (m % 64 or n % 64) and min(m, n) >= 8 and matrix.dtype == torch.bfloat16:
        # odd sizes (Mamba x_proj 160 x 4096, the 16 x 128 router of a small model): zero rows / columns stay zero
        # through the iteration, so the matrix is padded to whole 64-element blocks and the result cut back
        mp, np_ = -(-m // 64) * 64, -(-n // 64) * 64
        padded = torch.nn.functional.pad(Y, (0, np_ - n, 0, mp - m))
        out = newton_schulz(padded, iters, sumsq=sumsq)[:, :m, :n].contiguous()
        return out.squeeze(0) if squeeze else out
    if m % 64 or n % 64:
        return eager.newton_schulz(matrix, iters)
    s1 = s2 = None
    if sumsq is not None and matrix.dtype == torch.bfloat16 and Y.is_contiguous() and iters > 0:
        s1 = (1.0 / (sumsq.float().sqrt() + 1e-7)).contiguous()
        s2 = (s1 * s1).contiguous()
        Ya = Y
    else:
        Yf = Y.float()
        norms = Yf.reshape(b, -1).norm(dim=1).view(b, 1, 1)
        Ya = (Yf / (norms + 1e-7)).to(torch.bfloat16).contiguous()
    wide = m <= n
    g = m if wide else n
    if (iters >= 2 and 4 * max(m, n) >= 5 * g and g >= 256 and g % 64 == 0
            and os.environ.get("KMOE_NS_SMALL_SIDE", "1") != "0"):
        out = _newton_schulz_small_side(Ya, s1, s2, iters, wide).to(matrix.dtype)
        return out.squeeze(0) if squeeze else out
    Yb = torch.empty_like(Ya)
    Yc = torch.empty_like(Ya) if s1 is not None else None        # never write into the caller's tensor
    Gm = torch.empty(b, g, g, dtype=torch.bfloat16, device=Y.device)
    # Y' = 1.5 Y - 0.5 G Y = (1.5 I - 0.5 G) Y: the Gram GEMM's epilogue emits P = 1.5 I - 0.5 G directly, so
    # the second product is a plain GEMM that reads no addend
    for it in range(iters):
        first = it == 0 and s1 is not None
        ga = dict(alpha_dev=s2) if first else {}
        ya = dict(alpha_dev=s1) if first else {}
        if wide:
            # P = 1.5 I - 0.5 Y Y^T  (A, B K-major over n)
            gemm(Ya, Ya, Gm, mode=BATCHED, groups=b, M=m, N=m, Kd=n, lda=n, ldb=n, ldc=m, alpha=-0.5,
                 diag_add=1.5, a_gs=m * n, b_gs=m * n, c_gs=m * m, sym_upper=True, **ga)
            # Y' = P Y   (B = Y read MN-major)
            gemm(Gm, Ya, Yb, mode=BATCHED, groups=b, M=m, N=n, Kd=m,
                 b_major=MAJ_MN, lda=m, ldb=n, ldc=n, a_gs=m * m, b_gs=m * n, c_gs=m * n, **ya)
        else:
            # P = 1.5 I - 0.5 Y^T Y  (both MN-major over m)
            gemm(Ya, Ya, Gm, mode=BATCHED, groups=b, M=n, N=n, Kd=m, a_major=MAJ_MN, b_major=MAJ_MN,
                 lda=n, ldb=n, ldc=n, alpha=-0.5, diag_add=1.5, a_gs=m * n, b_gs=m * n, c_gs=n * n,
                 sym_upper=True, **ga)
            # Y' = Y P   (P symmetric: read K-major)
            gemm(Ya, Gm, Yb, mode=BATCHED, groups=b, M=m, N=n, Kd=n,
                 lda=n, ldb=n, ldc=n, a_gs=m * n, b_gs=n * n, c_gs=m * n, **ya)
        if first:
            Ya, Yb = Yb, Yc
        else:
            Ya, Yb = Yb, Ya
    out = Ya.to(matrix.dtype)
    return out.squeeze(0) if squeeze else out
