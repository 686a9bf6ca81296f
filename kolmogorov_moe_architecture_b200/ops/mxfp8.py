"""MXFP8 (OCP microscaling) support: e4m3 values with one power-of-two (e8m0) scale per 32
consecutive elements along the reduction dimension.

``quantize_mx`` / ``dequantize_mx`` define the number format exactly (they are the oracle for
any kernel that consumes it); ``fake_quant_mx`` is the straight-through estimator used for
training on devices without the kernels.  ``grouped_swiglu_mxfp8`` runs the expert FFN: on CUDA bf16
tensors whose widths are multiples of 128 every GEMM (forward, dgrad, wgrad) is a block-scaled
``tcgen05.mma.kind::mxf8f6f4`` GEMM on e4m3 operands quantised along that GEMM's reduction axis
(``csrc/gemm_mxfp8.cu``, ``csrc/mxfp8_quant.cu``); elsewhere the forward operands are fake-quantised
and the bf16 path multiplies them.  The reference's "FP8" experts clamp to +-448 and multiply in bf16
without ever casting to an fp8 dtype (reference: moe_arch/model/fp8_moe.py:247-266).
"""
from __future__ import annotations

import torch

E4M3_MAX = 448.0
BLOCK = 32


def _block_view(x: torch.Tensor, dim: int):
    x = x.movedim(dim, -1)
    K = x.shape[-1]
    pad = (-K) % BLOCK
    if pad:
        x = torch.nn.functional.pad(x, (0, pad))
    return x.reshape(*x.shape[:-1], -1, BLOCK), K


def quantize_mx(x: torch.Tensor, dim: int = -1):
    """Returns (q: float8_e4m3fn with x's shape, scale_exp: int8 exponents, one per 32-block along ``dim``).
    scale = 2^(floor(log2(amax)) - 8), the OCP rule for an element type with emax = 8."""
    xb, K = _block_view(x.float(), dim)
    amax = xb.abs().amax(dim=-1, keepdim=True)
    exp = torch.floor(torch.log2(amax.clamp(min=2.0 ** -127))) - 8.0
    exp = exp.clamp(-127, 127)
    scale = torch.exp2(exp)
    q = (xb / scale).clamp(-E4M3_MAX, E4M3_MAX).to(torch.float8_e4m3fn)
    q = q.reshape(*xb.shape[:-2], -1)[..., :K].movedim(-1, dim)
    return q, exp.squeeze(-1).to(torch.int8)


def dequantize_mx(q: torch.Tensor, scale_exp: torch.Tensor, dim: int = -1, dtype=torch.bfloat16) -> torch.Tensor:
    qb, K = _block_view(q.float(), dim)
    out = qb * torch.exp2(scale_exp.float()).unsqueeze(-1)
    return out.reshape(*qb.shape[:-2], -1)[..., :K].movedim(-1, dim).to(dtype)


class _FakeQuantMX(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, dim):
        q, e = quantize_mx(x, dim)
        return dequantize_mx(q, e, dim, x.dtype)

    @staticmethod
    def backward(ctx, g):
        return g, None


def fake_quant_mx(x: torch.Tensor, dim: int = -1) -> torch.Tensor:
    """Round to MXFP8 along ``dim`` and return in x's dtype; identity gradient."""
    return _FakeQuantMX.apply(x, dim)


def grouped_swiglu_mxfp8(x, w1, w2, w3, idx, weights, keep=None):
    """Expert FFN with MXFP8-rounded operands.  Reduction axes: x along d, w1/w2 along d (dim 1),
    the SwiGLU hidden along f, w3 along f (dim 1)."""
    from . import cuda_ops, eager
    if mx_kernel_ok(x, w1):
        return _GroupedSwiGLUMX.apply(x, w1.contiguous(), w2.contiguous(), w3.contiguous(), idx, weights, keep)
    xq = fake_quant_mx(x, -1)
    w1q, w2q, w3q = fake_quant_mx(w1, 1), fake_quant_mx(w2, 1), fake_quant_mx(w3, 1)
    if x.is_cuda and x.dtype == torch.bfloat16:
        return cuda_ops._GroupedSwiGLU.apply(xq, w1q.contiguous(), w2q.contiguous(), w3q.contiguous(), idx, weights, keep)
    return eager.grouped_swiglu(xq, w1q, w2q, w3q, idx, weights, keep)


# ----------------------------------------------------------------------------------------------
# Block-scaled tensor-core path (CUDA).  Operands are quantised by kernels that write the scale bytes
# in the arrangement the MMA reads from tensor memory; the GEMM is tcgen05 kind::mxf8f6f4.block_scale.

def decode_scale_chunks(sf: torch.Tensor, rows: int, K: int) -> torch.Tensor:
    """Scale chunks (uint8, 512 bytes per 128 rows x 128 reduction elements) -> int exponents (rows, K/32)."""
    rb, kc = (rows + 127) // 128, K // 128
    t = sf[: rb * kc * 512].view(rb, kc, 32, 4, 4)          # [row block, k chunk, row % 32, (row % 128) / 32, k group % 4]
    t = t.permute(0, 3, 2, 1, 4).reshape(rb * 128, kc * 4)
    return t[:rows].to(torch.int32) - 127


def quant_rows(x: torch.Tensor, x2=None, live_rows=None):
    """bf16 (..., C) -> (e4m3 same shape, scale chunks); reduction along the last dim.  With ``x2`` the
    quantised value is silu(x) * x2."""
    from . import cuda_ops
    q, sf = torch.ops.kmoe.mx_quant_rows(x, x2, live_rows)
    cuda_ops._count()
    return q, sf


def quant_cols(x: torch.Tensor, live_rows=None):
    """bf16 (R, C) or (G, R, C) -> (e4m3 (G, C, R), scale chunks); reduction along R, output transposed."""
    from . import cuda_ops
    q, sf = torch.ops.kmoe.mx_quant_cols(x.contiguous(), live_rows)
    cuda_ops._count()
    return q, sf


def gemm_mx(A, sfa, B, sfb, C, *, M, N, K, mode=0, groups=1, a_grouped=False, b_grouped=False, D=None,
            c_gs=0, tile_group=None, num_m_tiles=None, k_begin=None, k_len=None, alpha=1.0, beta=0.0):
    """C (M, N) = alpha * A (M, K) B (N, K)^T + beta * D with e4m3 operands and 1x32 e8m0 scales."""
    from . import cuda_ops
    ldc = C.stride(-2)
    ldd = D.stride(-2) if D is not None else 0
    torch.ops.kmoe.gemm_mxfp8(A, sfa, B, sfb, C, D, mode, M, N, K, groups, a_grouped, b_grouped, ldc, ldd, c_gs,
                              tile_group, num_m_tiles, k_begin, k_len, alpha, beta, cuda_ops.status_tensor(A.device))
    cuda_ops._count()
    return C


def mm_mx(a: torch.Tensor, b: torch.Tensor) -> torch.Tensor:
    """a (M, K) @ b (N, K)^T with both operands rounded to MXFP8 along K; bf16 in, bf16 out."""
    M, K = a.shape
    N = b.shape[0]
    aq, sa = quant_rows(a.contiguous())
    bq, sb = quant_rows(b.contiguous())
    return gemm_mx(aq, sa, bq, sb, torch.empty(M, N, dtype=torch.bfloat16, device=a.device), M=M, N=N, K=K)


class _LinearMX(torch.autograd.Function):
    """y = x W^T with all three GEMMs (forward, dgrad, wgrad) on the block-scaled fp8 path.
    x (M, in), W (out, in); M, in and out multiples of 128."""

    @staticmethod
    def forward(ctx, x, w):
        M, K = x.shape
        N = w.shape[0]
        xq, sx = quant_rows(x.contiguous())
        wq, sw = _weight_quant(w, "rows")                      # (out, in): reduction over in
        y = gemm_mx(xq, sx, wq, sw, torch.empty(M, N, dtype=x.dtype, device=x.device), M=M, N=N, K=K)
        ctx.save_for_backward(x, w)
        return y

    @staticmethod
    def backward(ctx, dy):
        x, w = ctx.saved_tensors
        M, K = x.shape
        N = w.shape[0]
        dy = dy.contiguous()
        dyq, sdy = quant_rows(dy)                              # reduction over out
        wT, swT = _weight_quant(w, "cols")                     # (in, out): reduction over out
        dx = gemm_mx(dyq, sdy, wT, swT, torch.empty(M, K, dtype=dy.dtype, device=dy.device), M=M, N=K, K=N)
        dyT, sdyT = quant_cols(dy)                             # (out, M): reduction over tokens
        xT, sxT = quant_cols(x.contiguous())                   # (in, M)
        dw = gemm_mx(dyT, sdyT, xT, sxT, torch.empty(N, K, dtype=w.dtype, device=w.device), M=N, N=K, K=M)
        return dx, dw


def linear_mx(x: torch.Tensor, w: torch.Tensor, bias=None) -> torch.Tensor:
    """``F.linear`` with MXFP8 operands.  Uses the tensor-core path for CUDA bf16 inputs whose token count and
    feature sizes are multiples of 128, fake-quantised operands with a bf16 multiply otherwise."""
    lead = x.shape[:-1]
    x2 = x.reshape(-1, x.shape[-1])
    ok = (x2.is_cuda and x2.dtype == torch.bfloat16 and w.dtype == torch.bfloat16 and x2.shape[0] % 128 == 0
          and x2.shape[1] % 128 == 0 and w.shape[0] % 128 == 0 and x2.shape[0] > 0)
    if ok:
        y = _LinearMX.apply(x2, w)
    else:
        y = torch.nn.functional.linear(fake_quant_mx(x2, -1), fake_quant_mx(w, -1))
    y = y.reshape(*lead, w.shape[0])
    return y if bias is None else y + bias


# Quantised copies of the expert weights are kept until the weights change, so a step with several
# micro-batches (or forward + backward of one) quantises each orientation once.  A copy is valid while the
# tensor's autograd version and the global epoch are unchanged; code that rewrites parameters through raw
# device pointers (the fused optimizer / all-gather kernels) calls ``invalidate_weight_cache``.
_WCACHE: dict = {}
_EPOCH = [0]


def invalidate_weight_cache() -> None:
    _EPOCH[0] += 1
    if len(_WCACHE) > 4096:
        _WCACHE.clear()


def _weight_quant(w: torch.Tensor, orient: str):
    import os
    if os.environ.get("KMOE_MXFP8_WEIGHT_CACHE", "1") != "1":
        return quant_cols(w) if orient == "cols" else quant_rows(w)
    key = (w.data_ptr(), tuple(w.shape), orient)
    stamp = (w._version, _EPOCH[0])
    hit = _WCACHE.get(key)
    if hit is not None and hit[0] == stamp:
        return hit[1]
    val = quant_cols(w) if orient == "cols" else quant_rows(w)
    _WCACHE[key] = (stamp, val)
    return val


class _GroupedSwiGLUMX(torch.autograd.Function):
    """Expert FFN with every GEMM (forward, dgrad, wgrad) on the block-scaled fp8 tensor-core path.
    Each operand is quantised along the reduction dimension of the GEMM that consumes it, so weights and
    activations are quantised once per orientation; accumulation is fp32, stored tensors stay bf16."""

    @staticmethod
    def forward(ctx, x, w1, w2, w3, idx, weights, keep):
        from . import cuda_ops as C
        K = torch.ops.kmoe
        T, d = x.shape
        E, _, f = w1.shape
        k = idx.shape[1]
        pos, row_src, counts, offsets, tile_group, meta = K.moe_plan(
            idx.reshape(-1).contiguous(), keep.reshape(-1) if keep is not None else None, E, 0)
        R = row_src.numel()
        nmt, live = meta[0:1], meta[1:2]
        Xp = K.moe_gather_rows(x.contiguous(), row_src, None, meta, k)
        Xq, sX = quant_rows(Xp, live_rows=live)
        W1q, s1 = _weight_quant(w1, "cols")                   # (E, f, d): reduction over d
        W2q, s2 = _weight_quant(w2, "cols")
        G = torch.empty(R, f, dtype=x.dtype, device=x.device)
        U = torch.empty_like(G)
        grp = dict(mode=C.GROUPED_M, groups=E, b_grouped=True, tile_group=tile_group, num_m_tiles=nmt)
        gemm_mx(Xq, sX, W1q, s1, G, M=R, N=f, K=d, **grp)
        gemm_mx(Xq, sX, W2q, s2, U, M=R, N=f, K=d, **grp)
        Hq, sH = quant_rows(G, U, live_rows=live)             # SwiGLU fused into the quantiser
        W3q, s3 = _weight_quant(w3, "cols")                   # (E, d, f): reduction over f
        Y = torch.empty(R, d, dtype=x.dtype, device=x.device)
        gemm_mx(Hq, sH, W3q, s3, Y, M=R, N=d, K=f, **grp)
        wf = weights.reshape(-1).float().contiguous()
        out = K.moe_combine(Y, pos, wf, T, k)
        C._count(3)
        ctx.save_for_backward(Xp, G, U, Y, w1, w2, w3, wf, pos, row_src, offsets, tile_group, meta)
        ctx.dims = (T, d, E, f, k, R)
        ctx.wdtype = weights.dtype
        return out

    @staticmethod
    def backward(ctx, dout):
        from . import cuda_ops as C
        K = torch.ops.kmoe
        Xp, G, U, Y, w1, w2, w3, wf, pos, row_src, offsets, tile_group, meta = ctx.saved_tensors
        T, d, E, f, k, R = ctx.dims
        nmt, live = meta[0:1], meta[1:2]
        dout = dout.contiguous()
        grp = dict(mode=C.GROUPED_M, groups=E, b_grouped=True, tile_group=tile_group, num_m_tiles=nmt)
        dYp = K.moe_gather_rows(dout, row_src, wf, meta, k)
        dwts = K.moe_combine_dw(Y, dout, pos, k).view(T, k).to(ctx.wdtype)
        dYq, sdY = quant_rows(dYp, live_rows=live)
        W3r, s3r = _weight_quant(w3, "rows")                  # (E, f, d): reduction over d
        dH = torch.empty(R, f, dtype=dout.dtype, device=dout.device)
        gemm_mx(dYq, sdY, W3r, s3r, dH, M=R, N=f, K=d, **grp)
        dG, dU = K.swiglu_bwd(G, U, dH, live)
        dGq, sdG = quant_rows(dG, live_rows=live)
        dUq, sdU = quant_rows(dU, live_rows=live)
        W1r, s1r = _weight_quant(w1, "rows")                  # (E, d, f): reduction over f
        W2r, s2r = _weight_quant(w2, "rows")
        dXp = torch.empty(R, d, dtype=dout.dtype, device=dout.device)
        gemm_mx(dGq, sdG, W1r, s1r, dXp, M=R, N=d, K=f, **grp)
        gemm_mx(dUq, sdU, W2r, s2r, dXp, D=dXp, beta=1.0, M=R, N=d, K=f, **grp)
        dx = K.moe_combine(dXp, pos, None, T, k)
        # weight gradients: reduction over each expert's (padded) token rows
        kb = offsets[:E].contiguous()
        kl = (offsets[1:] - offsets[:E]).contiguous()
        H = K.swiglu_fwd(G, U, live)
        XT, sXT = quant_cols(Xp, live_rows=live)              # (d, R)
        dGT, sdGT = quant_cols(dG, live_rows=live)            # (f, R)
        dUT, sdUT = quant_cols(dU, live_rows=live)
        HT, sHT = quant_cols(H, live_rows=live)
        dYT, sdYT = quant_cols(dYp, live_rows=live)           # (d, R)
        dw1, dw2, dw3 = torch.empty_like(w1), torch.empty_like(w2), torch.empty_like(w3)
        bat = dict(mode=C.BATCHED, groups=E, k_begin=kb, k_len=kl, K=R)
        gemm_mx(XT, sXT, dGT, sdGT, dw1, M=d, N=f, c_gs=d * f, **bat)
        gemm_mx(XT, sXT, dUT, sdUT, dw2, M=d, N=f, c_gs=d * f, **bat)
        gemm_mx(HT, sHT, dYT, sdYT, dw3, M=f, N=d, c_gs=f * d, **bat)
        C._count(5)
        return dx, dw1, dw2, dw3, None, dwts, None


def mx_kernel_ok(x, w1) -> bool:
    d, f = w1.shape[1], w1.shape[2]
    return x.is_cuda and x.dtype == torch.bfloat16 and w1.dtype == torch.bfloat16 and d % 128 == 0 and f % 128 == 0
