"""Expert-parallel SwiGLU FFN whose token exchange runs over NVLink peer pointers.

One autograd function covers the whole layer on both sides of the exchange:

    source rank                                      expert rank
    -----------                                      -----------
    plan (stable counting sort over all E experts)
    dispatch: token rows -> owner's receive slots    (permute and all-to-all in one kernel)
    ------------------------ flag barrier ------------------------
                                                     recv_plan: slot counts -> padded expert-major layout
                                                     compact slots -> Xp (+ table: packed row -> address
                                                             of its place in the source's return buffer)
                                                     grouped GEMM 1 (+SwiGLU epilogue)
                                                     grouped GEMM 2 whose epilogue stores every row
                                                             through that table into the source rank
    ------------------------ flag barrier ------------------------
    weighted top-k combine (local)

Backward is the same pipeline with ``w * dout`` rows travelling out, the dgrad GEMMs on the
expert rank, and ``dXp`` rows travelling back; weight gradients never leave the expert rank.
Counts, offsets and tile tables stay on the device - there is no host read and no NCCL call
in either direction (the all-to-all transport in :mod:`.ep` needs one host read per layer).

With ``moe_dtype="mxfp8"`` the expert rank quantises the compacted rows (e4m3, one e8m0 scale per 32
elements along each GEMM's reduction) and runs the block-scaled GEMMs of ``csrc/gemm_mxfp8.cu``; rows
travel in bf16 both ways and the second GEMM's rows go back with the return kernel.

Buffers are symmetric-memory allocations sized for the worst case (every token of every rank
routed to one rank) and shared by all layers of a model: a layer's receive buffer is free
again once the rank has compacted it, which the second barrier of the layer orders before any
peer's next dispatch.

The kernels are in ``csrc/comm.cu`` (``ep_dispatch``, ``ep_recv_plan``, ``ep_move``) and the
row-pointer epilogue of ``csrc/gemm_umma.cu``.  The
reference exchanges rows with ``all_to_all_single`` and a host-side loop
(moe_arch/model/sparse_moe.py:540-603).
"""
from __future__ import annotations

from typing import Dict, Optional, Tuple

import torch
import torch.distributed as dist

from .p2p import _group_name, enable_group, peer_ptrs


def _round_up(x: int, m: int) -> int:
    return (x + m - 1) // m * m


class EPBuffers:
    """Symmetric receive / return / meta / flag buffers for one (tokens, top_k, d_model, E) shape."""

    def __init__(self, T: int, k: int, d: int, E: int, dtype, device, group=None, cap: Optional[int] = None,
                 barrier_timeout_s: float = 30.0):
        import torch.distributed._symmetric_memory as symm
        from ..ops import cuda_ops
        self.group = group
        self.world = dist.get_world_size(group)
        self.rank = dist.get_rank(group)
        assert E % self.world == 0
        self.T, self.k, self.d, self.E = T, k, d, E
        self.n_local = E // self.world
        # top-k picks distinct experts, so one source sends an expert at most T rows
        self.cap = int(cap) if cap is not None else T
        n_slots = self.n_local * self.world
        self.max_rows_src = _round_up(T * k + E * 127, 128)
        self.max_rows_exp = _round_up(min(n_slots * self.cap, self.world * T * k) + self.n_local * 127, 128)
        name = _group_name(group)
        enable_group(name)
        self.recv = symm.empty((n_slots * self.cap, d), dtype=dtype, device=device)
        self.ret = symm.empty((self.max_rows_src, d), dtype=dtype, device=device)
        self.meta = symm.empty(n_slots * 2, dtype=torch.int32, device=device)
        self.flags = symm.empty(64, dtype=torch.int32, device=device)
        self.meta.zero_()
        self.flags.zero_()
        torch.cuda.synchronize(device)
        hs = [symm.rendezvous(t, name) for t in (self.recv, self.ret, self.meta, self.flags)]
        self._h = hs
        self.recv_ptrs = peer_ptrs(hs[0], self.recv, self.rank)
        self.ret_ptrs = peer_ptrs(hs[1], self.ret, self.rank)
        self.meta_ptrs = peer_ptrs(hs[2], self.meta, self.rank)
        self.flag_ptrs = peer_ptrs(hs[3], self.flags, self.rank)
        self.epoch = 0
        self.timeout_s = barrier_timeout_s
        self.status = cuda_ops.status_tensor(device)
        dist.barrier(group=group)

    def barrier(self) -> None:
        from ..ops import cuda_ops
        self.epoch += 1
        torch.ops.kmoe.p2p_barrier(self.flag_ptrs, self.rank, self.world, self.epoch, self.timeout_s, self.status)
        cuda_ops._count()

    def bytes(self) -> int:
        return sum(t.numel() * t.element_size() for t in (self.recv, self.ret, self.meta, self.flags))


class EPUnavailable(RuntimeError):
    """The symmetric buffers of the peer-pointer transport could not be set up on this machine."""


_CACHE: Dict[Tuple, EPBuffers] = {}


def get_buffers(T: int, k: int, d: int, E: int, dtype, device, group=None, cap: Optional[int] = None) -> EPBuffers:
    key = (T, k, d, E, dtype, str(device), _group_name(group), cap)
    buf = _CACHE.get(key)
    if buf is None:
        try:
            buf = EPBuffers(T, k, d, E, dtype, device, group, cap=cap)
        except Exception as e:
            raise EPUnavailable(f"{type(e).__name__}: {e}") from e
        _CACHE[key] = buf
    return buf


def release_buffers() -> None:
    """Drop the cached symmetric buffers (all ranks of the group must call it together)."""
    _CACHE.clear()


class _EPFusedFFN(torch.autograd.Function):
    @staticmethod
    def forward(ctx, x, w1, w2, w3, idx, weights, keep, buf: EPBuffers):
        from ..ops import cuda_ops as C
        K = torch.ops.kmoe
        T, d = x.shape
        nl, _, f = w1.shape
        k = idx.shape[1]
        E, ws = buf.E, buf.world
        idx_flat = idx.reshape(-1).contiguous()
        pos, row_src, counts, offsets, _tg, _meta = K.moe_plan(
            idx_flat, keep.reshape(-1) if keep is not None else None, E, 0)
        assert row_src.numel() <= buf.max_rows_src
        xc = x.contiguous()
        K.ep_dispatch(xc, row_src, None, offsets, counts, buf.recv_ptrs, buf.meta_ptrs, buf.rank, ws, E, buf.cap, k)
        buf.barrier()
        R = buf.max_rows_exp
        meta_in = buf.meta.clone()
        slot_dst, offs_l, tile_group, meta_l = K.ep_recv_plan(meta_in, nl, ws, R)
        Xp = torch.empty(R, d, dtype=x.dtype, device=x.device)
        # row_ptr: where each packed row's result belongs in its source rank's return buffer
        row_ptr = torch.empty(R, dtype=torch.int64, device=x.device)
        K.ep_move(buf.recv, Xp, meta_in, slot_dst, offs_l, buf.ret_ptrs, buf.rank, nl, ws, buf.cap, 0, row_ptr)
        H = torch.empty(R, f, dtype=x.dtype, device=x.device)
        G, U = torch.empty_like(H), torch.empty_like(H)
        nmt = meta_l[0:1]
        C.gemm(Xp, w1, H, B2=w2, G=G, U=U, mode=C.GROUPED_M, epi=C.EPI_SWIGLU, M=R, N=f, Kd=d, groups=nl,
               b_major=C.MAJ_MN, lda=d, ldb=f, ldc=f, b_gs=d * f, tile_group=tile_group, num_m_tiles=nmt)
        # GEMM 2 with the combine's transfer in its epilogue: every output row is stored straight into the
        # source rank's return buffer over NVLink (Xp only lends its dtype here)
        C.gemm(H, w3, Xp, mode=C.GROUPED_M, M=R, N=d, Kd=f, groups=nl, b_major=C.MAJ_MN, lda=f, ldb=d, ldc=d,
               b_gs=f * d, tile_group=tile_group, num_m_tiles=nmt, row_ptr=row_ptr)
        buf.barrier()
        wf = weights.reshape(-1).float().contiguous()
        out = K.moe_combine(buf.ret, pos, wf, T, k)
        # the return buffer is reused by the next layer; keep this layer's rows for d(loss)/d(weights)
        Yret = buf.ret[: row_src.numel()].clone() if ctx.needs_input_grad[5] else None
        C._count(6)
        ctx.save_for_backward(Xp, G, U, w1, w2, w3, wf, pos, row_src, counts, offsets, meta_in, slot_dst, offs_l,
                              tile_group, meta_l, Yret if Yret is not None else torch.empty(0, device=x.device),
                              row_ptr)
        ctx.buf = buf
        ctx.dims = (T, d, nl, f, k, R)
        ctx.wdtype = weights.dtype
        return out

    @staticmethod
    def backward(ctx, dout):
        from ..ops import cuda_ops as C
        K = torch.ops.kmoe
        (Xp, G, U, w1, w2, w3, wf, pos, row_src, counts, offsets, meta_in, slot_dst, offs_l, tile_group, meta_l,
         Yret, row_ptr) = ctx.saved_tensors
        buf = ctx.buf
        T, d, nl, f, k, R = ctx.dims
        E, ws = buf.E, buf.world
        dout = dout.contiguous()
        nmt = meta_l[0:1]
        # w * dout rows travel to the expert ranks (permute, scale and exchange in one kernel)
        K.ep_dispatch(dout, row_src, wf, offsets, counts, buf.recv_ptrs, buf.meta_ptrs, buf.rank, ws, E, buf.cap, k)
        buf.barrier()
        dYp = torch.empty(R, d, dtype=dout.dtype, device=dout.device)
        K.ep_move(buf.recv, dYp, meta_in, slot_dst, offs_l, buf.ret_ptrs, buf.rank, nl, ws, buf.cap, 0, None)
        dH = torch.empty(R, f, dtype=dout.dtype, device=dout.device)
        C.gemm(dYp, w3, dH, mode=C.GROUPED_M, M=R, N=f, Kd=d, groups=nl, lda=d, ldb=d, ldc=f, b_gs=f * d,
               tile_group=tile_group, num_m_tiles=nmt)
        dG, dU = K.swiglu_bwd(G, U, dH, meta_l[1:2])      # buffers are worst-case sized: touch live rows only
        dXp = torch.empty(R, d, dtype=dout.dtype, device=dout.device)
        C.gemm(dG, w1, dXp, mode=C.GROUPED_M, M=R, N=d, Kd=f, groups=nl, lda=f, ldb=f, ldc=d, b_gs=d * f,
               tile_group=tile_group, num_m_tiles=nmt)
        # second dgrad GEMM adds the first one's local result and stores the sum into the source ranks
        C.gemm(dU, w2, dXp, D=dXp, beta=1.0, mode=C.GROUPED_M, M=R, N=d, Kd=f, groups=nl, lda=f, ldb=f,
               ldc=d, ldd=d, b_gs=d * f, tile_group=tile_group, num_m_tiles=nmt, row_ptr=row_ptr)
        buf.barrier()
        dx = K.moe_combine(buf.ret, pos, None, T, k)
        dwts = None
        if Yret.numel():
            dwts = K.moe_combine_dw(Yret, dout, pos, k).view(T, k).to(ctx.wdtype)
        kb = offs_l[:nl].contiguous()
        kl = (offs_l[1:] - offs_l[:nl]).contiguous()
        H = K.swiglu_fwd(G, U, meta_l[1:2])
        dw1, dw2, dw3 = torch.empty_like(w1), torch.empty_like(w2), torch.empty_like(w3)
        common = dict(mode=C.BATCHED, groups=nl, a_major=C.MAJ_MN, b_major=C.MAJ_MN, Kd=R, k_begin=kb, k_len=kl)
        C.gemm(Xp, dG, dw1, M=d, N=f, lda=d, ldb=f, ldc=f, c_gs=d * f, **common)
        C.gemm(Xp, dU, dw2, M=d, N=f, lda=d, ldb=f, ldc=f, c_gs=d * f, **common)
        C.gemm(H, dYp, dw3, M=f, N=d, lda=f, ldb=d, ldc=d, c_gs=f * d, **common)
        C._count(8)
        return dx, dw1, dw2, dw3, None, dwts, None, None


class _EPFusedFFNMX(torch.autograd.Function):
    """Same exchange, expert GEMMs (forward, dgrad, wgrad) on the block-scaled fp8 path (e4m3 values, one
    e8m0 scale per 32 elements along the reduction, fp32 accumulation, bf16 results).  Rows cross NVLink in
    bf16 and are quantised on the expert rank, where each operand is quantised once per orientation; the
    second GEMM's rows go back to their source ranks with the return kernel instead of a GEMM epilogue."""

    @staticmethod
    def forward(ctx, x, w1, w2, w3, idx, weights, keep, buf: EPBuffers):
        from ..ops import cuda_ops as C
        from ..ops import mxfp8 as MX
        K = torch.ops.kmoe
        T, d = x.shape
        nl, _, f = w1.shape
        k = idx.shape[1]
        E, ws = buf.E, buf.world
        pos, row_src, counts, offsets, _tg, _meta = K.moe_plan(
            idx.reshape(-1).contiguous(), keep.reshape(-1) if keep is not None else None, E, 0)
        assert row_src.numel() <= buf.max_rows_src
        K.ep_dispatch(x.contiguous(), row_src, None, offsets, counts, buf.recv_ptrs, buf.meta_ptrs, buf.rank, ws, E,
                      buf.cap, k)
        buf.barrier()
        R = buf.max_rows_exp
        meta_in = buf.meta.clone()
        slot_dst, offs_l, tile_group, meta_l = K.ep_recv_plan(meta_in, nl, ws, R)
        nmt, live = meta_l[0:1], meta_l[1:2]
        Xp = torch.empty(R, d, dtype=x.dtype, device=x.device)
        K.ep_move(buf.recv, Xp, meta_in, slot_dst, offs_l, buf.ret_ptrs, buf.rank, nl, ws, buf.cap, 0, None)
        grp = dict(mode=C.GROUPED_M, groups=nl, b_grouped=True, tile_group=tile_group, num_m_tiles=nmt)
        Xq, sX = MX.quant_rows(Xp, live_rows=live)
        W1q, s1 = MX._weight_quant(w1, "cols")
        W2q, s2 = MX._weight_quant(w2, "cols")
        G = torch.empty(R, f, dtype=x.dtype, device=x.device)
        U = torch.empty_like(G)
        MX.gemm_mx(Xq, sX, W1q, s1, G, M=R, N=f, K=d, **grp)
        MX.gemm_mx(Xq, sX, W2q, s2, U, M=R, N=f, K=d, **grp)
        Hq, sH = MX.quant_rows(G, U, live_rows=live)          # SwiGLU fused into the quantiser
        W3q, s3 = MX._weight_quant(w3, "cols")
        Y = torch.empty(R, d, dtype=x.dtype, device=x.device)
        MX.gemm_mx(Hq, sH, W3q, s3, Y, M=R, N=d, K=f, **grp)
        K.ep_move(buf.recv, Y, meta_in, slot_dst, offs_l, buf.ret_ptrs, buf.rank, nl, ws, buf.cap, 1, None)
        buf.barrier()
        wf = weights.reshape(-1).float().contiguous()
        out = K.moe_combine(buf.ret, pos, wf, T, k)
        Yret = buf.ret[: row_src.numel()].clone() if ctx.needs_input_grad[5] else None
        C._count(6)
        ctx.save_for_backward(Xp, G, U, w1, w2, w3, wf, pos, row_src, counts, offsets, meta_in, slot_dst, offs_l,
                              tile_group, meta_l, Yret if Yret is not None else torch.empty(0, device=x.device))
        ctx.buf = buf
        ctx.dims = (T, d, nl, f, k, R)
        ctx.wdtype = weights.dtype
        return out

    @staticmethod
    def backward(ctx, dout):
        from ..ops import cuda_ops as C
        from ..ops import mxfp8 as MX
        K = torch.ops.kmoe
        (Xp, G, U, w1, w2, w3, wf, pos, row_src, counts, offsets, meta_in, slot_dst, offs_l, tile_group, meta_l,
         Yret) = ctx.saved_tensors
        buf = ctx.buf
        T, d, nl, f, k, R = ctx.dims
        E, ws = buf.E, buf.world
        dout = dout.contiguous()
        nmt, live = meta_l[0:1], meta_l[1:2]
        grp = dict(mode=C.GROUPED_M, groups=nl, b_grouped=True, tile_group=tile_group, num_m_tiles=nmt)
        K.ep_dispatch(dout, row_src, wf, offsets, counts, buf.recv_ptrs, buf.meta_ptrs, buf.rank, ws, E, buf.cap, k)
        buf.barrier()
        dYp = torch.empty(R, d, dtype=dout.dtype, device=dout.device)
        K.ep_move(buf.recv, dYp, meta_in, slot_dst, offs_l, buf.ret_ptrs, buf.rank, nl, ws, buf.cap, 0, None)
        dYq, sdY = MX.quant_rows(dYp, live_rows=live)
        W3r, s3r = MX._weight_quant(w3, "rows")
        dH = torch.empty(R, f, dtype=dout.dtype, device=dout.device)
        MX.gemm_mx(dYq, sdY, W3r, s3r, dH, M=R, N=f, K=d, **grp)
        dG, dU = K.swiglu_bwd(G, U, dH, live)
        dGq, sdG = MX.quant_rows(dG, live_rows=live)
        dUq, sdU = MX.quant_rows(dU, live_rows=live)
        W1r, s1r = MX._weight_quant(w1, "rows")
        W2r, s2r = MX._weight_quant(w2, "rows")
        dXp = torch.empty(R, d, dtype=dout.dtype, device=dout.device)
        MX.gemm_mx(dGq, sdG, W1r, s1r, dXp, M=R, N=d, K=f, **grp)
        MX.gemm_mx(dUq, sdU, W2r, s2r, dXp, D=dXp, beta=1.0, M=R, N=d, K=f, **grp)
        K.ep_move(buf.recv, dXp, meta_in, slot_dst, offs_l, buf.ret_ptrs, buf.rank, nl, ws, buf.cap, 1, None)
        buf.barrier()
        dx = K.moe_combine(buf.ret, pos, None, T, k)
        dwts = None
        if Yret.numel():
            dwts = K.moe_combine_dw(Yret, dout, pos, k).view(T, k).to(ctx.wdtype)
        kb = offs_l[:nl].contiguous()
        kl = (offs_l[1:] - offs_l[:nl]).contiguous()
        H = K.swiglu_fwd(G, U, live)
        XT, sXT = MX.quant_cols(Xp, live_rows=live)
        dGT, sdGT = MX.quant_cols(dG, live_rows=live)
        dUT, sdUT = MX.quant_cols(dU, live_rows=live)
        HT, sHT = MX.quant_cols(H, live_rows=live)
        dYT, sdYT = MX.quant_cols(dYp, live_rows=live)
        dw1, dw2, dw3 = torch.empty_like(w1), torch.empty_like(w2), torch.empty_like(w3)
        bat = dict(mode=C.BATCHED, groups=nl, k_begin=kb, k_len=kl, K=R)
        MX.gemm_mx(XT, sXT, dGT, sdGT, dw1, M=d, N=f, c_gs=d * f, **bat)
        MX.gemm_mx(XT, sXT, dUT, sdUT, dw2, M=d, N=f, c_gs=d * f, **bat)
        MX.gemm_mx(HT, sHT, dYT, sdYT, dw3, M=f, N=d, c_gs=f * d, **bat)
        C._count(8)
        return dx, dw1, dw2, dw3, None, dwts, None, None


def fused_available(x: torch.Tensor, w1: torch.Tensor, moe_dtype: str = "bf16") -> bool:
    from .p2p import p2p_available
    d, f = w1.shape[1], w1.shape[2]
    gran = 128 if moe_dtype == "mxfp8" else 64
    return (x.is_cuda and x.dtype == torch.bfloat16 and w1.dtype == torch.bfloat16 and d % gran == 0
            and f % gran == 0 and p2p_available(x.device))


def expert_parallel_ffn_fused(x, idx, weights, w1, w2, w3, n_experts: int, group=None, keep=None,
                              slot_cap: Optional[int] = None, moe_dtype: str = "bf16"):
    """x (T, d) bf16; idx, weights (T, k) with global expert ids; w* are this rank's expert weights
    (E / world, d, f) / (E / world, f, d).  Every rank of the group must call it with the same T.
    ``slot_cap``: upper bound on the assignments one rank sends to one expert (the capacity when ``keep``
    enforces one); it sizes the receive slots and the expert-side buffers, which default to the worst case T.
    ``moe_dtype="mxfp8"`` runs the expert GEMMs block-scaled in fp8 (d and f multiples of 128)."""
    from ..ops import checks
    if checks.enabled():
        checks.expert_indices(idx, n_experts)          # distinct per token: a source sends an expert at most T rows
        checks.routing_weights(weights)
        checks.keep_mask(keep, idx)
    T, d = x.shape
    cap = None if slot_cap is None else min(int(slot_cap), T)
    buf = get_buffers(T, idx.shape[1], d, n_experts, x.dtype, x.device, group, cap)
    fn = _EPFusedFFNMX if moe_dtype == "mxfp8" else _EPFusedFFN
    return fn.apply(x, w1.contiguous(), w2.contiguous(), w3.contiguous(), idx, weights, keep, buf)
