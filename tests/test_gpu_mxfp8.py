"""MXFP8 kernels: the quantisers against the PyTorch definition of the number format (bit-exact values
and scales), the block-scaled tcgen05 GEMM against an fp32 matmul of the dequantised operands, and the
expert FFN built from them against the bf16 path."""
import pytest
import torch

pytestmark = pytest.mark.gpu


def _mods():
    from kolmogorov_moe_architecture_b200.ops import cuda_ops, eager, mxfp8
    return cuda_ops, eager, mxfp8


def _deq(q, exps, dim=-1):
    """e4m3 tensor and per-32-block exponents along ``dim`` -> fp32."""
    qf = q.float().movedim(dim, -1)
    sc = torch.exp2(exps.float()).repeat_interleave(32, dim=-1)
    return (qf * sc).movedim(-1, dim)


def test_quant_rows_matches_definition():
    c, eager, mx = _mods()
    torch.manual_seed(0)
    x = (torch.randn(300, 384, device="cuda") * torch.logspace(-3, 2, 384, device="cuda")).bfloat16()
    x[5, 32:64] = 0                                       # an all-zero block
    q, sf = mx.quant_rows(x)
    qr, er = mx.quantize_mx(x, -1)
    assert torch.equal(q.view(torch.uint8), qr.view(torch.uint8))
    assert torch.equal(mx.decode_scale_chunks(sf, 300, 384), er.to(torch.int32))


def test_quant_cols_matches_definition():
    c, eager, mx = _mods()
    torch.manual_seed(1)
    x = (torch.randn(3, 256, 128, device="cuda") * 3).bfloat16()
    q, sf = mx.quant_cols(x)                              # (3, 128, 256), reduction along the 256
    qr, er = mx.quantize_mx(x, 1)                         # same values, untransposed
    assert torch.equal(q.view(torch.uint8), qr.transpose(1, 2).contiguous().view(torch.uint8))
    exps = mx.decode_scale_chunks(sf, 3 * 128, 256).view(3, 128, 8)
    assert torch.equal(exps, er.to(torch.int32))


def test_swiglu_quant_fused():
    c, eager, mx = _mods()
    torch.manual_seed(2)
    g = torch.randn(200, 256, device="cuda").bfloat16()
    u = torch.randn(200, 256, device="cuda").bfloat16()
    q, sf = mx.quant_rows(g, u)
    h = c.swiglu(g, u)
    qr, er = mx.quantize_mx(h, -1)
    same = (q.view(torch.uint8) == qr.view(torch.uint8)).float().mean().item()
    assert same > 0.995                                   # silu differs in the last bit now and then
    assert (mx.decode_scale_chunks(sf, 200, 256) - er.to(torch.int32)).abs().max().item() <= 1


@pytest.mark.parametrize("M,N,K", [(128, 128, 128), (300, 520, 384), (1024, 2048, 2816)])
def test_gemm_mxfp8_dense(M, N, K):
    c, eager, mx = _mods()
    torch.manual_seed(3)
    a = (torch.randn(M, K, device="cuda") * torch.logspace(-1, 1, K, device="cuda")).bfloat16()
    b = torch.randn(N, K, device="cuda").bfloat16()
    aq, sa = mx.quant_rows(a)
    bq, sb = mx.quant_rows(b)
    out = mx.gemm_mx(aq, sa, bq, sb, torch.empty(M, N, dtype=torch.float32, device="cuda"), M=M, N=N, K=K)
    c.check_status()
    ref = _deq(aq, mx.decode_scale_chunks(sa, M, K)) @ _deq(bq, mx.decode_scale_chunks(sb, N, K)).t()
    err = (out - ref).abs().max().item()
    assert err <= 2e-4 * ref.abs().max().item() + 1e-5, (err, ref.abs().max().item())
    # and with bf16 output + accumulate-into
    d0 = torch.randn(M, N, device="cuda").bfloat16()
    out2 = mx.gemm_mx(aq, sa, bq, sb, torch.empty(M, N, dtype=torch.bfloat16, device="cuda"), M=M, N=N, K=K, D=d0,
                      alpha=0.5, beta=1.0)
    ref2 = 0.5 * ref + d0.float()
    assert (out2.float() - ref2).abs().max().item() <= 1e-2 * ref2.abs().max().item()


def test_gemm_mxfp8_ragged_batched():
    """wgrad shape: per group g, C[g] = A[:, k0:k0+len] B[:, k0:k0+len]^T."""
    c, eager, mx = _mods()
    torch.manual_seed(4)
    M, N, R = 256, 128, 1024
    a = torch.randn(R, M, device="cuda").bfloat16()
    b = torch.randn(R, N, device="cuda").bfloat16()
    aT, sa = mx.quant_cols(a)                             # (M, R)
    bT, sb = mx.quant_cols(b)                             # (N, R)
    kb = torch.tensor([0, 384, 384, 640], dtype=torch.int32, device="cuda")
    kl = torch.tensor([384, 0, 256, 384], dtype=torch.int32, device="cuda")
    out = torch.full((4, M, N), 7.0, dtype=torch.float32, device="cuda")
    mx.gemm_mx(aT, sa, bT, sb, out, M=M, N=N, K=R, mode=c.BATCHED, groups=4, c_gs=M * N, k_begin=kb, k_len=kl)
    c.check_status()
    A = _deq(aT, mx.decode_scale_chunks(sa, M, R))
    B = _deq(bT, mx.decode_scale_chunks(sb, N, R))
    for g in range(4):
        k0, ln = int(kb[g]), int(kl[g])
        ref = A[:, k0:k0 + ln] @ B[:, k0:k0 + ln].t()
        assert (out[g] - ref).abs().max().item() <= 2e-4 * max(ref.abs().max().item(), 1.0)


def _fq(t, dim, mx):
    q, e = mx.quantize_mx(t, dim)
    return mx.dequantize_mx(q, e, dim, torch.float32)


@pytest.mark.parametrize("T,E,k", [(500, 4, 2), (64, 8, 2)])
def test_grouped_swiglu_mxfp8(T, E, k):
    """Forward against a PyTorch evaluation that rounds the same operands to MXFP8 at the same points
    (tight); gradients against the bf16 path (loose: three chained fp8 GEMMs carry a few percent of
    rounding noise, a layout error would be of order one)."""
    c, eager, mx = _mods()
    torch.manual_seed(5)
    d, f = 256, 384
    x = torch.randn(T, d, device="cuda").bfloat16().requires_grad_(True)
    ws = [(torch.randn(E, d, f, device="cuda") * 0.06).bfloat16().requires_grad_(True),
          (torch.randn(E, d, f, device="cuda") * 0.06).bfloat16().requires_grad_(True),
          (torch.randn(E, f, d, device="cuda") * 0.06).bfloat16().requires_grad_(True)]
    logits = torch.randn(T, E, device="cuda")
    wts, idx = torch.softmax(logits, -1).topk(k, dim=-1)
    wts = wts.bfloat16().requires_grad_(True)
    g = torch.randn(T, d, device="cuda").bfloat16()
    res = {}
    for mode in ("mxfp8", "bf16"):
        for t in [x, wts] + ws:
            t.grad = None
        out = c.grouped_swiglu(x, ws[0], ws[1], ws[2], idx, wts, None, mode)
        out.backward(g)
        c.check_status()
        res[mode] = [out.detach().float(), x.grad.float(), wts.grad.float()] + [w.grad.float() for w in ws]
    # forward oracle
    with torch.no_grad():
        xd = _fq(x.detach(), -1, mx)
        w1d, w2d, w3d = _fq(ws[0].detach(), 1, mx), _fq(ws[1].detach(), 1, mx), _fq(ws[2].detach(), 1, mx)
        ref = torch.zeros(T, d, device="cuda")
        for e in range(E):
            tok, slot = (idx == e).nonzero(as_tuple=True)
            if tok.numel() == 0:
                continue
            G = (xd[tok] @ w1d[e]).bfloat16().float()
            U = (xd[tok] @ w2d[e]).bfloat16().float()
            H = (torch.nn.functional.silu(G) * U).bfloat16()
            Y = (_fq(H, -1, mx) @ w3d[e]).bfloat16().float()
            ref.index_add_(0, tok, Y * wts.detach()[tok, slot].float().unsqueeze(1))
    err = (res["mxfp8"][0] - ref).norm().item() / ref.norm().item()
    assert err < 1e-2, ("forward vs MXFP8 oracle", err)
    for name, a, b in zip(["out", "dx", "dw", "dW1", "dW2", "dW3"], res["mxfp8"], res["bf16"]):
        err = (a - b).norm().item() / (b.norm().item() + 1e-9)
        assert err < 0.15, (name, err)


def test_linear_mxfp8_fwd_bwd():
    """FP8Linear on the tensor-core path: forward, dgrad and wgrad against the bf16 linear layer."""
    c, eager, mx = _mods()
    torch.manual_seed(6)
    x = torch.randn(256, 384, device="cuda").bfloat16().requires_grad_(True)
    w = (torch.randn(512, 384, device="cuda") * 0.05).bfloat16().requires_grad_(True)
    g = torch.randn(256, 512, device="cuda").bfloat16()
    y = mx.linear_mx(x, w)
    y.backward(g)
    c.check_status()
    xr, wr = x.detach().float().requires_grad_(True), w.detach().float().requires_grad_(True)
    yr = xr @ wr.t()
    yr.backward(g.float())
    for name, a, b in (("y", y, yr), ("dx", x.grad, xr.grad), ("dw", w.grad, wr.grad)):
        err = (a.float() - b).norm().item() / b.norm().item()
        assert err < 5e-2, (name, err)
    # odd sizes take the fake-quantised bf16 route
    x2 = torch.randn(10, 384, device="cuda").bfloat16()
    assert mx.linear_mx(x2, w).shape == (10, 512)
