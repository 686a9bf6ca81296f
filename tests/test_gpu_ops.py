"""Each CUDA kernel against the plain-PyTorch definition of the same op evaluated in fp32
(forward and backward), on small, ragged and empty-expert shapes."""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu


def _mods():
    from kolmogorov_moe_architecture_b200 import ops
    from kolmogorov_moe_architecture_b200.ops import cuda_ops, eager
    return ops, cuda_ops, eager


def _bf(*shape, scale=1.0, grad=False):
    t = (torch.randn(*shape, device="cuda") * scale).to(torch.bfloat16)
    return t.requires_grad_(grad)


def _rel(a, b):
    """Worst element of |a - b| / (|b| + rms(b)): a relative error where the reference is large and an
    absolute one, in units of the reference's typical magnitude, where it is small.  (Dividing by the
    largest reference value instead would let an op that is wrong on its small outputs pass.)"""
    a, b = a.float(), b.float()
    rms = b.pow(2).mean().sqrt() + 1e-12
    return ((a - b).abs() / (b.abs() + rms)).max().item()


def _f32_leaf(t):
    return t.detach().float().requires_grad_(True)


@pytest.mark.parametrize("d", [512, 2048, 1024, 256, 384])
def test_rmsnorm_fwd_bwd(d):
    """Widths 256 / 512 / 1024 / 2048 run the register-resident kernels (one pass, weight gradient included),
    384 the generic ones."""
    ops, c, eager = _mods()
    x, w = _bf(37, 5, d, grad=True), _bf(d, grad=True)
    y = ops.rmsnorm(x, w, 1e-5)
    g = _bf(37, 5, d)
    y.backward(g)
    xr, wr = _f32_leaf(x), _f32_leaf(w)
    yr = eager.rmsnorm(xr, wr, 1e-5)
    yr.backward(g.float())
    assert _rel(y, yr) < 1e-2 and _rel(x.grad, xr.grad) < 2e-2 and _rel(w.grad, wr.grad) < 2e-2


def test_rope_fwd_bwd():
    ops, c, eager = _mods()
    B, S, H, D = 2, 33, 3, 64
    cos, sin = eager.rope_tables(D, 64, 10000.0, device="cuda")
    x = _bf(B, S, H, D, grad=True)
    y = ops.rope_apply(x, cos[:S], sin[:S])
    g = _bf(B, S, H, D)
    y.backward(g)
    xr = _f32_leaf(x)
    yr = eager.rope_apply(xr, cos[:S], sin[:S])
    yr.backward(g.float())
    assert _rel(y, yr) < 1e-2 and _rel(x.grad, xr.grad) < 1e-2
    pid = torch.randint(0, 64, (B, S), device="cuda")
    y2 = ops.rope_apply(x.detach(), cos[pid], sin[pid])
    assert _rel(y2, eager.rope_apply(x.detach().float(), cos[pid], sin[pid])) < 1e-2


def test_swiglu_fwd_bwd_strided():
    ops, c, eager = _mods()
    gu = _bf(50, 2 * 264, grad=True)
    g_, u_ = gu.chunk(2, dim=-1)
    h = ops.swiglu(g_, u_)
    go = _bf(50, 264)
    h.backward(go)
    r = _f32_leaf(gu)
    a, b = r.chunk(2, dim=-1)
    hr = eager.swiglu(a, b)
    hr.backward(go.float())
    assert _rel(h, hr) < 1e-2 and _rel(gu.grad, r.grad) < 2e-2


@pytest.mark.parametrize("S", [7, 64, 130])
def test_causal_conv1d(S):
    ops, c, eager = _mods()
    B, C = 2, 192
    xz = _bf(B, S, 2 * C, grad=True)
    w = torch.randn(C, 4, device="cuda", requires_grad=True)
    b = torch.randn(C, device="cuda", requires_grad=True)
    x = xz[..., :C]
    y = ops.causal_conv1d(x, w, b, True)
    go = _bf(B, S, C)
    y.backward(go)
    xr, wr, br = _f32_leaf(xz), _f32_leaf(w), _f32_leaf(b)
    yr = eager.causal_conv1d(xr[..., :C], wr, br, True)
    yr.backward(go.float())
    assert _rel(y, yr) < 1e-2
    assert _rel(xz.grad, xr.grad) < 2e-2 and _rel(w.grad, wr.grad) < 2e-2 and _rel(b.grad, br.grad) < 2e-2


@pytest.mark.parametrize("S,C", [(16, 64), (45, 96), (128, 256)])
def test_selective_scan(S, C):
    ops, c, eager = _mods()
    B, N = 2, 16
    u = _bf(B, S, C, grad=True)
    delta = _bf(B, S, C, scale=0.5, grad=True)
    xz = _bf(B, S, 2 * C, grad=True)
    z = xz[..., C:]
    A = (-torch.exp(torch.randn(C, N, device="cuda") * 0.5)).requires_grad_(True)
    Bm = _bf(B, S, N, grad=True)
    Cm = _bf(B, S, N, grad=True)
    D = torch.randn(C, device="cuda", requires_grad=True)
    bias = torch.randn(C, device="cuda", requires_grad=True)
    y = ops.selective_scan(u, delta, A, Bm, Cm, D, z, bias, True)
    go = _bf(B, S, C)
    y.backward(go)
    leaves = [_f32_leaf(t) for t in (u, delta, A, Bm, Cm, D, xz, bias)]
    ur, dr, Ar, Br, Cr, Dr, xzr, br = leaves
    yr = eager.selective_scan(ur, dr, Ar, Br, Cr, Dr, xzr[..., C:], br, True)
    yr.backward(go.float())
    assert _rel(y, yr) < 2e-2
    for name, a, b in [("u", u, ur), ("delta", delta, dr), ("A", A, Ar), ("B", Bm, Br), ("C", Cm, Cr),
                       ("D", D, Dr), ("z", xz, xzr), ("bias", bias, br)]:
        assert _rel(a.grad, b.grad) < 4e-2, name


def test_conv_and_scan_with_parameter_sets_over_the_batch():
    """(G, C, ...) parameters: every slice of B / G batch entries uses its own set, forward and all gradients
    (the fp32 definition applies the sets slice by slice)."""
    ops, c, eager = _mods()
    G, Bg, S, C, N = 3, 2, 45, 96, 16
    B = G * Bg
    xz = _bf(B, S, 2 * C, grad=True)
    w = torch.randn(G, C, 4, device="cuda", requires_grad=True)
    b = torch.randn(G, C, device="cuda", requires_grad=True)
    y = ops.causal_conv1d(xz[..., :C], w, b, True)
    go = _bf(B, S, C)
    y.backward(go)
    xr, wr, br = _f32_leaf(xz), _f32_leaf(w), _f32_leaf(b)
    yr = eager.causal_conv1d(xr[..., :C], wr, br, True)
    yr.backward(go.float())
    assert _rel(y, yr) < 1e-2 and _rel(xz.grad, xr.grad) < 2e-2
    assert _rel(w.grad, wr.grad) < 2e-2 and _rel(b.grad, br.grad) < 2e-2
    u = _bf(B, S, C, grad=True)
    delta = _bf(B, S, C, scale=0.5, grad=True)
    z2 = _bf(B, S, 2 * C, grad=True)
    A = (-torch.exp(torch.randn(G, C, N, device="cuda") * 0.5)).requires_grad_(True)
    Bm, Cm = _bf(B, S, N, grad=True), _bf(B, S, N, grad=True)
    D = torch.randn(G, C, device="cuda", requires_grad=True)
    bias = torch.randn(G, C, device="cuda", requires_grad=True)
    y = ops.selective_scan(u, delta, A, Bm, Cm, D, z2[..., C:], bias, True)
    y.backward(go)
    ur, dr, Ar, Br, Cr, Dr, zr, bir = [_f32_leaf(t) for t in (u, delta, A, Bm, Cm, D, z2, bias)]
    yr = eager.selective_scan(ur, dr, Ar, Br, Cr, Dr, zr[..., C:], bir, True)
    yr.backward(go.float())
    assert _rel(y, yr) < 2e-2
    for name, a_, b_ in [("u", u, ur), ("delta", delta, dr), ("A", A, Ar), ("B", Bm, Br), ("C", Cm, Cr),
                         ("D", D, Dr), ("z", z2, zr), ("bias", bias, bir)]:
        assert _rel(a_.grad, b_.grad) < 4e-2, name
    # the sets really differ per slice: swapping two sets changes those slices only
    with torch.no_grad():
        A2 = A.detach().clone()
        A2[[0, 1]] = A2[[1, 0]]
        y2 = ops.selective_scan(u, delta, A2, Bm, Cm, D, z2[..., C:], bias, True)
    assert torch.equal(y2[2 * Bg:], y.detach()[2 * Bg:]) and not torch.equal(y2[:Bg], y.detach()[:Bg])


def test_routing_mamba_batched_pass_on_the_kernels():
    import kolmogorov_moe_architecture_b200 as kmoe
    from kolmogorov_moe_architecture_b200.models.mamba import RoutingMamba
    cfg = kmoe.get_tiny_debug_config(vocab_size=128, d_model=128, n_heads=2, n_kv_heads=1, head_dim=64, d_ff=256,
                                     d_ff_expert=128, max_seq_len=64, n_pred_tokens=1, aux_loss_weights=(1.0,))
    torch.manual_seed(0)
    m = RoutingMamba(cfg, 1).cuda().to(torch.bfloat16).train()
    x = _bf(2, 64, 128, grad=True)
    go = _bf(2, 64, 128)
    res = {}
    for flag in (False, True):
        m.batched = flag
        m.zero_grad()
        x.grad = None
        y = m(x)
        y.backward(go)
        res[flag] = (y.detach().float(), x.grad.float(), {n: p.grad.float() for n, p in m.named_parameters() if p.grad is not None})
    a, b = res[False], res[True]
    assert _rel(b[0], a[0]) < 2e-2 and _rel(b[1], a[1]) < 3e-2
    assert set(a[2]) == set(b[2]) and all(_rel(b[2][n], a[2][n]) < 5e-2 for n in a[2])


@pytest.mark.parametrize("T,E,k,drop", [(300, 4, 2, False), (64, 8, 2, False), (513, 4, 1, True)])
def test_grouped_swiglu_fwd_bwd(T, E, k, drop):
    ops, c, eager = _mods()
    d, f = 128, 192
    x = _bf(T, d, scale=0.5, grad=True)
    w1, w2 = _bf(E, d, f, scale=0.08, grad=True), _bf(E, d, f, scale=0.08, grad=True)
    w3 = _bf(E, f, d, scale=0.08, grad=True)
    logits = torch.randn(T, E, device="cuda")
    logits[:, 1] -= 100.0                      # expert 1 never selected: an empty group
    wts, idx = eager.topk_softmax_route(logits, k)
    wts = wts.requires_grad_(True)
    keep = eager.capacity_keep_mask(idx, E, max(1, T * k // E // 2)) if drop else None
    out = ops.grouped_swiglu(x, w1, w2, w3, idx, wts, keep)
    go = _bf(T, d)
    out.backward(go)
    c.check_status()
    xr, a1, a2, a3, wr = [_f32_leaf(t) for t in (x, w1, w2, w3, wts)]
    ref = eager.grouped_swiglu(xr, a1, a2, a3, idx, wr, keep)
    ref.backward(go.float())
    assert _rel(out, ref) < 2e-2
    for name, a, b in [("x", x, xr), ("w1", w1, a1), ("w2", w2, a2), ("w3", w3, a3), ("wts", wts, wr)]:
        assert _rel(a.grad, b.grad) < 4e-2, name
    # determinism: the same call twice gives identical bits
    out2 = ops.grouped_swiglu(x, w1, w2, w3, idx, wts, keep)
    assert torch.equal(out, out2)


def test_mtp_cross_entropy():
    ops, c, eager = _mods()
    B, S, d, V, nh = 2, 40, 128, 320, 3
    h = _bf(B, S, d, grad=True)
    Ws = [_bf(V, d, scale=0.2, grad=True) for _ in range(nh)]
    labels = torch.randint(0, V, (B, S), device="cuda")
    labels[0, 5:9] = -100
    wts = (0.5, 0.3, 0.2)
    total, per = ops.mtp_cross_entropy(h, Ws, labels, wts, -100)
    (total * 2.0).backward()
    c.check_status()
    hr = _f32_leaf(h)
    Wr = [_f32_leaf(w) for w in Ws]
    tr, pr = eager.mtp_cross_entropy(hr, Wr, labels, wts, -100)
    (tr * 2.0).backward()
    assert abs(total.item() - tr.item()) < 2e-2 * abs(tr.item())
    assert _rel(per, pr) < 2e-2
    assert _rel(h.grad, hr.grad) < 4e-2
    for a, b in zip(Ws, Wr):
        assert _rel(a.grad, b.grad) < 4e-2


@pytest.mark.parametrize("shape", [(256, 512), (512, 256), (3, 128, 320), (2, 320, 128), (3, 256, 704),
                                   (2, 704, 256), (2, 512, 512), (1, 512, 2048), (4, 160, 1024), (3, 16, 128),
                                   (5, 1, 256), (2, 192, 1)])
@pytest.mark.parametrize("with_sumsq", [False, True])
def test_newton_schulz(shape, with_sumsq):
    """Five cubic Newton-Schulz steps against the fp32 definition.  Shapes whose long side is at least 1.25x the
    short one (and at least 256 on the short side) take the path that iterates on the short side; the others
    the step-by-step path; sizes that are not multiples of 64 are zero-padded, vectors are only normalised.
    ``with_sumsq``: the norm comes in as a device scalar and is folded into the GEMMs."""
    ops, c, eager = _mods()
    torch.manual_seed(13)
    m = torch.randn(*shape, device="cuda").to(torch.bfloat16)
    if len(shape) == 3 and min(shape[1:]) > 4:
        m[0, :4] *= 20.0                                   # a few dominant directions in one matrix of the stack
    sumsq = None
    if with_sumsq:
        sumsq = m.float().reshape(1 if len(shape) == 2 else shape[0], -1).pow(2).sum(dim=-1)
    out = ops.newton_schulz(m, 5, sumsq=sumsq)
    c.check_status()
    ref = eager.newton_schulz(m.float(), 5)
    assert out.shape == m.shape and out.dtype == m.dtype
    assert _rel(out, ref) < 5e-2
    assert ((out.float() - ref).norm() / ref.norm()).item() < 1e-2


def test_model_step_bf16_matches_eager():
    """One forward/backward of a small hybrid model through the kernels vs the same
    weights through the PyTorch definitions in fp32."""
    import os
    from kolmogorov_moe_architecture_b200 import AdvancedMoEConfig, MoETransformer
    cfg = AdvancedMoEConfig(vocab_size=1024, d_model=256, n_layers=4, n_heads=4, n_kv_heads=2, head_dim=64,
                            d_ff=512, d_ff_expert=256, n_experts=4, moe_layers=(1, 2), mamba_layers=(1,),
                            max_seq_len=128, n_pred_tokens=2, aux_loss_weights=(1.0, 0.5),
                            mamba_moe_mode="moe_ffn", dropout=0.0, attention_dropout=0.0, residual_dropout=0.0)
    torch.manual_seed(0)
    ref = MoETransformer(cfg, verbose=False).cuda()
    model = MoETransformer(cfg, verbose=False).cuda()
    model.load_state_dict(ref.state_dict())
    model = model.to(torch.bfloat16)
    ids = torch.randint(0, cfg.vocab_size, (2, 128), device="cuda")
    model.train()
    ref.train()
    out = model(ids, labels=ids, return_logits=False)
    out["loss"].backward()
    os.environ["KMOE_STRICT"] = "0"
    o2 = ref(ids, labels=ids, return_logits=False)
    assert abs(out["lm_loss"].item() - o2["lm_loss"].item()) < 0.05
    assert all(p.grad is not None and torch.isfinite(p.grad).all() for p in model.parameters())


@pytest.mark.parametrize("B,S,H,Hkv,D", [(1, 128, 2, 1, 64), (2, 200, 4, 2, 128), (1, 512, 4, 1, 128),
                                         (2, 333, 2, 2, 64), (1, 1300, 8, 2, 128)])
def test_flash_attention_fwd_bwd(B, S, H, Hkv, D):
    ops, c, eager = _mods()
    torch.manual_seed(11)
    q, k, v = _bf(B, S, H, D, grad=True), _bf(B, S, Hkv, D, grad=True), _bf(B, S, Hkv, D, grad=True)
    out = ops.attention(q, k, v, causal=True)
    go = _bf(B, S, H, D)
    out.backward(go)
    c.check_status()
    qr, kr, vr = _f32_leaf(q), _f32_leaf(k), _f32_leaf(v)
    ref = eager.attention(qr, kr, vr, True)
    ref.backward(go.float())
    assert _rel(out, ref) < 2e-2
    # worst element over ~10^5 outputs: P, dS and the results themselves are rounded to bf16
    assert _rel(q.grad, qr.grad) < 5e-2, "dq"
    assert _rel(k.grad, kr.grad) < 5e-2, "dk"
    assert _rel(v.grad, vr.grad) < 5e-2, "dv"
    # and the bulk of the elements is far inside that bound
    for g, gr in ((q.grad, qr.grad), (k.grad, kr.grad), (v.grad, vr.grad)):
        assert ((g.float() - gr).abs().mean() / gr.abs().mean()).item() < 1e-2


@pytest.mark.parametrize("T,E,k", [(777, 16, 2), (64, 8, 1), (1500, 64, 4)])
def test_route_topk_fwd_bwd(T, E, k):
    ops, c, eager = _mods()
    torch.manual_seed(3)
    logits = (torch.randn(T, E, device="cuda") * 2).requires_grad_(True)
    w, idx, aux, counts = ops.route_topk(logits, k, 0.01, 0.001)
    gw = torch.randn(T, k, device="cuda")
    (w * gw).sum().add(aux * 3.0).backward()
    lr = logits.detach().clone().requires_grad_(True)
    wr, idxr, auxr, countsr = eager.route_topk(lr, k, 0.01, 0.001)
    (wr * gw).sum().add(auxr * 3.0).backward()
    assert torch.equal(idx, idxr)
    assert torch.allclose(counts, countsr)
    assert torch.allclose(w, wr, atol=1e-5) and torch.allclose(aux, auxr, rtol=1e-4, atol=1e-6)
    assert torch.allclose(logits.grad, lr.grad, atol=2e-5, rtol=1e-3)


@pytest.mark.parametrize("B,S,k", [(3, 2048, 1536), (2, 100, 37), (1, 5, 5)])
def test_mod_route_fwd_bwd(B, S, k):
    ops, c, eager = _mods()
    torch.manual_seed(4)
    logits = torch.randn(B, S, device="cuda").requires_grad_(True)
    sidx, w, _ = ops.mod_route(logits, k)
    gw = torch.randn(B, k, device="cuda")
    (w * gw).sum().backward()
    lr = logits.detach().clone().requires_grad_(True)
    sidxr, wr, _ = eager.mod_route(lr, k)
    (wr * gw).sum().backward()
    assert torch.equal(sidx, sidxr)
    assert torch.allclose(w, wr, atol=1e-6, rtol=1e-4)
    assert torch.allclose(logits.grad, lr.grad, atol=1e-6, rtol=1e-3)


@pytest.mark.parametrize("B,S,E,C", [(2, 2048, 16, 160), (3, 50, 4, 13)])
def test_expert_choice_route_fwd_bwd(B, S, E, C):
    ops, c, eager = _mods()
    torch.manual_seed(5)
    logits = torch.randn(B, S, E, device="cuda").requires_grad_(True)
    w, tok = ops.expert_choice_route(logits, C)
    gw = torch.randn(B, E, C, device="cuda")
    (w * gw).sum().backward()
    lr = logits.detach().clone().requires_grad_(True)
    wr, tokr = eager.expert_choice_route(lr, C)
    (wr * gw).sum().backward()
    assert torch.equal(tok, tokr)
    assert torch.allclose(w, wr, atol=1e-6, rtol=1e-4)
    assert torch.allclose(logits.grad, lr.grad, atol=1e-7, rtol=2e-3)


@pytest.mark.parametrize("B,S,k,d", [(3, 64, 48, 256), (2, 2048, 1536, 512), (1, 7, 1, 64)])
def test_mod_gather_combine_fwd_bwd(B, S, k, d):
    """Mixture-of-depths row movement: gather of the kept rows and residual + scatter(w * processed)."""
    ops, c, eager = _mods()
    torch.manual_seed(6)
    h = _bf(B, S, d, grad=True)
    res = _bf(B, S, d, grad=True)
    idx = torch.stack([torch.randperm(S, device="cuda")[:k].sort().values for _ in range(B)])
    w = torch.rand(B, k, device="cuda").bfloat16().requires_grad_(True)
    lin = _bf(d, d, scale=0.05)
    picked = ops.mod_gather(h, idx)
    proc = picked @ lin
    out = ops.mod_combine(res, proc, w, idx)
    g = _bf(B, S, d)
    out.backward(g)
    hr, rr, wr = _f32_leaf(h), _f32_leaf(res), _f32_leaf(w)
    pr = eager.mod_gather(hr, idx)
    outr = eager.mod_combine(rr, pr @ lin.float(), wr, idx)
    outr.backward(g.float())
    assert torch.equal(picked.float(), pr.detach())
    assert _rel(out, outr) < 1.5e-2     # `proc` is rounded to bf16 before the combine on this side only
    assert _rel(h.grad, hr.grad) < 2e-2 and _rel(res.grad, rr.grad) < 1e-6 and _rel(w.grad, wr.grad) < 2e-2


@pytest.mark.parametrize("B,S,H,Hkv,D", [(2, 384, 4, 2, 128), (1, 200, 2, 1, 64)])
def test_flash_attention_packed_documents(B, S, H, Hkv, D):
    """Document boundaries applied inside the flash kernels (forward, dQ, dK/dV) against eager attention with
    the dense block-diagonal mask; documents start in the middle of key blocks and span several of them."""
    ops, c, eager = _mods()
    torch.manual_seed(8)
    q, k, v = _bf(B, S, H, D, grad=True), _bf(B, S, Hkv, D, grad=True), _bf(B, S, Hkv, D, grad=True)
    cuts = [[0, 37, 101, 270], [0, 150]][:B] if B > 1 else [[0, 5, 77, 140]]
    doc_ids = torch.zeros(B, S, dtype=torch.long, device="cuda")
    for b, cs in enumerate(cuts):
        for i, s0 in enumerate(cs):
            doc_ids[b, s0:] = i
    ds = eager.doc_start_from_ids(doc_ids)
    out = ops.attention(q, k, v, causal=True, doc_start=ds)
    g = _bf(B, S, H, D)
    out.backward(g)
    c.check_status()
    qr, kr, vr = _f32_leaf(q), _f32_leaf(k), _f32_leaf(v)
    outr = eager.attention(qr, kr, vr, True, eager.doc_start_to_mask(ds))
    outr.backward(g.float())
    assert _rel(out, outr) < 2e-2
    assert _rel(q.grad, qr.grad) < 4e-2 and _rel(k.grad, kr.grad) < 4e-2 and _rel(v.grad, vr.grad) < 4e-2


def test_attention_and_routing_are_bitwise_deterministic():
    """No atomics on these paths: the same call twice gives identical bits (forward and gradients)."""
    ops, c, eager = _mods()
    torch.manual_seed(9)
    q, k, v = _bf(2, 300, 4, 128, grad=True), _bf(2, 300, 2, 128, grad=True), _bf(2, 300, 2, 128, grad=True)
    g = _bf(2, 300, 4, 128)
    runs = []
    for _ in range(2):
        q.grad = k.grad = v.grad = None
        o = ops.attention(q, k, v)
        o.backward(g)
        runs.append([o.detach().clone(), q.grad.clone(), k.grad.clone(), v.grad.clone()])
    assert all(torch.equal(a, b) for a, b in zip(*runs))
    logits = torch.randn(4, 512, device="cuda")
    a1, a2 = ops.mod_route(logits, 300), ops.mod_route(logits, 300)
    assert torch.equal(a1[0], a2[0]) and torch.equal(a1[1], a2[1])


@pytest.mark.parametrize("T,din,dout", [(256, 128, 192), (200, 256, 40), (64, 64, 16), (1024, 512, 1024),
                                        (4096, 2048, 64), (3000, 512, 160), (2048, 128, 1024)])
def test_linear_fwd_bwd(T, din, dout):
    """ops.linear (tcgen05 GEMM for y, dx and dW) against F.linear in fp32; dout = 40 / 16 takes the
    transposed-dy weight-gradient path, T = 200 a ragged last row tile.  The last three shapes have a weight
    gradient of few output tiles over thousands of tokens: it is computed in slices of the token dimension
    (one batched launch plus the sum of the partial results); 3000 tokens leave a ragged last slice."""
    ops, c, eager = _mods()
    x = _bf(2, T // 2, din, grad=True)
    w = _bf(dout, din, scale=din ** -0.5, grad=True)
    n0 = c.LAUNCHES["count"]
    y = ops.linear(x, w)
    g = _bf(2, T // 2, dout)
    y.backward(g)
    split = c.split_k_parts(dout, din, T) > 1
    assert split == (T >= 2048)
    assert c.LAUNCHES["count"] - n0 == 3 + int(split), "forward, dx and dW: one GEMM launch each (+ the sum)"
    xr, wr = _f32_leaf(x), _f32_leaf(w)
    yr = F.linear(xr, wr)
    yr.backward(g.float())
    assert _rel(y, yr) < 1e-2 and _rel(x.grad, xr.grad) < 1e-2 and _rel(w.grad, wr.grad) < 1e-2


def test_linear_strided_input_and_bias():
    ops, c, eager = _mods()
    xz = _bf(4, 32, 2 * 128, grad=True)
    x = xz[..., 128:]                                   # row stride 256, width 128
    w, b = _bf(64, 128, scale=0.1, grad=True), _bf(64, grad=True)
    y = ops.linear(x, w, b)
    g = _bf(4, 32, 64)
    y.backward(g)
    r, wr, br = _f32_leaf(xz), _f32_leaf(w), _f32_leaf(b)
    yr = F.linear(r[..., 128:], wr, br)
    yr.backward(g.float())
    assert _rel(y, yr) < 1e-2 and _rel(xz.grad, r.grad) < 1e-2 and _rel(w.grad, wr.grad) < 1e-2
    assert _rel(b.grad, br.grad) < 1e-2


def test_linear_single_output_column():
    """nn.Linear(d, 1): the mixture-of-depths scorer."""
    ops, c, eager = _mods()
    x, w = _bf(3, 50, 256, grad=True), _bf(1, 256, scale=0.06, grad=True)
    y = ops.linear(x, w)
    assert y.shape == (3, 50, 1)
    g = _bf(3, 50, 1)
    y.backward(g)
    xr, wr = _f32_leaf(x), _f32_leaf(w)
    yr = F.linear(xr, wr)
    yr.backward(g.float())
    assert _rel(y, yr) < 1e-2 and _rel(x.grad, xr.grad) < 1e-2 and _rel(w.grad, wr.grad) < 1e-2
    # input that needs no gradient (the auxiliary predictor sees detached activations)
    w2 = w.detach().clone().requires_grad_(True)
    ops.linear(x.detach(), w2).backward(g)
    assert _rel(w2.grad, wr.grad) < 1e-2


@pytest.mark.parametrize("T,d,f", [(256, 128, 256), (520, 256, 704)])
def test_dense_swiglu_fwd_bwd(T, d, f):
    ops, c, eager = _mods()
    x = _bf(T, d, grad=True)
    w1, w2 = _bf(f, d, scale=d ** -0.5, grad=True), _bf(f, d, scale=d ** -0.5, grad=True)
    w3 = _bf(d, f, scale=f ** -0.5, grad=True)
    y = ops.dense_swiglu(x, w1, w2, w3)
    g = _bf(T, d)
    y.backward(g)
    xr, r1, r2, r3 = (_f32_leaf(t) for t in (x, w1, w2, w3))
    yr = F.linear(F.silu(F.linear(xr, r1)) * F.linear(xr, r2), r3)
    yr.backward(g.float())
    assert _rel(y, yr) < 2e-2 and _rel(x.grad, xr.grad) < 2e-2
    for a, b in ((w1, r1), (w2, r2), (w3, r3)):
        assert _rel(a.grad, b.grad) < 2e-2


@pytest.mark.parametrize("B,S,E,C,d,f", [(2, 64, 4, 20, 128, 192), (3, 96, 8, 12, 64, 64)])
def test_expert_choice_swiglu_fwd_bwd(B, S, E, C, d, f):
    """Expert-choice experts on the grouped kernels (batched GEMMs over the experts, deterministic combine)
    against the gather / matmul / scatter-add definition in fp32; tokens picked by several experts included."""
    ops, c, eager = _mods()
    torch.manual_seed(3)
    x = _bf(B, S, d, grad=True)
    w1, w2 = _bf(E, d, f, scale=d ** -0.5, grad=True), _bf(E, d, f, scale=d ** -0.5, grad=True)
    w3 = _bf(E, f, d, scale=f ** -0.5, grad=True)
    logits = torch.randn(B, S, E, device="cuda")
    wts, tok = eager.expert_choice_route(logits, C)
    wts = wts.bfloat16().requires_grad_(True)
    assert torch.bincount(tok.reshape(B, -1)[0], minlength=S).max() > 1      # some token has several experts
    out = ops.expert_choice_swiglu(x, w1, w2, w3, wts, tok)
    g = _bf(B, S, d)
    out.backward(g)
    c.check_status()
    xr, a1, a2, a3, wr = [_f32_leaf(t) for t in (x, w1, w2, w3, wts)]
    ref = eager.expert_choice_swiglu(xr, a1, a2, a3, wr, tok)
    ref.backward(g.float())
    assert _rel(out, ref) < 2e-2
    for name, a, b in [("x", x, xr), ("w1", w1, a1), ("w2", w2, a2), ("w3", w3, a3), ("wts", wts, wr)]:
        assert _rel(a.grad, b.grad) < 4e-2, name
    out2 = ops.expert_choice_swiglu(x, w1, w2, w3, wts, tok)
    assert torch.equal(out, out2), "the combine must be deterministic"


@pytest.mark.parametrize("T,E,k,cap", [(1000, 8, 2, 130), (64, 4, 1, 3), (513, 16, 2, 10000)])
def test_capacity_mask_and_balanced_assignment_kernels(T, E, k, cap):
    """Device-side drop decision and balanced assignment against their PyTorch definitions (exact)."""
    ops, c, eager = _mods()
    torch.manual_seed(4)
    logits = torch.randn(T, E, device="cuda")
    logits[:, 1] += 1.0                                                      # a popular expert
    idx = logits.topk(k, dim=-1).indices
    keep = ops.capacity_keep_mask(idx, E, cap)
    assert keep.dtype == torch.bool and torch.equal(keep, eager.capacity_keep_mask(idx, E, cap))
    probs = torch.softmax(logits, -1)
    got, want = ops.balanced_assign(probs, k), eager.balanced_assign(probs, k)
    assert torch.equal(got, want)
    counts = torch.bincount(got.reshape(-1), minlength=E)
    assert counts.max() <= max((T * k) // E, 1) + T        # loose: fallback picks may exceed the capacity


@pytest.mark.parametrize("with_addend", [False, True])
@pytest.mark.parametrize("d", [512, 2048, 384])
def test_residual_rmsnorm_fwd_bwd(with_addend, d):
    """Residual add + RMSNorm in one op; the residual stream h is used twice downstream (through the norm and
    around it), and both gradient paths are summed inside the backward kernel."""
    ops, c, eager = _mods()
    x, w = _bf(3, 37, d, grad=True), _bf(d, grad=True)
    a = _bf(3, 37, d, grad=True) if with_addend else None
    h, y = ops.residual_rmsnorm(x, a, w, 1e-5)
    g1, g2 = _bf(3, 37, d), _bf(3, 37, d)
    ((h * g1).sum() + (y * g2).sum()).backward()
    xr, wr = _f32_leaf(x), _f32_leaf(w)
    ar = _f32_leaf(a) if with_addend else None
    hr, yr = eager.residual_rmsnorm(xr, ar, wr, 1e-5)
    ((hr * g1.float()).sum() + (yr * g2.float()).sum()).backward()
    assert _rel(h, hr) < 1e-2 and _rel(y, yr) < 1e-2
    assert _rel(x.grad, xr.grad) < 2e-2 and _rel(w.grad, wr.grad) < 2e-2
    if with_addend:
        assert _rel(a.grad, ar.grad) < 2e-2
    # only the residual branch used downstream
    x2 = x.detach().clone().requires_grad_(True)
    h2, _ = ops.residual_rmsnorm(x2, None, w.detach(), 1e-5)
    (h2 * g1).sum().backward()
    assert _rel(x2.grad, g1) < 1e-6


@pytest.mark.parametrize("B,S,d,k", [(2, 300, 256, 225), (3, 128, 512, 96)])
def test_mod_score_gather_fwd_bwd(B, S, d, k):
    """Scorer, top-k and gather of the kept rows as one op against the separate PyTorch definitions in fp32; the
    hidden states get the scatter of the picked rows' gradient plus the scorer's rank-one term from one kernel."""
    ops, c, eager = _mods()
    torch.manual_seed(21)
    h = _bf(B, S, d, grad=True)
    w = _bf(1, d, scale=d ** -0.5, grad=True)
    picked, idx, wts, logits = ops.mod_score_gather(h, w, k)
    g1, g2 = _bf(B, k, d), torch.randn(B, k, device="cuda")
    ((picked * g1).sum() + (wts.float() * g2).sum()).backward()
    c.check_status()
    hr, wr = _f32_leaf(h), _f32_leaf(w)
    lr = F.linear(hr, wr).squeeze(-1)
    # the kernel ranks the bf16-rounded logits: give the reference the same ranking
    lq = lr.detach().to(torch.bfloat16).float()
    idx_r, _, _ = eager.mod_route(lq, k)
    assert torch.equal(idx, idx_r)
    wts_r = torch.softmax(torch.gather(lr, 1, idx_r), dim=-1)
    pr = eager.mod_gather(hr, idx_r)
    ((pr * g1.float()).sum() + (wts_r * g2).sum()).backward()
    assert torch.equal(picked.float(), pr.detach())
    assert _rel(wts, wts_r) < 2e-2 and _rel(logits, lr) < 2e-2
    assert _rel(h.grad, hr.grad) < 2e-2 and _rel(w.grad, wr.grad) < 3e-2


def test_linear_multi_fwd_bwd():
    """q / k / v style projections of one input as one autograd node against three F.linear calls in fp32."""
    ops, c, eager = _mods()
    torch.manual_seed(5)
    x = _bf(2, 100, 256, grad=True)
    ws = [_bf(n, 256, scale=256 ** -0.5, grad=True) for n in (256, 64, 64)]
    ys = ops.linear_multi(x, ws)
    gs = [_bf(2, 100, n) for n in (256, 64, 64)]
    sum((y * g).sum() for y, g in zip(ys, gs)).backward()
    c.check_status()
    xr, wrs = _f32_leaf(x), [_f32_leaf(w) for w in ws]
    yrs = [F.linear(xr, w) for w in wrs]
    sum((y * g.float()).sum() for y, g in zip(yrs, gs)).backward()
    for y, yr in zip(ys, yrs):
        assert _rel(y, yr) < 1e-2
    assert _rel(x.grad, xr.grad) < 1e-2
    for w, wr in zip(ws, wrs):
        assert _rel(w.grad, wr.grad) < 1e-2
    # only one of the outputs used downstream
    x2 = x.detach().clone().requires_grad_(True)
    y0, _, _ = ops.linear_multi(x2, [w.detach() for w in ws])
    (y0 * gs[0]).sum().backward()
    assert _rel(x2.grad, (gs[0].float() @ wrs[0].detach())) < 1e-2


def test_mod_predictor_bce():
    """Fused selection-predictor loss against zeros + scatter_ + binary_cross_entropy_with_logits in fp32."""
    ops, c, eager = _mods()
    torch.manual_seed(17)
    B, S, k = 3, 333, 250
    logits = (torch.randn(B, S, device="cuda") * 3).to(torch.bfloat16).requires_grad_(True)
    idx = torch.stack([torch.randperm(S, device="cuda")[:k].sort().values for _ in range(B)])
    loss = ops.mod_bce(logits, idx)
    (loss * 2.5).backward()
    lr = logits.detach().float().requires_grad_(True)
    tgt = torch.zeros(B, S, device="cuda").scatter_(1, idx, 1.0)
    ref = F.binary_cross_entropy_with_logits(lr, tgt, reduction="mean")
    (ref * 2.5).backward()
    assert abs(loss.item() - ref.item()) < 1e-4 * max(1.0, abs(ref.item()))
    assert _rel(logits.grad, lr.grad) < 1e-2
