"""Properties of the routing definitions in ``ops/eager.py`` and of the MXFP8 rounding emulation - the oracles the kernels are compared
against - checked on generated shapes and values."""
import math

import pytest
import torch
from hypothesis import given, settings, strategies as st

from kolmogorov_moe_architecture_b200.ops import eager

SET = settings(max_examples=40, deadline=None)


@SET
@given(T=st.integers(1, 60), E=st.integers(2, 9), k=st.integers(1, 3), seed=st.integers(0, 10_000))
def test_token_choice_weights_sum_to_one_and_pick_distinct_largest(T, E, k, seed):
    k = min(k, E)
    logits = torch.randn(T, E, generator=torch.Generator().manual_seed(seed))
    w, idx = eager.topk_softmax_route(logits, k)
    assert w.shape == idx.shape == (T, k)
    assert torch.allclose(w.sum(-1), torch.ones(T), atol=1e-5) and (w > 0).all()
    assert all(len(set(r)) == k for r in idx.tolist())                      # distinct experts per token
    kth = logits.gather(1, idx).min(-1).values
    not_picked = torch.ones(T, E, dtype=torch.bool).scatter_(1, idx, False)
    assert (logits.masked_fill(~not_picked, -math.inf).max(-1).values <= kth + 1e-6).all()
    _, _, aux, counts = eager.route_topk(logits, k, 1.0, 0.0)
    assert int(counts.sum()) == T * k and float(aux) >= 0.0


@SET
@given(T=st.integers(1, 80), E=st.integers(1, 8), k=st.integers(1, 3), cap=st.integers(0, 30), seed=st.integers(0, 10_000))
def test_capacity_mask_keeps_the_first_assignments_of_each_expert(T, E, k, cap, seed):
    idx = torch.randint(0, E, (T, k), generator=torch.Generator().manual_seed(seed))
    keep = eager.capacity_keep_mask(idx, E, cap)
    flat, kf = idx.reshape(-1), keep.reshape(-1)
    for e in range(E):
        pos = (flat == e).nonzero().flatten()
        assert int(kf[pos].sum()) == min(cap, pos.numel())
        assert kf[pos[:cap]].all() and not kf[pos[cap:]].any()             # lowest (token, slot) order first


@SET
@given(B=st.integers(1, 4), S=st.integers(2, 40), frac=st.floats(0.1, 1.0), seed=st.integers(0, 10_000))
def test_mod_router_keeps_k_tokens_in_order_with_softmax_weights(B, S, frac, seed):
    k = max(1, min(S, int(S * frac)))
    logits = torch.randn(B, S, generator=torch.Generator().manual_seed(seed))
    sidx, w, topi = eager.mod_route(logits, k)
    assert sidx.shape == w.shape == (B, k)
    assert (sidx[:, 1:] > sidx[:, :-1]).all()                              # ascending, distinct positions
    assert torch.equal(sidx.sort(-1).values, topi.sort(-1).values)
    assert torch.allclose(w, torch.softmax(logits.gather(1, sidx), -1), atol=1e-6)
    dropped = torch.ones(B, S, dtype=torch.bool).scatter_(1, sidx, False)
    if k < S:
        assert (logits.masked_fill(~dropped, -math.inf).max(-1).values <= logits.gather(1, sidx).min(-1).values).all()
    # combine: positions that were not kept pass the residual through unchanged
    d = 3
    res = torch.randn(B, S, d)
    proc = torch.randn(B, k, d)
    out = eager.mod_combine(res, proc, w, sidx)
    assert torch.equal(out[dropped], res[dropped])
    assert torch.allclose(eager.mod_gather(out - res, sidx), proc * w.unsqueeze(-1), atol=1e-6)


@SET
@given(B=st.integers(1, 3), S=st.integers(2, 30), E=st.integers(1, 5), cf=st.floats(0.5, 2.0), seed=st.integers(0, 10_000))
def test_expert_choice_each_expert_takes_its_capacity(B, S, E, cf, seed):
    cap = min(S, int(math.ceil(S * cf / E)))
    logits = torch.randn(B, S, E, generator=torch.Generator().manual_seed(seed))
    w, tok = eager.expert_choice_route(logits, cap)
    assert w.shape == tok.shape == (B, E, cap)
    assert torch.allclose(w.sum(-1), torch.ones(B, E), atol=1e-4)
    assert all(len(set(r)) == cap for b in tok.tolist() for r in b)        # an expert takes a token once
    probs = torch.softmax(logits.transpose(1, 2), -1)
    kth = probs.gather(2, tok).min(-1).values
    rest = probs.scatter(2, tok, -1.0).max(-1).values
    assert (rest <= kth + 1e-7).all()


@SET
@given(T=st.integers(1, 40), E=st.integers(2, 6), seed=st.integers(0, 10_000))
def test_dropped_assignments_contribute_nothing(T, E, seed):
    g = torch.Generator().manual_seed(seed)
    d, f, k = 8, 12, 2
    x = torch.randn(T, d, generator=g)
    w1, w2, w3 = torch.randn(E, d, f, generator=g), torch.randn(E, d, f, generator=g), torch.randn(E, f, d, generator=g)
    wts, idx = eager.topk_softmax_route(torch.randn(T, E, generator=g), k)
    keep = eager.capacity_keep_mask(idx, E, max(1, T * k // (2 * E)))
    out = eager.grouped_swiglu(x, w1, w2, w3, idx, wts, keep)
    ref = eager.grouped_swiglu(x, w1, w2, w3, idx, wts * keep, None)       # zero weight == dropped, no renormalising
    assert torch.allclose(out, ref, atol=1e-5)
    all_dropped = ~keep.any(-1)
    assert torch.equal(out[all_dropped], torch.zeros_like(out[all_dropped]))


@SET
@given(R=st.integers(1, 6), K=st.integers(1, 100), scale=st.floats(1e-6, 1e4), dim=st.sampled_from([-1, 0]),
       seed=st.integers(0, 10_000))
def test_mx_rounding_is_a_projection_with_bounded_error(R, K, scale, dim, seed):
    """Block-scaled e4m3 (one power-of-two scale per 32 elements): quantising twice changes nothing more,
    the scale exponent follows the block maximum, the element error is within half an e4m3 step (values
    above 448 scales saturate), zero blocks stay zero, and the gradient passes straight through."""
    from kolmogorov_moe_architecture_b200.ops.mxfp8 import dequantize_mx, fake_quant_mx, quantize_mx
    x = torch.randn(R, K, generator=torch.Generator().manual_seed(seed)) * scale
    x[0, : min(K, 32)] = 0.0 if dim == -1 else x[0, : min(K, 32)]
    once = fake_quant_mx(x, dim)
    assert torch.equal(fake_quant_mx(once, dim), once)
    q, e = quantize_mx(x, dim)
    assert q.dtype == torch.float8_e4m3fn and q.shape == x.shape and e.dtype == torch.int8
    xm = x.movedim(dim, -1)
    nb = (xm.shape[-1] + 31) // 32
    assert e.shape[-1] == nb
    for b in range(nb):
        blk = xm[..., 32 * b: 32 * b + 32]
        amax = blk.abs().amax(-1)
        live = amax > 2.0 ** -100
        want = torch.floor(torch.log2(amax.clamp(min=2.0 ** -127))) - 8
        assert torch.equal(e[..., b].float()[live], want.clamp(-127, 127)[live])
        sc = torch.exp2(e[..., b].float()).unsqueeze(-1)
        got = once.movedim(dim, -1)[..., 32 * b: 32 * b + 32]
        err = (got - blk).abs()
        inside = blk.abs() <= 448.0 * sc                 # 3 mantissa bits; below 2^-6 of the scale a fixed step
        assert (err[inside] <= torch.maximum(2.0 ** -4 * blk.abs(), 2.0 ** -10 * sc.expand_as(blk))[inside]).all()
        assert torch.equal(got[~inside].abs(), (448.0 * sc.expand_as(blk))[~inside])     # saturates, never overflows
    assert torch.equal(dequantize_mx(q, e, dim, torch.float32), once)
    if dim == -1:
        assert torch.equal(once[0, : min(K, 32)], torch.zeros(min(K, 32)))
    xg = x.clone().requires_grad_(True)
    fake_quant_mx(xg, dim).sum().backward()
    assert torch.equal(xg.grad, torch.ones_like(x))


@SET
@given(m=st.integers(2, 24), n=st.integers(2, 24), b=st.integers(1, 3), seed=st.integers(0, 10_000))
def test_newton_schulz_moves_singular_values_towards_one(m, n, b, seed):
    """Wide, tall and batched inputs: the iteration keeps the singular vectors and pushes every singular
    value of the normalised matrix up towards 1 without overshooting, so the result is closer to an
    orthogonal factor after every additional step."""
    x = torch.randn(b, m, n, generator=torch.Generator().manual_seed(seed), dtype=torch.float64)
    y0 = x / x.reshape(b, -1).norm(dim=1).view(b, 1, 1)
    prev = torch.linalg.svdvals(y0)
    for iters in (1, 3, 6):
        y = eager.newton_schulz(x, iters)
        assert y.shape == x.shape
        sv = torch.linalg.svdvals(y)
        assert (sv <= 1.0 + 1e-9).all() and (sv >= prev - 1e-9).all()
        prev = sv
    one = eager.newton_schulz(x[0], 6)
    assert torch.allclose(one, y[0], atol=1e-12)                       # 2-D input = batch of one
    u, s, vh = torch.linalg.svd(y0[0], full_matrices=False)
    recon = u @ torch.diag(torch.linalg.svdvals(one)) @ vh
    assert torch.allclose(recon, one, atol=1e-8)                       # same singular vectors


@SET
@given(n=st.integers(1, 5000), scale=st.floats(1e-4, 1e3), seed=st.integers(0, 10_000))
def test_int8_block_quantisation_error_is_half_a_step_of_the_block_maximum(n, scale, seed):
    from kolmogorov_moe_architecture_b200.training.muon_optimizer import Muon8bit
    t = torch.randn(n, generator=torch.Generator().manual_seed(seed)) * scale
    q, scales, shape, numel = Muon8bit._quantize_to_8bit(t, block_size=256)
    back = Muon8bit._dequantize_from_8bit(q, scales, shape, numel)
    assert q.dtype == torch.int8 and back.shape == t.shape and scales.shape[0] == (n + 255) // 256
    bound = (scales / 127 * 0.5 * (1 + 1e-5)).expand(-1, 256).flatten()[:n]
    assert ((back - t).abs() <= bound).all()
    assert int(q.abs().max()) <= 127


@SET
@given(B=st.integers(1, 3), S=st.integers(1, 24), ndocs=st.integers(1, 5), seed=st.integers(0, 10_000))
def test_document_boundaries_and_mask_agree(B, S, ndocs, seed):
    """``doc_start`` is the first position of each token's document; the additive mask built from it hides
    exactly the keys of earlier documents (causality itself is the attention's job)."""
    g = torch.Generator().manual_seed(seed)
    cuts = torch.sort(torch.randint(0, S, (B, ndocs - 1), generator=g), dim=1).values if ndocs > 1 else torch.zeros(B, 0, dtype=torch.long)
    doc_ids = torch.zeros(B, S, dtype=torch.long)
    for b in range(B):
        for c in cuts[b].tolist():
            doc_ids[b, c:] += 1
    ds = eager.doc_start_from_ids(doc_ids)
    assert ds.dtype == torch.int32 and (ds <= torch.arange(S)).all()
    for b in range(B):
        for t in range(S):
            s0 = int(ds[b, t])
            assert (doc_ids[b, s0: t + 1] == doc_ids[b, t]).all() and (s0 == 0 or doc_ids[b, s0 - 1] != doc_ids[b, t])
    mask = eager.doc_start_to_mask(ds)
    same_or_later_doc = doc_ids.unsqueeze(2) <= doc_ids.unsqueeze(1)          # key's document is not an earlier one
    assert torch.equal(mask[:, 0] == 0, same_or_later_doc)


@SET
@given(B=st.integers(1, 3), S=st.integers(1, 12), n_heads=st.integers(1, 4), V=st.integers(2, 9), seed=st.integers(0, 10_000))
def test_multi_token_loss_scores_head_i_against_the_token_i_plus_one_ahead(B, S, n_heads, V, seed):
    """Head i (0-based) at position t is scored against labels[t + i + 1]; ignored targets do not count; heads
    that have no target inside the sequence contribute zero; a head whose logits put all mass on its targets
    has zero loss."""
    g = torch.Generator().manual_seed(seed)
    d = V                                                      # hidden = one-hot of a token: logits are readable
    labels = torch.randint(0, V, (B, S), generator=g)
    heads = [torch.eye(V) * 50.0 for _ in range(n_heads)]
    w = [1.0 / n_heads] * n_heads
    for i in range(n_heads):                                   # hidden state that is exactly right for head i
        hidden = torch.zeros(B, S, d)
        if i + 1 < S:
            hidden[:, : S - i - 1] = torch.nn.functional.one_hot(labels[:, i + 1:], V).float()
        total, per = eager.mtp_cross_entropy(hidden, heads, labels, w)
        assert per.shape == (n_heads,) and float(per[i]) < 1e-6
        assert abs(float(total) - float((per * torch.tensor(w)).sum())) < 1e-6
        for j in range(n_heads):
            if j + 1 >= S:
                assert float(per[j]) == 0.0
    hidden = torch.randn(B, S, d, generator=g)
    _, per = eager.mtp_cross_entropy(hidden, heads, labels, w)
    masked = labels.clone()
    masked[:, ::2] = -100
    _, per_m = eager.mtp_cross_entropy(hidden, heads, masked, w)
    i = 0
    if S > 1:
        keep = masked[:, 1:] != -100
        if keep.any():
            logits = hidden[:, : S - 1] @ heads[0].t()
            want = torch.nn.functional.cross_entropy(logits[keep], labels[:, 1:][keep])
            assert abs(float(per_m[i]) - float(want)) < 1e-4


def _get_tile(idx, num_m, num_n, groups, batched, sym_upper, BM=128, BN=256):
    """The work-index -> tile mapping of the persistent GEMM (``get_tile`` in csrc/gemm_umma.cu), restated."""
    per_group = num_m * num_n
    if sym_upper:
        first = [min(num_n, (m * BM) // BN) for m in range(num_m)]
        kept = sum(num_n - f for f in first)
        g, local = divmod(idx, kept)
        if g >= (groups if batched else 1):
            return None
        m = 0
        while local >= num_n - first[m]:
            local -= num_n - first[m]
            m += 1
        return g, m, first[m] + local
    g, local = 0, idx
    if batched:
        g, local = divmod(idx, per_group)
        if g >= groups:
            return None
    elif idx >= per_group:
        return None
    GM = 8
    band = local // (GM * num_n)
    first_m = band * GM
    gsz = min(num_m - first_m, GM)
    r = local - band * GM * num_n
    return g, first_m + r % gsz, r // gsz


@SET
@given(num_m=st.integers(1, 40), num_n=st.integers(1, 12), groups=st.integers(1, 4), batched=st.booleans(),
       grid=st.integers(1, 148))
def test_gemm_tile_scheduler_visits_every_tile_exactly_once(num_m, num_n, groups, batched, grid):
    """Persistent CTAs stride the work index by the grid size: together they cover every (group, m, n) tile
    once, in bands of eight m-tiles; the symmetric variant covers exactly the tiles that touch the upper
    triangle (the rest is mirrored afterwards)."""
    G = groups if batched else 1
    seen = []
    for cta in range(grid):
        idx = cta
        while (t := _get_tile(idx, num_m, num_n, groups, batched, False)) is not None:
            seen.append(t)
            idx += grid
    assert len(seen) == len(set(seen)) == G * num_m * num_n
    assert set(seen) == {(g, m, n) for g in range(G) for m in range(num_m) for n in range(num_n)}
    # symmetric product: BM = 128 rows against BN = 256 columns
    seen = []
    idx = 0
    while (t := _get_tile(idx, num_m, num_n, groups, batched, True)) is not None:
        seen.append(t)
        idx += 1
    want = {(g, m, n) for g in range(G) for m in range(num_m) for n in range(num_n) if (n + 1) * 256 > m * 128}
    assert len(seen) == len(set(seen)) and set(seen) == want


@SET
@given(rows=st.integers(1, 300), kchunks=st.integers(1, 4), seed=st.integers(0, 10_000))
def test_mx_scale_chunk_layout_round_trip(rows, kchunks, seed):
    """Scale bytes are stored in 512-byte chunks per 128 rows x 128 reduction elements, byte
    (row % 32) * 16 + (row % 128) / 32 * 4 + (k / 32) % 4 inside the chunk (the arrangement the tensor core
    reads from tensor memory); ``decode_scale_chunks`` undoes exactly that placement."""
    from kolmogorov_moe_architecture_b200.ops.mxfp8 import decode_scale_chunks
    K = 128 * kchunks
    exps = torch.randint(-20, 20, (rows, K // 32), generator=torch.Generator().manual_seed(seed))
    rb = (rows + 127) // 128
    sf = torch.zeros(rb * kchunks * 512, dtype=torch.uint8)
    for r in range(rows):
        for kg in range(K // 32):
            chunk = (r // 128) * kchunks + kg // 4
            sf[chunk * 512 + (r % 32) * 16 + ((r % 128) // 32) * 4 + kg % 4] = int(exps[r, kg]) + 127
    assert torch.equal(decode_scale_chunks(sf, rows, K), exps.to(torch.int32))


def test_extension_errors_raise_instead_of_crashing():
    """A failed entry point of the compiled library surfaces as a Python exception with its formatted message.
    (A library linked against a private copy of the C++ runtime crashes while formatting the number.)"""
    import pytest
    from kolmogorov_moe_architecture_b200.ops import loader
    if not loader.ext_available():
        pytest.skip("extension not built")
    with pytest.raises(RuntimeError, match="kmoe::self_test failed with code -7"):
        torch.ops.kmoe.raise_check(-7)
    torch.ops.kmoe.raise_check(0)


@settings(max_examples=60, deadline=None)
@given(out_f=st.sampled_from([8, 16, 40, 64, 128, 160, 512, 2048, 4096]),
       in_f=st.sampled_from([64, 128, 512, 2048, 4096]),
       T=st.integers(min_value=1, max_value=40000).map(lambda v: v * 8))
def test_weight_gradient_token_slices_cover_every_token_once(out_f, in_f, T):
    """The slices of a sliced weight gradient start on whole 64-row reduction blocks, do not overlap, and
    together cover exactly the T tokens; large results and short sequences are not sliced."""
    from kolmogorov_moe_architecture_b200.ops import cuda_ops as c
    parts = c.split_k_parts(out_f, in_f, T)
    assert 1 <= parts <= 32
    tiles = -(-out_f // 256) * -(-in_f // 256)
    if tiles >= 48 or T < 2048:
        assert parts == 1
        return
    begin, length = (t.tolist() for t in c._split_k_ranges(T, parts, torch.device("cpu")))
    assert 1 <= len(begin) <= parts and begin[0] == 0 and sum(length) == T
    for i in range(len(begin)):
        assert begin[i] % 64 == 0 and length[i] > 0
        if i + 1 < len(begin):
            assert begin[i] + length[i] == begin[i + 1]


def _score_key(v: float) -> int:
    """Order-preserving 32-bit image of an fp32 score, as in the selection kernel."""
    import struct
    u = struct.unpack("<I", struct.pack("<f", v))[0]
    return (~u & 0xFFFFFFFF) if (u & 0x80000000) else (u | 0x80000000)


def _radix_select_keep(scores, k):
    """Host restatement of the mixture-of-depths selection kernel: 4-pass radix selection of the k-th best key,
    then keep everything above it and the lowest-indexed ``need`` of the ties."""
    keys = [_score_key(float(v)) for v in scores]
    prefix, need = 0, k
    for p in range(4):
        shift = 24 - 8 * p
        mask = 0 if p == 0 else (0xFFFFFFFF << (shift + 8)) & 0xFFFFFFFF
        hist = [0] * 256
        for u in keys:
            if (u & mask) == prefix:
                hist[(u >> shift) & 255] += 1
        above = 0
        for b in range(255, -1, -1):
            if above + hist[b] >= need:
                prefix |= b << shift
                need -= above
                break
            above += hist[b]
    kept, ties = [], 0
    for i, u in enumerate(keys):
        if u > prefix or (u == prefix and ties < need):
            kept.append(i)
        if u == prefix:
            ties += 1
    return kept


@settings(max_examples=60, deadline=None)
@given(S=st.integers(min_value=2, max_value=300), frac=st.floats(min_value=0.05, max_value=1.0),
       levels=st.integers(min_value=2, max_value=50), seed=st.integers(min_value=0, max_value=10**6))
def test_radix_selection_equals_sorting_with_ties_to_the_lower_index(S, frac, levels, seed):
    """The selection used on the GPU (no sort) keeps exactly the positions a stable descending sort keeps, also
    when many scores are equal (few distinct levels) and for negative values."""
    g = torch.Generator().manual_seed(seed)
    scores = (torch.randint(0, levels, (S,), generator=g).float() - levels / 2) * 0.37
    k = max(1, min(S, int(S * frac)))
    kept = _radix_select_keep(scores.tolist(), k)
    order = sorted(range(S), key=lambda i: (-float(scores[i]), i))[:k]
    assert kept == sorted(order)
    # (torch.topk, which the eager definition uses, leaves the order among equal scores unspecified; without ties
    # the two agree)
    distinct = torch.randperm(S, generator=g).float() * 0.01 - 1.0
    idx, _, _ = eager.mod_route(distinct.unsqueeze(0), k)
    assert idx[0].tolist() == _radix_select_keep(distinct.tolist(), k)


@settings(max_examples=25, deadline=None)
@given(m=st.sampled_from([8, 16, 24]), ratio=st.sampled_from([1.25, 2.0, 3.5]), tall=st.booleans(),
       seed=st.integers(min_value=0, max_value=10**6))
def test_newton_schulz_on_the_short_side_is_the_same_iteration(m, ratio, tall, seed):
    """The identity behind the short-side form: with W = P - 1.5 I and V = Q - c I (c = 1.5^k),
    W' = W (W (W + 3 I) + 2.25 I), V' = W' V + 1.5 V + c W' and Y_5 = V Y + c Y reproduce five steps of
    Y <- 1.5 Y - 0.5 Y Y^T Y exactly (fp64 here)."""
    torch.manual_seed(seed)
    n = int(m * ratio)
    Y0 = torch.randn(m, n, dtype=torch.float64)
    if tall:
        Y0 = Y0.t().contiguous()
    ref = eager.newton_schulz(Y0, 5)
    Y = Y0 / (Y0.norm() + 1e-7)
    A = Y if not tall else Y.t()                     # iterate on the short side: A is (short, long)
    I = torch.eye(A.shape[0], dtype=torch.float64)
    W = -0.5 * (A @ A.t())
    V, c = W.clone(), 1.5
    for _ in range(4):
        W = W @ (W @ (W + 3.0 * I) + 2.25 * I)
        V = W @ V + 1.5 * V + c * W
        c *= 1.5
    out = V @ A + c * A
    out = out if not tall else out.t()
    assert torch.allclose(out, ref, rtol=1e-9, atol=1e-11)


# ---------------------------------------------------------------- opt-in validation of data-dependent inputs
def test_input_checks_name_the_first_offending_element(monkeypatch):
    from kolmogorov_moe_architecture_b200 import ops
    from kolmogorov_moe_architecture_b200.ops import checks
    monkeypatch.setenv("KMOE_CHECK_INPUTS", "1")
    assert checks.enabled()
    g = torch.Generator().manual_seed(0)
    T, d, f, E, k = 12, 16, 24, 4, 2
    x = torch.randn(T, d, generator=g)
    w1, w2, w3 = torch.randn(E, d, f, generator=g), torch.randn(E, d, f, generator=g), torch.randn(E, f, d, generator=g)
    idx = torch.stack([torch.randperm(E, generator=g)[:k] for _ in range(T)])
    wts = torch.softmax(torch.randn(T, k, generator=g), -1)
    ops.grouped_swiglu(x, w1, w2, w3, idx, wts)                       # valid input passes
    bad = idx.clone()
    bad[5, 1] = E
    with pytest.raises(IndexError, match=r"value 4 at position \(5, 1\) is outside \[0, 4\)"):
        ops.grouped_swiglu(x, w1, w2, w3, bad, wts)
    nanw = wts.clone()
    nanw[3, 0] = float("nan")
    with pytest.raises(ValueError, match=r"non-finite value at position \(3, 0\)"):
        ops.grouped_swiglu(x, w1, w2, w3, idx, nanw)
    with pytest.raises(ValueError, match="keep mask has 5 elements for 24 assignments"):
        ops.grouped_swiglu(x, w1, w2, w3, idx, wts, keep=torch.ones(5, dtype=torch.bool))
    dup = idx.clone()
    dup[7] = 2
    with pytest.raises(ValueError, match="token 7 is assigned to expert 2 twice"):
        checks.expert_indices(dup, E)
    checks.expert_indices(dup, E, top_k_distinct=False)

    # labels of the loss head
    V, B, S = 32, 2, 9
    hidden = torch.randn(B, S, d, generator=g)
    heads = [torch.randn(V, d, generator=g) for _ in range(2)]
    lab = torch.randint(0, V, (B, S), generator=g)
    lab[0, 2] = -100
    ops.mtp_cross_entropy(hidden, heads, lab, [0.7, 0.3])
    lab[1, 4] = V + 3
    with pytest.raises(IndexError, match=r"labels: value 35 at position \(1, 4\) is neither -100 nor in \[0, 32\)"):
        ops.mtp_cross_entropy(hidden, heads, lab, [0.7, 0.3])

    # mixture-of-depths positions: in range and strictly ascending
    h = torch.randn(B, S, d, generator=g)
    kept = torch.tensor([[0, 3, 4, 8], [1, 2, 5, 6]])
    ops.mod_gather(h, kept)
    with pytest.raises(IndexError, match=r"value 9 at position \(0, 3\) is outside \[0, 9\)"):
        ops.mod_gather(h, torch.tensor([[0, 3, 4, 9], [1, 2, 5, 6]]))
    with pytest.raises(ValueError, match=r"not strictly ascending at position \(1, 1\) \(5 is followed by 5\)"):
        ops.mod_gather(h, torch.tensor([[0, 3, 4, 8], [1, 5, 5, 6]]))
    with pytest.raises(ValueError, match="expected an integer tensor"):
        checks.kept_rows(kept.float(), S)

    # expert-choice: an expert takes a token at most once
    tok = torch.tensor([[[0, 1, 2], [3, 4, 5]], [[6, 7, 8], [1, 1, 0]]])
    with pytest.raises(ValueError, match=r"row 1 is selected twice in group \(1, 1\)"):
        checks.distinct_rows(tok, S, "expert-choice token index")

    # packed documents
    ds = torch.tensor([[0, 0, 0, 3, 3, 5], [0, 1, 1, 1, 4, 4]])
    checks.doc_start(ds)
    with pytest.raises(IndexError, match=r"value 4 at position \(0, 3\) is outside \[0, 3\]"):
        checks.doc_start(torch.tensor([[0, 0, 0, 4, 4, 5]]))
    with pytest.raises(ValueError, match=r"decreases after position \(0, 3\) \(3 -> 2\)"):
        checks.doc_start(torch.tensor([[0, 0, 0, 3, 2, 5]]))
    q = torch.randn(1, 6, 2, 8, generator=g)
    with pytest.raises(ValueError, match="decreases"):
        ops.attention(q, q, q, doc_start=torch.tensor([[0, 0, 0, 3, 2, 5]]))


def test_input_checks_are_off_by_default(monkeypatch):
    from kolmogorov_moe_architecture_b200 import ops
    from kolmogorov_moe_architecture_b200.ops import checks
    monkeypatch.delenv("KMOE_CHECK_INPUTS", raising=False)
    assert not checks.enabled()
    # no validation pass runs: a float index tensor, which the checks reject, reaches the op itself
    h = torch.randn(1, 4, 8)
    with pytest.raises(Exception) as e:
        ops.mod_gather(h, torch.tensor([[0.0, 1.0]]))
    assert "expected an integer tensor" not in str(e.value)
