"""CPU tests of the model, losses, routing rules, generation and gradient flow."""
import math

import pytest
import torch

import kolmogorov_moe_architecture_b200 as kmoe
from kolmogorov_moe_architecture_b200 import ops
from kolmogorov_moe_architecture_b200.ops import eager


def _tiny(**kw):
    base = dict(vocab_size=200, d_model=64, n_layers=4, n_heads=4, n_kv_heads=2, head_dim=16, d_ff=128,
                d_ff_expert=64, n_experts=4, moe_layers=(1, 2), mamba_layers=(1,), max_seq_len=32, n_pred_tokens=2,
                aux_loss_weights=(1.0, 0.5), dropout=0.0, attention_dropout=0.0, residual_dropout=0.0,
                device="cpu", dtype="float32")
    base.update(kw)
    return kmoe.AdvancedMoEConfig(**base)


@pytest.mark.parametrize("mode", ["routing_mamba", "moe_ffn"])
def test_forward_shapes_loss_composition_and_eval_aux(mode):
    cfg = _tiny(mamba_moe_mode=mode)
    m = kmoe.MoETransformer(cfg, verbose=False)
    ids = torch.randint(0, 200, (2, 32))
    m.train()
    out = m(ids, labels=ids)
    assert out["logits"].shape == (2, 32, 200) and len(out["logits_list"]) == 2
    assert torch.allclose(out["loss"], out["lm_loss"] + out["aux_loss"])
    out2 = m(ids, labels=ids, return_logits=False)
    assert torch.allclose(out2["lm_loss"], out["lm_loss"], atol=1e-5)
    m.eval()
    ev = m(ids, labels=ids)
    assert ev["aux_loss"] == 0.0 and torch.allclose(ev["loss"], ev["lm_loss"])
    kinds = [(l.mixer_kind, l.ffn_kind) for l in m.layers]
    assert kinds[1] == (("routing_mamba", "dense") if mode == "routing_mamba" else ("mamba", "moe"))


@pytest.mark.parametrize("mod", [True, False])
def test_every_parameter_gets_a_gradient(mod):
    m = kmoe.MoETransformer(_tiny(mod_enabled=mod, mamba_moe_mode="moe_ffn"), verbose=False)
    m.train()
    ids = torch.randint(0, 200, (2, 32))
    m(ids, labels=ids, return_logits=False)["loss"].backward()
    missing = [n for n, p in m.named_parameters() if p.grad is None or not torch.isfinite(p.grad).all()]
    assert not missing, missing
    zero = [n for n, p in m.named_parameters() if p.grad.abs().sum() == 0]
    assert not zero, zero


def test_state_dict_schema():
    m = kmoe.MoETransformer(_tiny(), verbose=False)
    keys = set(m.state_dict())
    for k in ["token_embedding.embedding.weight", "layers.0.seq_layer.q_proj.weight", "layers.0.ffn.w1.weight",
              "layers.0.ffn_mod_router.router.weight", "layers.0.ffn_mod_router.aux_router.2.weight",
              "layers.1.seq_layer.experts.0.mamba.mamba.in_proj.weight", "layers.1.seq_layer.router.0.weight",
              "layers.2.ffn.router.router.0.weight", "layers.2.ffn.grouped_experts.w3", "final_norm.weight",
              "lm_heads.0.weight", "lm_heads.1.weight"]:
        assert k in keys, k
    assert m.lm_heads[0].weight is m.token_embedding.embedding.weight
    assert m.state_dict()["layers.2.ffn.grouped_experts.w1"].shape == (4, 64, 64)
    assert not any("cos_cached" in k or "inv_freq" in k for k in keys)


def test_generate_length_and_sampling_filters():
    m = kmoe.MoETransformer(_tiny(), verbose=False).eval()
    ids = torch.randint(0, 200, (2, 5))
    out = m.generate(ids, max_new_tokens=4, temperature=0.8, top_k=10, top_p=0.9)
    assert out.shape == (2, 9) and torch.equal(out[:, :5], ids)


def test_mod_router_rule():
    from kolmogorov_moe_architecture_b200.models.mod import MoDRouter
    r = MoDRouter(_tiny(mod_capacity_factor=0.75)).train()
    x = torch.randn(3, 16, 64)
    idx, w, logits, topk = r(x)
    assert idx.shape == (3, 12) and torch.all(idx[:, 1:] > idx[:, :-1])
    assert torch.allclose(w.sum(-1), torch.ones(3), atol=1e-5)
    assert torch.allclose(w, torch.softmax(torch.gather(logits, 1, idx), -1), atol=1e-6)
    assert r.aux_loss > 0
    assert r.num_selected(1) == 1


def test_router_weights_and_balanced_capacity():
    from kolmogorov_moe_architecture_b200.models.moe import Router
    r = Router(_tiny())
    w, idx, logits = r(torch.randn(2, 16, 64))
    assert torch.allclose(w.sum(-1), torch.ones(2, 16), atol=1e-5) and idx.shape == (2, 16, 2)
    rb = Router(_tiny(moe_balanced_routing=True))
    wb, ib, _ = rb(torch.randn(4, 32, 64))
    assert torch.all(ib[..., 0] != ib[..., 1])
    counts = torch.bincount(ib.reshape(-1), minlength=4)
    assert counts.max() <= 2 * (4 * 32 * 2 // 4)


def test_capacity_drop_policy():
    idx = torch.tensor([[0, 1], [0, 1], [0, 2], [0, 1]])
    keep = eager.capacity_keep_mask(idx, 4, 2)
    assert keep.tolist() == [[True, True], [True, True], [False, True], [False, False]]
    x, w = torch.randn(4, 8), torch.full((4, 2), 0.5)
    w1, w2, w3 = torch.randn(4, 8, 6), torch.randn(4, 8, 6), torch.randn(4, 6, 8)
    out = eager.grouped_swiglu(x, w1, w2, w3, idx, w, keep)
    assert out[3].abs().sum() == 0


def test_expert_choice_capacity():
    from kolmogorov_moe_architecture_b200.models.moe import ExpertChoiceRouter
    r = ExpertChoiceRouter(_tiny(moe_capacity_factor=1.25))
    w, tok, _, cap = r(torch.randn(2, 16, 64))
    assert cap == math.ceil(16 * 1.25 / 4) and tok.shape == (2, 4, cap)
    assert torch.allclose(w.sum(-1), torch.ones(2, 4), atol=1e-4)


def test_selective_scan_matches_closed_form_for_constant_inputs():
    B, S, C, N = 1, 6, 2, 16
    u, dt = torch.ones(B, S, C), torch.full((B, S, C), 0.5)
    A = -torch.ones(C, N)
    Bm, Cm = torch.ones(B, S, N), torch.ones(B, S, N)
    y = eager.selective_scan(u, dt, A, Bm, Cm, None, None, None, delta_softplus=False)
    a, h, ref = math.exp(-0.5), 0.0, []
    for _ in range(S):
        h = a * h + 0.5
        ref.append(N * h)
    assert torch.allclose(y[0, :, 0], torch.tensor(ref), atol=1e-5)


def test_causal_conv_is_causal():
    x = torch.randn(1, 10, 4)
    w, b = torch.randn(4, 4), torch.randn(4)
    y1 = eager.causal_conv1d(x, w, b, True)
    x2 = x.clone(); x2[:, 7:] += 1.0
    y2 = eager.causal_conv1d(x2, w, b, True)
    assert torch.allclose(y1[:, :7], y2[:, :7])


def test_attention_gqa_equals_expanded_heads():
    q, k, v = torch.randn(2, 9, 4, 8), torch.randn(2, 9, 2, 8), torch.randn(2, 9, 2, 8)
    a = eager.attention(q, k, v)
    b = eager.attention(q, k.repeat_interleave(2, 2), v.repeat_interleave(2, 2))
    assert torch.allclose(a, b, atol=1e-6)


def test_count_parameters_and_presets():
    m = kmoe.MoETransformer(_tiny(mamba_moe_mode="moe_ffn"), verbose=False)
    c = m.count_parameters()
    assert c["total"] == sum(p.numel() for p in m.parameters()) and 0 < c["active"] < c["total"]
    assert kmoe.get_3b_config().n_experts == 64 and kmoe.get_test_config().n_layers == 4
    b = kmoe.get_bench_5b_config()
    assert len(b.moe_layers) == 16 and len(b.mamba_layers) == 8 and b.vocab_size == 50304
    d = b.to_dict(); d2 = kmoe.AdvancedMoEConfig.from_dict(d)
    assert d2.moe_layers == b.moe_layers
    with pytest.raises(TypeError):
        kmoe.AdvancedMoEConfig.from_dict({"not_a_field": 1})


def test_packed_docs_equals_dense_document_mask():
    """Document boundaries passed as ``PackedDocs`` give the same model output as the dense block-diagonal mask."""
    import kolmogorov_moe_architecture_b200 as kmoe
    from kolmogorov_moe_architecture_b200.data import PackedDocs, document_attention_mask
    cfg = kmoe.get_tiny_debug_config(vocab_size=128, d_model=64, n_heads=2, n_kv_heads=1, head_dim=32, d_ff=128,
                                     d_ff_expert=64, max_seq_len=24, n_pred_tokens=2, aux_loss_weights=(1.0, 0.5))
    torch.manual_seed(0)
    m = kmoe.MoETransformer(cfg, verbose=False).eval()
    ids = torch.randint(0, 128, (2, 24))
    doc_ids = torch.tensor([[0] * 5 + [1] * 10 + [2] * 9, [3] * 24])
    pd = PackedDocs(doc_ids=doc_ids)
    assert pd.doc_start[0].tolist() == [0] * 5 + [5] * 10 + [15] * 9 and pd.doc_start[1].tolist() == [0] * 24
    with torch.no_grad():
        a = m(ids, attention_mask=pd)["logits"]
        b = m(ids, attention_mask=document_attention_mask(doc_ids))["logits"]
        c = m(ids)["logits"]
    assert torch.allclose(a, b, atol=1e-5)
    assert not torch.allclose(a[0], c[0], atol=1e-3) and torch.allclose(a[1], c[1], atol=1e-5)


def test_packed_docs_sanitises_start_positions_given_from_outside():
    from kolmogorov_moe_architecture_b200.data import PackedDocs
    ds = torch.tensor([[0, 0, 5, -3, 4, 9]])
    p = PackedDocs(doc_start=ds)
    assert p.doc_start.dtype == torch.int32 and p.doc_start.tolist() == [[0, 0, 2, 2, 4, 5]]
    from kolmogorov_moe_architecture_b200.ops import checks
    checks.doc_start(p.doc_start)                      # what the validation mode demands of document starts
    assert p.to("cpu").doc_start.tolist() == p.doc_start.tolist() and len(p.chunk(1)) == 1
    ids = torch.tensor([[7, 7, 8, 8, 8, 9]])
    assert PackedDocs(doc_ids=ids).doc_start.tolist() == [[0, 0, 2, 2, 2, 5]]


def test_routing_mamba_batched_pass_equals_one_pass_per_expert():
    """All selected Mamba experts in one stacked pass (grouped convolution / scan parameters, batched
    projections) against the loop over experts: outputs, input gradient and every parameter gradient."""
    from kolmogorov_moe_architecture_b200.models.mamba import RoutingMamba
    cfg = kmoe.get_tiny_debug_config(vocab_size=128, d_model=32, n_heads=2, n_kv_heads=1, head_dim=16, d_ff=64,
                                     d_ff_expert=32, max_seq_len=16, n_pred_tokens=1, aux_loss_weights=(1.0,))
    torch.manual_seed(0)
    m = RoutingMamba(cfg, 1).train()
    x = torch.randn(2, 16, 32, requires_grad=True)
    res = {}
    for flag in (False, True):
        m.batched = flag
        m.zero_grad()
        x.grad = None
        y = m(x)
        (y * torch.arange(32.0)).sum().backward()
        res[flag] = (y.detach().clone(), x.grad.clone(),
                     {n: p.grad.clone() for n, p in m.named_parameters() if p.grad is not None})
    a, b = res[False], res[True]
    assert torch.allclose(a[0], b[0], atol=1e-5) and torch.allclose(a[1], b[1], atol=1e-5)
    assert set(a[2]) == set(b[2]) and all(torch.allclose(a[2][n], b[2][n], atol=1e-5) for n in a[2])


def test_tied_parameters_are_found_for_the_gradient_landing():
    """The embedding is tied to the first output head by default; the data-parallel plan must know, because such a
    tensor gets gradient from two nodes of the graph and may not be marked ready by the first one."""
    from kolmogorov_moe_architecture_b200 import AdvancedMoEConfig, MoETransformer
    from kolmogorov_moe_architecture_b200.parallel.zero import shared_parameter_ids
    cfg = AdvancedMoEConfig(vocab_size=256, d_model=64, n_layers=2, n_heads=4, n_kv_heads=2, head_dim=16, d_ff=128,
                            d_ff_expert=64, n_experts=4, moe_layers=(1,), mamba_layers=(), max_seq_len=32,
                            n_pred_tokens=2, aux_loss_weights=(1.0, 0.5))
    model = MoETransformer(cfg, verbose=False)
    shared = shared_parameter_ids(model)
    names = [n for n, p in model.named_parameters() if id(p) in shared]
    assert names == ["token_embedding.embedding.weight"]
    assert model.lm_heads[0].weight is model.token_embedding.embedding.weight
    assert id(model.lm_heads[1].weight) not in shared


def test_tied_embedding_gets_no_direct_gradient_destination():
    """The gradient-landing set-up of the data-parallel plan (exercised here with a stand-in device type, no GPU
    involved) registers a direct destination for every tensor except the tied embedding / first head."""
    import types
    from kolmogorov_moe_architecture_b200 import AdvancedMoEConfig, MoETransformer
    from kolmogorov_moe_architecture_b200.ops import cuda_ops
    from kolmogorov_moe_architecture_b200.parallel.zero import ShardedDataParallel
    cfg = AdvancedMoEConfig(vocab_size=256, d_model=64, n_layers=2, n_heads=4, n_kv_heads=2, head_dim=16, d_ff=128,
                            d_ff_expert=64, n_experts=4, moe_layers=(1,), mamba_layers=(), max_seq_len=32,
                            n_pred_tokens=2, aux_loss_weights=(1.0, 0.5))
    model = MoETransformer(cfg, verbose=False)
    dp = ShardedDataParallel(model)
    saved = dict(cuda_ops._GRAD_SINKS)
    try:
        cuda_ops._GRAD_SINKS.clear()
        dp.device = types.SimpleNamespace(type="cuda")
        dp._setup_grad_landing()
        tied = model.token_embedding.embedding.weight
        assert dp._landing and tied.data_ptr() not in cuda_ops._GRAD_SINKS
        assert len(cuda_ops._GRAD_SINKS) == len(dp.named) - 1
        assert all(p.grad is None for _, p in dp.named)
    finally:
        cuda_ops._GRAD_SINKS.clear()
        cuda_ops._GRAD_SINKS.update(saved)


def test_fused_op_entry_points_have_the_same_meaning_on_the_host():
    """``ops.linear_multi``, ``ops.mod_score_gather`` and ``ops.mod_bce`` fall back to plain PyTorch here; the
    definitions they fall back to are the ones the GPU kernels are tested against."""
    import torch.nn.functional as F
    from kolmogorov_moe_architecture_b200 import ops
    from kolmogorov_moe_architecture_b200.ops import eager
    torch.manual_seed(0)
    x = torch.randn(2, 10, 16)
    ws = [torch.randn(n, 16) for n in (16, 8, 8)]
    for y, w in zip(ops.linear_multi(x, ws), ws):
        assert torch.allclose(y, F.linear(x, w))
    w = torch.randn(1, 16)
    picked, idx, wts, logits = ops.mod_score_gather(x, w, 7)
    ref_logits = F.linear(x, w).squeeze(-1)
    ref_idx, ref_w, _ = eager.mod_route(ref_logits, 7)
    assert torch.equal(idx, ref_idx) and torch.allclose(wts, ref_w) and torch.allclose(logits, ref_logits)
    assert torch.equal(picked, eager.mod_gather(x, ref_idx))
    assert (idx[:, 1:] > idx[:, :-1]).all() and torch.allclose(wts.sum(-1), torch.ones(2))
    aux = torch.randn(2, 10)
    tgt = torch.zeros(2, 10).scatter_(1, idx, 1.0)
    assert torch.allclose(ops.mod_bce(aux, idx), F.binary_cross_entropy_with_logits(aux, tgt, reduction="mean"))


@pytest.mark.parametrize("kw", [dict(mamba_moe_mode="moe_ffn"), dict(mamba_moe_mode="routing_mamba"),
                                dict(moe_routing="expert_choice", mamba_layers=()),
                                dict(moe_balanced_routing=True, mamba_layers=()),
                                dict(moe_drop_tokens=True, moe_capacity_factor=1.0, mamba_layers=())])
def test_input_validation_mode_accepts_what_the_model_itself_produces(kw, monkeypatch):
    """``KMOE_CHECK_INPUTS=1`` validates every data-dependent kernel input; the model's own routers, the
    mixture-of-depths selection, the loss labels and packed-document starts must all pass it, and the result must
    not change."""
    from kolmogorov_moe_architecture_b200.data import PackedDocs
    torch.manual_seed(1)
    m = kmoe.MoETransformer(_tiny(**kw), verbose=False)
    m.train()
    ids = torch.randint(0, 200, (2, 32))
    labels = ids.clone()
    labels[0, :5] = -100
    pd = PackedDocs(doc_ids=torch.tensor([[0] * 7 + [1] * 25, [2] * 32]))
    torch.manual_seed(2)
    ref = m(ids, labels=labels, attention_mask=pd, return_logits=False)["loss"]
    monkeypatch.setenv("KMOE_CHECK_INPUTS", "1")
    torch.manual_seed(2)
    out = m(ids, labels=labels, attention_mask=pd, return_logits=False)["loss"]
    out.backward()
    assert torch.equal(out, ref)
    bad = labels.clone()
    bad[1, 3] = 200
    with pytest.raises(IndexError, match="labels: value 200"):
        m(ids, labels=bad, return_logits=False)
    with pytest.raises(IndexError, match="labels: value 200"):
        m(ids, labels=bad)                                  # the path through materialised logits as well
    toks = ids.clone()
    toks[0, 9] = 200
    with pytest.raises(IndexError, match=r"input_ids: value 200 at position \(0, 9\) is outside \[0, 200\)"):
        m(toks)
    with pytest.raises(IndexError, match="exceeds max_seq_len 32"):
        m(torch.zeros(1, 33, dtype=torch.long))
    with pytest.raises(IndexError, match="position_ids: value 32"):
        m(ids, position_ids=torch.arange(1, 33).expand(2, 32))
