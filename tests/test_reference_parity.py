"""Numerical parity with the reference implementation (imported from ``baseline/_ref`` when it is
installed there): same weights + same input => same loss, gradients and optimizer steps."""
import contextlib
import os as _os
_os.environ.setdefault("MOE_DISABLE_COMPILE", "1")   # the reference torch.compile()s its expert-choice body
import io
import os
import sys

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
REF = os.path.join(ROOT, "baseline", "_ref")
pytestmark = pytest.mark.skipif(not os.path.isdir(os.path.join(REF, "moe_arch")),
                                reason="reference package not installed under baseline/_ref")


@pytest.fixture(scope="module")
def ref():
    saved = {k: v for k, v in sys.modules.items() if k == "moe_arch" or k.startswith("moe_arch.")}
    for k in saved:
        del sys.modules[k]
    sys.path.insert(0, REF)
    with contextlib.redirect_stdout(io.StringIO()):
        import moe_arch.model.config as rc
        import moe_arch.model.transformer as rt
        import moe_arch.training.losses as rl
        import moe_arch.training.lr_schedule as rs
        import moe_arch.training.muon_optimizer as rm
    yield {"config": rc, "transformer": rt, "losses": rl, "sched": rs, "muon": rm}
    sys.path.remove(REF)
    for k in [k for k in sys.modules if k == "moe_arch" or k.startswith("moe_arch.")]:
        del sys.modules[k]
    sys.modules.update(saved)


KW = dict(vocab_size=512, d_model=64, n_layers=4, n_heads=4, n_kv_heads=1, head_dim=16, d_ff=128, d_ff_expert=96,
          n_experts=4, moe_top_k=2, moe_layers=(1, 2), mamba_layers=(1,), max_seq_len=32, n_pred_tokens=4,
          aux_loss_weights=(1.0, 0.5, 0.3, 0.2), dropout=0.0, attention_dropout=0.0, residual_dropout=0.0,
          use_flash_attention=False, device="cpu", dtype="float32")


def test_config_defaults_match(ref):
    from kolmogorov_moe_architecture_b200 import AdvancedMoEConfig
    a, b = AdvancedMoEConfig(), ref["config"].AdvancedMoEConfig()
    for k, v in b.to_dict().items():
        assert getattr(a, k) == v, k
    assert a.count_parameters() == b.count_parameters()


@pytest.mark.parametrize("routing,mod", [("token_choice", True), ("expert_choice", False)])
def test_model_loss_and_grads_match(ref, routing, mod):
    from kolmogorov_moe_architecture_b200 import AdvancedMoEConfig, MoETransformer
    kw = dict(KW, moe_routing=routing, mod_enabled=mod)
    torch.manual_seed(0)
    with contextlib.redirect_stdout(io.StringIO()):
        rmodel = ref["transformer"].MoETransformer(ref["config"].AdvancedMoEConfig(**kw))
    ours = MoETransformer(AdvancedMoEConfig(mamba_impl="simple", **kw), verbose=False)
    missing, unexpected = ours.load_state_dict(rmodel.state_dict(), strict=True)
    assert not missing and not unexpected
    ids = torch.randint(0, 512, (2, 32), generator=torch.Generator().manual_seed(1))
    rmodel.train(); ours.train()
    with contextlib.redirect_stdout(io.StringIO()):
        ro = rmodel(ids, labels=ids)
    oo = ours(ids, labels=ids, return_logits=False)
    assert torch.allclose(oo["lm_loss"], ro["lm_loss"], atol=1e-5), (oo["lm_loss"], ro["lm_loss"])
    assert torch.allclose(oo["loss"], ro["loss"], atol=1e-5)
    ro["loss"].backward(); oo["loss"].backward()
    rg = dict(rmodel.named_parameters())
    for n, p in ours.named_parameters():
        if rg[n].grad is None:
            assert p.grad is None or p.grad.abs().max() == 0, n
        else:
            assert torch.allclose(p.grad, rg[n].grad, atol=2e-5, rtol=1e-3), n
    rmodel.eval(); ours.eval()
    with torch.no_grad(), contextlib.redirect_stdout(io.StringIO()):
        assert torch.allclose(ours(ids)["logits"], rmodel(ids)["logits"], atol=1e-4)


def test_mtp_loss_matches(ref):
    from kolmogorov_moe_architecture_b200.training.losses import MultiTokenPredictionLoss
    g = torch.Generator().manual_seed(0)
    logits = [torch.randn(2, 16, 50, generator=g) for _ in range(3)]
    labels = torch.randint(0, 50, (2, 16), generator=g)
    mask = torch.ones(2, 16, dtype=torch.long); mask[0, 10:] = 0
    with contextlib.redirect_stdout(io.StringIO()):
        r = ref["losses"].MultiTokenPredictionLoss(3, (1.0, 0.5, 0.25))
    o = MultiTokenPredictionLoss(3, (1.0, 0.5, 0.25))
    a, _ = o(logits, labels, attention_mask=mask)
    b, _ = r(logits, labels, attention_mask=mask)
    assert torch.allclose(a, b, atol=1e-6)


@pytest.mark.parametrize("cls", ["Muon", "Muon8bit"])
def test_muon_steps_match(ref, cls):
    from kolmogorov_moe_architecture_b200.training import muon_optimizer as mo
    g = torch.Generator().manual_seed(0)
    shapes = [(24, 40), (40, 24), (3, 16, 24), (17,)]
    pa = [torch.randn(*s, generator=g).requires_grad_(True) for s in shapes]
    pb = [p.detach().clone().requires_grad_(True) for p in pa]
    with contextlib.redirect_stdout(io.StringIO()):
        oa = getattr(mo, cls)(pa, lr=1e-2)
        ob = getattr(ref["muon"], cls)(pb, lr=1e-2)
    for _ in range(3):
        for x, y in zip(pa, pb):
            gr = torch.randn(*x.shape, generator=g)
            x.grad, y.grad = gr.clone(), gr.clone()
        oa.step(); ob.step()
    for x, y in zip(pa, pb):
        assert torch.allclose(x, y, atol=1e-5), x.shape


def test_newton_schulz_orthogonality():
    from kolmogorov_moe_architecture_b200.ops import eager
    m = torch.randn(32, 64, generator=torch.Generator().manual_seed(0))
    q = eager.newton_schulz(m, 10)
    assert (q @ q.T - torch.eye(32)).abs().max() < 0.1


def test_schedule_matches(ref):
    from kolmogorov_moe_architecture_b200.training.lr_schedule import CosineScheduleWithWarmup
    p = [torch.zeros(1, requires_grad=True)]
    oa, ob = torch.optim.SGD(p, lr=1.0), torch.optim.SGD(p, lr=1.0)
    with contextlib.redirect_stdout(io.StringIO()):
        r = ref["sched"].CosineScheduleWithWarmup(ob, 5, 50, 1e-3, 1e-4)
    o = CosineScheduleWithWarmup(oa, 5, 50, 1e-3, 1e-4)
    for _ in range(60):
        assert abs(o.step() - r.step()) < 1e-12
    assert o.state_dict() == r.state_dict()


@pytest.mark.parametrize("fsdp_mode", [False, True])
def test_hybrid_optimizer_partition_matches(ref, fsdp_mode, monkeypatch):
    """Which tensors go to Muon and which to AdamW: the reference decides by name and dimension, and by name
    alone when it believes it runs distributed (it looks at WORLD_SIZE / LOCAL_RANK)."""
    from kolmogorov_moe_architecture_b200 import AdvancedMoEConfig, MoETransformer
    from kolmogorov_moe_architecture_b200.training.muon_optimizer import split_muon_params
    for k in ("WORLD_SIZE", "LOCAL_RANK"):
        monkeypatch.delenv(k, raising=False)
    if fsdp_mode:
        monkeypatch.setenv("WORLD_SIZE", "2")
    torch.manual_seed(0)
    with contextlib.redirect_stdout(io.StringIO()):
        rmodel = ref["transformer"].MoETransformer(ref["config"].AdvancedMoEConfig(**KW))
        ropt = ref["muon"].get_muon_optimizer(rmodel, lr=1e-3)
    ours = MoETransformer(AdvancedMoEConfig(mamba_impl="simple", **KW), verbose=False)
    rnames = {id(p): n for n, p in rmodel.named_parameters()}
    ref_muon = {rnames[id(p)] for g in ropt.muon_opt.param_groups for p in g["params"]}
    ref_adam = {rnames[id(p)] for g in ropt.adamw_opt.param_groups for p in g["params"]}
    mu, ad = split_muon_params(ours, fsdp_mode=fsdp_mode)
    onames = {id(p): n for n, p in ours.named_parameters()}
    assert {onames[id(p)] for p in mu} == ref_muon
    assert {onames[id(p)] for p in ad} == ref_adam


def test_memory_mapped_dataset_matches(ref, tmp_path):
    """Same ``.bin`` file, same samples: fixed strides of ``seq_len + n_pred_tokens`` tokens, labels equal to
    the inputs (the model shifts them itself)."""
    import numpy as np
    from kolmogorov_moe_architecture_b200.data import DolmaMemoryMappedDataset, write_token_file
    with contextlib.redirect_stdout(io.StringIO()):
        import moe_arch.data.dolma_dataset as rd
    path = str(tmp_path / "train.bin")
    toks = np.random.default_rng(0).integers(0, 50000, size=1000)
    write_token_file(path, toks)
    with contextlib.redirect_stdout(io.StringIO()):
        r = rd.DolmaMemoryMappedDataset(path, seq_len=32, n_pred_tokens=4)
    o = DolmaMemoryMappedDataset(path, seq_len=32, n_pred_tokens=4)
    assert len(o) == len(r) == 1000 // 36
    for i in (0, 5, len(o) - 1):
        a, b = o[i], r[i]
        assert torch.equal(a["input_ids"], b["input_ids"]) and torch.equal(a["labels"], b["labels"])
        assert a["input_ids"].dtype == torch.int64 and a["input_ids"].shape == (32,)


def test_expert_parallel_layer_single_process_matches(ref):
    """``ExpertParallelMoE`` with all experts on one rank: same router rule (softmax over the top-k logits),
    same experts, same auxiliary loss as the reference layer."""
    from kolmogorov_moe_architecture_b200 import AdvancedMoEConfig
    from kolmogorov_moe_architecture_b200.models.sparse_moe import ExpertParallelMoE
    with contextlib.redirect_stdout(io.StringIO()):
        import moe_arch.model.sparse_moe as rsm
        torch.manual_seed(0)
        r = rsm.ExpertParallelMoE(ref["config"].AdvancedMoEConfig(**dict(KW, moe_implementation="expert_parallel")), 1)
    o = ExpertParallelMoE(AdvancedMoEConfig(**dict(KW, moe_implementation="expert_parallel")), 1)
    missing, unexpected = o.load_state_dict(r.state_dict(), strict=True)
    assert not missing and not unexpected
    x = torch.randn(2, 16, 64, generator=torch.Generator().manual_seed(2))
    r.train(); o.train()
    with contextlib.redirect_stdout(io.StringIO()):
        yr = r(x)
    yo = o(x)
    assert torch.allclose(yo, yr, atol=1e-5), (yo - yr).abs().max()
    assert abs(float(o.aux_loss) - float(r.aux_loss)) < 1e-6


def test_stand_alone_moe_layer_variants_match(ref):
    """The stand-alone layer classes of ``fused_moe.py`` and ``triton_moe.py`` that run without a GPU: same
    state dict keys, same outputs."""
    from kolmogorov_moe_architecture_b200.models import fused_moe as of, triton_moe as ot
    with contextlib.redirect_stdout(io.StringIO()):
        import moe_arch.model.fused_moe as rf
        import moe_arch.model.triton_moe as rt
    torch.manual_seed(0)
    T, d, f, E, k = 20, 16, 32, 4, 2
    x = torch.randn(T, d)
    w, idx = torch.softmax(torch.randn(T, E), -1).topk(k, dim=-1)
    w = w / w.sum(-1, keepdim=True)
    for rcls, ocls in ((rf.OptimizedGroupedExperts, of.OptimizedGroupedExperts), (rt.BatchedMoE, ot.BatchedMoE),
                       (rt.BatchedMoEOptimized, ot.BatchedMoEOptimized)):
        with contextlib.redirect_stdout(io.StringIO()):
            r = rcls(E, d, f)
        o = ocls(E, d, f)
        assert not any(o.load_state_dict(r.state_dict(), strict=True))
        with contextlib.redirect_stdout(io.StringIO()):
            yr = r(x, idx, w)
        assert torch.allclose(o(x, idx, w), yr, atol=1e-5), rcls.__name__
    with contextlib.redirect_stdout(io.StringIO()):
        r = rf.FusedSparseMoE(d, f, E, k)
    o = of.FusedSparseMoE(d, f, E, k)
    assert not any(o.load_state_dict(r.state_dict(), strict=True))
    xb = torch.randn(2, 10, d)
    with contextlib.redirect_stdout(io.StringIO()):
        yr = r(xb)
    assert torch.allclose(o(xb), yr, atol=1e-5)


def test_reference_arm_builds_the_benchmark_layer(ref):
    """The benchmark's reference arm in ``moe_ffn`` mode (Mamba mixer + MoE FFN composed from the
    reference's own classes) holds exactly the parameters of this framework's model in that mode,
    loads into it strictly, and gives the same loss."""
    from baseline.run_reference import _build_model
    from kolmogorov_moe_architecture_b200 import AdvancedMoEConfig, MoETransformer
    kw = dict(KW, mod_enabled=True)
    torch.manual_seed(0)
    with contextlib.redirect_stdout(io.StringIO()):
        rmodel = _build_model(ref["transformer"].MoETransformer, ref["config"].AdvancedMoEConfig(**kw), "moe_ffn")
        stock = _build_model(ref["transformer"].MoETransformer, ref["config"].AdvancedMoEConfig(**kw), "routing_mamba")
    assert type(rmodel.layers[1]).__name__ == "MambaMoEBlock"
    assert type(rmodel.layers[1].seq_layer).__name__ == "MambaBlock"
    assert type(rmodel.layers[1].ffn).__name__ == "MoELayer"
    assert type(stock.layers[1].seq_layer).__name__ == "RoutingMamba"
    assert ref["transformer"].TransformerBlock.__name__ == "TransformerBlock"      # lookup restored
    ours = MoETransformer(AdvancedMoEConfig(mamba_impl="simple", mamba_moe_mode="moe_ffn", **kw), verbose=False)
    n_ref = sum(p.numel() for p in rmodel.parameters())
    assert n_ref == sum(p.numel() for p in ours.parameters())
    assert n_ref != sum(p.numel() for p in stock.parameters())
    missing, unexpected = ours.load_state_dict(rmodel.state_dict(), strict=True)
    assert not missing and not unexpected
    ids = torch.randint(0, 512, (2, 32), generator=torch.Generator().manual_seed(1))
    rmodel.train(); ours.train()
    with contextlib.redirect_stdout(io.StringIO()):
        ro = rmodel(ids, labels=ids)
    oo = ours(ids, labels=ids, return_logits=False)
    assert torch.allclose(oo["loss"], ro["loss"], atol=1e-5), (oo["loss"], ro["loss"])
