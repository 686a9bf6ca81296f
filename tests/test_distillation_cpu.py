"""Sparse distillation pipeline on a toy transformer (CPU)."""
import torch

from experiments.sparse_distillation.convert import convert_to_sparse
from experiments.sparse_distillation.distill import (DistillationConfig, MoEDistillationLayer,
                                                     SparseDistillationTrainer, cluster_quality, kmeans)
from experiments.sparse_distillation.dynamic_experts import (DynamicExpertLayer, interpolate_expert_weights,
                                                             reallocate_expert_layer)
from experiments.sparse_distillation.example_usage import ToyLM
from experiments.sparse_distillation.generate_config import choose_layer_config
from experiments.sparse_distillation.hooks import FFNActivationCache, find_ffn_modules


def _cfg(**kw):
    base = dict(n_experts=4, moe_top_k=2, data_free=True, data_free_steps=30, data_free_seq_len=32,
                data_free_batch_size=2, cluster_samples=512, router_train_steps=20, log_interval=0,
                learning_rate=2e-3)
    base.update(kw)
    return DistillationConfig(**base)


def test_hooks_capture_ffn_io():
    torch.manual_seed(0)
    m = ToyLM()
    assert len(find_ffn_modules(m)) == 2
    with FFNActivationCache(m) as c:
        m(torch.randint(0, 256, (2, 8)))
    assert c.inputs[0].shape == (2, 8, 64) and c.outputs[1].shape == (2, 8, 64)


def test_init_from_dense_makes_experts_tile_the_dense_ffn():
    torch.manual_seed(0)
    m = ToyLM()
    layer = MoEDistillationLayer(64, 64, _cfg())
    assert layer.init_from_dense_ffn(m.blocks[0].mlp, noise=0.0)
    assert torch.allclose(layer.experts.w1[1], m.blocks[0].mlp.gate_proj.weight[64:128].t())


def test_data_free_distillation_reduces_error_and_converts():
    torch.manual_seed(0)
    m = ToyLM().eval()
    tr = SparseDistillationTrainer(m, _cfg(), device="cpu")
    hist = tr.distill(steps=40)
    assert sum(hist[0][-5:]) < sum(hist[0][:5])
    ev = tr.evaluate(2)
    assert ev[0]["cosine"] > 0.5
    sparse = convert_to_sparse(m, trainer=tr)
    out = sparse(torch.randint(0, 256, (2, 16)))
    assert out["logits"].shape == (2, 16, 256)
    assert set(sparse.routing_stats()) == {0, 1}


def test_empirical_and_dynamic_and_expert_choice_modes_run():
    torch.manual_seed(0)
    for kw in (dict(empirical_routing=True, supervised_routing=False), dict(dynamic_experts=True, reallocate_every_n_steps=5, min_d_ff=16),
               dict(moe_routing="expert_choice", supervised_routing=False)):
        tr = SparseDistillationTrainer(ToyLM().eval(), _cfg(**kw), device="cpu")
        hist = tr.distill(steps=8)
        assert all(torch.isfinite(torch.tensor(v)).all() for v in hist.values())


def test_save_load_roundtrip(tmp_path):
    torch.manual_seed(0)
    m = ToyLM().eval()
    tr = SparseDistillationTrainer(m, _cfg(), device="cpu")
    tr.save(str(tmp_path / "d.pt"))
    sparse = convert_to_sparse(ToyLM().eval(), distilled_path=str(tmp_path / "d.pt"))
    assert sparse.count_parameters()["active"] < sparse.count_parameters()["total"]


def test_kmeans_and_quality_and_layer_config():
    g = torch.Generator().manual_seed(0)
    x = torch.cat([torch.randn(100, 8, generator=g) + 6 * i for i in range(3)])
    assign, cent = kmeans(x, 3)
    q = cluster_quality(x, assign, cent)
    assert q["silhouette"] > 0.5 and q["balance"] > 0.9
    cfg = choose_layer_config({"4": {"silhouette": 0.2, "balance": 0.9}, "8": {"silhouette": 0.4, "balance": 0.9}}, 1024)
    assert cfg["n_experts"] == 8 and cfg["d_ff_expert"] == 256 and cfg["top_k"] == 1


def test_dynamic_expert_resize():
    w1, w2, w3 = torch.randn(8, 32), torch.randn(8, 32), torch.randn(32, 8)
    a, b, c = interpolate_expert_weights(w1, w2, w3, 16)
    assert a.shape == (8, 16) and c.shape == (16, 8)
    a, b, c = interpolate_expert_weights(w1, w2, w3, 48)
    assert a.shape == (8, 48) and c.shape == (48, 8)
    layer = reallocate_expert_layer(DynamicExpertLayer(8, [32, 32]), {0: 48, 1: 16})
    out = layer(torch.randn(5, 8), torch.tensor([[0], [1], [0], [1], [0]]), torch.ones(5, 1))
    assert out.shape == (5, 8) and layer.d_ffs == [48, 16]


def test_router_supervision_from_real_activations():
    """Clusters of the dense FFN's outputs on real batches supervise the router: its loss against the
    cluster labels falls, and the collected activations are the hooked layer's own input/output."""
    torch.manual_seed(0)
    m = ToyLM().eval()
    tr = SparseDistillationTrainer(m, _cfg(cluster_samples=256), device="cpu")
    batches = [{"input_ids": torch.randint(0, 256, (4, 16))} for _ in range(6)]
    X, Y = tr._collect_ffn_activations_from_data(batches, 1, max_samples=200)
    assert X.shape == Y.shape == (200, 64)
    with torch.no_grad():
        assert torch.allclose(m.blocks[1].mlp(X[:8]), Y[:8], atol=1e-5)
    first = tr._train_router_supervised(1, steps=1, batches=batches)
    last = tr._train_router_supervised(1, steps=60, batches=batches)
    assert last < first
    q = tr.analyze_cluster_quality(0, ks=(2, 4), batches=batches)
    assert set(q) == {2, 4}


def test_finetune_eval_cli_and_routing_statistics(tmp_path):
    """Distil, save, then run the fine-tune/evaluate command line on the saved file: routing statistics over
    several batches, perplexity before/after, best and latest checkpoints, resume from the latest one."""
    from experiments.sparse_distillation import finetune_eval as fe
    torch.manual_seed(0)
    m = ToyLM().eval()
    tr = SparseDistillationTrainer(m, _cfg(), device="cpu")
    tr.distill(steps=10)
    ck = str(tmp_path / "distilled.pt")
    tr.save(ck)
    out = str(tmp_path / "ft")
    rep = fe.main(["--checkpoint", ck, "--max_steps", "8", "--eval_every", "4", "--moe_only", "--compare_dense",
                   "--output", out, "--seq_len", "16", "--eval_batches", "2", "--lr", "1e-3"])
    # random tokens carry nothing to learn: perplexity stays near the vocabulary size, for dense and sparse alike
    assert abs(rep["ppl_after"] - rep["ppl_before"]) < 0.05 * rep["ppl_before"]
    assert 100 < rep["dense_ppl"] < 600 and [h["step"] for h in rep["finetune"]["history"]] == [4, 8]
    assert 0.0 < rep["routing_before"]["mean_normalized_entropy"] <= 1.0
    assert (tmp_path / "ft" / "best_checkpoint.pt").exists() and (tmp_path / "ft" / "latest_checkpoint.pt").exists()
    rep2 = fe.main(["--checkpoint", ck, "--max_steps", "10", "--resume", out + "/latest_checkpoint.pt", "--moe_only",
                    "--seq_len", "16", "--eval_batches", "2"])
    assert len(rep2["finetune"]["history"]) >= 1 and rep2["finetune"]["history"][0]["step"] > 8
    # per-layer figures from hand-made counts
    st = fe._layer_stats(torch.tensor([10.0, 10.0, 0.0, 0.0]))
    assert st["active_experts"] == 2 and abs(st["normalized_entropy"] - 0.5) < 1e-3 and not st["collapsed"]
    assert fe._layer_stats(torch.tensor([100.0, 0.0, 0.0, 0.0]))["collapsed"]


def test_dynamic_expert_tracker_reallocation_keeps_the_budget():
    from experiments.sparse_distillation.dynamic_experts import (DynamicExpertConfig, DynamicExpertTracker,
                                                                 print_active_params_report)
    torch.manual_seed(0)
    cfg = DynamicExpertConfig(reallocate_every_n_steps=2, min_d_ff=16, max_d_ff=512, top_k_grow=1, top_k_shrink=1)
    layer = DynamicExpertLayer(32, [64, 64, 64, 64])
    tr = DynamicExpertTracker(4, initial_d_ff=64, d_model=32, config=cfg)
    x = torch.randn(40, 32)
    for step in range(2):
        outs = {e: layer.forward_expert(x[e * 10:(e + 1) * 10], e) for e in range(4)}
        tgts = {e: outs[e].detach() + (3.0 if e == 2 else 0.1 * (e + 1)) for e in range(4)}   # expert 2 is the worst
        tr.update_stats(outs, tgts)
    assert tr.should_reallocate()
    new = tr.compute_reallocation()
    assert new[2] == max(new.values()) and new[0] == min(new.values())
    assert abs(sum(new.values()) - 4 * 64) <= 4 * cfg.round_to and all(f % cfg.round_to == 0 for f in new.values())
    before = layer.get_total_params()
    reallocate_expert_layer(layer, {e: f for e, f in new.items() if f != layer.d_ffs[e]})
    tr.set_widths(layer.d_ffs)
    tr.reset_stats()
    assert abs(layer.get_total_params() - before) <= 3 * 32 * 4 * cfg.round_to
    assert "expert  2" in tr.get_report() and tr.expert_stats[2].token_count == 0
    rep = print_active_params_report({0: layer}, top_k=2, usage={0: torch.tensor([1.0, 1.0, 0.0, 0.0])})
    assert rep[0]["active"] == 2 * 0.5 * (layer.get_expert_params(0) + layer.get_expert_params(1))
    assert layer(x, torch.randint(0, 4, (40, 2)), torch.rand(40, 2)).shape == x.shape


def test_compute_layer_config_holds_the_ratios(tmp_path):
    import json
    from experiments.sparse_distillation.generate_config import compute_layer_config, main
    analysis = {"d_model": 64, "d_ff": 1024, "layers": {
        "0": {"n_experts": 8, "balance": 0.9, "silhouette": 0.2},
        "1": {"n_experts": 2, "balance": 0.8, "all_results": {"2": {"balance": 0.8}, "4": {"balance": 0.5}, "16": {"balance": 0.7}}},
        "2": {"n_experts": 2, "balance": 0.8}}}
    cfg = compute_layer_config(analysis, 3.0, 0.25, min_experts=4, verbose=False)
    L = cfg["layers"]
    assert L["0"] == {"n_experts": 8, "d_ff_expert": 384, "top_k": 1, "balance": 0.9, "silhouette": 0.2}
    assert L["1"]["n_experts"] == 16 and L["1"]["balance"] == 0.7 and L["1"]["d_ff_expert"] == 192
    assert L["2"]["n_experts"] == 4 and L["2"]["d_ff_expert"] == 768
    assert abs(cfg["stats"]["actual_expansion_ratio"] - 3.0) < 1e-6
    f = tmp_path / "a.json"
    f.write_text(json.dumps(analysis))
    out = main(["--analysis", str(f), "--output", str(tmp_path / "o.json")])
    assert json.load(open(tmp_path / "o.json"))["layers"] == out["layers"]
