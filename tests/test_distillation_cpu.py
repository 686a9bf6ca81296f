"""Sparse distillation pipeline on a toy transformer (CPU)."""
import pytest
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


def test_command_lines_take_the_reference_arguments(tmp_path, capsys):
    """analyse clusters -> per-layer configuration -> distil with it -> fine-tune / evaluate, each step driven through
    its command line with the argument names of the reference's scripts
    (Experiments/sparse_distillation/{example_usage,generate_config,finetune_eval}.py)."""
    import json
    from experiments.sparse_distillation import example_usage as eu, finetune_eval as fe, generate_config as gc
    out = str(tmp_path / "o")
    # every flag of the reference's example_usage parses, and lands in the configuration
    a = eu.build_parser().parse_args(
        "--model toy --dtype float32 --dataset wikitext --dataset_config wikitext-2-raw-v1 --max_samples 64 "
        "--seq_len 32 --batch_size 2 --n_experts 6 --moe_top_k 3 --capacity_factor 1.5 --d_ff_expert 0.5 "
        "--routing token_choice --epochs 2 --lr 3e-4 --max_steps 7 --sequential --no_data_free --data_free_steps 9 "
        "--data_free_batch_size 3 --data_free_seq_len 48 --no_compile --no_load_balance --load_balance_weight 0.02 "
        "--no_z_loss --z_loss_weight 0.002 --no_supervised_routing --cluster_samples 500 --router_train_steps 11 "
        "--empirical_routing --empirical_eval_interval 5 --empirical_temperature 0.2 --empirical_entropy_weight 0.03 "
        "--no_curriculum --curriculum_warmup_steps 50 --curriculum_initial_balance 0.8 --curriculum_final_balance 0.2 "
        "--no_gradient_routing --gradient_routing_exact --router_mlp --router_hidden_dim 32 --router_n_layers 3 "
        "--dynamic --reallocate_every 4 --growth_factor 1.5 --shrink_factor 0.7 --min_d_ff 16 --max_d_ff 512 "
        f"--output {out} --device cpu".split())
    c = eu.config_from_args(a)
    assert (c.n_experts, c.moe_top_k, c.moe_capacity_factor, c.d_ff_expert, c.learning_rate) == (6, 3, 1.5, 0.5, 3e-4)
    assert c.sequential_layers and not c.data_free and (c.data_free_steps, c.data_free_batch_size) == (9, 3)
    assert not c.use_load_balancing and c.load_balancing_weight == 0.02 and not c.use_z_loss and c.z_loss_weight == 0.002
    assert not c.supervised_routing and c.cluster_samples == 500 and c.router_train_steps == 11
    assert c.empirical_routing and c.empirical_eval_interval == 5 and c.empirical_temperature == 0.2
    assert not c.curriculum_routing and c.curriculum_warmup_steps == 50 and c.curriculum_final_balance == 0.2
    assert not c.gradient_routing and not c.gradient_routing_fast
    assert c.router_mlp and (c.router_hidden_dim, c.router_n_layers) == (32, 3)
    assert c.dynamic_experts and (c.reallocate_every_n_steps, c.growth_factor, c.min_d_ff, c.max_d_ff) == (4, 1.5, 16, 512)
    assert eu.parse_expert_width("2048") == 2048 and eu.parse_expert_width("0.075") == 0.075
    assert eu.parse_expert_width(None) is None and eu.parse_expert_width("auto") is None
    # 1. cluster analysis (stops after writing the file)
    _, sparse, analysis = eu.main(["--analyze_clusters", "--steps", "4", "--k_values", "2,4", "--output", out])
    assert sparse is None and set(analysis["layers"]) == {"0", "1"} and analysis["d_ff"] == 256
    # 2. per-layer configuration, positional path, default output beside it
    cfg = gc.main([out + "/cluster_analysis.json", "--expansion_ratio", "2", "--active_ratio", "0.5", "--min_experts",
                   "2", "--min_top_k", "1", "--max_top_k", "4"])
    saved = json.load(open(out + "/layer_config.json"))
    assert saved["layers"] == cfg["layers"] and abs(cfg["stats"]["actual_expansion_ratio"] - 2.0) < 1e-6
    # 3. distillation with that configuration, on token batches, two epochs
    tr, sparse, ev = eu.main(["--layer_config", out + "/layer_config.json", "--no_data_free", "--max_steps", "6",
                              "--epochs", "2", "--steps", "6", "--output", out])
    for i, lc in cfg["layers"].items():
        layer = tr.moe_layers[i]
        assert (layer.n_experts, layer.d_ff, layer.top_k) == (lc["n_experts"], lc["d_ff_expert"], lc["top_k"])
    assert set(ev) == {0, 1} and all(0 < v["rel_mse"] < 2 for v in ev.values())
    assert (tmp_path / "o" / "distilled_moe_layers.pt").exists() and (tmp_path / "o" / "sparse_model.pt").exists()
    # 4. fine-tune / evaluate with the reference's switches
    rep = fe.main(["--model", "toy", "--checkpoint", out + "/distilled_moe_layers.pt", "--layer_config",
                   out + "/layer_config.json", "--dtype", "float32", "--dataset", "wikitext", "--dataset_config",
                   "wikitext-2-raw-v1", "--max_samples", "32", "--epochs", "1", "--max_steps", "4", "--eval_every", "2",
                   "--eval_batches", "2", "--seq_len", "16", "--batch_size", "2", "--balanced-routing", "--no_8bit_adam",
                   "--moe_only", "--load_balance_weight", "0.01", "--z_loss_weight", "0.001", "--device", "cpu"])
    assert rep["balanced_routing_layers"] == 2 and rep["data"] == "random" and rep["finetune"]["optimizer"] == "adamw"
    capsys.readouterr()
    # a layer configuration that contradicts the checkpoint is refused
    bad = json.load(open(out + "/layer_config.json"))
    bad["layers"]["0"]["n_experts"] += 1
    json.dump(bad, open(out + "/bad.json", "w"))
    with pytest.raises(ValueError, match="layer 0: the layer configuration says"):
        fe.main(["--checkpoint", out + "/distilled_moe_layers.pt", "--layer_config", out + "/bad.json", "--eval_only"])


def test_balanced_routing_brings_unused_experts_into_use():
    """Two experts that every token prefers: plain top-2 leaves the other two without a token; with the capacity of
    T k / E checked at the start of each slot (the reference's rule, moe.py:353-421), whichever of the two is full
    after the first slot is closed in the second, and its tokens go to the idle experts."""
    from experiments.sparse_distillation.distill import MoEDistillationLayer
    torch.manual_seed(0)
    layer = MoEDistillationLayer(32, 16, _cfg(), n_experts=4, top_k=2)
    with torch.no_grad():
        layer.expert_bias[0] = 8.0
        layer.expert_bias[1] = 8.0
    x = torch.randn(2, 24, 32)
    layer(x)
    free = layer._last_expert_counts.clone()
    layer.balanced_routing = True
    out = layer(x)
    bal = layer._last_expert_counts
    assert free.tolist() == [48, 48, 0, 0]
    assert int(bal.sum()) == 96 and int((bal == 0).sum()) == 0 and out.shape == x.shape


def test_reference_names_of_hooks_wrapper_and_helpers():
    """The reference's spellings work: ``Experiments.sparse_distillation`` import path, ``register_hooks`` /
    ``get_activations`` / ``FFNActivation``, ``StreamingFFNExtractor.extract``, ``SparseModelWrapper.base_model`` /
    ``moe_layers`` / ``n_experts`` / ``get_active_parameters``, the loss helpers and ``freeze_non_moe_layers``."""
    import Experiments.sparse_distillation as ES
    from Experiments.sparse_distillation.finetune_eval import (compute_load_balancing_loss, compute_z_loss,
                                                               freeze_non_moe_layers)
    from Experiments.sparse_distillation.hooks import FFNActivation, StreamingFFNExtractor
    assert ES.SparseDistillationTrainer is SparseDistillationTrainer and ES.FFNActivationCache is FFNActivationCache
    torch.manual_seed(0)
    m = ToyLM().eval()
    ids = torch.randint(0, 256, (2, 12))
    cache = FFNActivationCache(m)
    cache.register_hooks()
    with torch.no_grad():
        m(ids)
    acts = cache.get_activations()
    cache.remove_hooks()
    assert cache.layer_indices == [0, 1] and set(acts) == {0, 1} and isinstance(acts[0], FFNActivation)
    with torch.no_grad():
        assert torch.allclose(m.blocks[1].mlp(acts[1].input), acts[1].output, atol=1e-6)
    assert cache.get_layer_activation(1).layer_idx == 1 and cache.get_layer_activation(7) is None
    only_first = FFNActivationCache(m, layer_filter=lambda name, mod: name == "blocks.0.mlp")
    assert [n for n, _ in only_first.ffn] == ["blocks.0.mlp"]
    ex = StreamingFFNExtractor(m)
    got = ex.extract(ids)
    assert ex.n_layers == 2 and ex.layer_indices == [0, 1] and torch.equal(got[0].input, acts[0].input)
    ex.close()
    with torch.no_grad():
        m(ids)                                   # hooks are gone: nothing is recorded any more
    seen = []
    with StreamingFFNExtractor(m, lambda i, x, y: seen.append((i, tuple(x.shape)))):
        with torch.no_grad():
            m(ids)
    assert seen == [(0, (2, 12, 64)), (1, (2, 12, 64))]
    tr = SparseDistillationTrainer(dense_model=m, config=_cfg(), device="cpu")
    wrapper = convert_to_sparse(dense_model=m, trainer=tr)
    assert wrapper.base_model is m and wrapper.n_experts == _cfg().n_experts
    assert set(wrapper.moe_layers.keys()) == {"0", "1"} and len(list(wrapper.parameters())) == len(list(m.parameters()))
    total = sum(p.numel() for p in m.parameters())
    experts = sum(p.numel() for l in wrapper.moe_layers.values() for p in l.experts.parameters())
    k, E = _cfg().moe_top_k, _cfg().n_experts
    assert wrapper.get_active_parameters() == int(total - experts * (1 - k / E))
    assert wrapper.get_active_parameters(top_k=E) == total
    logits, counts = torch.zeros(6, 4), torch.tensor([3, 3, 3, 3])
    assert abs(float(compute_load_balancing_loss(logits, counts)) - 1.0) < 1e-6      # uniform: E * sum (1/E)(1/E) = 1
    assert abs(float(compute_z_loss(logits)) - torch.log(torch.tensor(4.0)).pow(2).item()) < 1e-6
    kept = freeze_non_moe_layers(wrapper, moe_only=True)
    names = {n for n, p in wrapper.named_parameters() if p.requires_grad}
    assert kept and all(("experts" in n or "router" in n or "expert_bias" in n or "norm" in n) for n in names)
    assert not any(n.endswith("emb.weight") or n.endswith("head.weight") for n in names)
    assert len(freeze_non_moe_layers(wrapper, moe_only=False)) == len(list(wrapper.parameters()))


def test_call_forms_of_the_reference_are_accepted():
    """Constructors and functions of the package can be called the way the reference's are: argument order,
    keyword names, and what comes back."""
    from experiments.sparse_distillation import finetune_eval as fe
    from experiments.sparse_distillation.convert import SparseModelWrapper, replace_ffn_with_moe
    from experiments.sparse_distillation.dynamic_experts import DynamicExpertLayer
    from experiments.sparse_distillation.hooks import StreamingFFNExtractor
    torch.manual_seed(0)
    # layer with its settings spelled out
    layer = MoEDistillationLayer(32, 16, 4, capacity_factor=2.0, routing_type="token_choice", mlp_router=True,
                                 router_hidden_dim=8, router_n_layers=2, use_expert_bias=False)
    assert (layer.n_experts, layer.d_ff, layer.routing) == (4, 16, "token_choice") and layer.expert_bias is None
    assert layer.cfg.moe_capacity_factor == 2.0 and layer(torch.randn(2, 5, 32)).shape == (2, 5, 32)
    assert MoEDistillationLayer(d_model=32, d_ff=16, n_experts=4).routing == "expert_choice"
    # trainer: default configuration, layer filter, loss with and without metrics, a step on activations
    m = ToyLM().eval()
    tr = SparseDistillationTrainer(dense_model=m, config=_cfg(), device="cpu",
                                   layer_filter=lambda name, mod: name.endswith("mlp"))
    assert len(tr.ffn) == 2 and SparseDistillationTrainer(dense_model=ToyLM()).cfg.n_experts == 16
    x = torch.randn(2, 6, 64)
    y = tr._teacher(0, x)
    out, aux = tr.moe_layers["0"](x, return_aux=True)
    loss = tr.compute_loss(moe_output=out, target=y, aux_info=aux)
    loss2, metrics = tr.compute_loss(out, y, aux, return_metrics=True)
    assert torch.is_tensor(loss) and torch.equal(loss, loss2) and "mse" in metrics
    assert float(tr.compute_loss(out, y).detach()) > 0                              # no routing information: MSE (+ cosine)
    assert float(tr.compute_load_balancing_loss(router_logits=aux["router_logits"], expert_counts=aux["expert_counts"])) > 0
    assert float(tr.compute_z_loss(router_logits=aux["router_logits"])) >= 0
    ids = torch.randint(0, 256, (2, 10))
    acts = StreamingFFNExtractor(m).extract(ids)
    step = tr.train_step(acts)
    assert set(step) == {0, 1} and all(isinstance(v, float) for v in step.values())
    assert "mse" in tr.train_step(activations=acts, return_metrics=True)[0]
    q = tr.analyze_cluster_quality(acts[0].output, [2, 3])
    assert set(q) == {2, 3} and "balance" in q[2]
    assert set(tr.evaluate([ids, ids], max_batches=1)) == {0, 1} and set(tr.evaluate(dataloader=[{"input_ids": ids}])) == {0, 1}
    # conversion: the reference's argument order and keyword names
    wrapper = SparseModelWrapper(base_model=replace_ffn_with_moe(m, tr.get_moe_layers(), layer_indices=[0, 1],
                                                                 ffn_name_pattern="mlp", inplace=True),
                                 moe_layers=tr.get_moe_layers(), layer_indices=[0, 1])
    assert wrapper.moe_paths == {0: "blocks.0.mlp", 1: "blocks.1.mlp"}
    copy_ = replace_ffn_with_moe(ToyLM(), tr.get_moe_layers(), [0], inplace=False)
    assert type(copy_.blocks[0].mlp).__name__ == "MoEDistillationLayer" and type(copy_.blocks[1].mlp).__name__ != "MoEDistillationLayer"
    # perplexity and fine-tuning with data loaders, a device and the reference's keywords
    batches = [{"input_ids": torch.randint(0, 256, (2, 12))} for _ in range(3)]
    p1 = fe.compute_perplexity(wrapper, batches, "cpu", pad_token_id=None, max_batches=2, accumulate_routing=True)
    assert p1 == fe.compute_perplexity(model=wrapper, dataloader=batches, device="cpu", max_batches=2)
    rep = fe.finetune(wrapper, batches, batches[:1], "cpu", epochs=2, lr=1e-3, eval_every=3, max_steps=5,
                      use_8bit_adam=False, moe_only=True, load_balance_weight=0.01, z_loss_weight=0.001,
                      use_lr_schedule=True)
    assert rep["history"][-1]["step"] == 5 and rep["optimizer"] == "adamw"
    rep2 = fe.finetune(model=wrapper, train_dataloader=batches, eval_dataloader=batches[:1], device="cpu", epochs=1)
    assert rep2["history"][-1]["step"] == 3
    # dynamic experts in the reference's argument order and its expert-choice forward
    dyn = DynamicExpertLayer(3, 16, [8, 16, 24])
    assert dyn.n_experts == 3 and dyn.d_model == 16 and dyn.d_ff_per_expert == [8, 16, 24]
    assert dyn.get_expert_params(expert_idx=2) == 3 * 16 * 24
    xb = torch.randn(2, 7, 16)
    ti = torch.stack([torch.stack([torch.randperm(7)[:3] for _ in range(3)]) for _ in range(2)])
    ew = torch.rand(2, 3, 3)
    yb, per = dyn(xb, ew, ti)
    want = torch.zeros_like(xb)
    for b in range(2):
        for e in range(3):
            want[b].index_add_(0, ti[b, e], dyn.expert(e, xb[b, ti[b, e]]) * ew[b, e].unsqueeze(1))
    assert torch.allclose(yb, want, atol=1e-5) and per[1].shape == (2, 3, 16)
    a, b_, c = interpolate_expert_weights(old_w1=dyn.w1[0].data, old_w2=dyn.w2[0].data, old_w3=dyn.w3[0].data, new_d_ff=12)
    assert a.shape == (16, 12) and c.shape == (12, 16)
    assert reallocate_expert_layer(dyn, new_d_ff=[8, 32, 24], device="cpu").d_ffs == [8, 32, 24]


def test_finetune_checkpoints_carry_the_reference_keys_and_its_files_load(tmp_path):
    from experiments.sparse_distillation import finetune_eval as fe
    torch.manual_seed(0)
    m = ToyLM().eval()
    tr = SparseDistillationTrainer(m, _cfg(), device="cpu")
    wrapper = convert_to_sparse(m, trainer=tr)
    batches = [torch.randint(0, 256, (2, 12)) for _ in range(2)]
    fe.finetune(wrapper, batches, 2, lr=1e-3, out_dir=str(tmp_path), eval_batches=batches[:1], eval_every=1)
    ck = torch.load(tmp_path / "latest_checkpoint.pt", weights_only=False)
    assert {"moe_layers", "global_step", "best_ppl", "optimizer_state_dict"} <= set(ck)
    assert "0.experts.w1" in ck["moe_layers"] and ck["global_step"] == 2
    # a file with the reference's keys only (no "model") restores the MoE layers
    only_moe = {k: ck[k] for k in ("moe_layers", "global_step", "best_ppl")}
    torch.save(only_moe, tmp_path / "ref_style.pt")
    before = wrapper.moe_layers["0"].experts.w1.detach().clone()
    with torch.no_grad():
        wrapper.moe_layers["0"].experts.w1.add_(1.0)
    assert fe.load_finetuned(wrapper, str(tmp_path / "ref_style.pt")) == 2
    assert torch.equal(wrapper.moe_layers["0"].experts.w1, before)


def test_routing_statistics_have_the_reference_keys_and_values():
    """Golden figures: the reference's ``compute_routing_stats`` on the same three count vectors
    (reference: Experiments/sparse_distillation/finetune_eval.py:67-209)."""
    from experiments.sparse_distillation import finetune_eval as fe

    class Layer(torch.nn.Module):
        def __init__(self, counts):
            super().__init__()
            self._last_expert_counts = torch.tensor(counts, dtype=torch.float)
            self.n_experts = len(counts)

    layers = torch.nn.ModuleDict({"0": Layer([10, 10, 0, 0]), "1": Layer([5, 5, 5, 5]), "2": Layer([97, 1, 1, 1])})
    r = fe.compute_routing_stats(layers, verbose=False)
    golden = {
        0: dict(total_tokens=20, entropy=0.6931471825, max_entropy=1.3862943611, normalized_entropy=0.5, min_frac=0.0,
                max_frac=0.5, imbalance_ratio=5e9, active_experts=2, meaningful_experts=2, collapsed=False),
        1: dict(total_tokens=20, entropy=1.3862943649, normalized_entropy=1.0, min_frac=0.25, max_frac=0.25,
                imbalance_ratio=1.0, active_experts=4, meaningful_experts=4, collapsed=False),
        2: dict(total_tokens=100, entropy=0.1677004993, normalized_entropy=0.1209703393, min_frac=0.01, max_frac=0.97,
                imbalance_ratio=97.0, active_experts=4, meaningful_experts=1, collapsed=True),
    }
    for i, want in golden.items():
        got = r["per_layer"][i]
        for k, v in want.items():
            assert got[k] == pytest.approx(v, rel=1e-5, abs=1e-7), (i, k, got[k], v)
    agg = r["aggregate"]
    assert agg["mean_normalized_entropy"] == pytest.approx(0.5403234478, rel=1e-5)
    assert agg["min_normalized_entropy"] == pytest.approx(0.1209703393, rel=1e-5)
    assert agg["mean_active_expert_frac"] == pytest.approx(10 / 12)
    assert agg["worst_min_frac"] == 0.0 and agg["worst_max_frac"] == pytest.approx(0.97)
    assert agg["collapsed_layers"] == [2] and agg["n_collapsed"] == 1


def test_the_guide_snippet_runs_as_written(tmp_path, monkeypatch):
    """The Python example of the package's user guide is executed verbatim (in a scratch directory)."""
    import os
    import re
    here = os.path.dirname(os.path.abspath(__file__))
    guide = os.path.join(here, "..", "experiments", "sparse_distillation", "README.md")
    code = re.search(r"```python\n(.*?)```", open(guide).read(), re.S).group(1)
    monkeypatch.chdir(tmp_path)
    torch.manual_seed(0)
    scope = {}
    exec(compile(code, "guide-snippet", "exec"), scope)
    assert scope["logits"].shape == (2, 16, 256)
    assert os.path.exists(tmp_path / "distilled.pt")
    assert set(scope["quality"]) == {0, 1} and set(scope["sparse"].count_parameters()) >= {"total", "active"}


def test_finetuning_auxiliary_losses_match_the_reference_figures():
    """Golden figures: the reference's ``compute_load_balancing_loss`` / ``compute_z_loss`` on the same seeded
    logits (reference: Experiments/sparse_distillation/finetune_eval.py:28-64)."""
    from experiments.sparse_distillation import finetune_eval as fe
    torch.manual_seed(0)
    golden = [(1.071408748626709, 12.736410140991211), (1.010005235671997, 10.339591979980469),
              (1.4494478702545166, 23.843008041381836)]
    for shape, (lb, z) in zip(((2, 16, 8), (64, 4), (3, 5, 16)), golden):
        lg = torch.randn(*shape) * 2
        E = shape[-1]
        cnt = torch.bincount(lg.reshape(-1, E).topk(2, -1).indices.reshape(-1), minlength=E).float()
        assert float(fe.compute_load_balancing_loss(lg, cnt)) == pytest.approx(lb, rel=1e-5)
        assert float(fe.compute_z_loss(lg)) == pytest.approx(z, rel=1e-5)
