"""The evaluation, analysis and diagnosis command lines run end to end on CPU on a tiny model."""
import json
import os
import sys

import pytest
import torch
import yaml

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


@pytest.fixture(scope="module")
def tiny(tmp_path_factory):
    """A small YAML config (same schema as configs/*.yaml) and a checkpoint of a model built from it."""
    d = tmp_path_factory.mktemp("tools")
    cfg = yaml.safe_load(open(os.path.join(ROOT, "configs", "test.yaml")))
    cfg["model"].update(d_model=64, d_ff=128, d_ff_expert=64, head_dim=16, n_heads=4, n_kv_heads=2,
                        max_seq_len=64, vocab_size=300, moe_layers=[1, 2, 3])
    cfg_path = str(d / "tiny.yaml")
    yaml.safe_dump(cfg, open(cfg_path, "w"))
    from kolmogorov_moe_architecture_b200 import MoETransformer
    from kolmogorov_moe_architecture_b200.utils.config_io import load_yaml, model_config_tolerant
    torch.manual_seed(0)
    model = MoETransformer(model_config_tolerant(load_yaml(cfg_path)), verbose=False)
    ck_path = str(d / "ck.pt")
    torch.save({"model_state_dict": model.state_dict(), "global_step": 3, "tokens_seen": 123}, ck_path)
    return {"dir": str(d), "config": cfg_path, "checkpoint": ck_path}


def test_evaluate_perplexity_synthetic(tiny):
    from eval import evaluate_perplexity as ev
    out = os.path.join(tiny["dir"], "results.md")
    ev.main(["--checkpoint", tiny["checkpoint"], "--config", tiny["config"], "--device", "cpu", "--synthetic",
             "--tokens", "2000", "--seq-len", "32", "--stride", "16", "--output", out])
    assert os.path.exists(out) and os.path.exists(out.replace(".md", ".json"))
    res = json.load(open(out.replace(".md", ".json")))
    text = json.dumps(res)
    assert "perplexity" in text
    # the layout of the reference's committed results: checkpoint / config / settings / results[dataset]
    assert {"checkpoint", "config", "settings", "results"} <= set(res)
    assert res["settings"] == {"tokens_per_dataset": 2000, "seq_len": 32, "stride": 16}
    assert {"perplexity", "loss"} <= set(res["results"]["synthetic"])
    md = open(out).read()
    assert "| Dataset | Perplexity | Loss | Tokens | Time (s) |" in md and "| **Average** |" in md
    ev.write_reports({"wikipedia": {"perplexity": float("nan"), "loss": float("nan"), "num_tokens": 0}},
                     {"checkpoint": "c.pt", "config": "c.yaml"}, out)
    assert "| wikipedia | N/A | N/A | - | - | *Could not load data* |" in open(out).read()
    # strided windows cover the stream with the requested overlap
    w = ev.windows(list(range(100)), 32, 16)
    assert all(len(x) == 32 for x in w) and w[1][0] == 16


def test_diagnose_training_reports_every_section(tiny):
    from tools import diagnose_training as dt
    rep = dt.main(["--checkpoint", tiny["checkpoint"], "--config", tiny["config"], "--device", "cpu", "--synthetic",
                   "--eval-batches", "2"])
    quick = dt.main(["--checkpoint", tiny["checkpoint"], "--config", tiny["config"], "--device", "cpu", "--gpu", "0",
                     "--skip-eval", "--skip-generation"])
    assert "evaluation" not in quick and "gradients" in quick
    assert set(rep) >= {"router", "routing_in_model", "movement", "trainability", "evaluation", "gradients", "findings"}
    assert rep["trainability"]["trainable"] == rep["trainability"]["total"]
    assert abs(rep["evaluation"]["lm_loss"] - rep["evaluation"]["uniform_loss"]) < 1.0   # untrained model
    assert rep["routing_in_model"] and all(0.0 <= s["gini"] <= 1.0 for s in rep["routing_in_model"].values())
    # the checkpoint is the seed-0 initialisation itself: nothing has moved
    assert max(rep["movement"].values()) < 1e-6
    assert any("did not move" in line for line in rep["findings"])
    assert dt.calculate_gini([1, 1, 1, 1]) == 0.0 and dt.calculate_gini([0, 0, 0, 8]) == 0.75


def test_reallocate_experts_copies_w123_and_resets_routers(tiny):
    """A layer whose router has collapsed gets its experts from a healthy layer (the stacked w1/w2/w3 tensors
    are what is copied) and every router is re-initialised; the optimizer state is dropped."""
    from tools import reallocate_experts as re_
    from eval.evaluate_perplexity import load_model
    model, _ = load_model(tiny["checkpoint"], tiny["config"], "cpu", dtype=torch.float32)
    moe_layers = [i for i, l in enumerate(model.layers) if hasattr(l.ffn, "grouped_experts")]
    assert len(moe_layers) >= 2
    sick = model.layers[moe_layers[0]].ffn
    with torch.no_grad():                                      # collapse: every token prefers expert 0
        last = sick.router.router[2].weight
        last.zero_()
        last[0].fill_(5.0)
        sick.router.router[0].weight.normal_(0.0, 1.0)       # large hidden activations: silu ~ relu >= 0
    bad_ck = os.path.join(tiny["dir"], "collapsed.pt")
    torch.save({"model_state_dict": model.state_dict(), "optimizer_state_dict": {"x": 1}}, bad_ck)
    out = os.path.join(tiny["dir"], "reallocated.pt")
    info = re_.reallocate_experts(bad_ck, tiny["config"], out, "cpu")
    assert moe_layers[0] in info["collapsed"] and info["source"] in info["healthy"]
    ck = torch.load(out, map_location="cpu", weights_only=False)
    assert "optimizer_state_dict" not in ck
    sd = ck["model_state_dict"]
    a, b = f"layers.{moe_layers[0]}.ffn.grouped_experts.w1", f"layers.{info['source']}.ffn.grouped_experts.w1"
    assert torch.equal(sd[a], sd[b])
    assert not torch.equal(sd[f"layers.{moe_layers[0]}.ffn.router.router.2.weight"], last)


def test_param_calculator_matches_the_model(tiny):
    from tools import param_calculator as pc
    from kolmogorov_moe_architecture_b200 import MoETransformer
    from kolmogorov_moe_architecture_b200.utils.config_io import load_yaml, model_config_tolerant
    cfg = model_config_tolerant(load_yaml(tiny["config"]))
    r = pc.analyze(cfg, world=2)
    n = sum(p.numel() for p in MoETransformer(cfg, verbose=False).parameters())
    total = next(v for k, v in r.items() if "total" in k and isinstance(v, (int, float)))
    assert abs(total - n) <= 0.02 * n, (total, n)
    rep = pc.print_report(cfg, world=2)
    b = rep["breakdown"]
    assert b["total"] == n and b["experts"] > 0 and b["mamba"] > 0 and b["mod_router"] > 0 and "other" not in b
    assert pc.format_params(5.87e9) == "5.87B" and pc.format_params(1500) == "1.50K"
    found = pc.design(5e9, 1.5e9, tol=0.3, limit=3)
    assert isinstance(found, list)
    # the reference's manual options: experts in every layer, totals equal to the instantiated model
    rep = pc.main(["--vocab-size", "1000", "--d-model", "256", "--n-layers", "4", "--n-heads", "2", "--n-kv-heads", "1",
                   "--head-dim", "128", "--d-ff", "512", "--d-ff-expert", "256", "--n-experts", "4", "--top-k", "2",
                   "--all-moe", "--world", "2"])
    bd = rep["breakdown"]
    assert bd["experts"] == 4 * 4 * 3 * 256 * 256 and bd["dense_ffn"] == 0 and bd["mamba"] == 0 and bd["mod_router"] == 0
    assert bd["embedding"] == 1000 * 256
    assert isinstance(pc.main(["--design", "--target-total", "5", "--target-active", "1.5"]), list)


def test_plateau_memory_debug_and_active_param_tools(tiny, capsys):
    import analyze_active_params
    import check_memory
    import debug_training
    import diagnose_memory
    import diagnose_plateau
    rep = diagnose_plateau.main(["--config", tiny["config"], "--checkpoint", tiny["checkpoint"], "--device", "cpu",
                                 "--batches", "2", "--batch-size", "1", "--seq-len", "16"])
    assert rep, "router hooks recorded nothing"
    rows = check_memory.main(["--config", tiny["config"], "--seq-len", "32"])
    assert [r[0] for r in rows][:2] == ["start", "model"] and len(rows) >= 6
    rep = diagnose_memory.main([tiny["config"], "--seq-len", "32", "--steps", "6", "--accum", "2"])
    assert rep["opt_steps"] == 3 and rep["leak"] is False
    assert diagnose_memory.growth_per_step([1.0, 2.0, 2.5, 3.0, 3.5]) == pytest.approx(0.5)
    info = debug_training.inspect(tiny["checkpoint"], top=3)
    assert info["non_finite"] == [] and info["n_tensors"] > 10 and info["meta"]["global_step"] == 3
    analyze_active_params.main(["--preset", "test"])
    assert "active" in capsys.readouterr().out.lower()


def test_expert_choice_scatter_benchmark_variants_agree():
    from tools import benchmark_expert_choice as bec
    torch.manual_seed(0)
    B, E, C, S, d = 2, 3, 4, 10, 8
    w_out = torch.randn(B, E, C, d)
    idx = torch.randint(0, S, (B, E, C))
    a = bec.scatter_loop(torch.zeros(B, S, d), w_out, idx)
    b = bec.scatter_vectorised(torch.zeros(B, S, d), w_out, idx)
    assert torch.allclose(a, b, atol=1e-6)
    times = bec.main(["--device", "cpu", "--batch-size", "2", "--seq-len", "64", "--d-model", "32", "--n-experts", "4",
                      "--capacity-factor", "1.25", "--warmup", "1", "--iters", "3"])
    assert set(times) == {"loop", "scatter_add"} and all(t > 0 for t in times.values())


def test_bench_clock_sampler_parses_nvidia_smi_lines_and_flags():
    """The benchmark's clock record: median SM clock under load, maximum clock, and the throttle reasons that
    were active in any sample; the argument defaults are the contract's (1 GPU, >= 3 warm-up steps)."""
    import bench
    s = bench.ClockSampler(0)
    s.proc = type("P", (), {"terminate": lambda self: None})()
    s.lines = ["0, 1965, 1965, 950.1, 0x0000000000000004, Not Active, Not Active, Not Active, Active",
               "0, 1890, 1965, 990.0, 0x0000000000000004, Not Active, Not Active, Not Active, Active",
               "0, 1920, 1965, 980.0, 0x0000000000000000, Not Active, Not Active, Not Active, Not Active",
               "garbage line", "0, [N/A], 1965, 1, 0, Not Active, Not Active, Not Active, Not Active"]
    out = s.stop()
    assert out == {"sm_mhz": 1920.0, "sm_max_mhz": 1965.0, "samples": 3, "reasons": ["sw_power_cap"]}
    s.lines = ["0, 1200, 1965, 500, 0x8, Active, Active, Not Active, Not Active"]
    assert s.stop()["reasons"] == ["hw_slowdown", "hw_thermal_slowdown"]
    none = bench.ClockSampler(0).stop()
    assert none["sm_mhz"] is None
    import sys
    argv, sys.argv = sys.argv, ["bench.py"]
    try:
        a = bench.parse_args()
    finally:
        sys.argv = argv
    assert (a.gpus, a.impl, a.micro_batch, a.seq_len, a.layers) == (1, "ours", 4, 2048, 32) and a.warmup >= 3


def test_every_shipped_config_builds_a_model_on_the_meta_device():
    """All YAML files under configs/ (the Accelerate launcher file aside) go through both loaders and describe
    a model that can be instantiated; every one has the training sections the entry points read."""
    import glob
    from kolmogorov_moe_architecture_b200 import MoETransformer
    from kolmogorov_moe_architecture_b200.utils.config_io import load_yaml, model_config_tolerant, section
    paths = sorted(p for p in glob.glob(os.path.join(ROOT, "configs", "*.yaml")) if not p.endswith("fsdp_config.yaml"))
    assert len(paths) >= 18
    for p in paths:
        y = load_yaml(p)
        cfg = model_config_tolerant(y)
        with torch.device("meta"):
            m = MoETransformer(cfg, verbose=False)
        c = m.count_parameters()
        assert c["total"] > 0 and 0 < c["active"] <= c["total"], p
        tr = section(y, "training")
        assert {"batch_size", "gradient_accumulation_steps", "max_lr", "warmup_steps"} <= set(tr), p
        assert section(y, "optimizer").get("type", "adamw") in ("muon", "adamw", "adam"), p
    big = model_config_tolerant(load_yaml(os.path.join(ROOT, "configs", "bench_5b_hybrid.yaml")))
    with torch.device("meta"):
        n = sum(p.numel() for p in MoETransformer(big, verbose=False).parameters())
    assert abs(n - 5.87e9) < 0.01e9
    acc = yaml.safe_load(open(os.path.join(ROOT, "configs", "fsdp_config.yaml")))
    assert acc["distributed_type"] == "FSDP" and acc["fsdp_config"]["fsdp_sharding_strategy"] == "FULL_SHARD"


def test_hf_entrypoint_fsdp_settings():
    """The shipped Accelerate-style FSDP file is consumed: a torchrun launch asks the HF Trainer for FULL_SHARD
    over the transformer blocks, an Accelerate launch leaves FSDP to Accelerate, one process needs nothing."""
    import train_production as tp
    path = os.path.join(ROOT, "configs", "fsdp_config.yaml")
    one = tp.fsdp_settings(path, env={})
    assert one["distributed"] is False and one["hf_kwargs"] == {}
    tr = tp.fsdp_settings(path, env={"WORLD_SIZE": "2"})
    assert tr["distributed"] and tr["hf_kwargs"]["fsdp"] == "full_shard auto_wrap"
    assert tr["hf_kwargs"]["fsdp_config"]["transformer_layer_cls_to_wrap"] == ["TransformerBlock"]
    assert tr["hf_kwargs"]["fsdp_config"]["backward_prefetch"] == "backward_pre" and tr["cpu_offload"] is False
    acc = tp.fsdp_settings(path, env={"WORLD_SIZE": "2", "ACCELERATE_USE_FSDP": "true"})
    assert acc["accelerate_owns_fsdp"] and acc["hf_kwargs"] == {}
    assert tr["sharding_strategy"] == "full_shard" and tr["sharded_state_dict"]
    assert tr["hf_kwargs"]["fsdp_config"]["state_dict_type"] == "SHARDED_STATE_DICT"
    # other strategies, wrap policies and offload in the file change the request accordingly
    import tempfile
    import yaml
    with tempfile.NamedTemporaryFile("w", suffix=".yaml", delete=False) as f:
        yaml.safe_dump({"fsdp_config": {"fsdp_sharding_strategy": "SHARD_GRAD_OP", "fsdp_auto_wrap_policy": "SIZE_BASED_WRAP",
                                        "fsdp_min_num_params": 5000, "fsdp_offload_params": True,
                                        "fsdp_state_dict_type": "FULL_STATE_DICT"}}, f)
    alt = tp.fsdp_settings(f.name, env={"WORLD_SIZE": "4"})
    os.unlink(f.name)
    assert alt["hf_kwargs"]["fsdp"] == "shard_grad_op auto_wrap offload" and alt["cpu_offload"]
    assert alt["hf_kwargs"]["fsdp_config"]["min_num_params"] == 5000 and not alt["sharded_state_dict"]
    assert "transformer_layer_cls_to_wrap" not in alt["hf_kwargs"]["fsdp_config"]


def test_tools_expose_the_reference_helper_names(tiny, capsys):
    """Helper functions that the reference's tools define at module level exist here under the same names and do
    the same job."""
    import analyze_active_params
    import check_memory
    import debug_training
    import diagnose_memory
    import diagnose_plateau
    from eval import evaluate_perplexity as ev
    from tools import benchmark_expert_choice as bec, diagnose_training as dt, param_calculator as pc, reallocate_experts as re_
    raw = diagnose_plateau.load_config(tiny["config"])
    assert raw == ev.load_config(tiny["config"]) == check_memory.load_config(tiny["config"]) == diagnose_memory.load_config(tiny["config"])
    model, cfg = diagnose_plateau.create_model_from_config(raw)
    assert cfg.d_model == raw["model"]["d_model"] and re_.create_model_config(raw).d_model == cfg.d_model
    assert dt.create_model_config(raw).n_layers == cfg.n_layers
    an = diagnose_plateau.RouterAnalyzer(model)
    assert an.register_hooks() is an
    ids = torch.randint(0, cfg.vocab_size, (2, 16))
    model.train()
    model(ids, labels=ids, return_logits=False)["loss"].backward()
    assert an.get_stats() and diagnose_plateau.analyze_gradients(model)
    an.remove_hooks()
    assert check_memory.print_memory(3, "after forward")[0] == "3:after forward"
    assert diagnose_memory.get_mem() == (0.0, 0.0) and diagnose_memory.print_mem("x", 0.0) == 0.0
    assert debug_training.analyze_checkpoint(tiny["checkpoint"])["non_finite"] == []
    c = analyze_active_params.analyze_config(cfg, "tiny")
    assert c["total"] == sum(p.numel() for p in model.parameters())
    loaded, lcfg = ev.load_model_from_checkpoint(tiny["checkpoint"], tiny["config"], "cpu")
    assert not loaded.training and lcfg.d_model == cfg.d_model
    trained, tcfg = dt.load_checkpoint(tiny["checkpoint"], tiny["config"], "cpu")
    fresh = dt.create_fresh_model(tcfg, "cpu")
    mv = dt.analyze_parameter_movement(trained, fresh)
    assert mv and max(mv.values()) < 1e-6                       # the checkpoint is the seed-0 initialisation
    with torch.no_grad():
        next(trained.parameters()).add_(1.0)
    assert max(dt.analyze_parameter_movement(trained, fresh).values()) > 0.1
    assert dt.analyze_trainability(trained)["trainable"] == dt.analyze_trainability(trained)["total"]
    assert len(dt.test_generation(trained, tcfg, "cpu", prompt_len=4, new_tokens=3)) == 7
    assert dt.check_gradient_flow(trained, tcfg, "cpu")
    # the plain attention + MoE calculator against a model of that shape
    mp = pc.ModelParams(vocab_size=500, d_model=64, n_layers=4, n_heads=2, n_kv_heads=1, head_dim=32, d_ff=128,
                        d_ff_expert=64, n_experts=4, moe_top_k=2, moe_layers=[1, 3], tie_embeddings=True)
    r = pc.calculate_params(mp)
    import kolmogorov_moe_architecture_b200 as kmoe
    twin = kmoe.MoETransformer(kmoe.AdvancedMoEConfig(
        vocab_size=500, d_model=64, n_layers=4, n_heads=2, n_kv_heads=1, head_dim=32, d_ff=128, d_ff_expert=64,
        n_experts=4, moe_top_k=2, moe_layers=(1, 3), mamba_enabled=False, mamba_layers=(), mod_enabled=False,
        n_pred_tokens=1, aux_loss_weights=(1.0,), max_seq_len=16), verbose=False)
    assert r["total_params"] == sum(p.numel() for p in twin.parameters())
    assert r["n_moe_layers"] == 2 and r["active_params"] == r["total_params"] - r["expert_params"] / 2
    assert pc.print_report(r, mp) is r
    assert pc.load_config(tiny["config"]).d_model == cfg.d_model
    best = pc.design_model(0.1, 0.05, vocab_size=32000)
    assert best is None or isinstance(best, pc.ModelParams)
    assert bec.original_scatter_add is bec.scatter_loop and bec.vectorized_scatter_add is bec.scatter_vectorised
    w, idx = torch.randn(1, 2, 3, 4), torch.tensor([[[0, 1, 2], [2, 3, 4]]])
    assert bec.benchmark_fn(bec.vectorized_scatter_add, torch.zeros(1, 6, 4), w, idx, warmup=1, iters=2) > 0
    capsys.readouterr()
