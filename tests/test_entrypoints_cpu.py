"""Every training entry point runs a few steps on CPU from a YAML config, writes the checkpoint layout its
counterpart in the reference writes, and resumes from it."""
import os
import subprocess
import sys

import pytest
import torch
import yaml

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)


@pytest.fixture(scope="module")
def tiny_cfg(tmp_path_factory):
    d = tmp_path_factory.mktemp("entry")
    cfg = yaml.safe_load(open(os.path.join(ROOT, "configs", "test.yaml")))
    cfg["model"].update(d_model=64, d_ff=128, d_ff_expert=64, head_dim=16, n_heads=4, n_kv_heads=2,
                        max_seq_len=32, vocab_size=300)
    cfg["training"].update(checkpoint_dir=str(d / "from_yaml"), save_interval=2, log_interval=1,
                           gradient_accumulation_steps=1, batch_size=2)
    path = str(d / "tiny.yaml")
    yaml.safe_dump(cfg, open(path, "w"))
    return {"dir": str(d), "config": path}


def test_train_py_format_b_checkpoints_and_resume(tiny_cfg):
    import train
    ck = os.path.join(tiny_cfg["dir"], "b")
    out = train.main(["--config", tiny_cfg["config"], "--steps", "4", "--batch-size", "2", "--seq-len", "32",
                      "--grad-accum", "1", "--synthetic", "--checkpoint-dir", ck, "--save-interval", "2"])
    assert out["steps"] == 4 and out["final_loss"] is not None
    files = sorted(os.listdir(os.path.join(ck, "tiny")))
    assert files == ["checkpoint-2.pt", "checkpoint-4-final.pt"]
    sd = torch.load(os.path.join(ck, "tiny", "checkpoint-2.pt"), map_location="cpu", weights_only=False)
    assert {"step", "model_state_dict", "optimizer_state_dict", "total_tokens", "config_path"} <= set(sd)
    assert isinstance(sd["optimizer_state_dict"], list) and len(sd["optimizer_state_dict"]) == 2   # Muon + AdamW
    out2 = train.main(["--config", tiny_cfg["config"], "--steps", "5", "--batch-size", "2", "--seq-len", "32",
                       "--grad-accum", "1", "--synthetic", "--checkpoint-dir", ck, "--save-interval", "0",
                       "--resume", os.path.join(ck, "tiny", "checkpoint-2.pt")])
    assert out2["steps"] == 5


def test_train_custom_format_c_and_scripts_train_format_a(tiny_cfg):
    import train_custom
    ck = os.path.join(tiny_cfg["dir"], "c")
    out = train_custom.main(["--config", tiny_cfg["config"], "--steps", "4", "--batch-size", "2", "--synthetic",
                             "--checkpoint-dir", ck])
    assert out["steps"] == 4
    dirs = sorted(n for n in os.listdir(ck) if n.startswith("checkpoint-"))
    assert dirs and set(os.listdir(os.path.join(ck, dirs[-1]))) >= {"model.pt", "optimizer.pt", "training_state.pt"}
    out = train_custom.main(["--config", tiny_cfg["config"], "--steps", "5", "--batch-size", "2", "--synthetic",
                             "--checkpoint-dir", ck, "--resume", os.path.join(ck, dirs[-1])])
    assert out["steps"] == 5
    sys.path.insert(0, os.path.join(ROOT, "scripts"))
    import importlib.util
    spec = importlib.util.spec_from_file_location("scripts_train", os.path.join(ROOT, "scripts", "train.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    mod.main(["--config", tiny_cfg["config"], "--max_steps", "3", "--device", "cpu", "--synthetic"])


def test_train_production_native_fallback(tiny_cfg):
    import train_production
    out = train_production.main(["--config", tiny_cfg["config"], "--max_steps", "3", "--synthetic",
                                 "--output_dir", os.path.join(tiny_cfg["dir"], "hf")])
    assert out is None or out.get("steps", 3) == 3


def _torchrun(args, port):
    env = dict(os.environ, PYTHONPATH=ROOT, KMOE_OFFLINE="1")
    r = subprocess.run([sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node=2",
                        "--master-addr", "127.0.0.1", "--master-port", str(port),
                        os.path.join(ROOT, "train_distributed.py")] + args,
                       env=env, capture_output=True, text=True, timeout=900, cwd=ROOT)
    assert r.returncode == 0, r.stdout[-2000:] + r.stderr[-3000:]
    return r.stdout


@pytest.mark.parametrize("sharded", [False, True])
def test_train_distributed_two_ranks_background_checkpoints_and_resume(tiny_cfg, sharded):
    """Two gloo ranks: replicated-parameter plan and parameter-sharded plan, checkpoints written in the
    background with completion markers, then a second launch that resumes from the checkpoint root."""
    ck = os.path.join(tiny_cfg["dir"], "dist_sharded" if sharded else "dist")
    extra = ["--shard-params"] if sharded else []
    out = _torchrun(["--config", tiny_cfg["config"], "--steps", "4", "--synthetic", "--checkpoint-dir", ck,
                     "--async-checkpoint"] + extra, 29711 + int(sharded))
    assert "Step 4/4" in out
    from kolmogorov_moe_architecture_b200.training import checkpoint as ckpt
    last = ckpt.latest_complete_checkpoint(ck, world=2)
    assert last is not None and last.endswith("checkpoint-4")
    names = set(os.listdir(last))
    per_rank = "shards-rank{}.pt" if sharded else "optimizer-rank{}.pt"
    assert {"model.pt", "training_state.pt", "complete-rank0", "complete-rank1",
            per_rank.format(0), per_rank.format(1)} <= names
    out = _torchrun(["--config", tiny_cfg["config"], "--steps", "6", "--synthetic", "--checkpoint-dir", ck,
                     "--resume", ck] + extra, 29713 + int(sharded))
    assert "Step 5/6" in out and "Step 4/6" not in out


def test_expert_parallel_checkpoint_keeps_every_ranks_experts(tiny_cfg):
    """Experts split over two ranks: each rank's experts and their optimizer state go to its own file, the
    job resumes from them, and the directory consolidates into one state dict for a model with all experts
    on one rank."""
    cfg = yaml.safe_load(open(tiny_cfg["config"]))
    cfg["model"].update(moe_implementation="expert_parallel", ep_size=2, moe_layers=[1, 2, 3])
    path = os.path.join(tiny_cfg["dir"], "tiny_ep.yaml")
    yaml.safe_dump(cfg, open(path, "w"))
    ck = os.path.join(tiny_cfg["dir"], "dist_ep")
    _torchrun(["--config", path, "--steps", "4", "--synthetic", "--checkpoint-dir", ck, "--async-checkpoint"], 29715)
    from kolmogorov_moe_architecture_b200.training import checkpoint as ckpt
    last = ckpt.latest_complete_checkpoint(ck, world=2)
    assert {"experts-rank0.pt", "experts-rank1.pt", "model.pt"} <= set(os.listdir(last))
    e0 = torch.load(os.path.join(last, "experts-rank0.pt"), weights_only=False)
    e1 = torch.load(os.path.join(last, "experts-rank1.pt"), weights_only=False)
    assert (e0["ep_rank"], e1["ep_rank"], e0["ep_size"]) == (0, 1, 2) and e0["optimizer"] is not None
    name = next(iter(e0["params"]))
    assert "local_experts" in name and not torch.equal(e0["params"][name], e1["params"][name])
    model_sd = torch.load(os.path.join(last, "model.pt"), weights_only=False)
    assert not any("local_experts" in k for k in model_sd)
    full = ckpt.consolidate_expert_checkpoint(last)
    assert full[name].shape[0] == 2 * e0["params"][name].shape[0]
    assert torch.equal(full[name][: e0["params"][name].shape[0]], e0["params"][name])
    # a single-process model with all experts local loads the consolidated state
    import kolmogorov_moe_architecture_b200 as kmoe
    from kolmogorov_moe_architecture_b200.utils.config_io import load_yaml, model_config_tolerant
    y = load_yaml(path)
    y["model"]["ep_size"] = 1
    one = kmoe.MoETransformer(model_config_tolerant(y), verbose=False)
    missing, unexpected = one.load_state_dict(full, strict=False)
    assert not unexpected and not [k for k in missing if "local_experts" in k]
    out = _torchrun(["--config", path, "--steps", "6", "--synthetic", "--checkpoint-dir", ck, "--resume", ck], 29716)
    assert "Step 5/6" in out and "Step 4/6" not in out
    # the same split of the experts under the parameter-sharded plan for the dense parameters
    ck2 = os.path.join(tiny_cfg["dir"], "dist_ep_sharded")
    _torchrun(["--config", path, "--steps", "4", "--synthetic", "--checkpoint-dir", ck2, "--shard-params"], 29717)
    last = ckpt.latest_complete_checkpoint(ck2, world=2)
    assert {"experts-rank0.pt", "experts-rank1.pt", "shards-rank0.pt", "shards-rank1.pt", "model.pt"} <= set(os.listdir(last))


def test_elastic_launcher_restarts_from_the_newest_complete_checkpoint(tiny_cfg, monkeypatch):
    """Rank 1 exits on the host after step 3 (once); the launcher starts the job again, which resumes from
    checkpoint-2 and runs to the end.  A second scenario shrinks to one process after two failures."""
    import elastic_launch
    ck = os.path.join(tiny_cfg["dir"], "elastic")
    marker = os.path.join(tiny_cfg["dir"], "failed_once")
    env = dict(os.environ, PYTHONPATH=ROOT, KMOE_OFFLINE="1", KMOE_FAULT_INJECT="1:3:exit", KMOE_FAULT_ONCE=marker)
    lines = []
    rc = elastic_launch.supervise(2, ["train_distributed.py", "--config", tiny_cfg["config"], "--steps", "6",
                                      "--synthetic"], ck, max_restarts=2, port=29741, env=env, log=lines.append)
    assert rc == 0, lines
    assert os.path.exists(marker)
    assert any("starting fresh" in l for l in lines) and any("resuming from checkpoint-2" in l for l in lines)
    assert any("finished after 1 restart" in l for l in lines)
    from kolmogorov_moe_architecture_b200.training import checkpoint as ckpt
    assert ckpt.latest_complete_checkpoint(ck, world=2).endswith("checkpoint-6")
    # a rank that fails every time: two failures at two processes, then one process finishes the job
    # (the launches are replaced by a stub: what is checked is the launcher's own bookkeeping)
    calls, codes = [], iter([17, 17, 0])

    def fake_call(cmd, env=None, cwd=None):
        calls.append(cmd)
        return next(codes)

    monkeypatch.setattr(elastic_launch.subprocess, "call", fake_call)
    lines = []
    rc = elastic_launch.supervise(2, ["train_distributed.py", "--steps", "6"], ck, max_restarts=3, port=29751,
                                  shrink=True, log=lines.append, backoff_s=0.0)
    assert rc == 0 and any("continuing with 1 processes" in l for l in lines)
    assert [c[4] for c in calls] == ["--nproc-per-node=2", "--nproc-per-node=2", "--nproc-per-node=1"]
    assert all(c[-2:] == ["--resume", ck] for c in calls)                   # the finished run left checkpoints there
    codes = iter([3, 3])
    assert elastic_launch.supervise(2, ["t.py"], ck, max_restarts=1, log=lines.append, backoff_s=0.0) == 3
    cmd = elastic_launch.build_command(4, 29500, ["t.py", "--resume", "old", "--checkpoint-dir=x", "--steps", "3"], "ck", "ck")
    assert cmd[-4:] == ["--checkpoint-dir", "ck", "--resume", "ck"] and "old" not in cmd and "--steps" in cmd


def _records(path):
    import json
    return {r["step"]: r for r in map(json.loads, open(path)) if "loss" in r}


@pytest.mark.parametrize("fmt", ["B", "C"])
def test_resume_continues_schedule_and_data(tiny_cfg, fmt):
    """After a resume the learning rate and the loss of the next steps equal those of the run that was
    never interrupted: the schedule continues at the saved step and the consumed batches are not replayed."""
    from kolmogorov_moe_architecture_b200.training.runner import RunSpec, run_training
    base = os.path.join(tiny_cfg["dir"], f"resume_{fmt}")
    common = dict(config_path=tiny_cfg["config"], steps=6, batch_size=2, data_mode="synthetic",
                  checkpoint_format=fmt, save_interval=3, optimizer_family="adamw")
    run_training(RunSpec(checkpoint_dir=os.path.join(base, "a"), jsonl=os.path.join(base, "a.jsonl"), **common))
    cdir = os.path.join(base, "a") if fmt == "C" else os.path.join(base, "a", "tiny")
    ck = os.path.join(cdir, "checkpoint-3" if fmt == "C" else "checkpoint-3.pt")
    assert os.path.exists(ck)
    run_training(RunSpec(checkpoint_dir=os.path.join(base, "b"), jsonl=os.path.join(base, "b.jsonl"), resume=ck,
                         **common))
    full, tail = _records(os.path.join(base, "a.jsonl")), _records(os.path.join(base, "b.jsonl"))
    assert sorted(tail) == [4, 5, 6]
    lrs = [full[s]["lr"] for s in range(1, 7)]
    assert len(set(lrs)) == 6, "the warm-up should move the rate at every step of this run"
    for s in (4, 5, 6):
        assert tail[s]["lr"] == pytest.approx(full[s]["lr"], rel=1e-12), (s, tail[s]["lr"], full[s]["lr"])
        assert tail[s]["loss"] == pytest.approx(full[s]["loss"], rel=1e-5), (s, tail[s]["loss"], full[s]["loss"])
    saved = torch.load(ck if fmt == "B" else os.path.join(ck, "training_state.pt"), map_location="cpu",
                       weights_only=False)
    assert saved["data_idx"] == 3


def test_checkpoint_completeness_rules(tmp_path):
    """A directory is a checkpoint only when every writer named in rank 0's manifest has finished."""
    from kolmogorov_moe_architecture_b200.training import checkpoint as ck
    d = tmp_path / "checkpoint-5"
    d.mkdir()
    # rank 0 has written its state, no rank has dropped a marker yet (killed in that window)
    ck._write_manifest(str(d), "sharded", 2, ck._expected_files("optimizer", 2, False))
    for n in ("model.pt", "training_state.pt", "optimizer-rank0.pt"):
        (d / n).write_bytes(b"x")
    assert not ck.checkpoint_complete(str(d), 2)
    ck._mark_complete(str(d), 0)
    assert not ck.checkpoint_complete(str(d), 2)            # rank 1 still writing
    (d / "optimizer-rank1.pt").write_bytes(b"x")
    ck._mark_complete(str(d), 1)
    assert ck.checkpoint_complete(str(d), 2)
    assert ck.checkpoint_complete(str(d), 1)                # a smaller job recognises it too
    # per-rank files without a manifest: rank 0 has not begun
    e = tmp_path / "checkpoint-7"
    e.mkdir()
    (e / "optimizer-rank1.pt").write_bytes(b"x")
    (e / "training_state.pt").write_bytes(b"x")
    assert not ck.checkpoint_complete(str(e), 2)
    # single-writer layout (format C)
    f = tmp_path / "checkpoint-9"
    f.mkdir()
    (f / "model.pt").write_bytes(b"x")
    assert not ck.checkpoint_complete(str(f), 1)
    (f / "training_state.pt").write_bytes(b"x")
    assert ck.checkpoint_complete(str(f), 1)
    assert ck.latest_complete_checkpoint(str(tmp_path), 2).endswith("checkpoint-9")
    # pruning never deletes on the strength of an unfinished directory
    ck.prune_checkpoints(str(tmp_path), keep=1, world=2)
    assert sorted(os.listdir(tmp_path)) == ["checkpoint-7", "checkpoint-9"]


def test_missing_optimizer_shard_is_an_error_at_the_same_world_size(tmp_path):
    from kolmogorov_moe_architecture_b200.training import checkpoint as ck

    class Pool:
        world = 2
        def load_optimizer_state_dict(self, sd):
            raise AssertionError("not reached")

    model = torch.nn.Linear(4, 4)
    d = tmp_path / "checkpoint-1"
    d.mkdir()
    torch.save(model.state_dict(), d / "model.pt")
    torch.save({"step": 1}, d / "training_state.pt")
    ck._write_manifest(str(d), "sharded", 2, ck._expected_files("optimizer", 2, False))
    with pytest.raises(FileNotFoundError, match="optimizer state of rank 1"):
        ck.load_sharded(str(d), model, Pool(), rank=1)
    # written by a job of another size: parameters carry over, moments start fresh
    ck._write_manifest(str(d), "sharded", 4, ck._expected_files("optimizer", 4, False))
    assert ck.load_sharded(str(d), model, Pool(), rank=1)["step"] == 1


def test_elastic_launcher_environment_and_shrink_refusal(tmp_path, monkeypatch):
    import elastic_launch
    from kolmogorov_moe_architecture_b200.training.runner import fault_injection_refusal
    seen = {}

    def fake_call(cmd, env=None, cwd=None):
        seen.setdefault("envs", []).append(dict(env))
        seen.setdefault("cmds", []).append(cmd)
        return 1
    monkeypatch.setattr(elastic_launch.subprocess, "call", fake_call)
    d = tmp_path / "ck" / "checkpoint-2"
    d.mkdir(parents=True)
    (d / "experts-rank0.pt").write_bytes(b"x")
    logs = []
    rc = elastic_launch.supervise(4, ["train_distributed.py"], str(tmp_path / "ck"), max_restarts=3, shrink=True,
                                  backoff_s=0.0, env={}, log=logs.append)
    assert rc == 1
    env = seen["envs"][0]
    assert env["NCCL_NVLS_ENABLE"] == "0" and env["KMOE_MULTIMEM"] == "0"
    assert env["TORCH_SYMM_MEM_DISABLE_MULTICAST"] == "1"
    assert all("--nproc-per-node=4" in c for c in seen["cmds"]), "expert-parallel checkpoints keep the job size"
    assert any("--shrink refused" in m for m in logs)
    # the injector's own guard
    assert "NCCL_NVLS_ENABLE" in fault_injection_refusal({}, None)
    assert "TORCH_SYMM_MEM_DISABLE_MULTICAST" in fault_injection_refusal({"NCCL_NVLS_ENABLE": "0"}, "p2p")
    assert fault_injection_refusal({"NCCL_NVLS_ENABLE": "0"}, "nccl") is None
    assert fault_injection_refusal({"NCCL_NVLS_ENABLE": "0", "TORCH_SYMM_MEM_DISABLE_MULTICAST": "1"}, None) is None


def test_debug_mode_profile_phases_and_token_weighting(tiny_cfg, capsys):
    """``--debug`` prints the gradient-flow table (every category got gradients) and the router / stuck-norm
    line; ``--profile`` reports forward / backward / optimizer next to data / step; token weighting changes
    the loss that is optimised."""
    from kolmogorov_moe_architecture_b200.training.runner import RunSpec, run_training
    base = os.path.join(tiny_cfg["dir"], "dbg")
    common = dict(config_path=tiny_cfg["config"], steps=3, batch_size=2, data_mode="synthetic", checkpoint_format="C",
                  save_interval=0, optimizer_family="adamw")
    run_training(RunSpec(checkpoint_dir=os.path.join(base, "a"), jsonl=os.path.join(base, "a.jsonl"), debug=True,
                         debug_interval=2, profile=True, use_8bit_optimizer=True, compile=True, **common))
    out = capsys.readouterr().out
    assert "Gradient flow summary (aggregated across 1 ranks)" in out
    assert "All parameters received gradients!" in out and "MISSING" not in out
    for group in ("attention", "expert_weights", "moe_router", "mod_router", "lm_head", "norms", "embeddings"):
        assert f"  {group}" in out, group
    assert "[debug step 2] router:" in out and "norm weights still at their initial value" in out
    assert "bitsandbytes not available, falling back to standard AdamW" in out or "Using 8-bit AdamW" in out
    assert "--compile: accepted" in out
    rec = _records(os.path.join(base, "a.jsonl"))[3]
    for k in ("time_data_ms", "time_step_ms", "time_forward_ms", "time_backward_ms", "time_optimizer_ms"):
        assert rec[k] >= 0.0, k
    run_training(RunSpec(checkpoint_dir=os.path.join(base, "b"), jsonl=os.path.join(base, "b.jsonl"),
                         token_weight_decay=2.0, **common))
    plain, weighted = _records(os.path.join(base, "a.jsonl")), _records(os.path.join(base, "b.jsonl"))
    assert weighted[1]["loss"] != pytest.approx(plain[1]["loss"], rel=1e-6)
    assert abs(weighted[1]["loss"] - plain[1]["lm_loss"]) < 1.0      # still a next-token loss near ln(vocab)


def test_script_level_helpers_of_the_reference_work_on_this_framework(tmp_path, monkeypatch):
    """Code that imports the helpers the reference's scripts define (``from train_distributed import
    create_model, wrap_model_with_fsdp, create_optimizer, create_scheduler, train_step`` and so on) keeps
    working: a few steps under the parameter-sharded plan and under a plain optimizer, schedule landmarks,
    checkpoints, diagnostics, token weights, timing."""
    import math
    import yaml
    monkeypatch.setenv("KMOE_OFFLINE", "1")
    import train as t1
    import train_custom as tc
    import train_distributed as td
    cfg = {"model": dict(vocab_size=128, d_model=32, n_layers=2, n_heads=2, n_kv_heads=1, head_dim=16, d_ff=64,
                         d_ff_expert=32, n_experts=4, moe_top_k=2, moe_layers=[1], mamba_enabled=False,
                         mamba_layers=[], mod_enabled=False, max_seq_len=16, n_pred_tokens=2,
                         aux_loss_weights=[1.0, 0.5], moe_implementation="batched"),
           "training": dict(max_lr=1e-2, warmup_steps=2, min_lr_ratio=0.1, batch_size=2),
           "optimizer": dict(type="adamw", weight_decay=0.1), "data": dict(tokenizer_name="gpt2")}
    path = tmp_path / "c.yaml"
    path.write_text(yaml.safe_dump(cfg))
    assert td.load_config(str(path))["model"]["d_model"] == 32 and t1.load_config(str(path)) == td.load_config(str(path))
    rank, world, local = td.setup_distributed()
    assert (rank, world, local) == (0, 1, 0) and tc.is_main_process()
    torch.manual_seed(0)
    model, mcfg = td.create_model(cfg, rank, world)
    assert mcfg.d_model == 32 and sum(p.numel() for p in model.parameters()) > 0
    loader = td.create_dataloader(cfg, td.load_tokenizer(cfg), 16, 2, rank, world)
    batch = next(iter(loader))
    assert batch["input_ids"].shape == (2, 16) and torch.equal(batch["input_ids"], batch["labels"])
    # plain optimizer: decay / no-decay groups, warm-up then cosine to the floor
    opt = td.create_optimizer(model, cfg)
    assert [g["weight_decay"] for g in opt.param_groups] == [0.1, 0.0]
    no_decay = {id(p) for p in opt.param_groups[1]["params"]}
    assert all(("norm" in n or "embedding" in n or "bias" in n) == (id(p) in no_decay) for n, p in model.named_parameters())
    sched = td.create_scheduler(opt, cfg, total_steps=10)
    lrs = []
    losses = []
    for step in range(10):
        lrs.append(sched.get_last_lr()[0])
        m = td.train_step(model, batch, opt, sched, grad_clip=1.0, accumulation_steps=2, step=step, debug=(step == 1))
        losses.append(m["loss"])
    assert lrs[0] == 0.0 and lrs[1] == 0.0 and lrs[2] == pytest.approx(5e-3)        # two calls per optimizer step
    assert sched.last_step == 5 and sched.factor(10) == pytest.approx(0.1) and sched.factor(2) == pytest.approx(1.0)
    assert losses[-1] < losses[0] and "grad_norm" in m
    stats = td.collect_router_stats(model, batch)
    assert stats and all(0.0 <= s["entropy"] <= 1.0 for s in stats.values())
    census = td.check_parameter_gradients(model, 0, 0)
    assert "census" in census and "flow" in census
    # the same calls with the model under the parameter-sharded plan (one rank: the shard is the whole unit)
    torch.manual_seed(0)
    m2, _ = td.create_model(cfg, 0, 1)
    m2 = td.wrap_model_with_fsdp(m2, 0, use_bf16=False, cpu_offload=False, activation_checkpointing=False)
    opt2 = td.create_optimizer(m2, cfg)
    assert opt2 is m2._kmoe_plan.optimizer and opt2.param_groups[0]["lr"] == 1e-2
    sched2 = td.create_scheduler(opt2, cfg, total_steps=8)
    first = last = None
    for step in range(8):
        out = td.train_step(m2, batch, opt2, sched2, grad_clip=1.0, accumulation_steps=1, step=step)
        first = out["loss"] if first is None else first
        last = out["loss"]
    assert last < first and sched2.last_step == 8
    # checkpoints in train_custom's directory layout, for both kinds of model
    d = tc.save_checkpoint(model, opt, sched, 5, checkpoint_dir=str(tmp_path / "ck"))
    assert sorted(os.listdir(d)) == ["model.pt", "optimizer.pt", "training_state.pt"]
    before = {k: v.clone() for k, v in model.state_dict().items()}
    with torch.no_grad():
        next(model.parameters()).add_(1.0)
    assert tc.load_checkpoint(model, opt, sched, d) == 5
    assert all(torch.equal(v, model.state_dict()[k]) for k, v in before.items())
    d2 = tc.save_checkpoint(m2, opt2, sched2, 8, checkpoint_dir=str(tmp_path / "ck2"))
    full = torch.load(os.path.join(d2, "model.pt"))
    assert set(full) == set(model.state_dict()) and tc.load_checkpoint(m2, opt2, sched2, d2) == 8
    assert set(t1.get_model_state_dict(m2)) == set(full)
    # train.py's single-file checkpoint and cache path
    st = {"model": model, "optimizer": opt, "step": 7, "epoch": 0, "data_idx": 3, "losses": [1.0, 0.5],
          "total_tokens": 99, "config_path": str(path), "checkpoint_saved": False}
    assert t1.save_checkpoint(st, str(tmp_path / "b" / "checkpoint-7.pt"), reason="test") and st["checkpoint_saved"]
    ck = torch.load(tmp_path / "b" / "checkpoint-7.pt", weights_only=False)
    assert ck["step"] == 7 and ck["data_idx"] == 3 and "model_state_dict" in ck
    assert not t1.save_checkpoint({"model": None}, str(tmp_path / "none.pt"))
    p1, p2 = t1.get_cache_path("a/b", 128, 1000, True), t1.get_cache_path("a/b", 256, 1000, True)
    assert p1 != p2 and p1.endswith(".pt") and "packed" in p1
    stats_, collapsed, summary = t1.check_router_collapse_fast(model, "cpu", 0.7)
    assert isinstance(summary, str) and isinstance(collapsed, list)
    # token weights, weighted loss, evaluation, timing, scheduler with absolute rates, prefetcher, configuration
    w = tc.compute_token_weights(8, 0.5)
    assert w.mean().item() == pytest.approx(1.0) and w[-1] > w[0] and torch.equal(tc.compute_token_weights(4, 0), torch.ones(4))
    model.eval()
    plain, met = tc.compute_loss(model, batch)
    weighted, _ = tc.compute_loss(model, batch, tc.compute_token_weights(16, 0.0))
    assert met["ppl"] == pytest.approx(math.exp(float(plain)), rel=1e-4)
    with torch.no_grad():
        out = model(batch["input_ids"], labels=batch["labels"])
        ce = torch.nn.functional.cross_entropy(out["logits"][:, :-1].reshape(-1, 128), batch["labels"][:, 1:].reshape(-1))
    assert float(weighted) == pytest.approx(float(ce), rel=1e-5)          # uniform weights: the first head's loss
    ev = tc.evaluate(model, [batch, batch], max_batches=1)
    assert ev["batches"] == 1 and ev["ppl"] == pytest.approx(math.exp(ev["loss"]))
    ts = tc.TimingStats()
    ts.update(data=0.1, forward=0.3)
    ts.update("forward", 0.1)
    assert ts.counts == {"data": 1, "forward": 2} and "forward" in ts.summary()
    s3 = tc.CosineWarmupScheduler(torch.optim.SGD([torch.nn.Parameter(torch.zeros(1))], lr=1.0), 2, 10, max_lr=0.5, min_lr=0.05)
    for _ in range(10):
        s3.step()
    assert s3.get_lr()[0] == pytest.approx(0.05)
    assert [b["input_ids"].shape for b in tc.CUDAPrefetcher([batch, batch], "cpu")] == [(2, 16), (2, 16)]
    tcfg = tc.TrainConfig.from_yaml(str(path))
    assert tcfg.learning_rate == 1e-2 and tcfg.min_lr == pytest.approx(1e-3) and tcfg.max_seq_len == 16
    assert tcfg.model["d_model"] == 32 and tcfg.optimizer == "adamw" and tcfg.weight_decay == 0.1
    td.cleanup_distributed()


def test_names_of_the_hugging_face_scripts(monkeypatch):
    """``train_production`` (and its two variants) expose the wrapper, the collator, the data set loader and -
    built on first use - the Trainer subclasses under the reference's names."""
    monkeypatch.setenv("KMOE_OFFLINE", "1")
    import train_fineweb_working as tfw
    import train_production as tp
    from scripts import train_hf
    assert tfw.SimpleModelWrapper is tp.MoEModelWrapper and train_hf.MoEModelWrapper is tp.MoEModelWrapper
    trainer_cls, cb_cls = tp.MoETrainer, tp.TrueLossLoggingCallback
    assert trainer_cls.__name__ == "MoETrainer" and tfw.MuonTrainer.__name__ == "MoETrainer"
    logs = {"loss": 8.0}
    cb_cls(4).on_log(None, None, None, logs=logs)
    assert logs["true_loss"] == 2.0 and logs["accumulated_loss"] == 8.0

    class Tok:
        def __call__(self, texts, truncation=True, max_length=8, padding="max_length", return_tensors=None):
            texts = [texts] if isinstance(texts, str) else texts
            rows = [[ord(c) % 50 + 1 for c in t][:max_length] for t in texts]
            if padding == "max_length":
                mask = [[1] * len(r) + [0] * (max_length - len(r)) for r in rows]
                rows = [r + [0] * (max_length - len(r)) for r in rows]
                return {"input_ids": torch.tensor(rows), "attention_mask": torch.tensor(mask)}
            return {"input_ids": rows}

    batch = tp.OnTheFlyDataCollator(Tok(), 8)([{"text": "abc"}, {"text": "a much longer text"}])
    assert batch["input_ids"].shape == (2, 8) and batch["labels"][0].tolist()[3:] == [-100] * 5
    assert torch.equal(batch["labels"][1], batch["input_ids"][1])
    ds = tp.load_and_prepare_dataset({"data": {"dataset_name": "wikitext", "max_examples": 6},
                                      "model": {"max_seq_len": 12, "vocab_size": 64}}, Tok())
    assert len(ds) == 6 and ds[0]["input_ids"].shape == (12,) and int(ds[0]["input_ids"].max()) < 64
    assert tfw.tokenize_function({"text": ["hello"]}, Tok(), 4)["input_ids"] == [[ord(c) % 50 + 1 for c in "hell"]]
    with pytest.raises(AttributeError):
        tp.no_such_name
