"""Parameter-sharded data parallelism on CPU ranks (gloo): two ranks with different data must follow the
replicated-parameter plan (same ranks, same data, AdamW) step for step; parameters are released between
uses; full and sharded state round-trips."""
import os

import torch

from dist_utils import run_ranks

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _tiny_cfg():
    import kolmogorov_moe_architecture_b200 as kmoe
    return kmoe.get_tiny_debug_config(vocab_size=256, d_model=64, n_heads=2, n_kv_heads=1, head_dim=32, d_ff=128,
                                      d_ff_expert=64, max_seq_len=32, n_pred_tokens=2, aux_loss_weights=(1.0, 0.5),
                                      mamba_moe_mode="moe_ffn", mod_capacity_factor=1.0)


def _worker(rank, world, tmp):
    import torch.distributed as dist
    import kolmogorov_moe_architecture_b200 as kmoe
    from kolmogorov_moe_architecture_b200.parallel.fsdp import FullyShardedDataParallel
    from kolmogorov_moe_architecture_b200.training.engine import TrainEngine
    cfg = _tiny_cfg()
    torch.manual_seed(0)
    model = kmoe.MoETransformer(cfg, verbose=False)
    ref = kmoe.MoETransformer(cfg, verbose=False)
    ref.load_state_dict(model.state_dict())
    from kolmogorov_moe_architecture_b200.parallel.zero import ShardedDataParallel
    rdp = ShardedDataParallel(ref, optimizer_kind="adamw", adamw_lr=1e-2, weight_decay=0.01)
    reng = TrainEngine(ref, rdp.optimizer, grad_clip=1.0, dp=rdp)
    n_full = sum(p.numel() for p in model.parameters())
    plan = FullyShardedDataParallel(model, lr=1e-2, weight_decay=0.01, overlap=(tmp.endswith("prefetch")))
    assert all(p.numel() == 0 for p in model.parameters()), "parameters must be released outside their unit"
    assert plan.param_bytes_per_rank() < 0.6 * n_full * 4
    eng = TrainEngine(model, plan.optimizer, grad_clip=1.0, dp=plan)
    g = torch.Generator().manual_seed(3)
    for step in range(3):
        ids = torch.randint(0, 256, (2 * world, 32), generator=g)
        a = eng.step(ids[rank * 2: rank * 2 + 2])
        b = reng.step(ids[rank * 2: rank * 2 + 2])
        assert abs(a.loss_value() - b.loss_value()) < 1e-3, (step, a.loss_value(), b.loss_value())
    if plan.overlap:     # per step: every block but the first ahead of its forward, every block but the last ahead of its backward
        assert plan.early_gathers == 3 * 2 * (len(plan.units) - 1) + 3, plan.early_gathers
    full = plan.full_state_dict()
    rs = dict(ref.named_parameters(remove_duplicate=False))
    worst = max((full[n] - rs[n].detach()).abs().max().item() for n in full)
    assert worst < 2e-3, worst
    # state round trip
    sd = plan.shard_state_dict()
    torch.save(sd, os.path.join(tmp, f"shard{rank}.pt"))
    plan.load_shard_state_dict(torch.load(os.path.join(tmp, f"shard{rank}.pt"), weights_only=False))
    plan.load_full_state_dict(full)
    again = plan.full_state_dict()
    assert all(torch.equal(full[n], again[n]) for n in full)
    model.eval()
    with torch.no_grad():
        out = model(torch.randint(0, 256, (1, 32)), return_logits=True)
    assert torch.isfinite(out["logits"]).all()
    dist.barrier()


def test_fsdp_two_ranks_follow_single_process(tmp_path):
    run_ranks(_worker, 2, str(tmp_path))


def test_fsdp_with_early_gathers_follows_single_process(tmp_path):
    """Same check with the next unit's gather issued ahead of its use (buffer-free bookkeeping)."""
    d = tmp_path / "prefetch"
    d.mkdir()
    run_ranks(_worker, 2, str(d))


def _ckpt_worker(rank, world, tmp):
    """Checkpoint of the sharded plan: resume from the shard files, and from model.pt alone."""
    import torch.distributed as dist
    import kolmogorov_moe_architecture_b200 as kmoe
    from kolmogorov_moe_architecture_b200.parallel.fsdp import FullyShardedDataParallel
    from kolmogorov_moe_architecture_b200.training import checkpoint as ckpt
    from kolmogorov_moe_architecture_b200.training.engine import TrainEngine
    cfg = _tiny_cfg()

    def fresh(seed):
        torch.manual_seed(seed)
        m = kmoe.MoETransformer(cfg, verbose=False)
        p = FullyShardedDataParallel(m, lr=1e-2)
        return m, p, TrainEngine(m, p.optimizer, grad_clip=1.0, dp=p)

    g = torch.Generator().manual_seed(5 + rank)
    data = [torch.randint(0, 256, (2, 32), generator=g) for _ in range(4)]
    m, p, e = fresh(0)
    for b in data[:2]:
        e.step(b)
    d = ckpt.save_param_sharded(tmp, 2, p, {"step": 2}, rank)
    after = [e.step(b).loss_value() for b in data[2:]]
    m2, p2, e2 = fresh(1)                                   # different init: everything must come from the files
    st = ckpt.load_param_sharded(d, p2, rank)
    assert st["step"] == 2
    again = [e2.step(b).loss_value() for b in data[2:]]
    assert max(abs(a - b) for a, b in zip(after, again)) < 1e-5, (after, again)
    # model.pt is an ordinary state dict of the unsharded model
    plain = kmoe.MoETransformer(cfg, verbose=False)
    plain.load_state_dict(torch.load(os.path.join(d, "model.pt"), weights_only=False))
    dist.barrier()


def test_fsdp_checkpoint_resume(tmp_path):
    run_ranks(_ckpt_worker, 2, str(tmp_path))


def test_fsdp_cpu_offload_single_process():
    """World size 1 with host-resident shards: parameters live in host memory between uses and training works."""
    import kolmogorov_moe_architecture_b200 as kmoe
    from kolmogorov_moe_architecture_b200.parallel.fsdp import FullyShardedDataParallel
    from kolmogorov_moe_architecture_b200.training.engine import TrainEngine
    cfg = _tiny_cfg()
    torch.manual_seed(0)
    m = kmoe.MoETransformer(cfg, verbose=False)
    p = FullyShardedDataParallel(m, lr=1e-2, cpu_offload=True)
    e = TrainEngine(m, p.optimizer, grad_clip=1.0, dp=p)
    ids = torch.randint(0, 256, (2, 32))
    l0 = e.step(ids).loss_value()
    for _ in range(5):
        l1 = e.step(ids).loss_value()
    assert l1 < l0


def _ep_worker(rank, world, tmp):
    """Dense parameters sharded per block, experts split over the expert-parallel group: same losses and
    parameters as the replicated-parameter plan with the same expert pool, one global-norm clip over both."""
    import kolmogorov_moe_architecture_b200 as kmoe
    from kolmogorov_moe_architecture_b200.parallel import mesh as pmesh
    from kolmogorov_moe_architecture_b200.parallel.fsdp import FullyShardedDataParallel
    from kolmogorov_moe_architecture_b200.parallel.zero import ParallelPlan, ShardedDataParallel
    from kolmogorov_moe_architecture_b200.training.engine import TrainEngine
    mesh = pmesh.make_mesh(2)
    cfg = kmoe.get_tiny_debug_config(vocab_size=256, d_model=64, n_heads=2, n_kv_heads=1, head_dim=32, d_ff=128,
                                     d_ff_expert=64, max_seq_len=32, n_pred_tokens=2, aux_loss_weights=(1.0, 0.5),
                                     mamba_moe_mode="moe_ffn", mod_capacity_factor=1.0,
                                     moe_implementation="expert_parallel", ep_size=2)

    def build(sharded):
        torch.manual_seed(0)
        m = kmoe.MoETransformer(cfg, verbose=False)
        n_ep = sum(p.numel() for p in m.parameters() if getattr(p, "_kmoe_expert_parallel", False))
        assert n_ep > 0
        experts = ShardedDataParallel(m, optimizer_kind="adamw", group=mesh.expert_dp_group, adamw_lr=1e-2,
                                      weight_decay=0.01, expert_params=True, grad_scale=0.5, broadcast_from_rank0=False)
        dense = (FullyShardedDataParallel(m, lr=1e-2, weight_decay=0.01, overlap=True) if sharded
                 else ShardedDataParallel(m, optimizer_kind="adamw", adamw_lr=1e-2, weight_decay=0.01))
        plan = ParallelPlan([dense, experts])
        return m, dense, TrainEngine(m, plan, grad_clip=0.5, dp=plan)

    ma, _, ea = build(False)
    mb, fsdp, eb = build(True)
    assert all(p.numel() > 0 for p in mb.parameters() if getattr(p, "_kmoe_expert_parallel", False))
    assert all(p.numel() == 0 for p in mb.parameters() if not getattr(p, "_kmoe_expert_parallel", False))
    g = torch.Generator().manual_seed(11 + rank)
    for step in range(3):
        ids = torch.randint(0, 256, (2, 32), generator=g)
        la, lb = ea.step(ids).loss_value(), eb.step(ids).loss_value()
        assert abs(la - lb) < 1e-3, (step, la, lb)
    full = fsdp.full_state_dict()
    ref = dict(ma.named_parameters(remove_duplicate=False))
    assert max((full[n] - ref[n].detach()).abs().max().item() for n in full) < 2e-3
    for (n, pa), (_, pb) in zip(ma.named_parameters(), mb.named_parameters()):
        if getattr(pa, "_kmoe_expert_parallel", False):
            assert torch.allclose(pa, pb, atol=2e-3), n
    # checkpoint of both pools, restored into a freshly built job: the next step gives the same loss
    from kolmogorov_moe_architecture_b200.training import checkpoint as ckpt
    d = ckpt.save_param_sharded(tmp, 3, eb.dp, {"step": 3}, rank, ep_rank=mesh.ep_rank, ep_size=2)
    mc, _, ec = build(True)
    st = ckpt.load_param_sharded(d, ec.dp, rank, ep_rank=mesh.ep_rank, ep_size=2)
    assert st["step"] == 3
    ids = torch.randint(0, 256, (2, 32), generator=g)
    assert abs(eb.step(ids).loss_value() - ec.step(ids).loss_value()) < 1e-4


def test_sharded_dense_parameters_with_expert_parallel_experts(tmp_path):
    run_ranks(_ep_worker, 2, str(tmp_path))


def _accum_worker(rank, world, tmp):
    """Two micro-batches per step: each one's gradients are reduced and added to the shards (the sharded plan
    against the replicated plan with the same accumulation)."""
    import kolmogorov_moe_architecture_b200 as kmoe
    from kolmogorov_moe_architecture_b200.parallel.fsdp import FullyShardedDataParallel
    from kolmogorov_moe_architecture_b200.parallel.zero import ShardedDataParallel
    from kolmogorov_moe_architecture_b200.training.engine import TrainEngine
    cfg = _tiny_cfg()
    torch.manual_seed(0)
    a = kmoe.MoETransformer(cfg, verbose=False)
    b = kmoe.MoETransformer(cfg, verbose=False)
    b.load_state_dict(a.state_dict())
    pa = ShardedDataParallel(a, optimizer_kind="adamw", adamw_lr=1e-2, weight_decay=0.01)
    pb = FullyShardedDataParallel(b, lr=1e-2, weight_decay=0.01, overlap=True)
    ea = TrainEngine(a, pa.optimizer, grad_clip=1.0, grad_accum=2, dp=pa)
    eb = TrainEngine(b, pb.optimizer, grad_clip=1.0, grad_accum=2, dp=pb)
    g = torch.Generator().manual_seed(7 + rank)
    for step in range(3):
        ids = torch.randint(0, 256, (4, 32), generator=g)          # two micro-batches of two sequences
        la, lb = ea.step(ids).loss_value(), eb.step(ids).loss_value()
        assert abs(la - lb) < 1e-3, (step, la, lb)
    full = pb.full_state_dict()
    ref = dict(a.named_parameters(remove_duplicate=False))
    assert max((full[n] - ref[n].detach()).abs().max().item() for n in full) < 2e-3
    assert all(p.numel() == 0 for p in b.layers.parameters())      # every block is released again


def test_fsdp_gradient_accumulation_reduces_every_micro_batch(tmp_path):
    run_ranks(_accum_worker, 2, str(tmp_path))


def _recompute_worker(rank, world, tmp):
    """Activation recomputation: a block's forward runs again inside the backward pass, with its parameters
    gathered for it and kept until its gradients are reduced."""
    import kolmogorov_moe_architecture_b200 as kmoe
    from kolmogorov_moe_architecture_b200.parallel.fsdp import FullyShardedDataParallel
    from kolmogorov_moe_architecture_b200.parallel.zero import ShardedDataParallel
    from kolmogorov_moe_architecture_b200.training.engine import TrainEngine
    cfg = _tiny_cfg()
    cfg.use_gradient_checkpointing = True
    torch.manual_seed(0)
    a = kmoe.MoETransformer(cfg, verbose=False)
    b = kmoe.MoETransformer(cfg, verbose=False)
    b.load_state_dict(a.state_dict())
    pa = ShardedDataParallel(a, optimizer_kind="adamw", adamw_lr=1e-2, weight_decay=0.01)
    pb = FullyShardedDataParallel(b, lr=1e-2, weight_decay=0.01, overlap=True)
    ea = TrainEngine(a, pa.optimizer, grad_clip=1.0, dp=pa)
    eb = TrainEngine(b, pb.optimizer, grad_clip=1.0, dp=pb)
    g = torch.Generator().manual_seed(9 + rank)
    for step in range(3):
        ids = torch.randint(0, 256, (2, 32), generator=g)
        la, lb = ea.step(ids).loss_value(), eb.step(ids).loss_value()
        assert abs(la - lb) < 1e-3, (step, la, lb)
    assert all(p.numel() == 0 for p in b.layers.parameters())


def test_fsdp_with_activation_recomputation(tmp_path):
    run_ranks(_recompute_worker, 2, str(tmp_path))


def _script_api_worker(rank, world, tmp):
    """The reference's launcher spelled with its own helper names, on two ranks: every rank builds the model,
    shards it, steps on its own batches, and the two ranks end with the same full state dict and checkpoint."""
    import torch.distributed as dist
    import yaml
    os.environ["KMOE_OFFLINE"] = "1"
    import train_custom as tc
    import train_distributed as td
    cfg = {"model": dict(vocab_size=128, d_model=32, n_layers=2, n_heads=2, n_kv_heads=1, head_dim=16, d_ff=64,
                         d_ff_expert=32, n_experts=4, moe_top_k=2, moe_layers=[1], mamba_enabled=False,
                         mamba_layers=[], mod_enabled=False, max_seq_len=16, n_pred_tokens=1,
                         aux_loss_weights=[1.0], moe_implementation="batched"),
           "training": dict(max_lr=5e-3, warmup_steps=1, min_lr_ratio=0.1), "optimizer": dict(weight_decay=0.01)}
    r, w, _ = td.setup_distributed()                   # the group exists already: ranks are read from it
    assert (r, w) == (rank, world)
    torch.manual_seed(0)
    model, _ = td.create_model(cfg, r, w)
    model = td.wrap_model_with_fsdp(model, r, use_bf16=False, activation_checkpointing=False)
    opt = td.create_optimizer(model, cfg)
    sched = td.create_scheduler(opt, cfg, total_steps=6)
    loader = iter(td.create_dataloader(cfg, td.load_tokenizer(cfg), 16, 2, r, w))
    first = next(loader)
    other = [torch.empty_like(first["input_ids"]) for _ in range(w)]
    dist.all_gather(other, first["input_ids"])
    assert not torch.equal(other[0], other[1]), "ranks must see different rows"
    losses = []
    batch = first
    for step in range(6):
        losses.append(td.train_step(model, batch, opt, sched, grad_clip=1.0, accumulation_steps=1, step=step)["loss"])
    assert losses[-1] < losses[0]
    import train as single_gpu_script
    full = single_gpu_script.get_model_state_dict(model)          # gathers the sharded model in full
    flat = torch.cat([v.reshape(-1).float() for _, v in sorted(full.items())])
    both = [torch.empty_like(flat) for _ in range(w)]
    dist.all_gather(both, flat)
    assert torch.equal(both[0], both[1]), "ranks hold different parameters after the same steps"
    d = tc.save_checkpoint(model, opt, sched, 6, checkpoint_dir=os.path.join(tmp, "ck"))
    dist.barrier()
    ck = os.path.join(tmp, "ck", "checkpoint-6")
    assert (d == ck) if r == 0 else (d is None)
    assert sorted(os.listdir(ck)) == ["model.pt", "optimizer.pt", "training_state.pt"]
    assert tc.load_checkpoint(model, opt, sched, ck) == 6


def test_reference_launcher_helpers_on_two_ranks(tmp_path):
    run_ranks(_script_api_worker, 2, str(tmp_path))
