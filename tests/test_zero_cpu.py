"""Sharded data parallelism on 2 and 3 CPU ranks (gloo) against a single process."""
import torch

from dist_utils import run_ranks


def _cfg():
    from kolmogorov_moe_architecture_b200 import AdvancedMoEConfig
    return AdvancedMoEConfig(vocab_size=128, d_model=64, n_layers=2, n_heads=2, n_kv_heads=1, head_dim=32, d_ff=128,
                             d_ff_expert=64, n_experts=4, moe_layers=(), mamba_layers=(1,), mod_enabled=False,
                             max_seq_len=32, n_pred_tokens=2, aux_loss_weights=(1.0, 0.5), dtype="float32",
                             device="cpu", dropout=0.0, attention_dropout=0.0, residual_dropout=0.0)


def _data(world):
    g = torch.Generator().manual_seed(7)
    return torch.randint(0, 128, (3, 2 * world, 32), generator=g)     # steps x global batch x seq


def _worker(rank, world, kind, ref_state, accum=1):
    from kolmogorov_moe_architecture_b200 import MoETransformer
    from kolmogorov_moe_architecture_b200.parallel.zero import ShardedDataParallel
    from kolmogorov_moe_architecture_b200.training.engine import TrainEngine
    torch.manual_seed(0)
    model = MoETransformer(_cfg(), verbose=False)
    dp = ShardedDataParallel(model, optimizer_kind=kind, lr=1e-2, adamw_lr=1e-2)
    eng = TrainEngine(model, dp.optimizer, grad_clip=1.0, grad_accum=accum, dp=dp)
    data = _data(world)
    for s in range(3):
        eng.step(data[s, 2 * rank: 2 * rank + 2])       # with accum = 2: two micro-batches of one sequence
    sd = model.state_dict()
    for k, v in ref_state.items():
        assert torch.allclose(sd[k], v, atol=5e-4, rtol=1e-3), (k, (sd[k] - v).abs().max())
    # every tensor has exactly one owner and the owners cover everything
    import torch.distributed as dist
    owned = [None] * world
    dist.all_gather_object(owned, dp.owned_names())
    flat = [n for o in owned for n in o]
    assert len(flat) == len(set(flat)) == len(dp.named)


def _reference(kind, world):
    from kolmogorov_moe_architecture_b200 import MoETransformer
    from kolmogorov_moe_architecture_b200.training.engine import TrainEngine
    from kolmogorov_moe_architecture_b200.training.optim_factory import build_optimizer
    torch.manual_seed(0)
    model = MoETransformer(_cfg(), verbose=False)
    eng = TrainEngine(model, build_optimizer(model, kind, lr=1e-2, adamw_lr=1e-2), grad_clip=1.0)
    data = _data(world)
    for s in range(3):
        eng.step(data[s])
    return {k: v.clone() for k, v in model.state_dict().items()}


def test_zero_matches_single_process_adamw_2ranks():
    run_ranks(_worker, 2, "adamw", _reference("adamw", 2))


def test_zero_with_gradient_accumulation_reduces_once_per_step():
    """Micro-batches of equal size: accumulating two of them is the same step as one batch of both, and the
    ranks exchange gradients only after the last one."""
    run_ranks(_worker, 2, "adamw", _reference("adamw", 2), 2)


def test_zero_matches_single_process_muon_3ranks():
    run_ranks(_worker, 3, "muon", _reference("muon", 3))


def test_owner_assignment_is_balanced():
    from kolmogorov_moe_architecture_b200.parallel.zero import assign_owners
    sizes = [100, 90, 80, 10, 10, 10, 5, 5]
    own = assign_owners(sizes, 3)
    loads = [sum(s for s, o in zip(sizes, own) if o == r) for r in range(3)]
    assert max(loads) - min(loads) <= 128 * 3
