"""Sharded data parallelism on 2 and 3 CPU ranks (gloo) against a single process."""
import pytest
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


def test_grouped_reduction_launches_in_order_and_refuses_a_gradient_completed_twice():
    """Host logic of the reduce-scatter that overlaps the backward pass (GPU transport only), on a stand-in object:
    a group goes when its last tensor is complete and every earlier group has gone; a tensor that is marked complete
    twice in one step is an error, because its group could otherwise go before the second contribution exists."""
    from kolmogorov_moe_architecture_b200.parallel.zero import ShardedDataParallel
    ps = [torch.nn.Parameter(torch.zeros(2)) for _ in range(5)]
    pool = ShardedDataParallel.__new__(ShardedDataParallel)
    pool.named = [(f"p{i}", p) for i, p in enumerate(ps)]
    pool._sync = True
    pool._chunks = [[(0, 8)], [(8, 8)], [(16, 8)]]
    pool._chunk_of = {id(ps[4]): 0, id(ps[3]): 0, id(ps[2]): 1, id(ps[1]): 2, id(ps[0]): 2}   # backward order
    pool._group_sizes = [2, 1, 2]
    pool._pending = list(pool._group_sizes)
    pool._ready_seen = set()
    pool._launched = 0
    launched = []
    pool._launch_chunk = launched.append
    pool._grad_ready(ps[2])                      # group 1 is complete, but group 0 has not gone yet
    assert launched == []
    pool._grad_ready(ps[4])
    assert launched == []
    pool._grad_ready(ps[3])                      # group 0 complete: 0 and the waiting 1 go, in order
    assert launched == [0, 1]
    pool._grad_ready(ps[1])
    with pytest.raises(RuntimeError, match="gradient of p1 was marked complete twice"):
        pool._grad_ready(ps[1])
    assert launched == [0, 1]                    # the second mark did not let group 2 go
    pool._grad_ready(ps[0])
    assert launched == [0, 1, 2]
    # micro-batches that only accumulate do not count
    pool._pending, pool._launched = list(pool._group_sizes), 0
    pool._ready_seen.clear()
    pool.set_sync(False)
    for p in ps:
        pool._grad_ready(p)
        pool._grad_ready(p)
    assert launched == [0, 1, 2] and pool._pending == [2, 1, 2]


def test_only_tied_weights_are_written_by_more_than_one_node_of_the_graph():
    """The direct gradient destinations (an op writes a weight's gradient into the flat buffer and marks it
    complete) are sound only for weights that a single node of the autograd graph writes.  For the model family,
    in every layer mix, the weights with several consumers are exactly the ones ``shared_parameter_ids`` finds
    (the tied embedding / first head); the per-expert slices of the eager expert loop are a CPU-path detail."""
    import collections
    import kolmogorov_moe_architecture_b200 as kmoe
    from kolmogorov_moe_architecture_b200.parallel.zero import shared_parameter_ids
    base = dict(vocab_size=200, d_model=64, n_layers=4, n_heads=4, n_kv_heads=2, head_dim=16, d_ff=128,
                d_ff_expert=64, n_experts=4, moe_layers=(1, 2), mamba_layers=(1,), max_seq_len=32, n_pred_tokens=2,
                aux_loss_weights=(1.0, 0.5), dropout=0.0, attention_dropout=0.0, residual_dropout=0.0,
                device="cpu", dtype="float32")
    for kw in [dict(mamba_moe_mode="moe_ffn"), dict(mamba_moe_mode="routing_mamba"), dict(mod_enabled=False),
               dict(tie_word_embeddings=False), dict(moe_routing="expert_choice", mamba_layers=()),
               dict(use_gradient_checkpointing=True)]:
        m = kmoe.MoETransformer(kmoe.AdvancedMoEConfig(**{**base, **kw}), verbose=False).train()
        ids = torch.randint(0, 200, (2, 32))
        loss = m(ids, labels=ids, return_logits=False)["loss"]
        names = {id(p): n for n, p in m.named_parameters()}
        uses = collections.Counter()
        seen, stack = set(), [loss.grad_fn]
        while stack:
            fn = stack.pop()
            if fn is None or fn in seen:
                continue
            seen.add(fn)
            for nxt, _ in fn.next_functions:
                if nxt is not None:
                    if hasattr(nxt, "variable"):
                        uses[id(nxt.variable)] += 1
                    stack.append(nxt)
        multi = {names[k] for k, c in uses.items() if c > 1 and k in names}
        multi = {n for n in multi if ".grouped_experts.w" not in n}
        shared = {names[k] for k in shared_parameter_ids(m)}
        assert multi == shared, (kw, multi, shared)
        assert shared == ({"token_embedding.embedding.weight"} if kw.get("tie_word_embeddings", True) else set())
