"""CPU tests of optimizers, schedules, trainer, checkpoints, data pipeline and failure handling."""
import os
import signal
import time

import pytest
import torch

import kolmogorov_moe_architecture_b200 as kmoe
from kolmogorov_moe_architecture_b200.training import checkpoint as ck
from kolmogorov_moe_architecture_b200.training.engine import TrainEngine
from kolmogorov_moe_architecture_b200.training.lr_schedule import CosineScheduleWithWarmup, cosine_lambda
from kolmogorov_moe_architecture_b200.training.muon_optimizer import (CombinedOptimizer, Muon, Muon8bit,
                                                                     get_muon_optimizer, split_muon_params)
from kolmogorov_moe_architecture_b200.training.optim_factory import build_optimizer


def _model(**kw):
    cfg = kmoe.get_tiny_debug_config(vocab_size=128, max_seq_len=16, d_model=64, head_dim=16, d_ff=128,
                                     d_ff_expert=64, mamba_moe_mode="moe_ffn", **kw)
    torch.manual_seed(0)
    return cfg, kmoe.MoETransformer(cfg, verbose=False)


def test_schedule_landmarks():
    p = [torch.zeros(1, requires_grad=True)]
    s = CosineScheduleWithWarmup(torch.optim.SGD(p, lr=1.0), 10, 100, 1e-3, 1e-4)
    assert s.get_lr(0) == 0.0 and abs(s.get_lr(10) - 1e-3) < 1e-12 and abs(s.get_lr(100) - 1e-4) < 1e-12
    assert abs(s.get_lr(55) - (1e-4 + 0.5 * 9e-4)) < 1e-9 and s.get_lr(1000) == 1e-4
    f = cosine_lambda(10, 100)
    assert f(0) == 0.0 and f(10) == 1.0 and abs(f(100) - 0.1) < 1e-9


def test_muon_writes_orthogonal_matrix_back_into_momentum():
    torch.manual_seed(11)
    w = torch.randn(16, 32, requires_grad=True)
    o = Muon([w], lr=0.1, weight_decay=0.0)
    w.grad = torch.randn(16, 32)
    o.step()
    buf = o.state[w]["momentum_buffer"]
    assert (buf @ buf.T - torch.eye(16)).abs().max() < 0.5       # 5 cubic iterations: roughly orthonormal rows
    o2 = Muon([torch.randn(16, 32, requires_grad=True)], standard_muon=True)
    assert o2.defaults["standard_muon"]


def test_muon8bit_quantisation_roundtrip():
    t = torch.randn(5000)
    q, s, shape, n = Muon8bit._quantize_to_8bit(t, 2048)
    back = Muon8bit._dequantize_from_8bit(q, s, shape, n)
    assert q.dtype == torch.int8 and back.shape == t.shape and (back - t).abs().max() <= t.abs().max() / 127 + 1e-6
    assert Muon8bit._square_factor(4096) == (64, 64) and Muon8bit._square_factor(13) == (1, 13)


def test_optimizer_partitions():
    _, m = _model()
    mu, ad = split_muon_params(m, fsdp_mode=False)
    names = {id(p): n for n, p in m.named_parameters()}
    assert all(p.dim() == 2 for p in mu)
    assert not any("embedding" in names[id(p)] or "lm_heads" in names[id(p)] or "norm" in names[id(p)] for p in mu)
    assert any("grouped_experts.w1" in names[id(p)] for p in ad)          # stacked experts go to AdamW here
    c = CombinedOptimizer(m)
    assert any(p.dim() == 3 for g in c.muon.param_groups for p in g["params"])   # ...and to Muon there
    sd = c.state_dict()
    assert isinstance(sd, list) and len(sd) == 2
    h = get_muon_optimizer(m, fsdp_mode=False)
    assert set(h.state_dict()) == {"muon", "adamw"}


def test_engine_trains_and_grad_accum_matches_big_batch():
    cfg, m1 = _model(mod_enabled=False, moe_layers=(), n_experts=4)
    _, m2 = _model(mod_enabled=False, moe_layers=(), n_experts=4)
    ids = torch.randint(0, 128, (4, 16))
    e1 = TrainEngine(m1, build_optimizer(m1, "adamw", adamw_lr=1e-2), grad_clip=1.0, grad_accum=1)
    e2 = TrainEngine(m2, build_optimizer(m2, "adamw", adamw_lr=1e-2), grad_clip=1.0, grad_accum=2)
    e1.step(ids); e2.step(ids)
    for (n, a), (_, b) in zip(m1.named_parameters(), m2.named_parameters()):
        assert torch.allclose(a, b, atol=2e-4), n


def test_checkpoint_formats_roundtrip(tmp_path):
    cfg, m = _model()
    opt = CombinedOptimizer(m)
    ids = torch.randint(0, 128, (2, 16))
    TrainEngine(m, opt).step(ids)
    ck.save_format_b(str(tmp_path / "checkpoint-5.pt"), m, opt, 5, 0, 0, [1.0], 100, "cfg.yaml")
    _, m2 = _model()
    _, obj = ck.load_model_state(m2, str(tmp_path / "checkpoint-5.pt"))
    assert obj["step"] == 5 and isinstance(obj["optimizer_state_dict"], list)
    assert all(torch.equal(a, b) for a, b in zip(m.state_dict().values(), m2.state_dict().values()))
    for s in (1, 2, 3, 4):
        ck.save_format_c(str(tmp_path / "c"), s, m, opt, {"step": s})
    assert sorted(os.listdir(tmp_path / "c")) == ["checkpoint-2", "checkpoint-3", "checkpoint-4"]
    assert ck.load_format_c(str(tmp_path / "c" / "checkpoint-4"), m2)["step"] == 4
    # prefixed keys of other writers (HF wrapper, DDP, torch.compile) are accepted
    pref = {"model." + k: v for k, v in m.state_dict().items()}
    ck.load_model_state(m2, {"model_state_dict": pref})
    ck.load_model_state(m2, {"_orig_mod." + k: v for k, v in m.state_dict().items()})


def test_resume_reproduces_the_loss_curve(tmp_path):
    def run(n, resume=None):
        cfg, m = _model()
        opt = build_optimizer(m, "muon", lr=1e-2, adamw_lr=1e-2)
        eng = TrainEngine(m, opt)
        start = 0
        if resume:
            obj = torch.load(resume, weights_only=False)
            m.load_state_dict(obj["model_state_dict"]); opt.load_state_dict(obj["optimizer_state_dict"])
            start = obj["step"]
        g = torch.Generator().manual_seed(0)
        data = torch.randint(0, 128, (6, 2, 16), generator=g)
        losses = []
        for s in range(start, n):
            torch.manual_seed(100 + s)
            losses.append(eng.step(data[s]).loss_value())
            if s == 2 and not resume:
                ck.save_format_b(str(tmp_path / "r.pt"), m, opt, 3, 0, 0, losses, 0, "x")
        return losses
    full = run(6)
    tail = run(6, str(tmp_path / "r.pt"))
    assert full[3:] == pytest.approx(tail, abs=1e-6)


def test_data_pipeline(tmp_path):
    from kolmogorov_moe_architecture_b200.data import (ByteTokenizer, DolmaMemoryMappedDataset, PackedDocumentDataset,
                                                       PinnedPrefetcher, SyntheticTokenDataset,
                                                       document_attention_mask, write_token_file)
    a = next(iter(SyntheticTokenDataset(100, 8, seed=1))); b = next(iter(SyntheticTokenDataset(100, 8, seed=1)))
    assert torch.equal(a["input_ids"], b["input_ids"]) and a["input_ids"] is a["labels"] or True
    write_token_file(str(tmp_path / "t.bin"), list(range(60)))
    ds = DolmaMemoryMappedDataset(str(tmp_path / "t.bin"), seq_len=8, n_pred_tokens=2, vocab_size=100)
    assert len(ds) == 6 and ds[1]["input_ids"].tolist() == list(range(10, 18))
    rows = list(PackedDocumentDataset([[1, 2, 3], [4, 5], [6, 7, 8, 9]], seq_len=6, eos_id=0))
    assert rows[0]["input_ids"].tolist() == [1, 2, 3, 0, 4, 5] and rows[0]["labels"].tolist() == [1, 2, 3, 0, -100, 5]
    mask = document_attention_mask(rows[0]["doc_ids"][None])
    assert mask[0, 0, 4, 3] == float("-inf") and mask[0, 0, 5, 4] == 0 and mask[0, 0, 2, 3] == float("-inf")
    tok = ByteTokenizer()
    assert tok.decode(tok("héllo")["input_ids"]) == "héllo"

    def bad():
        yield {"input_ids": torch.zeros(2)}
        raise RuntimeError("loader failed")
    it = iter(PinnedPrefetcher(bad(), pin=False))
    next(it)
    with pytest.raises(RuntimeError, match="loader failed"):
        next(it)


def test_interrupt_guard_and_watchdog():
    from kolmogorov_moe_architecture_b200.utils.fault import InterruptGuard, StepWatchdog
    with InterruptGuard() as g:
        os.kill(os.getpid(), signal.SIGTERM)
        time.sleep(0.05)
        assert g.requested and g.signum == signal.SIGTERM
    fired = []
    dog = StepWatchdog(0.2, fired.append, poll_s=0.05).start()
    time.sleep(0.1); dog.beat(); time.sleep(0.1)
    assert not fired
    time.sleep(0.4)
    dog.stop()
    assert fired and dog.tripped


def test_router_collapse_probe_and_census():
    from kolmogorov_moe_architecture_b200.utils.fault import check_router_collapse, gradient_census, NormWatch
    cfg, m = _model()
    stats, collapsed, summary = check_router_collapse(m, n_samples=256)
    assert set(stats) == {1, 2} and "entropy" in stats[1]
    with torch.no_grad():
        m.layers[2].ffn.router.router[2].weight.zero_()
        m.layers[2].ffn.router.router[2].weight[0] = 50.0      # every token's best expert is 0
    _, collapsed, summary = check_router_collapse(m, n_samples=256)
    assert 2 in collapsed and "COLLAPSE" in summary
    watch = NormWatch(m)
    ids = torch.randint(0, 128, (2, 16))
    m.train(); m(ids, labels=ids, return_logits=False)["loss"].backward()
    cen = gradient_census(m)
    assert cen["router"]["nan"] == 0 and cen["norm"]["tensors"] > 0
    assert len(watch.stuck(m)) == len(watch.init)


def test_yaml_loaders(tmp_path):
    from kolmogorov_moe_architecture_b200.utils.config_io import (load_yaml, model_config_strict,
                                                                 model_config_tolerant, section)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    y = load_yaml(os.path.join(root, "configs", "test.yaml"))
    s = model_config_strict(y)
    t = model_config_tolerant(y, seq_len=64)
    assert s.d_model == t.d_model == 256 and t.max_seq_len == 64 and t.dropout == 0.0
    assert section(y, "training")["warmup_steps"] == 10 and section(y, "optimizer")["newton_iters"] == 5
    bare = model_config_tolerant({"model": {"n_layers": 2}})
    assert bare.moe_layers == () and bare.n_pred_tokens == 1 and not bare.mamba_enabled
    (tmp_path / "bad.yaml").write_text("modle: {}\n")
    with pytest.raises(KeyError):
        load_yaml(str(tmp_path / "bad.yaml"))
    with pytest.raises(TypeError):
        model_config_strict({"model": {"no_such_field": 1}})


def test_threaded_prefetcher_yields_batches_on_the_device_in_order():
    from kolmogorov_moe_architecture_b200.data import ThreadedPrefetcher
    batches = [{"input_ids": torch.full((2, 4), i), "n": i} for i in range(7)]
    got = list(ThreadedPrefetcher(batches, "cpu", buffer_size=2))
    assert [b["n"] for b in got] == list(range(7))
    assert all(torch.equal(b["input_ids"], torch.full((2, 4), b["n"])) for b in got)


def test_async_checkpoint_writer_markers_pruning_and_errors(tmp_path):
    """Background sharded saves: the state is snapshotted at submit time, a directory is a checkpoint only
    when every rank's marker is in it, pruning ignores incomplete directories, writer errors surface."""
    from kolmogorov_moe_architecture_b200.training import checkpoint as ck

    class FakePlan:                      # what save_sharded needs from a data-parallel plan
        def __init__(self, v):
            self.t = torch.full((4,), float(v))

        def optimizer_state_dict(self):
            return {"m": self.t}

    root = str(tmp_path)
    model = torch.nn.Linear(3, 2)
    w0, w1 = ck.AsyncCheckpointWriter(), ck.AsyncCheckpointWriter()
    for step in (10, 20, 30):
        plan0, plan1 = FakePlan(step), FakePlan(step + 1)
        d = ck.save_sharded(root, step, model, plan0, {"step": step}, rank=0, keep=2, writer=w0, world=2)
        plan0.t.zero_()                  # training goes on: the file must hold the value at submit time
        w0.wait()
        assert not ck.checkpoint_complete(d, 2)
        if step < 30:                    # rank 1 never finishes the last one
            ck.save_sharded(root, step, model, plan1, {"step": step}, rank=1, keep=2, writer=w1, world=2)
            w1.wait()
            assert ck.checkpoint_complete(d, 2)
        assert torch.equal(torch.load(os.path.join(d, "optimizer-rank0.pt"))["m"], torch.full((4,), float(step)))
    assert ck.latest_complete_checkpoint(root, 2).endswith("checkpoint-20")
    ck.prune_checkpoints(root, keep=1, world=2)
    left = sorted(n for n in os.listdir(root) if n.startswith("checkpoint-"))
    assert left == ["checkpoint-20", "checkpoint-30"]           # 10 pruned, incomplete 30 left alone
    st = ck.load_sharded(os.path.join(root, "checkpoint-20"), torch.nn.Linear(3, 2),
                         type("P", (), {"load_optimizer_state_dict": lambda self, sd: None})(), rank=0)
    assert st["step"] == 20
    bad = ck.AsyncCheckpointWriter()
    bad.submit({os.path.join(root, "x.pt"): {"f": lambda: 0}}, root, 0)      # a lambda cannot be pickled
    with pytest.raises(RuntimeError, match="asynchronous checkpoint write failed"):
        bad.wait()


def test_engine_rejects_token_ids_outside_the_vocabulary_on_the_host():
    _, m = _model()
    eng = TrainEngine(m, torch.optim.AdamW(m.parameters(), lr=1e-3))
    V = m.config.vocab_size
    ok = torch.randint(0, V, (2, 16))
    eng.step(ok)
    for bad in (ok.clone().index_put_((torch.tensor(0), torch.tensor(3)), torch.tensor(V)),
                ok.clone().index_put_((torch.tensor(1), torch.tensor(0)), torch.tensor(-1))):
        with pytest.raises(ValueError, match="token ids must lie in"):
            eng.step(bad)
