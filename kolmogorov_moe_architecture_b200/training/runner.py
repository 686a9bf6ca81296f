"""The training loop shared by the command-line entrypoints.

Each entrypoint (``train.py``, ``train_distributed.py``, ``train_custom.py``, ``scripts/train.py``)
parses its own flags - kept from the reference's scripts - into a :class:`RunSpec` and calls
:func:`run_training`.  What a spec selects:

* weight regime: ``bf16`` weights (train.py:508-509) or fp32 master weights with bf16 autocast
  (scripts/train.py); fp16 weights are accepted for parity.
* optimizer family: ``combined`` (Muon on ndim >= 2 + AdamW groups, train.py:566-705), ``hybrid``
  (name-based Muon + AdamW, muon_optimizer.py:468-616), ``muon8bit_all`` (train_custom.py:1035-1049),
  ``adamw`` (decay / no-decay groups).
* parallelism: one process, or torchrun with the sharded data-parallel plan (+ expert parallelism
  when the model config says ``moe_implementation: expert_parallel``).
* checkpoint format B (single file) or C (directory, newest three kept), sharded when distributed.
* data: synthetic ids, streaming text, packed documents with cross-document label masking.

Unlike the reference's distributed script the loop seeds every rank, clips with the global norm
across shards, does not shift labels twice, and can resume.
"""
from __future__ import annotations

import math
import os
import time
from dataclasses import dataclass, field
from typing import Any, Dict, Optional

import torch

from ..config import AdvancedMoEConfig
from ..data import (DolmaStreamingDataset, PackedDocumentDataset, PinnedPrefetcher, SyntheticTokenDataset,
                    TokenizerWrapper, PackedDocs)
from ..models.transformer import MoETransformer
from ..parallel import mesh as pmesh
from ..utils.config_io import load_yaml, model_config_strict, model_config_tolerant, section
from ..utils.fault import InterruptGuard, StepWatchdog, check_router_collapse
from ..utils.logging import MetricLogger
from ..utils.profiling import PhaseTimer
from . import checkpoint as ckpt
from .engine import TrainEngine
from .lr_schedule import CosineScheduleWithWarmup
from .muon_optimizer import CombinedOptimizer, Muon8bit, get_muon_optimizer


@dataclass
class RunSpec:
    config_path: str
    steps: Optional[int] = None
    batch_size: Optional[int] = None
    seq_len: Optional[int] = None
    grad_accum: Optional[int] = None
    strict_config: bool = False
    weights: str = "bf16"                  # bf16 | fp16 | fp32_autocast
    optimizer_family: str = "auto"         # auto | combined | hybrid | muon8bit_all | adamw
    checkpoint_format: str = "B"           # B | C
    checkpoint_dir: Optional[str] = None
    save_interval: Optional[int] = None
    resume: Optional[str] = None
    data_mode: str = "auto"                # auto | synthetic | streaming | packed
    document_mask: bool = False
    grad_checkpoint: bool = False
    compile: bool = False
    wandb: bool = False
    wandb_project: str = "Kolmogorov-Testing"
    wandb_run: Optional[str] = None
    lr_scale: float = 1.0
    gpu: Optional[int] = None
    balanced_routing: bool = False
    collapse_check_interval: int = 0
    collapse_entropy_threshold: float = 0.7
    reallocate: bool = False
    entropy_threshold: float = 0.85
    constant_lr: bool = False              # train.py trains at a fixed LR (no scheduler)
    profile: bool = False
    debug: bool = False                    # gradient-flow table, router statistics and stuck-norm check
    debug_interval: int = 100
    use_8bit_optimizer: bool = False       # bitsandbytes AdamW8bit when installed (one process, AdamW family)
    token_weight_decay: float = 0.0        # > 0: later positions weigh more in the loss (train_custom.py:690-707)
    use_lr_schedule: bool = True
    step_deadline_s: float = 0.0           # > 0 arms the step watchdog
    transport: Optional[str] = None
    jsonl: Optional[str] = None
    shard_params: bool = False             # ZeRO-3 / FULL_SHARD plan (AdamW) instead of replicated parameters
    cpu_offload: bool = False              # with shard_params: shards and optimizer state in pinned host memory
    async_checkpoint: bool = False         # sharded saves: copy to pinned memory, write files in the background
    extra: Dict[str, Any] = field(default_factory=dict)


def _build_optimizer(spec: RunSpec, model, opt_cfg, train_cfg):
    fam = spec.optimizer_family
    kind = opt_cfg.get("type", "adamw")
    if fam == "auto":
        fam = "combined" if kind == "muon" else "adamw"
    s = spec.lr_scale
    wd = opt_cfg.get("weight_decay", train_cfg.get("weight_decay", 0.01))
    if fam == "combined":
        adamw_lr = opt_cfg.get("adamw_lr", 3e-4) * s
        norm_lr = opt_cfg.get("norm_lr")
        return CombinedOptimizer(model, muon_lr=opt_cfg.get("muon_lr", 0.02) * s, adamw_lr=adamw_lr,
                                 momentum=opt_cfg.get("momentum", 0.95), weight_decay=wd,
                                 nesterov=opt_cfg.get("nesterov", True), backend=opt_cfg.get("backend", "newton"),
                                 newton_iters=opt_cfg.get("newton_iters", 5),
                                 norm_lr=(norm_lr * s) if norm_lr is not None else None,
                                 betas=tuple(opt_cfg.get("adamw_betas", (0.9, 0.95))))
    if fam == "hybrid":
        return get_muon_optimizer(model, lr=train_cfg.get("max_lr", 1e-3) * s, momentum=opt_cfg.get("momentum", 0.95),
                                  weight_decay=wd)
    if fam == "muon8bit_all":
        return Muon8bit(model.parameters(), lr=train_cfg.get("max_lr", 1e-3) * s, momentum=opt_cfg.get("momentum", 0.95),
                        weight_decay=wd)
    decay, no_decay = [], []
    for n, p in model.named_parameters():
        if p.requires_grad:
            (no_decay if (p.dim() < 2 or "norm" in n or "bias" in n) else decay).append(p)
    lr = train_cfg.get("max_lr", opt_cfg.get("adamw_lr", 3e-4)) * s
    on_cuda = next(model.parameters()).is_cuda
    if spec.use_8bit_optimizer:
        # reference: train_distributed.py:368-383 - AdamW8bit when bitsandbytes is there, else plain AdamW
        try:
            import bitsandbytes as bnb
            print("Using 8-bit AdamW (4x memory savings for optimizer states)")
            return bnb.optim.AdamW8bit([{"params": decay, "weight_decay": wd}, {"params": no_decay, "weight_decay": 0.0}],
                                       lr=lr, betas=tuple(opt_cfg.get("adamw_betas", (0.9, 0.95))), eps=1e-8)
        except ImportError:
            print("Warning: bitsandbytes not available, falling back to standard AdamW")
    return torch.optim.AdamW([{"params": decay, "weight_decay": wd}, {"params": no_decay, "weight_decay": 0.0}],
                             lr=lr, betas=tuple(opt_cfg.get("adamw_betas", (0.9, 0.95))), fused=on_cuda)


def _documents(tokenizer, max_examples):
    from ..data.dolma_dataset import _open_first_available
    ds = _open_first_available("train", True)
    if ds is None:
        return None

    def gen():
        for i, ex in enumerate(ds):
            if max_examples and i >= max_examples:
                return
            t = ex.get("text", "")
            if t:
                enc = tokenizer.encode(t, truncation=False)
                yield enc["input_ids"] if isinstance(enc, dict) else enc
    return gen()


class _SkipFirst:
    """An iterable that drops the first ``n`` batches of ``loader`` (resume: the batches consumed
    before the checkpoint are not replayed; the reference stores and restores ``data_idx`` for
    the same purpose, train.py:195, 811, 869)."""

    def __init__(self, loader, n: int):
        self.loader, self.n = loader, int(n)

    def __iter__(self):
        import itertools
        return itertools.islice(iter(self.loader), self.n, None)


def _make_loader(spec, cfg, data_cfg, batch, rank, world, skip_batches: int = 0):
    loader, kind = _make_loader_from_start(spec, cfg, data_cfg, batch, rank, world)
    return (_SkipFirst(loader, skip_batches) if skip_batches > 0 else loader), kind


def _make_loader_from_start(spec, cfg, data_cfg, batch, rank, world):
    from torch.utils.data import DataLoader
    mode = spec.data_mode
    tok = None
    if mode in ("auto", "streaming", "packed"):
        tok = TokenizerWrapper(data_cfg.get("tokenizer_name", "gpt2"), vocab_size=None, verbose=(rank == 0))
    if mode == "packed" or (mode == "auto" and spec.checkpoint_format == "C"):
        docs = _documents(tok, data_cfg.get("max_examples"))
        if docs is not None:
            ds = PackedDocumentDataset(docs, cfg.max_seq_len, tok.eos_token_id, cfg.n_pred_tokens)
            return DataLoader(ds, batch_size=batch), "packed"
    if mode in ("auto", "streaming"):
        ds = DolmaStreamingDataset(tok, cfg.max_seq_len, cfg.n_pred_tokens, "train", True, cfg.vocab_size,
                                   rank=rank, world_size=world)
        if ds.dataset is not None:
            return DataLoader(ds, batch_size=batch), "streaming"
    ds = SyntheticTokenDataset(cfg.vocab_size, cfg.max_seq_len, seed=1234, rank=rank, low=1)
    return DataLoader(ds, batch_size=batch), "synthetic"


def run_training(spec: RunSpec) -> Dict[str, Any]:
    mesh = pmesh.init_distributed(ep_size=1) if int(os.environ.get("WORLD_SIZE", "1")) > 1 else pmesh.Mesh(
        1, 0, spec.gpu or 0, 1, 1)
    rank, world = mesh.rank, mesh.world
    is_main = rank == 0
    use_cuda = torch.cuda.is_available()
    device = torch.device("cuda", mesh.local_rank if world > 1 else (spec.gpu or 0)) if use_cuda else torch.device("cpu")
    if use_cuda:
        torch.cuda.set_device(device)
    y = load_yaml(spec.config_path)
    train_cfg, opt_cfg, data_cfg = section(y, "training"), section(y, "optimizer"), section(y, "data")
    over = {}
    if spec.balanced_routing:
        over["moe_balanced_routing"] = True
    cfg: AdvancedMoEConfig = (model_config_strict(y, **over) if spec.strict_config
                              else model_config_tolerant(y, seq_len=spec.seq_len, **over))
    if spec.seq_len and spec.strict_config:
        cfg.max_seq_len = spec.seq_len
    if cfg.moe_implementation == "expert_parallel" and world > 1 and cfg.ep_size == 1:
        cfg.ep_size = math.gcd(world, cfg.n_experts)
    if cfg.ep_size > 1 and world > 1:
        mesh = pmesh.make_mesh(cfg.ep_size)
    torch.manual_seed(1234)                                    # identical initial weights on every rank
    model = MoETransformer(cfg, verbose=is_main)
    if cfg.ep_size > 1 and mesh.ep_group is not None:
        for m in model.modules():
            if hasattr(m, "expert_parallel_layer") and m.expert_parallel_layer is not None:
                m.expert_parallel_layer.process_group = mesh.ep_group
    wdtype = {"bf16": torch.bfloat16, "fp16": torch.float16, "fp32_autocast": torch.float32}[spec.weights]
    model = model.to(device).to(wdtype)
    if spec.grad_checkpoint:
        model.gradient_checkpointing_enable()
    start_step, tokens_seen, losses, data_idx = 0, 0, [], None
    resume = spec.resume or train_cfg.get("resume_from")
    if resume and not os.path.isdir(resume):
        _, ck = ckpt.load_model_state(model, resume, map_location=device)
        start_step = ck.get("step", ck.get("global_step", 0)) if isinstance(ck, dict) else 0
        tokens_seen = ck.get("total_tokens", ck.get("tokens_seen", 0)) if isinstance(ck, dict) else 0
        data_idx = ck.get("data_idx") if isinstance(ck, dict) else None
    if spec.reallocate:
        from tools.reallocate_experts import reallocate_model_experts
        reallocate_model_experts(model, entropy_threshold=spec.entropy_threshold, verbose=is_main)

    dp = None
    if spec.shard_params:
        # the reference's train_distributed.py regime: parameters sharded per block, AdamW on the shards
        from ..parallel.fsdp import FullyShardedDataParallel
        dp = FullyShardedDataParallel(model, lr=opt_cfg.get("adamw_lr", train_cfg.get("max_lr", 3e-4)) * spec.lr_scale,
                                      betas=tuple(opt_cfg.get("adamw_betas", (0.9, 0.95))),
                                      weight_decay=opt_cfg.get("weight_decay", train_cfg.get("weight_decay", 0.01)),
                                      cpu_offload=spec.cpu_offload)
        optimizer = dp.optimizer
        if is_main:
            print(f"parameter-sharded plan: {dp.param_bytes_per_rank() / 2**20:.1f} MiB of parameters per rank"
                  f"{' (host memory)' if spec.cpu_offload else ''}")
        if cfg.ep_size > 1 and any(getattr(p, "_kmoe_expert_parallel", False) for p in model.parameters()):
            # experts are already split over the expert-parallel group; their replicas form a second pool
            from ..parallel.zero import ParallelPlan, ShardedDataParallel
            experts = ShardedDataParallel(model, optimizer_kind="adamw", group=mesh.expert_dp_group,
                                          adamw_lr=opt_cfg.get("adamw_lr", 3e-4) * spec.lr_scale,
                                          weight_decay=opt_cfg.get("weight_decay", 0.01), expert_params=True,
                                          grad_scale=1.0 / cfg.ep_size, broadcast_from_rank0=False,
                                          transport="nccl" if use_cuda else "gloo")
            dp = ParallelPlan([dp, experts])
            optimizer = dp
    elif world > 1:
        from ..parallel.zero import ParallelPlan, ShardedDataParallel
        okind = "muon" if opt_cfg.get("type", "adamw") == "muon" else "adamw"
        pools = [ShardedDataParallel(model, optimizer_kind=okind, lr=opt_cfg.get("muon_lr", 1e-3) * spec.lr_scale,
                                     adamw_lr=opt_cfg.get("adamw_lr", 3e-4) * spec.lr_scale,
                                     momentum=opt_cfg.get("momentum", 0.95),
                                     weight_decay=opt_cfg.get("weight_decay", 0.01),
                                     newton_iters=opt_cfg.get("newton_iters", 5), transport=spec.transport)]
        if cfg.ep_size > 1 and any(getattr(p, "_kmoe_expert_parallel", False) for p in model.parameters()):
            pools.append(ShardedDataParallel(model, optimizer_kind="adamw", group=mesh.expert_dp_group,
                                             adamw_lr=opt_cfg.get("adamw_lr", 3e-4) * spec.lr_scale,
                                             weight_decay=opt_cfg.get("weight_decay", 0.01), expert_params=True,
                                             grad_scale=1.0 / cfg.ep_size, broadcast_from_rank0=False,
                                             transport="nccl" if use_cuda else "gloo"))
        dp = ParallelPlan(pools)
        optimizer = dp
    else:
        optimizer = _build_optimizer(spec, model, opt_cfg, train_cfg)
        if resume and not os.path.isdir(resume) and isinstance(ck, dict) and ck.get("optimizer_state_dict") is not None:
            try:
                optimizer.load_state_dict(ck["optimizer_state_dict"])
            except Exception as e:
                if is_main:
                    print(f"optimizer state not restored: {e}")

    batch = spec.batch_size or train_cfg["batch_size"]
    accum = spec.grad_accum or train_cfg["gradient_accumulation_steps"]
    tokens_per_step = batch * cfg.max_seq_len * world * accum
    total_steps = spec.steps or max(1, train_cfg["total_tokens"] // tokens_per_step)
    sched = None
    if spec.use_lr_schedule and not spec.constant_lr:
        max_lr = train_cfg["max_lr"] * spec.lr_scale
        sched = CosineScheduleWithWarmup(optimizer, min(train_cfg["warmup_steps"], max(total_steps - 1, 1)),
                                         total_steps, max_lr, max_lr * train_cfg["min_lr_ratio"],
                                         preserve_ratios=True)
        sched.current_step = start_step
    amp = torch.bfloat16 if (spec.weights == "fp32_autocast" and use_cuda) else None
    engine = TrainEngine(model, optimizer, sched, train_cfg["gradient_clip_norm"], accum, amp, dp, device)
    engine.global_step, engine.tokens_seen = start_step, tokens_seen
    if spec.use_8bit_optimizer and dp is not None and is_main:
        print("--8bit-optimizer: ignored under the sharded plans (optimizer state is already split over the "
              f"{world} ranks and kept in fp32 by their fused update kernels)")
    twd = spec.token_weight_decay or (train_cfg.get("token_weight_decay", 0.0)
                                      if train_cfg.get("use_token_weights", False) else 0.0)
    if twd > 0:
        pos = torch.arange(cfg.max_seq_len, dtype=torch.float32, device=device)
        w = 1.0 + twd * pos / cfg.max_seq_len
        engine.token_weights = w / w.mean()
        if is_main:
            print(f"  Token weighting: enabled (decay={twd})")
    if resume and os.path.isdir(resume) and not os.path.exists(os.path.join(resume, "model.pt")):
        # a checkpoint root: continue from the newest directory that every rank finished writing
        found = ckpt.latest_complete_checkpoint(resume, world)
        if found is None:
            raise FileNotFoundError(f"no complete checkpoint under {resume}")
        resume = found
    if resume and os.path.isdir(resume):
        if spec.shard_params:
            st = ckpt.load_param_sharded(resume, dp, rank, ep_rank=mesh.ep_rank, ep_size=mesh.ep)
        else:
            st = (ckpt.load_sharded(resume, model, dp, rank, device, ep_rank=mesh.ep_rank, ep_size=mesh.ep)
                  if dp is not None
                  else ckpt.load_format_c(resume, model, optimizer, device))
        engine.global_step = start_step = st.get("step", 0)
        engine.tokens_seen = st.get("tokens_seen", 0)
        data_idx = st.get("data_idx")
        if sched is not None:
            if st.get("lr_scheduler") is not None:
                sched.load_state_dict(st["lr_scheduler"])
            sched.current_step = start_step        # warm-up and cosine phase continue, they do not restart
            sched.apply()
    elif sched is not None and start_step:
        sched.apply()
    # one loader batch feeds one optimizer step; a checkpoint from before ``data_idx`` existed
    # (or one that stored 0) falls back to the step count
    consumed = data_idx if data_idx else start_step
    loader, data_kind = _make_loader(spec, cfg, data_cfg, batch * accum, rank, world, skip_batches=consumed)
    it = iter(PinnedPrefetcher(loader, depth=4, pin=use_cuda))
    cdir = spec.checkpoint_dir or train_cfg["checkpoint_dir"]
    if spec.checkpoint_format == "B":
        cdir = os.path.join(cdir, os.path.splitext(os.path.basename(spec.config_path))[0])
    save_every = spec.save_interval if spec.save_interval is not None else train_cfg["save_interval"]
    wb = y.get("wandb") or {}                  # the YAML's ``wandb:`` section: enabled / project / entity / run_name
    hf = y.get("huggingface") or {}
    logger = MetricLogger(spec.jsonl, spec.wandb or bool(wb.get("enabled", False)) or bool(hf.get("use_wandb", False)),
                          wb.get("project", spec.wandb_project), spec.wandb_run or wb.get("run_name"), y,
                          rank=rank, entity=wb.get("entity"))
    timer = PhaseTimer(enabled=spec.profile, device=device)
    if spec.profile:
        engine.timer = timer                   # forward / backward / optimizer next to data / step
    watch = None
    if spec.debug:
        from ..utils.fault import NormWatch, format_flow_report, gradient_flow_report
        watch = NormWatch(model)
        if is_main:
            print(f"DEBUG MODE: diagnostics every {spec.debug_interval} steps; gradient statistics are summed "
                  f"over the {world} rank(s) with one all-reduce")

        def _flow(m):
            # first step and then every debug_interval-th: which parameter groups received gradients
            if engine.global_step == start_step or (engine.global_step + 1) % spec.debug_interval == 0:
                rep = gradient_flow_report(m)
                if is_main:
                    print(format_flow_report(rep, world), flush=True)
        engine.before_update.append(_flow)
    if spec.profile and os.environ.get("KMOE_NVTX_BLOCKS", "0") == "1":
        from ..utils.profiling import annotate_blocks
        annotate_blocks(model)                 # per-layer ranges for a timeline capture
    dog = StepWatchdog(spec.step_deadline_s, lambda idle: print(f"[watchdog] no step for {idle:.0f}s on rank {rank}",
                                                                flush=True)).start() if spec.step_deadline_s > 0 else None
    if spec.compile and is_main:
        print("--compile: accepted for command-line compatibility and not used (the hot operations are this "
              "library's fused CUDA kernels; nothing is traced)")
    if is_main:
        print(f"training: {total_steps} steps, {tokens_per_step:,} tokens/step, data={data_kind}, world={world}, "
              f"ep={cfg.ep_size}, weights={spec.weights}")

    writer = ckpt.AsyncCheckpointWriter() if spec.async_checkpoint else None

    def save(step: int, suffix: Optional[str] = None):
        state = {"step": step, "tokens_seen": engine.tokens_seen, "config_path": spec.config_path,
                 "data_idx": batches_consumed,
                 "lr_scheduler": sched.state_dict() if sched is not None else None}
        if spec.shard_params:
            ckpt.save_param_sharded(cdir, step, dp, state, rank, writer=writer, ep_rank=mesh.ep_rank, ep_size=mesh.ep)
        elif dp is not None:
            ckpt.save_sharded(cdir, step, model, dp, state, rank, writer=writer, world=world,
                              ep_rank=mesh.ep_rank, ep_size=mesh.ep)
        elif spec.checkpoint_format == "C":
            ckpt.save_format_c(cdir, step, model, optimizer, state)
        else:
            ckpt.save_format_b(os.path.join(cdir, ckpt.format_b_name(step, suffix)), model, optimizer, step, 0,
                               batches_consumed, losses, engine.tokens_seen, spec.config_path)

    injector = _fault_from_env(spec.transport)
    log_every = train_cfg["log_interval"]
    t_last, tok_last = time.time(), engine.tokens_seen
    last_stats = None
    batches_consumed = consumed
    with InterruptGuard() as guard:
        step = start_step
        while step < total_steps:
            with timer.phase("data"):
                b = next(it)
            batches_consumed += 1
            am = None
            if spec.document_mask and "doc_ids" in b:
                # boundaries instead of a dense (B, 1, S, S) mask: attention stays on the flash kernels
                am = PackedDocs(doc_ids=b["doc_ids"].to(device))
            with timer.phase("step"):
                if am is not None:
                    last_stats = engine.step(b["input_ids"], b.get("labels"), attention_mask=am)
                else:
                    last_stats = engine.step(b["input_ids"], b.get("labels"))
            step += 1
            if dog is not None:
                dog.beat()
            if injector is not None:
                injector(rank, step)           # host-side failure between steps (tests of restart / resume)
            if step % log_every == 0 or step == total_steps:
                lv = last_stats.loss_value()
                losses.append(lv)
                now = time.time()
                tps = (engine.tokens_seen - tok_last) * world / max(now - t_last, 1e-9)
                t_last, tok_last = now, engine.tokens_seen
                rec = {"loss": lv, "lm_loss": float(last_stats.lm_loss), "lr": optimizer.param_groups[0]["lr"],
                       "aux_loss": float(last_stats.aux_loss) if torch.is_tensor(last_stats.aux_loss) else 0.0,
                       "grad_norm": float(last_stats.grad_norm) if last_stats.grad_norm is not None else None,
                       "tokens_seen": engine.tokens_seen * world, "tokens_per_sec": tps}
                if use_cuda:
                    rec["mem_allocated_gb"] = torch.cuda.memory_allocated() / 2**30
                    rec["mem_reserved_gb"] = torch.cuda.memory_reserved() / 2**30
                for k, v in (last_stats.per_head or {}).items():
                    rec[f"mt_{k}"] = float(v)
                if spec.profile:
                    rec.update({f"time_{k}_ms": v for k, v in timer.summary(reduce_max=world > 1).items()})
                    timer.reset()
                logger.log(rec, step=step)
                if is_main:
                    print(f"Step {step}/{total_steps} | Loss: {lv:.4f} | LR: {rec['lr']:.2e} | Tok/s: {tps:,.0f}", flush=True)
            if spec.debug and step % spec.debug_interval == 0:
                stats, collapsed, summary = check_router_collapse(model, entropy_threshold=spec.collapse_entropy_threshold)
                stuck = watch.stuck(model) if watch is not None else []
                if is_main:
                    print(f"  [debug step {step}] router: {summary}; "
                          f"norm weights still at their initial value: {len(stuck)}"
                          + (f" (e.g. {stuck[0]})" if stuck else ""), flush=True)
            if spec.collapse_check_interval and step % spec.collapse_check_interval == 0:
                stats, collapsed, summary = check_router_collapse(model, entropy_threshold=spec.collapse_entropy_threshold)
                if stats:
                    logger.log({"router/avg_entropy": sum(s["entropy"] for s in stats.values()) / len(stats),
                                "router/max_usage": max(s["max_usage"] for s in stats.values()),
                                "router/collapsed_layers": len(collapsed)}, step=step)
                if is_main and collapsed:
                    print(f"  [router] {summary}")
            if save_every and step % save_every == 0 and step < total_steps:
                save(step)
            if guard.requested:
                if is_main:
                    print(f"signal {guard.signum}: saving checkpoint at step {step} and stopping")
                save(step, "interrupted")
                break
        else:
            save(step, "final")
    if writer is not None:
        writer.wait()                          # the last save must be on disk before the job reports success
    if dog is not None:
        dog.stop()
    logger.close()
    if use_cuda:
        from ..ops import cuda_ops
        cuda_ops.check_status()
    out = {"steps": step, "final_loss": losses[-1] if losses else None, "tokens_seen": engine.tokens_seen * world,
           "checkpoint_dir": cdir}
    if world > 1:
        pmesh.destroy()
    return out


def fault_injection_refusal(env, transport: Optional[str]) -> Optional[str]:
    """Why host-side fault injection may not run on GPUs with this environment (None = it may).  A rank that
    leaves while its memory is bound to an NVLink multicast object can fault its peers' GPUs."""
    if env.get("NCCL_NVLS_ENABLE", "1") != "0":
        return "KMOE_FAULT_INJECT on GPUs needs NCCL_NVLS_ENABLE=0 (plain peer loads and stores only)"
    if transport not in ("nccl", "gloo") and env.get("TORCH_SYMM_MEM_DISABLE_MULTICAST", "0") != "1":
        return ("KMOE_FAULT_INJECT on GPUs needs TORCH_SYMM_MEM_DISABLE_MULTICAST=1 (or --transport nccl): the "
                "symmetric-memory rendezvous of the p2p transport otherwise binds the buffers to a multicast object")
    return None


def _fault_from_env(transport: Optional[str] = None):
    """``KMOE_FAULT_INJECT=rank:step:kind`` (kind = raise | exit | stall) makes that rank fail on the host
    right after that step, with no kernel or collective of its own in flight.  With ``KMOE_FAULT_ONCE=<file>``
    the failure happens only while the file does not exist (it is created first), so a restarted job runs
    through.  On GPUs nothing of the job may be bound to an NVLink multicast object: ``NCCL_NVLS_ENABLE=0`` (NCCL;
    this library's kernels obey it too) and either ``TORCH_SYMM_MEM_DISABLE_MULTICAST=1`` (torch's symmetric-memory
    allocator, which backs the ``p2p`` transport's buffers, otherwise creates and binds one at rendezvous) or a
    transport that allocates no symmetric memory (``transport`` = ``nccl`` / ``gloo``)."""
    spec = os.environ.get("KMOE_FAULT_INJECT")
    if not spec:
        return None
    if torch.cuda.is_available():
        refusal = fault_injection_refusal(os.environ, transport)
        if refusal:
            raise RuntimeError(refusal)
    from ..utils.fault import FaultInjector
    r, s_, kind = (spec.split(":") + ["raise"])[:3]
    inj = FaultInjector(int(r), int(s_), kind)
    once = os.environ.get("KMOE_FAULT_ONCE")

    def fire(rank: int, step: int) -> None:
        if rank != inj.rank or step != inj.step:
            return
        if once:
            if os.path.exists(once):
                return
            with open(once, "w") as f:
                f.write(f"rank {rank} step {step}\n")
        if torch.cuda.is_available():
            torch.cuda.synchronize()           # nothing of this rank is in flight when it leaves
        inj.maybe_fail(rank, step)

    return fire
