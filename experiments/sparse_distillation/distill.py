"""Sparse distillation: replace the dense FFNs of a pretrained transformer by MoE layers trained
to reproduce the dense FFN's output (counterpart of the reference's
``Experiments/sparse_distillation/distill.py``).

Training modes of :class:`SparseDistillationTrainer`:
* ``distill``            - all layers in parallel on real batches (teacher forward with hooks).
* ``sequential_layers``  - one layer at a time, the others kept off the training device.
* ``data_free``          - inputs are random unit vectors scaled by sqrt(d); no dataset needed.
* ``supervised_routing`` - k-means (k-means++ init, spherical option) on dense-FFN outputs, then the
  router is trained with KL against the cluster assignment before / while experts train.
* ``empirical_routing``  - two passes: evaluate every expert on every token (loss or, with
  ``gradient_routing``, error magnitude), turn that into balanced top-k targets blended with the
  uniform distribution on a curriculum, train the router on those targets with the expert loss
  detached from it.
* ``dynamic_experts``    - experts of unequal width, periodically grown / shrunk by tracked loss.
Loss: MSE + lambda (1 - cos) + load-balance + z-loss.
"""
from __future__ import annotations

import json
import math
import os
import sys
from dataclasses import asdict, dataclass
from typing import Dict, List, Optional, Tuple, Union

import torch
import torch.nn as nn
import torch.nn.functional as F

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))))

from kolmogorov_moe_architecture_b200.config import AdvancedMoEConfig  # noqa: E402
from kolmogorov_moe_architecture_b200.models.moe import (ExpertChoiceRouter, GroupedExperts,  # noqa: E402
                                                         GroupedExpertsExpertChoice, Router)

from .dynamic_experts import DynamicExpertLayer, DynamicExpertTracker, reallocate_expert_layer  # noqa: E402
from .hooks import FFNActivationCache, find_ffn_modules  # noqa: E402


@dataclass
class DistillationConfig:
    n_experts: int = 16
    moe_top_k: int = 2
    moe_capacity_factor: float = 1.25
    moe_routing: str = "token_choice"
    d_ff_expert: Optional[Union[int, float]] = None     # int = width, float = fraction of the dense width
    layer_config_path: Optional[str] = None             # per-layer {n_experts, d_ff_expert, top_k} JSON
    learning_rate: float = 1e-4
    weight_decay: float = 0.01
    warmup_steps: int = 100
    max_grad_norm: float = 1.0
    use_cosine_loss: bool = True
    cosine_loss_weight: float = 0.1
    use_load_balancing: bool = True
    load_balancing_weight: float = 0.01
    use_z_loss: bool = True
    z_loss_weight: float = 0.001
    init_from_dense: bool = True
    sequential_layers: bool = False
    dynamic_experts: bool = False
    reallocate_every_n_steps: int = 500
    growth_factor: float = 1.25
    shrink_factor: float = 0.8
    min_d_ff: int = 256
    max_d_ff: int = 8192
    top_k_grow: int = 2
    top_k_shrink: int = 2
    log_interval: int = 100
    data_free: bool = True
    data_free_batch_size: int = 4
    data_free_seq_len: int = 512
    data_free_steps: int = 1000
    use_compile: bool = False
    supervised_routing: bool = True
    cluster_samples: int = 10000
    cluster_batch_size: int = 32
    router_train_steps: int = 2000
    empirical_routing: bool = False
    empirical_eval_interval: int = 10
    empirical_temperature: float = 0.1
    empirical_entropy_weight: float = 0.01
    curriculum_routing: bool = True
    curriculum_warmup_steps: int = 5000
    curriculum_initial_balance: float = 0.9
    curriculum_final_balance: float = 0.3
    target_max_prob: float = 0.25
    target_temperature_schedule: bool = True
    target_initial_temperature: float = 1.0
    target_final_temperature: float = 0.1
    detach_router_from_expert_loss: bool = True
    router_loss_weight: float = 1.0
    use_expert_bias: bool = True
    gradient_routing: bool = True
    gradient_routing_fast: bool = True
    router_mlp: bool = False
    router_hidden_dim: int = 256
    router_n_layers: int = 2


class MLPRouter(nn.Module):
    """Router with ``n_layers`` linear layers (with biases) and GELU between them; parameters ``mlp.{0,2,...}``
    (reference: distill.py:212-243)."""

    def __init__(self, d_model: int, n_experts: int, hidden_dim: int = 256, n_layers: int = 2):
        super().__init__()
        self.d_model, self.n_experts = d_model, n_experts
        dims = [d_model] + [hidden_dim] * (n_layers - 1)
        layers: List[nn.Module] = []
        for a, b in zip(dims[:-1], dims[1:]):
            layers += [nn.Linear(a, b), nn.GELU()]
        layers.append(nn.Linear(dims[-1], n_experts))
        self.mlp = nn.Sequential(*layers)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        return self.mlp(x)


def _dense_ffn_weights(ffn: nn.Module):
    """(gate, up, down) Linear weights of a SwiGLU-style FFN under the common naming schemes."""
    for names in (("gate_proj", "up_proj", "down_proj"), ("w1", "w2", "w3"), ("w1", "w3", "w2")):
        if all(hasattr(ffn, n) and hasattr(getattr(ffn, n), "weight") for n in names):
            g, u, d = (getattr(ffn, n).weight for n in names)
            if g.shape == u.shape and d.shape == (g.shape[1], g.shape[0]):
                return g, u, d
    return None


class MoEDistillationLayer(nn.Module):
    """Router (+ optional learnable per-expert logit bias) and stacked experts."""

    def __init__(self, d_model: int, d_ff_expert: int = None, cfg=None, n_experts=None, top_k=None, *,
                 d_ff: int = None, capacity_factor: float = None, routing_type: str = None, mlp_router: bool = None,
                 router_hidden_dim: int = None, router_n_layers: int = None, use_expert_bias: bool = None):
        """``MoEDistillationLayer(d_model, d_ff_expert, config[, n_experts, top_k])``, or with the settings spelled
        out as in the reference (distill.py:253): ``MoEDistillationLayer(d_model, d_ff, n_experts,
        capacity_factor=..., routing_type=..., mlp_router=..., router_hidden_dim=..., router_n_layers=...,
        use_expert_bias=...)`` - a configuration is then made from the defaults and these values."""
        super().__init__()
        if isinstance(cfg, int):                             # third positional is the expert count
            n_experts, cfg = cfg, None
        d_ff_expert = d_ff if d_ff_expert is None else d_ff_expert
        if cfg is None:
            cfg = DistillationConfig(moe_routing=routing_type or "expert_choice")
        over = {k: v for k, v in dict(moe_capacity_factor=capacity_factor, moe_routing=routing_type,
                                      router_mlp=mlp_router, router_hidden_dim=router_hidden_dim,
                                      router_n_layers=router_n_layers, use_expert_bias=use_expert_bias).items()
                if v is not None}
        if over:
            import dataclasses
            cfg = dataclasses.replace(cfg, **over)
        self.cfg, self.d_model, self.d_ff = cfg, d_model, d_ff_expert
        self.n_experts, self.top_k = n_experts or cfg.n_experts, top_k or cfg.moe_top_k
        self.routing = cfg.moe_routing
        # The router is the model family's own: a d -> 128 -> E network without biases (``Router`` for token choice,
        # ``ExpertChoiceRouter`` for expert choice; parameters ``router.router.{0,2}.weight``, the keys of the
        # reference's distillation checkpoints), or the deeper ``MLPRouter`` when asked for.  Only its logits are
        # used here: selection, bias and weights are this layer's business.
        if cfg.router_mlp:
            self.router = MLPRouter(d_model, self.n_experts, cfg.router_hidden_dim, cfg.router_n_layers)
        else:
            mini = AdvancedMoEConfig(d_model=d_model, n_experts=self.n_experts, d_ff_expert=d_ff_expert,
                                     moe_capacity_factor=cfg.moe_capacity_factor, moe_top_k=min(self.top_k, self.n_experts))
            self.router = ExpertChoiceRouter(mini) if self.routing == "expert_choice" else Router(mini)
        self.expert_bias = nn.Parameter(torch.zeros(self.n_experts)) if cfg.use_expert_bias else None
        if self.routing == "expert_choice":
            self.experts = GroupedExpertsExpertChoice(self.n_experts, d_model, d_ff_expert)
        else:
            self.experts = GroupedExperts(self.n_experts, d_model, d_ff_expert)
        self._last_router_logits: Optional[torch.Tensor] = None
        self._last_expert_counts: Optional[torch.Tensor] = None
        # token choice under a per-expert capacity of T k / E (greedy, slot by slot): keeps every expert in use
        # while fine-tuning (reference: finetune_eval.py:812-826 switches it on, moe.py:353-421 defines it)
        self.balanced_routing = False

    def router_net(self) -> nn.Module:
        """The network that maps hidden states to expert logits."""
        return self.router if isinstance(self.router, MLPRouter) else self.router.router

    def get_router_logits(self, x: torch.Tensor) -> torch.Tensor:
        logits = self.router_net()(x)
        return logits + self.expert_bias if self.expert_bias is not None else logits

    def forward(self, x: torch.Tensor, return_aux: bool = False):
        shape = x.shape
        x3 = x if x.dim() == 3 else x.unsqueeze(0)
        rin = x3.detach() if (self.cfg.detach_router_from_expert_loss and self.cfg.empirical_routing) else x3
        logits = self.get_router_logits(rin)
        self._last_router_logits = logits
        if self.routing == "expert_choice":
            S = x3.shape[1]
            cap = min(S, int(math.ceil(S * self.cfg.moe_capacity_factor / self.n_experts)))
            probs = F.softmax(logits.transpose(1, 2), dim=-1)
            w, tok = torch.topk(probs, cap, dim=-1)
            w = w / (w.sum(-1, keepdim=True) + 1e-9)
            out = self.experts(x3, w, tok)
            self._last_expert_counts = torch.full((self.n_experts,), cap * x3.shape[0], device=x.device)
        else:
            probs = F.softmax(logits, dim=-1)
            if self.balanced_routing:
                from kolmogorov_moe_architecture_b200 import ops
                idx = ops.balanced_assign(probs.reshape(-1, self.n_experts).float(), self.top_k).view(
                    *probs.shape[:-1], self.top_k)
                w = probs.gather(-1, idx)
            else:
                w, idx = torch.topk(probs, self.top_k, dim=-1)
            w = w / w.sum(-1, keepdim=True)
            flat = x3.reshape(-1, self.d_model)
            out = self.experts(flat, idx.reshape(-1, self.top_k), w.reshape(-1, self.top_k)).view_as(x3)
            self._last_expert_counts = torch.bincount(idx.reshape(-1), minlength=self.n_experts)
        out = out.view(shape)
        return (out, {"router_logits": logits, "expert_counts": self._last_expert_counts}) if return_aux else out

    def expert_outputs_all(self, x: torch.Tensor) -> torch.Tensor:
        """Every expert on every token: (E, T, d).  Used by empirical routing."""
        flat = x.reshape(-1, self.d_model)
        e = self.experts
        h = F.silu(torch.einsum("td,edf->etf", flat, e.w1)) * torch.einsum("td,edf->etf", flat, e.w2)
        return torch.einsum("etf,efd->etd", h, e.w3)

    @torch.no_grad()
    def init_from_dense_ffn(self, dense_ffn: nn.Module, noise: float = 0.01):
        """Each expert takes a contiguous slice of the dense hidden units (wrapping around when the
        experts together are wider than the dense layer), plus 1 % relative noise to break symmetry."""
        w = _dense_ffn_weights(dense_ffn)
        if w is None:
            return False
        g, u, d = (t.detach().float() for t in w)            # (F, d), (F, d), (d, F)
        Fd = g.shape[0]
        for e in range(self.n_experts):
            cols = (torch.arange(self.d_ff) + e * self.d_ff) % Fd
            for dst, src in ((self.experts.w1, g[cols].t()), (self.experts.w2, u[cols].t()), (self.experts.w3, d[:, cols].t())):
                s = src.to(dst.dtype).to(dst.device)
                dst[e].copy_(s + noise * s.std() * torch.randn_like(s))
        return True


def print_layer_routing_stats(moe_layer: MoEDistillationLayer, layer_idx: int, prefix: str = ""):
    c = moe_layer._last_expert_counts
    if c is None:
        return None
    u = c.float() / c.sum().clamp(min=1)
    ent = float(-(u * torch.log(u + 1e-10)).sum() / math.log(max(len(u), 2)))
    print(f"{prefix}layer {layer_idx}: usage entropy {ent:.3f}, max {float(u.max()):.3f}, dead {int((u == 0).sum())}")
    return ent


def kmeans(x: torch.Tensor, k: int, iters: int = 25, spherical: bool = False, seed: int = 0) -> Tuple[torch.Tensor, torch.Tensor]:
    """k-means with k-means++ seeding, pure torch. Returns (assignments, centroids)."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    x = F.normalize(x.float(), dim=-1) if spherical else x.float()
    n = x.shape[0]
    cent = x[torch.randint(0, n, (1,), generator=g)].clone()
    for _ in range(1, k):
        d2 = torch.cdist(x, cent).pow(2).min(dim=1).values
        p = (d2 / d2.sum().clamp(min=1e-12)).cpu()
        cent = torch.cat([cent, x[torch.multinomial(p, 1, generator=g)].to(x.device)])
    assign = torch.zeros(n, dtype=torch.long, device=x.device)
    for _ in range(iters):
        assign = torch.cdist(x, cent).argmin(dim=1)
        for j in range(k):
            m = assign == j
            if m.any():
                cent[j] = x[m].mean(0)
                if spherical:
                    cent[j] = F.normalize(cent[j], dim=0)
    return assign, cent


def cluster_quality(x: torch.Tensor, assign: torch.Tensor, cent: torch.Tensor) -> Dict[str, float]:
    """Calinski-Harabasz index, a centroid-based silhouette estimate and the size-entropy balance."""
    k, n = cent.shape[0], x.shape[0]
    x = x.float()
    sizes = torch.bincount(assign, minlength=k).float()
    mean = x.mean(0)
    between = (sizes[:, None] * (cent - mean).pow(2)).sum()
    within = (x - cent[assign]).pow(2).sum()
    ch = float((between / max(k - 1, 1)) / (within / max(n - k, 1)).clamp(min=1e-12))
    d = torch.cdist(x, cent)
    a = d.gather(1, assign[:, None]).squeeze(1)
    d.scatter_(1, assign[:, None], float("inf"))
    b = d.min(dim=1).values
    sil = float(((b - a) / torch.maximum(a, b).clamp(min=1e-12)).mean())
    p = sizes / n
    bal = float(-(p * torch.log(p + 1e-10)).sum() / math.log(max(k, 2)))
    return {"calinski_harabasz": ch, "silhouette": sil, "balance": bal}


def balanced_topk_targets(scores: torch.Tensor, k: int, max_prob: float, temperature: float, balance: float):
    """scores (T, E), lower is better -> routing target distribution: softmax(-score / T), clipped to
    ``max_prob`` and renormalised, then blended with uniform by ``balance``."""
    t = F.softmax(-scores / max(temperature, 1e-6), dim=-1)
    t = t.clamp(max=max_prob)
    t = t / t.sum(-1, keepdim=True)
    E = scores.shape[-1]
    return (1 - balance) * t + balance / E


def checkpoint_layers(ck: Dict) -> Dict[str, Dict[str, torch.Tensor]]:
    """Per-layer state dicts of a distillation checkpoint: this file's layout (``{"layers": {i: state}}``) or the
    reference's (``{"moe_layers": {"<i>.<key>": tensor}}``, distill.py:2924-2950)."""
    if "layers" in ck:
        return {str(k): v for k, v in ck["layers"].items()}
    out: Dict[str, Dict[str, torch.Tensor]] = {}
    for key, t in ck["moe_layers"].items():
        i, rest = key.split(".", 1)
        out.setdefault(i, {})[rest] = t
    return out


def checkpoint_config(ck: Dict) -> "DistillationConfig":
    """The configuration stored in a checkpoint: a dict of fields (this file's layout) or the object itself."""
    c = ck.get("config")
    if isinstance(c, dict):
        known = {f for f in DistillationConfig.__dataclass_fields__}
        return DistillationConfig(**{k: v for k, v in c.items() if k in known})
    return c if c is not None else DistillationConfig()


def load_layer_state(layer: nn.Module, state: Dict[str, torch.Tensor]) -> None:
    """Load one layer.  Keys of a helper module the reference keeps beside an MLP router (``_base_router.*``, its
    routing logic; unused weights) are ignored; everything else must match."""
    state = {k: v for k, v in state.items() if not k.startswith("_base_router.")}
    layer.load_state_dict(state)


def _ids_of_batch(b) -> torch.Tensor:
    """Token ids of a batch given as a tensor, a tuple whose first entry is one, or a dict with ``input_ids``."""
    if isinstance(b, dict):
        return b.get("input_ids", b.get("tokens"))
    return b[0] if isinstance(b, (list, tuple)) else b


class SparseDistillationTrainer:
    def __init__(self, model: nn.Module = None, config: DistillationConfig = None, device: str = "cpu",
                 dense_model: nn.Module = None, layer_filter=None):
        model = dense_model if model is None else model          # the reference's keyword for the teacher
        config = DistillationConfig() if config is None else config
        self.model, self.cfg, self.device = model, config, torch.device(device)
        self.ffn = find_ffn_modules(model, layer_filter=layer_filter)
        assert self.ffn, "no FFN modules found in the model"
        self.d_model, self.d_ff_dense, self.dtype = self._infer_dimensions()
        self.layer_cfg = json.load(open(config.layer_config_path)) if config.layer_config_path else {}
        if isinstance(self.layer_cfg.get("layers"), dict):      # file written by generate_config.compute_layer_config
            self.layer_cfg = self.layer_cfg["layers"]
        self.moe_layers = nn.ModuleDict()
        self._create_moe_layers()
        self.optimizers: Dict[int, torch.optim.Optimizer] = {}
        self.step_count = 0

    # ------------------------------------------------------------------ set-up
    def _infer_dimensions(self):
        w = _dense_ffn_weights(self.ffn[0][1])
        if w is not None:
            return w[0].shape[1], w[0].shape[0], w[0].dtype
        lin = [m for m in self.ffn[0][1].modules() if isinstance(m, nn.Linear)]
        return lin[0].in_features, lin[0].out_features, lin[0].weight.dtype

    def _compute_expert_dim(self, layer_idx: int) -> int:
        lc = self.layer_cfg.get(str(layer_idx), {})
        v = lc.get("d_ff_expert", self.cfg.d_ff_expert)
        if v is None:
            v = max(8, self.d_ff_dense // max(1, self.cfg.n_experts // self.cfg.moe_top_k))
        elif isinstance(v, float) and v <= 4.0:
            v = int(self.d_ff_dense * v)
        return max(8, int(v) // 8 * 8)

    def _create_moe_layers(self):
        for i, (_, dense) in enumerate(self.ffn):
            lc = self.layer_cfg.get(str(i), {})
            layer = MoEDistillationLayer(self.d_model, self._compute_expert_dim(i), self.cfg, lc.get("n_experts"),
                                         lc.get("top_k"))
            if self.cfg.init_from_dense:
                layer.init_from_dense_ffn(dense)
            self.moe_layers[str(i)] = layer

    def _get_optimizer(self, i: int):
        if i not in self.optimizers:
            self.optimizers[i] = torch.optim.AdamW(self.moe_layers[str(i)].parameters(), lr=self.cfg.learning_rate,
                                                   weight_decay=self.cfg.weight_decay)
        return self.optimizers[i]

    def get_moe_layers(self) -> nn.ModuleDict:
        return self.moe_layers

    # ------------------------------------------------------------------ losses
    @staticmethod
    def compute_load_balancing_loss(router_logits: torch.Tensor, expert_counts: torch.Tensor) -> torch.Tensor:
        logits, counts = router_logits, expert_counts
        E = logits.shape[-1]
        P = F.softmax(logits.reshape(-1, E).float(), -1).mean(0)
        f = counts.float() / counts.sum().clamp(min=1)
        return E * (f * P).sum()

    @staticmethod
    def compute_z_loss(router_logits: torch.Tensor) -> torch.Tensor:
        return torch.logsumexp(router_logits.float(), dim=-1).pow(2).mean()

    def compute_loss(self, moe_output: torch.Tensor, target: torch.Tensor, aux_info: Optional[Dict] = None,
                     return_metrics: bool = False):
        """MSE (+ cosine, load-balance and z terms as configured) of the MoE output against the dense FFN's.
        Returns the loss, or (loss, {"mse", "cos", "lb", "z"}) with ``return_metrics``."""
        student, teacher, aux = moe_output, target, aux_info
        have_aux = aux is not None and aux.get("router_logits") is not None
        mse = F.mse_loss(student.float(), teacher.float())
        loss, parts = mse, {"mse": float(mse.detach())}
        if self.cfg.use_cosine_loss:
            cos = 1 - F.cosine_similarity(student.float().reshape(-1, student.shape[-1]),
                                          teacher.float().reshape(-1, teacher.shape[-1]), dim=-1).mean()
            loss = loss + self.cfg.cosine_loss_weight * cos
            parts["cos"] = float(cos.detach())
        if have_aux and self.cfg.use_load_balancing and self.cfg.moe_routing == "token_choice":
            lb = self.compute_load_balancing_loss(aux["router_logits"], aux["expert_counts"])
            loss = loss + self.cfg.load_balancing_weight * lb
            parts["lb"] = float(lb.detach())
        if have_aux and self.cfg.use_z_loss:
            z = self.compute_z_loss(aux["router_logits"])
            loss = loss + self.cfg.z_loss_weight * z
            parts["z"] = float(z.detach())
        return (loss, parts) if return_metrics else loss

    def train_step(self, i=None, x: torch.Tensor = None, target: torch.Tensor = None, return_metrics: bool = False,
                   activations=None):
        """One update of layer ``i`` on (FFN input, FFN output): returns the loss parts of that layer.  In the
        reference's form, ``train_step(activations)`` with ``{layer: FFNActivation}`` from a forward pass of the
        dense model, every layer in the dict gets one update and the result is ``{layer: loss}`` (the parts
        instead of the loss with ``return_metrics``)."""
        i = activations if i is None else i
        if isinstance(i, dict):
            out = {}
            for k, act in i.items():
                parts = self.train_step(int(k), act.input, act.output)
                out[int(k)] = parts if return_metrics else parts["loss"]
            self.step_count += 1
            return out
        layer = self.moe_layers[str(i)].to(self.device).train()
        opt = self._get_optimizer(i)
        out, aux = layer(x.to(self.device), return_aux=True)
        loss, parts = self.compute_loss(out, target.to(self.device), aux, return_metrics=True)
        opt.zero_grad(set_to_none=True)
        loss.backward()
        torch.nn.utils.clip_grad_norm_(layer.parameters(), self.cfg.max_grad_norm)
        lr = self.cfg.learning_rate * min(1.0, (self.step_count + 1) / max(self.cfg.warmup_steps, 1))
        for g in opt.param_groups:
            g["lr"] = lr
        opt.step()
        parts["loss"] = float(loss.detach())
        return parts

    # ------------------------------------------------------------------- modes
    def distill(self, batches=None, steps: Optional[int] = None, epochs: int = 1, max_steps: Optional[int] = None,
                dataloader=None) -> Dict[int, List[float]]:
        """Dispatch on the configuration.  ``batches`` (or ``dataloader``, the reference's name for it): iterable of
        input-id tensors or of dicts with ``input_ids``, walked ``epochs`` times in the real-data modes;
        ``steps`` / ``max_steps`` bound the number of updates (reference: distill.py:929-1094)."""
        batches = dataloader if batches is None else batches
        steps = max_steps if steps is None else steps
        if batches is not None and epochs > 1:
            once = list(batches)
            batches = [b for _ in range(epochs) for b in once]
        if batches is not None:
            batches = [_ids_of_batch(b) for b in batches]
        if self.cfg.dynamic_experts:
            return self._distill_dynamic(steps or self.cfg.data_free_steps)
        if self.cfg.empirical_routing:
            return self._distill_empirical_routing(steps or self.cfg.data_free_steps)
        if self.cfg.data_free or batches is None:
            return self._distill_data_free(steps or self.cfg.data_free_steps)
        if self.cfg.sequential_layers:
            return self._distill_sequential(batches, steps)
        hist: Dict[int, List[float]] = {i: [] for i in range(len(self.ffn))}
        self.model.eval()
        for n, ids in enumerate(batches):
            if steps is not None and n >= steps:
                break
            with torch.no_grad(), FFNActivationCache(self.model) as cache:
                self.model(ids.to(next(self.model.parameters()).device))
            for i in range(len(self.ffn)):
                hist[i].append(self.train_step(i, cache.inputs[i], cache.outputs[i])["loss"])
            self.step_count += 1
        return hist

    def _distill_sequential(self, batches, steps=None) -> Dict[int, List[float]]:
        batches = list(batches)
        hist: Dict[int, List[float]] = {}
        for i in range(len(self.ffn)):
            hist[i] = []
            self.step_count = 0
            for n, ids in enumerate(batches):
                if steps is not None and n >= steps:
                    break
                with torch.no_grad(), FFNActivationCache(self.model, layers=[i]) as cache:
                    self.model(ids.to(next(self.model.parameters()).device))
                hist[i].append(self.train_step(i, cache.inputs[i], cache.outputs[i])["loss"])
                self.step_count += 1
            self.moe_layers[str(i)].to("cpu")
            self.optimizers.pop(i, None)
        return hist

    def _random_inputs(self, g=None) -> torch.Tensor:
        x = torch.randn(self.cfg.data_free_batch_size, self.cfg.data_free_seq_len, self.d_model, generator=g)
        return (F.normalize(x, dim=-1) * math.sqrt(self.d_model)).to(self.device).to(self.dtype)

    @torch.no_grad()
    def _teacher(self, i: int, x: torch.Tensor) -> torch.Tensor:
        ffn = self.ffn[i][1]
        dev = next(ffn.parameters()).device
        out = ffn(x.to(dev))
        return (out[0] if isinstance(out, tuple) else out).to(self.device)

    @torch.no_grad()
    def _collect_ffn_activations_from_data(self, batches, i: int, max_samples: int = 10000):
        """(inputs, outputs) of dense FFN ``i`` on real batches, flattened to (N, d_model) on the host
        (reference: Experiments/sparse_distillation/distill.py:1261-1319).  A batch is a tensor of input
        ids, a tuple whose first entry is one, or a dict with ``input_ids`` (and optionally
        ``attention_mask``)."""
        xs, ys, n = [], [], 0
        dev = next(self.model.parameters()).device
        self.model.eval()
        for b in batches:
            if n >= max_samples:
                break
            kw = {}
            if isinstance(b, dict):
                ids = b.get("input_ids", b.get("tokens"))
                if b.get("attention_mask") is not None:
                    kw["attention_mask"] = b["attention_mask"].to(dev)
            else:
                ids = b[0] if isinstance(b, (list, tuple)) else b
            with FFNActivationCache(self.model, layers=[i]) as cache:
                self.model(ids.to(dev), **kw)
            xs.append(cache.inputs[i].reshape(-1, self.d_model).float().cpu())
            ys.append(cache.outputs[i].reshape(-1, self.d_model).float().cpu())
            n += xs[-1].shape[0]
        if not xs:
            raise ValueError(f"no activations collected for layer {i}")
        return torch.cat(xs)[:max_samples], torch.cat(ys)[:max_samples]

    def _cluster_ffn_outputs(self, i: int, n_clusters: int, batches=None):
        """Spherical k-means of the dense FFN's outputs: on activations from ``batches`` when given,
        otherwise on its responses to random unit-norm inputs scaled by sqrt(d)."""
        if batches is not None:
            X, Y = self._collect_ffn_activations_from_data(batches, i, self.cfg.cluster_samples)
            X, Y = X.to(self.dtype), Y.to(self.dtype)
        else:
            xs, ys = [], []
            n = 0
            while n < self.cfg.cluster_samples:
                x = self._random_inputs()
                xs.append(x.reshape(-1, self.d_model))
                ys.append(self._teacher(i, x).reshape(-1, self.d_model))
                n += xs[-1].shape[0]
            X, Y = torch.cat(xs)[: self.cfg.cluster_samples], torch.cat(ys)[: self.cfg.cluster_samples]
        assign, cent = kmeans(Y, n_clusters, spherical=True)
        return X, Y, assign, cent

    def analyze_cluster_quality(self, i=None, ks=(4, 8, 16), batches=None, outputs: torch.Tensor = None,
                                k_values=None) -> Dict[int, Dict[str, float]]:
        """Cluster quality of layer ``i``'s FFN outputs for each cluster count in ``ks``.  In the reference's form,
        ``analyze_cluster_quality(outputs, k_values)``, the (N, d_model) outputs are given directly
        (distill.py:1394-1536)."""
        if torch.is_tensor(i):
            outputs, i = i, None
            if not isinstance(ks, tuple) or ks != (4, 8, 16):
                k_values = ks if k_values is None else k_values
        if outputs is not None:
            res = {}
            Y = outputs.reshape(-1, outputs.shape[-1]).float()
            for k in (k_values or range(4, 65, 2)):
                if k > Y.shape[0]:
                    break
                assign, cent = kmeans(Y, int(k), spherical=True)
                res[int(k)] = cluster_quality(F.normalize(Y, dim=-1), assign, cent)
            return res
        ks = k_values if k_values is not None else ks
        out = {}
        batches = list(batches) if batches is not None else None
        for k in ks:
            _, Y, assign, cent = self._cluster_ffn_outputs(i, k, batches)
            out[k] = cluster_quality(F.normalize(Y.float(), dim=-1), assign, cent)
        return out

    def _train_router_supervised(self, i: int, steps: Optional[int] = None, batches=None) -> float:
        layer = self.moe_layers[str(i)].to(self.device).train()
        X, _, assign, _ = self._cluster_ffn_outputs(i, layer.n_experts, batches)
        params = list(layer.router.parameters()) + ([layer.expert_bias] if layer.expert_bias is not None else [])
        opt = torch.optim.AdamW(params, lr=self.cfg.learning_rate * 10)
        last = 0.0
        for s in range(steps or self.cfg.router_train_steps):
            sel = torch.randint(0, X.shape[0], (min(1024, X.shape[0]),))
            loss = F.cross_entropy(layer.get_router_logits(X[sel].to(self.device)).float(), assign[sel].to(self.device))
            opt.zero_grad(set_to_none=True)
            loss.backward()
            opt.step()
            last = float(loss.detach())
        return last

    def _distill_data_free(self, steps: int) -> Dict[int, List[float]]:
        hist: Dict[int, List[float]] = {}
        for i in range(len(self.ffn)):
            hist[i] = []
            if self.cfg.supervised_routing and self.cfg.moe_routing == "token_choice":
                self._train_router_supervised(i, min(self.cfg.router_train_steps, max(steps, 1)))
            self.step_count = 0
            for s in range(steps):
                x = self._random_inputs()
                hist[i].append(self.train_step(i, x, self._teacher(i, x))["loss"])
                self.step_count += 1
                if self.cfg.log_interval and (s + 1) % self.cfg.log_interval == 0:
                    print_layer_routing_stats(self.moe_layers[str(i)], i, prefix=f"  step {s + 1} ")
            if self.cfg.sequential_layers:
                self.moe_layers[str(i)].to("cpu")
        return hist

    def _expert_scores(self, layer: MoEDistillationLayer, x: torch.Tensor, target: torch.Tensor) -> torch.Tensor:
        """(T, E): per-token cost of sending the token to each expert alone."""
        with torch.no_grad():
            allo = layer.expert_outputs_all(x)                                   # E, T, d
            err = (allo.float() - target.reshape(1, -1, self.d_model).float())
            if self.cfg.gradient_routing and self.cfg.gradient_routing_fast:
                return err.abs().mean(-1).t()                                    # error magnitude ~ gradient norm
            return err.pow(2).mean(-1).t()

    def _distill_empirical_routing(self, steps: int) -> Dict[int, List[float]]:
        c = self.cfg
        hist: Dict[int, List[float]] = {}
        for i in range(len(self.ffn)):
            layer = self.moe_layers[str(i)].to(self.device).train()
            opt = self._get_optimizer(i)
            hist[i] = []
            targets = None
            for s in range(steps):
                frac = min(1.0, s / max(c.curriculum_warmup_steps, 1))
                bal = (c.curriculum_initial_balance + frac * (c.curriculum_final_balance - c.curriculum_initial_balance)
                       if c.curriculum_routing else 0.0)
                temp = (c.target_initial_temperature + frac * (c.target_final_temperature - c.target_initial_temperature)
                        if c.target_temperature_schedule else c.empirical_temperature)
                x = self._random_inputs()
                y = self._teacher(i, x)
                if targets is None or s % max(c.empirical_eval_interval, 1) == 0:
                    targets = balanced_topk_targets(self._expert_scores(layer, x, y), layer.top_k, c.target_max_prob,
                                                    temp, bal)
                    xt = x
                out, aux = layer(x, return_aux=True)
                loss, parts = self.compute_loss(out, y, aux, return_metrics=True)
                logp = F.log_softmax(layer.get_router_logits(xt.detach()).reshape(-1, layer.n_experts).float(), -1)
                kl = F.kl_div(logp, targets, reduction="batchmean")
                ent = -(logp.exp() * logp).sum(-1).mean()
                total = loss + c.router_loss_weight * kl - c.empirical_entropy_weight * ent
                opt.zero_grad(set_to_none=True)
                total.backward()
                torch.nn.utils.clip_grad_norm_(layer.parameters(), c.max_grad_norm)
                opt.step()
                hist[i].append(float(loss.detach()))
        return hist

    def _distill_dynamic(self, steps: int) -> Dict[int, List[float]]:
        c = self.cfg
        hist: Dict[int, List[float]] = {}
        for i in range(len(self.ffn)):
            base = self.moe_layers[str(i)]
            dyn = DynamicExpertLayer(self.d_model, [base.d_ff] * base.n_experts).to(self.device)
            with torch.no_grad():
                for e in range(base.n_experts):
                    dyn.w1[e].copy_(base.experts.w1[e]); dyn.w2[e].copy_(base.experts.w2[e]); dyn.w3[e].copy_(base.experts.w3[e])
            router = base.router_net().to(self.device)
            tracker = DynamicExpertTracker(base.n_experts)
            make_opt = lambda: torch.optim.AdamW(list(dyn.parameters()) + list(router.parameters()), lr=c.learning_rate)
            opt = make_opt()
            hist[i] = []
            for s in range(steps):
                x = self._random_inputs()
                y = self._teacher(i, x)
                flat, ty = x.reshape(-1, self.d_model).float(), y.reshape(-1, self.d_model).float()
                w, idx = torch.topk(F.softmax(router(flat.to(x.dtype)).float(), -1), base.top_k, dim=-1)
                w = w / w.sum(-1, keepdim=True)
                out = dyn(flat, idx, w)
                per_tok = (out - ty).pow(2).mean(-1)
                loss = per_tok.mean()
                opt.zero_grad(set_to_none=True)
                loss.backward()
                opt.step()
                hist[i].append(float(loss.detach()))
                pe = torch.zeros(base.n_experts, device=x.device).index_add_(0, idx[:, 0], per_tok.detach())
                cnt = torch.bincount(idx[:, 0], minlength=base.n_experts)
                tracker.update(pe / cnt.clamp(min=1), cnt)
                if c.reallocate_every_n_steps and (s + 1) % c.reallocate_every_n_steps == 0:
                    plan = tracker.plan(dyn.d_ffs, c.top_k_grow, c.top_k_shrink, c.growth_factor, c.shrink_factor,
                                        c.min_d_ff, c.max_d_ff)
                    if plan:
                        reallocate_expert_layer(dyn, plan)
                        opt = make_opt()
            self.moe_layers[str(i)].dynamic = dyn
        return hist

    # -------------------------------------------------------------- evaluation
    @torch.no_grad()
    def evaluate(self, n_batches=4, batches=None, max_batches: Optional[int] = 100,
                 dataloader=None) -> Dict[int, Dict[str, float]]:
        """Per layer: MSE, cosine similarity and relative MSE of the MoE layer against the dense FFN - on what the
        FFN sees when the model runs on ``batches`` (token ids; reference: distill.py:2849-2922) or, without
        batches, on ``n_batches`` random unit-norm inputs."""
        if not isinstance(n_batches, int):                       # evaluate(dataloader, max_batches): the reference's form
            batches, n_batches = n_batches, 4
        batches = dataloader if batches is None else batches
        if batches is not None:
            return self._evaluate_on_data(batches, max_batches if max_batches is not None else 10 ** 9)
        out = {}
        for i in range(len(self.ffn)):
            layer = self.moe_layers[str(i)].to(self.device).eval()
            mse = cos = 0.0
            for _ in range(n_batches):
                x = self._random_inputs()
                y, s = self._teacher(i, x).float(), layer(x).float()
                mse += float(F.mse_loss(s, y))
                cos += float(F.cosine_similarity(s.reshape(-1, self.d_model), y.reshape(-1, self.d_model), dim=-1).mean())
            out[i] = {"mse": mse / n_batches, "cosine": cos / n_batches,
                      "rel_mse": (mse / n_batches) / max(float(y.pow(2).mean()), 1e-12)}
        return out

    @torch.no_grad()
    def _evaluate_on_data(self, batches, max_batches: int) -> Dict[int, Dict[str, float]]:
        n = 0
        acc = {i: [0.0, 0.0, 0.0] for i in range(len(self.ffn))}
        dev = next(self.model.parameters()).device
        self.model.eval()
        for b in batches:
            if n >= max_batches:
                break
            with FFNActivationCache(self.model) as cache:
                self.model(_ids_of_batch(b).to(dev))
            for i in range(len(self.ffn)):
                layer = self.moe_layers[str(i)].to(self.device).eval()
                x, y = cache.inputs[i].to(self.device), cache.outputs[i].to(self.device).float()
                s = layer(x).float()
                acc[i][0] += float(F.mse_loss(s, y))
                acc[i][1] += float(F.cosine_similarity(s.reshape(-1, self.d_model), y.reshape(-1, self.d_model),
                                                       dim=-1).mean())
                acc[i][2] += float(y.pow(2).mean())
            n += 1
        n = max(n, 1)
        return {i: {"mse": a[0] / n, "cosine": a[1] / n, "rel_mse": (a[0] / n) / max(a[2] / n, 1e-12)}
                for i, a in acc.items()}

    def save(self, path: str):
        """``layers`` / ``dims`` / ``config`` (a plain dict) are what this package reads back; ``moe_layers`` (flat
        ``"<layer>.<key>"`` state dict), ``d_model``, ``d_ff``, ``layer_indices``, ``layer_dimensions``,
        ``global_step`` and ``layer_config`` are the reference's keys for the same content (distill.py:2924-2950)."""
        torch.save({"layers": {k: v.state_dict() for k, v in self.moe_layers.items()}, "config": asdict(self.cfg),
                    "dims": {k: (v.d_model, v.d_ff, v.n_experts, v.top_k) for k, v in self.moe_layers.items()},
                    "moe_layers": self.moe_layers.state_dict(), "d_model": self.d_model, "d_ff": self.d_ff_dense,
                    "dtype": str(self.dtype), "layer_indices": [int(k) for k in self.moe_layers],
                    "layer_dimensions": {int(k): {"n_experts": v.n_experts, "d_ff": v.d_ff}
                                         for k, v in self.moe_layers.items()},
                    "global_step": self.step_count, "layer_config": self.layer_cfg or None}, path)

    def load(self, path: str):
        ck = torch.load(path, map_location="cpu", weights_only=False)
        for k, sd in checkpoint_layers(ck).items():
            load_layer_state(self.moe_layers[k], sd)
        return ck
