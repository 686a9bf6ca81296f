"""``MoETransformer``: embedding -> N blocks -> final norm -> n_pred_tokens LM heads
(reference: moe_arch/model/transformer.py:20-414).

Same constructor, ``forward`` signature, result dict and state-dict keys as the
reference.  With ``labels`` given and ``return_logits=False`` the loss is computed
from the final hidden state by the fused LM-head + cross-entropy op, so the four
(B, S, V) logits tensors of the reference (transformer.py:201-204) never exist.
"""
from __future__ import annotations

from typing import Dict, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..config import AdvancedMoEConfig
from ..training.losses import MultiTokenPredictionLoss
from .embeddings import TokenEmbedding, get_norm_layer
from .layers import TransformerBlock
from .linear import Linear


def _numel(module_or_params) -> int:
    ps = module_or_params.parameters() if isinstance(module_or_params, nn.Module) else module_or_params
    return sum(p.numel() for p in ps)


class MoETransformer(nn.Module):
    def __init__(self, config: AdvancedMoEConfig, verbose: bool = True):
        super().__init__()
        self.config = config
        self.gradient_checkpointing = False
        from .linear import deferred_init
        with deferred_init():                    # every Linear is initialised by ``_init_weights`` below
            self.token_embedding = TokenEmbedding(config)
            self.layers = nn.ModuleList([TransformerBlock(config, i) for i in range(config.n_layers)])
            self.final_norm = get_norm_layer(config)
            self.lm_heads = nn.ModuleList([Linear(config.d_model, config.vocab_size, bias=False)
                                           for _ in range(config.n_pred_tokens)])
        self.tie_word_embeddings = getattr(config, "tie_word_embeddings", True)
        if self.tie_word_embeddings:
            self.lm_heads[0].weight = self.token_embedding.embedding.weight
        self.multitoken_loss = MultiTokenPredictionLoss(config.n_pred_tokens, config.aux_loss_weights)
        self.apply(self._init_weights)
        if verbose:
            n, a = _numel(self), self.count_active_parameters()
            print(f"Initialized MoETransformer with {n / 1e9:.2f}B parameters "
                  f"({a / 1e9:.2f}B active, {config.n_pred_tokens} prediction heads)")

    def _init_weights(self, module: nn.Module) -> None:
        """normal(0, init_std) for every Linear/Embedding, zero Linear biases; stacked
        expert tensors, conv kernels and SSM vectors keep their own initialisation
        (reference: transformer.py:97-104)."""
        if isinstance(module, nn.Linear):
            nn.init.normal_(module.weight, mean=0.0, std=self.config.init_std)
            if module.bias is not None:
                nn.init.zeros_(module.bias)
        elif isinstance(module, nn.Embedding):
            nn.init.normal_(module.weight, mean=0.0, std=self.config.init_std)

    def gradient_checkpointing_enable(self):
        self.gradient_checkpointing = True

    def gradient_checkpointing_disable(self):
        self.gradient_checkpointing = False

    @staticmethod
    def _checkpointed_layer_forward(layer, hidden_states, attention_mask, position_ids):
        return layer(hidden_states, attention_mask, position_ids, return_aux_loss=True)

    # ------------------------------------------------------------------ trunk
    def forward_hidden(self, input_ids: torch.Tensor, attention_mask: Optional[torch.Tensor] = None,
                       position_ids: Optional[torch.Tensor] = None):
        """Embedding + blocks + final norm. Returns (hidden, summed aux loss)."""
        h = self.token_embedding(input_ids)
        add_mask = None
        if hasattr(attention_mask, "doc_start"):            # PackedDocs: handed to the attention layers as is
            add_mask = attention_mask
        elif attention_mask is not None and attention_mask.dim() == 4:    # already additive (B, 1, S, S)
            add_mask = attention_mask.to(h.dtype).clamp(min=torch.finfo(h.dtype).min)
        elif attention_mask is not None:
            add_mask = (1.0 - attention_mask[:, None, None, :].to(h.dtype)) * torch.finfo(h.dtype).min
        aux = 0.0
        for layer in self.layers:
            if self.gradient_checkpointing and self.training:
                from torch.utils.checkpoint import checkpoint
                h, a = checkpoint(self._checkpointed_layer_forward, layer, h, add_mask, position_ids,
                                  use_reentrant=False)
                aux = aux + a
            else:
                h = layer(h, attention_mask=add_mask, position_ids=position_ids)
                if self.training:
                    aux = aux + layer.aux_loss
        return self.final_norm(h), aux

    def forward(self, input_ids: torch.Tensor, attention_mask: Optional[torch.Tensor] = None,
                position_ids: Optional[torch.Tensor] = None, labels: Optional[torch.Tensor] = None,
                return_logits: bool = True) -> Dict[str, torch.Tensor]:
        from ..ops import checks
        if checks.enabled():       # out-of-range ids would otherwise end in a device-side assertion of the lookup
            checks.index_range(input_ids, self.config.vocab_size, "input_ids")
            if labels is not None:
                checks.labels(labels, self.config.vocab_size)
            if position_ids is not None:
                checks.index_range(position_ids, self.config.max_seq_len, "position_ids")
            elif input_ids.shape[1] > self.config.max_seq_len:
                raise IndexError(f"sequence length {input_ids.shape[1]} exceeds max_seq_len "
                                 f"{self.config.max_seq_len} (the rotary tables end there)")
        hidden, aux = self.forward_hidden(input_ids, attention_mask, position_ids)
        if hasattr(attention_mask, "doc_start") or (attention_mask is not None and attention_mask.dim() == 4):
            attention_mask = None                           # attention structure, not a padding mask for the loss
        loss = lm_loss = None
        info: Dict[str, torch.Tensor] = {}
        logits_list = None
        if return_logits:
            logits_list = [head(hidden) for head in self.lm_heads]
        if labels is not None:
            if logits_list is not None:
                lm_loss, info = self.multitoken_loss(logits_list, labels, attention_mask=attention_mask)
            else:
                lm_loss, info = self.multitoken_loss.from_hidden(
                    hidden, [h.weight for h in self.lm_heads], labels, attention_mask=attention_mask)
            loss = lm_loss + aux if (self.training and torch.is_tensor(aux)) else lm_loss
        result = {"loss": loss, "lm_loss": lm_loss, "aux_loss": aux if self.training else 0.0}
        if return_logits:
            result["logits"] = logits_list[0]
            result["logits_list"] = logits_list
            result["multitoken_loss_dict"] = info
        elif labels is not None:
            result["multitoken_loss_dict"] = info
        return result

    # ------------------------------------------------------------- generation
    @torch.no_grad()
    def generate(self, input_ids: torch.Tensor, max_new_tokens: int = 100, temperature: float = 1.0,
                 top_k: Optional[int] = None, top_p: Optional[float] = None) -> torch.Tensor:
        """Sampling loop with temperature / top-k / nucleus filtering.  Like the
        reference there is no KV cache: every step re-runs the prompt; only the last
        position is projected to the vocabulary."""
        for _ in range(max_new_tokens):
            ctx = input_ids[:, -self.config.max_seq_len:]
            hidden, _ = self.forward_hidden(ctx)
            logits = self.lm_heads[0](hidden[:, -1, :]).float() / temperature
            if top_k is not None:
                kth = torch.topk(logits, min(top_k, logits.size(-1)), dim=-1).values[:, -1:]
                logits = logits.masked_fill(logits < kth, float("-inf"))
            if top_p is not None:
                s_logits, s_idx = torch.sort(logits, descending=True, dim=-1)
                cum = torch.cumsum(F.softmax(s_logits, dim=-1), dim=-1)
                remove = cum > top_p
                remove[..., 1:] = remove[..., :-1].clone()
                remove[..., 0] = False
                logits = logits.masked_fill(remove.scatter(1, s_idx, remove), float("-inf"))
            nxt = torch.multinomial(F.softmax(logits, dim=-1), num_samples=1)
            input_ids = torch.cat([input_ids, nxt], dim=-1)
        return input_ids

    # ------------------------------------------------------------- accounting
    def count_active_parameters(self) -> int:
        """Parameters touched per token: everything except the unselected fraction
        (1 - top_k / n_experts) of each expert stack (FFN experts and RoutingMamba
        experts alike).  MoD changes compute, not this count."""
        c = self.config
        active = _numel(self.token_embedding) + _numel(self.final_norm) + _numel(self.lm_heads)
        if self.tie_word_embeddings:
            active -= self.lm_heads[0].weight.numel()
        for layer in self.layers:
            active += _numel(layer.seq_norm) + _numel(layer.ffn_norm)
            if layer.mixer_kind == "routing_mamba":
                active += _numel(layer.seq_layer.router)
                active += int(_numel(layer.seq_layer.experts) * c.moe_top_k / c.n_experts)
            else:
                active += _numel(layer.seq_layer)
            if layer.ffn_kind == "moe":
                ffn = layer.ffn
                if ffn._use_expert_parallel:
                    ep = ffn.expert_parallel_layer
                    active += _numel(ep.router)
                    active += int(_numel(ep.local_experts) * c.moe_top_k / ep.n_local_experts)
                else:
                    active += _numel(ffn.router)
                    experts = ffn.grouped_experts if ffn.grouped_experts is not None else ffn.grouped_experts_ec
                    active += int(_numel(experts) * c.moe_top_k / c.n_experts)
            else:
                active += _numel(layer.ffn)
            if layer.ffn_mod_router is not None:
                active += _numel(layer.ffn_mod_router)
        return active

    def count_parameters(self) -> Dict[str, float]:
        total = _numel(self)
        moe_p = std_p = n_moe = n_std = n_mamba = n_attn = 0
        for layer in self.layers:
            n = _numel(layer)
            if layer.use_moe:
                moe_p, n_moe = moe_p + n, n_moe + 1
            else:
                std_p, n_std = std_p + n, n_std + 1
            if layer.use_mamba:
                n_mamba += 1
            else:
                n_attn += 1
        active = self.count_active_parameters()
        return {
            "embedding": _numel(self.token_embedding), "layers": _numel(self.layers),
            "moe_layers": moe_p, "standard_layers": std_p, "n_moe_layers": n_moe,
            "n_standard_layers": n_std, "n_mamba_layers": n_mamba, "n_attention_layers": n_attn,
            "final_norm": _numel(self.final_norm), "lm_heads": _numel(self.lm_heads),
            "lm_head": _numel(self.lm_heads),          # the single-head name older callers (and the reference's tests) use
            "total": total, "total_billions": total / 1e9, "active": active,
            "active_billions": active / 1e9, "sparsity": 1.0 - active / max(total, 1),
        }
