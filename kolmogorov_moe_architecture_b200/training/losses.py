"""Multi-token-prediction loss (reference: moe_arch/training/losses.py:13-123).

Head i (0-based) is scored on positions [0, S-i-1) against ``labels[:, i+1:]``;
the caller passes unshifted labels.  Head weights are normalised to sum to 1.
Two entry points: :meth:`forward` takes materialised logits (API parity) and
:meth:`from_hidden` takes the final hidden state plus the head matrices and goes
through the fused linear+cross-entropy op, which never builds a (B, S, V) tensor.
Neither synchronises with the host: the per-head values in the returned dict are
0-d tensors (the reference calls ``.item()`` five times per step, losses.py:113,121).
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence, Tuple

import torch
import torch.nn as nn
import torch.nn.functional as F

from .. import ops


class MultiTokenPredictionLoss(nn.Module):
    def __init__(self, n_pred_tokens: int = 4, aux_loss_weights: Sequence[float] = (1.0, 0.5, 0.3, 0.2),
                 ignore_index: int = -100):
        super().__init__()
        assert len(aux_loss_weights) == n_pred_tokens, (
            f"aux_loss_weights length ({len(aux_loss_weights)}) must match n_pred_tokens ({n_pred_tokens})")
        self.n_pred_tokens = n_pred_tokens
        s = float(sum(aux_loss_weights))
        self.aux_loss_weights = tuple(w / s for w in aux_loss_weights)
        self.ignore_index = ignore_index

    def _masked_labels(self, labels: torch.Tensor, attention_mask: Optional[torch.Tensor]) -> torch.Tensor:
        if attention_mask is None:
            return labels
        return labels.masked_fill(attention_mask == 0, self.ignore_index)

    def forward(self, logits_list: List[torch.Tensor], labels: torch.Tensor,
                attention_mask: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, Dict[str, torch.Tensor]]:
        assert len(logits_list) == self.n_pred_tokens, (
            f"Expected {self.n_pred_tokens} logits tensors, got {len(logits_list)}")
        labels = self._masked_labels(labels, attention_mask)
        S = labels.shape[1]
        total = None
        info: Dict[str, torch.Tensor] = {}
        for i, (logits, w) in enumerate(zip(logits_list, self.aux_loss_weights)):
            if i + 1 >= S:
                loss = logits.new_zeros(())
            else:
                lg = logits[:, : S - i - 1]
                loss = F.cross_entropy(lg.reshape(-1, lg.size(-1)), labels[:, i + 1:].reshape(-1),
                                       ignore_index=self.ignore_index, reduction="mean")
            info[f"loss_t{i + 1}"] = loss.detach()
            total = w * loss if total is None else total + w * loss
        info["total_multitoken_loss"] = total.detach()
        return total, info

    def from_hidden(self, hidden: torch.Tensor, head_weights: Sequence[torch.Tensor], labels: torch.Tensor,
                    attention_mask: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, Dict[str, torch.Tensor]]:
        labels = self._masked_labels(labels, attention_mask)
        total, per = ops.mtp_cross_entropy(hidden, list(head_weights), labels, self.aux_loss_weights,
                                           self.ignore_index)
        info = {f"loss_t{i + 1}": per[i].detach() for i in range(self.n_pred_tokens)}
        info["total_multitoken_loss"] = total.detach()
        return total, info
