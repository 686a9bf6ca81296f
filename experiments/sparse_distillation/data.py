"""Token batches for the distillation command lines.

The reference's scripts tokenise a Hugging Face data set with the model's tokenizer
(Experiments/sparse_distillation/example_usage.py:214-291, finetune_eval.py:880-960).  The same arguments are
accepted here (``--dataset``, ``--dataset_config``, ``--max_samples``, ``--seq_len``, ``--batch_size``); where the
data set or the tokenizer cannot be had (no network, ``--model toy``) the batches come from a uint16 token file
(``--data``) or, failing that, are uniform random ids from a seed, and the source is reported.
"""
from __future__ import annotations

import os
from typing import List, Optional, Tuple

import torch

TEXT_DATASETS = {"c4": ("c4", "en"), "fineweb-edu": ("HuggingFaceFW/fineweb-edu", None),
                 "HuggingFaceFW/fineweb-edu": ("HuggingFaceFW/fineweb-edu", None)}


def _offline() -> bool:
    return os.environ.get("HF_HUB_OFFLINE") == "1" or os.environ.get("KMOE_OFFLINE") == "1"


def _from_hub(model: str, dataset: str, dataset_config: Optional[str], max_samples: int, seq_len: int):
    """(rows of token ids, pad id) from a Hugging Face data set, or None when it cannot be loaded."""
    if _offline() or model == "toy":
        return None
    try:
        from datasets import load_dataset
        from transformers import AutoTokenizer
        tok = AutoTokenizer.from_pretrained(model)
        if tok.pad_token is None:
            tok.pad_token = tok.eos_token
        if dataset in TEXT_DATASETS:
            name, cfg = TEXT_DATASETS[dataset]
            ds = load_dataset(name, cfg, split="train", streaming=True) if cfg else \
                load_dataset(name, split="train", streaming=True)
            rows_text = [r["text"] for r, _ in zip(ds, range(max_samples))]
        else:
            ds = load_dataset(dataset, dataset_config, split="train") if dataset_config else \
                load_dataset(dataset, split="train")
            col = "text" if "text" in ds.column_names else ds.column_names[0]
            rows_text = [ds[i][col] for i in range(min(len(ds), max_samples))]
        enc = tok(rows_text, truncation=True, max_length=seq_len, padding="max_length", return_tensors="pt")
        return enc["input_ids"], tok.pad_token_id
    except Exception as e:                      # no network, no cache, unknown data set: say so and fall back
        print(f"[sparse_distillation] data set '{dataset}' unavailable ({type(e).__name__}); using fallback tokens")
        return None


def load_token_batches(model: str, vocab: int, *, dataset: str = "wikitext",
                       dataset_config: Optional[str] = "wikitext-2-raw-v1", data_file: Optional[str] = None,
                       max_samples: int = 10000, seq_len: int = 2048, batch_size: int = 1, n_batches: Optional[int] = None,
                       seed: int = 0, device: str = "cpu") -> Tuple[List[torch.Tensor], str, Optional[int]]:
    """Returns (batches of (batch_size, seq_len) ids, source, pad id).  ``source`` is ``"dataset"``, ``"file"`` or
    ``"random"``.  ``n_batches`` bounds the number of batches (default: what ``max_samples`` rows give)."""
    g = torch.Generator().manual_seed(seed)
    want = n_batches if n_batches is not None else max(max_samples // batch_size, 1)
    hub = _from_hub(model, dataset, dataset_config, min(max_samples, want * batch_size), seq_len)
    pad = None
    if hub is not None:
        rows, pad = hub
        source = "dataset"
    elif data_file:
        import numpy as np
        arr = np.memmap(data_file, dtype=np.uint16, mode="r")
        n_seq = (len(arr) - 1) // seq_len
        pick = torch.randperm(n_seq, generator=g)[: want * batch_size].tolist()
        rows = torch.stack([torch.from_numpy(np.asarray(arr[i * seq_len: (i + 1) * seq_len], dtype=np.int64))
                            for i in pick])
        source = "file"
    else:
        rows = torch.randint(0, vocab, (want * batch_size, seq_len), generator=g)
        source = "random"
    rows = rows[torch.randperm(rows.shape[0], generator=g)] if source == "dataset" else rows
    batches = [rows[i: i + batch_size].to(device) for i in range(0, rows.shape[0] - batch_size + 1, batch_size)]
    return batches[:want], source, pad
