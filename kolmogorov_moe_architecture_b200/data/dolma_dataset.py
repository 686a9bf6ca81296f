"""Datasets and loaders (reference: moe_arch/data/dolma_dataset.py:19-336, the packed /
document-aware streaming of train_custom.py:216-335 and its prefetcher, 519-594).

* ``SyntheticTokenDataset``   - uniform-random token ids from a seed (the benchmark's data).
* ``DolmaStreamingDataset``   - FineWeb -> FineWeb-Edu -> OpenWebText -> Pile, falling back to
  random ids when none can be opened; yields ``input_ids == labels`` chunks of ``seq_len``.
* ``PackedDocumentDataset``   - packs documents into fixed-length rows with ``doc_ids`` and labels
  masked (-100) where the next-token targets would cross a document boundary.
* ``DolmaMemoryMappedDataset``- uint16 ``.bin`` memmap in strides of ``seq_len + n_pred_tokens``.
* ``PinnedPrefetcher``        - background thread that collates the next batches into pinned host
  memory so the step's host-to-device copy is a single asynchronous DMA.
"""
from __future__ import annotations

import os
import queue
import threading
from pathlib import Path
from typing import Dict, Iterable, Iterator, List, Optional

import numpy as np
import torch
from torch.utils.data import DataLoader, Dataset, IterableDataset


class SyntheticTokenDataset(IterableDataset):
    def __init__(self, vocab_size: int, seq_len: int, seed: int = 1234, rank: int = 0, low: int = 0):
        super().__init__()
        self.vocab_size, self.seq_len, self.seed, self.rank, self.low = vocab_size, seq_len, seed, rank, low

    def __iter__(self) -> Iterator[Dict[str, torch.Tensor]]:
        g = torch.Generator().manual_seed(self.seed + self.rank)
        while True:
            ids = torch.randint(self.low, self.vocab_size, (self.seq_len,), generator=g)
            yield {"input_ids": ids, "labels": ids}


_SOURCES = [("HuggingFaceFW/fineweb", "sample-10BT"), ("HuggingFaceFW/fineweb-edu", "sample-10BT"),
            ("Skylion007/openwebtext", None), ("monology/pile-uncopyrighted", None)]


def _open_first_available(split: str, streaming: bool, names=None):
    try:
        from datasets import load_dataset
    except Exception:
        return None
    if os.environ.get("HF_HUB_OFFLINE") == "1" or os.environ.get("KMOE_OFFLINE") == "1":
        return None
    for name, cfg in (names or _SOURCES):
        try:
            ds = load_dataset(name, cfg, split="train" if split == "train" else "train", streaming=streaming)
            return ds
        except Exception:
            continue
    return None


class DolmaStreamingDataset(IterableDataset):
    def __init__(self, tokenizer, seq_len: int = 2048, n_pred_tokens: int = 4, split: str = "train",
                 streaming: bool = True, vocab_size: Optional[int] = None, use_dummy_if_no_split: bool = True,
                 rank: int = 0, world_size: int = 1, seed: int = 0):
        super().__init__()
        self.tokenizer, self.seq_len, self.n_pred_tokens = tokenizer, seq_len, n_pred_tokens
        self.split, self.streaming = split, streaming
        self.vocab_size = vocab_size if vocab_size is not None else tokenizer.vocab_size
        self.rank, self.world_size, self.seed = rank, world_size, seed
        self.dataset = _open_first_available(split, streaming)
        if self.dataset is not None and world_size > 1 and hasattr(self.dataset, "shard"):
            try:
                self.dataset = self.dataset.shard(num_shards=world_size, index=rank)
            except Exception:
                pass
        if self.dataset is None and not use_dummy_if_no_split:
            raise RuntimeError("no dataset could be opened and dummy data is disabled")

    def __iter__(self) -> Iterator[Dict[str, torch.Tensor]]:
        n = self.seq_len + self.n_pred_tokens
        if self.dataset is None:
            g = torch.Generator().manual_seed(self.seed + 7919 * self.rank)
            while True:
                ids = torch.randint(1, self.vocab_size, (n,), generator=g)
                yield {"input_ids": ids[:-self.n_pred_tokens], "labels": ids[:-self.n_pred_tokens]}
        for ex in self.dataset:
            text = ex.get("text", "")
            if not text:
                continue
            enc = self.tokenizer.encode(text, truncation=False)
            toks = enc["input_ids"] if isinstance(enc, dict) else enc
            if len(toks) < n:
                continue
            for i in range(0, len(toks) - n, self.seq_len):
                chunk = torch.tensor(toks[i: i + n])
                yield {"input_ids": chunk[:-self.n_pred_tokens], "labels": chunk[:-self.n_pred_tokens]}


class PackedDocumentDataset(IterableDataset):
    """Packs an iterable of token lists (documents, each ended by ``eos_id``) into rows of
    ``seq_len``.  Yields ``input_ids``, ``labels`` (with -100 at positions whose any of the next
    ``n_pred_tokens`` targets belongs to another document when ``mask_cross_doc``) and ``doc_ids``."""

    def __init__(self, documents: Iterable[List[int]], seq_len: int, eos_id: int, n_pred_tokens: int = 1,
                 mask_cross_doc: bool = True):
        super().__init__()
        self.documents, self.seq_len, self.eos_id = documents, seq_len, eos_id
        self.n_pred_tokens, self.mask_cross_doc = n_pred_tokens, mask_cross_doc

    def __iter__(self):
        buf: List[int] = []
        docs: List[int] = []
        d = 0
        for toks in self.documents:
            toks = list(toks)
            if not toks or toks[-1] != self.eos_id:
                toks.append(self.eos_id)
            buf.extend(toks)
            docs.extend([d] * len(toks))
            d += 1
            while len(buf) >= self.seq_len:
                ids = torch.tensor(buf[: self.seq_len])
                did = torch.tensor(docs[: self.seq_len])
                did = did - did[0]
                labels = ids.clone()
                if self.mask_cross_doc:
                    # MTP head i reads labels[t + i + 1]; mask a label whose position starts a new document
                    # so no target is predicted across a boundary
                    boundary = torch.zeros_like(ids, dtype=torch.bool)
                    boundary[1:] = did[1:] != did[:-1]
                    labels = labels.masked_fill(boundary, -100)
                yield {"input_ids": ids, "labels": labels, "doc_ids": did}
                buf, docs = buf[self.seq_len:], docs[self.seq_len:]


def document_attention_mask(doc_ids: torch.Tensor) -> torch.Tensor:
    """Additive block-diagonal causal mask (B,1,S,S) from (B,S) document ids
    (reference: train_custom.py:429-463)."""
    same = doc_ids[:, :, None] == doc_ids[:, None, :]
    S = doc_ids.shape[1]
    causal = torch.tril(torch.ones(S, S, dtype=torch.bool, device=doc_ids.device))
    ok = same & causal
    return torch.zeros(ok.shape, dtype=torch.float32, device=doc_ids.device).masked_fill(~ok, float("-inf"))[:, None]


class PackedDocs:
    """Document boundaries of a packed batch, for attention that must not cross documents.

    Pass an instance as ``attention_mask`` to ``MoETransformer``: on CUDA the flash-attention kernels apply the
    boundaries directly (each query row only needs the first position of its document), so packed
    training keeps the fast path; elsewhere it becomes the additive mask of ``document_attention_mask``.
    The reference builds the dense (B, 1, S, S) mask and falls off its flash path (train_custom.py:429-463)."""

    def __init__(self, doc_ids: Optional[torch.Tensor] = None, doc_start: Optional[torch.Tensor] = None,
                 _checked: bool = False):
        from ..ops import eager
        assert (doc_ids is None) != (doc_start is None), "give document ids or start positions"
        if doc_start is None:
            self.doc_start = eager.doc_start_from_ids(doc_ids)
        elif _checked:
            self.doc_start = doc_start
        else:
            # start positions from outside: a start is neither negative nor after its own position (the
            # attention kernels index key blocks with it), and starts never move backwards along a sequence
            # (the kernels skip the key blocks before the start of a tile's first query for the whole tile)
            ds = doc_start.to(torch.int32)
            pos = torch.arange(ds.shape[-1], device=ds.device, dtype=torch.int32)
            ds = torch.minimum(ds.clamp(min=0), pos.expand_as(ds))
            self.doc_start = torch.cummax(ds, dim=-1).values

    @property
    def device(self):
        return self.doc_start.device

    def to(self, device, non_blocking: bool = False) -> "PackedDocs":
        return PackedDocs(doc_start=self.doc_start.to(device, non_blocking=non_blocking), _checked=True)

    def chunk(self, n: int, dim: int = 0):
        return [PackedDocs(doc_start=t, _checked=True) for t in self.doc_start.chunk(n, dim=dim)]

    def dense_mask(self, dtype=torch.float32) -> torch.Tensor:
        from ..ops import eager
        return eager.doc_start_to_mask(self.doc_start, dtype)


class DolmaMemoryMappedDataset(Dataset):
    def __init__(self, data_path: str, seq_len: int = 2048, n_pred_tokens: int = 4, vocab_size: int = 50257):
        super().__init__()
        self.data_path = Path(data_path)
        self.seq_len, self.n_pred_tokens, self.vocab_size = seq_len, n_pred_tokens, vocab_size
        if not self.data_path.exists():
            raise FileNotFoundError(f"Pre-tokenized data file not found: {data_path}")
        self.data = np.memmap(self.data_path, dtype=np.uint16, mode="r")
        self.n_samples = len(self.data) // (seq_len + n_pred_tokens)

    def __len__(self) -> int:
        return self.n_samples

    def __getitem__(self, idx: int) -> Dict[str, torch.Tensor]:
        n = self.seq_len + self.n_pred_tokens
        chunk = torch.from_numpy(self.data[idx * n: (idx + 1) * n].astype(np.int64))
        return {"input_ids": chunk[:-self.n_pred_tokens], "labels": chunk[:-self.n_pred_tokens]}


def write_token_file(path: str, tokens) -> None:
    """Write a uint16 ``.bin`` token file readable by ``DolmaMemoryMappedDataset``."""
    np.asarray(tokens, dtype=np.uint16).tofile(path)


def get_dataloaders(tokenizer, config, batch_size: int = 8, num_workers: int = 4, use_memory_mapped: bool = False,
                    data_path: Optional[str] = None, synthetic: bool = False, rank: int = 0, world_size: int = 1):
    if synthetic:
        tr = SyntheticTokenDataset(config.vocab_size, config.max_seq_len, seed=1234, rank=rank)
        va = SyntheticTokenDataset(config.vocab_size, config.max_seq_len, seed=4321, rank=rank)
        return DataLoader(tr, batch_size=batch_size), DataLoader(va, batch_size=batch_size)
    if use_memory_mapped:
        if data_path is None:
            raise ValueError("data_path must be provided when use_memory_mapped=True")
        mk = lambda f: DolmaMemoryMappedDataset(os.path.join(data_path, f), config.max_seq_len,
                                                config.n_pred_tokens, config.vocab_size)
        tr, va = mk("train.bin"), mk("val.bin")
        return (DataLoader(tr, batch_size=batch_size, shuffle=True, num_workers=num_workers, pin_memory=True),
                DataLoader(va, batch_size=batch_size, shuffle=False, num_workers=num_workers, pin_memory=True))
    mk = lambda split: DolmaStreamingDataset(tokenizer, config.max_seq_len, config.n_pred_tokens, split, True,
                                             config.vocab_size, rank=rank, world_size=world_size)
    return DataLoader(mk("train"), batch_size=batch_size, num_workers=0), \
        DataLoader(mk("validation"), batch_size=batch_size, num_workers=0)


class PinnedPrefetcher:
    """Iterates a loader from a background thread, staging each batch in pinned host memory.
    ``depth`` batches are kept ready.  An exception in the loader thread is re-raised in the
    consumer (so a failing data source surfaces as an error, not as a stalled step)."""

    _END = object()

    def __init__(self, loader: Iterable, depth: int = 4, pin: Optional[bool] = None):
        self.loader, self.depth = loader, depth
        self.pin = torch.cuda.is_available() if pin is None else pin
        self.q: "queue.Queue" = queue.Queue(maxsize=depth)
        self.stop_flag = threading.Event()
        self.thread = threading.Thread(target=self._run, daemon=True)
        self.thread.start()

    def _stage(self, batch):
        if isinstance(batch, dict):
            return {k: self._stage(v) for k, v in batch.items()}
        if torch.is_tensor(batch) and self.pin:
            return batch.pin_memory()
        return batch

    def _run(self):
        try:
            for b in self.loader:
                if self.stop_flag.is_set():
                    return
                self.q.put(self._stage(b))
            self.q.put(self._END)
        except BaseException as e:   # surfaced to the consumer
            self.q.put(e)

    def __iter__(self):
        return self

    def __next__(self):
        item = self.q.get()
        if item is self._END:
            raise StopIteration
        if isinstance(item, BaseException):
            raise item
        return item

    def close(self):
        self.stop_flag.set()
        try:
            while True:
                self.q.get_nowait()
        except queue.Empty:
            pass


class ThreadedPrefetcher(PinnedPrefetcher):
    """``PinnedPrefetcher`` with the constructor and behaviour of the reference's custom-training
    prefetcher (reference: train_custom.py:519-594): ``buffer_size`` batches are produced ahead by a
    background thread and every batch handed out is already on ``device`` (the copy from pinned
    memory is asynchronous, so it overlaps the step that is still running)."""

    def __init__(self, dataloader: Iterable, device, buffer_size: int = 3):
        self.device = torch.device(device)
        super().__init__(dataloader, depth=buffer_size, pin=self.device.type == "cuda")

    def _to_device(self, batch):
        if isinstance(batch, dict):
            return {k: self._to_device(v) for k, v in batch.items()}
        if torch.is_tensor(batch):
            return batch.to(self.device, non_blocking=True)
        return batch

    def __next__(self):
        return self._to_device(super().__next__())

    def stop(self):
        """End the producer thread and drop what it has staged (the reference's name for ``close``)."""
        self.close()
