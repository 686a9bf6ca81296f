"""Tokenizer wrapper (reference: moe_arch/data/tokenizer.py:12-145).

Wraps a HuggingFace ``AutoTokenizer`` (pad token = eos when missing).  When the named
tokenizer cannot be loaded (no network, no local files) and ``allow_byte_fallback`` is set,
a self-contained byte-level tokenizer is used so the data pipeline and the tests run offline.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Union


class ByteTokenizer:
    """256 byte values + <eos>=256, <pad>=257.  Deterministic, dependency-free."""

    eos_token, pad_token, bos_token = "<eos>", "<pad>", None
    eos_token_id, pad_token_id, bos_token_id = 256, 257, None

    def __len__(self) -> int:
        return 258

    def __call__(self, text, add_special_tokens=True, max_length=None, truncation=False, padding=False,
                 return_tensors=None, **_):
        single = isinstance(text, str)
        texts = [text] if single else list(text)
        ids = []
        for t in texts:
            row = list(t.encode("utf-8"))
            if add_special_tokens:
                row.append(self.eos_token_id)
            if truncation and max_length is not None:
                row = row[:max_length]
            ids.append(row)
        if padding:
            L = max(len(r) for r in ids) if padding is True or padding == "longest" else max_length
            mask = [[1] * len(r) + [0] * (L - len(r)) for r in ids]
            ids = [r + [self.pad_token_id] * (L - len(r)) for r in ids]
        else:
            mask = [[1] * len(r) for r in ids]
        if return_tensors == "pt":
            import torch
            return {"input_ids": torch.tensor(ids), "attention_mask": torch.tensor(mask)}
        if single:
            return {"input_ids": ids[0], "attention_mask": mask[0]}
        return {"input_ids": ids, "attention_mask": mask}

    def decode(self, ids, skip_special_tokens=True, **_):
        if hasattr(ids, "tolist"):
            ids = ids.tolist()
        return bytes(i for i in ids if i < 256).decode("utf-8", errors="replace")

    def batch_decode(self, batch, skip_special_tokens=True, **_):
        return [self.decode(r, skip_special_tokens) for r in batch]


class TokenizerWrapper:
    def __init__(self, tokenizer_name: str = "gpt2", vocab_size: Optional[int] = None,
                 add_special_tokens: bool = True, allow_byte_fallback: bool = True, verbose: bool = True):
        self.add_special_tokens = add_special_tokens
        try:
            from transformers import AutoTokenizer
            self.tokenizer = AutoTokenizer.from_pretrained(tokenizer_name)
            if self.tokenizer.pad_token is None:
                self.tokenizer.pad_token = self.tokenizer.eos_token
        except Exception as e:
            if not allow_byte_fallback:
                raise
            if verbose:
                print(f"Warning: tokenizer '{tokenizer_name}' unavailable ({type(e).__name__}); "
                      "using the built-in byte tokenizer")
            self.tokenizer = ByteTokenizer()
        if vocab_size is not None and len(self.tokenizer) != vocab_size and verbose:
            print(f"Warning: Tokenizer vocab size ({len(self.tokenizer)}) differs from config vocab size ({vocab_size})")

    @property
    def vocab_size(self) -> int:
        return len(self.tokenizer)

    @property
    def pad_token_id(self) -> int:
        return self.tokenizer.pad_token_id

    @property
    def eos_token_id(self) -> int:
        return self.tokenizer.eos_token_id

    @property
    def bos_token_id(self):
        return self.tokenizer.bos_token_id

    def encode(self, text: Union[str, Sequence[str]], max_length: Optional[int] = None, truncation: bool = True,
               padding: Union[bool, str] = False, return_tensors: Optional[str] = None):
        return self.tokenizer(text, add_special_tokens=self.add_special_tokens, max_length=max_length,
                              truncation=truncation, padding=padding, return_tensors=return_tensors)

    def decode(self, token_ids, skip_special_tokens: bool = True) -> str:
        return self.tokenizer.decode(token_ids, skip_special_tokens=skip_special_tokens)

    def batch_decode(self, token_ids, skip_special_tokens: bool = True) -> List[str]:
        return self.tokenizer.batch_decode(token_ids, skip_special_tokens=skip_special_tokens)
