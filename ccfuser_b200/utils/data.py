"""Token-stream batching for language-model training.

``LMOrderedIterator`` cuts one long token stream into ``batch_size`` parallel streams and yields consecutive
``[batch, tgt_len]`` segments with next-token targets, so that the hidden-state memory of Transformer-XL stays aligned
from one step to the next (same contract as the iterator the reference vendors in
mix_moe/mix_moe/examples/transformer-xl/data_utils.py:9-60, batch-first here). ``synthetic_corpus`` provides token
streams when no dataset is available.
"""
from __future__ import annotations

from typing import Iterator, Optional, Tuple

import torch


def synthetic_corpus(n_tokens: int, vocab_size: int, seed: int = 0, zipf: float = 1.1) -> torch.Tensor:
    """A reproducible token stream with a Zipf-like unigram distribution (ids in [0, vocab_size))."""
    g = torch.Generator().manual_seed(seed)
    ranks = torch.arange(1, vocab_size + 1, dtype=torch.float64)
    p = ranks.pow(-zipf)
    return torch.multinomial(p / p.sum(), n_tokens, replacement=True, generator=g)


class LMOrderedIterator:
    """Consecutive ``[batch, tgt_len]`` segments of ``batch`` parallel streams cut from one token stream; see the module docstring."""
    def __init__(self, data: torch.Tensor, batch_size: int, tgt_len: int, device=None, rank: int = 0, world: int = 1):
        """`data`: 1-D token ids. Each data-parallel rank takes its own contiguous share of the stream."""
        share = data.numel() // world
        data = data[rank * share:(rank + 1) * share]
        n_step = data.numel() // batch_size
        self.data = data[:n_step * batch_size].view(batch_size, n_step).contiguous()
        self.batch_size, self.tgt_len, self.device = batch_size, tgt_len, device
        self.n_batch = max(0, (n_step - 1) // tgt_len)
        if device is not None and torch.device(device).type == "cuda":
            self.data = self.data.pin_memory()

    def get_batch(self, i: int) -> Tuple[torch.Tensor, torch.Tensor]:
        beg = i * self.tgt_len
        end = min(beg + self.tgt_len, self.data.shape[1] - 1)
        x, y = self.data[:, beg:end], self.data[:, beg + 1:end + 1]
        if self.device is not None:
            x, y = x.to(self.device, non_blocking=True), y.to(self.device, non_blocking=True)
        return x.contiguous(), y.contiguous()

    def __len__(self) -> int:
        return self.n_batch

    def __iter__(self) -> Iterator[Tuple[torch.Tensor, torch.Tensor]]:
        for i in range(self.n_batch):
            yield self.get_batch(i)


def evaluate_lm(model_step, iterator: LMOrderedIterator, max_batches: Optional[int] = None) -> float:
    """Mean loss of ``model_step(x, y) -> loss`` over an iterator, without gradients."""
    total, n = 0.0, 0
    with torch.no_grad():
        for i, (x, y) in enumerate(iterator):
            if max_batches is not None and i >= max_batches:
                break
            total += float(model_step(x, y))
            n += 1
    return total / max(1, n)


class Vocab:
    """Word-level vocabulary built from text: ids by descending frequency (ties by first appearance), optional
    ``<unk>`` / ``<eos>`` symbols, frequency and size limits. Covers what the training scripts need from the
    vocabulary helper the reference vendors (mix_moe/mix_moe/examples/transformer-xl/utils/vocabulary.py)."""

    def __init__(self, min_freq: int = 1, max_size: Optional[int] = None, lower: bool = False, add_eos: bool = True,
                 unk: str = "<unk>", eos: str = "<eos>"):
        self.min_freq, self.max_size, self.lower, self.add_eos = min_freq, max_size, lower, add_eos
        self.unk, self.eos = unk, eos
        self.counter: dict = {}
        self.idx2sym: list = []
        self.sym2idx: dict = {}

    def tokenize(self, line: str):
        line = line.strip()
        if self.lower:
            line = line.lower()
        toks = line.split()
        return toks + [self.eos] if (self.add_eos and toks) else toks

    def count_lines(self, lines):
        for line in lines:
            for t in self.tokenize(line):
                self.counter[t] = self.counter.get(t, 0) + 1

    def build(self):
        self.idx2sym, self.sym2idx = [], {}
        for sym in (self.unk,) + ((self.eos,) if self.add_eos else ()):
            self._add(sym)
        order = sorted(self.counter.items(), key=lambda kv: -kv[1])      # stable: first appearance breaks ties
        for sym, n in order:
            if n < self.min_freq or (self.max_size is not None and len(self.idx2sym) >= self.max_size):
                break
            self._add(sym)
        return self

    def _add(self, sym):
        if sym not in self.sym2idx:
            self.sym2idx[sym] = len(self.idx2sym)
            self.idx2sym.append(sym)

    def encode_lines(self, lines) -> torch.Tensor:
        unk = self.sym2idx[self.unk]
        ids = [self.sym2idx.get(t, unk) for line in lines for t in self.tokenize(line)]
        return torch.tensor(ids, dtype=torch.int64)

    def decode(self, ids) -> str:
        return " ".join(self.idx2sym[int(i)] for i in ids)

    def __len__(self):
        return len(self.idx2sym)


class Corpus:
    """train / valid / test token streams from three text files (or three lists of lines) sharing one vocabulary built
    on the training split; ``iterator(split, ...)`` gives an ``LMOrderedIterator`` over it."""

    def __init__(self, train, valid=None, test=None, **vocab_kw):
        def lines(src):
            if src is None:
                return []
            if isinstance(src, str):
                with open(src, encoding="utf-8") as f:
                    return f.readlines()
            return list(src)
        splits = {"train": lines(train), "valid": lines(valid), "test": lines(test)}
        self.vocab = Vocab(**vocab_kw)
        self.vocab.count_lines(splits["train"])
        self.vocab.build()
        self.data = {k: self.vocab.encode_lines(v) for k, v in splits.items()}

    def iterator(self, split: str, batch_size: int, tgt_len: int, device=None, rank: int = 0, world: int = 1):
        return LMOrderedIterator(self.data[split], batch_size, tgt_len, device=device, rank=rank, world=world)
