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
