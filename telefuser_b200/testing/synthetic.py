"""Synthetic stand-ins for benchmarks and tests that run without checkpoints or a network:
random initialisation of real architectures and a deterministic hash tokenizer."""

from __future__ import annotations

import hashlib

import torch


def random_init_(model: torch.nn.Module, seed: int = 0, std: float = 0.02) -> torch.nn.Module:
    """Fills parameters in place: N(0, std) matrices, small biases, unit norm scales, N(0, 1/sqrt(d)) modulation tables."""
    dev = next(model.parameters()).device
    g = torch.Generator(device=dev).manual_seed(seed)
    for name, p in model.named_parameters():
        if "modulation" in name:
            p.data.normal_(0.0, 1.0 / p.shape[-1] ** 0.5, generator=g)
        elif name.endswith("gamma") or (p.dim() == 1 and not name.endswith("bias")):
            p.data.fill_(1.0)
        elif p.dim() >= 2:
            p.data.normal_(0.0, std, generator=g)
        else:
            p.data.normal_(0.0, 0.01, generator=g)
    return model


class HashTokenizer:
    """Maps whitespace-separated words to ids by hashing; pads to a fixed length. Deterministic, no files."""

    def __init__(self, vocab_size: int, seq_len: int):
        self.vocab_size, self.seq_len = vocab_size, seq_len

    def __call__(self, sequence, return_mask: bool = False, **kwargs):
        if isinstance(sequence, str):
            sequence = [sequence]
        ids = torch.zeros(len(sequence), self.seq_len, dtype=torch.long)
        mask = torch.zeros(len(sequence), self.seq_len, dtype=torch.long)
        for i, s in enumerate(sequence):
            words = s.split()[: self.seq_len - 1]
            toks = [2 + int(hashlib.md5(w.encode()).hexdigest(), 16) % (self.vocab_size - 2) for w in words] + [1]
            ids[i, : len(toks)] = torch.tensor(toks)
            mask[i, : len(toks)] = 1
        return (ids, mask) if return_mask else ids
