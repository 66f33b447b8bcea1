"""Bit-sequence "circuit" tasks: parity, majority, vocabulary majority and their cumulative (per-position) versions
(zoology/data/circuits.py:8-258). Tokens: 0 / 1 are bits, 2 is the end marker; only the last position is supervised in
the non-cumulative tasks."""
from __future__ import annotations

import numpy as np
import torch

from ..config import DataSegmentConfig
from .utils import DataSegment


def _final_answer(bits: np.ndarray, end: int, answer: np.ndarray, slices: dict | None):
    n = len(bits)
    inputs = np.concatenate([bits, np.full((n, 1), end, dtype=np.int64)], axis=1)
    labels = np.full_like(inputs, -100)
    labels[:, -1] = answer
    return DataSegment(torch.from_numpy(inputs), torch.from_numpy(labels), slices=slices)


class ParityConfig(DataSegmentConfig):
    name: str = "parity"

    def build(self, seed: int) -> DataSegment:
        return parity(**self.model_dump(), seed=seed)


def parity(vocab_size: int, num_examples: int, input_seq_len: int, seed: int, **kwargs) -> DataSegment:
    bits = np.random.RandomState(seed).randint(0, 2, size=(num_examples, input_seq_len - 1)).astype(np.int64)
    return _final_answer(bits, 2, bits.sum(1) % 2, {"input_seq_len": input_seq_len})


class MajorityConfig(DataSegmentConfig):
    name: str = "majority"

    def build(self, seed: int) -> DataSegment:
        return majority(**self.model_dump(), seed=seed)


def majority(vocab_size: int, num_examples: int, input_seq_len: int, seed: int, **kwargs) -> DataSegment:
    bits = np.random.RandomState(seed).randint(0, 2, size=(num_examples, input_seq_len - 1)).astype(np.int64)
    return _final_answer(bits, 2, (bits.mean(1) > 0.5).astype(np.int64), None)


class VocabMajorityConfig(DataSegmentConfig):
    name: str = "vocab_majority"

    def build(self, seed: int) -> DataSegment:
        return vocab_majority(**self.model_dump(), seed=seed)


def vocab_majority(vocab_size: int, num_examples: int, input_seq_len: int, seed: int, **kwargs) -> DataSegment:
    """Most frequent token of a random sequence over ``[1, V)``; ties are broken towards the smallest token by
    overwriting one occurrence of another token, so the answer is unique."""
    rng = np.random.RandomState(seed)
    seqs = rng.randint(1, vocab_size, size=(num_examples, input_seq_len - 1)).astype(np.int64)
    answers = np.zeros(num_examples, dtype=np.int64)
    for i, seq in enumerate(seqs):
        vals, counts = np.unique(seq, return_counts=True)
        top = vals[counts == counts.max()]
        answers[i] = top.min()
        if len(top) > 1:
            seq[np.argmax(seq != answers[i])] = answers[i]
    return _final_answer(seqs, 0, answers, {"vocab_size": vocab_size})


class CumulativeParityConfig(DataSegmentConfig):
    name: str = "cumulative_parity"

    def build(self, seed: int) -> DataSegment:
        return cumulative_parity(**self.model_dump(), seed=seed)


def cumulative_parity(vocab_size: int, num_examples: int, input_seq_len: int, seed: int, **kwargs) -> DataSegment:
    bits = np.random.RandomState(seed).randint(0, 2, size=(num_examples, input_seq_len - 1)).astype(np.int64)
    return DataSegment(torch.from_numpy(bits), torch.from_numpy(bits.cumsum(1) % 2), slices={"input_seq_len": input_seq_len})


class CumulativeMajorityConfig(DataSegmentConfig):
    num_examples: int = 1_000
    input_seq_len: int = 16
    name: str = "cumulative_majority"

    def build(self, seed: int) -> DataSegment:
        return cumulative_majority(self, seed=seed)


def cumulative_majority(config: CumulativeMajorityConfig, seed: int, **kwargs) -> DataSegment:
    bits = np.random.RandomState(seed).randint(0, 2, size=(config.num_examples, config.input_seq_len)).astype(np.int64)
    labels = ((bits * 2 - 1).cumsum(axis=1) >= 0).astype(np.int64)
    return DataSegment(torch.from_numpy(bits), torch.from_numpy(labels), slices={"input_seq_len": config.input_seq_len})
