"""Compositional MQAR: compound keys ``(K1, K2) -> V`` laid out on a ``g x g`` grid so that neither key component alone
determines the value (zoology/data/compositional_mqar.py:8-150). Vocabulary thirds: K1, K2, values."""
from __future__ import annotations

import numpy as np
import torch

from ..config import DataSegmentConfig
from .utils import DataSegment, choice_without_replacement, fill_random_non_queries, power_law_gaps


class CompositionalMQARConfig(DataSegmentConfig):
    name: str = "compositional_mqar"
    power_a: float = 0.01
    num_kv_pairs: int = 4  # a perfect square
    random_non_queries: bool = True
    include_slices: bool = True

    def build(self, seed: int) -> DataSegment:
        return compositional_mqar(**self.model_dump(), seed=seed)


def compositional_mqar(vocab_size: int, num_examples: int, input_seq_len: int, seed: int, power_a: float = 0.01,
                       num_kv_pairs: int = 4, random_non_queries: bool = True, include_slices: bool = True, **kwargs) -> DataSegment:
    assert input_seq_len % 2 == 0, "input_seq_len must be even"
    assert vocab_size > input_seq_len
    assert num_kv_pairs * 6 <= input_seq_len, f"Need at least 6 tokens per kv pair. Got {input_seq_len} for {num_kv_pairs} pairs."
    g = int(round(np.sqrt(num_kv_pairs)))
    assert g * g == num_kv_pairs, f"num_kv_pairs must be a perfect square (e.g., 4, 9, 16). Got {num_kv_pairs}."
    rng = np.random.RandomState(seed)
    context, third = num_kv_pairs * 3, vocab_size // 3
    k1_set = choice_without_replacement(rng, np.arange(1, third), num_examples, g)
    k2_set = choice_without_replacement(rng, np.arange(third, 2 * third), num_examples, g)
    perm = np.argsort(rng.random_sample((num_examples, num_kv_pairs)), axis=1)
    k1s = np.take_along_axis(np.repeat(k1_set, g, axis=1), perm, axis=1)
    k2s = np.take_along_axis(np.tile(k2_set, (1, g)), perm, axis=1)
    values = choice_without_replacement(rng, np.arange(2 * third, vocab_size), num_examples, num_kv_pairs)
    kvs = np.zeros((num_examples, context), dtype=np.int64)
    kvs[:, 0::3], kvs[:, 1::3], kvs[:, 2::3] = k1s, k2s, values
    gaps = power_law_gaps(rng, (input_seq_len - context) // 3, power_a, num_examples, num_kv_pairs)
    queries = np.zeros((num_examples, input_seq_len - context + 1), dtype=np.int64)
    np.put_along_axis(queries, gaps * 3, k1s, axis=1)
    np.put_along_axis(queries, gaps * 3 + 1, k2s, axis=1)
    examples = np.concatenate([kvs, queries], axis=1)
    labels = np.full((num_examples, input_seq_len + 1), -100, dtype=np.int64)
    np.put_along_axis(labels, gaps * 3 + context + 2, values, axis=1)
    inputs, labels = torch.from_numpy(examples[:, :-1].copy()), torch.from_numpy(labels[:, 1:].copy())
    if random_non_queries:
        inputs = fill_random_non_queries(inputs, vocab_size, seed)
    return DataSegment(inputs, labels, slices={"num_kv_pairs": num_kv_pairs, "input_seq_len": input_seq_len} if include_slices else {})
