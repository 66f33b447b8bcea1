"""Forgetting MQAR: ``num_updates`` of the keys are bound a second time to a new value after the first pass; queries
must return the most recent binding (zoology/data/forgetting_mqar.py:8-170)."""
from __future__ import annotations

import numpy as np
import torch

from ..config import DataSegmentConfig
from .utils import DataSegment, choice_without_replacement, fill_random_non_queries, power_law_gaps


class ForgettingMQARConfig(DataSegmentConfig):
    name: str = "forgetting_mqar"
    power_a: float = 0.01
    num_kv_pairs: int = 8
    num_updates: int = 4
    random_non_queries: bool = True
    include_slices: bool = True

    def build(self, seed: int) -> DataSegment:
        return forgetting_mqar(**self.model_dump(), seed=seed)


def forgetting_mqar(vocab_size: int, num_examples: int, input_seq_len: int, seed: int, power_a: float = 0.01, num_kv_pairs: int = 8,
                    num_updates: int = 4, random_non_queries: bool = True, include_slices: bool = True, **kwargs) -> DataSegment:
    assert input_seq_len % 2 == 0, "input_seq_len must be even"
    assert vocab_size > input_seq_len
    assert num_updates <= num_kv_pairs, "num_updates must be <= num_kv_pairs"
    context = (num_kv_pairs + num_updates) * 2
    assert context + num_kv_pairs * 2 <= input_seq_len, "sequence too short for the context, the updates and the queries"
    rng = np.random.RandomState(seed)
    half = vocab_size // 2
    keys = choice_without_replacement(rng, np.arange(1, half), num_examples, num_kv_pairs)
    # distinct old and new values: draw num_kv_pairs + num_updates distinct values, the tail are the replacements
    vals = choice_without_replacement(rng, np.arange(half, vocab_size), num_examples, num_kv_pairs + num_updates)
    original, updated = vals[:, :num_kv_pairs], vals[:, num_kv_pairs:]
    upd_idx = choice_without_replacement(rng, np.arange(num_kv_pairs), num_examples, num_updates)
    final = original.copy()
    np.put_along_axis(final, upd_idx, updated, axis=1)
    first = np.zeros((num_examples, num_kv_pairs * 2), dtype=np.int64)
    first[:, 0::2], first[:, 1::2] = keys, original
    second = np.zeros((num_examples, num_updates * 2), dtype=np.int64)
    second[:, 0::2], second[:, 1::2] = np.take_along_axis(keys, upd_idx, axis=1), updated
    kvs = np.concatenate([first, second], axis=1)
    gaps = power_law_gaps(rng, (input_seq_len - context) // 2, power_a, num_examples, num_kv_pairs)
    queries = np.zeros((num_examples, input_seq_len - context + 1), dtype=np.int64)
    np.put_along_axis(queries, gaps * 2, keys, axis=1)
    examples = np.concatenate([kvs, queries], axis=1)
    labels = np.full((num_examples, input_seq_len + 1), -100, dtype=np.int64)
    np.put_along_axis(labels, gaps * 2 + context + 1, final, axis=1)
    inputs, labels = torch.from_numpy(examples[:, :-1].copy()), torch.from_numpy(labels[:, 1:].copy())
    if random_non_queries:
        inputs = fill_random_non_queries(inputs, vocab_size, seed)
    slices = {"num_kv_pairs": num_kv_pairs, "num_updates": num_updates, "input_seq_len": input_seq_len}
    return DataSegment(inputs, labels, slices=slices if include_slices else {})
