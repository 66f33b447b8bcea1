"""Multi-query associative recall (Arora, Eyuboglu et al., "Zoology"): key/value pairs, then the keys re-appear as
queries at power-law distributed gaps and the model must emit the bound value (zoology/data/multiquery_ar.py:8-142).

Layout for ``num_kv_pairs=2, input_seq_len=16, random_non_queries=False``::

    inputs  k1 v1 k2 v2 0 0 k2 0 0 0 0 0 k1 0 0 ...      labels  -100 ... v2 ... v1 ...

Keys come from ``[1, V/2)``, values from ``[V/2, V)``; ``num_passes`` repeats the context (JRT). The generator is
vectorised over examples (no per-row ``np.random.choice``).
"""
from __future__ import annotations

import numpy as np
import torch

from ..config import DataSegmentConfig
from .utils import DataSegment, choice_without_replacement, fill_random_non_queries, power_law_gaps


class MQARConfig(DataSegmentConfig):
    name: str = "multiquery_ar"
    power_a: float = 0.01
    num_kv_pairs: int = 8
    num_passes: int = 1
    random_non_queries: bool = True
    include_slices: bool = True

    def build(self, seed: int) -> DataSegment:
        return multiquery_ar(**self.model_dump(), seed=seed)


def multiquery_ar(vocab_size: int, num_examples: int, input_seq_len: int, seed: int, power_a: float = 0.01, num_kv_pairs: int = 8,
                  num_passes: int = 1, random_non_queries: bool = True, include_slices: bool = True, **kwargs) -> DataSegment:
    assert input_seq_len % 2 == 0, "input_seq_len must be even"
    assert vocab_size > input_seq_len
    assert num_kv_pairs * 2 * num_passes + num_kv_pairs * 2 <= input_seq_len
    rng = np.random.RandomState(seed)
    context = num_kv_pairs * 2 * num_passes
    half = vocab_size // 2
    keys = choice_without_replacement(rng, np.arange(1, half), num_examples, num_kv_pairs)
    values = choice_without_replacement(rng, np.arange(half, vocab_size), num_examples, num_kv_pairs)
    kvs = np.zeros((num_examples, num_kv_pairs * 2), dtype=np.int64)
    kvs[:, 0::2], kvs[:, 1::2] = keys, values
    kvs = np.tile(kvs, (1, num_passes))
    gaps = power_law_gaps(rng, (input_seq_len - context) // 2, power_a, num_examples, num_kv_pairs)
    queries = np.zeros((num_examples, input_seq_len - context + 1), dtype=np.int64)
    np.put_along_axis(queries, gaps * 2, keys, axis=1)
    examples = np.concatenate([kvs, queries], axis=1)
    labels = np.full((num_examples, input_seq_len + 1), -100, dtype=np.int64)
    np.put_along_axis(labels, gaps * 2 + context + 1, values, axis=1)
    inputs, labels = torch.from_numpy(examples[:, :-1].copy()), torch.from_numpy(labels[:, 1:].copy())
    if random_non_queries:
        inputs = fill_random_non_queries(inputs, vocab_size, seed)
    slices = {"num_kv_pairs": num_kv_pairs, "input_seq_len": input_seq_len, "num_passes": num_passes}
    return DataSegment(inputs, labels, slices=slices if include_slices else {})
