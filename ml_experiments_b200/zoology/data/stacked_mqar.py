"""Continuous ("stacked") MQAR: every context position carries the concatenation of a key embedding and a value
embedding; query positions carry only the key half and the target is the index of the bound value
(zoology/data/stacked_mqar.py:8-96)."""
from __future__ import annotations

from typing import Any

import torch

from ..config import DataSegmentConfig
from .utils import DataSegment


class ContinuousMQARConfig(DataSegmentConfig):
    name: str = "continuous_mqar"
    num_kv_pairs: int = 8
    num_passes: int = 1
    per_sequence_mapping: bool = True
    embeddings: Any = None

    def build(self, seed: int) -> DataSegment:
        return continuous_mqar(self.num_examples, self.num_kv_pairs, self.num_passes, self.per_sequence_mapping, self.embeddings, seed)


def continuous_mqar(num_examples: int, num_kv_pairs: int, num_passes: int = 1, per_sequence_mapping: bool = True,
                    embeddings: torch.Tensor | None = None, seed: int = 42) -> DataSegment:
    g = torch.Generator().manual_seed(seed)
    embeddings = embeddings.detach().cpu()
    num_keys, dim = embeddings.shape[0] // 2, embeddings.shape[1]
    key_emb, value_emb = embeddings[:num_keys], embeddings[num_keys:]
    n, k = num_examples, num_kv_pairs
    rand_perm = lambda cols: torch.rand(n, cols, generator=g).argsort(dim=1)
    sel_keys, sel_vals = rand_perm(num_keys)[:, :k], rand_perm(num_keys)[:, :k]
    mapping = rand_perm(k) if per_sequence_mapping else torch.randperm(k, generator=g).expand(n, k)
    bound_vals = torch.gather(sel_vals, 1, mapping)  # value bound to local key j
    inputs = torch.zeros(n, (num_passes + 1) * k, 2 * dim)
    for p in range(num_passes):
        order = rand_perm(k)
        inputs[:, p * k:(p + 1) * k, :dim] = key_emb[torch.gather(sel_keys, 1, order)]
        inputs[:, p * k:(p + 1) * k, dim:] = value_emb[torch.gather(bound_vals, 1, order)]
    order = rand_perm(k)
    inputs[:, num_passes * k:, :dim] = key_emb[torch.gather(sel_keys, 1, order)]
    labels = torch.gather(bound_vals, 1, order)
    return DataSegment(inputs=inputs, labels=labels, slices={"num_kv_pairs": num_kv_pairs, "num_passes": num_passes})
