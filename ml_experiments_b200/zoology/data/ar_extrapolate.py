"""Length / pair-count extrapolation splits for associative recall: several MQAR segments with different settings for
train and test, each tagged with its own configuration as slice keys (zoology/data/ar_extrapolate.py:10-64, whose
``_mqar`` helper no longer exists upstream; the segments here come from ``multiquery_ar``)."""
from __future__ import annotations

from typing import List

from pydantic import BaseModel

from .multiquery_ar import multiquery_ar
from .utils import DataSegment


class ARConfig(BaseModel):
    input_seq_len: int = 64
    num_examples: int = 1_000
    num_kv_pairs: int = 4
    num_queries: int = 4
    random_non_queries: bool = True


def ar_extrapolate(train_configs: List[ARConfig], test_configs: List[ARConfig], vocab_size: int = 8_192, seed: int = 0):
    """Returns ``(train_segments, test_segments)``; every segment's ``slices`` is its ``ARConfig`` as a dict."""
    def build(cfgs, offset):
        out = []
        for i, c in enumerate(cfgs):
            seg = multiquery_ar(vocab_size=vocab_size, num_examples=c.num_examples, input_seq_len=c.input_seq_len,
                                seed=seed + offset + i, num_kv_pairs=c.num_kv_pairs, random_non_queries=c.random_non_queries)
            out.append(DataSegment(seg.inputs, seg.labels, slices=c.model_dump()))
        return out
    return build(train_configs, 0), build(test_configs, len(train_configs))
