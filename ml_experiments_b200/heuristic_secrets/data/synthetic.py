"""Synthetic sequence tasks (vectorised numpy generators): ``mqar``, ``compositional_mqar``, ``forgetting_mqar``,
``parity``, ``cumulative_parity``, ``majority``, ``cumulative_majority``, ``copying``, ``selective_copying``,
``induction_heads``; labels are ``-100`` wherever no prediction is scored.

Task definitions, argument names, ``TASKS`` and ``load_task`` follow the reference
(src/heuristic_secrets/data/synthetic.py:33-522). Whole batches of examples are generated with array operations
instead of a Python loop per example, so the random streams differ from the reference at equal seed while the task
distributions are the same.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np
import torch
from torch.utils.data import DataLoader, Dataset

IGNORE = -100


@dataclass
class SyntheticData:
    inputs: torch.Tensor
    labels: torch.Tensor
    task: str
    config: dict = field(default_factory=dict)


class SyntheticDataset(Dataset):
    def __init__(self, data: SyntheticData):
        self.data = data

    def __len__(self):
        return self.data.inputs.shape[0]

    def __getitem__(self, i):
        return self.data.inputs[i], self.data.labels[i]


def _pack(inp, lab, task, **cfg) -> SyntheticData:
    return SyntheticData(torch.from_numpy(np.ascontiguousarray(inp)).long(), torch.from_numpy(np.ascontiguousarray(lab)).long(), task, cfg)


def _distinct(rng, n, hi, k):
    """``n`` rows of ``k`` distinct integers from ``[0, hi)``."""
    return np.argsort(rng.random((n, hi)), axis=1)[:, :k]


def mqar(vocab_size=256, seq_len=64, num_kv_pairs=8, num_examples=10000, power_a=0.01, random_non_queries=True, seed=42):
    rng = np.random.default_rng(seed)
    kv, n, half = num_kv_pairs, num_examples, vocab_size // 2
    keys = _distinct(rng, n, half, kv)
    vals = rng.integers(half, vocab_size, size=(n, kv))
    p = None
    if power_a > 0:
        p = np.arange(1, kv + 1, dtype=np.float64) ** (-power_a)
        p /= p.sum()
    qi = rng.choice(kv, size=(n, kv), replace=True, p=p)
    inp = rng.integers(0, half, size=(n, seq_len)) if random_non_queries else np.zeros((n, seq_len), dtype=np.int64)
    inp[:, 0:2 * kv:2], inp[:, 1:2 * kv:2] = keys, vals
    inp[:, seq_len - kv:] = np.take_along_axis(keys, qi, 1)
    lab = np.full((n, seq_len), IGNORE, dtype=np.int64)
    lab[:, seq_len - kv:] = np.take_along_axis(vals, qi, 1)
    return _pack(inp, lab, "mqar", vocab_size=vocab_size, seq_len=seq_len, num_kv_pairs=kv)


def compositional_mqar(vocab_size=256, seq_len=64, num_kv_pairs=8, num_examples=10000, seed=42):
    """Two-hop recall: pairs ``(k, m)`` and ``(m, v)`` are given; a query ``k`` must return ``v``."""
    rng = np.random.default_rng(seed)
    kv, n, third = num_kv_pairs, num_examples, vocab_size // 3
    keys = _distinct(rng, n, third, kv)
    mids = _distinct(rng, n, third, kv) + third
    vals = rng.integers(2 * third, vocab_size, size=(n, kv))
    inp = rng.integers(0, third, size=(n, seq_len))
    inp[:, 0:2 * kv:2], inp[:, 1:2 * kv:2] = keys, mids
    inp[:, 2 * kv:4 * kv:2], inp[:, 2 * kv + 1:4 * kv:2] = mids, vals
    qi = rng.integers(0, kv, size=(n, kv))
    inp[:, seq_len - kv:] = np.take_along_axis(keys, qi, 1)
    lab = np.full((n, seq_len), IGNORE, dtype=np.int64)
    lab[:, seq_len - kv:] = np.take_along_axis(vals, qi, 1)
    return _pack(inp, lab, "compositional_mqar", vocab_size=vocab_size, seq_len=seq_len, num_kv_pairs=kv)


def forgetting_mqar(vocab_size=256, seq_len=64, num_kv_pairs=8, num_examples=10000, overwrite_frac=0.5, seed=42):
    """Some keys are bound twice; the later binding is the answer."""
    rng = np.random.default_rng(seed)
    kv, n, half = num_kv_pairs, num_examples, vocab_size // 2
    keys = _distinct(rng, n, half, kv)
    v1 = rng.integers(half, vocab_size, size=(n, kv))
    v2 = rng.integers(half, vocab_size, size=(n, kv))
    over = rng.random((n, kv)) < overwrite_frac
    inp = rng.integers(0, half, size=(n, seq_len))
    inp[:, 0:2 * kv:2], inp[:, 1:2 * kv:2] = keys, v1
    inp[:, 2 * kv:4 * kv:2] = np.where(over, keys, inp[:, 2 * kv:4 * kv:2])
    inp[:, 2 * kv + 1:4 * kv:2] = np.where(over, v2, inp[:, 2 * kv + 1:4 * kv:2])
    qi = rng.integers(0, kv, size=(n, kv))
    inp[:, seq_len - kv:] = np.take_along_axis(keys, qi, 1)
    lab = np.full((n, seq_len), IGNORE, dtype=np.int64)
    lab[:, seq_len - kv:] = np.take_along_axis(np.where(over, v2, v1), qi, 1)
    return _pack(inp, lab, "forgetting_mqar", vocab_size=vocab_size, seq_len=seq_len, num_kv_pairs=kv)


def parity(seq_len=64, num_examples=10000, seed=42, vocab_size=2):
    rng = np.random.default_rng(seed)
    inp = rng.integers(0, 2, size=(num_examples, seq_len))
    lab = np.full((num_examples, seq_len), IGNORE, dtype=np.int64)
    lab[:, -1] = inp.sum(1) % 2
    return _pack(inp, lab, "parity", vocab_size=2, seq_len=seq_len)


def cumulative_parity(seq_len=64, num_examples=10000, seed=42, vocab_size=2):
    rng = np.random.default_rng(seed)
    inp = rng.integers(0, 2, size=(num_examples, seq_len))
    return _pack(inp, np.cumsum(inp, 1) % 2, "cumulative_parity", vocab_size=2, seq_len=seq_len)


def majority(seq_len=64, num_examples=10000, seed=42, vocab_size=2):
    rng = np.random.default_rng(seed)
    inp = rng.integers(0, 2, size=(num_examples, seq_len))
    lab = np.full((num_examples, seq_len), IGNORE, dtype=np.int64)
    lab[:, -1] = (inp.sum(1) * 2 > seq_len).astype(np.int64)
    return _pack(inp, lab, "majority", vocab_size=2, seq_len=seq_len)


def cumulative_majority(seq_len=64, num_examples=10000, seed=42, vocab_size=2):
    rng = np.random.default_rng(seed)
    inp = rng.integers(0, 2, size=(num_examples, seq_len))
    ones = np.cumsum(inp, 1)
    lab = (ones * 2 > np.arange(1, seq_len + 1)[None, :]).astype(np.int64)
    return _pack(inp, lab, "cumulative_majority", vocab_size=2, seq_len=seq_len)


def copying(vocab_size=256, seq_len=64, num_tokens=16, num_examples=10000, seed=42):
    """``tokens ... blanks ... <copy> blanks``; the model must reproduce the tokens after the copy marker."""
    rng = np.random.default_rng(seed)
    num_tokens = min(num_tokens, (seq_len - 1) // 2)
    n, blank, marker = num_examples, vocab_size - 2, vocab_size - 1
    toks = rng.integers(0, vocab_size - 2, size=(n, num_tokens))
    inp = np.full((n, seq_len), blank, dtype=np.int64)
    inp[:, :num_tokens] = toks
    inp[:, seq_len - num_tokens - 1] = marker
    lab = np.full((n, seq_len), IGNORE, dtype=np.int64)
    lab[:, seq_len - num_tokens:] = toks
    return _pack(inp, lab, "copying", vocab_size=vocab_size, seq_len=seq_len, num_tokens=num_tokens)


def selective_copying(vocab_size=256, seq_len=64, num_tokens=16, num_examples=10000, seed=42):
    """Tokens are scattered among blanks at random positions and must be reproduced in order."""
    rng = np.random.default_rng(seed)
    num_tokens = min(num_tokens, (seq_len - 1) // 2)
    n, blank, marker = num_examples, vocab_size - 2, vocab_size - 1
    body = seq_len - num_tokens - 1
    toks = rng.integers(0, vocab_size - 2, size=(n, num_tokens))
    where = np.sort(_distinct(rng, n, body, num_tokens), axis=1)
    inp = np.full((n, seq_len), blank, dtype=np.int64)
    np.put_along_axis(inp, where, toks, 1)
    inp[:, body] = marker
    lab = np.full((n, seq_len), IGNORE, dtype=np.int64)
    lab[:, seq_len - num_tokens:] = toks
    return _pack(inp, lab, "selective_copying", vocab_size=vocab_size, seq_len=seq_len, num_tokens=num_tokens)


def induction_heads(vocab_size=256, seq_len=64, num_examples=10000, seed=42, num_triggers=1):
    """A trigger token appears once mid-sequence followed by a payload; at the end the trigger reappears and the
    payload must be predicted."""
    rng = np.random.default_rng(seed)
    n, trigger = num_examples, vocab_size - 1
    inp = rng.integers(0, vocab_size - 1, size=(n, seq_len))
    pos = rng.integers(1, seq_len - 3, size=n)
    rows = np.arange(n)
    inp[rows, pos] = trigger
    payload = inp[rows, pos + 1]
    inp[:, -1] = trigger
    lab = np.full((n, seq_len), IGNORE, dtype=np.int64)
    lab[:, -1] = payload
    return _pack(inp, lab, "induction_heads", vocab_size=vocab_size, seq_len=seq_len)


TASKS = {"mqar": mqar, "compositional_mqar": compositional_mqar, "forgetting_mqar": forgetting_mqar, "parity": parity,
         "cumulative_parity": cumulative_parity, "majority": majority, "cumulative_majority": cumulative_majority,
         "copying": copying, "selective_copying": selective_copying, "induction_heads": induction_heads}
_BINARY = ("parity", "cumulative_parity", "majority", "cumulative_majority")


def load_task(task: str, seq_len: int = 128, num_train: int = 50000, num_test: int = 10000, batch_size: int = 64,
              seed: int = 42, **kwargs):
    if task not in TASKS:
        raise ValueError(f"Unknown task: {task}. Available: {list(TASKS.keys())}")
    common = dict(seq_len=seq_len, **kwargs)
    if "vocab_size" not in kwargs and task not in _BINARY:
        common["vocab_size"] = 256
    train = TASKS[task](num_examples=num_train, seed=seed, **common)
    test = TASKS[task](num_examples=num_test, seed=seed + 1000, **common)
    return (DataLoader(SyntheticDataset(train), batch_size=batch_size, shuffle=True, num_workers=0),
            DataLoader(SyntheticDataset(test), batch_size=batch_size, shuffle=False, num_workers=0), train.config)
