"""``DataSegment`` (with an md5-keyed on-disk cache), per-segment seeding and the batch-returning dataset
(zoology/data/utils.py:14-177). Train segments draw seeds from the lower half of the 32-bit range and test segments
from the upper half, so a train and a test segment can never share a seed."""
from __future__ import annotations

import hashlib
import json
import os
from dataclasses import asdict, dataclass
from pathlib import Path
from typing import Any, Dict, List, Tuple

import numpy as np
import torch
from torch.utils.data import DataLoader, Dataset

from ..config import DataConfig, DataSegmentConfig


@dataclass
class DataSegment:
    inputs: torch.Tensor
    labels: torch.Tensor
    slices: Dict[str, Any] | None = None

    def __len__(self):
        assert len(self.inputs) == len(self.labels)
        return len(self.inputs)

    @classmethod
    def from_config(cls, config: DataSegmentConfig, cache_dir: str | None = None, force_cache: bool = False, seed: int = 123):
        path = None
        if cache_dir is not None:
            try:
                Path(cache_dir).mkdir(exist_ok=True, parents=True)
                dump = {k: v for k, v in config.model_dump().items() if not isinstance(v, torch.Tensor)}
                key = hashlib.md5(json.dumps({**dump, "_seed": seed}, sort_keys=True, default=str).encode()).hexdigest()
                path = os.path.join(cache_dir, f"data_{key}.pt")
            except OSError:
                print(f"Could not create cache directory {cache_dir}")
        if path is not None and os.path.exists(path) and not force_cache:
            return cls(**torch.load(path, weights_only=False))
        data = config.build(seed=seed)
        if path is not None:
            tmp = f"{path}.tmp.{os.getpid()}"
            torch.save(asdict(data), tmp)
            os.replace(tmp, path)
        return data


class _SyntheticDataset(Dataset):
    """Returns whole batches; a batch never mixes two segments."""

    def __init__(self, segments: List[DataSegment], batch_size: int):
        self.segments, self.batch_size = segments, batch_size
        self.batches = [(i, s) for i, seg in enumerate(segments) for s in range(0, len(seg), batch_size)]

    def __getitem__(self, idx: int):
        seg_idx, start = self.batches[idx]
        seg = self.segments[seg_idx]
        sl = slice(start, start + self.batch_size)
        inputs = seg.inputs[sl]
        return inputs, seg.labels[sl], [seg.slices or {}] * len(inputs)

    def __len__(self):
        return len(self.batches)


def _split_batch_size(bs) -> Tuple[int, int]:
    return (bs, bs) if isinstance(bs, int) else tuple(bs)


def _loaders(config: DataConfig, factory_kwargs: dict):
    train_bs, test_bs = _split_batch_size(config.batch_size)
    rng = np.random.RandomState(config.seed)
    max_seed = 2 ** 32
    train_seeds = rng.randint(0, max_seed // 2, size=len(config.train_configs), dtype=np.int64)
    test_seeds = rng.randint(max_seed // 2, max_seed, size=len(config.test_configs), dtype=np.int64)
    make = lambda cfgs, seeds, bs: DataLoader(
        _SyntheticDataset([DataSegment.from_config(c, seed=int(s), **factory_kwargs) for c, s in zip(cfgs, seeds)], bs),
        batch_size=None, num_workers=0, shuffle=False)
    return make(config.train_configs, train_seeds, train_bs), make(config.test_configs, test_seeds, test_bs)


def prepare_data(config: DataConfig):
    return _loaders(config, {"cache_dir": config.cache_dir, "force_cache": config.force_cache})


def prepare_continuous_data(config: DataConfig, embeddings: torch.Tensor):
    for cfg in list(config.train_configs) + list(config.test_configs):
        cfg.embeddings = embeddings
    return _loaders(config, {"cache_dir": None, "force_cache": False})


# --- vectorised sampling helpers shared by the task generators --------------------------------------------------------
def choice_without_replacement(rng: np.random.RandomState, pool: np.ndarray, rows: int, k: int) -> np.ndarray:
    """``rows`` independent draws of ``k`` distinct items from ``pool`` (uniform)."""
    keys = rng.random_sample((rows, len(pool)))
    idx = np.argpartition(keys, k - 1, axis=1)[:, :k]
    order = np.take_along_axis(keys, idx, axis=1).argsort(axis=1)  # random order among the k chosen
    return pool[np.take_along_axis(idx, order, axis=1)]


def weighted_choice_without_replacement(rng: np.random.RandomState, p: np.ndarray, rows: int, k: int) -> np.ndarray:
    """``rows`` draws of ``k`` distinct indices with probabilities ``p`` (successive sampling, via Gumbel top-k)."""
    g = np.log(p)[None, :] + rng.gumbel(size=(rows, len(p)))
    return np.argsort(-g, axis=1)[:, :k]


def power_law_gaps(rng, space: int, power_a: float, rows: int, k: int) -> np.ndarray:
    p = power_a * np.arange(1, space + 1) ** (power_a - 1)
    return weighted_choice_without_replacement(rng, p / p.sum(), rows, k)


def fill_random_non_queries(inputs: torch.Tensor, vocab_size: int, seed: int) -> torch.Tensor:
    g = torch.Generator().manual_seed(seed)
    noise = torch.randint(vocab_size, inputs.shape, generator=g)
    return torch.where(inputs == 0, noise, inputs)
