"""Validator dataset: JSONL samples -> heuristic features + byte ids, length-bucketed batches, md5-keyed cache
(reference: src/heuristic_secrets/validator/dataset.py:31-346)."""
from __future__ import annotations

import hashlib
import json
import random
from dataclasses import dataclass
from pathlib import Path

import torch
from torch.utils.data import Dataset

from ..data.types import ValidatorSample
from .features import FrequencyTable, extract_features

BUCKETS = (64, 128, 256, 512, 1024, 2048, 4096)
CACHE_DIR = Path(".cache/validator")
VALIDATOR_MAX_BYTE_LEN = 4096
LENGTH_BINS = list(BUCKETS)      # the name the reference uses for the same edges


@dataclass
class ValidatorDatasetStats:
    total: int = 0
    positives: int = 0
    negatives: int = 0


def load_jsonl(path: Path) -> list[ValidatorSample]:
    with open(path) as f:
        return [ValidatorSample.from_dict(json.loads(line)) for line in f if line.strip()]


def build_frequency_table(samples: list[ValidatorSample], label: int | None = None) -> FrequencyTable:
    data = b"".join(s.text.encode("utf-8") for s in samples if label is None or s.label == label)
    return FrequencyTable.from_data(data)


def build_text_freq_from_documents(data_dir: Path) -> FrequencyTable:
    """Byte frequencies of the non-secret parts of the training documents."""
    path = Path(data_dir) / "splits" / "documents" / "train.jsonl"
    chunks = []
    if path.exists():
        for line in open(path):
            if not line.strip():
                continue
            d = json.loads(line)
            raw, pos = d["text"].encode("utf-8"), 0
            for s, e in sorted(zip(d.get("starts", []), d.get("ends", []))):
                chunks.append(raw[pos:s])
                pos = max(pos, e)
            chunks.append(raw[pos:])
    return FrequencyTable.from_data(b"".join(chunks))


class ValidatorDataset(Dataset):
    def __init__(self, samples: list[ValidatorSample], text_freq: FrequencyTable, innocuous_freq: FrequencyTable,
                 secret_freq: FrequencyTable, feature_indices: list[int] | None = None, max_byte_len: int = 4096):
        self.samples, self.max_byte_len, self.feature_indices = samples, max_byte_len, feature_indices
        feats, ids = [], []
        for s in samples:
            raw = s.text.encode("utf-8")[:max_byte_len]
            f = extract_features(raw, text_freq, innocuous_freq, secret_freq).to_list()
            feats.append([f[i] for i in feature_indices] if feature_indices is not None else f)
            ids.append(torch.frombuffer(bytearray(raw), dtype=torch.uint8).long() if raw else torch.zeros(0, dtype=torch.long))
        self.features = torch.tensor(feats, dtype=torch.float32).reshape(len(samples), -1)
        self.byte_ids = ids
        self.labels = torch.tensor([s.label for s in samples], dtype=torch.float32)

    def stats(self) -> ValidatorDatasetStats:
        pos = int(self.labels.sum())
        return ValidatorDatasetStats(len(self.samples), pos, len(self.samples) - pos)

    def __len__(self):
        return len(self.samples)

    def __getitem__(self, i):
        return self.features[i], self.byte_ids[i], self.labels[i]


def create_bucketed_batches(ds: ValidatorDataset, batch_size: int = 64, shuffle: bool = True, seed: int | None = None):
    """Batches ``(features, byte_ids, lengths, labels)`` whose members share a length bucket (less padding)."""
    rng = random.Random(seed)
    buckets: dict[int, list[int]] = {}
    for i, ids in enumerate(ds.byte_ids):
        b = next((x for x in BUCKETS if len(ids) <= x), BUCKETS[-1])
        buckets.setdefault(b, []).append(i)
    batches = []
    for members in buckets.values():
        if shuffle:
            rng.shuffle(members)
        for k in range(0, len(members), batch_size):
            idx = members[k:k + batch_size]
            lengths = torch.tensor([max(len(ds.byte_ids[i]), 1) for i in idx])
            ids = torch.zeros(len(idx), int(lengths.max()), dtype=torch.long)
            for r, i in enumerate(idx):
                ids[r, : len(ds.byte_ids[i])] = ds.byte_ids[i]
            batches.append((ds.features[idx], ids, lengths, ds.labels[idx]))
    if shuffle:
        rng.shuffle(batches)
    return batches


def _cache_key(data_dir: Path, split: str, feature_indices, max_byte_len: int) -> str:
    p = Path(data_dir) / "splits" / "validator" / f"{split}.jsonl"
    h = hashlib.md5()
    h.update(f"{p}:{p.stat().st_mtime_ns if p.exists() else 0}:{feature_indices}:{max_byte_len}".encode())
    return h.hexdigest()


def load_validator_dataset(data_dir: Path, split: str = "train", feature_indices: list[int] | None = None,
                           max_byte_len: int = 4096, tables: dict | None = None, cache: bool = True):
    """Returns ``(dataset, tables)``; frequency tables are built from the training split when not supplied."""
    data_dir = Path(data_dir)
    cache_file = data_dir / ".cache" / "validator" / f"{_cache_key(data_dir, split, feature_indices, max_byte_len)}.pt"
    if cache and cache_file.exists() and tables is None:
        return torch.load(cache_file, weights_only=False)
    samples = load_jsonl(data_dir / "splits" / "validator" / f"{split}.jsonl")
    own_tables = tables is None
    if tables is None:
        train = samples if split == "train" else load_jsonl(data_dir / "splits" / "validator" / "train.jsonl")
        tables = {"text": build_text_freq_from_documents(data_dir), "innocuous": build_frequency_table(train, 0),
                  "secret": build_frequency_table(train, 1)}
    ds = ValidatorDataset(samples, tables["text"], tables["innocuous"], tables["secret"], feature_indices, max_byte_len)
    if cache and own_tables:
        cache_file.parent.mkdir(parents=True, exist_ok=True)
        torch.save((ds, tables), cache_file)
    return ds, tables
