"""SpanFinder dataset: documents -> overlapping chunks with per-byte [start, inclusive end] labels
(reference: src/heuristic_secrets/spanfinder/dataset.py:44-205)."""
from __future__ import annotations

import json
import random
from dataclasses import dataclass
from pathlib import Path

import torch
from torch.utils.data import Dataset

from ..data.types import SpanFinderSample
from ..pipeline.chunker import Chunker


@dataclass
class ChunkedSample:
    """One chunk of a document with its span labels (the record type of the reference's dataset; this dataset keeps
    ``(byte_ids, targets)`` pairs and builds the record on request: :meth:`SpanFinderDataset.chunk`)."""
    byte_ids: torch.Tensor
    targets: torch.Tensor
    length: int
    is_first: bool = False
    is_last: bool = False


def load_jsonl(path) -> list[SpanFinderSample]:
    return [SpanFinderSample.from_dict(json.loads(line)) for line in open(path) if line.strip()]


class SpanFinderDataset(Dataset):
    def __init__(self, samples: list[SpanFinderSample], chunk_size: int = 512, chunk_overlap: int = 64):
        self.chunker = Chunker(chunk_size, chunk_overlap)
        self.items: list[tuple[torch.Tensor, torch.Tensor]] = []
        for s in samples:
            raw = s.text.encode("utf-8")
            for c in self.chunker.chunk(raw):
                ids = torch.frombuffer(bytearray(c.data), dtype=torch.uint8).long()
                tgt = torch.zeros(len(c.data), 2)
                for st, en in zip(s.starts, s.ends):
                    if c.start <= st < c.end:
                        tgt[st - c.start, 0] = 1.0
                    if c.start <= en - 1 < c.end:
                        tgt[en - 1 - c.start, 1] = 1.0
                self.items.append((ids, tgt))

    def __len__(self):
        return len(self.items)

    def chunk(self, i: int) -> ChunkedSample:
        ids, tgt = self.items[i]
        return ChunkedSample(ids, tgt, len(ids))

    def __getitem__(self, i):
        return self.items[i]


def collate_chunks(items):
    lengths = torch.tensor([len(x) for x, _ in items])
    L = int(lengths.max())
    ids = torch.zeros(len(items), L, dtype=torch.long)
    tgt = torch.zeros(len(items), L, 2)
    for i, (x, t) in enumerate(items):
        ids[i, : len(x)], tgt[i, : len(x)] = x, t
    return ids, tgt, lengths


def create_batches(ds: SpanFinderDataset, batch_size: int = 1024, shuffle: bool = True, seed: int | None = None):
    order = list(range(len(ds)))
    if shuffle:
        random.Random(seed).shuffle(order)
    return [collate_chunks([ds[i] for i in order[k:k + batch_size]]) for k in range(0, len(order), batch_size)]


@dataclass
class SpanFinderDatasetStats:
    total_samples: int
    total_chunks: int
    total_spans: int
    avg_chunks_per_sample: float
    chunk_size: int
    chunk_overlap: int


def load_spanfinder_dataset(data_dir: Path, split: str = "train", chunk_size: int = 512,
                            chunk_overlap: int = 64) -> tuple[SpanFinderDataset, SpanFinderDatasetStats]:
    """``(dataset, stats)`` of ``<data_dir>/splits/documents/<split>.jsonl`` cut into overlapping chunks."""
    path = Path(data_dir) / "splits" / "documents" / f"{split}.jsonl"
    samples = [SpanFinderSample.from_dict(json.loads(line)) for line in open(path) if line.strip()]
    ds = SpanFinderDataset(samples, chunk_size, chunk_overlap)
    stats = SpanFinderDatasetStats(len(samples), len(ds), sum(len(s.starts) for s in samples), len(ds) / len(samples) if samples else 0.0,
                                   chunk_size, chunk_overlap)
    return ds, stats
