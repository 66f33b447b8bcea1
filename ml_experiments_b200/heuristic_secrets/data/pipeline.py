"""De-duplication, stratified splitting and JSONL IO of samples (reference: src/heuristic_secrets/data/pipeline.py)."""
from __future__ import annotations

import json
import random
from collections import defaultdict
from pathlib import Path
from typing import Iterator, Type, TypeVar

from .types import SpanFinderSample, ValidatorSample

T = TypeVar("T", ValidatorSample, SpanFinderSample)


def deduplicate_samples(samples: list[T]) -> list[T]:
    seen: set[str] = set()
    out = []
    for s in samples:
        if s.text not in seen:
            seen.add(s.text)
            out.append(s)
    return out


def split_samples(samples: list[T], train: float = 0.8, val: float = 0.1, test: float = 0.1, seed: int | None = None,
                  stratify: bool = True) -> tuple[list[T], list[T], list[T]]:
    assert abs(train + val + test - 1.0) < 0.01, "Splits must sum to 1.0"
    rng = random.Random(seed)
    groups: dict[str, list[T]] = defaultdict(list)
    for s in samples:
        groups[getattr(s, "category", "unknown") if stratify else "all"].append(s)
    parts: tuple[list[T], list[T], list[T]] = ([], [], [])
    for members in groups.values():
        members = list(members)
        rng.shuffle(members)
        a = int(len(members) * train)
        b = a + int(len(members) * val)
        parts[0].extend(members[:a])
        parts[1].extend(members[a:b])
        parts[2].extend(members[b:])
    for p in parts:
        rng.shuffle(p)
    return parts


def write_jsonl(samples: list[T], filepath: Path) -> None:
    filepath = Path(filepath)
    filepath.parent.mkdir(parents=True, exist_ok=True)
    with open(filepath, "w") as f:
        for s in samples:
            f.write(json.dumps(s.to_dict()) + "\n")


def read_jsonl(filepath: Path, sample_type: Type[T]) -> Iterator[T]:
    with open(filepath) as f:
        for line in f:
            if line.strip():
                yield sample_type.from_dict(json.loads(line))
