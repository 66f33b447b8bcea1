"""ByteMasker dataset: line / multi-line windows with per-byte secret masks and a leakage-free split.

Follows the reference's design (src/heuristic_secrets/bytemasker/dataset.py:23-922): windows are single lines,
multi-line windows of 2-9 lines (at most ``max_len`` bytes) or secret-only windows; every secret gets a content id
(``sha256[:16]``); windows that share a secret are connected (union-find) and whole components are assigned to
train / val / test so that no secret appears in two splits; batches are length-bucketed.
"""
from __future__ import annotations

import hashlib
import random
from dataclasses import dataclass, field

import torch

from ..data.types import SpanFinderSample

BUCKETS = (48, 80, 128, 288, 384, 512)


@dataclass
class MaskWindow:
    data: bytes
    mask: list[int]
    secret_ids: list[str] = field(default_factory=list)
    kind: str = "line"


def secret_id(raw: bytes) -> str:
    return hashlib.sha256(raw).hexdigest()[:16]


def windows_from_document(s: SpanFinderSample, max_len: int = 512, rng: random.Random | None = None) -> list[MaskWindow]:
    rng = rng or random.Random(0)
    raw = s.text.encode("utf-8")
    mask = bytearray(len(raw))
    spans = sorted(zip(s.starts, s.ends))
    for a, b in spans:
        mask[a:b] = b"\x01" * (b - a)
    # line boundaries
    bounds, pos = [], 0
    for line in raw.split(b"\n"):
        bounds.append((pos, pos + len(line)))
        pos += len(line) + 1
    out = []

    def make(a, b, kind):
        ids = [secret_id(raw[x:y]) for x, y in spans if x >= a and y <= b]
        out.append(MaskWindow(raw[a:b], list(mask[a:b]), ids, kind))

    for a, b in bounds:
        if 0 < b - a <= max_len:
            make(a, b, "line")
    i = 0
    while i < len(bounds):
        n = rng.randint(2, 9)
        a, b = bounds[i][0], bounds[min(i + n, len(bounds)) - 1][1]
        if 0 < b - a <= max_len:
            make(a, b, "multi")
        i += n
    for a, b in spans:
        if 0 < b - a <= max_len:
            make(a, b, "secret")
    return out


def stratified_component_split(windows: list[MaskWindow], fractions=(0.8, 0.1, 0.1), seed: int = 0):
    """Connected components over shared secret ids, assigned greedily to the split furthest below its quota."""
    parent = list(range(len(windows)))

    def find(x):
        while parent[x] != x:
            parent[x] = parent[parent[x]]
            x = parent[x]
        return x

    owner: dict[str, int] = {}
    for i, w in enumerate(windows):
        for sid in w.secret_ids:
            if sid in owner:
                ra, rb = find(i), find(owner[sid])
                if ra != rb:
                    parent[ra] = rb
            else:
                owner[sid] = i
    comps: dict[int, list[int]] = {}
    for i in range(len(windows)):
        comps.setdefault(find(i), []).append(i)
    groups = list(comps.values())
    random.Random(seed).shuffle(groups)
    groups.sort(key=len, reverse=True)
    splits: tuple[list, list, list] = ([], [], [])
    total = len(windows)
    for g in groups:
        deficits = [fractions[k] - len(splits[k]) / max(total, 1) for k in range(3)]
        k = max(range(3), key=lambda j: deficits[j])
        splits[k].extend(windows[i] for i in g)
    return splits


def create_bucketed_batches(windows: list[MaskWindow], batch_size: int = 64, shuffle: bool = True, seed: int | None = None):
    """Batches ``(byte_ids, masks, lengths)`` grouped by length bucket."""
    rng = random.Random(seed)
    buckets: dict[int, list[MaskWindow]] = {}
    for w in windows:
        b = next((x for x in BUCKETS if len(w.data) <= x), BUCKETS[-1])
        buckets.setdefault(b, []).append(w)
    batches = []
    for members in buckets.values():
        if shuffle:
            rng.shuffle(members)
        for k in range(0, len(members), batch_size):
            part = members[k:k + batch_size]
            lengths = torch.tensor([len(w.data) for w in part])
            L = int(lengths.max())
            ids = torch.zeros(len(part), L, dtype=torch.long)
            masks = torch.zeros(len(part), L)
            for r, w in enumerate(part):
                ids[r, : len(w.data)] = torch.frombuffer(bytearray(w.data), dtype=torch.uint8).long()
                masks[r, : len(w.data)] = torch.tensor(w.mask, dtype=torch.float32)
            batches.append((ids, masks, lengths))
    if shuffle:
        rng.shuffle(batches)
    return batches
