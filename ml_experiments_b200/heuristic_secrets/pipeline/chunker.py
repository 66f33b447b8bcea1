"""Fixed-size overlapping byte windows (reference: src/heuristic_secrets/pipeline/chunker.py:5-55)."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Iterator


@dataclass
class Chunk:
    data: bytes
    start: int
    end: int
    is_first: bool
    is_last: bool


class Chunker:
    def __init__(self, chunk_size: int = 512, overlap: int = 64):
        if overlap >= chunk_size:
            raise ValueError("overlap must be less than chunk_size")
        self.chunk_size, self.overlap = chunk_size, overlap
        self.stride = chunk_size - overlap

    def chunk(self, data: bytes) -> Iterator[Chunk]:
        n = len(data)
        if n == 0:
            return
        pos = 0
        while True:
            end = min(pos + self.chunk_size, n)
            last = end >= n
            yield Chunk(data=data[pos:end], start=pos, end=end, is_first=pos == 0, is_last=last)
            if last:
                return
            pos += self.stride
