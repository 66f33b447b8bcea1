"""Turns per-byte [start, end] probabilities into spans (reference: src/heuristic_secrets/pipeline/assembler.py).

For every predicted start the first predicted end that gives a length in ``[min_length, max_length]`` closes the span;
unmatched starts / leading ends at chunk edges become partial spans. Span ``end`` is exclusive.
"""
from __future__ import annotations

import bisect
from dataclasses import dataclass
from typing import Optional

import torch


@dataclass
class Span:
    start: Optional[int]
    end: Optional[int]

    @property
    def is_partial(self) -> bool:
        return self.start is None or self.end is None

    @property
    def length(self) -> Optional[int]:
        return None if self.is_partial else self.end - self.start


class SpanAssembler:
    def __init__(self, threshold: float = 0.5, min_length: int = 8, max_length: int = 256):
        self.threshold, self.min_length, self.max_length = threshold, min_length, max_length

    def extract_spans(self, predictions: torch.Tensor, chunk_start: int = 0, is_first_chunk: bool = True,
                      is_last_chunk: bool = True) -> list[Span]:
        if predictions.numel() and (predictions.min() < 0 or predictions.max() > 1):
            predictions = torch.sigmoid(predictions)
        hits = predictions >= self.threshold
        starts = hits[:, 0].nonzero(as_tuple=True)[0].tolist()
        ends = hits[:, 1].nonzero(as_tuple=True)[0].tolist()
        spans: list[Span] = []
        if not is_first_chunk and ends and (not starts or starts[0] > ends[0]):
            spans.append(Span(start=None, end=chunk_start + ends[0] + 1))
        for s in starts:
            # first end position e with min_length <= e - s + 1 <= max_length (ends is sorted)
            k = bisect.bisect_left(ends, s + self.min_length - 1)
            if k < len(ends) and ends[k] - s + 1 <= self.max_length:
                spans.append(Span(start=chunk_start + s, end=chunk_start + ends[k] + 1))
            elif not is_last_chunk:
                spans.append(Span(start=chunk_start + s, end=None))
        return spans
