"""The six heuristic features of the Validator, computed on 256-bin byte histograms.

Same definitions and values as the reference (src/heuristic_secrets/validator/features.py:7-182): Shannon entropy in
bits per byte, Huffman-coded size over raw size ("kolmogorov complexity"), L2 distance between the byte-frequency
vector and three reference tables (text / innocuous / secret), and the fraction of adjacent byte pairs whose character
class (letter / digit / other) differs. Histograms and table distances are numpy vectors instead of Python dicts; the
Huffman size is the sum of the merged weights of the code tree, so no code strings are built.
"""
from __future__ import annotations

import heapq
import math
from dataclasses import dataclass, field
from typing import NamedTuple

import numpy as np

_CLASS = np.full(256, 2, dtype=np.int8)
_CLASS[65:91] = 0
_CLASS[97:123] = 0
_CLASS[48:58] = 1


def _hist(data: bytes) -> np.ndarray:
    return np.bincount(np.frombuffer(data, dtype=np.uint8), minlength=256)


def shannon_entropy(data: bytes) -> float:
    if len(data) == 0:
        return 0.0
    c = _hist(data)
    p = c[c > 0] / len(data)
    return float(-(p * np.log2(p)).sum())


def _huffman_encoded_length(data: bytes) -> int:
    if len(data) == 0:
        return 0
    weights = [int(w) for w in _hist(data) if w > 0]
    if len(weights) == 1:
        return len(data)
    heapq.heapify(weights)
    bits = 0
    while len(weights) > 1:
        merged = heapq.heappop(weights) + heapq.heappop(weights)
        bits += merged  # every symbol below this node gets one more code bit
        heapq.heappush(weights, merged)
    return bits


def kolmogorov_complexity(data: bytes) -> float:
    if len(data) == 0:
        return 0.0
    if len(data) == 1:
        return 1.0
    return _huffman_encoded_length(data) / (len(data) * 8)


@dataclass
class FrequencyTable:
    frequencies: dict[int, float] = field(default_factory=dict)

    def get(self, byte: int) -> float:
        return self.frequencies.get(byte, 0.0)

    def as_vector(self) -> np.ndarray:
        v = np.zeros(256, dtype=np.float64)
        for k, x in self.frequencies.items():
            v[int(k)] = x
        return v

    def to_dict(self) -> dict[str, float]:
        return {str(k): v for k, v in self.frequencies.items()}

    @classmethod
    def from_dict(cls, d: dict) -> "FrequencyTable":
        return cls({int(k): float(v) for k, v in d.items()})

    @classmethod
    def from_data(cls, data: bytes) -> "FrequencyTable":
        if len(data) == 0:
            return cls({})
        c = _hist(data)
        nz = np.nonzero(c)[0]
        return cls({int(b): float(c[b]) / len(data) for b in nz})


def char_frequency_difference(data: bytes, reference: FrequencyTable) -> float:
    if len(data) == 0:
        return 0.0
    d = _hist(data) / len(data) - reference.as_vector()
    return float(math.sqrt(float((d * d).sum())))


def char_type_mix(data: bytes) -> float:
    if len(data) <= 1:
        return 0.0
    t = _CLASS[np.frombuffer(data, dtype=np.uint8)]
    return float((t[1:] != t[:-1]).sum()) / (len(data) - 1)


class FeatureSet(NamedTuple):
    shannon_entropy: float
    kolmogorov_complexity: float
    text_freq_diff: float
    innocuous_freq_diff: float
    secret_freq_diff: float
    char_type_mix: float

    def to_list(self) -> list[float]:
        return list(self)


def extract_features(data: bytes, text_freq: FrequencyTable, innocuous_freq: FrequencyTable,
                     secret_freq: FrequencyTable) -> FeatureSet:
    return FeatureSet(shannon_entropy(data), kolmogorov_complexity(data),
                      char_frequency_difference(data, text_freq), char_frequency_difference(data, innocuous_freq),
                      char_frequency_difference(data, secret_freq), char_type_mix(data))
