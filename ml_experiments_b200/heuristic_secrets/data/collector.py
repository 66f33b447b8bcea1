"""Collector interface of the dataset builder (reference: src/heuristic_secrets/data/collector.py:12-50)."""
from __future__ import annotations

import os
from abc import ABC, abstractmethod
from pathlib import Path
from typing import Iterator

from .types import SpanFinderSample, ValidatorSample

Sample = ValidatorSample | SpanFinderSample


def get_cache_dir() -> Path:
    return Path(os.environ.get("HEURISTIC_SECRETS_CACHE", Path.home() / ".cache" / "heuristic-secrets"))


class Collector(ABC):
    name: str
    data_type: str  # "validator" or "spanfinder"

    @abstractmethod
    def collect(self) -> Iterator[Sample]:
        ...

    def setup(self, force: bool = False) -> None:
        """Fetch the data source if it has one (git clone / download); a no-op for generators."""

    def cache_path(self) -> Path:
        return get_cache_dir() / "sources" / self.name

    def is_available(self) -> bool:
        return True

    def collect_spans(self) -> Iterator[SpanFinderSample]:
        return iter(())
