"""What a data source of the dataset builder has to provide (reference interface: src/heuristic_secrets/data/collector.py:12-50).

A collector is named, declares which model its samples train (``data_type``: ``"validator"`` or ``"spanfinder"``),
yields samples from :meth:`Collector.collect` and, when it reads files that must be fetched first, does the fetching
in :meth:`Collector.setup` into its own folder below the cache directory.
"""
from __future__ import annotations

import os
from abc import ABC, abstractmethod
from pathlib import Path
from typing import Iterator

from .types import SpanFinderSample, ValidatorSample

Sample = ValidatorSample | SpanFinderSample
_CACHE_ENV = "HEURISTIC_SECRETS_CACHE"


def get_cache_dir() -> Path:
    """``$HEURISTIC_SECRETS_CACHE`` if set, else ``~/.cache/heuristic-secrets``."""
    override = os.environ.get(_CACHE_ENV)
    return Path(override) if override else Path.home() / ".cache" / "heuristic-secrets"


class Collector(ABC):
    name: str
    data_type: str

    # -- where the source's files live, and whether they are there -------------------------------------------------
    def cache_path(self) -> Path:
        return get_cache_dir() / "sources" / self.name

    def is_available(self) -> bool:
        """Generators are always available; file-backed sources override this with a check of ``cache_path()``."""
        return True

    def setup(self, force: bool = False) -> None:
        """Fetch the source (clone / download) if it has one; nothing to do for generators."""

    # -- samples ---------------------------------------------------------------------------------------------------
    @abstractmethod
    def collect(self) -> Iterator[Sample]:
        """All samples of the source, in a deterministic order."""

    def collect_spans(self) -> Iterator[SpanFinderSample]:
        """Span-annotated texts for the SpanFinder, for sources that have them (none by default)."""
        return iter(())
