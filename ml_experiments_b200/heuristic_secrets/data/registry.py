"""Registry of collectors (reference: src/heuristic_secrets/data/registry.py:17-65)."""
from __future__ import annotations

from typing import Type

from .collector import Collector
from .collectors.generated import Base64Generator, HashGenerator, UUIDGenerator
from .collectors.scrapers import CredDataCollector
from .collectors.tools import DetectSecretsCollector, GitleaksCollector, TrufflehogCollector


class CollectorRegistry:
    def __init__(self):
        self._collectors: dict[str, Collector] = {}

    def register(self, collector_class: Type[Collector], **kwargs) -> None:
        inst = collector_class(**kwargs)
        self._collectors[inst.name] = inst

    def get(self, name: str) -> Collector | None:
        return self._collectors.get(name)

    def names(self) -> list[str]:
        return list(self._collectors)

    def all(self) -> list[Collector]:
        return list(self._collectors.values())


def get_default_registry() -> CollectorRegistry:
    r = CollectorRegistry()
    r.register(UUIDGenerator)
    for h in ("md5", "sha1", "sha256"):
        r.register(HashGenerator, hash_type=h)
    r.register(Base64Generator)
    for c in (DetectSecretsCollector, GitleaksCollector, TrufflehogCollector, CredDataCollector):
        r.register(c)
    return r
