"""Synthetic non-secrets: UUIDs, hash digests and base64 blobs (reference: data/collectors/generated.py:13-90).
A ``seed`` makes the streams reproducible; without one they use OS entropy like the reference."""
from __future__ import annotations

import base64
import hashlib
import random
import uuid
from typing import Iterator

from ..collector import Collector
from ..types import SecretCategory, ValidatorSample


class _Seeded(Collector):
    data_type = "validator"

    def _rng(self) -> random.Random:
        return random.Random(self.seed) if getattr(self, "seed", None) is not None else random.SystemRandom()


class UUIDGenerator(_Seeded):
    name = "generated_uuids"

    def __init__(self, count: int = 5000, seed: int | None = None):
        self.count, self.seed = count, seed

    def collect(self) -> Iterator[ValidatorSample]:
        rng = self._rng()
        for _ in range(self.count):
            text = str(uuid.UUID(int=rng.getrandbits(128), version=4))
            yield ValidatorSample(text, 0, self.name, SecretCategory.FP_UUID.value)


class HashGenerator(_Seeded):
    def __init__(self, hash_type: str = "sha256", count: int = 3000, seed: int | None = None):
        if hash_type not in ("md5", "sha1", "sha256"):
            raise ValueError(f"Unknown hash type: {hash_type}")
        self.hash_type, self.count, self.seed = hash_type, count, seed
        self.name = f"generated_{hash_type}"

    def collect(self) -> Iterator[ValidatorSample]:
        rng = self._rng()
        for _ in range(self.count):
            digest = hashlib.new(self.hash_type, rng.getrandbits(256).to_bytes(32, "little")).hexdigest()
            yield ValidatorSample(digest, 0, self.name, SecretCategory.FP_HASH.value)


class Base64Generator(_Seeded):
    name = "generated_base64"

    def __init__(self, count: int = 2000, min_length: int = 20, max_length: int = 100, seed: int | None = None):
        self.count, self.min_length, self.max_length, self.seed = count, min_length, max_length, seed

    def collect(self) -> Iterator[ValidatorSample]:
        rng = self._rng()
        for _ in range(self.count):
            n = (rng.randint(self.min_length, self.max_length) * 3) // 4
            text = base64.b64encode(rng.getrandbits(8 * n).to_bytes(n, "little")).decode("ascii")
            yield ValidatorSample(text, 0, self.name, SecretCategory.FP_ENCODED.value)
