"""Sample records and secret categories (reference: src/heuristic_secrets/data/types.py:6-106)."""
from __future__ import annotations

import json
from dataclasses import asdict, dataclass, field
from enum import Enum


class SecretCategory(str, Enum):
    PRIVATE_KEY = "private_key"
    API_KEY = "api_key"
    AUTH_TOKEN = "auth_token"
    PASSWORD = "password"
    CONNECTION_STRING = "connection_string"
    GENERIC_SECRET = "generic_secret"
    FP_UUID = "fp_uuid"
    FP_HASH = "fp_hash"
    FP_ENCODED = "fp_encoded"
    FP_PLACEHOLDER = "fp_placeholder"
    FP_OTHER = "fp_other"
    UNKNOWN = "unknown"


CATEGORY_LABELS = {c: (0 if c.value.startswith("fp_") or c is SecretCategory.UNKNOWN else 1) for c in SecretCategory}


def category_to_label(category: SecretCategory) -> int:
    return CATEGORY_LABELS[category]


@dataclass
class ValidatorSample:
    text: str
    label: int
    source: str = ""
    category: str = SecretCategory.UNKNOWN.value

    def to_dict(self) -> dict:
        return asdict(self)

    def to_json(self) -> str:
        return json.dumps(self.to_dict())

    @classmethod
    def from_dict(cls, d: dict) -> "ValidatorSample":
        return cls(text=d["text"], label=int(d["label"]), source=d.get("source", ""),
                   category=d.get("category", SecretCategory.UNKNOWN.value))


@dataclass
class SpanFinderSample:
    text: str
    starts: list[int] = field(default_factory=list)
    ends: list[int] = field(default_factory=list)
    source: str = ""
    categories: list[str] | None = None

    def to_dict(self) -> dict:
        d = {"text": self.text, "starts": self.starts, "ends": self.ends, "source": self.source}
        if self.categories is not None:
            d["categories"] = self.categories
        return d

    def to_json(self) -> str:
        return json.dumps(self.to_dict())

    @classmethod
    def from_dict(cls, d: dict) -> "SpanFinderSample":
        return cls(text=d["text"], starts=list(d.get("starts", [])), ends=list(d.get("ends", [])),
                   source=d.get("source", ""), categories=d.get("categories"))
