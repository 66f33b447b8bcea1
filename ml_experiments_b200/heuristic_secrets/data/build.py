"""``heuristic-secrets-data`` command: fetch sources, run collectors, de-duplicate, split 80/10/10, write JSONL splits and
a manifest (reference: src/heuristic_secrets/data/build.py:23-216; same constructor arguments, same manifest fields).

Additions to the manifest the reference writes: ``skipped`` (sources that could not be fetched or are not present:
the build goes on without them; the reference lets the first failing ``collect()`` end the build) and ``categories``
(label histogram of the validator samples after de-duplication).
"""
from __future__ import annotations

import argparse
import json
import sys
from collections import Counter
from dataclasses import asdict, dataclass, field
from datetime import datetime, timezone
from pathlib import Path
from typing import Any

from .pipeline import deduplicate_samples, split_samples, write_jsonl
from .registry import CollectorRegistry, get_default_registry
from .types import SpanFinderSample, ValidatorSample


@dataclass
class Manifest:
    """What a build read and wrote: per-source counts, split sizes per sample kind, de-duplication before / after."""
    created_at: str = ""
    sources: dict[str, dict[str, Any]] = field(default_factory=dict)
    splits: dict[str, dict[str, int]] = field(default_factory=dict)
    deduplication: dict[str, int] = field(default_factory=dict)
    skipped: list = field(default_factory=list)
    categories: dict[str, int] = field(default_factory=dict)

    def to_dict(self) -> dict[str, Any]:
        return asdict(self)


class DataBuilder:
    def __init__(self, output_dir: Path, sources: list[str] | None = None, no_fetch: bool = False, force_download: bool = False,
                 seed: int = 42, registry: CollectorRegistry | None = None):
        self.output_dir, self.no_fetch, self.force_download, self.seed = Path(output_dir), no_fetch, force_download, seed
        self.registry = registry or get_default_registry()
        if sources:
            self._filter_sources(sources)

    def _filter_sources(self, sources: list[str]) -> None:
        kept = CollectorRegistry()
        for name in sources:
            c = self.registry.get(name)
            if c is None:
                print(f"[warn] Unknown source: {name}", file=sys.stderr)
            else:
                kept._collectors[name] = c
        self.registry = kept

    def _setup_collectors(self, manifest: Manifest) -> set[str]:
        """``setup`` of every collector (clone / download); returns the names whose setup failed."""
        failed = set()
        for c in self.registry.all():
            try:
                c.setup(force=self.force_download)
            except Exception as e:          # no network, no git, a moved repository: skip the source, keep building
                manifest.skipped.append([c.name, f"setup failed: {e}"])
                failed.add(c.name)
        return failed

    def _write_splits(self, kind: str, samples: list, manifest: Manifest, stratify: bool) -> None:
        if not samples:
            return
        parts = dict(zip(("train", "val", "test"), split_samples(samples, seed=self.seed, stratify=stratify)))
        manifest.splits[kind] = {k: len(v) for k, v in parts.items()}
        for split, part in parts.items():
            write_jsonl(part, self.output_dir / "splits" / kind / f"{split}.jsonl")

    def build(self) -> Manifest:
        manifest = Manifest(created_at=datetime.now(timezone.utc).isoformat())
        failed = set() if self.no_fetch else self._setup_collectors(manifest)
        validator: list[ValidatorSample] = []
        documents: list[SpanFinderSample] = []
        for c in self.registry.all():
            if c.name in failed:
                continue
            if not c.is_available():
                manifest.skipped.append([c.name, "not available"])
                continue
            samples = list(c.collect())
            wanted = ValidatorSample if c.data_type == "validator" else SpanFinderSample
            (validator if wanted is ValidatorSample else documents).extend(s for s in samples if isinstance(s, wanted))
            spans = list(c.collect_spans())
            documents.extend(spans)
            manifest.sources[c.name] = {"samples": len(samples), "spans": len(spans)}
        before = len(validator)
        validator = deduplicate_samples(validator)
        documents = deduplicate_samples(documents)
        manifest.deduplication = {"validator_before": before, "validator_after": len(validator)}
        manifest.categories = dict(Counter(s.category for s in validator))
        self._write_splits("validator", validator, manifest, stratify=True)
        self._write_splits("documents", documents, manifest, stratify=False)
        self.output_dir.mkdir(parents=True, exist_ok=True)
        (self.output_dir / "manifest.json").write_text(json.dumps(manifest.to_dict(), indent=2))
        return manifest


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="heuristic-secrets-data", description="Build the training data of the secret detector.")
    ap.add_argument("--output", "-o", default="data")
    ap.add_argument("--seed", type=int, default=42)
    ap.add_argument("--sources", nargs="*", default=None, help="only these sources (default: all registered)")
    ap.add_argument("--no-fetch", action="store_true", help="do not clone / download; use what is already cached")
    ap.add_argument("--force-download", action="store_true", help="fetch the sources again even if cached")
    ap.add_argument("--list", action="store_true", help="print the registered sources and exit")
    a = ap.parse_args(argv)
    if a.list:
        print("\n".join(get_default_registry().names()))
        return 0
    m = DataBuilder(Path(a.output), a.sources, a.no_fetch, a.force_download, a.seed).build()
    print(json.dumps({"splits": m.splits, "deduplication": m.deduplication, "skipped": m.skipped}))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
