"""``heuristic-secrets-data`` command: run collectors, de-duplicate, split 80/10/10, write JSONL splits and a manifest
(reference: src/heuristic_secrets/data/build.py:23-216)."""
from __future__ import annotations

import argparse
import json
import time
from collections import Counter
from dataclasses import dataclass, field
from pathlib import Path

from .pipeline import deduplicate_samples, split_samples, write_jsonl
from .registry import CollectorRegistry, get_default_registry
from .types import SpanFinderSample, ValidatorSample


@dataclass
class BuildResult:
    validator_counts: dict = field(default_factory=dict)
    document_counts: dict = field(default_factory=dict)
    per_source: dict = field(default_factory=dict)
    skipped: list = field(default_factory=list)


class DataBuilder:
    def __init__(self, output_dir: Path, registry: CollectorRegistry | None = None, seed: int = 42,
                 sources: list[str] | None = None, setup: bool = False):
        self.output_dir, self.registry, self.seed = Path(output_dir), registry or get_default_registry(), seed
        self.sources, self.do_setup = sources, setup

    def build(self) -> BuildResult:
        res = BuildResult()
        val_samples: list[ValidatorSample] = []
        docs: list[SpanFinderSample] = []
        for c in self.registry.all():
            if self.sources is not None and c.name not in self.sources:
                continue
            if self.do_setup:
                try:
                    c.setup()
                except Exception as e:  # network / git unavailable: the source is skipped, the build goes on
                    res.skipped.append((c.name, f"setup failed: {e}"))
                    continue
            if not c.is_available():
                res.skipped.append((c.name, "not available"))
                continue
            got = [s for s in c.collect() if isinstance(s, ValidatorSample)]
            res.per_source[c.name] = len(got)
            val_samples += got
            docs += list(c.collect_spans())
        val_samples = deduplicate_samples(val_samples)
        docs = deduplicate_samples(docs)
        for kind, samples, counts, stratify in (("validator", val_samples, res.validator_counts, True),
                                                 ("documents", docs, res.document_counts, False)):
            tr, va, te = split_samples(samples, seed=self.seed, stratify=stratify)
            for split, part in (("train", tr), ("val", va), ("test", te)):
                write_jsonl(part, self.output_dir / "splits" / kind / f"{split}.jsonl")
                counts[split] = len(part)
        manifest = {"created": time.strftime("%Y-%m-%dT%H:%M:%S"), "seed": self.seed, "per_source": res.per_source,
                    "validator": res.validator_counts, "documents": res.document_counts, "skipped": res.skipped,
                    "categories": dict(Counter(s.category for s in val_samples))}
        (self.output_dir / "manifest.json").write_text(json.dumps(manifest, indent=2))
        return res


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(prog="heuristic-secrets-data")
    ap.add_argument("--output", default="data")
    ap.add_argument("--seed", type=int, default=42)
    ap.add_argument("--sources", nargs="*", default=None)
    ap.add_argument("--setup", action="store_true", help="clone / download the external sources first")
    ap.add_argument("--list", action="store_true")
    a = ap.parse_args(argv)
    reg = get_default_registry()
    if a.list:
        print("\n".join(reg.names()))
        return 0
    r = DataBuilder(Path(a.output), reg, a.seed, a.sources, a.setup).build()
    print(json.dumps({"validator": r.validator_counts, "documents": r.document_counts, "skipped": r.skipped}))
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
