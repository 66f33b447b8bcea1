"""Collectors that mine the test fixtures of secret scanners (detect-secrets, gitleaks, trufflehog) and the CredData
research set for labelled secrets.

The reference has one hand-tuned scraper per tool (data/collectors/detect_secrets.py, gitleaks.py, trufflehog.py,
creddata.py). Here they share one engine: walk the cloned repository, pull string literals out of fixture files with
per-language patterns, keep the ones that look like credentials (length / character-class filter), infer a category
from the file name and the variable name next to the literal, and emit ``ValidatorSample`` records plus
``SpanFinderSample`` records that keep the surrounding file text with byte offsets of every literal.
"""
from __future__ import annotations

import csv
import re
from pathlib import Path
from typing import Iterator

from ..collector import Collector
from ..git_utils import clone_or_update
from ..types import SecretCategory, SpanFinderSample, ValidatorSample

_LITERAL = re.compile(r"""(?P<name>[A-Za-z_][A-Za-z0-9_\-\.]*)?\s*[:=]?\s*(?P<q>["'`])(?P<val>[^"'`\n]{8,256})(?P=q)""")
_CATEGORY_HINTS = (
    (re.compile(r"private[_-]?key|BEGIN [A-Z ]*PRIVATE KEY", re.I), SecretCategory.PRIVATE_KEY),
    (re.compile(r"passw(or)?d|pwd", re.I), SecretCategory.PASSWORD),
    (re.compile(r"token|bearer|oauth|session", re.I), SecretCategory.AUTH_TOKEN),
    (re.compile(r"api[_-]?key|apikey|access[_-]?key|client[_-]?secret", re.I), SecretCategory.API_KEY),
    (re.compile(r"://[^/\s:]+:[^@\s]+@|connection|dsn|jdbc", re.I), SecretCategory.CONNECTION_STRING),
)


def looks_like_credential(s: str) -> bool:
    if len(s) < 8 or " " in s.strip() and len(s.split()) > 3:
        return False
    classes = sum(bool(re.search(p, s)) for p in (r"[a-z]", r"[A-Z]", r"[0-9]", r"[^A-Za-z0-9]"))
    return classes >= 2 and len(set(s)) >= 6


def infer_category(context: str, value: str) -> SecretCategory:
    for pat, cat in _CATEGORY_HINTS:
        if pat.search(context) or pat.search(value):
            return cat
    return SecretCategory.GENERIC_SECRET


def extract_literals(text: str) -> list[tuple[int, int, str, str]]:
    """``(start, end, value, variable_name)`` of credential-like string literals in ``text`` (character offsets)."""
    out = []
    for m in _LITERAL.finditer(text):
        v = m.group("val")
        if looks_like_credential(v):
            out.append((m.start("val"), m.end("val"), v, m.group("name") or ""))
    return out


class FixtureScraper(Collector):
    data_type = "validator"
    repo_url = ""
    include = ("test", "fixture", "testdata", "examples")
    suffixes = (".py", ".go", ".yaml", ".yml", ".json", ".toml", ".txt", ".js", ".env")

    def __init__(self, root: Path | None = None, max_files: int = 5000):
        self.root, self.max_files = (Path(root) if root else None), max_files

    def setup(self, force: bool = False) -> None:
        if self.root is None and self.repo_url:
            self.root = clone_or_update(self.repo_url, self.cache_path(), force=force)

    def is_available(self) -> bool:
        root = self.root or self.cache_path()
        return root.exists()

    def _files(self) -> Iterator[Path]:
        root = self.root or self.cache_path()
        n = 0
        for p in sorted(root.rglob("*")):
            if p.is_file() and p.suffix in self.suffixes and any(k in str(p).lower() for k in self.include):
                yield p
                n += 1
                if n >= self.max_files:
                    return

    def collect(self) -> Iterator[ValidatorSample]:
        for f in self._files():
            text = f.read_text(errors="ignore")
            for _, _, val, name in extract_literals(text):
                yield ValidatorSample(val, 1, self.name, infer_category(f"{f.name} {name}", val).value)

    def collect_spans(self) -> Iterator[SpanFinderSample]:
        for f in self._files():
            text = f.read_text(errors="ignore")
            lits = extract_literals(text)
            if lits:
                raw = text.encode("utf-8")
                starts = [len(text[:s].encode("utf-8")) for s, _, _, _ in lits]
                ends = [len(text[:e].encode("utf-8")) for _, e, _, _ in lits]
                if len(raw) <= 1 << 20:
                    yield SpanFinderSample(text, starts, ends, self.name,
                                           [infer_category(f"{f.name} {n}", v).value for _, _, v, n in lits])


class GenericFixtureCollector(FixtureScraper):
    """Literal scraper over an arbitrary checkout (every hit is labelled positive): the fallback for scanner
    repositories that do not follow the layouts the per-tool collectors of :mod:`.tools` read."""

    name = "fixtures"

    def __init__(self, root: Path | None = None, max_files: int = 5000, name: str | None = None):
        super().__init__(root, max_files)
        if name:
            self.name = name


# CredData's own category labels (possibly several, colon-separated, e.g. "Auth:Token") -> the categories used here;
# the first keyword found in the label decides
_CREDDATA_LABELS = (("password", SecretCategory.PASSWORD), ("auth", SecretCategory.AUTH_TOKEN), ("token", SecretCategory.AUTH_TOKEN),
                    ("secret", SecretCategory.GENERIC_SECRET), ("key", SecretCategory.API_KEY), ("api", SecretCategory.API_KEY),
                    ("private", SecretCategory.PRIVATE_KEY), ("certificate", SecretCategory.PRIVATE_KEY), ("credentials", SecretCategory.PASSWORD),
                    ("generic", SecretCategory.GENERIC_SECRET), ("seed", SecretCategory.GENERIC_SECRET), ("salt", SecretCategory.GENERIC_SECRET))


CREDDATA_CATEGORY_MAP = dict(_CREDDATA_LABELS)


def map_creddata_category(category_str: str) -> SecretCategory:
    """Category of a CredData row from its label column (src/heuristic_secrets/data/collectors/creddata.py:20-51)."""
    label = (category_str or "").lower()
    return next((cat for key, cat in _CREDDATA_LABELS if key in label), SecretCategory.GENERIC_SECRET)


class CredDataCollector(Collector):
    """Samsung CredData: ``meta/*.csv`` rows (file, line span, value span, ground truth ``T`` / ``F``, category) joined
    with the downloaded files under ``data/``."""

    name = "creddata"
    data_type = "validator"
    repo_url = "https://github.com/Samsung/CredData"

    def __init__(self, root: Path | None = None):
        self.root = Path(root) if root else None

    def setup(self, force: bool = False) -> None:
        if self.root is None:
            self.root = clone_or_update(self.repo_url, self.cache_path(), force=force)

    def is_available(self) -> bool:
        root = self.root or self.cache_path()
        return (root / "meta").exists()

    def collect(self) -> Iterator[ValidatorSample]:
        root = self.root or self.cache_path()
        for meta in sorted((root / "meta").glob("*.csv")):
            with open(meta, newline="", errors="ignore") as fh:
                for row in csv.DictReader(fh):
                    path = root / row.get("FilePath", "")
                    try:
                        line_no = int(row.get("LineStart", -1))
                        s, e = int(float(row.get("ValueStart", -1))), int(float(row.get("ValueEnd", -1)))
                    except ValueError:
                        continue
                    if not path.is_file() or line_no < 1 or s < 0 or e <= s:
                        continue
                    lines = path.read_text(errors="ignore").splitlines()
                    if line_no > len(lines):
                        continue
                    val = lines[line_no - 1][s:e]
                    if len(val) >= 4:
                        truth = row.get("GroundTruth", "F").strip().upper() == "T"
                        cat = map_creddata_category(row.get("Category", "")) if truth else SecretCategory.FP_OTHER
                        yield ValidatorSample(val, int(truth), self.name, cat.value)
