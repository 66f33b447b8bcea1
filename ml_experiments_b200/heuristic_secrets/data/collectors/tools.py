"""Per-tool collectors: each secret scanner keeps labelled examples in a different place and notation, and each keeps
*negative* examples (strings its rule must not flag) next to the positive ones. These collectors read the notations
the tools themselves use, so both labels come out:

* gitleaks (``cmd/generate/config/rules/*.go``): ``utils.GenerateSampleSecrets("id", "secret")`` and the ``tps`` string
  slices are true positives, the ``fps`` slices are false positives; ``testdata/`` Go literals and ``.env`` files add
  positives (reference: src/heuristic_secrets/data/collectors/gitleaks.py:36-170, which labels everything 1).
* detect-secrets (``tests/plugins/*_test.py``): parametrised ``(line, should_flag)`` tuples give both labels; module
  constants in capitals are positives; ``test_data/`` YAML / INI / ``.env`` files add positives
  (reference: data/collectors/detect_secrets.py:30-300).
* trufflehog (``pkg/detectors/**/_test.go``): ``validPattern`` / ``want: []string{...}`` are positives,
  ``invalidPattern`` literals and test cases whose ``want`` is empty are negatives
  (reference: data/collectors/trufflehog.py:33-112).

Every collector also yields ``SpanFinderSample`` records: the fixture file's text with the byte offsets of each
positive literal found in it. The generic literal scraper (:mod:`.scrapers`) stays available as a fallback for
repositories laid out differently from what is described above.
"""
from __future__ import annotations

import re
from pathlib import Path
from typing import Iterable, Iterator

from ..collector import Collector
from ..git_utils import clone_or_update
from ..types import SecretCategory, SpanFinderSample, ValidatorSample
from .scrapers import infer_category

_STOPWORDS = frozenset("true false null none undefined test example sample demo placeholder password secret token key api "
                       "changeme foobar username".split())
_GO_STRING = re.compile(r'"((?:[^"\\\n]|\\.)*)"|`([^`]*)`')
_PY_STRING = re.compile(r"""(?P<q>'''|\"\"\"|'|")(?P<v>(?:\\.|(?!(?P=q)).)*)(?P=q)""", re.S)


def plausible(value: str, min_len: int = 10) -> bool:
    """Filters out literals that cannot be credential material: too short, prose, stop words, one repeated symbol."""
    v = value.strip()
    if len(v) < min_len or len(v) > 4096 or v.lower() in _STOPWORDS:
        return False
    if len(set(v)) < 5 or v.count(" ") > 3:
        return False
    return any(c.isalnum() for c in v)


def clean_literal(value: str, min_len: int = 8) -> bool:
    """A literal that can stand alone as a sample: one line without tabs or escape sequences (what is left of a
    mis-parsed multi-line construct has them), not a stop word, a few distinct symbols, not prose."""
    if not min_len <= len(value) <= 4096 or value != value.strip():
        return False
    if any(c in value for c in "\n\t\r\\") or value.lower() in _STOPWORDS:
        return False
    return len(set(value)) >= 3 and value.count(" ") <= 3 and any(c.isalnum() for c in value)


def go_strings(block: str) -> list[str]:
    out = []
    for m in _GO_STRING.finditer(block):
        raw = m.group(1) if m.group(1) is not None else m.group(2)
        if m.group(1) is not None:
            raw = re.sub(r'\\(["\\])', r"\1", raw)
        out.append(raw)
    return out


def _byte_spans(text: str, needles: Iterable[str]) -> tuple[list[int], list[int], list[str]]:
    """Byte offsets of every occurrence of every needle in ``text`` (non-overlapping, sorted)."""
    found = []
    for n in set(needles):
        at = text.find(n)
        while at >= 0:
            found.append((at, at + len(n), n))
            at = text.find(n, at + len(n))
    found.sort()
    starts, ends, vals, last = [], [], [], -1
    for s, e, n in found:
        if s < last:
            continue
        starts.append(len(text[:s].encode()))
        ends.append(len(text[:e].encode()))
        vals.append(n)
        last = e
    return starts, ends, vals


class _RepoCollector(Collector):
    """Shared plumbing: a local checkout (``root``) or a shallow clone into the cache; de-duplicated labelled values."""

    data_type = "validator"
    repo_url = ""
    min_len = 10

    def __init__(self, root: Path | None = None):
        self.root = Path(root) if root else None

    def setup(self, force: bool = False) -> None:
        if self.root is None and self.repo_url:
            self.root = clone_or_update(self.repo_url, self.cache_path(), force=force)

    def repo(self) -> Path:
        return self.root or self.cache_path()

    def is_available(self) -> bool:
        return self.repo().exists()

    def labelled(self) -> Iterator[tuple[str, int, str]]:
        """``(value, label, file name)`` before filtering and de-duplication."""
        raise NotImplementedError

    # -- text-level helpers (one file's text in, literals or spans out) ----------------------------------------------
    def _is_valid_secret(self, value: str) -> bool:
        return clean_literal(value)

    @staticmethod
    def _find_all_positions(text: str, secret: str) -> list[tuple[int, int]]:
        """Character offsets ``(start, end)`` of every non-overlapping occurrence of ``secret`` in ``text``."""
        out, at = [], text.find(secret) if secret else -1
        while at >= 0:
            out.append((at, at + len(secret)))
            at = text.find(secret, at + len(secret))
        return out

    def _positives_in(self, text: str, filename: str = "") -> Iterator[str]:
        """Positive literals of one fixture file (per tool: see the sub-classes)."""
        return iter(())

    def _file_to_span_sample(self, text: str, filename: str = "") -> SpanFinderSample | None:
        """The file's text with the byte offsets of every positive literal found in it; ``None`` without any."""
        starts, ends, vals = _byte_spans(text, {v for v in self._positives_in(text, filename) if v})
        if not starts:
            return None
        return SpanFinderSample(text, starts, ends, self.name, [infer_category(filename, v).value for v in vals])

    def span_files(self) -> Iterator[Path]:
        return iter(())

    def collect(self) -> Iterator[ValidatorSample]:
        seen: dict[str, int] = {}
        for value, label, fname in self.labelled():
            if not plausible(value, self.min_len) or value in seen:
                continue
            seen[value] = label
            cat = infer_category(fname, value) if label else SecretCategory.FP_OTHER
            yield ValidatorSample(value, label, self.name, cat.value)

    def collect_spans(self) -> Iterator[SpanFinderSample]:
        positives = {s.text for s in self.collect() if s.label == 1}
        for f in self.span_files():
            text = f.read_text(errors="ignore")
            if len(text) > 1 << 20:
                continue
            starts, ends, vals = _byte_spans(text, (p for p in positives if p in text))
            if starts:
                yield SpanFinderSample(text, starts, ends, self.name, [infer_category(f.name, v).value for v in vals])


class GitleaksCollector(_RepoCollector):
    name = "gitleaks"
    repo_url = "https://github.com/gitleaks/gitleaks"
    _SAMPLE = re.compile(r'GenerateSampleSecrets?\s*\(\s*"[^"]*"\s*,\s*("(?:[^"\\]|\\.)*"|`[^`]*`)')
    _SLICE = re.compile(r"\b(tps|fps)\s*(?::=|=)\s*(?:append\([^,]+,\s*)?\[\]string\s*\{(.*?)\n\s*\}", re.S)

    _LITERAL = re.compile(r':=\s*("(?:[^"\\]|\\.)*"|`[^`]*`)')

    def _extract_secrets_from_go(self, code: str) -> Iterator[str]:
        """True positives of a rule file: second arguments of ``GenerateSampleSecrets`` and the ``tps`` string slices."""
        for m in self._SAMPLE.finditer(code):
            yield from (v for v in go_strings(m.group(1)) if self._is_valid_secret(v))
        for m in self._SLICE.finditer(code):
            if m.group(1) == "tps":
                yield from (v for v in go_strings(m.group(2)) if self._is_valid_secret(v))

    def _extract_string_literals_from_go(self, code: str) -> Iterator[str]:
        """String literals assigned with ``:=`` in ``testdata`` Go files."""
        for m in self._LITERAL.finditer(code):
            yield from (v for v in go_strings(m.group(1)) if self._is_valid_secret(v))

    def _positives_in(self, text, filename=""):
        yield from self._extract_secrets_from_go(text)
        yield from self._extract_string_literals_from_go(text)

    def _rule_files(self):
        d = self.repo() / "cmd" / "generate" / "config" / "rules"
        return sorted(d.glob("*.go")) if d.exists() else []

    def _testdata(self):
        d = self.repo() / "testdata"
        return d if d.exists() else None

    def labelled(self):
        for f in self._rule_files():
            code = f.read_text(errors="ignore")
            for m in self._SAMPLE.finditer(code):
                for v in go_strings(m.group(1)):
                    yield v, 1, f.name
            for m in self._SLICE.finditer(code):
                label = 1 if m.group(1) == "tps" else 0
                for v in go_strings(m.group(2)):
                    yield v, label, f.name
        td = self._testdata()
        if td is not None:
            for f in sorted(td.rglob("*.go")):
                for m in re.finditer(r':=\s*("(?:[^"\\]|\\.)*"|`[^`]*`)', f.read_text(errors="ignore")):
                    for v in go_strings(m.group(1)):
                        yield v, 1, f.name
            for f in sorted(td.rglob("*.env*")):
                for line in f.read_text(errors="ignore").splitlines():
                    m = re.match(r"\s*(?:export\s+)?([A-Za-z_][A-Za-z0-9_]*)\s*=\s*(.+?)\s*$", line)
                    if m and not line.lstrip().startswith("#"):
                        yield m.group(2).strip("\"'"), 1, f"{f.name} {m.group(1)}"      # the variable name hints at the category

    def span_files(self):
        td = self._testdata()
        files = list(self._rule_files())
        if td is not None:
            files += [p for p in sorted(td.rglob("*")) if p.is_file() and p.suffix in (".go", ".env", ".txt", ".yaml", ".yml", ".json", ".toml")]
        return iter(files)


class DetectSecretsCollector(_RepoCollector):
    name = "detect_secrets"
    repo_url = "https://github.com/Yelp/detect-secrets"
    _PAIR = re.compile(r"""\(\s*(?:[rRbBuUfF]{0,2})(?P<q>'|")(?P<v>(?:\\.|(?!(?P=q)).)*)(?P=q)\s*,\s*(?P<flag>True|False)\s*,?\s*\)""")
    _CONST = re.compile(r"""^(?P<name>[A-Z][A-Z0-9_]{2,})\s*=\s*(?:[rRbBuU]{0,2})(?P<q>'|")(?P<v>(?:\\.|(?!(?P=q)).)*)(?P=q)\s*$""", re.M)

    _ASSIGN = re.compile(r"""^[ \t]*(?:self\.)?[A-Za-z_]\w*[ \t]*=[ \t]*(?:[rRbBuU]{0,2})(?P<q>'|")(?P<v>(?:\\.|(?!(?P=q)).)*)(?P=q)[ \t]*$""", re.M)
    _INI = re.compile(r"""^[ \t]*[^\[\]#;=\n][^=\n]*?=[ \t]*['"]?([^'"\n#;]+?)['"]?[ \t]*(?:[#;].*)?$""", re.M)
    _ENV = re.compile(r"""^[ \t]*(?:export[ \t]+)?[A-Za-z_][A-Za-z0-9_]*=['"]?([^'"\n]+?)['"]?[ \t]*$""", re.M)
    _YAML = re.compile(r"""^\s*[\w.-]*(?:key|secret|token|password|passwd|credential)[\w.-]*\s*:\s*['"]?([^'"#\n]+?)['"]?\s*(?:#.*)?$""", re.M | re.I)

    def _extract_constants_from_python(self, code: str) -> Iterator[str]:
        """Positive literals of a plugin test: string constants assigned to a name or a ``self.`` attribute, and the
        first element of parametrised ``(line, should_flag)`` cases whose flag is ``True``."""
        seen = set()
        for m in self._ASSIGN.finditer(code):
            seen.add(m.group("v"))
        for m in self._PAIR.finditer(code):
            if m.group("flag") == "True":
                seen.add(self._secret_in(m.group("v")))
        negatives = {self._secret_in(m.group("v")) for m in self._PAIR.finditer(code) if m.group("flag") == "False"}
        yield from (v for v in seen if self._is_valid_secret(v) and v not in negatives)

    def _extract_secrets_from_ini(self, content: str) -> Iterator[str]:
        yield from (m.group(1).strip() for m in self._INI.finditer(content) if self._is_valid_secret(m.group(1).strip()))

    def _extract_secrets_from_env(self, content: str) -> Iterator[str]:
        yield from (m.group(1).strip() for m in self._ENV.finditer(content) if self._is_valid_secret(m.group(1).strip()))

    def _extract_secrets_from_yaml(self, content: str) -> Iterator[str]:
        yield from (m.group(1).strip() for m in self._YAML.finditer(content) if self._is_valid_secret(m.group(1).strip()))

    def _positives_in(self, text, filename=""):
        name = filename.lower()
        if name.endswith((".yaml", ".yml")):
            return self._extract_secrets_from_yaml(text)
        if name.endswith((".ini", ".cfg", ".conf")):
            return self._extract_secrets_from_ini(text)
        if ".env" in name:
            return self._extract_secrets_from_env(text)
        return self._extract_constants_from_python(text)

    def _plugin_tests(self):
        d = self.repo() / "tests" / "plugins"
        return sorted(d.glob("*_test.py")) if d.exists() else []

    def _test_data(self):
        d = self.repo() / "test_data"
        return [p for p in sorted(d.rglob("*")) if p.is_file()] if d.exists() else []

    @staticmethod
    def _secret_in(line: str) -> str:
        """A parametrised case is a whole source line; the credential is its right-hand side if it has one."""
        m = re.search(r"""[:=]\s*['"]?([^'"\s][^'"]*?)['"]?\s*;?\s*$""", line)
        return (m.group(1) if m else line).strip()

    def labelled(self):
        for f in self._plugin_tests():
            code = f.read_text(errors="ignore")
            for m in self._PAIR.finditer(code):
                yield self._secret_in(m.group("v")), int(m.group("flag") == "True"), f.name
            for m in self._CONST.finditer(code):
                yield m.group("v"), 1, f.name
        for f in self._test_data():
            if f.suffix in (".yaml", ".yml", ".ini", ".cfg", ".conf") or ".env" in f.name:
                for v in self._positives_in(f.read_text(errors="ignore"), f.name):
                    yield v, 1, f.name

    def span_files(self):
        return iter(self._plugin_tests() + [p for p in self._test_data() if p.suffix in (".yaml", ".yml", ".ini", ".cfg", ".conf", ".py", ".txt") or ".env" in p.name])


class TrufflehogCollector(_RepoCollector):
    name = "trufflehog"
    repo_url = "https://github.com/trufflesecurity/trufflehog"
    min_len = 12
    _ASSIGN = re.compile(r"\b(validPattern|invalidPattern|secret|token|key|password|complexPattern)\w*\s*(?::=|=)\s*(\"(?:[^\"\\]|\\.)*\"|`[^`]*`)")
    _CASE = re.compile(r"input:\s*(\"(?:[^\"\\]|\\.)*\"|`[^`]*`|\w+)\s*,\s*want:\s*(nil|\[\]string\s*\{(.*?)\})", re.S)

    @staticmethod
    def _longest_token(snippet: str) -> str:
        """Patterns are usually whole config snippets: the credential is the longest token without spaces or punctuation."""
        return max(re.findall(r"[^\s\"'=:,;{}\[\]()<>]+", snippet) or [snippet], key=len)

    def _extract_from_go_test(self, code: str) -> Iterator[str]:
        """Positive literals of a detector's unit test: ``validPattern`` / ``secret`` / ``token`` ... assignments of a
        string literal and the ``want: []string{...}`` lists. Integration tests fetch their secrets at run time
        (``common.GetSecret`` / ``MustGetField``): no literal is assigned there, so nothing is taken from them."""
        for m in self._ASSIGN.finditer(code):
            if not m.group(1).startswith("invalid"):
                yield from (t for t in (self._longest_token(v) for v in go_strings(m.group(2))) if self._is_valid_secret(t))
        for m in self._CASE.finditer(code):
            yield from (v for v in go_strings(m.group(3) or "") if self._is_valid_secret(v))

    def _positives_in(self, text, filename=""):
        return self._extract_from_go_test(text)

    def _tests(self):
        d = self.repo() / "pkg" / "detectors"
        return sorted(d.rglob("*_test.go")) if d.exists() else []

    def labelled(self):
        for f in self._tests():
            code = f.read_text(errors="ignore")
            for m in self._ASSIGN.finditer(code):
                label = 0 if m.group(1).startswith("invalid") else 1
                for v in go_strings(m.group(2)):
                    yield self._longest_token(v), label, f.parent.name + "_" + f.name
            for m in self._CASE.finditer(code):
                wants = go_strings(m.group(3) or "")
                for v in wants:
                    yield v, 1, f.parent.name + "_" + f.name
                if not wants and m.group(1)[0] in "\"`":         # a case that must stay silent: its input is a negative
                    for v in go_strings(m.group(1)):
                        yield self._longest_token(v), 0, f.parent.name + "_" + f.name

    def span_files(self):
        return iter(self._tests())
