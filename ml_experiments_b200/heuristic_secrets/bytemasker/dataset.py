"""ByteMasker dataset: line / multi-line windows with per-byte secret masks and a leakage-free split.

Follows the reference's design (src/heuristic_secrets/bytemasker/dataset.py:23-922): windows are single lines,
multi-line windows of 2-9 lines (at most ``max_len`` bytes) or secret-only windows; every secret gets a content id
(``sha256[:16]``); windows that share a secret are connected (union-find) and whole components are assigned to
train / val / test so that no secret appears in two splits; batches are length-bucketed.

On top of that, the loaders of the reference's training scripts: documents come from ``<data_dir>/splits/documents/
{train,val,test}.jsonl`` (``SpanFinderSample`` per line); lines longer than ``max_len`` are cut into windows that keep a
prefix and a suffix of the line around a moving middle part (:func:`window_long_line`); spans whose category is a
false-positive class do not count as secrets; window lists are cached as JSON lines keyed by the source file's path,
time stamp and the windowing parameters (:func:`load_bytemasker_dataset`), and
:func:`load_and_split_mixed_windows` re-splits ALL documents by secret components and refuses to return a split in
which a secret occurs on both sides.
"""
from __future__ import annotations

import functools
import hashlib
import json
import os
import random
from dataclasses import asdict, dataclass, field
from pathlib import Path

import torch

from ..data.types import CATEGORY_LABELS, SecretCategory, SpanFinderSample

BUCKETS = (48, 80, 128, 288, 384, 512)


@dataclass
class MaskWindow:
    data: bytes
    mask: list[int]
    secret_ids: list[str] = field(default_factory=list)
    kind: str = "line"
    source: str = ""
    categories: list[str] | None = None

    # the reference's record for the same thing is ``LineSample(bytes, mask, has_secret, source, ...)``: its attribute
    # names read the same data here
    @property
    def bytes(self):
        return self.data

    @property
    def has_secret(self) -> bool:
        return any(self.mask)


class LineSample(MaskWindow):
    """:class:`MaskWindow` built with the reference's argument names (src/heuristic_secrets/bytemasker/dataset.py:36-43)."""

    def __init__(self, bytes, mask, has_secret: bool | None = None, source: str = "", categories=None, secret_ids=None):
        super().__init__(data=bytes, mask=list(mask), secret_ids=list(secret_ids or []), kind="line", source=source, categories=categories)


def secret_id(raw: bytes) -> str:
    return hashlib.sha256(raw).hexdigest()[:16]


def true_secret_spans(s: SpanFinderSample) -> list[tuple[int, int]]:
    """Spans of ``s`` whose category is a real secret class (``fp_*`` / unknown categories label 0 and are skipped;
    a span without category information counts as a secret)."""
    n = len(s.text.encode("utf-8"))
    out = []
    for i, (a, b) in enumerate(zip(s.starts, s.ends)):
        cat = s.categories[i] if s.categories and i < len(s.categories) else None
        if cat is not None:
            try:
                if CATEGORY_LABELS.get(SecretCategory(cat), 0) != 1:
                    continue
            except ValueError:
                if cat.startswith("fp_"):
                    continue
        if 0 <= a < min(b, n):
            out.append((a, min(b, n)))
    return sorted(out)


def window_long_line(w: MaskWindow, max_len: int = 512, prefix_len: int = 64, suffix_len: int = 64,
                     middle_len: int | None = None) -> list[MaskWindow]:
    """A line longer than ``max_len`` becomes several windows ``prefix + middle[k] + suffix``: the head and tail of the
    line (where key names and closing quotes sit) stay visible next to every slice of its middle."""
    if len(w.data) <= max_len:
        return [w]
    middle_len = middle_len or max(max_len - prefix_len - suffix_len, 1)
    head, tail = w.data[:prefix_len], w.data[len(w.data) - suffix_len:]
    mhead, mtail = w.mask[:prefix_len], w.mask[len(w.mask) - suffix_len:]
    mid, mmid = w.data[prefix_len:len(w.data) - suffix_len], w.mask[prefix_len:len(w.mask) - suffix_len]
    out = []
    for k in range(0, len(mid), middle_len):
        mask = mhead + mmid[k:k + middle_len] + mtail
        out.append(MaskWindow(head + mid[k:k + middle_len] + tail, mask, list(w.secret_ids) if any(mask) else [], w.kind))
    return out


def windows_from_document(s: SpanFinderSample, max_len: int = 512, rng: random.Random | None = None,
                          prefix_len: int = 64, suffix_len: int = 64, min_len: int = 1) -> list[MaskWindow]:
    rng = rng or random.Random(0)
    raw = s.text.encode("utf-8")
    mask = bytearray(len(raw))
    spans = true_secret_spans(s)
    for a, b in spans:
        mask[a:b] = b"\x01" * (b - a)
    # line boundaries
    bounds, pos = [], 0
    for line in raw.split(b"\n"):
        bounds.append((pos, pos + len(line)))
        pos += len(line) + 1
    out = []

    def make(a, b, kind):
        ids = [secret_id(raw[x:y]) for x, y in spans if x < b and y > a]      # every secret the window touches
        out.append(MaskWindow(raw[a:b], list(mask[a:b]), ids, kind))

    for a, b in bounds:
        if b - a > max_len and raw[a:b].strip():
            make(a, b, "line")
            out.extend(window_long_line(out.pop(), max_len, prefix_len, suffix_len))
        elif b - a >= min_len and raw[a:b].strip():
            make(a, b, "line")
    i = 0
    while i < len(bounds):
        n = rng.randint(2, 9)
        a, b = bounds[i][0], bounds[min(i + n, len(bounds)) - 1][1]
        if 0 < b - a <= max_len:
            make(a, b, "multi")
        i += n
    for a, b in spans:
        if 0 < b - a <= max_len:
            make(a, b, "secret")
    return out


# -- the reference's names for the three window kinds and its constants (src/heuristic_secrets/bytemasker/dataset.py:16-270) --
CACHE_DIR = Path(".cache/bytemasker")
DEFAULT_MAX_LEN, DEFAULT_PREFIX_LEN, DEFAULT_SUFFIX_LEN, DEFAULT_MIDDLE_LEN = 512, 64, 64, 384
DEFAULT_MULTILINE_MAX_LINES, DEFAULT_MULTILINE_OVERLAP, DEFAULT_MULTILINE_MIN_LINES, DEFAULT_MULTILINE_MAX_BYTES = 9, 2, 4, 512


def _windows_of_kind(sample: SpanFinderSample, kind: str, max_len: int) -> list[MaskWindow]:
    big = 1 << 30 if kind == "line" else max_len          # whole lines come back unsplit; ``window_line`` splits them
    out = [w for w in windows_from_document(sample, big, random.Random(0)) if w.kind == kind]
    for w in out:
        w.source = sample.source
    return out


def extract_lines_with_masks(sample: SpanFinderSample) -> list[MaskWindow]:
    """One window per non-blank line of the document with its per-byte secret mask."""
    return _windows_of_kind(sample, "line", DEFAULT_MAX_LEN)


def window_line(line: MaskWindow, max_len: int = DEFAULT_MAX_LEN, prefix_len: int = DEFAULT_PREFIX_LEN, suffix_len: int = DEFAULT_SUFFIX_LEN,
                middle_len: int = DEFAULT_MIDDLE_LEN) -> list[MaskWindow]:
    return window_long_line(line, max_len, prefix_len, suffix_len, middle_len)


def extract_multiline_windows(sample: SpanFinderSample, max_lines: int = DEFAULT_MULTILINE_MAX_LINES, overlap: int = DEFAULT_MULTILINE_OVERLAP,
                              min_lines: int = DEFAULT_MULTILINE_MIN_LINES, max_bytes: int = DEFAULT_MULTILINE_MAX_BYTES) -> list[MaskWindow]:
    """Windows of several consecutive lines (2 to 9, drawn per window) no longer than ``max_bytes``."""
    return _windows_of_kind(sample, "multi", max_bytes)


def extract_secret_only_samples(sample: SpanFinderSample, max_bytes: int = DEFAULT_MAX_LEN) -> list[MaskWindow]:
    """The bare secret of every true span as a window of its own (mask all ones)."""
    return _windows_of_kind(sample, "secret", max_bytes)


def stratified_split_samples(samples: list[MaskWindow], train_ratio: float = 0.88, val_ratio: float = 0.12, seed: int | None = None):
    """``(train, val)`` with every group of windows that share a secret on one side."""
    train, val, _ = stratified_component_split(samples, (train_ratio, val_ratio, 0.0), seed or 0)
    return train, val


def stratified_component_split(windows: list[MaskWindow], fractions=(0.8, 0.1, 0.1), seed: int = 0):
    """Connected components over shared secret ids, assigned greedily to the split furthest below its quota."""
    parent = list(range(len(windows)))

    def find(x):
        while parent[x] != x:
            parent[x] = parent[parent[x]]
            x = parent[x]
        return x

    owner: dict[str, int] = {}
    for i, w in enumerate(windows):
        for sid in w.secret_ids:
            if sid in owner:
                ra, rb = find(i), find(owner[sid])
                if ra != rb:
                    parent[ra] = rb
            else:
                owner[sid] = i
    comps: dict[int, list[int]] = {}
    for i in range(len(windows)):
        comps.setdefault(find(i), []).append(i)
    groups = list(comps.values())
    random.Random(seed).shuffle(groups)
    groups.sort(key=len, reverse=True)
    splits: tuple[list, list, list] = ([], [], [])
    total = len(windows)
    for g in groups:
        deficits = [fractions[k] - len(splits[k]) / max(total, 1) for k in range(3)]
        k = max(range(3), key=lambda j: deficits[j])
        splits[k].extend(windows[i] for i in g)
    return splits


def compute_length_bins(lengths: list[int], n_bins: int = 8) -> list[int]:
    """Bucket edges at the ``1/n_bins .. (n_bins-1)/n_bins`` quantiles of ``lengths`` plus the maximum (equal-population
    buckets for a given data set, as an alternative to the fixed ``BUCKETS``)."""
    if not lengths:
        return [512]
    ordered = sorted(lengths)
    return sorted({ordered[len(ordered) * i // n_bins] for i in range(1, n_bins)} | {ordered[-1]})


def create_bucketed_batches(windows, batch_size: int = 64, shuffle: bool = True, seed: int | None = None, indices: list[int] | None = None,
                            show_progress: bool = False, length_bins: list[int] | None = None):
    """Batches ``(byte_ids, masks, lengths)`` grouped by length bucket. ``windows``: a list of :class:`MaskWindow` or a
    :class:`LineMaskDataset` (then ``indices`` selects windows of it, the call form of the reference,
    src/heuristic_secrets/bytemasker/dataset.py:351-416); ``length_bins`` replaces the default bucket edges."""
    if isinstance(windows, LineMaskDataset):
        windows = windows.windows if indices is None else [windows.windows[i] for i in indices]
    elif indices is not None:
        windows = [windows[i] for i in indices]
    edges = tuple(sorted(length_bins)) if length_bins else BUCKETS
    rng = random.Random(seed)
    buckets: dict[int, list[MaskWindow]] = {}
    for w in windows:
        b = next((x for x in edges if len(w.data) <= x), edges[-1] + 1)
        buckets.setdefault(b, []).append(w)
    batches = []
    for members in buckets.values():
        if shuffle:
            rng.shuffle(members)
        for k in range(0, len(members), batch_size):
            part = members[k:k + batch_size]
            lengths = torch.tensor([len(w.data) for w in part])
            L = int(lengths.max())
            ids = torch.zeros(len(part), L, dtype=torch.long)
            masks = torch.zeros(len(part), L)
            for r, w in enumerate(part):
                ids[r, : len(w.data)] = torch.frombuffer(bytearray(w.data), dtype=torch.uint8).long()
                masks[r, : len(w.data)] = torch.tensor(w.mask, dtype=torch.float32)
            batches.append((ids, masks, lengths))
    if shuffle:
        rng.shuffle(batches)
    return batches


# ------------------------------------------------------------------------------------------------ files, caches, stats
def load_spanfinder_samples(path) -> list[SpanFinderSample]:
    with open(path) as fh:
        return [SpanFinderSample.from_dict(json.loads(line)) for line in fh if line.strip()]


def load_all_documents(data_dir, show_progress: bool = False) -> list[SpanFinderSample]:
    docs = []
    for split in ("train", "val", "test"):
        path = Path(data_dir) / "splits" / "documents" / f"{split}.jsonl"
        if path.exists():
            part = load_spanfinder_samples(path)
            docs.extend(part)
            if show_progress:
                print(f"  {split}: {len(part):,} documents")
    return docs


class LineMaskDataset(torch.utils.data.Dataset):
    """``(byte ids int64 [L], mask float32 [L])`` per window."""

    def __init__(self, windows: list[MaskWindow]):
        self.windows = windows

    # the attribute names the reference's dataset exposes (src/heuristic_secrets/bytemasker/dataset.py:281-313), computed
    # on first use: index lists of windows with / without a secret, per-window tensors and lengths
    @property
    def lines(self) -> list[MaskWindow]:
        return self.windows

    @functools.cached_property
    def secret_lines(self) -> list[int]:
        return [i for i, w in enumerate(self.windows) if w.has_secret]

    @functools.cached_property
    def clean_lines(self) -> list[int]:
        return [i for i, w in enumerate(self.windows) if not w.has_secret]

    @functools.cached_property
    def lengths(self) -> list[int]:
        return [len(w.data) for w in self.windows]

    @functools.cached_property
    def byte_tensors(self) -> list[torch.Tensor]:
        return [self[i][0] for i in range(len(self))]

    @functools.cached_property
    def mask_tensors(self) -> list[torch.Tensor]:
        return [self[i][1] for i in range(len(self))]

    def __len__(self) -> int:
        return len(self.windows)

    def __getitem__(self, i: int):
        w = self.windows[i]
        return torch.frombuffer(bytearray(w.data), dtype=torch.uint8).long(), torch.tensor(w.mask, dtype=torch.float32)

    @classmethod
    def from_spanfinder_file(cls, path, max_len: int = 512, seed: int = 0) -> "LineMaskDataset":
        rng = random.Random(seed)
        return cls([w for s in load_spanfinder_samples(path) for w in windows_from_document(s, max_len, rng)])


@dataclass
class DatasetStats:
    windows: int = 0
    with_secret: int = 0
    total_bytes: int = 0
    secret_bytes: int = 0
    unique_secrets: int = 0
    by_kind: dict = field(default_factory=dict)

    def __str__(self) -> str:
        frac = self.secret_bytes / max(self.total_bytes, 1)
        kinds = ", ".join(f"{k} {v:,}" for k, v in sorted(self.by_kind.items()))
        return (f"{self.windows:,} windows ({self.with_secret:,} with a secret; {kinds}), {self.total_bytes:,} bytes, "
                f"{100 * frac:.2f} % secret bytes, {self.unique_secrets:,} distinct secrets")


def compute_stats(windows) -> DatasetStats:
    windows = windows.windows if isinstance(windows, LineMaskDataset) else windows
    st = DatasetStats(windows=len(windows))
    ids = set()
    for w in windows:
        n = sum(w.mask)
        st.with_secret += n > 0
        st.total_bytes += len(w.data)
        st.secret_bytes += n
        st.by_kind[w.kind] = st.by_kind.get(w.kind, 0) + 1
        ids.update(w.secret_ids)
    st.unique_secrets = len(ids)
    return st


def cache_dir() -> Path:
    return Path(os.environ.get("HEURISTIC_SECRETS_CACHE", Path.home() / ".cache" / "heuristic-secrets")) / "bytemasker"


def _cache_file(source: Path, split: str, params: dict, secrets_only: bool) -> Path:
    parts = [str(source.resolve()), split] + [f"{k}={params[k]}" for k in sorted(params)]
    if source.exists():
        parts.append(f"{source.stat().st_mtime_ns}:{source.stat().st_size}")
    key = hashlib.md5("|".join(parts).encode()).hexdigest()[:12]
    return cache_dir() / f"windows_{split}_{'secrets_' if secrets_only else ''}{key}.jsonl"


def _write_cache(path: Path, windows: list[MaskWindow], stats: DatasetStats) -> None:
    path.parent.mkdir(parents=True, exist_ok=True)
    tmp = path.with_suffix(f".tmp{os.getpid()}")
    with open(tmp, "w") as fh:
        fh.write(json.dumps({"stats": asdict(stats)}) + "\n")
        for w in windows:
            # run-length coded mask: secrets are a few long runs, a list of 0/1 per byte would dominate the file
            runs, last, start = [], 0, 0
            for i, m in enumerate(w.mask + [0]):
                if m != last:
                    if last:
                        runs.append([start, i])
                    start, last = i, m
            fh.write(json.dumps({"d": w.data.hex(), "r": runs, "s": w.secret_ids, "k": w.kind}) + "\n")
    os.replace(tmp, path)


def _read_cache(path: Path, secrets_only: bool = False):
    try:
        with open(path) as fh:
            header = json.loads(fh.readline())
            windows = []
            for line in fh:
                o = json.loads(line)
                data = bytes.fromhex(o["d"])
                mask = [0] * len(data)
                for a, b in o["r"]:
                    mask[a:b] = [1] * (b - a)
                if secrets_only and not o["r"]:
                    continue
                windows.append(MaskWindow(data, mask, o["s"], o["k"]))
    except (OSError, ValueError, KeyError):
        return None                     # unreadable or truncated cache: rebuild
    stats = compute_stats(windows) if secrets_only else DatasetStats(**header["stats"])
    return windows, stats


def load_bytemasker_dataset(data_dir, split: str = "train", max_len: int = 512, prefix_len: int = 64, suffix_len: int = 64,
                            use_cache: bool = True, secrets_only: bool = False, seed: int = 0):
    """``(LineMaskDataset, DatasetStats)`` of one document split, through the JSON-lines window cache. A request for
    ``secrets_only`` is served from the full cache of the same split when that exists."""
    source = Path(data_dir) / "splits" / "documents" / f"{split}.jsonl"
    params = dict(max_len=max_len, prefix_len=prefix_len, suffix_len=suffix_len, seed=seed)
    own, full = _cache_file(source, split, params, secrets_only), _cache_file(source, split, params, False)
    if use_cache:
        for path, filt in ((own, False), (full, secrets_only)):
            if path.exists():
                got = _read_cache(path, secrets_only=filt)
                if got is not None:
                    if path is not own:
                        _write_cache(own, *got)
                    return LineMaskDataset(got[0]), got[1]
    rng = random.Random(seed)
    windows = [w for s in load_spanfinder_samples(source) for w in windows_from_document(s, max_len, rng, prefix_len, suffix_len)]
    if secrets_only:
        windows = [w for w in windows if any(w.mask)]
    stats = compute_stats(windows)
    if use_cache:
        _write_cache(own, windows, stats)
    return LineMaskDataset(windows), stats


MIN_WINDOW_LENGTH = 8


def load_mixed_windows(data_dir, split: str = "train", max_len: int = 512, seed: int = 0, **window_kw):
    """All window kinds (lines, multi-line, secret-only) of one split plus the set of secret ids they contain."""
    source = Path(data_dir) / "splits" / "documents" / f"{split}.jsonl"
    rng = random.Random(seed)
    windows = [w for s in load_spanfinder_samples(source) for w in windows_from_document(s, max_len, rng, **window_kw)
               if len(w.data) >= MIN_WINDOW_LENGTH]
    return windows, {i for w in windows for i in w.secret_ids}


def load_and_split_mixed_windows(data_dir, train_ratio: float = 0.88, val_ratio: float = 0.12, seed: int = 42,
                                 max_len: int = 512, show_progress: bool = False, **window_kw):
    """Ignores the document-level split on disk: windows of ALL documents are re-split by secret components.
    Returns ``((train windows, train secret ids), (val windows, val secret ids))`` and raises if a secret leaks."""
    rng = random.Random(seed)
    windows = [w for s in load_all_documents(data_dir, show_progress) for w in windows_from_document(s, max_len, rng, **window_kw)
               if len(w.data) >= MIN_WINDOW_LENGTH]
    rest = max(1.0 - train_ratio - val_ratio, 0.0)
    train, val, extra = stratified_component_split(windows, (train_ratio, val_ratio, rest), seed)
    train = train + extra if rest == 0.0 else train
    ids = lambda ws: {i for w in ws for i in w.secret_ids}
    leak = ids(train) & ids(val)
    if leak:
        raise RuntimeError(f"secret leakage: {len(leak)} secrets occur in both train and val")
    if show_progress:
        print(f"  train {compute_stats(train)}\n  val   {compute_stats(val)}")
    return (train, ids(train)), (val, ids(val))
