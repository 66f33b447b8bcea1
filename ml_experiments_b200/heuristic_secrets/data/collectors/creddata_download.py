"""Materialises the Samsung CredData corpus from its ``snapshot.json``: every listed repository is fetched at the
pinned commit, its files are copied under ``data/<new repo id>/<scope>/<file id><ext>`` with the obfuscation the corpus
applies, and failures of single repositories are logged and skipped instead of ending the run.

Counterpart of the reference's patched download script (src/heuristic_secrets/data/collectors/creddata_download.py:26-279,
itself based on CredData's ``download_data.py``). Layout rules restated from there: the new repository id is the CRC-32 of
the 20-byte commit hash in hex; a file's id is the first 8 hex digits of the SHA-256 of ``<new repo id>/<path>``; the
scope folder is built from the ``word_in_path.json`` keywords that occur in the lower-cased path (``/_/`` when none does).
Fetching needs network access and ``git``; everything else is pure file handling and is tested on local repositories.
"""
from __future__ import annotations

import binascii
import hashlib
import json
import logging
import shutil
import subprocess
from dataclasses import dataclass, field
from pathlib import Path

log = logging.getLogger(__name__)


def new_repo_id(repo_id: str) -> str:
    return f"{binascii.crc32(binascii.unhexlify(repo_id[:40])):08x}"


def file_scope(path_without_ext: str, words: list[str]) -> str:
    probe = "./" + path_without_ext.lower()
    parts = [w.strip("/") for w in words if w in probe]
    return "/" + "/".join(p for p in parts if p) + "/" if parts else "/_/"


def file_id(repo: str, rel_path: str) -> str:
    return hashlib.sha256(f"{repo}/{rel_path}".encode()).hexdigest()[:8]


@dataclass
class DownloadReport:
    fetched: list[str] = field(default_factory=list)
    failed: dict[str, str] = field(default_factory=dict)
    files: int = 0


def fetch_repo(repo_id: str, url: str, tmp: Path, timeout: int = 900) -> Path:
    """Checks out ``repo_id[:40]`` of ``url`` under ``tmp/repo_id`` (re-used when already present)."""
    dest = tmp / repo_id
    sha = repo_id[:40]

    def git(*args, cwd=dest):
        subprocess.run(["git", *args], cwd=cwd, check=True, capture_output=True, timeout=timeout)

    if not (dest / ".git").exists():
        dest.mkdir(parents=True, exist_ok=True)
        git("init", "-q")
        git("remote", "add", "origin", url)
    try:
        git("fetch", "-q", "--depth", "1", "origin", sha)
    except subprocess.CalledProcessError:
        git("fetch", "-q", "origin")                     # servers that refuse fetching a bare commit id
    git("checkout", "-q", "-f", sha)
    return dest


def copy_repo_files(repo_dir: Path, repo_id: str, out: Path, words: list[str], max_bytes: int = 1 << 22) -> int:
    """Copies the tracked text files of one checkout into the corpus layout; returns how many were written."""
    rid = new_repo_id(repo_id)
    n = 0
    for f in sorted(p for p in repo_dir.rglob("*") if p.is_file() and ".git" not in p.relative_to(repo_dir).parts):
        rel = f.relative_to(repo_dir).as_posix()
        if f.stat().st_size > max_bytes:
            continue
        scope = file_scope(str(Path(rel).with_suffix("")), words)
        dst = out / "data" / rid / scope.strip("/") / (file_id(rid, rel) + f.suffix)
        dst.parent.mkdir(parents=True, exist_ok=True)
        shutil.copyfile(f, dst)
        n += 1
    return n


def download(creddata_dir: Path, out: Path | None = None, tmp: Path | None = None, limit: int | None = None) -> DownloadReport:
    """Fetches every repository of ``creddata_dir/snapshot.json``; a failing repository is recorded and skipped."""
    creddata_dir = Path(creddata_dir)
    out = Path(out or creddata_dir)
    tmp = Path(tmp or creddata_dir / "tmp")
    snapshot = json.loads((creddata_dir / "snapshot.json").read_text())
    words_file = creddata_dir / "word_in_path.json"
    words = json.loads(words_file.read_text()) if words_file.exists() else []
    report = DownloadReport()
    for i, (repo_id, url) in enumerate(sorted(snapshot.items())):
        if limit is not None and i >= limit:
            break
        try:
            repo = fetch_repo(repo_id, url, tmp)
            report.files += copy_repo_files(repo, repo_id, out, words)
            report.fetched.append(repo_id)
        except (subprocess.SubprocessError, OSError, ValueError) as e:
            log.warning("repository %s (%s) skipped: %s", repo_id, url, e)
            report.failed[repo_id] = f"{type(e).__name__}: {e}"[:300]
    return report


# -- the helper names of the reference's downloader (src/heuristic_secrets/data/collectors/creddata_download.py:26-240) --
def get_words_in_path(creddata_dir: Path) -> list[str]:
    return json.loads((Path(creddata_dir) / "word_in_path.json").read_text())


get_file_scope = file_scope
get_new_repo_id = new_repo_id


def download_repo(repo_id: str, repo_url: str, tmp_dir: Path) -> bool:
    """True when the pinned commit could be checked out under ``tmp_dir``."""
    try:
        fetch_repo(repo_id, repo_url, Path(tmp_dir))
        return True
    except (subprocess.SubprocessError, OSError):
        return False


def read_meta_csv(meta_file: Path) -> list[dict]:
    import csv
    if not Path(meta_file).exists():
        return []
    with open(meta_file, newline="", errors="ignore") as fh:
        return list(csv.DictReader(fh))


def process_repo(repo_id: str, repo_url: str, tmp_dir: Path, meta_dir: Path, data_dir: Path, words_in_path: list[str]) -> int:
    """Fetch one repository and copy its files into the corpus layout; returns the number of files written (0 when the
    fetch failed). ``meta_dir`` is not needed here: the copy keeps every text file, the labels are joined at collection."""
    if not download_repo(repo_id, repo_url, tmp_dir):
        return 0
    return copy_repo_files(Path(tmp_dir) / repo_id, repo_id, Path(data_dir).parent, words_in_path)


def run_download(creddata_dir: Path, skip_download: bool = False, jobs: int = 1) -> dict:
    """The whole download as a dictionary of counts (``jobs`` is accepted; repositories are fetched one after another)."""
    if skip_download:
        return {"fetched": 0, "failed": 0, "files": 0, "skipped": True}
    r = download(Path(creddata_dir))
    return {"fetched": len(r.fetched), "failed": len(r.failed), "files": r.files, "skipped": False}


def main(argv=None) -> int:
    import argparse

    ap = argparse.ArgumentParser(description="Fetch the CredData repositories at their pinned commits")
    ap.add_argument("creddata_dir", type=Path)
    ap.add_argument("--out", type=Path, default=None)
    ap.add_argument("--limit", type=int, default=None)
    a = ap.parse_args(argv)
    logging.basicConfig(level="INFO", format="%(asctime)s | %(levelname)s | %(message)s")
    rep = download(a.creddata_dir, a.out, limit=a.limit)
    print(json.dumps({"fetched": len(rep.fetched), "failed": len(rep.failed), "files": rep.files}))
    return 0 if rep.fetched or not rep.failed else 1


if __name__ == "__main__":
    raise SystemExit(main())
