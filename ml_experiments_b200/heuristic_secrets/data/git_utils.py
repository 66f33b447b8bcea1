"""``git`` helpers for collectors that read scanner repositories (reference: src/heuristic_secrets/data/git_utils.py:5-48)."""
from __future__ import annotations

import shutil
import subprocess
from pathlib import Path


def _git(*args: str, cwd: Path | None = None, timeout: int = 600) -> subprocess.CompletedProcess:
    return subprocess.run(["git", *args], cwd=None if cwd is None else str(cwd), check=True, capture_output=True, text=True, timeout=timeout)


def clone_or_update(url: str, dest: Path, force: bool = False, timeout: int = 600) -> Path:
    """Shallow clone into ``dest`` unless something is already there (``force`` removes it first); returns ``dest``."""
    dest = Path(dest)
    if dest.exists() and force:
        shutil.rmtree(dest)
    if dest.exists() and any(dest.iterdir()):
        return dest
    dest.parent.mkdir(parents=True, exist_ok=True)
    _git("clone", "--depth", "1", url, str(dest), timeout=timeout)
    return dest


def clone_or_pull(repo_url: str, dest: Path) -> None:
    """Clone ``repo_url`` into ``dest``, or fast-forward the checkout that is already there."""
    dest = Path(dest)
    if (dest / ".git").exists():
        _git("pull", "--ff-only", cwd=dest)
        return
    dest.parent.mkdir(parents=True, exist_ok=True)
    _git("clone", "--depth", "1", repo_url, str(dest))


def get_repo_version(repo_path: Path) -> str:
    """Commit hash of the checkout's ``HEAD`` (40 hex digits)."""
    return _git("rev-parse", "HEAD", cwd=Path(repo_path)).stdout.strip()
