"""Shallow ``git clone`` helper for collectors that scrape tool repositories
(reference: src/heuristic_secrets/data/git_utils.py:5-48)."""
from __future__ import annotations

import shutil
import subprocess
from pathlib import Path


def clone_or_update(url: str, dest: Path, force: bool = False, timeout: int = 600) -> Path:
    dest = Path(dest)
    if dest.exists() and force:
        shutil.rmtree(dest)
    if dest.exists() and any(dest.iterdir()):
        return dest
    dest.parent.mkdir(parents=True, exist_ok=True)
    subprocess.run(["git", "clone", "--depth", "1", url, str(dest)], check=True, capture_output=True, timeout=timeout)
    return dest
