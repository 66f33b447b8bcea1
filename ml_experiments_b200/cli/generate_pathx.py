"""Write Path-X style splits as ``<output-dir>/{train,val,test}.npz`` (``x`` uint8 ``[n, size, size]``, ``y`` int64)
(role of the reference's ``scripts/generate_pathx.py``; the images come from :mod:`ml_experiments_b200.data.pathfinder`).

    python -m ml_experiments_b200.cli.generate_pathx --n-train 160000 --n-val 20000 --n-test 20000 --size 256
"""
from __future__ import annotations

import argparse
from pathlib import Path

import numpy as np

from ..data import pathfinder


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--output-dir", default=".cache/pathx")
    ap.add_argument("--n-train", type=int, default=160000)
    ap.add_argument("--n-val", type=int, default=20000)
    ap.add_argument("--n-test", type=int, default=20000)
    ap.add_argument("--size", type=int, default=256)
    ap.add_argument("--contour-length", type=int, default=14)
    ap.add_argument("--marker-radius", type=int, default=5)
    ap.add_argument("--continuity", type=float, default=1.8)
    ap.add_argument("--seed", type=int, default=0)
    a = ap.parse_args(argv)
    out = Path(a.output_dir)
    out.mkdir(parents=True, exist_ok=True)
    for i, (split, n) in enumerate((("train", a.n_train), ("val", a.n_val), ("test", a.n_test))):
        if n <= 0:
            continue
        x, y = pathfinder.generate(n, a.size, a.seed + 1000 * i, contour_length=a.contour_length, marker_radius=a.marker_radius,
                                   continuity=a.continuity)
        np.savez_compressed(out / f"{split}.npz", x=x, y=y)
        # the flat per-split cache the reference's trainer reads (scripts/train_pathx.py:48-60): pixel rows, labels and
        # the index lists of the two classes
        np.savez_compressed(out / f"pathx_{split}_cache.npz", pixels=x.reshape(len(x), -1), labels=y.astype(np.int64),
                            pos_indices=np.flatnonzero(y == 1), neg_indices=np.flatnonzero(y == 0))
        print(f"{split}: {n} images of {a.size}x{a.size} -> {out / (split + '.npz')} ({y.mean():.2f} positive)")
    return out


if __name__ == "__main__":
    main()
