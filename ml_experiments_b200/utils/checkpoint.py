"""Checkpoint IO: atomic ``torch.save`` of state-dict dictionaries, per-rank shards of sharded optimizer state, and
re-sharding on load when the world size changed.

The reference saves plain ``torch.save`` dictionaries (src/heuristic_secrets/models/train.py:862-896,
scripts/train_line_filter.py:893-914, modded-nanogpt/train_gpt.py:1890-1894); its sharded optimizer state exists only
on the owning rank and a rank-0 save loses the other shards. Here every rank writes ``<path>.rank{r}`` for its shard,
rank 0 writes the replicated part, and ``load_sharded`` concatenates the shards along dim 0 and re-slices them for the
current world size. RNG state and a loader position can be stored alongside.
"""
from __future__ import annotations

import os
import random

import numpy as np
import torch


def save_checkpoint(obj: dict, path) -> None:
    tmp = f"{path}.tmp.{os.getpid()}"
    torch.save(obj, tmp)
    os.replace(tmp, path)


def load_checkpoint(path, map_location="cpu") -> dict:
    return torch.load(path, map_location=map_location, weights_only=False)


def rng_state() -> dict:
    st = {"python": random.getstate(), "numpy": np.random.get_state(), "torch": torch.get_rng_state()}
    if torch.cuda.is_available():
        st["cuda"] = torch.cuda.get_rng_state_all()
    return st


def set_rng_state(st: dict) -> None:
    random.setstate(st["python"])
    np.random.set_state(st["numpy"])
    torch.set_rng_state(st["torch"])
    if "cuda" in st and torch.cuda.is_available():
        torch.cuda.set_rng_state_all(st["cuda"])


def save_sharded(replicated: dict, shard: dict, path, rank: int, world_size: int, rows: dict | None = None) -> None:
    """``replicated`` is written by rank 0 to ``path``; every rank writes its ``shard`` (name -> tensor sliced along
    dim 0) to ``path.rank{rank}``. ``rows`` (name -> number of meaningful rows of the concatenated tensor) is stored
    when the shards are padded to a multiple of the world size, so that a load under another world size can drop the
    padding before it re-partitions."""
    if rank == 0:
        save_checkpoint({**replicated, "world_size": world_size, "shard_rows": dict(rows or {})}, path)
    save_checkpoint({"rank": rank, "world_size": world_size, "shard": shard}, f"{path}.rank{rank}")


def load_sharded(path, rank: int, world_size: int, map_location="cpu") -> tuple[dict, dict]:
    """Returns ``(replicated, shard_for_this_rank)``; shards saved under another world size are re-partitioned
    (padding rows recorded at save time are dropped first and the result is zero-padded to a multiple of the new
    world size)."""
    rep = load_checkpoint(path, map_location)
    old = rep.get("world_size", 1)
    rows = rep.get("shard_rows", {}) or {}
    parts = [load_checkpoint(f"{path}.rank{r}", map_location)["shard"] for r in range(old)]
    out = {}
    for name in parts[0]:
        full = torch.cat([p[name] for p in parts], dim=0)
        if name in rows:
            full = full[: rows[name]]
            pad = (-full.shape[0]) % world_size
            if pad:
                full = torch.cat([full, full.new_zeros((pad, *full.shape[1:]))], dim=0)
        assert full.shape[0] % world_size == 0, f"{name}: {full.shape[0]} rows do not divide over {world_size} ranks"
        per = full.shape[0] // world_size
        out[name] = full[rank * per:(rank + 1) * per].clone()
    return rep, out
