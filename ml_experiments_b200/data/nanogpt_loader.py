"""Token-shard data loader of the GPT trainers.

File format and batch semantics follow the reference (modded-nanogpt/train_gpt.py:1304-1495, data/fineweb.py): a
``.bin`` shard is a 256 x int32 header (magic 20240520, version 1, token count) followed by uint16 tokens. Batches are
assembled from whole documents: every sequence starts at a BOS token (id 50256), is cut at ``max_seq_len`` and the
per-rank token budget, ranks take consecutive documents, and the generator accepts ``.send((num_tokens, max_seq_len,
grad_accum_steps))`` to change the batch size between steps. Each item is ``(inputs int32, targets int64, cum_seqlens
int32 padded to a multiple of 128 documents, bigram hash int32)``.

Differences by design: the shard is memory-mapped and the document cut points of a batch are computed with
vectorised numpy (no Python loop over the shard), the next shard is opened by a background thread, and host buffers
are pinned once and reused; with ``device=None`` the tensors stay on the host (used by CPU tests).
"""
from __future__ import annotations

import glob
import threading
from pathlib import Path

import numpy as np
import torch

MAGIC, VERSION, BOS_ID = 20240520, 1, 50256


def write_data_shard(path, tokens) -> None:
    toks = np.asarray(tokens, dtype=np.uint16)
    header = np.zeros(256, dtype=np.int32)
    header[0], header[1], header[2] = MAGIC, VERSION, len(toks)
    with open(path, "wb") as f:
        f.write(header.tobytes())
        f.write(toks.tobytes())


def load_data_shard(file) -> np.ndarray:
    header = np.fromfile(str(file), dtype=np.int32, count=256)
    assert header[0] == MAGIC, "magic number mismatch in the data .bin file"
    assert header[1] == VERSION, "unsupported version"
    n = int(header[2])
    toks = np.memmap(str(file), dtype=np.uint16, mode="r", offset=256 * 4, shape=(n,))
    assert toks.shape[0] == n, "number of tokens read does not match header"
    return toks


def next_multiple_of_n(v, *, n: int) -> int:
    return next(x for x in range(n, int(v) + 1 + n, n) if x >= v)


class BOSFinder:
    """Document-aligned batch assembly over one shard."""

    def __init__(self, tokens: np.ndarray, world_size: int = 1):
        self.tokens, self.size, self.world_size = tokens, len(tokens), world_size
        self.bos_idx = np.flatnonzero(np.asarray(tokens) == BOS_ID).astype(np.int64)
        self.i = 0

    def next_batch(self, num_tokens_local: int, max_seq_len: int):
        n = len(self.bos_idx)
        starts = [[] for _ in range(self.world_size)]
        ends = [[] for _ in range(self.world_size)]
        idx = self.i
        nxt = np.append(self.bos_idx[1:], self.size)
        for r in range(self.world_size):
            cur_len = 0
            while cur_len <= num_tokens_local:
                if idx >= n:
                    raise StopIteration("Insufficient BOS ahead; hit tail of shard.")
                cur = int(self.bos_idx[idx])
                end = min(int(nxt[idx]), cur + max_seq_len, cur + num_tokens_local - cur_len + 1)
                starts[r].append(cur)
                ends[r].append(end)
                cur_len += end - cur
                idx += 1
            assert cur_len == num_tokens_local + 1
        self.i = idx
        return starts, ends


def get_bigram_hash(x: torch.Tensor, bigram_vocab_size: int) -> torch.Tensor:
    """``xor(36313 * cur, 27191 * prev) % (V - 1)``; position 0 maps to the reserved index ``V - 1``."""
    mod = bigram_vocab_size - 1
    x = x.to(torch.int32).clone()
    out = x.clone()
    out[0] = mod
    out[1:] = torch.bitwise_xor(36313 * x[1:], 27191 * x[:-1]) % mod
    return out


class _Preloader:
    def __init__(self, file_iter, world_size):
        self.file_iter, self.world_size, self.thread, self.data = file_iter, world_size, None, None

    def _load(self):
        try:
            toks = load_data_shard(next(self.file_iter))
            self.data = (toks, BOSFinder(toks, self.world_size))
        except StopIteration:
            self.data = None

    def start(self):
        self.thread = threading.Thread(target=self._load, daemon=True)
        self.thread.start()

    def get(self):
        if self.thread:
            self.thread.join()
        return self.data


def distributed_data_generator(filename_pattern: str, num_tokens: int, max_seq_len: int, grad_accum_steps: int = 1,
                               align_to_bos: bool = True, rank: int = 0, world_size: int = 1, device="cuda",
                               bigram_vocab_size: int = 50304 * 5):
    assert num_tokens % (world_size * grad_accum_steps) == 0, "Batch size must be divisible by world size"
    num_tokens //= grad_accum_steps
    files = [Path(f) for f in sorted(glob.glob(filename_pattern))]
    if not files:
        raise FileNotFoundError(f"No files found for pattern: {filename_pattern}")
    file_iter = iter(files)
    tokens = load_data_shard(next(file_iter))
    finder = BOSFinder(tokens, world_size) if align_to_bos else None
    pre = _Preloader(file_iter, world_size)
    pre.start()
    pos = 0
    pin = device is not None and torch.cuda.is_available()
    while True:
        local = num_tokens // world_size
        max_docs = next_multiple_of_n(local // 300, n=128)
        if align_to_bos:
            try:
                seq_starts, seq_ends = finder.next_batch(local, max_seq_len)
            except StopIteration:
                nxt = pre.get()
                if nxt is None:
                    return
                tokens, finder = nxt
                pre.start()
                continue
            s, e = np.asarray(seq_starts[rank]), np.asarray(seq_ends[rank])
            buf = np.concatenate([tokens[a:b] for a, b in zip(s, e)]).astype(np.int64)
            e = e.copy()
            e[-1] -= 1
            cum = np.cumsum(e - s)
        else:
            if pos + num_tokens + 1 >= len(tokens):
                nxt = pre.get()
                if nxt is None:
                    return
                tokens, _ = nxt
                pre.start()
                pos = 0
            lo = pos + rank * local
            buf = np.asarray(tokens[lo:lo + local + 1]).astype(np.int64)
            cum = np.flatnonzero(buf[:-1] == BOS_ID)
            pos += num_tokens
        cum_lengths = np.full(max(max_docs, len(cum) + 1), local, dtype=np.int32)
        cum_lengths[0] = 0
        cum_lengths[1:len(cum) + 1] = cum
        inputs = torch.from_numpy(buf[:-1].astype(np.int32))
        targets = torch.from_numpy(buf[1:].copy())
        cl = torch.from_numpy(cum_lengths)
        bigram = get_bigram_hash(inputs, bigram_vocab_size)
        items = (inputs, targets, cl, bigram)
        if device is not None:
            items = tuple((t.pin_memory() if pin else t).to(device, non_blocking=True) for t in items)
        new = yield items
        if new is not None:
            new_tokens, max_seq_len, new_accum = new
            assert new_tokens % (world_size * new_accum) == 0, "Num tokens must be divisible by world size"
            num_tokens = new_tokens // new_accum
