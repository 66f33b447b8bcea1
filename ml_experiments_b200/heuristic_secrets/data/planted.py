"""Seeded synthetic span data: printable-ASCII noise with planted hex / base64 runs.

Each sequence is ``seq_len`` bytes drawn uniformly from 0x20-0x7E; 0-3 runs of random hex or base64 characters,
16-64 bytes long, are written at uniform-random offsets. Labels follow the SpanFinder dataset convention of the
reference (src/heuristic_secrets/spanfinder/dataset.py:72-91): channel 0 marks the first byte of a run, channel 1 its
inclusive last byte.
"""
from __future__ import annotations

import torch

_HEX = torch.tensor(list(b"0123456789abcdef"), dtype=torch.long)
_B64 = torch.tensor(list(b"ABCDEFGHIJKLMNOPQRSTUVWXYZabcdefghijklmnopqrstuvwxyz0123456789+/"), dtype=torch.long)


def planted_span_batch(batch: int = 16, seq_len: int = 512, seed: int = 0, max_spans: int = 3, min_len: int = 16,
                       max_len: int = 64):
    """Returns ``(byte_ids [B, L] int64, targets [B, L, 2] float32, lengths [B] int64, spans)``."""
    g = torch.Generator().manual_seed(seed)
    ids = torch.randint(0x20, 0x7F, (batch, seq_len), generator=g, dtype=torch.long)
    targets = torch.zeros(batch, seq_len, 2)
    spans: list[list[tuple[int, int]]] = []
    for b in range(batch):
        n = int(torch.randint(0, max_spans + 1, (1,), generator=g))
        row = []
        for _ in range(n):
            ln = int(torch.randint(min_len, max_len + 1, (1,), generator=g))
            off = int(torch.randint(0, seq_len - ln + 1, (1,), generator=g))
            alphabet = _HEX if int(torch.randint(0, 2, (1,), generator=g)) == 0 else _B64
            ids[b, off:off + ln] = alphabet[torch.randint(0, len(alphabet), (ln,), generator=g)]
            targets[b, off, 0] = 1.0
            targets[b, off + ln - 1, 1] = 1.0
            row.append((off, off + ln))
        spans.append(row)
    lengths = torch.full((batch,), seq_len, dtype=torch.long)
    return ids, targets, lengths, spans
