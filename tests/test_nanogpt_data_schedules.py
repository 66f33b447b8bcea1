"""Shard format, document-aligned batches, bigram hash and the speedrun schedules (CPU)."""
import numpy as np
import torch

from ml_experiments_b200.data.nanogpt_loader import (BOS_ID, BOSFinder, distributed_data_generator, get_bigram_hash,
                                                     load_data_shard, write_data_shard)
from ml_experiments_b200.trainers import schedules as S


def _shard(tmp_path, name, n_docs=200, seed=0):
    rng = np.random.default_rng(seed)
    toks = []
    for _ in range(n_docs):
        toks += [BOS_ID] + rng.integers(0, 50000, size=rng.integers(20, 400)).tolist()
    write_data_shard(tmp_path / name, toks)
    return np.asarray(toks, dtype=np.uint16)


def test_shard_roundtrip_and_batches(tmp_path):
    toks = _shard(tmp_path, "train_000.bin")
    _shard(tmp_path, "train_001.bin", seed=1)
    assert np.array_equal(load_data_shard(tmp_path / "train_000.bin"), toks)
    f = BOSFinder(toks, world_size=2)
    starts, ends = f.next_batch(1024, 256)
    for r in range(2):
        assert sum(e - s for s, e in zip(starts[r], ends[r])) == 1025
        assert all(toks[s] == BOS_ID and e - s <= 256 for s, e in zip(starts[r], ends[r]))
    assert starts[1][0] > starts[0][-1]
    gen = distributed_data_generator(str(tmp_path / "train_*.bin"), 2048, 256, rank=1, world_size=2, device=None)
    x, y, cl, bg = next(gen)
    assert x.dtype == torch.int32 and y.dtype == torch.int64 and cl.dtype == torch.int32 and x.numel() == 1024 == y.numel()
    assert torch.equal(x[1:].long(), y[:-1]) and x[0] == BOS_ID and cl[0] == 0 and cl.numel() % 128 == 0
    assert bool((x[cl[1:4].long()] == BOS_ID).all())
    x2, *_ = gen.send((4096, 512, 1))
    assert x2.numel() == 2048
    n = sum(1 for _ in gen)  # runs into the second shard and stops cleanly at the end of the data
    assert n >= 1


def test_bigram_hash():
    x = torch.tensor([5, 7, 9, 11], dtype=torch.int32)
    h = get_bigram_hash(x, 1000)
    assert h[0] == 999 and h[1] == ((36313 * 7) ^ (27191 * 5)) % 999 and h[3] == ((36313 * 11) ^ (27191 * 9)) % 999


def test_schedules():
    a = S.ScheduleArgs()
    assert S.get_bs(0, a) == 8 * 2048 * 8 and S.get_bs(600, a) == 16 * 2048 * 8 and S.get_bs(1540, a) == 24 * 2048 * 8
    assert S.get_ws(0, a) == (1, 3) and S.get_ws(1200, a) == (5, 11) and S.get_ws(1560, a) == (6, 13)
    assert S.get_lr(0, a) == 1.0 and abs(S.get_lr(a.num_scheduled_iterations, a) - 0.1) < 1e-9 and S.get_lr(1536, a) == 0.1
    assert S.get_lr(600, a) == 1.52
    assert S.get_muon_momentum(0, a) == 0.85 and S.get_muon_momentum(400, a) == 0.95 and S.get_muon_momentum(a.num_iterations, a) == 0.85
    assert len(S.mtp_weights(0, a)) == 3 and len(S.mtp_weights(700, a)) == 2 and S.mtp_weights(1500, a) == [1.0]
    y = S.Yarn(128, 4096)
    f0, s0 = y.angular_freq.clone(), y.attn_scale
    m = S.TrainingManager(a, y)
    i0 = m.advance_schedule(0)
    assert i0["batch_changed"] and i0["window_changed"] and not i0["do_adam"]
    i1 = m.advance_schedule(1)
    assert not i1["batch_changed"] and i1["do_adam"]
    m.advance_schedule(600)
    assert y.attn_scale > s0 and (y.angular_freq <= f0 + 1e-9).all() and y.cos.shape == (8192, 64)
