import torch

from ml_experiments_b200.utils import checkpoint as C


def test_atomic_and_resharding(tmp_path):
    path = tmp_path / "ck.pt"
    full = torch.arange(24.0).view(8, 3)
    for r in range(4):
        C.save_sharded({"step": 7, "model": {"w": torch.ones(2)}}, {"momentum": full[r * 2:(r + 1) * 2]}, path, r, 4)
    assert not list(tmp_path.glob("*.tmp*"))
    rep, shard = C.load_sharded(path, rank=1, world_size=2)
    assert rep["step"] == 7 and torch.equal(shard["momentum"], full[4:8])
    rep, shard = C.load_sharded(path, rank=0, world_size=1)
    assert torch.equal(shard["momentum"], full)
    st = C.rng_state()
    a = torch.rand(3)
    C.set_rng_state(st)
    assert torch.equal(a, torch.rand(3))
