import torch
import torch.nn as nn

from ml_experiments_b200.models import unified as U
from ml_experiments_b200.models.unified import ensemble, features, ponder, train as T


def _toy(n=96, seed=0):
    g = torch.Generator().manual_seed(seed)
    xs, ys, ls = [], [], []
    for i in range(n):
        L = int(torch.randint(10, 60, (1,), generator=g))
        y = i % 2
        x = torch.randint(97, 123, (L,), generator=g)
        if y:
            x[L // 2:L // 2 + 4] = torch.tensor([48, 49, 50, 51])  # "0123" marks a positive
        xs.append(x), ys.append(float(y)), ls.append(L)
    return xs, ys, ls


def _small_cfg(head="classifier", n_classes=2):
    return U.ModelConfig(n_layers=1, layer=U.LayerConfig(embed_width=16, dropout=0.0, attn_heads=2, ssm_n_heads=2, ssm_state_size=8,
                                                         ssm_kernel_sizes=(3, 5)), head=U.HeadConfig(head, n_classes))


def test_trainer_learns_checkpoints_and_bins(tmp_path):
    xs, ys, ls = _toy()
    batches = T.create_binary_batches(xs, ys, ls, batch_size=16, seed=1)
    assert sum(len(b.labels) for b in batches) == len(xs)
    assert all((b.lengths <= b.bytes.shape[1]).all() for b in batches)
    cfg = T.TrainConfig(lr=3e-3, epochs=6, warmup_epochs=1, seed=0, threshold_search=True, curriculum_start_epoch=1)
    tr = T.Trainer(U.Model(_small_cfg()), batches, batches[:3], cfg, device=torch.device("cpu"))
    decay, no_decay = tr._get_param_groups(tr.model)
    names = {id(p): n for n, p in tr.model.named_parameters()}
    assert all("bias" not in names[id(p)] for p in decay) and any("A_log" in names[id(p)] for p in no_decay)
    first = tr.train_epoch(0)
    for e in range(1, 6):
        last = tr.train_epoch(e)
    assert last.loss < first.loss
    assert tr.swa_active and tr.get_batch_time_stats()["count"] >= len(batches)
    m = tr.validate(optimize_threshold=True)
    assert 0.1 <= tr.optimal_threshold <= 0.9 and m.eval_tokens_per_sec > 0 and "loss=" in str(m)
    tr.finalize_swa()
    tr.save_checkpoint(tmp_path / "ck.pt", extra={"epoch": 5}, with_optimizer=True)
    model, tr2, data = T.Trainer.load_checkpoint(tmp_path / "ck.pt", device=torch.device("cpu"))
    assert data["epoch"] == 5 and "optimizer" in data and tr2.optimal_threshold == tr.optimal_threshold
    prof = tr.profile_batch(0, warmup=0, runs=1)
    assert "profile_table" in prof and prof["mean_time"] > 0


def test_mask_and_multiclass_losses():
    xs, ys, ls = _toy(32)
    masks = [torch.zeros(L) for L in ls]
    mb = T.create_mask_batches(xs, masks, ls, batch_size=8, seed=0)
    tr = T.Trainer(U.Model(_small_cfg("mask")), mb, mb, T.TrainConfig(epochs=1, use_swa=False, pos_weight=3.0), device=torch.device("cpu"))
    assert tr.train_epoch(0).loss > 0 and tr.validate().loss > 0
    bb = [T.BinaryBatch(b.bytes, torch.randint(0, 3, (b.bytes.shape[0],)).float(), b.lengths) for b in mb]
    tr = T.Trainer(U.Model(_small_cfg("classifier", 3)), bb, bb, T.TrainConfig(epochs=1, use_swa=False), device=torch.device("cpu"))
    m = tr.train_epoch(0)
    assert 0 <= m.accuracy <= 1 and tr.validate().accuracy >= 0


def test_threshold_search_objectives():
    import numpy as np
    probs = np.array([0.2, 0.3, 0.55, 0.6, 0.8, 0.95])
    truth = np.array([0, 0, 1, 0, 1, 1])
    assert 0.3 < T.find_optimal_threshold(probs, truth, optimize_for="f1") <= 0.55
    assert T.find_optimal_threshold(probs, truth, optimize_for="recall", min_precision=0.7) <= 0.55


def test_ensemble_matches_member_mean():
    torch.manual_seed(0)
    ens = ensemble.Ensemble(_small_cfg(), n_members=3).eval()
    x = torch.randint(0, 256, (4, 20))
    mean, var = ens.forward_with_variance(x)
    want = torch.stack([torch.sigmoid(m(x)[0]) for m in ens.models])
    assert torch.allclose(mean, want.mean(0), atol=1e-5) and torch.allclose(var, want.var(0), atol=1e-5)
    assert torch.allclose(ens(x), mean)


def test_feature_zoo_and_combiner():
    torch.manual_seed(0)
    feats = nn.ModuleList([features.ConvFeature(16, (3, 5), groups=2, dropout=0.0), features.AttentionFeature(16, 1, 2, dropout=0.0),
                           features.HeuristicFeature(lambda b: float(len(b))), features.PrecomputedFeature(1)])
    comb = features.FeatureCombiner(feats, hidden_dims=(8, 4), use_gates=True)
    x = torch.randint(0, 256, (3, 12))
    mask = torch.arange(12)[None] >= torch.tensor([12, 7, 3])[:, None]
    out = comb(x, mask, precomputed=torch.randn(3, 2))
    assert out.shape == (3, 4) and comb.output_dim == 4
    assert feats[2](x, mask).view(-1).tolist() == [12.0, 7.0, 3.0]
    out.sum().backward()


def test_ponder_trainer_runs():
    torch.manual_seed(0)
    class Base(nn.Module):
        def __init__(self):
            super().__init__()
            self.head = nn.Linear(16, 4)

        def forward(self, x):
            return self.head(x.flatten(1))

    base = Base()
    pw = ponder.PonderWrapper(base)
    assert pw.n_classes == 4
    data = [(torch.randn(8, 1, 4, 4), torch.randint(0, 4, (8,))) for _ in range(4)]
    tr = ponder.PonderTrainer(pw, data, data, torch.device("cpu"), ponder.PonderTrainConfig(epochs=3, meta_warmup_epochs=1, meta_wean_epochs=1),
                              flatten_input=True)
    assert tr._reinforce_alpha(0) == 0.0 and tr._reinforce_alpha(2) == 1.0
    acc = tr.train(3, verbose=False)
    assert 0.0 <= acc <= 1.0
    logits, pl, raw = pw(torch.randn(2, 16), torch.tensor([0, 1]))
    assert (raw > 0).all() and pl.shape == (2,)
