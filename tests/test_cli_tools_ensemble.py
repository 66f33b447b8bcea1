"""Command-line tools around trained 1-D models: ensemble training, distillation, hard-negative mining, kernel inspection."""
import json

import torch


def test_vote_threshold_and_segments():
    from ml_experiments_b200.cli.mine_hard_negatives import mask_segments
    from ml_experiments_b200.cli.train_ensemble import best_vote_threshold, prf, vote_counts

    probs = torch.tensor([[0.9, 0.2, 0.6, 0.1], [0.8, 0.7, 0.4, 0.2], [0.7, 0.1, 0.7, 0.6]])
    y = torch.tensor([1.0, 0.0, 1.0, 0.0])
    assert vote_counts(probs, y, 0.5) == (2, 0, 0, 2)           # majority of three members per column
    assert vote_counts(probs, y, 0.05) == (2, 2, 0, 0)
    assert prf(2, 0, 0, 2)["f1"] == 1.0
    assert 0.1 <= best_vote_threshold(probs, y) <= 0.9
    m = torch.tensor([[0, 1, 1, 0, 1, 1], [1, 1, 0, 0, 0, 1]], dtype=torch.bool)
    assert mask_segments(m, torch.tensor([6, 4])) == [(0, 1, 3), (0, 4, 6), (1, 0, 2)]   # the run past row 1's length is cut


def test_distillation_loss_matches_its_definition():
    from ml_experiments_b200.cli.distill_1d import distillation_loss

    s, t, y = torch.tensor([0.5, -1.0, 2.0]), torch.tensor([1.5, -2.0, 0.5]), torch.tensor([1.0, 0.0, 1.0])
    T, alpha = 4.0, 0.7
    kl = torch.nn.functional.binary_cross_entropy(torch.sigmoid(s / T), torch.sigmoid(t / T)) * T * T
    task = torch.nn.functional.binary_cross_entropy_with_logits(s, y)
    loss, kl_, task_ = distillation_loss(s, t, y, T, alpha)
    assert torch.allclose(loss, alpha * kl + (1 - alpha) * task) and torch.allclose(kl_, kl) and torch.allclose(task_, task)
    only_kl, _, _ = distillation_loss(s, t, None, T, alpha)
    assert torch.allclose(only_kl, kl)


def test_ensemble_distill_and_mining_tools(tmp_path):
    from ml_experiments_b200.cli import distill_1d, mine_hard_negatives, train_bytemasker, train_ensemble, train_line_filter

    ens = train_ensemble.main(["--synthetic", "128", "--n-members", "2", "--epochs", "1", "--embed-width", "16", "--max-len", "64",
                               "--output", str(tmp_path / "ens.pt"), "--device", "cpu"])
    ck = torch.load(tmp_path / "ens.pt", weights_only=False)
    assert ck["n_members"] == 2 and len(ck["state_dicts"]) == 2 and 0.1 <= ck["optimal_threshold"] <= 0.9 and 0 <= ens["final"]["f1"] <= 1
    train_line_filter.main(["--synthetic", "128", "--head", "classifier", "--embed-width", "16", "--epochs", "1", "--max-len", "64", "--no-swa",
                            "--output", str(tmp_path / "teacher"), "--device", "cpu"])
    d = distill_1d.main(["--teacher", str(tmp_path / "teacher" / "final.pt"), "--synthetic", "128", "--student-width", "8", "--student-features", "4",
                         "--student-mlp-dim", "16", "--epochs", "1", "--max-len", "64", "--output", str(tmp_path / "student.pt"), "--device", "cpu"])
    assert d["student_params"] < d["teacher_params"] and 0.0 <= d["final"]["teacher_agreement"] <= 1.0
    st = torch.load(tmp_path / "student.pt", weights_only=False)
    assert st["model_config"]["layer"]["embed_width"] == 8 and st["distillation"] == {"temperature": 4.0, "alpha": 0.7}
    train_bytemasker.main(["--synthetic", "128", "--epochs", "1", "--width", "16", "--depth", "1", "--max-len", "64", "--output", str(tmp_path / "bm.pt"),
                           "--device", "cpu"])
    out = tmp_path / "hn.jsonl"
    s = mine_hard_negatives.main(["--masker-checkpoint", str(tmp_path / "bm.pt"), "--synthetic", "128", "--max-len", "64", "--threshold", "0.0",
                                  "--min-segment-len", "4", "--max-segment-len", "64", "--output", str(out), "--device", "cpu"])
    rows = [json.loads(l) for l in out.read_text().splitlines()]
    # threshold 0 marks every byte: each clean window that decodes as UTF-8 becomes one label-0 sample
    assert s["hard_negatives"] == len(rows) and all(r["label"] == 0 and r["source"] == "bytemasker_fp" for r in rows)
    assert s["clean_windows"] >= len(rows)


def test_inspect_kernels_reports_every_adaptive_branch(tmp_path, capsys):
    from ml_experiments_b200.cli import inspect_kernels
    from ml_experiments_b200.models.unified import HeadConfig, LayerConfig, Model, ModelConfig

    assert "all values" in inspect_kernels.ascii_histogram([1.0, 1.0]) and "#" in inspect_kernels.ascii_histogram([0.0, 1.0, 1.0, 2.0], bins=4)
    torch.manual_seed(0)
    cfg = ModelConfig(n_layers=1, layer=LayerConfig(embed_width=16, arch_type="unified", adaptive_conv=True, n_adaptive_branches=2, attn_window_size=64),
                      head=HeadConfig(head_type="classifier", n_classes=2))
    torch.save({"model_config": cfg.to_dict(), "state_dict": Model(cfg).state_dict()}, tmp_path / "m.pt")
    summary = inspect_kernels.main([str(tmp_path / "m.pt"), "--synthetic", "64", "--max-len", "64", "--batch-size", "16", "--device", "cpu"])
    assert len(summary) >= 2
    shares = [v["share"] for v in summary.values()]
    assert abs(sum(shares) - 1.0) < 1e-5 and all("sigma" in v for v in summary.values())
    assert "branch contribution" in capsys.readouterr().out


def test_vision_2d_trainer_augments_on_device_and_resumes(tmp_path):
    from ml_experiments_b200.cli import train_vision_2d as V

    g = torch.Generator().manual_seed(0)
    grey, colour = torch.rand(4, 1, 28, 28), torch.rand(4, 3, 32, 32)
    assert V.augment(grey, g).shape == grey.shape and V.augment(colour, g).shape == colour.shape
    # colour augmentation only moves pixels: every output value exists in the zero-padded input
    out = V.augment(colour, g)
    assert set(out[0, 0].flatten().tolist()) <= set(colour[0, 0].flatten().tolist()) | {0.0}
    x, y = V.synthetic_images(V.DATASET_CONFIGS["mnist"], 32, 0)
    assert x.shape == (32, 1, 28, 28) and x.dtype == torch.uint8 and int(y.max()) < 10
    assert V.to_gray(torch.full((1, 3, 2, 2), 100, dtype=torch.uint8)).unique().tolist() == [100]
    args = ["--dataset", "mnist", "--source", "synthetic", "--n-train", "64", "--n-val", "32", "--width", "8", "--n-layers", "1", "--batch-size", "32",
            "--adaptive", "--n-branches", "2", "--output", str(tmp_path / "m.pt"), "--device", "cpu"]
    s1 = V.main(args + ["--epochs", "1"])
    assert (tmp_path / "m.last.pt").exists() and 0.0 <= s1["best_acc"] <= 1.0
    ck = torch.load(tmp_path / "m.last.pt", weights_only=False)
    assert ck["epoch"] == 1 and ck["model_config"]["layer"]["adaptive_conv"] is True


def test_arch_search_grids_and_pareto(tmp_path):
    from ml_experiments_b200.cli import arch_search as A

    rows = [{"arch": "a", "params": 10, "f1": 0.5}, {"arch": "b", "params": 20, "f1": 0.4}, {"arch": "c", "params": 30, "f1": 0.9},
            {"arch": "d", "params": 30, "f1": 0.7}]
    assert [r["arch"] for r in A.pareto_front(rows, "f1")] == ["a", "c"]
    assert len(A.line_filter_space(True)) == 8 and len({c.name() for c in A.line_filter_space(False)}) == len(A.line_filter_space(False))
    assert all(c.width % c.groups == 0 for c in A.bytemasker_space(False))
    summary, res = A.main(["--task", "line-filter", "--quick", "--max-candidates", "2", "--synthetic", "96", "--epochs", "1", "--max-len", "64",
                           "--no-swa", "--device", "cpu", "--output", str(tmp_path / "lf.csv")])
    assert summary["candidates"] == 2 and res[0]["params"] != res[1]["params"]        # the axes change the model
    assert (tmp_path / "lf.csv").read_text().startswith("arch,arch_type,embed_width")
    summary, res = A.main(["--task", "bytemasker", "--quick", "--max-candidates", "2", "--synthetic", "96", "--epochs", "1", "--max-len", "64",
                           "--device", "cpu"])
    assert summary["task"] == "bytemasker" and all(0.0 <= r["recall"] <= 1.0 and r["samples_per_sec"] > 0 for r in res)


def test_memory_diagnostics_run_every_strategy_on_the_host():
    from ml_experiments_b200.cli import diagnose_memory as D

    rows = D.main(["--what", "gather", "--lengths", "32", "--batch", "2", "--channels", "16", "--heads", "2", "--samples", "3", "--device", "cpu"])
    assert set(rows[0]) >= {"materialise", "per_tap", "fused"}
    cases, x = D.gather_cases(2, 32, 16, 2, 3, torch.device("cpu"), torch.float32)
    a, b = cases["materialise"](), cases["per_tap"]()
    assert torch.allclose(a, b, atol=1e-5)                  # both strategies compute the same nearest-tap gather
    rows = D.main(["--what", "telephone", "--lengths", "64", "--batch", "1", "--channels", "16", "--heads", "2", "--device", "cpu"])
    assert set(rows[0]) == {"L", "fused_or_whole", "chunked_checkpoint"}
