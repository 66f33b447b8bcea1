"""Command-line tools: the scatter benchmark harness, the crossover sweep, the Ripple profiler and the SpanFinder trainer."""
import json

import torch


def test_bench_scatter_builds_every_model_at_a_matched_budget_and_trains():
    from ml_experiments_b200.cli import bench_scatter as B

    for kind in B.MODEL_TYPES:
        m = B.build_model(kind, layers=2, n_out=2, seq_len=64, num_channels=2, target_params=20_000, jacobi_iters=1)
        n = B.count_params(m)
        assert 5_000 < n < 80_000, (kind, n)
        assert m(torch.rand(2, 64)).shape == (2, 2)
    res = B.main(["--model", "conv,ripple", "--dataset", "mqar", "--seq-len", "32", "--epochs", "2", "--layers", "1", "--num-train", "32",
                  "--num-test", "16", "--batch-size", "16", "--target-params", "8000", "--device", "cpu", "--swa", "--swa-start", "0.5",
                  "--hard-mining", "--self-distill", "--distill-merge", "slerp", "--task-vocab-size", "32"])
    assert set(res) == {"conv", "ripple"} and all(0.0 <= r["mean"] <= 1.0 for r in res.values())


def test_schedule_and_weight_merges():
    from ml_experiments_b200.cli.bench_scatter import lerp_weights, lr_lambda, slerp_weights

    assert lr_lambda(0, 100, 10, 0.1) == 0.1 and lr_lambda(9, 100, 10, 0.1) == 1.0 and lr_lambda(15, 100, 10, 0.1) == 1.0
    assert lr_lambda(99, 100, 10, 0.1) < 0.01
    a, b = {"w": torch.tensor([1.0, 0.0])}, {"w": torch.tensor([0.0, 1.0])}
    assert torch.allclose(lerp_weights(a, b, 0.25)["w"], torch.tensor([0.75, 0.25]))
    s = slerp_weights(a, b, 0.5)["w"]
    assert torch.allclose(s, torch.full((2,), 0.5 ** 0.5), atol=1e-6)   # stays on the unit circle


def test_crossover_profile_and_spanfinder_tools(tmp_path, capsys):
    from ml_experiments_b200.cli import bench_crossover, profile_ripple, train_spanfinder

    rows = bench_crossover.main(["--lengths", "64", "--ops", "attention,conv,lowrank", "--width", "32", "--heads", "2", "--batch", "2", "--iters", "1",
                                 "--warmup", "0", "--device", "cpu"])
    assert [r["op"] for r in rows] == ["attention", "conv", "lowrank"] and all(r["fwd_ms"] > 0 for r in rows)
    out = profile_ripple.main(["--seq-len", "64", "--width", "32", "--layers", "1", "--heads", "2", "--batch", "2", "--iters", "1", "--device", "cpu"])
    assert {"telephone", "conv", "lowrank"} <= set(out["forward_by_operator"]) and out["forward_ms"] > 0
    meta = train_spanfinder.main(["--preset", "tiny", "--synthetic", "32", "--batch-size", "16", "--epochs", "1", "--output", str(tmp_path / "sf"),
                                  "--device", "cpu", "--chunk-size", "128"])
    assert (tmp_path / "sf.safetensors").exists() and json.loads((tmp_path / "sf.meta.json").read_text())["parameters"] == meta["parameters"]


def test_validator_trainer_tool(tmp_path):
    from ml_experiments_b200.cli import train_validator

    meta = train_validator.main(["--synthetic", "120", "--epochs", "2", "--output", str(tmp_path / "val"), "--device", "cpu"])
    saved = json.loads((tmp_path / "val.meta.json").read_text())
    assert (tmp_path / "val.safetensors").exists() and set(saved["frequencies"]) == {"text", "innocuous", "secret"}
    assert saved["config"]["num_features"] == 6 and meta["parameters"] > 0


def test_line_filter_trainer_checkpoints_and_resumes(tmp_path):
    from ml_experiments_b200.cli import train_line_filter as T

    common = ["--synthetic", "96", "--arch", "conv", "--embed-width", "16", "--output", str(tmp_path), "--device", "cpu", "--batch-size", "32"]
    T.main(common + ["--epochs", "2", "--neg-ratio", "1.0"])
    assert (tmp_path / "epoch002.pt").exists() and (tmp_path / "final.pt").exists()
    s = T.main(common + ["--epochs", "3", "--resume", str(tmp_path / "epoch002.pt")])
    assert (tmp_path / "epoch003.pt").exists() and s["parameters"] > 0
    assert abs(T.pos_weight_at(0, 10, 4.0, 1.0) - 4.0) < 1e-6 and abs(T.pos_weight_at(9, 10, 4.0, 1.0) - 1.0) < 1e-6
    m = T.main(common + ["--epochs", "1", "--head", "classifier", "--no-swa"])
    assert 0.0 <= float(m["best_metric"]) <= 1.0


def test_pathfinder_generator_and_pathx_trainers(tmp_path):
    import numpy as np

    from ml_experiments_b200.cli import generate_pathx, train_pathx
    from ml_experiments_b200.data import pathfinder

    x, y = pathfinder.generate(12, 64, seed=3)
    x2, y2 = pathfinder.generate(12, 64, seed=3)
    assert x.shape == (12, 64, 64) and x.dtype == np.uint8 and (x == x2).all() and (y == y2).all() and y.sum() == 6
    assert 0.005 < (x > 0).mean() < 0.5                       # sparse strokes on a dark canvas
    generate_pathx.main(["--output-dir", str(tmp_path / "gen"), "--n-train", "8", "--n-val", "4", "--n-test", "0", "--size", "32"])
    assert np.load(tmp_path / "gen" / "train.npz")["x"].shape == (8, 32, 32)
    flat = np.load(tmp_path / "gen" / "pathx_train_cache.npz")      # the per-split cache the reference's Path-X trainer reads
    assert flat["pixels"].shape == (8, 1024) and sorted(flat["pos_indices"].tolist() + flat["neg_indices"].tolist()) == list(range(8))
    assert (flat["labels"][flat["pos_indices"]] == 1).all()
    common = ["--size", "16", "--n-train", "32", "--n-val", "16", "--embed-width", "16", "--attn-window", "16", "--data-dir", str(tmp_path / "d"),
              "--device", "cpu", "--batch-size", "16"]
    s1 = train_pathx.main(common + ["--epochs", "2", "--mode", "1d", "--arch", "conv", "--output", str(tmp_path / "o1")])
    assert s1["tokens"] == 256 and (tmp_path / "o1" / "epoch002.pt").exists()
    train_pathx.main(common + ["--epochs", "2", "--mode", "2d", "--output", str(tmp_path / "o2")])
    s2 = train_pathx.main(common + ["--epochs", "2", "--mode", "2d", "--output", str(tmp_path / "o2"), "--resume", str(tmp_path / "o2" / "epoch001.pt")])
    assert len(s2["history"]) == 2 and s2["history"][0]["epoch"] == 1     # the second epoch was run again from the first one's checkpoint


def test_pipeline_evaluation_and_feature_subset_search(tmp_path):
    from ml_experiments_b200.cli import evaluate_pipeline, heuristic_search
    from ml_experiments_b200.heuristic_secrets.io import save_model_bundle
    from ml_experiments_b200.heuristic_secrets.pipeline.detector import DetectorConfig
    from ml_experiments_b200.heuristic_secrets.spanfinder.model import SpanFinderConfig, SpanFinderModel
    from ml_experiments_b200.heuristic_secrets.validator.features import FrequencyTable
    from ml_experiments_b200.heuristic_secrets.validator.model import ValidatorConfig, ValidatorModel

    assert evaluate_pipeline.match_spans([(0, 10), (50, 60)], [(1, 10), (100, 120)]) == (1, 1, 1)
    save_model_bundle(tmp_path / "b", SpanFinderModel(SpanFinderConfig.tiny()), ValidatorModel(ValidatorConfig()), DetectorConfig(),
                      {k: FrequencyTable({65: 1.0}) for k in ("text", "innocuous", "secret")})
    out = evaluate_pipeline.main(["--bundle", str(tmp_path / "b"), "--synthetic", "6"])
    assert out["documents"] == 6 and 0.0 <= out["f1"] <= 1.0 and out["bytes_per_second"] > 0
    assert len(list(heuristic_search.subsets(6))) == 63
    res = heuristic_search.main(["--synthetic", "60", "--epochs", "1", "--max-size", "1", "--device", "cpu"])
    assert len(res) == 6 and res[0]["f1"] >= res[-1]["f1"]


def test_checkpoint_ensemble_evaluation(tmp_path):
    from ml_experiments_b200.cli import eval_checkpoints, train_line_filter

    train_line_filter.main(["--synthetic", "96", "--arch", "conv", "--embed-width", "16", "--output", str(tmp_path), "--device", "cpu",
                            "--batch-size", "32", "--epochs", "2", "--no-swa"])
    rows, summary = eval_checkpoints.main(["--checkpoints", str(tmp_path / "epoch00*.pt"), "--synthetic", "48", "--device", "cpu"])
    assert len(rows) == 2 and summary["ensemble"]["members"] == 2
    assert summary["mean_disagreement"] == summary["mean_disagreement"] and 0.0 <= summary["ensemble"]["f1"] <= 1.0


def test_bytemasker_and_joint_trainer_tool(tmp_path):
    from ml_experiments_b200.cli import train_bytemasker

    s = train_bytemasker.main(["--synthetic", "64", "--epochs", "1", "--width", "16", "--depth", "2", "--output", str(tmp_path / "bm.pt"), "--device", "cpu"])
    assert s["kind"] == "bytemasker" and (tmp_path / "bm.pt").exists() and 0.0 <= s["clean_fp_rate"] <= 1.0
    j = train_bytemasker.main(["--joint", "--synthetic", "64", "--epochs", "1", "--width", "16", "--depth", "2", "--output", str(tmp_path / "j.pt"),
                               "--device", "cpu"])
    assert j["kind"] == "joint" and (tmp_path / "j.pt").exists()


def test_scatter_harness_selection_duo_and_ponder_modes():
    import torch

    from ml_experiments_b200.cli import bench_scatter as B

    per = torch.tensor([0.1, 2.0, 0.5, 1.0])
    assert B.selection_weights(per, None).tolist() == [1, 1, 1, 1]
    assert B.selection_weights(per, "top", 0.5).tolist() == [0, 1, 0, 1]
    assert B.selection_weights(per, "easy", 0.5).tolist() == [1, 0, 1, 0]
    assert B.selection_weights(per, "wtf").tolist() == [-1, 1, -1, 1]
    assert abs(B.hard_fraction(0, 5, 0.5, 0.1) - 0.5) < 1e-9 and abs(B.hard_fraction(4, 5, 0.5, 0.1) - 0.1) < 1e-9
    duo = B.DuoModel(torch.nn.Linear(4, 3), torch.nn.Linear(4, 3), "logsum")
    merged, a, b = duo.forward_both(torch.randn(2, 4))
    assert torch.allclose(merged, torch.log_softmax(a, -1) + torch.log_softmax(b, -1))
    common = ["--model", "ripple", "--dataset", "random-image", "--layers", "1", "--num-train", "32", "--num-test", "16", "--batch-size", "16",
              "--device", "cpu", "--target-params", "20000", "--seq-len", "64"]
    for extra in (["--epochs", "2", "--hard-start", "0.5", "--hard-end", "0.25"], ["--epochs", "1", "--duo"],
                  ["--epochs", "2", "--self-distill", "--distill-adaptive"], ["--epochs", "1", "--ponder"],
                  ["--epochs", "1", "--first-epoch-pct", "0.3", "--workers", "2", "--compile"]):
        r = B.main(common + extra)
        assert 0.0 <= r["ripple"]["mean"] <= 1.0


def test_scatter_harness_grid_models_ssm_stage_heads_and_ensemble_teacher():
    import torch

    from ml_experiments_b200.cli import bench_scatter as B
    from ml_experiments_b200.cli import scatter_grid as G

    # per-sample ensemble teacher: best-k correctly classified epochs, weights 1 / loss
    lg = [torch.tensor([[1.0, 0.0], [0.0, 1.0]]), torch.tensor([[3.0, 0.0], [0.0, 5.0]]), torch.tensor([[9.0, 0.0], [0.0, 7.0]])]
    ls = [torch.tensor([1.0, float("inf")]), torch.tensor([0.5, float("inf")]), torch.tensor([4.0, float("inf")])]
    t = B.ensemble_teacher_logits(lg, ls, top_k=2)
    assert torch.allclose(t[0], (torch.tensor([3.0, 0.0]) * 2 + torch.tensor([1.0, 0.0]) * 1) / 3) and t[1].abs().sum() == 0
    # the query-group head reads all tokens; the state-space stage keeps the block's shape on every grid rank
    head = G.QueryGroupHead(32, 250)
    assert head(torch.randn(2, 5, 7, 32)).shape == (2, 250) and head.groups == 100 and head.per_group == 3
    for nd, shape in ((1, (2, 16, 32)), (2, (2, 4, 4, 32)), (3, (2, 4, 4, 3, 32))):
        blk = G.WithSSM(torch.nn.Identity(), 32, 4, nd)
        assert blk(torch.randn(*shape)).shape == shape
    common = ["--dataset", "random-image", "--layers", "1", "--num-train", "32", "--num-test", "16", "--batch-size", "16", "--device", "cpu",
              "--target-params", "20000", "--epochs", "1", "--kernel-size", "3"]
    runs = [(["--model", "hier,conv", "--2d", "--seq-len", "64", "--merge-mode", "gate", "--conv-position", "pre", "--no-attn-residual", "--no-lowrank-hier"], ("hier", "conv")),
            (["--model", "attention,local", "--3d", "--seq-len", "48", "--ssm", "--ml-decoder"], ("attention", "local")),
            (["--model", "ripple", "--2d", "--seq-len", "64"], ("ripple",)),
            (["--model", "attention,hier", "--seq-len", "32", "--ssm", "--ml-decoder", "--merge-mode", "learned"], ("attention", "hier")),
            (["--model", "conv", "--seq-len", "32", "--epochs", "3", "--self-distill", "--distill-ensemble", "--distill-ensemble-k", "2"], ("conv",)),
            (["--model", "conv", "--seq-len", "32", "--epochs", "3", "--self-distill", "--distill-from-merged"], ("conv",))]
    for extra, kinds in runs:
        r = B.main(common + extra)
        assert set(r) == set(kinds) and all(0.0 <= v["mean"] <= 1.0 for v in r.values()), (extra, r)
