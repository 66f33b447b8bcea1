"""The published sweeps of the recall harness: every sweep builds, its run ids are unique, and one model of every
architecture family that occurs in it can be constructed from its config and run forward on CPU."""
import pytest
import torch

from ml_experiments_b200.zoology.experiments import paper_configs as P


@pytest.mark.parametrize("name", sorted(P.SWEEPS))
def test_sweep_builds_with_unique_run_ids(name):
    configs = P.build(name, scale=1e-4)
    assert len(configs) > 0
    ids = [c.run_id + "|" + str(c.model.sequence_mixer) for c in configs]
    assert len(set(ids)) == len(ids)
    assert all(c.data.train_configs and c.data.test_configs for c in configs)
    assert len({c.sweep_id for c in configs}) == 1


def test_reference_grid_sizes():
    """Counts that follow from the grids of the reference's scripts: 3 lengths x 4 widths x 4 rates x 7 mixers; the Taylor
    exploration has 2 widths x 4 rates x 3 feature sizes x 2 head counts at one length."""
    assert len(P.iclr24_zoology_figure2(scale=1e-4)) == 3 * 4 * 4 * 7
    assert len(P.iclr24_explore_taylor(scale=1e-4)) == 2 * 4 * 3 * 2
    fig2 = P.arxiv24_based_figure2(scale=1e-4)
    per_family = {}
    for c in fig2:
        per_family[c.model.name] = per_family.get(c.model.name, 0) + 1
    assert per_family == {"attention": 2 * 4, "based": 9 * 4, "sliding-window-attention": 8 * 4, "mamba": 9 * 4, "mamba2": 9 * 4, "hyena": 3 * 4,
                          "h3": 3 * 4}


def test_one_model_per_family_runs_forward():
    from ml_experiments_b200.zoology.model import LanguageModel

    torch.manual_seed(0)
    seen = set()
    todo = P.arxiv24_based_appendix(scale=1e-4) + P.arxiv24_based_figure3(scale=1e-4) + P.iclr24_explore_dmodel(scale=1e-4, seq_kv=((64, 4),))
    for c in todo:
        fm = str(c.model.sequence_mixer.kwargs.get("configs", [{}])[-1].get("kwargs", {}).get("feature_name", ""))
        key = (c.model.name, fm)
        if key in seen or c.model.d_model > 128:
            continue
        seen.add(key)
        m = c.model.model_copy(update={"vocab_size": 64})
        # sequences of the smallest segment keep the test quick; every mixer takes l_max >= the length it sees
        model = LanguageModel(m).eval()
        x = torch.randint(0, 64, (2, 32))
        with torch.no_grad():
            y = model(x)
        assert y.shape == (2, 32, model.backbone.embeddings.word_embeddings.num_embeddings if hasattr(model, "backbone") else y.shape[-1])
        assert torch.isfinite(y).all(), key
    assert len(seen) >= 15


def test_module_level_configs_follow_the_environment(monkeypatch):
    monkeypatch.setenv("ZOOLOGY_PAPER_SWEEP", "iclr24_explore_configs/mqar_taylor_kv")
    monkeypatch.setenv("ZOOLOGY_PAPER_SCALE", "0.0001")
    assert len(P.configs) == 3 * 4 * 4


def test_state_tradeoff_table_marks_the_frontier(tmp_path):
    import pandas as pd

    from ml_experiments_b200.zoology.analysis.results import plot_state_tradeoff, state_tradeoff_table

    df = pd.DataFrame({"model": ["based"] * 4 + ["mamba"] * 3, "mixer": ["x"] * 7, "state_size": [100, 200, 400, 400, 64, 128, 256],
                       "best_acc": [0.5, 0.4, 0.9, 0.8, 0.3, 0.6, 0.6]})
    t = state_tradeoff_table(df)
    assert t["on_frontier"].tolist() == [True, False, True, True, True, False]      # a larger state has to buy accuracy
    assert t.loc[2, "best_acc"] == 0.9                                             # best run of the duplicated point
    out = tmp_path / "tradeoff.svg"
    assert plot_state_tradeoff(df, str(out)) and out.read_text().startswith("<svg")


def test_continuous_input_sweep_shapes():
    from ml_experiments_b200.zoology.experiments.mqar_examples import continuous_sweep

    cs = continuous_sweep(scale=1e-4)
    assert cs and all(c.input_type == "continuous" and c.model.n_layers == 1 and not c.model.learnable_word_embeddings for c in cs)
    assert {c.model.name for c in cs} == {"attention", "sliding-window-attention", "gated_delta_net", "ttt_linear", "ttt_mlp"}


def test_spiky_feature_maps():
    """Shapes, positivity and normalisation of the exponential feature maps; they resolve under the reference's path."""
    from ml_experiments_b200.zoology.mixers import feature_maps as F
    from ml_experiments_b200.zoology.utils import import_from_str

    torch.manual_seed(0)
    x = torch.randn(2, 3, 5, 8)
    assert import_from_str("zoology.mixers.feature_maps.exp_dim.SoftmaxDim") is F.SoftmaxDim
    for name, width in (("ExpDim", 16), ("ExpMaxNorm", 16), ("SoftmaxDim", 16), ("SoftmaxDimHalfspace", 8), ("ExpSumNorm", 16), ("ExpSumNormHalfspace", 8)):
        m = getattr(F, name)(input_dim=8, temp=0.7)
        y = m(x)
        assert y.shape == (2, 3, 5, width) == (2, 3, 5, m.expanded_size()) and (y > 0).all()
    assert torch.allclose(F.ExpDim(input_dim=8)(x), torch.cat([x, -x], -1).clamp(min=1e-12).exp())      # the doubling clamps first
    assert torch.allclose(F.ExpMaxNorm(input_dim=8, fullspace=False)(x).amax(-1), torch.ones(2, 3, 5))
    assert torch.allclose(F.SoftmaxDim(input_dim=8)(x).sum(-1), torch.full((2, 3, 5), 2.0), atol=1e-5)
    assert torch.allclose(F.ExpSumNorm(input_dim=8)(x).sum(-1), torch.ones(2, 3, 5), atol=1e-5)      # each |x| weight lands in one half
