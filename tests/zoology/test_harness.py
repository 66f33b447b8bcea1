"""Synthetic-recall harness: configs, data, models, trainer, sweep launcher and the mixers' causality."""
import pytest
import torch

from ml_experiments_b200.zoology.config import DataConfig, ModelConfig, ModuleConfig, TrainConfig
from ml_experiments_b200.zoology.data.circuits import CumulativeMajorityConfig, ParityConfig, VocabMajorityConfig
from ml_experiments_b200.zoology.data.compositional_mqar import CompositionalMQARConfig
from ml_experiments_b200.zoology.data.forgetting_mqar import ForgettingMQARConfig
from ml_experiments_b200.zoology.data.multiquery_ar import MQARConfig
from ml_experiments_b200.zoology.data.stacked_mqar import ContinuousMQARConfig
from ml_experiments_b200.zoology.data.utils import DataSegment, prepare_data
from ml_experiments_b200.zoology.model import LanguageModel
from ml_experiments_b200.zoology.utils import flatten, import_from_str, unflatten

MIXERS = [
    ("zoology.mixers.attention.MHA", dict(num_heads=2)),
    ("zoology.mixers.attention.SlidingAttn", dict(block_size=4)),
    ("zoology.mixers.base_conv.BaseConv", dict(l_max=32, kernel_size=3)),
    ("zoology.mixers.base_conv.BaseConv", dict(l_max=32, kernel_size=-1)),
    ("zoology.mixers.based.Based", dict(feature_dim=4, num_heads=2, num_key_value_heads=2)),
    ("zoology.mixers.mamba.Mamba", dict(d_state=8)),
    ("zoology.mixers.mamba2.Mamba2", dict(d_state=8, headdim=8, chunk_size=8)),
    ("zoology.mixers.rwkv.RWKVTimeMixer", dict(l_max=32, n_layer=2)),
    ("zoology.mixers.rwkv.RWKV5TimeMixer", dict(l_max=32, n_layer=2, head_size=16)),
    ("zoology.mixers.mra.MRAAttention", dict(max_position_embeddings=32, num_heads=2, num_block_per_row=1)),
    ("zoology.mixers.linear_attn.GatedLinearAttention", dict(num_heads=2)),
    ("zoology.mixers.linear_attn.GatedLinearAttention", dict(num_heads=4, num_kv_heads=2, use_short_conv=True)),
    ("zoology.mixers.linear_attn.DeltaNet", dict(num_heads=2)),
    ("zoology.mixers.linear_attn.DeltaNet", dict(num_heads=2, use_gate=True, allow_neg_eigval=True, qk_activation="relu")),
    ("zoology.mixers.linear_attn.GatedDeltaNet", dict(num_heads=2)),
    ("zoology.mixers.linear_attn.RWKV7Attention", dict(head_dim=16)),
    ("zoology.mixers.hyena.Hyena", dict(l_max=32, filter_order=8, num_heads=2)),
    ("zoology.mixers.h3.H3", dict(l_max=32, d_state=8, head_dim=2)),
    ("zoology.mixers.scatterbrain.SBLocalAttention", dict(num_heads=2, window_size=4, feature_dim=8, dropout=0.0)),
    ("zoology.mixers.scatterbrain.ScatterBrain", dict(feature_dim=4, num_heads=4, num_key_value_heads=2)),
    ("zoology.mixers.selective.SigmoidLookups", dict(num_heads=2)),
    ("zoology.mixers.selective.SMA", dict(num_heads=2)),
    ("zoology.mixers.nsa.SparseAttention", dict(num_heads=2, sliding_window_size=4, compress_block_size=4, selection_block_size=4, num_selected_blocks=2)),
    ("zoology.mixers.nsa.SparseAttention", dict(num_heads=2, kv_heads=1, sliding_window_size=4, compress_block_size=4, selection_block_size=4, num_selected_blocks=2, query_heads_share_selected_kv=False)),
    ("zoology.mixers.bigbird.BigBIRDAttention", dict(block_size=2)),
    ("zoology.mixers.nystrom.NystromAttention", dict(num_heads=2, num_landmarks=64)),
    ("zoology.mixers.ttt.TTT", dict(num_heads=2)),
    ("zoology.mixers.ttt.TTT", dict(num_heads=2, ttt_layer_type="mlp", use_gate=True, mini_batch_size=8)),
    ("zoology.mixers.ttt.TTT", dict(num_heads=2, share_qk=True)),
    ("zoology.mixers.hybrid.Hybrid", dict(configs=[dict(name="zoology.mixers.attention.MHA", kwargs=dict(num_heads=1)),
                                                   dict(name="zoology.mixers.base_conv.BaseConv", kwargs=dict(l_max=32))])),
]


@pytest.mark.parametrize("name,kwargs", MIXERS)
def test_mixer_is_causal_and_differentiable(name, kwargs):
    torch.manual_seed(0)
    mixer = import_from_str(name)(d_model=32, layer_idx=1, **kwargs).train()
    x = torch.randn(2, 24, 32, requires_grad=True)
    y = mixer(x)
    assert y.shape == x.shape
    x2 = x.detach().clone()
    x2[:, 15:] += 1.0
    y2 = mixer(x2)
    assert torch.allclose(y[:, :15], y2[:, :15], atol=1e-4), "output before position 15 depends on later inputs"
    y.sum().backward()
    assert torch.isfinite(x.grad).all()
    assert mixer.state_size(sequence_length=24) >= 0


def test_tasks_are_well_formed(tmp_path):
    seg = MQARConfig(vocab_size=64, num_examples=50, input_seq_len=32, num_kv_pairs=4).build(seed=1)
    assert seg.inputs.shape == (50, 32) and seg.labels.shape == (50, 32)
    for x, y in zip(seg.inputs, seg.labels):  # every supervised position holds the value bound to the queried key
        ctx = dict(zip(x[0:8:2].tolist(), x[1:8:2].tolist()))
        pos = (y != -100).nonzero().flatten()
        assert len(pos) == 4 and all(ctx[int(x[p])] == int(y[p]) for p in pos)
    comp = CompositionalMQARConfig(vocab_size=150, num_examples=20, input_seq_len=30, num_kv_pairs=4).build(seed=2)
    for x, y in zip(comp.inputs, comp.labels):
        ctx = {(int(x[i]), int(x[i + 1])): int(x[i + 2]) for i in range(0, 12, 3)}
        for p in (y != -100).nonzero().flatten():
            assert ctx[(int(x[p - 1]), int(x[p]))] == int(y[p])
    forg = ForgettingMQARConfig(vocab_size=100, num_examples=20, input_seq_len=32, num_kv_pairs=4, num_updates=2).build(seed=3)
    for x, y in zip(forg.inputs, forg.labels):
        ctx = {}
        for i in range(0, 12, 2):
            ctx[int(x[i])] = int(x[i + 1])  # later bindings overwrite
        for p in (y != -100).nonzero().flatten():
            assert ctx[int(x[p])] == int(y[p])
    par = ParityConfig(num_examples=10, input_seq_len=9).build(seed=0)
    assert ((par.inputs[:, :-1].sum(1) % 2) == par.labels[:, -1]).all()
    cm = CumulativeMajorityConfig(num_examples=5, input_seq_len=8).build(seed=0)
    assert cm.labels.shape == (5, 8)
    vm = VocabMajorityConfig(vocab_size=6, num_examples=10, input_seq_len=12).build(seed=0)
    for x, y in zip(vm.inputs, vm.labels):
        counts = torch.bincount(x[:-1], minlength=6)
        assert counts[y[-1]] == counts.max() and (counts == counts.max()).sum() == 1
    emb = torch.randn(40, 8)
    cont = ContinuousMQARConfig(num_examples=6, num_kv_pairs=3, embeddings=emb).build(seed=0)
    assert cont.inputs.shape == (6, 6, 16) and cont.labels.shape == (6, 3)
    # cache round trip and seed separation
    cfg = DataConfig(train_configs=[MQARConfig(vocab_size=64, num_examples=20, input_seq_len=32, num_kv_pairs=4)],
                     test_configs=[MQARConfig(vocab_size=64, num_examples=10, input_seq_len=32, num_kv_pairs=4)], batch_size=(8, 4),
                     cache_dir=str(tmp_path))
    tr, te = prepare_data(cfg)
    assert len(tr) == 3 and len(te) == 3 and len(list(tmp_path.glob("data_*.pt"))) == 2
    tr2, _ = prepare_data(cfg)
    assert torch.equal(next(iter(tr))[0], next(iter(tr2))[0])


def test_config_cli_and_helpers(tmp_path):
    (tmp_path / "c.yaml").write_text("data:\n  train_configs: []\n  test_configs: []\nmodel:\n  d_model: 48\n")
    cfg = TrainConfig.from_cli(["--config", str(tmp_path / "c.yaml"), "--model.n_layers=3", "--learning-rate=0.01", "--run_id", "abc"])
    assert cfg.model.d_model == 48 and cfg.model.n_layers == 3 and cfg.learning_rate == 0.01 and cfg.run_id == "abc"
    nested = {"a": 1, "b": {"c": 2, "d": {"e": 3}}, "f": [4, 5]}
    assert flatten(nested) == {"a": 1, "b.c": 2, "b.d.e": 3, "f.0": 4, "f.1": 5} and unflatten(flatten(nested)) == nested
    assert import_from_str("zoology.mixers.mlp.MLP").__name__ == "MLP"


def _mqar_config(run_id, mixer, tmp_path, epochs=40):
    seg = dict(vocab_size=32, input_seq_len=16, num_kv_pairs=2)
    return TrainConfig(
        data=DataConfig(train_configs=[MQARConfig(num_examples=512, **seg)], test_configs=[MQARConfig(num_examples=64, **seg)], batch_size=64),
        model=ModelConfig(d_model=32, n_layers=2, max_position_embeddings=16, vocab_size=32, sequence_mixer=mixer),
        max_epochs=epochs, learning_rate=3e-3, slice_keys=["num_kv_pairs"], run_id=run_id)


def test_trainer_learns_small_mqar(tmp_path, monkeypatch):
    from ml_experiments_b200.zoology.train import train
    monkeypatch.setenv("ZOOLOGY_CSV", str(tmp_path / "r.csv"))
    monkeypatch.setenv("ZOOLOGY_LOG_DIR", str(tmp_path))
    best = train(_mqar_config("mha", ModuleConfig(name="zoology.mixers.attention.MHA", kwargs={"num_heads": 2}), tmp_path), device="cpu")
    # chance is 1/16 (values come from half of a 32-token vocabulary); full recall needs far more data than a unit test
    assert best["valid/accuracy"] > 0.4 and "valid/num_kv_pairs/accuracy-2" in best
    rows = (tmp_path / "r.csv").read_text().strip().splitlines()
    assert rows[0].startswith("run_id,mixer") and rows[1].startswith("mha,zoology.mixers.attention.MHA")
    assert (tmp_path / "mha.jsonl").exists()


def test_language_model_blocks_and_state_size():
    for block, mixer in (("TransformerBlock", ModuleConfig(name="zoology.mixers.based.Based", kwargs=dict(feature_dim=4, num_heads=2, num_key_value_heads=2))),
                         ("MambaBlock", ModuleConfig(name="zoology.mixers.mamba.Mamba", kwargs=dict(d_state=8))),
                         ("Mamba2Block", ModuleConfig(name="zoology.mixers.mamba2.Mamba2", kwargs=dict(d_state=8, headdim=8, chunk_size=8)))):
        m = LanguageModel(ModelConfig(d_model=32, n_layers=2, vocab_size=50, max_position_embeddings=0, sequence_mixer=mixer, block_type=block,
                                      pad_vocab_size_multiple=8))
        logits = m(torch.randint(0, 50, (2, 12)))
        assert logits.shape == (2, 12, 56) and m.state_size(12) > 0
        assert m.lm_head.weight is m.backbone.embeddings.word_embeddings.weight


def test_sweep_launcher_runs_every_config(tmp_path, monkeypatch):
    from ml_experiments_b200.zoology.launch import run_sweep
    monkeypatch.setenv("ZOOLOGY_CSV", str(tmp_path / "sweep.csv"))
    sweep = tmp_path / "sweep.py"
    sweep.write_text(
        "from ml_experiments_b200.zoology.config import *\nfrom ml_experiments_b200.zoology.data.multiquery_ar import MQARConfig\n"
        "seg = dict(vocab_size=32, input_seq_len=16, num_kv_pairs=2)\nconfigs = [TrainConfig(\n"
        "    data=DataConfig(train_configs=[MQARConfig(num_examples=64, **seg)], test_configs=[MQARConfig(num_examples=32, **seg)], batch_size=32),\n"
        "    model=ModelConfig(d_model=16, n_layers=1, max_position_embeddings=16, vocab_size=32,\n"
        "                      sequence_mixer=ModuleConfig(name=name, kwargs=kw)), max_epochs=1, run_id=rid)\n"
        "    for rid, name, kw in [('a', 'zoology.mixers.attention.MHA', {}), ('b', 'zoology.mixers.does_not_exist.X', {}),\n"
        "                          ('c', 'zoology.mixers.base_conv.BaseConv', {'l_max': 16})]]\n")
    out = run_sweep(str(sweep), name="t")
    assert [o[0] for o in out] == ["a", "b", "c"]
    assert out[0][2] is None and out[2][2] is None and "not found" in out[1][2]


def test_chunked_recurrences_match_step_by_step():
    from ml_experiments_b200.ops import linear_recurrence as R
    torch.manual_seed(0)
    B, T, H, dk, dv = 2, 150, 2, 16, 24
    q, k, v = torch.randn(B, T, H, dk), torch.randn(B, T, H, dk), torch.randn(B, T, H, dv)
    g = torch.nn.functional.logsigmoid(torch.randn(B, T, H, dk) * 3)
    o1, s1 = R.gla_recurrent(q, k, v, g)
    o2, s2 = R.chunk_gla(q, k, v, g)
    assert torch.allclose(o1, o2, atol=1e-4) and torch.allclose(s1, s2, atol=1e-4)
    kn, beta = torch.nn.functional.normalize(k, dim=-1), torch.rand(B, T, H)
    for gate in (None, torch.nn.functional.logsigmoid(torch.randn(B, T, H) + 2)):
        o1, s1 = R.delta_rule_recurrent(q, kn, v, beta, gate)
        o2, s2 = R.chunk_delta_rule(q, kn, v, beta, gate)
        assert torch.allclose(o1, o2, atol=1e-4) and torch.allclose(s1, s2, atol=1e-4)


def test_state_space_kernels_match_their_recurrences():
    from ml_experiments_b200.zoology.mixers.h3 import SSKernel
    torch.manual_seed(0)
    for mode, extra in (("diag", dict(disc="bilinear")), ("diag", dict(disc="zoh")), ("diag", dict(measure="diag")), ("shift", {})):
        k = SSKernel(4, N=8, L=20, mode=mode, **extra)
        K = k(L=20)[0][0]
        state, ys = k.default_state(1), []
        for t in range(20):
            y, state = k.step(torch.ones(1, 4) * (t == 0), state)
            ys.append(y[0, 0])
        assert torch.allclose(torch.stack(ys, -1), K, atol=1e-5)


def test_mixers_that_look_ahead_by_design():
    """The landmark Nystrom approximation and the eval-mode top-k of the selective look-ups see the whole sequence, as
    in the reference; they are checked for shape, gradients and their exact special cases only."""
    from ml_experiments_b200.zoology.mixers.nystrom import NystromAttention, iterative_pinv
    from ml_experiments_b200.zoology.mixers.selective import SelectiveLookups
    from ml_experiments_b200.zoology.mixers.scatterbrain import SBLocalAttention
    torch.manual_seed(0)
    x = torch.randn(2, 24, 32, requires_grad=True)
    for m in (NystromAttention(32, num_heads=2, num_landmarks=8), NystromAttention(32, num_heads=2, num_landmarks=8, split_heads=True, conv_kernel_size=3),
              SelectiveLookups(32, 2).eval(), SelectiveLookups(32, 2).train()):
        y = m(x)
        assert y.shape == x.shape
        y.sum().backward()
        assert torch.isfinite(x.grad).all()
    a = torch.softmax(torch.randn(3, 8, 8), dim=-1)
    assert torch.allclose(iterative_pinv(a, 20) @ a, torch.eye(8).expand(3, 8, 8), atol=1e-2)
    # a window covering the whole sequence makes the sparse + low-rank decomposition exact softmax attention
    m = SBLocalAttention(32, 2, window_size=64, feature_dim=8, dropout=0.0)
    q, k, v = m.Wqkv(x).view(2, 24, 3, 2, 16).permute(2, 0, 3, 1, 4)
    ref = torch.nn.functional.scaled_dot_product_attention(q, k, v, is_causal=True).transpose(1, 2).reshape(2, 24, 32)
    assert torch.allclose(m(x), m.out_proj(ref), atol=1e-5)


def test_mamba_decode_steps_match_the_parallel_forward():
    from ml_experiments_b200.zoology.mixers.mamba import Mamba
    torch.manual_seed(0)
    m = Mamba(32, d_state=8).eval()
    x = torch.randn(2, 12, 32)
    full = m(x)
    conv_state, ssm_state = m.allocate_inference_cache(2)
    outs = [m.step(x[:, t:t + 1], conv_state, ssm_state)[0] for t in range(12)]
    assert torch.allclose(torch.cat(outs, 1), full, atol=1e-5)


def test_experiment_definitions_build_and_instantiate():
    """The sweep files produce configs whose every mixer can be built and run (tiny widths, one per family)."""
    from ml_experiments_b200.zoology.experiments import models_repo, ripple_mqar
    cfgs = ripple_mqar.build_configs(seq_kv=[(64, 4)], d_models=[32], lrs=[1e-3], mixers=["attention", "mamba", *ripple_mqar.RIPPLE_VARIANTS],
                                     num_train=8, num_test=8, vocab_size=64)
    assert len(cfgs) == 2 + len(ripple_mqar.RIPPLE_VARIANTS)
    assert len(ripple_mqar.configs) == 5 * 5 * 3 * len(ripple_mqar.DEFAULT_MIXERS)
    x = torch.randint(0, 64, (2, 64))
    for c in cfgs[:4] + cfgs[-2:]:
        assert LanguageModel(c.model)(x).shape == (2, 64, 64)
    seen = set()
    for add in models_repo.ALL_FAMILIES:
        models = add([], dict(name="zoology.mixers.base_conv.BaseConv", kwargs={"l_max": 64, "kernel_size": 3}), 64, dict(vocab_size=64))
        assert models
        m = min(models, key=lambda mc: mc.d_model)
        if m.name in seen:
            continue
        seen.add(m.name)
        assert LanguageModel(m)(x).shape == (2, 64, 64), m.name


def test_analysis_tables_and_wall_clock(tmp_path):
    import json

    import pandas as pd

    from ml_experiments_b200.zoology.analysis import results as R
    from ml_experiments_b200.zoology.analysis import wall_clock as W

    rows = [dict(run_id=f"r{i}", mixer=m, d_model=d, seq_len=L, lr=lr, best_acc=acc)
            for i, (m, d, L, lr, acc) in enumerate([("a.b.MHA", 64, 128, 1e-3, 0.5), ("a.b.MHA", 64, 128, 1e-2, 0.9), ("a.b.MHA", 128, 128, 1e-3, 0.95),
                                                    ("x.Mamba", 64, 128, 1e-3, 0.7), ("x.Mamba", 64, 256, 1e-3, 0.4)])]
    pd.DataFrame(rows).to_csv(tmp_path / "res.csv", index=False)
    log = tmp_path / "logs"
    log.mkdir()
    with open(log / "z1.jsonl", "w") as f:
        f.write(json.dumps({"config": {"run_id": "z1", "learning_rate": 3e-3, "model": {"d_model": 256, "n_layers": 2, "sequence_mixer": {"name": "x.Mamba"}},
                                       "data": {"train_configs": [{"input_seq_len": 256}]}}}) + "\n")
        f.write(json.dumps({"num_parameters": 1234, "state_size": 99}) + "\n")
        f.write(json.dumps({"epoch": 0, "valid/accuracy": 0.3, "valid/loss": 2.0}) + "\n")
        f.write(json.dumps({"epoch": 1, "valid/accuracy": 0.8, "valid/loss": 1.0}) + "\n")
    df = R.load_results(str(tmp_path / "res.csv"), str(log))
    assert len(df) == 6 and df[df.run_id == "z1"].iloc[0].best_acc == 0.8 and df[df.run_id == "z1"].iloc[0].n_params == 1234
    t = R.mqar_table(df)
    assert t.loc[(128, "MHA"), 64] == 0.9 and t.loc[(128, "MHA"), 128] == 0.95          # best learning rate per point
    assert t.loc[(256, "Mamba"), 256] == 0.8 and t.loc[(256, "Mamba"), 64] == 0.4
    assert len(R.best_by(df)) == 5
    assert R.load_results(str(tmp_path / "none.csv")).empty
    assert R.plot_mqar(df, str(tmp_path / "fig.svg"))                                     # the figure needs no plotting library
    svg = (tmp_path / "fig.svg").read_text()
    assert svg.startswith("<svg") and svg.count("<polyline") == 3 and "seq_len 256" in svg and "Mamba" in svg
    table = W.wall_clock_table(("mamba1", "mamba2", "attention", "gla", "long_conv"), (32,), batch=1, heads=2, head_dim=8, dstate=8, iters=1, warmup=0,
                               backward=True, device="cpu")
    assert table[0]["seq_len"] == 32 and all(table[0][k] > 0 for k in W.OPERATORS)


def test_example_sweeps_build_train_configs(tmp_path, monkeypatch):
    """The ready-made sweeps yield one config per (model, learning rate); a shrunken one trains through the harness."""
    from ml_experiments_b200.zoology.experiments import mqar_examples as E
    assert len(E.configs) == 1 and len(E.basic_sweep()) == 4
    sweep = E.mqar_sweep(families=("attention", "mamba2"), scale=1e-3)
    assert len({c.sweep_id for c in sweep}) == 1 and len(sweep) % 4 == 0
    assert [s.num_kv_pairs for s in sweep[0].data.train_configs] == [4, 8, 16, 32, 64]
    assert max(s.input_seq_len for s in sweep[0].data.test_configs) == 1024 and sweep[0].slice_keys == ["num_kv_pairs"]
    forget = E.forgetting_sweep(families=("attention",), scale=1e-3)
    assert isinstance(forget[0].data.train_configs[0], ForgettingMQARConfig) and forget[0].data.test_configs[-1].input_seq_len == 2048
    comp = E.composition_sweep(families=("based",), scale=1e-3)
    assert isinstance(comp[0].data.train_configs[0], CompositionalMQARConfig)
    circ = E.circuits_sweep("majority", seq_lens=(8, 16), families=("attention",), num_train=16, num_test=8)
    assert circ and circ[0].model.vocab_size == 3 and circ[0].slice_keys == ["input_seq_len"]
    # a tiny instance of the multi-length sweep steps through the trainer
    from ml_experiments_b200.zoology.train import train
    monkeypatch.chdir(tmp_path)
    tiny = E.mqar_sweep(families=("attention",), lrs=[1e-3], max_epochs=1, batch_size=8, vocab_size=64,
                        train=((16, 16, 2),), test=((16, 8, 2),))
    c = min(tiny, key=lambda t: t.model.d_model)
    c.data.cache_dir = str(tmp_path)
    train(c)
