"""The published sweeps of the recall harness as builder functions that return ``list[TrainConfig]``.

The reference keeps one script per figure or ablation (zoology/experiments/paper_configs/: ``iclr24_zoology_figure2``,
``iclr24_explore_configs/{mqar_dmodel,mqar_taylor,mqar_taylor_kv}``, ``arxiv24_based_figure2``, ``_figure3``,
``_appendix``, ``_rebuttal_circuits`` and the dated files of ``arxiv24_based_ablations``). All of them are one of two
shapes, so here each shape is one function and every script is a call with that script's grids as defaults:

* **single-length recall** (:func:`single_length_sweep`): one MQAR segment per (sequence length, key-value count),
  batch size chosen by length, every mixer at every width and learning rate;
* **mixed-length recall** (:func:`mixed_length_sweep`): the multi-length training mixture with test segments out to
  four times the longest training length, a list of ``ModelConfig`` s from the family builders below.

``SWEEPS`` maps the reference's folder / file names to the builders; ``python -m
ml_experiments_b200.zoology.launch ml_experiments_b200/zoology/experiments/paper_configs.py`` runs ``configs``, which is
the sweep named by ``$ZOOLOGY_PAPER_SWEEP`` (default ``iclr24_zoology_figure2``) scaled by ``$ZOOLOGY_PAPER_SCALE``
(fraction of the example counts; default 1).
"""
from __future__ import annotations

import os
import uuid
from typing import Callable, Iterable, Sequence

import numpy as np

from ..config import DataConfig, LoggerConfig, ModelConfig, TrainConfig
from ..data.circuits import CumulativeMajorityConfig, CumulativeParityConfig, MajorityConfig, ParityConfig
from ..data.multiquery_ar import MQARConfig
from .mqar_examples import MQAR_TEST, MQAR_TRAIN, VOCAB_SIZE

IDENTITY_STATE = dict(name="torch.nn.Identity", kwargs={})
# the older mixture of the dated ablation files: short sequences only up to 16 pairs, fewer long examples
EXTRAP_TRAIN = ((64, 100_000, 4), (64, 20_000, 8), (64, 20_000, 16), (128, 10_000, 32), (256, 5_000, 64))


def _short_conv(l_max: int) -> dict:
    return dict(name="zoology.mixers.base_conv.BaseConv", kwargs={"l_max": l_max, "kernel_size": 3, "implicit_long_conv": True})


def _hybrid(*mixers: dict) -> dict:
    return dict(name="zoology.mixers.hybrid.Hybrid", kwargs={"configs": list(mixers)})


def _based(l_max: int, feature_dim: int = 8, heads: int = 1, feature_name: str = "taylor_exp", **extra) -> dict:
    kw = {"l_max": l_max, "feature_dim": feature_dim, "feature_name": feature_name, "num_key_value_heads": heads, "num_heads": heads,
          "train_view": "quadratic"}
    kw.update(extra)
    return dict(name="zoology.mixers.based.Based", kwargs=kw)


# ------------------------------------------------------------------------------------------------ single-length recall
def single_mixers(l_max: int, based_feature_dim: int = 8, based_heads: int = 1) -> dict[str, dict]:
    """The sequence mixers of the single-length figures, keyed by the names the result tables use."""
    return {
        "attention": dict(name="zoology.mixers.attention.MHA", kwargs={"dropout": 0.1, "num_heads": 1}),
        "hyena": dict(name="zoology.mixers.hyena.Hyena", kwargs={"l_max": l_max}),
        "rwkv": dict(name="zoology.mixers.rwkv.RWKVTimeMixer", kwargs={"l_max": l_max}),
        "base_conv": dict(name="zoology.mixers.base_conv.BaseConv", kwargs={"l_max": l_max, "kernel_size": [3, -1, 3, -1]}),
        "base_conv_act": dict(name="zoology.mixers.base_conv.BaseConv", kwargs={"l_max": l_max, "kernel_size": [3, -1, 3, -1], "use_act": True}),
        "h3": dict(name="zoology.mixers.h3.H3", kwargs={"l_max": l_max, "d_state": l_max, "head_dim": 2}),   # d_state = l_max: Hyena-equivalent
        "based": _hybrid(_short_conv(l_max), _based(l_max, based_feature_dim, based_heads)),
        "mamba": dict(name="zoology.mixers.mamba.Mamba", kwargs={}),
    }


def _batch_for(seq_len: int, largest: int = 512) -> int:
    """Halve the batch for every doubling of the length beyond 128 (``largest`` at 128 and below), never under 64."""
    b = largest
    for limit in (256, 512, 1024):
        if seq_len >= limit:
            b //= 2
    return max(b, 64)


def single_length_sweep(seq_kv: Iterable[tuple[int, int]] = ((128, 8), (64, 4), (256, 16)), d_models: Sequence[int] = (64, 128, 256, 512),
                        lrs=None, mixers: Sequence[str] = ("attention", "hyena", "rwkv", "base_conv", "h3", "based", "mamba"),
                        n_layers: int = 2, max_epochs: int = 64, num_train: int = 100_000, num_test: int = 3_000, scale: float = 1.0,
                        largest_batch: int = 512, based_grid: Sequence[tuple[int, int]] = ((8, 1),), sweep: str = "figure2",
                        vocab_size: int = VOCAB_SIZE) -> list[TrainConfig]:
    """One run per (length, width, learning rate, mixer). ``based_grid``: (feature_dim, heads) pairs tried for the
    ``based`` entry (the Taylor-feature explorations sweep it; everything else ignores it)."""
    lrs = np.logspace(-4, -2, 4) if lrs is None else lrs
    sweep_id = f"{sweep}-{uuid.uuid4().hex[:6]}"
    out = []
    for seq_len, kv in seq_kv:
        seg = dict(vocab_size=vocab_size, input_seq_len=seq_len, num_kv_pairs=kv, power_a=0.01, random_non_queries=False)
        data = DataConfig(train_configs=[MQARConfig(num_examples=max(int(num_train * scale), 8), **seg)],
                          test_configs=[MQARConfig(num_examples=max(int(num_test * scale), 8), **seg)], batch_size=_batch_for(seq_len, largest_batch))
        for d_model in d_models:
            for lr in lrs:
                for name in mixers:
                    for ftr, heads in (based_grid if name == "based" else ((8, 1),)):
                        mixer = single_mixers(seq_len, ftr, heads)[name]
                        model = ModelConfig(d_model=d_model, n_layers=n_layers, vocab_size=vocab_size, sequence_mixer=mixer, state_mixer=IDENTITY_STATE,
                                            block_type="MambaBlock" if name == "mamba" else "TransformerBlock", name=name,
                                            max_position_embeddings=seq_len if name == "attention" else 0)
                        tag = f"-ftr{ftr}-heads{heads}" if name == "based" and len(tuple(based_grid)) > 1 else ""
                        out.append(TrainConfig(model=model, data=data, learning_rate=float(lr), max_epochs=max_epochs, sweep_id=sweep_id,
                                               run_id=f"{name}-seqlen{seq_len}-dmodel{d_model}-lr{lr:.1e}-kv{kv}{tag}",
                                               logger=LoggerConfig(project_name="zoology")))
    return out


def iclr24_zoology_figure2(**kw) -> list[TrainConfig]:
    return single_length_sweep(**kw)


def iclr24_explore_dmodel(**kw) -> list[TrainConfig]:
    """Wider models, longer sequences, the two larger learning rates, and the gated variant of the long convolution."""
    kw.setdefault("seq_kv", ((64, 4), (128, 8), (256, 16), (512, 64)))
    kw.setdefault("d_models", (128, 256, 512))
    kw.setdefault("lrs", np.logspace(-4, -2, 4)[2:])
    kw.setdefault("mixers", ("attention", "hyena", "rwkv", "base_conv", "base_conv_act", "h3", "based", "mamba"))
    return single_length_sweep(sweep="explore-dmodel", **kw)


def iclr24_explore_taylor(**kw) -> list[TrainConfig]:
    """Taylor-feature linear attention alone: feature dimension x head count at one length."""
    kw.setdefault("seq_kv", ((256, 16),))
    kw.setdefault("d_models", (64, 128))
    kw.setdefault("based_grid", tuple((f, h) for f in (8, 16, 32) for h in (1, 4)))
    return single_length_sweep(mixers=("based",), largest_batch=256, sweep="explore-taylor", **kw)


def iclr24_explore_taylor_kv(**kw) -> list[TrainConfig]:
    """The same mixer against the number of key-value pairs at fixed length."""
    kw.setdefault("seq_kv", ((256, 8), (256, 32), (256, 64)))
    kw.setdefault("based_grid", ((16, 4),))
    return single_length_sweep(mixers=("based",), largest_batch=256, sweep="explore-taylor-kv", **kw)


# ------------------------------------------------------------------------------------------------- mixed-length recall
Family = Callable[[int, dict], list[ModelConfig]]


def _model(name: str, mixer: dict, d_model: int, common: dict, block_type: str = "TransformerBlock", n_layers: int = 2) -> ModelConfig:
    return ModelConfig(block_type=block_type, d_model=d_model, n_layers=n_layers, sequence_mixer=mixer, max_position_embeddings=0, name=name, **common)


def fam_attention(d_models=(64, 128)) -> Family:
    mha = dict(name="zoology.mixers.attention.MHA", kwargs={"dropout": 0.1, "num_heads": 1})
    return lambda L, c: [_model("attention", _hybrid(_short_conv(L), mha), d, c) for d in d_models]


def fam_based(d_models=(48, 64, 128), feature_dims=(8, 16, 24), feature_names=("taylor_exp",), conv: bool = True) -> Family:
    def build(L, c):
        pre = (_short_conv(L),) if conv else ()
        return [_model("based" if fn == "taylor_exp" else f"based-{fn.rsplit('.', 1)[-1]}", _hybrid(*pre, _based(L, f, feature_name=fn)), d, c)
                for d in d_models for fn in feature_names for f in feature_dims]
    return build


def fam_based_feature_maps(d_models=(64, 128, 192, 256, 320, 384, 448, 512)) -> Family:
    """Taylor features at two sizes against full-width maps (positive ELU, identity, ReLU, square, cosFormer, Performer)
    and a learned polynomial map, all inside the same hybrid."""
    full = ("zoology.mixers.feature_maps.base.PosELU", "zoology.mixers.feature_maps.base.Identity", "zoology.mixers.feature_maps.base.ReLU",
            "zoology.mixers.feature_maps.base.Square", "zoology.mixers.feature_maps.cosformer.CosFormerFeatureMap",
            "zoology.mixers.feature_maps.performer.PerformerFeatureMap")

    def build(L, c):
        out = []
        for d in d_models:
            variants = [dict(feature_name="zoology.mixers.feature_maps.taylor.TaylorExp", feature_dim=f) for f in (16, 24)]
            variants += [dict(feature_name=n, feature_dim=d) for n in full]
            variants.append(dict(feature_name="all_poly", feature_dim=d, feature_kwargs={"output_dim": d, "learnable": True, "init": "kaiming"}))
            for v in variants:
                extra = {k: v[k] for k in v if k not in ("feature_name", "feature_dim")}
                out.append(_model("based", _hybrid(_short_conv(L), _based(L, v["feature_dim"], feature_name=v["feature_name"], **extra)), d, c))
        return out
    return build


def fam_sliding(d_models=(128,), widths=(8, 16, 32, 64, 128, 256, 512, 1024)) -> Family:
    return lambda L, c: [_model("sliding-window-attention", _hybrid(_short_conv(L), dict(name="zoology.mixers.slide_attn.SlidingAttn",
                                kwargs={"block_size": w, "attention_dropout": 0.0})), d, c) for d in d_models for w in widths]


def fam_state(kind: str = "mamba", d_models=(64, 128, 256), d_states=(8, 16, 24)) -> Family:
    path, block = {"mamba": ("zoology.mixers.mamba.Mamba", "MambaBlock"), "mamba2": ("zoology.mixers.mamba2.Mamba2", "Mamba2Block")}[kind]
    return lambda L, c: [_model(kind, dict(name=path, kwargs={"d_state": s}), d, c, block) for d in d_models for s in d_states]


def fam_hyena(d_models=(64, 128, 256)) -> Family:
    return lambda L, c: [_model("hyena", dict(name="zoology.mixers.hyena.Hyena", kwargs={"l_max": L}), d, c) for d in d_models]


def fam_h3(d_models=(64, 128, 256)) -> Family:
    return lambda L, c: [_model("h3", dict(name="zoology.mixers.h3.H3", kwargs={"l_max": L, "d_state": d // 4, "head_dim": 2}), d, c) for d in d_models]


def fam_scatterbrain(d_models=(64, 128, 256), windows=(4, 16, 64, 256, 1024), feature_dims=(32, 64, 128)) -> Family:
    def build(L, c):
        return [_model("scatter-brain", _hybrid(_short_conv(L), dict(name="zoology.mixers.scatterbrain.SBLocalAttention",
                       kwargs={"num_heads": 1, "window_size": w, "feature_dim": f})), d, c)
                for d in d_models for w in windows for f in feature_dims if f <= d]
    return build


def fam_bigbird(d_models=(64,), block_sizes=(4, 8, 16, 32, 64, 128)) -> Family:
    return lambda L, c: [_model("bigbird", _hybrid(_short_conv(L), dict(name="zoology.mixers.bigbird.BigBIRDAttention", kwargs={"block_size": b})), d, c)
                         for d in d_models for b in block_sizes]


def _segments(cls, table, vocab_size, scale, **extra):
    return [cls(vocab_size=vocab_size, input_seq_len=L, num_examples=max(int(n * scale), 8), num_kv_pairs=kv, **extra) for L, n, kv in table]


def mixed_length_sweep(families: Sequence[Family], lrs=None, max_epochs: int = 32, batch_size: int = 256, scale: float = 1.0, train=MQAR_TRAIN,
                       test=MQAR_TEST, vocab_size: int = VOCAB_SIZE, state_mixer: dict = IDENTITY_STATE, sweep: str = "based",
                       slice_keys=("num_kv_pairs",)) -> list[TrainConfig]:
    lrs = np.logspace(-3, -1.5, 4) if lrs is None else lrs
    tr, te = _segments(MQARConfig, train, vocab_size, scale), _segments(MQARConfig, test, vocab_size, scale)
    return _runs(DataConfig(train_configs=tr, test_configs=te, batch_size=(batch_size, max(batch_size // 8, 1))), families,
                 {"state_mixer": state_mixer, "vocab_size": vocab_size}, lrs, max_epochs, sweep, slice_keys)


def _runs(data: DataConfig, families, common, lrs, max_epochs, sweep, slice_keys) -> list[TrainConfig]:
    L = max(c.input_seq_len for c in data.train_configs + data.test_configs)
    models = [m for fam in families for m in fam(L, common)]
    sweep_id = f"{sweep}-{uuid.uuid4().hex[:6]}"
    return [TrainConfig(model=m, data=data, learning_rate=float(lr), max_epochs=max_epochs, slice_keys=list(slice_keys), sweep_id=sweep_id,
                        run_id=f"{m.name}-d{m.d_model}-lr{lr:.1e}", logger=LoggerConfig(project_name="zoology")) for m in models for lr in lrs]


def arxiv24_based_figure2(**kw) -> list[TrainConfig]:
    """Recall against state size: attention, Based, sliding window, Mamba, Mamba-2, Hyena, H3."""
    fams = (fam_attention(), fam_based(), fam_sliding(), fam_state("mamba"), fam_state("mamba2"), fam_hyena(), fam_h3())
    return mixed_length_sweep(kw.pop("families", fams), sweep="based-figure2", **kw)


def arxiv24_based_figure3(**kw) -> list[TrainConfig]:
    """Which feature map: the linear-attention block with each map over eight widths."""
    return mixed_length_sweep(kw.pop("families", (fam_based_feature_maps(),)), sweep="based-figure3", **kw)


def arxiv24_based_appendix(**kw) -> list[TrainConfig]:
    """Figure 2's families plus the sparse / low-rank attention approximations (ScatterBrain windows, BigBird blocks)."""
    fams = (fam_attention(), fam_based(), fam_sliding(), fam_state("mamba"), fam_hyena(), fam_h3(), fam_scatterbrain(), fam_bigbird())
    return mixed_length_sweep(kw.pop("families", fams), sweep="based-appendix", **kw)


_ABLATIONS: dict[str, Callable[[], tuple]] = {
    # name -> (families, overrides): the dated files of arxiv24_based_ablations
    "extrap": lambda: ((fam_based((64, 128, 256), (8, 16, 24, 32)), fam_attention((64, 128, 256)), fam_state("mamba"), fam_hyena(), fam_h3()),
                       dict(train=EXTRAP_TRAIN, max_epochs=64)),
    "feature_map": lambda: ((fam_based((64, 128, 256), (8, 16, 24), ("taylor_exp", "pos_elu", "relu", "square", "performer", "cosformer")),
                             fam_attention((64, 128, 256))), dict(train=EXTRAP_TRAIN, max_epochs=64)),
    "tradeoff": lambda: ((fam_based((32, 64, 128, 256), (4, 8, 16, 24, 32)), fam_attention((32, 64, 128, 256)), fam_sliding((64, 128)),
                          fam_state("mamba", (32, 64, 128, 256))), dict(train=EXTRAP_TRAIN, max_epochs=64)),
    "taylor_low": lambda: ((fam_based((64, 128, 256), (4, 8, 16)), fam_attention((64, 128, 256))), dict(train=EXTRAP_TRAIN, max_epochs=64)),
    "sliding": lambda: ((fam_sliding((64, 128, 256)), fam_based((64, 128), (8, 16)), fam_attention()), dict(max_epochs=64)),
    "harder_yet": lambda: ((fam_based((64, 128, 256), (8, 16, 24)), fam_attention(), fam_sliding(), fam_state("mamba")),
                           dict(train=MQAR_TRAIN + ((512, 20_000, 128),), test=MQAR_TEST + ((2048, 1_000, 512),), max_epochs=64)),
    "new_feature_maps": lambda: ((fam_based_feature_maps((64, 128, 256)), fam_attention()), dict(max_epochs=64)),
    "no_conv": lambda: ((fam_based((64, 128), (8, 16, 24), conv=False), fam_based((64, 128), (8, 16, 24), conv=True)), dict(max_epochs=64)),
}


def arxiv24_based_ablation(which: str = "tradeoff", **kw) -> list[TrainConfig]:
    """One of ``extrap`` (older training mixture), ``feature_map``, ``tradeoff`` (width x feature size against windows and
    state sizes), ``taylor_low`` (small Taylor features), ``sliding``, ``harder_yet`` (512-token training, 2048-token
    test), ``new_feature_maps``, ``no_conv`` (the block with and without its short convolution)."""
    fams, overrides = _ABLATIONS[which]()
    overrides.update(kw)
    return mixed_length_sweep(overrides.pop("families", fams), sweep=f"based-{which}", **overrides)


def arxiv24_based_rebuttal_circuits(task: str = "cumulative_parity", seq_lens=(16, 32, 64, 128), lrs=None, max_epochs: int = 128, scale: float = 1.0,
                                    included=("attention", "based", "mamba")) -> list[TrainConfig]:
    """State-tracking probes with a gated MLP after every mixer: running parity / majority of a bit string, or their
    whole-sequence forms (``parity``, ``majority``), at several lengths."""
    cls = {"cumulative_parity": CumulativeParityConfig, "cumulative_majority": CumulativeMajorityConfig, "parity": ParityConfig,
           "majority": MajorityConfig}[task]
    vocab = 3
    seg = lambda n: [cls(vocab_size=vocab, input_seq_len=k, num_examples=max(int(n * scale), 8)) for k in seq_lens]
    data = DataConfig(train_configs=seg(100_000), test_configs=seg(1_000), batch_size=(256, 32))
    fams = {"attention": fam_attention((128,)), "based": fam_based((64, 128, 256), (16,)), "mamba": fam_state("mamba", (512,), (16,))}
    common = {"state_mixer": dict(name="zoology.mixers.mlp.GLU", kwargs={"hidden_mult": 4}), "vocab_size": vocab}
    lrs = np.logspace(-3.5, -2, 4) if lrs is None else lrs
    return _runs(data, [fams[n] for n in included], common, lrs, max_epochs, f"circuits-{task}", ("input_seq_len",))


SWEEPS: dict[str, Callable[..., list[TrainConfig]]] = {
    "iclr24_zoology_figure2": iclr24_zoology_figure2,
    "iclr24_explore_configs/mqar_dmodel": iclr24_explore_dmodel,
    "iclr24_explore_configs/mqar_taylor": iclr24_explore_taylor,
    "iclr24_explore_configs/mqar_taylor_kv": iclr24_explore_taylor_kv,
    "arxiv24_based_figure2": arxiv24_based_figure2,
    "arxiv24_based_figure3": arxiv24_based_figure3,
    "arxiv24_based_appendix": arxiv24_based_appendix,
    "arxiv24_based_rebuttal_circuits": arxiv24_based_rebuttal_circuits,
    **{f"arxiv24_based_ablations/{k}": (lambda k=k, **kw: arxiv24_based_ablation(k, **kw)) for k in _ABLATIONS},
}


def build(name: str, **kw) -> list[TrainConfig]:
    if name not in SWEEPS:
        raise KeyError(f"unknown sweep {name!r}; have {sorted(SWEEPS)}")
    return SWEEPS[name](**kw)


def __getattr__(attr: str):
    # `configs` is built on first access (the launcher reads it; importing the builders must stay cheap)
    if attr == "configs":
        return build(os.environ.get("ZOOLOGY_PAPER_SWEEP", "iclr24_zoology_figure2"), scale=float(os.environ.get("ZOOLOGY_PAPER_SCALE", "1")))
    raise AttributeError(attr)
