"""Ready-made experiment definitions of the recall harness, as builder functions that return ``list[TrainConfig]``.

The reference keeps these as one script per sweep (zoology/experiments/basic_examples/basic.py, basic_sweep.py,
mqar_example_configs/{original_mqar,forgetting,composition}_configs.py, paper_configs/.../{parity,majority}.py):
every script repeats the same three steps (data segments of growing length, a model list from ``models_repo``, a
learning-rate grid). Here the steps are functions with the scripts' values as defaults, so a sweep is one call and a
reduced version of it (fewer lengths, fewer mixers, fewer examples) is the same call with arguments:

    python -m ml_experiments_b200.zoology.launch ml_experiments_b200/zoology/experiments/mqar_examples.py          # `configs` = basic()
    python -c "from ml_experiments_b200.zoology.experiments.mqar_examples import mqar_sweep; print(len(mqar_sweep()))"
"""
from __future__ import annotations

import uuid

import numpy as np

from ..config import DataConfig, LoggerConfig, ModelConfig, ModuleConfig, TrainConfig
from ..data.circuits import MajorityConfig, ParityConfig
from ..data.compositional_mqar import CompositionalMQARConfig
from ..data.forgetting_mqar import ForgettingMQARConfig
from ..data.multiquery_ar import MQARConfig
from . import models_repo

VOCAB_SIZE = 8_192
ALL_FAMILIES = ("attention", "sliding_window", "based", "mamba2", "delta_net", "rwkv7", "gla", "gated_delta_net", "deepseek_nsa", "ttt")
# (input_seq_len, num_examples, num_kv_pairs) of the multi-length MQAR mixture: short sequences dominate training, the test
# segments extend to four times the longest training length
MQAR_TRAIN = ((64, 100_000, 4), (128, 20_000, 8), (256, 20_000, 16), (256, 20_000, 32), (256, 20_000, 64))
MQAR_TEST = ((64, 1_000, 4), (64, 1_000, 8), (64, 1_000, 16), (128, 1_000, 32), (256, 1_000, 64), (512, 1_000, 128), (1024, 1_000, 256))
FORGET_TRAIN = ((64, 100_000, 4), (128, 20_000, 9), (256, 20_000, 16), (256, 20_000, 25), (256, 20_000, 36))
FORGET_TEST = ((64, 1_000, 4), (64, 1_000, 9), (128, 1_000, 16), (256, 1_000, 36), (512, 1_000, 64), (1024, 1_000, 144), (2048, 1_000, 256))


def basic(num_train: int = 10_000, num_test: int = 1_000) -> list[TrainConfig]:
    """One attention model on one MQAR segment: the smallest complete run."""
    seg = lambda n: MQARConfig(num_examples=n, vocab_size=256, input_seq_len=64, num_kv_pairs=4)
    model = ModelConfig(vocab_size=256, max_position_embeddings=64,
                        sequence_mixer=ModuleConfig(name="zoology.mixers.attention.MHA", kwargs={"dropout": 0.1, "num_heads": 1}))
    return [TrainConfig(data=DataConfig(train_configs=[seg(num_train)], test_configs=[seg(num_test)]), model=model)]


def basic_sweep(d_models=(64, 128), lrs=(1e-3, 3e-3), **kw) -> list[TrainConfig]:
    """The same task over a small width x learning-rate grid."""
    out = []
    for d in d_models:
        for lr in lrs:
            c = basic(**kw)[0]
            c.model.d_model, c.learning_rate, c.run_id = d, float(lr), f"mha-d{d}-lr{lr:.0e}"
            out.append(c)
    return out


def _segments(cls, table, vocab_size, scale: float = 1.0, **extra):
    return [cls(vocab_size=vocab_size, input_seq_len=L, num_examples=max(int(n * scale), 8), num_kv_pairs=kv, **extra) for L, n, kv in table]


def model_zoo(input_seq_len: int, vocab_size: int = VOCAB_SIZE, families=ALL_FAMILIES, num_layers: int = 2) -> list[ModelConfig]:
    """Every architecture family of ``models_repo`` over its own width / hyper-parameter grid, each mixer preceded by a
    short convolution (the harness' standard hybrid) and followed by an identity state mixer."""
    conv = dict(name="zoology.mixers.base_conv.BaseConv", kwargs={"l_max": input_seq_len, "kernel_size": 3, "implicit_long_conv": True})
    factory_kwargs = {"state_mixer": dict(name="torch.nn.Identity", kwargs={}), "vocab_size": vocab_size}
    models: list = []
    for fam in families:
        models = getattr(models_repo, f"add_{fam}")(models, conv, input_seq_len, factory_kwargs, num_layers=num_layers)
    return models


def _sweep(data: DataConfig, models, lrs, max_epochs, project, sweep_name, slice_keys=("num_kv_pairs",)) -> list[TrainConfig]:
    sweep_id = f"{sweep_name}-{uuid.uuid4().hex[:6]}"
    return [TrainConfig(model=m, data=data, learning_rate=float(lr), max_epochs=max_epochs, slice_keys=list(slice_keys), sweep_id=sweep_id,
                        run_id=f"{m.name}-lr{lr:.1e}", logger=LoggerConfig(project_name=project))
            for m in models for lr in lrs]


def mqar_sweep(families=ALL_FAMILIES, lrs=None, max_epochs: int = 32, batch_size: int = 256, scale: float = 1.0,
               train=MQAR_TRAIN, test=MQAR_TEST, vocab_size: int = VOCAB_SIZE, segment=MQARConfig, name: str = "mqar") -> list[TrainConfig]:
    """Multi-length associative recall: trains on a mixture of lengths / key-value counts, tests out to longer
    sequences; ``scale`` shrinks every segment's example count (``scale=0.01`` is a smoke run)."""
    lrs = np.logspace(-3, -1.5, 4) if lrs is None else lrs
    tr, te = _segments(segment, train, vocab_size, scale), _segments(segment, test, vocab_size, scale)
    L = max(c.input_seq_len for c in tr + te)
    data = DataConfig(train_configs=tr, test_configs=te, batch_size=(batch_size, max(batch_size // 8, 1)))
    return _sweep(data, model_zoo(L, vocab_size, families), lrs, max_epochs, "zoology-mqar", name)


def forgetting_sweep(**kw) -> list[TrainConfig]:
    """Recall with overwritten keys (the later binding of a key must win)."""
    kw.setdefault("train", FORGET_TRAIN)
    kw.setdefault("test", FORGET_TEST)
    return mqar_sweep(segment=ForgettingMQARConfig, name="forgetting", **kw)


def composition_sweep(**kw) -> list[TrainConfig]:
    """Two-hop recall (the value of one pair is the key of another)."""
    return mqar_sweep(segment=CompositionalMQARConfig, name="composition", **kw)


def continuous_sweep(kv_train=((4, 100_000), (8, 20_000), (16, 20_000), (32, 20_000), (64, 20_000)), kv_test=(4, 8, 16, 32, 64, 128, 256),
                     families=("attention", "sliding_window", "gated_delta_net", "ttt"), lrs=None, max_epochs: int = 32, batch_size: int = 256,
                     scale: float = 1.0, vocab_size: int = VOCAB_SIZE) -> list[TrainConfig]:
    """Recall on continuous inputs (zoology/experiments/011126/mqar_continuous.py): keys and values are fixed unit
    vectors instead of learned token embeddings (``input_type="continuous"``, spherical frozen embeddings), one-layer
    models without the short convolution, the sequence as long as its key-value pairs need."""
    from ..data.stacked_mqar import ContinuousMQARConfig

    lrs = np.logspace(-3, -1.5, 4) if lrs is None else lrs
    tr = [ContinuousMQARConfig(num_examples=max(int(n * scale), 8), num_kv_pairs=kv) for kv, n in kv_train]
    te = [ContinuousMQARConfig(num_examples=max(int(1_000 * scale), 8), num_kv_pairs=kv) for kv in kv_test]
    L = max((c.num_passes + 1) * c.num_kv_pairs for c in tr + te)
    factory_kwargs = {"state_mixer": dict(name="torch.nn.Identity", kwargs={}), "vocab_size": vocab_size}
    models: list = []
    for fam in families:
        models = getattr(models_repo, f"add_{fam}")(models, None, L, factory_kwargs, num_layers=1)
    for m in models:
        m.embedding_init_type, m.learnable_word_embeddings = "spherical", False
    data = DataConfig(train_configs=tr, test_configs=te, batch_size=(batch_size, max(batch_size // 8, 1)))
    out = _sweep(data, models, lrs, max_epochs, "zoology-continuous", "continuous-mqar")
    for c in out:
        c.input_type = "continuous"
    return out


def circuits_sweep(task: str = "parity", seq_lens=(8, 16, 32, 64), families=("attention", "based", "mamba2"), lrs=(1e-3, 3e-3),
                   num_train: int = 100_000, num_test: int = 1_000, max_epochs: int = 32) -> list[TrainConfig]:
    """Parity / majority over bit strings of several lengths (state-tracking probes)."""
    cls = {"parity": ParityConfig, "majority": MajorityConfig}[task]
    tr = [cls(vocab_size=3, input_seq_len=L, num_examples=num_train) for L in seq_lens]
    te = [cls(vocab_size=3, input_seq_len=L, num_examples=num_test) for L in seq_lens]
    data = DataConfig(train_configs=tr, test_configs=te, batch_size=(256, 32))
    return _sweep(data, model_zoo(max(seq_lens), 3, families), lrs, max_epochs, "zoology-circuits", task, slice_keys=("input_seq_len",))


configs = basic()
