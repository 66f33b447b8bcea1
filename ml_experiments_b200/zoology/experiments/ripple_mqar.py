"""Ripple variants against attention (and Mamba) on multi-query associative recall, the grid of the reference's
``zoology/experiments/ripple_mqar.py:20-300``: sequence length / key-value pairs in {64/4, 256/16, 512/32, 1024/64,
4096/256}, d_model in {32..512}, three learning rates, two layers, vocabulary 8192, 64 epochs.

    python -m ml_experiments_b200.zoology.launch ml_experiments_b200/zoology/experiments/ripple_mqar.py [-p]

``build_configs(...)`` takes reduced grids for smoke runs.
"""
from __future__ import annotations

import uuid

import numpy as np

from ..config import DataConfig, LoggerConfig, ModelConfig, TrainConfig
from ..data.multiquery_ar import MQARConfig

VOCAB_SIZE = 8_192
SEQ_KV = [(64, 4), (256, 16), (512, 32), (1024, 64), (4096, 256)]
D_MODELS = [32, 64, 128, 256, 512]

_J = dict(diffuse_se=True)
# name -> (operator order, extra RippleMixer kwargs)
RIPPLE_VARIANTS = {
    "ripple-tcl": ("tele,conv,lowrank", {}),
    "ripple-tclj": ("tele,conv,lowrank,jacobi", {}),
    "ripple-aj": ("attn,jacobi", {}),
    "ripple-ca": ("conv,attn", {}),
    "ripple-ca-plain": ("conv,attn", dict(differential=False, embed_residual=False)),
    "ripple-ca-nodiff": ("conv,attn", dict(differential=False)),
    "ripple-ca-noembed": ("conv,attn", dict(embed_residual=False)),
    "ripple-a": ("attn", {}),
    "ripple-caj": ("conv,attn,jacobi", {}),
    "ripple-ja": ("jacobi,attn", {}),
    "ripple-cja": ("conv,jacobi,attn", {}),
    "ripple-ja-di": ("jacobi,attn", dict(_J, diff_inject=True)),
    "ripple-ja-dr": ("jacobi,attn", dict(_J, diff_readout=True)),
    "ripple-ja-dir": ("jacobi,attn", dict(_J, diff_inject=True, diff_readout=True)),
    "ripple-ja-dir-bcn": ("jacobi,attn", dict(_J, diff_inject=True, diff_readout=True, bc_norm=True)),
    "ripple-ja-se": ("jacobi,attn", dict(_J)),
    "ripple-ja-dir-bcn-r2": ("jacobi,attn", dict(_J, diff_inject=True, diff_readout=True, bc_norm=True, relu2=True)),
    "ripple-jl": ("jacobi,lowrank", {}),
    "ripple-cl": ("conv,lowrank", {}),
}
# the mixers the reference's sweep actually runs (it defines "mamba", "ripple-tclj" and "ripple-aj" without running them)
DEFAULT_MIXERS = ["attention", "ripple-tcl", "ripple-ca", "ripple-ca-plain", "ripple-ca-nodiff", "ripple-ca-noembed", "ripple-a",
                  "ripple-caj", "ripple-ja", "ripple-ja-di", "ripple-ja-dr", "ripple-ja-dir", "ripple-ja-dir-bcn", "ripple-ja-se",
                  "ripple-ja-dir-bcn-r2", "ripple-cja", "ripple-jl", "ripple-cl"]


def batch_size_for(seq_len: int) -> int:
    return 512 if seq_len <= 128 else 256 if seq_len <= 512 else 128 if seq_len <= 2048 else 64 if seq_len <= 4096 else 32


def heads_for(d_model: int) -> int:
    return 2 if d_model <= 32 else 4 if d_model <= 64 else 8 if d_model <= 256 else 16


def mixer_config(name: str, d_model: int, seq_len: int) -> dict:
    if name == "attention":
        return dict(name="zoology.mixers.attention.MHA", kwargs={"dropout": 0.1, "num_heads": 1})
    if name == "mamba":
        return dict(name="zoology.mixers.mamba.Mamba", kwargs={})
    order, extra = RIPPLE_VARIANTS[name]
    return dict(name="zoology.mixers.ripple.RippleMixer", kwargs=dict(num_heads=heads_for(d_model), order=order, max_seq_len=seq_len, **extra))


def build_configs(seq_kv=SEQ_KV, d_models=D_MODELS, lrs=None, mixers=DEFAULT_MIXERS, max_epochs: int = 64, num_train: int = 100_000,
                  num_test: int = 3_000, vocab_size: int = VOCAB_SIZE, sweep_id: str | None = None):
    lrs = np.logspace(-4, -2, 4)[1:] if lrs is None else lrs
    sweep_id = sweep_id or f"ripple_mqar_{uuid.uuid4().hex[:6]}"
    out = []
    for seq_len, kv in seq_kv:
        task = dict(num_kv_pairs=kv, train_power_a=0.01, test_power_a=0.01, random_non_queries=False)
        data = DataConfig(train_configs=[MQARConfig(num_examples=num_train, vocab_size=vocab_size, input_seq_len=seq_len, **task)],
                          test_configs=[MQARConfig(num_examples=num_test, vocab_size=vocab_size, input_seq_len=seq_len, **task)],
                          batch_size=batch_size_for(seq_len))
        for d_model in d_models:
            for lr in lrs:
                for name in mixers:
                    model = ModelConfig(d_model=d_model, n_layers=2, block_type="MambaBlock" if "mamba" in name else "TransformerBlock",
                                        max_position_embeddings=seq_len if name == "attention" else 0, vocab_size=vocab_size,
                                        sequence_mixer=mixer_config(name, d_model, seq_len), state_mixer=dict(name="torch.nn.Identity", kwargs={}))
                    out.append(TrainConfig(model=model, data=data, learning_rate=float(lr), max_epochs=max_epochs, sweep_id=sweep_id,
                                           run_id=f"{name}-seqlen{seq_len}-dmodel{d_model}-lr{lr:.6f}-kv{kv}",
                                           logger=LoggerConfig(project_name="ripple-zoology")))
    return out


configs = build_configs()
