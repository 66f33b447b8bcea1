"""Model factories of the reference's comparison sweeps (zoology/experiments/models_repo.py:5-390): each ``add_*``
appends ``ModelConfig``s for one architecture family over its width / state-size grid, optionally preceded by a short
convolution mixer (``conv_mixer``) inside a ``Hybrid`` sequence mixer."""
from __future__ import annotations

from ..config import ModelConfig, ModuleConfig


def _append(models, name, mixer, conv_mixer, d_model, num_layers, model_factory_kwargs, block_type="TransformerBlock"):
    mixers = [conv_mixer, mixer] if conv_mixer is not None else [mixer]
    seq = ModuleConfig(name="zoology.mixers.hybrid.Hybrid", kwargs={"configs": mixers})
    models.append(ModelConfig(block_type=block_type, d_model=d_model, n_layers=num_layers, sequence_mixer=seq, max_position_embeddings=0,
                              name=name, **model_factory_kwargs))


def add_attention(models, conv_mixer, input_seq_len, model_factory_kwargs, num_layers=2):
    for d_model in [32, 64, 128]:
        _append(models, "attention", dict(name="zoology.mixers.attention.MHA", kwargs={"dropout": 0.1, "num_heads": 2}), conv_mixer, d_model,
                num_layers, model_factory_kwargs)
    return models


def add_based(models, conv_mixer, input_seq_len, model_factory_kwargs, num_layers=2):
    for d_model in [48, 64, 128]:
        for ftr_dim in [8, 16, 24]:
            mixer = dict(name="zoology.mixers.based.Based", kwargs={"l_max": input_seq_len, "feature_dim": ftr_dim, "feature_name": "taylor_exp",
                                                                      "num_key_value_heads": 1, "num_heads": 1, "train_view": "quadratic"})
            _append(models, "based", mixer, conv_mixer, d_model, num_layers, model_factory_kwargs)
    return models


def add_sliding_window(models, conv_mixer, input_seq_len, model_factory_kwargs, num_layers=2):
    for d_model in [128]:
        for width in [8, 16, 32, 64, 128, 256, 512, 1024]:
            mixer = dict(name="zoology.mixers.slide_attn.SlidingAttn", kwargs={"block_size": width, "attention_dropout": 0.0})
            _append(models, "sliding-window-attention", mixer, conv_mixer, d_model, num_layers, model_factory_kwargs)
    return models


def _state_family(models, path, name, input_seq_len, model_factory_kwargs, num_layers, block_type):
    for d_model in [64, 128, 256]:
        for d_state in [8, 16, 24]:
            models.append(ModelConfig(block_type=block_type, d_model=d_model, n_layers=num_layers,
                                      sequence_mixer=dict(name=path, kwargs={"d_state": d_state}), max_position_embeddings=0, name=name,
                                      **model_factory_kwargs))
    return models


def add_mamba(models, conv_mixer, input_seq_len, model_factory_kwargs, num_layers=2):
    return _state_family(models, "zoology.mixers.mamba.Mamba", "mamba", input_seq_len, model_factory_kwargs, num_layers, "MambaBlock")


def add_mamba2(models, conv_mixer, input_seq_len, model_factory_kwargs, num_layers=2):
    return _state_family(models, "zoology.mixers.mamba2.Mamba2", "mamba2", input_seq_len, model_factory_kwargs, num_layers, "Mamba2Block")


def add_hyena(models, conv_mixer, input_seq_len, model_factory_kwargs, num_layers=2):
    for d_model in [64, 128, 256]:
        models.append(ModelConfig(block_type="TransformerBlock", d_model=d_model, n_layers=num_layers,
                                  sequence_mixer=dict(name="zoology.mixers.hyena.Hyena", kwargs={"l_max": input_seq_len}),
                                  max_position_embeddings=0, name="hyena", **model_factory_kwargs))
    return models


def add_h3(models, conv_mixer, input_seq_len, model_factory_kwargs, num_layers=2):
    for d_model in [64, 128, 256]:
        models.append(ModelConfig(block_type="TransformerBlock", d_model=d_model, n_layers=num_layers,
                                  sequence_mixer=dict(name="zoology.mixers.h3.H3", kwargs={"l_max": input_seq_len, "d_state": d_model // 4, "head_dim": 2}),
                                  max_position_embeddings=0, name="h3", **model_factory_kwargs))
    return models


def _grid(models, name, path, kwargs, conv_mixer, model_factory_kwargs, num_layers, d_models=(64, 128, 256)):
    for d_model in d_models:
        _append(models, name, dict(name=path, kwargs=dict(kwargs)), conv_mixer, d_model, num_layers, model_factory_kwargs)
    return models


def add_rwkv7(models, conv_mixer, input_seq_len, model_factory_kwargs, num_layers=2):
    kw = {"l_max": input_seq_len, "head_dim": 64, "decay_low_rank_dim": 16, "gate_low_rank_dim": 64, "a_low_rank_dim": 16, "v_low_rank_dim": 16}
    return _grid(models, "rwkv7", "zoology.mixers.rwkv7.RWKV7Attention", kw, conv_mixer, model_factory_kwargs, num_layers)


def add_delta_net(models, conv_mixer, input_seq_len, model_factory_kwargs, num_layers=2):
    kw = {"l_max": input_seq_len, "num_heads": 2, "use_beta": True, "use_gate": False, "use_short_conv": True, "conv_size": 4}
    return _grid(models, "delta_net", "zoology.mixers.delta_net.DeltaNet", kw, conv_mixer, model_factory_kwargs, num_layers)


def add_gated_delta_net(models, conv_mixer, input_seq_len, model_factory_kwargs, num_layers=2):
    kw = {"l_max": input_seq_len, "num_heads": 2, "use_gate": False, "use_short_conv": True, "conv_size": 4}
    return _grid(models, "gated_delta_net", "zoology.mixers.gated_delta_net.GatedDeltaNet", kw, conv_mixer, model_factory_kwargs, num_layers)


def add_gla(models, conv_mixer, input_seq_len, model_factory_kwargs, num_layers=2):
    return _grid(models, "gla", "zoology.mixers.gla.GatedLinearAttention", {"num_heads": 2, "use_short_conv": False}, conv_mixer,
                 model_factory_kwargs, num_layers)


def add_deepseek_nsa(models, conv_mixer, input_seq_len, model_factory_kwargs, num_layers=2):
    kw = {"num_heads": 2, "sliding_window_size": 16, "compress_block_size": 8, "selection_block_size": 8, "num_selected_blocks": 4}
    return _grid(models, "deepseek_nsa", "zoology.mixers.deepseek_nsa.SparseAttention", kw, conv_mixer, model_factory_kwargs, num_layers)


def add_ttt(models, conv_mixer, input_seq_len, model_factory_kwargs, num_layers=2):
    for d_model in [64, 128, 256]:
        for ttt_type in ["mlp", "linear"]:
            for mini_batch_size in [16, 32]:
                kw = {"num_heads": 2, "ttt_layer_type": ttt_type, "ttt_base_lr": 1.0, "mini_batch_size": mini_batch_size, "use_gate": False,
                      "share_qk": False, "pre_conv": False, "conv_kernel": 4}
                _append(models, f"ttt_{ttt_type}", dict(name="zoology.mixers.ttt.TTT", kwargs=kw), conv_mixer, d_model, num_layers, model_factory_kwargs)
    return models


ALL_FAMILIES = [add_attention, add_based, add_sliding_window, add_mamba, add_mamba2, add_hyena, add_h3, add_rwkv7, add_delta_net,
                add_gated_delta_net, add_gla, add_deepseek_nsa, add_ttt]
