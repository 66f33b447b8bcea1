"""Configuration objects (pydantic). ``BaseConfig.from_cli`` reads ``--config file.yaml`` and dotted ``--a.b=v``
overrides; ``ModuleConfig`` / ``FunctionConfig`` name a class or function by import string and instantiate it.
Same fields and defaults as zoology/config.py:12-142 of the reference."""
from __future__ import annotations

import argparse
from datetime import datetime
from functools import partial
from typing import List, Literal, Optional, Tuple, Union

from pydantic import BaseModel, ConfigDict

from .utils import import_from_str


class BaseConfig(BaseModel):
    model_config = ConfigDict(arbitrary_types_allowed=True, protected_namespaces=())

    @classmethod
    def from_cli(cls, argv: list[str] | None = None):
        import yaml
        parser = argparse.ArgumentParser(allow_abbrev=False)
        parser.add_argument("--config", type=str, default=None)
        parser.add_argument("--run_id", type=str, default=None)
        args, extra = parser.parse_known_args(argv)
        config: dict = {}
        if args.config is not None:
            with open(args.config) as f:
                config = yaml.safe_load(f) or {}
        for item in extra:
            key, value = item.lstrip("-").split("=", 1)
            node = config
            parts = key.replace("-", "_").split(".")
            for part in parts[:-1]:
                node = node.setdefault(part, {})
            node[parts[-1]] = yaml.safe_load(value)
        if args.run_id is not None:
            config["run_id"] = args.run_id
        obj = cls.model_validate(config)
        if getattr(obj, "run_id", "x") is None:
            obj.run_id = datetime.now().strftime("%Y-%m-%d-%H-%M-%S")
        return obj

    def print(self):
        try:
            import rich
            rich.print(self)
        except ImportError:
            print(self)


class _ByImportString(BaseConfig):
    """``name``: dotted import path of a class or function; ``kwargs``: keyword arguments bound at instantiation."""
    name: str
    kwargs: dict = {}

    def _target(self):
        return import_from_str(self.name)


class ModuleConfig(_ByImportString):
    def instantiate(self, **kwargs):
        return self._target()(**kwargs, **self.kwargs)


class FunctionConfig(_ByImportString):
    def instantiate(self):
        return partial(self._target(), **self.kwargs)


class DataSegmentConfig(BaseConfig):
    """Subclass per task (e.g. ``MQARConfig``) and implement ``build(seed) -> DataSegment``."""
    vocab_size: int = 8_192
    num_examples: int = 1_000
    input_seq_len: int = 64

    def build(self, **kwargs):
        raise NotImplementedError()


class DataConfig(BaseConfig):
    train_configs: List[DataSegmentConfig]
    test_configs: List[DataSegmentConfig]
    batch_size: Union[int, Tuple[int, int]] = 32  # (train, test) when a tuple
    seed: int = 123
    cache_dir: Optional[str] = None
    force_cache: bool = False
    num_passes: int = 1


class ModelConfig(BaseConfig):
    name: str = "default"
    # size
    d_model: int = 128
    n_layers: int = 2
    vocab_size: int = 8_192
    pad_vocab_size_multiple: int = 1
    max_position_embeddings: int = 64
    # blocks
    block_type: Literal["TransformerBlock", "MambaBlock", "Mamba2Block"] = "TransformerBlock"
    sequence_mixer: Optional[ModuleConfig] = None
    state_mixer: ModuleConfig = ModuleConfig(name="zoology.mixers.mlp.MLP", kwargs={"hidden_mult": 4})
    layer_norm_epsilon: float = 1e-5
    # embeddings and regularisation
    learnable_word_embeddings: bool = True
    embedding_init_type: Literal["default", "spherical", "normal"] = "default"
    embed_dropout: float = 0.1
    resid_dropout: float = 0.0
    drop_path: float = 0.0


class LoggerConfig(BaseConfig):
    project_name: Optional[str] = None
    entity: Optional[str] = None


class TrainConfig(BaseConfig):
    model: ModelConfig
    data: DataConfig
    logger: LoggerConfig = LoggerConfig()
    # identification of a run inside a sweep
    run_id: Optional[str] = "default"
    sweep_id: Optional[str] = None
    launch_id: Optional[str] = None
    seed: int = 123
    # optimisation
    learning_rate: float = 1e-3
    weight_decay: float = 0.1
    max_epochs: int = 100
    input_type: Literal["discrete", "continuous"] = "discrete"
    loss_type: Literal["ce", "mse", "ce_embed"] = "ce"
    # evaluation
    slice_keys: List[str] = []
    early_stopping_metric: Optional[str] = "valid/accuracy"  # None disables early stopping
    early_stopping_threshold: float = 0.99
