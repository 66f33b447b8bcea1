"""Run logger: Weights & Biases when configured and importable (zoology/logger.py:9-56), always a JSON-lines file when
``ZOOLOGY_LOG_DIR`` is set, otherwise silent."""
from __future__ import annotations

import json
import os


class WandbLogger:
    def __init__(self, config):
        self.run = None
        self._file = None
        log_dir = os.environ.get("ZOOLOGY_LOG_DIR")
        if log_dir:
            os.makedirs(log_dir, exist_ok=True)
            self._file = open(os.path.join(log_dir, f"{config.run_id}.jsonl"), "a")
        lc = config.logger
        self.no_logger = lc.project_name is None or lc.entity is None
        if not self.no_logger:
            try:
                import wandb
                self.run = wandb.init(name=config.run_id, entity=lc.entity, project=lc.project_name)
            except ImportError:
                print("wandb is not installed, logging to file only")
                self.no_logger = True

    def log_config(self, config):
        if self._file:
            self._file.write(json.dumps({"config": config.model_dump()}, default=str) + "\n")
        if self.run is not None:
            self.run.config.update(config.model_dump(), allow_val_change=True)

    def log_model(self, model, config):
        seq = max(c.input_seq_len for c in config.data.test_configs)
        info = {"num_parameters": sum(p.numel() for p in model.parameters() if p.requires_grad),
                "state_size": model.state_size(sequence_length=seq)}
        self.log(info)

    def log(self, metrics: dict):
        if self._file:
            self._file.write(json.dumps(metrics, default=float) + "\n")
            self._file.flush()
        if self.run is not None:
            import wandb
            wandb.log(metrics)

    def finish(self):
        if self._file:
            self._file.close()
            self._file = None
        if self.run is not None:
            self.run.finish()
