"""``heuristic_secrets.models.train``: generic trainer, batches, metrics (reference:
src/heuristic_secrets/models/train.py). Re-exports."""
# ruff: noqa: F401
from ...models.unified.train import (
    BinaryBatch, MaskBatch, Metrics, TrainConfig, Trainer, compute_length_bins, create_binary_batches, create_mask_batches, get_device,
    set_seed, setup_cuda
)
