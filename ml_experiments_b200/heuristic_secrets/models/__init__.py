"""``heuristic_secrets.models`` under the reference's module names (src/heuristic_secrets/models/__init__.py:1-54).

The implementations live in :mod:`ml_experiments_b200.models` (one rank-generic class per operator instead of a file
per dimensionality, CUDA kernels of this package instead of Triton programs). Code written against the reference
imports ``heuristic_secrets.models``, ``heuristic_secrets.models.backbone``, ``...scatter_attention``,
``...triton_scatter`` and so on; every such module exists here and re-exports the same public names.
"""
from ...models.unified import (AttentionBackbone, BinaryHead, ByteEmbedding, ConvBackbone, HeadConfig, LayerConfig, MaskHead, Model,
                               ModelConfig)
from ...models.unified.features import AttentionFeature, ConvFeature, FeatureCombiner, HeuristicFeature, PrecomputedFeature
from ...models.unified.train import (Batch, BinaryBatch, MaskBatch, Metrics, TrainConfig, Trainer, create_binary_batches,
                                     create_mask_batches, get_device, set_seed, setup_cuda)

__all__ = ["ByteEmbedding", "ConvBackbone", "AttentionBackbone", "ConvFeature", "AttentionFeature", "HeuristicFeature", "PrecomputedFeature",
           "BinaryHead", "MaskHead", "FeatureCombiner", "Model", "ModelConfig", "LayerConfig", "HeadConfig", "Trainer", "TrainConfig", "Metrics",
           "MaskBatch", "BinaryBatch", "Batch", "create_mask_batches", "create_binary_batches", "get_device", "set_seed", "setup_cuda"]
