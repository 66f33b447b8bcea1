"""Multi-GPU building blocks: symmetric memory, fused collectives, sharded optimizers, DDP wrapper."""
