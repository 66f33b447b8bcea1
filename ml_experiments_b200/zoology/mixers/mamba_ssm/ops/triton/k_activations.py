"""``swiglu(x, y) = silu(x) * y`` (zoology/mixers/mamba_ssm/ops/triton/k_activations.py)."""
import torch.nn.functional as F


def swiglu(x, y):
    return F.silu(x) * y
