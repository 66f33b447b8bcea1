"""Joint detector: ByteMasker and Validator stages trained as one model (public names of the reference's package,
src/heuristic_secrets/joint/__init__.py)."""
from .model import JointConfig, JointSecretDetector
from .train import JointTrainer, load_checkpoint

__all__ = ["JointConfig", "JointSecretDetector", "JointTrainer", "load_checkpoint"]
