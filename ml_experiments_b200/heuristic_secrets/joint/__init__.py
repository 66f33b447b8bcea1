from .model import JointConfig, JointSecretDetector  # noqa: F401
