"""Byte-level secret detection: SpanFinder -> Validator pipeline, ByteMasker, Joint detector, data tooling.

Public names match the reference package (src/heuristic_secrets/__init__.py:3-16).
"""
from .pipeline.detector import Detection, Detector, DetectorConfig
from .spanfinder.model import SpanFinderConfig
from .validator.model import ValidatorConfig

__version__ = "0.1.0"
__all__ = ["Detector", "Detection", "DetectorConfig", "SpanFinderConfig", "ValidatorConfig", "__version__"]
