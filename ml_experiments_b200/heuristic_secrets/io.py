"""Deployment bundle: a directory of ``config.json``, ``spanfinder.safetensors`` + ``.meta.json`` and
``validator.safetensors`` + ``.meta.json`` (model config plus the three byte-frequency tables).

File names, JSON keys and tensor names are those of the reference (src/heuristic_secrets/io.py:15-109), so bundles are
interchangeable. Files are written to a temporary name and renamed, so a crashed save never leaves a half bundle.
"""
from __future__ import annotations

import json
import os
from dataclasses import asdict, dataclass
from pathlib import Path

from safetensors.torch import load_file, save_file

from .pipeline.detector import DetectorConfig
from .spanfinder.model import SpanFinderConfig, SpanFinderModel
from .validator.features import FrequencyTable
from .validator.model import ValidatorConfig, ValidatorModel


@dataclass
class ModelBundle:
    spanfinder: SpanFinderModel
    validator: ValidatorModel
    config: DetectorConfig
    frequencies: dict[str, FrequencyTable]


def _write_json(path: Path, obj) -> None:
    tmp = path.with_suffix(path.suffix + ".tmp")
    tmp.write_text(json.dumps(obj, indent=2))
    os.replace(tmp, path)


def _write_tensors(path: Path, state: dict) -> None:
    tmp = path.with_suffix(path.suffix + ".tmp")
    save_file({k: v.detach().cpu().contiguous() for k, v in state.items()}, str(tmp))
    os.replace(tmp, path)


def save_model_bundle(path: Path, spanfinder: SpanFinderModel, validator: ValidatorModel,
                      detector_config: DetectorConfig, frequencies: dict[str, FrequencyTable],
                      version: str = "1.0.0") -> None:
    path = Path(path)
    path.mkdir(parents=True, exist_ok=True)
    _write_json(path / "config.json", {"version": version, **asdict(detector_config)})
    _write_tensors(path / "spanfinder.safetensors", spanfinder.state_dict())
    _write_json(path / "spanfinder.meta.json", spanfinder.config.to_dict())
    val_state = {k: v for k, v in validator.state_dict().items() if not k.startswith("attention.")}
    _write_tensors(path / "validator.safetensors", val_state)
    _write_json(path / "validator.meta.json",
                {**validator.config.to_dict(), "frequencies": {n: t.to_dict() for n, t in frequencies.items()}})


def load_model_bundle(path: Path) -> ModelBundle:
    path = Path(path)
    cfg = json.loads((path / "config.json").read_text())
    det = DetectorConfig(**{k: cfg[k] for k in ("chunk_size", "chunk_overlap", "spanfinder_threshold",
                                                 "validator_threshold", "min_span_length", "max_span_length")})
    spanfinder = SpanFinderModel(SpanFinderConfig.from_dict(json.loads((path / "spanfinder.meta.json").read_text())))
    spanfinder.load_state_dict(load_file(str(path / "spanfinder.safetensors")))
    vmeta = json.loads((path / "validator.meta.json").read_text())
    freqs = {n: FrequencyTable.from_dict(t) for n, t in vmeta.pop("frequencies").items()}
    validator = ValidatorModel(ValidatorConfig.from_dict(vmeta))
    validator.load_state_dict(load_file(str(path / "validator.safetensors")), strict=False)
    return ModelBundle(spanfinder, validator, det, freqs)
