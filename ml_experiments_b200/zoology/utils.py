"""Small helpers: import-by-string, seeding, flatten / unflatten of nested dictionaries (zoology/utils.py:8-36 and the
wandb table helpers of the reference)."""
from __future__ import annotations

import importlib
import random
from typing import Callable, Union

import numpy as np
import torch

# reference module paths keep working in configs written for the vendored package
_ALIASES = {"zoology.": "ml_experiments_b200.zoology."}
# modules of the reference's mixer zoo that live under another file name here
_MODULE_ALIASES = {
    "ml_experiments_b200.zoology.mixers.delta_net": "ml_experiments_b200.zoology.mixers.linear_attn",
    "ml_experiments_b200.zoology.mixers.gated_delta_net": "ml_experiments_b200.zoology.mixers.linear_attn",
    "ml_experiments_b200.zoology.mixers.gla": "ml_experiments_b200.zoology.mixers.linear_attn",
    "ml_experiments_b200.zoology.mixers.rwkv7": "ml_experiments_b200.zoology.mixers.linear_attn",
    "ml_experiments_b200.zoology.mixers.deepseek_nsa": "ml_experiments_b200.zoology.mixers.nsa",
    "ml_experiments_b200.zoology.mixers.slide_attn": "ml_experiments_b200.zoology.mixers.attention",
    "ml_experiments_b200.zoology.mixers.scatterbrain_new": "ml_experiments_b200.zoology.mixers.scatterbrain",
    "ml_experiments_b200.zoology.mixers.scatterbrain.attn": "ml_experiments_b200.zoology.mixers.scatterbrain",
    "ml_experiments_b200.zoology.mixers.nystromformer.nystromformer": "ml_experiments_b200.zoology.mixers.nystrom",
    "ml_experiments_b200.zoology.mixers.mra.mra": "ml_experiments_b200.zoology.mixers.mra",
    "ml_experiments_b200.zoology.mixers.h3.h3": "ml_experiments_b200.zoology.mixers.h3",
    "ml_experiments_b200.zoology.mixers.rwkv5": "ml_experiments_b200.zoology.mixers.rwkv",
    **{f"ml_experiments_b200.zoology.mixers.h3.{m}": "ml_experiments_b200.zoology.mixers.h3" for m in ("ss_kernel", "ss_kernel_diag", "ss_kernel_shift", "ssm_utils")},
    "ml_experiments_b200.zoology.mixers.scatterbrain.feature_maps_sb": "ml_experiments_b200.zoology.mixers.scatterbrain",
    "ml_experiments_b200.zoology.mixers.scatterbrain.projection_utils": "ml_experiments_b200.zoology.mixers.scatterbrain",
    "ml_experiments_b200.zoology.analysis.utils": "ml_experiments_b200.zoology.utils",
    # the reference's feature-map package is one module here
    **{f"ml_experiments_b200.zoology.mixers.feature_maps.{m}": "ml_experiments_b200.zoology.mixers.feature_maps"
       for m in ("base", "taylor", "performer", "cosformer", "all_poly", "exp_dim")},
}


def import_from_str(path: str) -> Union[type, Callable]:
    """``"pkg.module.Name"`` -> the object; paths starting with ``zoology.`` resolve inside this package."""
    for old, new in _ALIASES.items():
        if path.startswith(old):
            path = new + path[len(old):]
    module_name, obj_name = path.rsplit(".", 1)
    module_name = _MODULE_ALIASES.get(module_name, module_name)
    try:
        module = importlib.import_module(module_name)
    except ImportError as e:
        raise ImportError(f"Module '{module_name}' not found.") from e
    try:
        return getattr(module, obj_name)
    except AttributeError as e:
        raise AttributeError(f"Class '{obj_name}' not found in module '{module_name}'.") from e


def set_determinism(seed: int) -> None:
    random.seed(seed)
    np.random.seed(seed)
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed(seed)


def flatten(data, parent_key: str | None = None, sep: str = ".") -> dict:
    """``{"a": {"b": 1}, "f": [4, 5]}`` -> ``{"a.b": 1, "f.0": 4, "f.1": 5}``."""
    items = {}
    if isinstance(data, (list, tuple)):
        pairs = ((str(i), v) for i, v in enumerate(data))
    elif isinstance(data, dict):
        pairs = data.items()
    else:
        return {parent_key: data}
    for k, v in pairs:
        items.update(flatten(v, k if parent_key is None else f"{parent_key}{sep}{k}", sep))
    return items


def unflatten(d: dict, sep: str = ".") -> dict:
    """Inverse of ``flatten``; dictionaries whose keys are ``0..n-1`` become lists; NaN values are dropped."""
    root: dict = {}
    for key, value in d.items():
        if isinstance(value, float) and np.isnan(value):
            continue
        node = root
        parts = key.split(sep)
        for part in parts[:-1]:
            node = node.setdefault(part, {})
        node[parts[-1]] = value

    def listify(node):
        if not isinstance(node, dict):
            return node
        node = {k: listify(v) for k, v in node.items()}
        if node and all(k.isdigit() for k in node) and sorted(int(k) for k in node) == list(range(len(node))):
            return [node[str(i)] for i in range(len(node))]
        return node

    return listify(root)


def fetch_wandb_runs(project_name: str | None = None, filters: dict | None = None, csv_path: str | None = None, log_dir: str | None = None, **kwargs):
    """Runs of a sweep as a ``pandas.DataFrame``, one row per run. The reference downloads them from a wandb project
    (zoology/analysis/utils.py); training boxes here have no network, so the rows come from what the trainer writes
    locally (results CSV, JSON-lines logs: :func:`ml_experiments_b200.zoology.analysis.results.load_results`).
    ``filters``: column -> value (or list of values) to keep, e.g. ``{"sweep_id": "based-figure2-1a2b3c"}``."""
    import os

    from .analysis.results import load_results
    df = load_results(csv_path or os.environ.get("ZOOLOGY_CSV", "zoology_results.csv"), log_dir or os.environ.get("ZOOLOGY_LOG_DIR"))
    for col, want in (filters or {}).items():
        if col in df.columns:
            df = df[df[col].isin(want if isinstance(want, (list, tuple, set)) else [want])]
    return df.reset_index(drop=True)
