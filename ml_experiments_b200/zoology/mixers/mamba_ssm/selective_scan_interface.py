"""Same names one level up, as in the reference's tree (zoology/mixers/mamba_ssm/selective_scan_interface.py)."""
# ruff: noqa: F401
from .ops.selective_scan_interface import MambaInnerFn, SelectiveScanFn, mamba_inner_fn, mamba_inner_ref, selective_scan_fn, selective_scan_ref
