"""One decode step of the selective recurrence (zoology/mixers/mamba_ssm/ops/triton/selective_state_update.py:121-240)."""
# ruff: noqa: F401
from ml_experiments_b200.ops.selective_scan import selective_state_update
from ml_experiments_b200.ops.selective_scan import selective_state_update as selective_state_update_ref
