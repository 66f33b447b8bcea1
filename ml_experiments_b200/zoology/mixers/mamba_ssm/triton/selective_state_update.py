# ruff: noqa: F401
from ..ops.triton.selective_state_update import selective_state_update, selective_state_update_ref
