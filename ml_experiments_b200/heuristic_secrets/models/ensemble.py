"""``heuristic_secrets.models.ensemble``: majority-vote ensemble (reference: src/heuristic_secrets/models/ensemble.py).
Re-exports."""
# ruff: noqa: F401
from ...models.unified.ensemble import Ensemble
