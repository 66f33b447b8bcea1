"""``heuristic_secrets.data.collectors.gitleaks`` of the reference: the collector lives in :mod:`.tools` with the other scanner-repository readers."""
# ruff: noqa: F401
from .tools import GitleaksCollector
