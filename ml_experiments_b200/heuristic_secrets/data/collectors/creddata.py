"""``heuristic_secrets.data.collectors.creddata`` of the reference: the Samsung CredData collector and its label mapping."""
# ruff: noqa: F401
from .scrapers import CREDDATA_CATEGORY_MAP, CredDataCollector, map_creddata_category
