"""Synthetic-recall benchmark harness (the reference vendors HazyResearch "zoology" for this): pydantic configs,
token / continuous language models assembled from pluggable sequence and state mixers, a trainer with per-slice
accuracy, a sweep launcher that spreads configs over the GPUs of a node, synthetic tasks, and the mixer zoo."""
