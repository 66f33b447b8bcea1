"""Command-line entry points (``python -m ml_experiments_b200.cli.<name>``)."""
