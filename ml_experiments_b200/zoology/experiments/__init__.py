"""Sweep definitions: python files whose module-level ``configs`` list the launcher runs."""
