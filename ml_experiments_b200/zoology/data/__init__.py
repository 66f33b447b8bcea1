"""Synthetic tasks and the batch-returning dataset of the recall harness."""
