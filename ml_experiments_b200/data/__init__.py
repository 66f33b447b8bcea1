"""Data loading: token shard reader / document-aligned batch assembly for the GPT trainers."""
