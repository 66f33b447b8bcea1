"""Reference arm of bench.py: runs the unmodified reference classes installed under ``baseline/_ref``."""
import json


def run(args, rank, local, world, seq_len, window_blocks, baseline_tokens_per_s, ClockSampler):
    if rank == 0:
        print(json.dumps({"impl": "reference", "unavailable": "reference arm not wired up yet"}), flush=True)
