"""Reference arm of bench.py.

The reference is installed with one offline ``pip install --no-index --no-build-isolation --find-links /opt/wheelhouse
--target baseline/_ref <reference>``. Its build backend (hatchling) is not in the offline wheelhouse, so that install
fails and nothing exists under ``baseline/_ref``; in addition the benchmarked GPT trainer of the reference is not part
of its installable package (it only exists as source embedded in a run log). The arm therefore reports itself as
unavailable and the published 8xH100 number stays the bar.
"""
import json
import os


def run(args, rank, local, world, seq_len, window_blocks, baseline_tokens_per_s, ClockSampler):
    here = os.path.dirname(os.path.abspath(__file__))
    ref = os.path.join(here, "_ref", "heuristic_secrets")
    why = ("offline pip install of the reference failed: build backend 'hatchling' is not in /opt/wheelhouse"
           if not os.path.isdir(ref) else
           "the reference's installable package does not contain the GPT trainer (modded-nanogpt is a script tree)")
    if rank == 0:
        print(json.dumps({"impl": "reference", "unavailable": why}), flush=True)
