"""Mine hard negatives for the Validator from a trained ByteMasker's false positives (role of the reference's
``scripts/mine_hard_negatives.py``): run the masker over windows without any secret byte, cut every run of bytes it
marks above its threshold, keep runs of a sane length that decode as UTF-8 and write them as label-0 validator samples.

Runs of marked bytes are found for the whole batch at once from the edges of the thresholded mask (a shifted compare on
the device), not by a per-byte Python loop.

    python -m ml_experiments_b200.cli.mine_hard_negatives --masker-checkpoint models/bytemasker.pt --synthetic 2000 \
        --output data/hard_negatives.jsonl
"""
from __future__ import annotations

import argparse
import json
from pathlib import Path

import torch

from ..heuristic_secrets.bytemasker.dataset import create_bucketed_batches
from ..heuristic_secrets.bytemasker.model import ByteMaskerConfig, ByteMaskerModel
from ..heuristic_secrets.data.types import ValidatorSample
from .train_bytemasker import jsonl_mask_windows, mask_windows


def mask_segments(mask: torch.Tensor, lengths: torch.Tensor) -> list[tuple[int, int, int]]:
    """``mask [B, L]`` bool, ``lengths [B]`` -> ``(row, start, end)`` of every maximal run of True inside each row's length."""
    B, L = mask.shape
    m = mask & (torch.arange(L, device=mask.device)[None, :] < lengths[:, None].to(mask.device))
    z = torch.zeros(B, 1, dtype=torch.bool, device=mask.device)
    edges = torch.cat([z, m, z], 1)
    rise = (edges[:, 1:] & ~edges[:, :-1]).nonzero()          # run starts at column c
    fall = (~edges[:, 1:] & edges[:, :-1]).nonzero()          # run ends before column c
    return [(int(r), int(s), int(e)) for (r, s), (_, e) in zip(rise.tolist(), fall.tolist())]


def load_masker(path, device):
    ck = torch.load(path, map_location=device, weights_only=False)
    model = ByteMaskerModel(ByteMaskerConfig.from_dict(ck["config"]))
    model.load_state_dict(ck.get("best_state") or ck["state_dict"])
    return model.to(device).eval(), float(ck.get("threshold", ck.get("optimal_threshold", 0.5)))


@torch.no_grad()
def mine(model, threshold, windows, batch_size, min_len, max_len, device):
    clean = [w for w in windows if not any(w.mask)]
    samples = []
    for i in range(0, len(clean), batch_size):
        part = clean[i:i + batch_size]
        lengths = torch.tensor([len(w.data) for w in part])
        ids = torch.zeros(len(part), int(lengths.max()), dtype=torch.long)
        for r, w in enumerate(part):
            ids[r, : len(w.data)] = torch.frombuffer(bytearray(w.data), dtype=torch.uint8).long()
        probs = torch.sigmoid(model(ids.to(device)))
        for r, s, e in mask_segments(probs >= threshold, lengths):
            if not (min_len <= e - s <= max_len):
                continue
            try:
                text = part[r].data[s:e].decode("utf-8")
            except UnicodeDecodeError:
                continue
            samples.append(ValidatorSample(text=text, label=0, source="bytemasker_fp", category="hard_negative"))
    return samples, len(clean)


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--masker-checkpoint", required=True)
    ap.add_argument("--data-dir", default=None)
    ap.add_argument("--split", default="train", choices=["train", "val"])
    ap.add_argument("--synthetic", type=int, default=0)
    ap.add_argument("--output", required=True)
    ap.add_argument("--min-segment-len", type=int, default=4)
    ap.add_argument("--max-segment-len", type=int, default=512)
    ap.add_argument("--max-len", type=int, default=512)
    ap.add_argument("--batch-size", type=int, default=64)
    ap.add_argument("--threshold", type=float, default=None, help="override the checkpoint's threshold")
    ap.add_argument("--seed", type=int, default=7)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    a = ap.parse_args(argv)
    device = torch.device(a.device)
    model, thr = load_masker(a.masker_checkpoint, device)
    if a.threshold is not None:
        thr = a.threshold
    if a.data_dir and not a.synthetic:
        windows = jsonl_mask_windows(Path(a.data_dir) / "splits" / "documents" / f"{a.split}.jsonl", a.max_len, a.seed)
    else:
        windows = mask_windows(a.synthetic or 2000, a.max_len, a.seed)
    samples, n_clean = mine(model, thr, windows, a.batch_size, a.min_segment_len, a.max_segment_len, device)
    out = Path(a.output)
    out.parent.mkdir(parents=True, exist_ok=True)
    out.write_text("".join(s.to_json() + "\n" for s in samples))
    lens = [len(s.text) for s in samples]
    summary = {"clean_windows": n_clean, "hard_negatives": len(samples), "threshold": thr,
               "len_min": min(lens) if lens else 0, "len_max": max(lens) if lens else 0, "len_mean": sum(lens) / len(lens) if lens else 0.0}
    print(json.dumps(summary))
    return summary


if __name__ == "__main__":
    main()
