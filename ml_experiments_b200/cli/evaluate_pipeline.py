"""End-to-end evaluation of the secret Detector (SpanFinder -> span assembly -> Validator) on documents with labelled
spans: span-level precision / recall / F1 at an overlap threshold, per-stage recall, throughput (role of the reference's
``scripts/evaluate_pipeline.py``).

    python -m ml_experiments_b200.cli.evaluate_pipeline --bundle models/bundle --data data/splits/documents/test.jsonl
    python -m ml_experiments_b200.cli.evaluate_pipeline --bundle models/bundle --synthetic 200

``--synthetic N`` evaluates on N printable-ASCII documents with planted hex / base64 runs.
"""
from __future__ import annotations

import argparse
import json
import time
from pathlib import Path

from ..heuristic_secrets.data.planted import planted_span_batch
from ..heuristic_secrets.pipeline.detector import Detector


def _iou(a, b):
    inter = max(0, min(a[1], b[1]) - max(a[0], b[0]))
    return inter / max((a[1] - a[0]) + (b[1] - b[0]) - inter, 1)


def match_spans(pred, truth, min_iou: float = 0.5):
    """Greedy one-to-one matching by overlap -> ``(true positives, false positives, false negatives)``."""
    used, tp = set(), 0
    for p in pred:
        best, bi = 0.0, None
        for i, t in enumerate(truth):
            if i not in used and _iou(p, t) > best:
                best, bi = _iou(p, t), i
        if bi is not None and best >= min_iou:
            used.add(bi)
            tp += 1
    return tp, len(pred) - tp, len(truth) - tp


def load_documents(path: Path):
    docs = []
    for line in path.read_text().splitlines():
        if line.strip():
            d = json.loads(line)
            docs.append((d["text"], list(zip(d.get("starts", []), d.get("ends", [])))))
    return docs


def synthetic_documents(n: int, length: int = 512, seed: int = 0):
    ids, _, _, spans = planted_span_batch(n, length, seed=seed)
    return [(bytes(ids[i].tolist()).decode("ascii"), spans[i]) for i in range(n)]


def evaluate(detector: Detector, docs, min_iou: float = 0.5):
    tp = fp = fn = 0
    cand_tp = cand_total = nbytes = 0
    t0 = time.perf_counter()
    for text, truth in docs:
        data = text.encode("utf-8")
        nbytes += len(data)
        cands = [(s.start, s.end) for s in detector._find_spans(data)]
        c_tp, _, _ = match_spans(cands, truth, min_iou)
        cand_tp, cand_total = cand_tp + c_tp, cand_total + len(cands)
        det = [(d.start, d.end) for d in detector.scan(text)]
        a, b, c = match_spans(det, truth, min_iou)
        tp, fp, fn = tp + a, fp + b, fn + c
    dt = time.perf_counter() - t0
    n_truth = tp + fn
    prec, rec = tp / max(tp + fp, 1), tp / max(n_truth, 1)
    return {"documents": len(docs), "labelled_spans": n_truth, "precision": prec, "recall": rec, "f1": 2 * prec * rec / max(prec + rec, 1e-12),
            "spanfinder_recall": cand_tp / max(n_truth, 1), "candidates_per_document": cand_total / max(len(docs), 1),
            "bytes_per_second": nbytes / max(dt, 1e-9), "seconds": dt}


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--bundle", required=True, help="directory written by save_model_bundle")
    ap.add_argument("--data", default=None)
    ap.add_argument("--synthetic", type=int, default=0)
    ap.add_argument("--min-iou", type=float, default=0.5)
    ap.add_argument("--device", default="cpu")
    a = ap.parse_args(argv)
    detector = Detector.load(a.bundle, device=a.device)
    docs = load_documents(Path(a.data)) if a.data and not a.synthetic else synthetic_documents(a.synthetic or 100)
    out = evaluate(detector, docs, a.min_iou)
    print(json.dumps(out))
    return out


if __name__ == "__main__":
    main()
