"""Two-stage secret detector: SpanFinder proposes byte spans, Validator accepts or rejects them.

Behaviour of ``scan`` follows the reference (src/heuristic_secrets/pipeline/detector.py:16-143): utf-8 bytes are cut
into overlapping chunks, SpanFinder probabilities are assembled into spans, partial spans are dropped, every remaining
span gets the six heuristic features and is scored by the Validator. Differences by design: all chunks of a document
run through SpanFinder as one padded batch and all candidate spans through the Validator as one padded batch (the
reference runs batch size 1 in Python loops), the Validator receives the span bytes and lengths (the reference's
one-argument call no longer matches its own model), and duplicate spans from overlapping chunks are merged.
"""
from __future__ import annotations

from dataclasses import dataclass
from pathlib import Path
from typing import Optional

import torch

from ..spanfinder.model import SpanFinderModel
from ..validator.features import FrequencyTable, extract_features
from ..validator.model import ValidatorModel
from .assembler import Span, SpanAssembler
from .chunker import Chunker


@dataclass
class Detection:
    start: int
    end: int
    text: str
    probability: float


@dataclass
class DetectorConfig:
    chunk_size: int = 512
    chunk_overlap: int = 64
    spanfinder_threshold: float = 0.5
    validator_threshold: float = 0.5
    min_span_length: int = 8
    max_span_length: int = 256


class Detector:
    def __init__(self, spanfinder: SpanFinderModel, validator: ValidatorModel, config: DetectorConfig,
                 text_freq: FrequencyTable, innocuous_freq: FrequencyTable, secret_freq: FrequencyTable,
                 device: str | torch.device = "cpu"):
        self.device = torch.device(device)
        self.spanfinder = spanfinder.to(self.device).eval()
        self.validator = validator.to(self.device).eval()
        self.config = config
        self.text_freq, self.innocuous_freq, self.secret_freq = text_freq, innocuous_freq, secret_freq
        self.chunker = Chunker(config.chunk_size, config.chunk_overlap)
        self.assembler = SpanAssembler(config.spanfinder_threshold, config.min_span_length, config.max_span_length)

    @torch.no_grad()
    def _find_spans(self, data: bytes) -> list[Span]:
        chunks = list(self.chunker.chunk(data))
        if not chunks:
            return []
        L = max(len(c.data) for c in chunks)
        ids = torch.zeros(len(chunks), L, dtype=torch.long)
        for i, c in enumerate(chunks):
            ids[i, : len(c.data)] = torch.frombuffer(bytearray(c.data), dtype=torch.uint8).long()
        probs = torch.sigmoid(self.spanfinder(ids.to(self.device))).cpu()
        spans, seen = [], set()
        for i, c in enumerate(chunks):
            for s in self.assembler.extract_spans(probs[i, : len(c.data)], chunk_start=c.start,
                                                  is_first_chunk=c.is_first, is_last_chunk=c.is_last):
                key = (s.start, s.end)
                if key not in seen:
                    seen.add(key)
                    spans.append(s)
        return spans

    @torch.no_grad()
    def _validate_spans(self, pieces: list[bytes]) -> list[float]:
        if not pieces:
            return []
        feats = torch.tensor([extract_features(p, self.text_freq, self.innocuous_freq, self.secret_freq).to_list()
                              for p in pieces], dtype=torch.float32)
        nf = self.validator.config.num_features
        feats = feats[:, :nf] if feats.shape[1] >= nf else torch.nn.functional.pad(feats, (0, nf - feats.shape[1]))
        lengths = torch.tensor([len(p) for p in pieces], dtype=torch.long)
        ids = torch.zeros(len(pieces), int(lengths.max()), dtype=torch.long)
        for i, p in enumerate(pieces):
            ids[i, : len(p)] = torch.frombuffer(bytearray(p), dtype=torch.uint8).long()
        logits = self.validator(feats.to(self.device), ids.to(self.device), lengths.to(self.device))
        return torch.sigmoid(logits.squeeze(-1)).cpu().tolist()

    def _validate_span(self, data: bytes) -> float:
        return self._validate_spans([data])[0]

    def scan(self, text: str) -> list[Detection]:
        if not text:
            return []
        data = text.encode("utf-8")
        spans = [s for s in self._find_spans(data) if not s.is_partial]
        probs = self._validate_spans([data[s.start:s.end] for s in spans])
        return [Detection(s.start, s.end, data[s.start:s.end].decode("utf-8", errors="replace"), p)
                for s, p in zip(spans, probs) if p >= self.config.validator_threshold]

    def scan_batch(self, texts: list[str]) -> list[list[Detection]]:
        return [self.scan(t) for t in texts]

    @classmethod
    def load(cls, path: str | Path, config: Optional[DetectorConfig] = None, device="cpu") -> "Detector":
        from ..io import load_model_bundle

        b = load_model_bundle(Path(path))
        return cls(b.spanfinder, b.validator, config or b.config, b.frequencies["text"], b.frequencies["innocuous"],
                   b.frequencies["secret"], device=device)
