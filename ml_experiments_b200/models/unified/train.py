"""Generic trainer for ``unified.Model`` (binary / multi-class / per-byte mask heads).

Capabilities follow src/heuristic_secrets/models/train.py: AdamW with a no-decay name filter (:180-214), OneCycleLR sized
for 1.5x the batch count (:216-231), SWA (:233-253), hard-batch curriculum (:259-271,391-402), the three losses plus
deformable-conv regularisers (:273-355), per-batch ms/token statistics with slow-batch detection and on-demand
``torch.profiler`` (:451-497,499-586), threshold search in numpy (:819-857), checkpoint dictionary (:862-896) and the
length-binned batch builders (:899-1035). Checkpoints are written atomically.
"""
from __future__ import annotations

import random
import time
from dataclasses import dataclass, fields
from pathlib import Path
from typing import Literal, NamedTuple, Sequence

import numpy as np
import torch
import torch.nn.functional as F
from torch.nn.utils.rnn import pad_sequence
from torch.optim.swa_utils import SWALR, AveragedModel, update_bn

from ...utils.checkpoint import load_checkpoint, save_checkpoint
from .composed import Model, ModelConfig

NO_DECAY_KEYWORDS = ("bias", "LayerNorm.weight", "norm.weight", "log_sigma", "A_log", ".D", "b_bias", "c_bias", "pool_query",
                     "pool_queries", "lambda_proj.bias", "dt_proj.bias")
LENGTH_BINS = (48, 80, 128, 288, 384, 512)


def get_device(device: str | None = None) -> torch.device:
    if device is not None:
        return torch.device(device)
    return torch.device("cuda" if torch.cuda.is_available() else "cpu")


def setup_cuda(allow_tf32: bool = False) -> None:
    if torch.cuda.is_available():
        torch.backends.cudnn.benchmark = True
        torch.backends.cuda.matmul.allow_tf32 = allow_tf32
        torch.backends.cudnn.allow_tf32 = allow_tf32


def set_seed(seed: int) -> None:
    random.seed(seed)
    np.random.seed(seed)
    torch.manual_seed(seed)
    if torch.cuda.is_available():
        torch.cuda.manual_seed_all(seed)


class MaskBatch(NamedTuple):
    bytes: torch.Tensor
    masks: torch.Tensor
    lengths: torch.Tensor


class BinaryBatch(NamedTuple):
    bytes: torch.Tensor
    labels: torch.Tensor
    lengths: torch.Tensor | None = None
    features: torch.Tensor | None = None
    secret_ids: list | None = None


Batch = MaskBatch | BinaryBatch


@dataclass
class TrainConfig:
    lr: float = 1e-3
    epochs: int = 20
    warmup_epochs: int = 2
    grad_clip: float = 1.0
    weight_decay: float = 0.01
    pos_weight: float = 1.0
    use_swa: bool = True
    swa_start_pct: float = 0.4
    swa_lr_mult: float = 0.05
    swa_anneal_epochs: int = 5
    hard_example_ratio: float = 0.3
    curriculum_start_epoch: int = 2
    curriculum_end_epoch: int | None = None
    threshold_search: bool = False
    threshold_search_steps: int = 50
    threshold_optimize_for: Literal["f1", "recall", "gmean_r_f1"] = "gmean_r_f1"
    threshold_min_precision: float = 0.5
    preload_to_device: bool = False
    offset_reg_weight: float = 0.01
    entropy_reg_weight: float = 0.001
    seed: int | None = None

    def to_dict(self) -> dict:
        return dict(self.__dict__)

    @classmethod
    def from_dict(cls, d: dict) -> "TrainConfig":
        known = {f.name for f in fields(cls)}
        return cls(**{k: v for k, v in d.items() if k in known})


@dataclass
class Metrics:
    loss: float
    precision: float
    recall: float
    f1: float
    accuracy: float = 0.0
    fp_rate: float = 0.0
    fn_rate: float = 0.0
    eval_time: float = 0.0
    eval_tokens_per_sec: float = 0.0

    def __str__(self) -> str:
        parts = [f"loss={self.loss:.4f}"]
        if self.accuracy > 0:
            parts.append(f"acc={self.accuracy:.4f}")
        if self.precision > 0 or self.recall > 0 or self.f1 > 0:
            parts += [f"P={self.precision:.4f}", f"R={self.recall:.4f}", f"F1={self.f1:.4f}"]
        if self.fp_rate > 0 or self.fn_rate > 0:
            parts += [f"FP%={self.fp_rate * 100:.1f}", f"FN%={self.fn_rate * 100:.1f}"]
        if self.eval_time > 0:
            parts.append(f"[{self.eval_time:.2f}s {self.eval_tokens_per_sec:.0f}tok/s]")
        return " ".join(parts)


def _prf(tp, fp, fn):
    p = tp / (tp + fp) if tp + fp else 0.0
    r = tp / (tp + fn) if tp + fn else 0.0
    return p, r, (2 * p * r / (p + r) if p + r else 0.0)


def find_optimal_threshold(probs: np.ndarray, targets: np.ndarray, steps: int = 50, optimize_for: str = "gmean_r_f1",
                           min_precision: float = 0.5) -> float:
    """Scan thresholds in [0.1, 0.9]; objective ``f1``, ``recall`` (subject to a precision floor) or sqrt(recall * f1)."""
    best, best_t = 0.0, 0.5
    pos = targets == 1
    for t in np.linspace(0.1, 0.9, steps):
        pred = probs >= t
        p, r, f1 = _prf(int((pred & pos).sum()), int((pred & ~pos).sum()), int((~pred & pos).sum()))
        if optimize_for == "recall":
            score = r if p >= min_precision else 0.0
        elif optimize_for == "gmean_r_f1":
            score = (r * f1) ** 0.5
        else:
            score = f1
        if score > best:
            best, best_t = score, float(t)
    return best_t


class Trainer:
    def __init__(self, model: Model, train_data: Sequence[Batch], val_data: Sequence[Batch] | None = None,
                 config: TrainConfig | None = None, device: torch.device | None = None):
        self.config = cfg = config or TrainConfig()
        if cfg.seed is not None:
            set_seed(cfg.seed)
        self.device = device or get_device()
        self.model = model.to(self.device)
        self.head_type, self.n_classes = model.config.head.head_type, model.config.head.n_classes
        self._data_on_device = cfg.preload_to_device
        move = self._move if self._data_on_device else (lambda b: b)
        self.train_data = [move(b) for b in train_data]
        self.val_data = [move(b) for b in val_data] if val_data else None
        decay, no_decay = self._get_param_groups(model)
        self.optimizer = torch.optim.AdamW([{"params": decay, "weight_decay": cfg.weight_decay},
                                            {"params": no_decay, "weight_decay": 0.0}], lr=cfg.lr)
        # one-cycle schedule sized for the curriculum's extra (re-added hard) batches
        self._max_batches = int(len(self.train_data) * 1.5)
        self._scheduler_total = cfg.epochs * self._max_batches
        self._scheduler_steps = 0
        self.scheduler = None
        if self._scheduler_total > 0:
            pct = min(cfg.warmup_epochs * self._max_batches / self._scheduler_total, 0.3)
            self.scheduler = torch.optim.lr_scheduler.OneCycleLR(self.optimizer, max_lr=cfg.lr, total_steps=self._scheduler_total,
                                                                 pct_start=pct, anneal_strategy="cos")
        self.swa_active, self.swa_model, self.swa_scheduler = False, None, None
        self.swa_start_epoch = cfg.epochs + 1
        if cfg.use_swa:
            self.swa_start_epoch = int(cfg.epochs * cfg.swa_start_pct)
            self.swa_model = AveragedModel(self.model)
            self.swa_scheduler = SWALR(self.optimizer, swa_lr=cfg.lr * cfg.swa_lr_mult, anneal_epochs=cfg.swa_anneal_epochs,
                                       anneal_strategy="cos")
        self.best_metric, self.best_state, self.optimal_threshold = 0.0, None, 0.5
        self._batch_losses = [0.0] * len(self.train_data)
        self._batch_times: list[tuple[int, float]] = []
        self._slow_batches: list[tuple[int, int, int, float, float, float]] = []
        self._ms_per_token_history: list[float] = []

    # ---- setup helpers -------------------------------------------------------------------------------------------
    @staticmethod
    def _get_param_groups(model) -> tuple[list, list]:
        decay, no_decay = [], []
        for name, p in model.named_parameters():
            if p.requires_grad:
                (no_decay if any(k in name for k in NO_DECAY_KEYWORDS) else decay).append(p)
        return decay, no_decay

    def set_train_data(self, train_data: Sequence[Batch]) -> None:
        self.train_data = train_data
        if len(train_data) != len(self._batch_losses):
            self._batch_losses = [0.0] * len(train_data)

    def _get_hard_ratio(self, epoch: int) -> float:
        cfg = self.config
        end = cfg.curriculum_end_epoch or cfg.epochs // 2
        if epoch < cfg.curriculum_start_epoch:
            return 0.0
        if epoch >= end:
            return cfg.hard_example_ratio
        return cfg.hard_example_ratio * (epoch - cfg.curriculum_start_epoch) / (end - cfg.curriculum_start_epoch)

    def _move(self, batch: Batch) -> Batch:
        to = lambda t: None if t is None else t.to(self.device, non_blocking=True)
        if isinstance(batch, MaskBatch):
            return MaskBatch(to(batch.bytes), to(batch.masks), to(batch.lengths))
        return BinaryBatch(to(batch.bytes), to(batch.labels), to(batch.lengths), to(batch.features), batch.secret_ids)

    def _to_device(self, batch: Batch) -> Batch:
        return batch if self._data_on_device else self._move(batch)

    # ---- forward / loss -------------------------------------------------------------------------------------------
    def _valid_positions(self, batch: Batch, L: int) -> torch.Tensor:
        return torch.arange(L, device=self.device).unsqueeze(0) < batch.lengths.unsqueeze(1)

    def _forward_batch(self, batch: Batch):
        if self.head_type == "mask":
            out = self.model(batch.bytes)
        else:
            pad = None if batch.lengths is None else ~self._valid_positions(batch, batch.bytes.shape[1])
            out = self.model(batch.bytes, mask=pad, precomputed=batch.features)
        return out if isinstance(out, tuple) else (out, {})

    def _compute_loss(self, logits, batch: Batch, aux: dict) -> torch.Tensor:
        pw = self.config.pos_weight
        if self.head_type == "mask":
            valid = self._valid_positions(batch, logits.shape[1])
            bce = F.binary_cross_entropy_with_logits(logits, batch.masks, reduction="none")
            if pw != 1.0:
                bce = bce * torch.where(batch.masks == 1, pw, 1.0)
            loss = (bce * valid).sum() / valid.sum()
        elif self.n_classes > 2:
            loss = F.cross_entropy(logits, batch.labels.long())
        else:
            logits = logits.squeeze(-1) if logits.dim() > 1 else logits
            weight = torch.where(batch.labels == 1, pw, 1.0) if pw != 1.0 else None
            loss = F.binary_cross_entropy_with_logits(logits, batch.labels, weight=weight)
        # the model prefixes aux names with the layer index; sum every layer's regulariser
        for key, w in (("offset_reg", self.config.offset_reg_weight), ("entropy_reg", self.config.entropy_reg_weight)):
            terms = [v for k, v in aux.items() if k == key or k.endswith("_" + key)]
            if terms and w:
                loss = loss + w * torch.stack(terms).mean()
        return loss

    @torch.no_grad()
    def _compute_confusion(self, logits, batch: Batch, threshold: float = 0.5):
        """(tp, fp, fn, tn, n) as device tensors -- no host synchronisation inside the training loop."""
        if self.head_type == "mask":
            valid = self._valid_positions(batch, logits.shape[1])
            pred, truth = (torch.sigmoid(logits) >= threshold)[valid], batch.masks[valid] == 1
        elif self.n_classes > 2:
            correct = (logits.argmax(-1) == batch.labels.long()).sum()
            n = torch.tensor(len(batch.labels), device=self.device)
            zero = torch.zeros((), dtype=torch.long, device=self.device)
            return torch.stack([correct, n - correct, zero, zero, n])
        else:
            pred, truth = torch.sigmoid(logits).view(-1) >= threshold, batch.labels == 1
        return torch.stack([(pred & truth).sum(), (pred & ~truth).sum(), (~pred & truth).sum(), (~pred & ~truth).sum(),
                            torch.tensor(pred.numel(), device=self.device)])

    def _build_metrics(self, total_loss, n_batches, tp, fp, fn, tn, n) -> Metrics:
        loss = total_loss / n_batches if n_batches else 0.0
        if self.n_classes > 2 and self.head_type != "mask":
            return Metrics(loss, 0.0, 0.0, 0.0, accuracy=tp / n if n else 0.0)
        p, r, f1 = _prf(tp, fp, fn)
        return Metrics(loss, p, r, f1, accuracy=(tp + tn) / n if n else 0.0, fp_rate=fp / (fp + tn) if fp + tn else 0.0,
                       fn_rate=fn / (fn + tp) if fn + tp else 0.0)

    # ---- training ---------------------------------------------------------------------------------------------------
    def _step(self, batch: Batch):
        self.optimizer.zero_grad(set_to_none=True)
        logits, aux = self._forward_batch(batch)
        loss = self._compute_loss(logits, batch, aux)
        loss.backward()
        return logits, loss

    def train_epoch(self, epoch: int = 0, profile_slow: bool = False) -> Metrics:
        self.model.train()
        cfg = self.config
        if cfg.use_swa and epoch >= self.swa_start_epoch:
            self.swa_active = True
        order = list(range(len(self.train_data)))
        if cfg.seed is not None:
            random.seed(cfg.seed + epoch)
        random.shuffle(order)
        n_hard = int(len(order) * self._get_hard_ratio(epoch)) if epoch > 0 else 0
        if n_hard > 0:
            order += sorted(range(len(self._batch_losses)), key=self._batch_losses.__getitem__, reverse=True)[:n_hard]
            random.shuffle(order)
        total_loss = torch.zeros((), device=self.device)
        confusion = torch.zeros(5, dtype=torch.long, device=self.device)
        losses = []
        self._batch_times, self._ms_per_token_history = [], []
        sync = torch.cuda.synchronize if self.device.type == "cuda" else (lambda: None)
        for loop_idx, idx in enumerate(order):
            t0 = time.perf_counter()
            batch = self._to_device(self.train_data[idx])
            logits, loss = self._step(batch)
            if cfg.grad_clip > 0:
                torch.nn.utils.clip_grad_norm_(self.model.parameters(), cfg.grad_clip)
            self.optimizer.step()
            if self.swa_active and self.swa_scheduler is not None:
                self.swa_scheduler.step()
            elif self.scheduler is not None and self._scheduler_steps < self._scheduler_total:
                self.scheduler.step()
                self._scheduler_steps += 1
            losses.append((idx, loss.detach()))
            total_loss += loss.detach()
            confusion += self._compute_confusion(logits.detach(), batch)
            sync()
            dt = time.perf_counter() - t0
            self._batch_times.append((idx, dt))
            tokens = int(batch.lengths.sum()) if batch.lengths is not None else batch.bytes.numel()
            mpt = dt * 1000 / max(tokens, 1)
            hist = self._ms_per_token_history
            hist.append(mpt)
            if len(hist) >= 50:
                mean = sum(hist) / len(hist)
                std = (sum((v - mean) ** 2 for v in hist) / len(hist)) ** 0.5
                if mpt > mean + std:
                    self._slow_batches.append((epoch, loop_idx, idx, mpt, mean, std))
                    if profile_slow:
                        self.profile_batch(idx, warmup=0, runs=1)
        if self.swa_active and self.swa_model is not None:
            self.swa_model.update_parameters(self.model)
        for idx, l in losses:  # one host transfer per epoch
            self._batch_losses[idx] = float(l)
        tp, fp, fn, tn, n = (int(v) for v in confusion.tolist())
        return self._build_metrics(float(total_loss), len(order), tp, fp, fn, tn, n)

    def profile_batch(self, batch_idx: int, warmup: int = 2, runs: int = 5, trace_path: str | None = None) -> dict:
        """Time one batch's forward+backward and collect a ``torch.profiler`` table (optionally a chrome trace)."""
        from torch.profiler import ProfilerActivity, profile
        batch = self._to_device(self.train_data[batch_idx])
        sync = torch.cuda.synchronize if self.device.type == "cuda" else (lambda: None)
        for _ in range(warmup):
            self._step(batch)
        sync()
        times = []
        for _ in range(runs):
            t0 = time.perf_counter()
            self._step(batch)
            sync()
            times.append(time.perf_counter() - t0)
        acts = [ProfilerActivity.CPU] + ([ProfilerActivity.CUDA] if self.device.type == "cuda" else [])
        with profile(activities=acts, record_shapes=True) as prof:
            self._step(batch)
            sync()
        if trace_path:
            prof.export_chrome_trace(trace_path)
        key = "cuda_time_total" if self.device.type == "cuda" else "cpu_time_total"
        return {"batch_idx": batch_idx, "batch_size": batch.bytes.shape[0], "seq_len": batch.bytes.shape[1], "times": times,
                "mean_time": sum(times) / len(times), "min_time": min(times), "max_time": max(times),
                "profile_table": prof.key_averages().table(sort_by=key, row_limit=20)}

    def get_batch_time_stats(self) -> dict:
        if not self._batch_times:
            return {}
        t = sorted(v for _, v in self._batch_times)
        n = len(t)
        out = {"count": n, "mean": sum(t) / n, "median": t[n // 2], "p95": t[int(n * 0.95)], "p99": t[int(n * 0.99)],
               "min": t[0], "max": t[-1], "slow_batches": len(self._slow_batches)}
        m = sorted(self._ms_per_token_history)
        if m:
            mean = sum(m) / len(m)
            out.update(ms_per_token_mean=mean, ms_per_token_std=(sum((v - mean) ** 2 for v in m) / len(m)) ** 0.5,
                       ms_per_token_median=m[len(m) // 2], ms_per_token_p95=m[int(len(m) * 0.95)])
        return out

    def finalize_swa(self) -> None:
        if not self.swa_active or self.swa_model is None:
            return
        update_bn((b.bytes.to(self.device) for b in self.train_data), self.swa_model, device=self.device)
        self.model.load_state_dict(self.swa_model.module.state_dict())

    # ---- evaluation ---------------------------------------------------------------------------------------------------
    @torch.no_grad()
    def validate(self, optimize_threshold: bool = False) -> Metrics:
        if self.val_data is None:
            raise ValueError("No validation data provided")
        self.model.eval()
        cfg = self.config
        scores, targets = [], []
        total_loss = torch.zeros((), device=self.device)
        tokens = 0
        t0 = time.perf_counter()
        for batch in self.val_data:
            batch = self._to_device(batch)
            tokens += int(batch.lengths.sum()) if batch.lengths is not None else batch.bytes.numel()
            logits, aux = self._forward_batch(batch)
            total_loss += self._compute_loss(logits, batch, aux)
            if self.head_type == "mask":
                valid = self._valid_positions(batch, logits.shape[1])
                scores.append(torch.sigmoid(logits)[valid])
                targets.append(batch.masks[valid])
            elif self.n_classes > 2:
                scores.append(logits.argmax(-1))
                targets.append(batch.labels)
            else:
                scores.append(torch.sigmoid(logits).view(-1))
                targets.append(batch.labels)
        y = torch.cat(targets).cpu()
        s = torch.cat(scores).cpu()
        if self.n_classes > 2 and self.head_type != "mask":
            metrics = Metrics(float(total_loss) / len(self.val_data), 0.0, 0.0, 0.0,
                              accuracy=float((s == y.long()).float().mean()) if len(y) else 0.0)
        else:
            probs, truth = s.numpy(), y.numpy()
            if optimize_threshold and cfg.threshold_search:
                self.optimal_threshold = find_optimal_threshold(probs, truth, cfg.threshold_search_steps,
                                                                cfg.threshold_optimize_for, cfg.threshold_min_precision)
            pred, pos = probs >= self.optimal_threshold, truth == 1
            metrics = self._build_metrics(float(total_loss), len(self.val_data), int((pred & pos).sum()), int((pred & ~pos).sum()),
                                          int((~pred & pos).sum()), int((~pred & ~pos).sum()), len(truth))
        metrics.eval_time = time.perf_counter() - t0
        metrics.eval_tokens_per_sec = tokens / metrics.eval_time if metrics.eval_time > 0 else 0.0
        target = metrics.accuracy if self.n_classes > 2 else (metrics.recall if cfg.threshold_optimize_for == "recall" else metrics.f1)
        if target > self.best_metric + 0.001:
            self.best_metric = target
            self.best_state = {k: v.detach().clone() for k, v in self.model.state_dict().items()}
        return metrics

    def load_best_model(self) -> None:
        if self.best_state is not None:
            self.model.load_state_dict(self.best_state)

    # ---- checkpoints --------------------------------------------------------------------------------------------------
    def save_checkpoint(self, path: Path, extra: dict | None = None, with_optimizer: bool = False) -> None:
        data = {"model_config": self.model.config.to_dict(), "train_config": self.config.to_dict(),
                "state_dict": self.model.state_dict(), "best_metric": self.best_metric, "best_state": self.best_state,
                "optimal_threshold": self.optimal_threshold}
        if with_optimizer:  # what a bit-exact resume needs beyond the reference's dictionary
            data["optimizer"] = self.optimizer.state_dict()
            data["scheduler_steps"] = self._scheduler_steps
            if self.scheduler is not None:
                data["scheduler"] = self.scheduler.state_dict()
        data.update(extra or {})
        save_checkpoint(data, path)

    @classmethod
    def load_checkpoint(cls, path: Path, device: torch.device | None = None):
        device = device or get_device()
        data = load_checkpoint(path, map_location=device)
        model = Model(ModelConfig.from_dict(data["model_config"]))
        model.load_state_dict(data.get("best_state") or data["state_dict"])
        trainer = cls(model.to(device), [], config=TrainConfig.from_dict(data.get("train_config", {})), device=device)
        trainer.best_metric = data.get("best_metric", 0.0)
        trainer.optimal_threshold = data.get("optimal_threshold", 0.5)
        return model, trainer, data


def compute_length_bins(lengths: list[int]) -> list[int]:
    """Bucket edges tuned for line-level data (dense below 70 bytes, long sparse tail)."""
    if not lengths:
        return [512]
    longest = max(lengths)
    return [b for b in LENGTH_BINS if b <= longest] or [longest]


def _binned_groups(lengths, batch_size, indices):
    """Yield index groups: samples bucketed by length bin, sorted by length inside a bin, cut into batches."""
    indices = list(range(len(lengths))) if indices is None else indices
    edges = compute_length_bins([lengths[i] for i in indices])
    bins: dict[int, list[int]] = {e: [] for e in edges}
    bins[-1] = []
    for i in indices:
        bins[next((e for e in edges if lengths[i] <= e), -1)].append(i)
    for members in bins.values():
        members.sort(key=lengths.__getitem__)
        for s in range(0, len(members), batch_size):
            yield members[s:s + batch_size]


def create_mask_batches(byte_tensors, mask_tensors, lengths, batch_size, indices=None, shuffle=True, seed=None,
                        show_progress=True) -> list[MaskBatch]:
    if seed is not None:
        random.seed(seed)
    batches = [MaskBatch(pad_sequence([byte_tensors[j] for j in g], batch_first=True, padding_value=0),
                         pad_sequence([mask_tensors[j] for j in g], batch_first=True, padding_value=0.0),
                         torch.tensor([lengths[j] for j in g])) for g in _binned_groups(lengths, batch_size, indices)]
    if shuffle:
        random.shuffle(batches)
    return batches


def create_binary_batches(byte_tensors, labels, lengths, batch_size, feature_tensors=None, secret_ids=None, indices=None,
                          shuffle=True, seed=None, show_progress=True) -> list[BinaryBatch]:
    if seed is not None:
        random.seed(seed)
    batches = []
    for g in _binned_groups(lengths, batch_size, indices):
        batches.append(BinaryBatch(
            pad_sequence([byte_tensors[j] for j in g], batch_first=True, padding_value=0),
            torch.tensor([labels[j] for j in g]), torch.tensor([lengths[j] for j in g]),
            None if feature_tensors is None else torch.stack([feature_tensors[j] for j in g]),
            None if secret_ids is None else [secret_ids[j] for j in g]))
    if shuffle:
        random.shuffle(batches)
    return batches
