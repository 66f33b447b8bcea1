"""Benchmark harness of the long-sequence operator family: trains attention / hierarchical / SGSB / conv / telephone
("gather") / Ripple / Ripple-channel / flat-Ripple classifiers (or per-token LMs on the synthetic recall tasks) at a
matched parameter budget and prints per-epoch accuracy. Role of the reference's ``scripts/bench_scatter_vs_attn.py``:
model builders with a binary search on width (:1229-1338), sequence classifier / LM shells (:418-503), AdamW with
warm-up -> plateau -> cosine (:1080-1105), label smoothing, SWA, hard-example mining, self-distillation with
EMA / lerp / slerp weight merging (:768-806, 870-874), bf16 autocast, one-batch profiling (:1756) and the determinism
switches (:1798-1810).

    python -m ml_experiments_b200.cli.bench_scatter --model ripple --dataset random-image --seq-len 1024 --epochs 2
    python -m ml_experiments_b200.cli.bench_scatter --model all --dataset mqar --seq-len 128 --target-params 200000

Datasets: the synthetic tasks of ``heuristic_secrets.data.synthetic`` (mqar, parity, copying, ...), ``random-image``
(uniform pixels, Bernoulli labels: the shape of the long-sequence benchmark config) and ``npz:<path>`` (arrays
``x_train, y_train, x_test, y_test``; images are flattened to pixel sequences in [0, 1]).
"""
from __future__ import annotations

import argparse
import copy
import math
import os
import time

import numpy as np
import torch
import torch.nn as nn
import torch.nn.functional as F

from ..heuristic_secrets.data import synthetic
from ..models.ripple import RippleClassifier
from ..models.ripple_channel import RippleChannelClassifier
from ..models.ripple_ops import RMSNorm, TelephoneAttentionND
from ..models.scatter import FlatRippleClassifierND, HierarchicalLocalBlock, SGSBBlockND

MODEL_TYPES = ["attention", "hier", "sgsb", "conv", "gather", "ripple", "ripple-channel", "flat"]
SYNTHETIC_TASKS = ["mqar", "compositional_mqar", "forgetting_mqar", "parity", "cumulative_parity", "majority", "cumulative_majority",
                   "copying", "selective_copying", "induction_heads"]


# ------------------------------------------------------------------------------------------------------------ blocks
class SwiGLU(nn.Module):
    def __init__(self, width: int, mult: float = 4.0):
        super().__init__()
        hidden = int(width * mult * 2 / 3)
        self.w12, self.w3 = nn.Linear(width, 2 * hidden), nn.Linear(hidden, width)

    def forward(self, x):
        a, b = self.w12(x).chunk(2, dim=-1)
        return self.w3(F.silu(a) * b)


class AttentionBlock(nn.Module):
    """Pre-norm full softmax attention + SwiGLU."""

    def __init__(self, width: int, num_heads: int = 4):
        super().__init__()
        self.n1, self.n2, self.h = RMSNorm(width), RMSNorm(width), num_heads
        self.qkv, self.out, self.mlp = nn.Linear(width, 3 * width), nn.Linear(width, width), SwiGLU(width)

    def forward(self, x):
        B, L, C = x.shape
        q, k, v = self.qkv(self.n1(x)).view(B, L, 3, self.h, C // self.h).permute(2, 0, 3, 1, 4)
        x = x + self.out(F.scaled_dot_product_attention(q, k, v).transpose(1, 2).reshape(B, L, C))
        return x + self.mlp(self.n2(x))


class ConvBlock(nn.Module):
    """Depthwise conv + squeeze-excite + pointwise MLP."""

    def __init__(self, width: int, kernel_size: int = 17):
        super().__init__()
        self.n1, self.n2 = RMSNorm(width), RMSNorm(width)
        self.conv = nn.Conv1d(width, width, kernel_size, padding=kernel_size // 2, groups=width)
        self.se = nn.Sequential(nn.Linear(width, max(width // 4, 1)), nn.SiLU(), nn.Linear(max(width // 4, 1), width), nn.Sigmoid())
        self.mlp = SwiGLU(width)

    def forward(self, x):
        h = self.conv(self.n1(x).transpose(1, 2)).transpose(1, 2)
        x = x + h * self.se(h.mean(dim=1, keepdim=True))
        return x + self.mlp(self.n2(x))


class TelephoneAttentionBlock(nn.Module):
    def __init__(self, width: int, num_heads: int = 4, max_seq_len: int = 8192):
        super().__init__()
        self.n1, self.n2 = RMSNorm(width), RMSNorm(width)
        self.attn, self.mlp = TelephoneAttentionND(width, ndim=1, num_heads=num_heads, max_seq_len=max_seq_len), SwiGLU(width)

    def forward(self, x):
        x = x + self.attn(self.n1(x))[0]
        return x + self.mlp(self.n2(x))


class SequenceClassifier(nn.Module):
    """Scalar inputs in [0, 1] (or token ids when ``vocab_size`` is given) -> blocks -> mean pool -> classes; with
    ``per_token`` the head is applied at every position (the LM shell)."""

    def __init__(self, block_fn, width: int, n_layers: int, n_out: int, seq_len: int, vocab_size: int | None = None, per_token: bool = False,
                 token_head: nn.Module | None = None):
        super().__init__()
        self.per_token, self.token_head = per_token, token_head
        self.embed = nn.Embedding(vocab_size, width) if vocab_size else nn.Linear(1, width)
        self.embed_norm, self.pos_norm, self.norm = RMSNorm(width), RMSNorm(width), RMSNorm(width)
        self.pos_embed = nn.Parameter(torch.randn(1, seq_len, width) * 0.02)
        self.layers = nn.ModuleList([block_fn() for _ in range(n_layers)])
        self.head = nn.Linear(width, n_out)

    def forward(self, x):
        h = self.embed(x) if isinstance(self.embed, nn.Embedding) else F.silu(self.embed(x.unsqueeze(-1)))
        h = self.embed_norm(h) + self.pos_norm(F.silu(self.pos_embed[:, : h.shape[1]]))
        for layer in self.layers:
            h = layer(h)
        h = self.norm(h)
        if self.token_head is not None and not self.per_token:
            return self.token_head(h)          # a head that reads all tokens (query-group head) instead of mean pool + linear
        return self.head(h) if self.per_token else self.head(h.mean(dim=1))


class _PerToken(nn.Module):
    """Adapts a pooled classifier class to per-token outputs by replacing its pooling (used for the Ripple LMs)."""

    def __init__(self, core, width, n_out):
        super().__init__()
        self.core, self.head = core, nn.Linear(width, n_out)

    def forward(self, x):
        feats = []
        handle = self.core.norm.register_forward_hook(lambda m, i, o: feats.append(o))
        try:
            self.core(x)
        finally:
            handle.remove()
        return self.head(feats[-1])


class _AsImage(nn.Module):
    """Hands the flat ``(B, H * W)`` rows of the resident dataset to a model that wants ``(B, H, W)``."""

    def __init__(self, core: nn.Module, grid):
        super().__init__()
        self.core, self.grid = core, tuple(grid)

    def forward(self, x):
        return self.core(x.view(x.shape[0], *self.grid))


def count_params(model: nn.Module) -> int:
    return sum(p.numel() for p in model.parameters())


def find_config_for_params(make, target_params: int, head_options=(2, 4, 8), min_w: int = 16, max_w: int = 512):
    """Binary search on the width (kept a multiple of ``2 * heads``) for the parameter count closest to the target."""
    best, best_diff = (min_w, head_options[0]), float("inf")
    for heads in head_options:
        align = 2 * heads
        lo, hi = max(min_w, align), max_w
        while lo <= hi:
            mid = max((lo + hi) // 2 // align * align, align)
            try:
                params = count_params(make(mid, heads))
            except Exception:
                hi = mid - align
                continue
            if abs(params - target_params) < best_diff:
                best, best_diff = (mid, heads), abs(params - target_params)
            if params < target_params:
                lo = mid + align
            elif params > target_params:
                hi = mid - align
            else:
                return best
    return best


def build_model(model_type: str, layers: int, n_out: int, seq_len: int, num_channels: int = 4, kernel_size: int = 17,
                attn_order: str = "tele,conv,lowrank", target_params: int = 400_000, cross_layer: bool = False, router_top_k: int = 0,
                jacobi_iters: int = 12, siren_conv: bool = False, vocab_size: int | None = None, per_token: bool = False,
                embed_2d: tuple[int, int] | None = None, use_ssm: bool = False, ml_decoder: bool = False, hier_kw: dict | None = None):
    """``use_ssm``: a chunk-scan state-space mixer after every attention / hierarchical block; ``ml_decoder``: query-group
    head instead of mean pool + linear; ``hier_kw``: ``conv_position`` / ``attn_residual`` / ``merge_mode`` /
    ``lowrank_hier`` of the hierarchical block."""
    from .scatter_grid import QueryGroupHead, WithSSM
    max_len = max(seq_len, 64)
    hier_kw = hier_kw or {}
    ssm = (lambda make_block, w, h: (lambda: WithSSM(make_block(), w, h, 1))) if use_ssm else (lambda make_block, w, h: make_block)
    if model_type in ("ripple", "ripple-channel", "flat"):
        def make(w, _h):
            if model_type == "ripple":
                return RippleClassifier(width=w, n_layers=layers, n_classes=n_out, seq_len=seq_len, num_heads=num_channels, order=attn_order,
                                        cross_layer=cross_layer, vocab_size=vocab_size, jacobi_iters=jacobi_iters, siren_conv=siren_conv,
                                        max_seq_len=max_len, embed_2d=embed_2d)
            if model_type == "ripple-channel":
                return RippleChannelClassifier(width=w, n_channels=layers, n_classes=n_out, seq_len=seq_len, topology=attn_order,
                                               num_heads=num_channels, vocab_size=vocab_size, router_top_k=router_top_k, siren_conv=siren_conv,
                                               jacobi_iters=jacobi_iters, max_seq_len=max_len, embed_2d=embed_2d)
            return FlatRippleClassifierND(embed_dim=w, n_classes=n_out, iterations=layers, kernel_size=kernel_size, ndim=1, num_channels=num_channels)
        width, _ = find_config_for_params(make, target_params, head_options=(num_channels,))
        core = make(width, num_channels)
        return _PerToken(core, width, n_out) if per_token else core
    blocks = {
        "attention": lambda w, h: ssm(lambda: AttentionBlock(w, num_heads=h), w, h),
        "hier": lambda w, h: ssm(lambda: HierarchicalLocalBlock(w, window_size=kernel_size, num_channels=h, **hier_kw), w, h),
        "sgsb": lambda w, h: (lambda: SGSBBlockND(w, kernel_size=kernel_size, ndim=1, num_channels=h)),
        "conv": lambda w, h: (lambda: ConvBlock(w, kernel_size=kernel_size)),
        "gather": lambda w, h: (lambda: TelephoneAttentionBlock(w, num_heads=h, max_seq_len=max_len)),
    }
    if model_type not in blocks:
        raise ValueError(f"Unknown model type: {model_type}")
    make = lambda w, h: SequenceClassifier(blocks[model_type](w, h), w, layers, n_out, seq_len, vocab_size=vocab_size, per_token=per_token,
                                           token_head=QueryGroupHead(w, n_out) if ml_decoder and not per_token else None)
    width, heads = find_config_for_params(make, target_params)
    return make(width, heads)


# -------------------------------------------------------------------------------------------------------------- data
class PreloadedDataset:
    """Whole dataset resident on the device; ``batches()`` yields shuffled slices (no host round trips)."""

    def __init__(self, x: torch.Tensor, y: torch.Tensor, device, batch_size: int, shuffle: bool, seed: int = 0):
        self.x, self.y, self.batch_size, self.shuffle = x.to(device), y.to(device), batch_size, shuffle
        self.gen = torch.Generator(device="cpu").manual_seed(seed)

    def __len__(self):
        return (len(self.x) + self.batch_size - 1) // self.batch_size

    def batches(self, weights: torch.Tensor | None = None):
        n = len(self.x)
        if weights is not None:      # hard-example mining: sample with probability proportional to the previous loss
            order = torch.multinomial(weights.cpu(), n, replacement=True, generator=self.gen)
        else:
            order = torch.randperm(n, generator=self.gen) if self.shuffle else torch.arange(n)
        order = order.to(self.x.device)
        for i in range(0, n, self.batch_size):
            idx = order[i:i + self.batch_size]
            yield idx, self.x[idx], self.y[idx]


def load_dataset(name: str, seq_len: int | None, num_train: int, num_test: int, seed: int, vocab_size: int | None = None):
    """-> ``(x_train, y_train, x_test, y_test, n_out, task_type, vocab, seq_len)``; ``task_type`` is ``classification`` or ``lm``."""
    if name in SYNTHETIC_TASKS:
        L = seq_len or 128
        kw = {} if vocab_size is None or name in ("parity", "cumulative_parity", "majority", "cumulative_majority") else {"vocab_size": vocab_size}
        tr = synthetic.TASKS[name](num_examples=num_train, seed=seed, seq_len=L, **kw)
        te = synthetic.TASKS[name](num_examples=num_test, seed=seed + 1000, seq_len=L, **kw)
        vocab = int(max(tr.inputs.max(), tr.labels.max()).item()) + 1
        per_token = tr.labels.dim() == 2
        return tr.inputs, tr.labels, te.inputs, te.labels, vocab if per_token else int(tr.labels.max().item()) + 1, "lm" if per_token else "classification", vocab, L
    if name == "random-image":
        L = seq_len or 1024
        g = torch.Generator().manual_seed(seed)
        mk = lambda n: (torch.randint(0, 256, (n, L), generator=g).float() / 255, (torch.rand(n, generator=g) < 0.5).long())
        (xa, ya), (xb, yb) = mk(num_train), mk(num_test)
        return xa, ya, xb, yb, 2, "classification", None, L
    if name.startswith("npz:"):
        d = np.load(name[4:])
        f = lambda a: torch.from_numpy(a.reshape(len(a), -1)).float() / (255.0 if a.dtype == np.uint8 else 1.0)
        xa, xb = f(d["x_train"]), f(d["x_test"])
        ya, yb = torch.from_numpy(d["y_train"]).long(), torch.from_numpy(d["y_test"]).long()
        if seq_len:
            xa, xb = xa[:, :seq_len], xb[:, :seq_len]
        return xa, ya, xb, yb, int(ya.max()) + 1, "classification", None, xa.shape[1]
    raise ValueError(f"Unknown dataset {name}; available: {SYNTHETIC_TASKS + ['random-image', 'npz:<path>']}")


# ---------------------------------------------------------------------------------------------------------- training
def lr_lambda(step: int, total: int, warmup: int, cosine_start: float):
    """Linear warm-up, plateau for ``cosine_start`` of the remainder, cosine decay to zero."""
    if step < warmup:
        return (step + 1) / max(warmup, 1)
    rest = max(total - warmup, 1)
    hold = int(rest * cosine_start)
    if step - warmup < hold:
        return 1.0
    return 0.5 * (1 + math.cos(math.pi * (step - warmup - hold) / max(rest - hold, 1)))


def lerp_weights(a, b, t):
    return {k: torch.lerp(a[k].float(), b[k].float(), t).to(a[k].dtype) if a[k].is_floating_point() else b[k] for k in a}


def slerp_weights(a, b, t):
    out = {}
    for k in a:
        if not a[k].is_floating_point() or a[k].numel() < 2:
            out[k] = b[k]
            continue
        x, y = a[k].float().flatten(), b[k].float().flatten()
        cos = torch.clamp(F.cosine_similarity(x, y, dim=0), -1 + 1e-7, 1 - 1e-7)
        om = torch.acos(cos)
        if om.abs() < 1e-4:
            out[k] = torch.lerp(a[k].float(), b[k].float(), t).to(a[k].dtype)
        else:
            out[k] = ((torch.sin((1 - t) * om) * x + torch.sin(t * om) * y) / torch.sin(om)).view_as(a[k]).to(a[k].dtype)
    return out


def merge_teacher_student(teacher_sd, student_sd, alpha: float, method: str = "ema"):
    """``alpha`` = share of the student (0 keeps the teacher)."""
    return slerp_weights(teacher_sd, student_sd, alpha) if method == "slerp" else lerp_weights(teacher_sd, student_sd, alpha)


def _loss_per_sample(logits, y, task_type, label_smoothing=0.0):
    if task_type == "lm":
        l = F.cross_entropy(logits.flatten(0, 1).float(), y.flatten(), ignore_index=-100, reduction="none", label_smoothing=label_smoothing)
        l = l.view_as(y)
        return l.sum(1) / (y != -100).sum(1).clamp(min=1)
    return F.cross_entropy(logits.float(), y, reduction="none", label_smoothing=label_smoothing)


def _accuracy(logits, y, task_type):
    pred = logits.argmax(-1)
    if task_type == "lm":
        m = y != -100
        return (pred[m] == y[m]).float().sum().item(), int(m.sum().item())
    return (pred == y).float().sum().item(), y.numel()


@torch.no_grad()
def evaluate(model, data: PreloadedDataset, task_type, amp: bool):
    model.eval()
    correct = total = 0
    losses = torch.zeros(len(data.x), device=data.x.device)
    for idx, x, y in data.batches():
        with torch.autocast(x.device.type, dtype=torch.bfloat16, enabled=amp):
            logits = model(x)
        c, n = _accuracy(logits, y, task_type)
        correct, total = correct + c, total + n
        losses[idx] = _loss_per_sample(logits, y, task_type)
    return correct / max(total, 1), losses


# ------------------------------------------------------------------------------------------------ sample selection
def ensemble_teacher_logits(logit_history, loss_history, top_k: int = 3) -> torch.Tensor:
    """``logit_history``: per epoch ``[N, classes]``; ``loss_history``: per epoch ``[N]`` (``inf`` where the sample was
    misclassified). Per sample the ``top_k`` lowest-loss epochs are averaged with weights proportional to 1 / loss;
    a sample never classified correctly gets zero logits (a uniform teacher)."""
    logits, losses = torch.stack(logit_history), torch.stack(loss_history)
    k = min(top_k, losses.shape[0])
    best, where = losses.topk(k, dim=0, largest=False)
    picked = torch.gather(logits, 0, where.unsqueeze(-1).expand(-1, -1, logits.shape[-1]))
    w = torch.where(torch.isfinite(best), 1.0 / (best + 1e-8), torch.zeros_like(best))
    w = w / w.sum(dim=0, keepdim=True).clamp_min(1e-8)
    return (picked * w.unsqueeze(-1)).sum(dim=0)


@torch.no_grad()
def _logits_and_losses(model, data: "PreloadedDataset", amp: bool):
    """Logits and per-sample cross entropy of every sample of ``data`` in storage order."""
    model.eval()
    outs = []
    for i in range(0, len(data.x), data.batch_size):
        with torch.autocast(data.x.device.type, dtype=torch.bfloat16, enabled=amp):
            outs.append(model(data.x[i:i + data.batch_size]).float())
    logits = torch.cat(outs)
    model.train()
    return logits, F.cross_entropy(logits, data.y, reduction="none")


def hard_fraction(epoch: int, epochs: int, start: float, end: float) -> float:
    """Share of each batch that is back-propagated at ``epoch``: linear from ``start`` to ``end`` over the run."""
    t = epoch / max(epochs - 1, 1)
    return start + (end - start) * t


def selection_weights(per_sample: torch.Tensor, mode: str | None, fraction: float = 1.0) -> torch.Tensor:
    """Per-sample weights for one batch from the (detached) per-sample losses.

    ``None``: all ones. ``"top"``: ones on the hardest ``fraction`` of the batch, zeros elsewhere (in-batch hard mining,
    ``--hard-start`` / ``--hard-end`` / ``--first-epoch-pct``). ``"wtf"``: +1 above the batch median, -1 below, i.e.
    descent on the hard half and ascent on the easy half. ``"easy"``: complement of ``"top"`` (the second model of a duo)."""
    n = per_sample.numel()
    if mode is None or n == 0:
        return torch.ones_like(per_sample)
    if mode == "wtf":
        return torch.where(per_sample > per_sample.median(), 1.0, -1.0).to(per_sample.dtype)   # torch.median: the lower middle
    k = min(max(int(round(n * fraction)), 1), n)
    hard = torch.zeros_like(per_sample)
    hard[per_sample.topk(k).indices] = 1.0
    if mode == "top":
        return hard
    if mode == "easy":
        easy = 1.0 - hard
        return easy if easy.sum() > 0 else hard
    raise ValueError(f"unknown selection mode {mode}")


def weighted_mean(per_sample: torch.Tensor, w: torch.Tensor) -> torch.Tensor:
    return (per_sample * w).sum() / w.abs().sum().clamp(min=1.0)


class DuoModel(nn.Module):
    """Two copies of an architecture trained on complementary parts of every batch (one on the hardest share, the
    other on the rest, ranked by the merged prediction's loss) and merged at inference (``--duo``)."""

    MERGE_STRATEGIES = ("mean", "max", "logsum", "harmonic")

    def __init__(self, model_hard: nn.Module, model_easy: nn.Module, merge: str = "mean"):
        super().__init__()
        if merge not in self.MERGE_STRATEGIES:
            raise ValueError(f"merge must be one of {self.MERGE_STRATEGIES}")
        self.model_hard, self.model_easy, self.merge = model_hard, model_easy, merge

    def merge_logits(self, a, b):
        if self.merge == "mean":
            return 0.5 * (a + b)
        if self.merge == "max":
            return torch.maximum(a, b)
        if self.merge == "logsum":
            return F.log_softmax(a.float(), -1) + F.log_softmax(b.float(), -1)
        return 2 * a * b / (a + b + 1e-8)

    def forward_both(self, x):
        a, b = self.model_hard(x), self.model_easy(x)
        return self.merge_logits(a, b), a, b

    def forward(self, x):
        return self.forward_both(x)[0]


def train_model(model, train: PreloadedDataset, test: PreloadedDataset, epochs: int, lr: float, task_type: str = "classification",
                warmup_epochs: int = 2, cosine_start: float = 0.1, swa: bool = False, swa_start: float = 0.8, swa_lr: float = 1e-5,
                hard_mining: bool = False, amp: bool = False, label_smoothing: float = 0.1, self_distill: bool = False,
                distill_alpha: float = 0.5, distill_temp: float = 2.0, distill_merge: str | None = None, distill_merge_alpha: float = 0.5,
                checkpoint_dir: str | None = None, model_name: str = "model", verbose: bool = True, weight_decay: float = 0.01,
                hard_start: float | None = None, hard_end: float | None = None, first_epoch_pct: float | None = None,
                wtf_mode: bool = False, distill_adaptive: bool = False, distill_from_merged: bool = False, distill_ensemble: bool = False,
                distill_ensemble_k: int = 3):
    """Trains ``model`` (or both halves of a :class:`DuoModel`). In-batch selection: with ``hard_start`` / ``hard_end`` only
    the hardest share of each batch is back-propagated (share moving linearly over the epochs), ``first_epoch_pct``
    does that for the first epoch only, ``wtf_mode`` ascends on the easy half. ``distill_adaptive`` blends the
    teacher and the labels per sample: easy samples follow the teacher, hard ones the labels. ``distill_from_merged``:
    the teacher of the next epoch is the weight merge of the previous teacher and the current model (``distill_merge``
    names the rule, exponential average by default). ``distill_ensemble``: the teacher is no model but a table of
    logits per training sample, the inverse-loss-weighted mean over the ``distill_ensemble_k`` epochs in which that sample
    was classified correctly with the lowest loss (:func:`ensemble_teacher_logits`)."""
    duo = isinstance(model, DuoModel)
    opt = torch.optim.AdamW(model.parameters(), lr=lr, weight_decay=weight_decay)
    steps = epochs * len(train)
    sched = torch.optim.lr_scheduler.LambdaLR(opt, lambda s: lr_lambda(s, steps, min(warmup_epochs, max(epochs - 1, 0)) * len(train), cosine_start))
    swa_model = torch.optim.swa_utils.AveragedModel(model) if swa else None
    swa_epoch = int(epochs * swa_start)
    teacher, weights, history = None, None, []
    if distill_from_merged and not distill_merge:
        distill_merge = "ema"
    table, logit_hist, loss_hist = None, [], []      # ensemble distillation: teacher logits per training sample
    for epoch in range(epochs):
        model.train()
        t0, seen, correct, total = time.perf_counter(), 0, 0.0, 0
        in_swa = swa and epoch >= swa_epoch
        if in_swa:
            for gp in opt.param_groups:
                gp["lr"] = swa_lr
        for idx, x, y in train.batches(weights if hard_mining else None):
            frac, mode = 1.0, None
            if wtf_mode:
                mode = "wtf"
            elif first_epoch_pct is not None and epoch == 0:
                frac, mode = first_epoch_pct, "top"
            elif hard_start is not None:
                frac, mode = hard_fraction(epoch, epochs, hard_start, hard_end if hard_end is not None else hard_start), "top"
            with torch.autocast(x.device.type, dtype=torch.bfloat16, enabled=amp):
                if duo:
                    logits, la, lb = model.forward_both(x)
                    rank_by = _loss_per_sample(logits, y, task_type).detach()
                    f = frac if mode == "top" else 0.5
                    pa, pb = _loss_per_sample(la, y, task_type, label_smoothing), _loss_per_sample(lb, y, task_type, label_smoothing)
                    loss = weighted_mean(pa, selection_weights(rank_by, "top", f)) + weighted_mean(pb, selection_weights(rank_by, "easy", f))
                else:
                    logits = model(x)
                    per = _loss_per_sample(logits, y, task_type, label_smoothing)
                    w = selection_weights(per.detach(), mode, frac)
                    loss = weighted_mean(per, w)
                if (teacher is not None or table is not None) and not duo:
                    with torch.no_grad():
                        tl = table[idx] if table is not None else teacher(x)
                    kd_rows = F.kl_div(F.log_softmax(logits.float() / distill_temp, -1), F.softmax(tl.float() / distill_temp, -1),
                                       reduction="none").sum(-1)
                    if kd_rows.dim() > 1:
                        kd_rows = kd_rows.mean(tuple(range(1, kd_rows.dim())))
                    if distill_adaptive:
                        # rank of each sample's label loss inside the batch in [0, 1]: 0 (easy) -> all teacher, 1 (hard) -> all labels
                        r = per.detach().argsort().argsort().float() / max(per.numel() - 1, 1)
                        loss = (r * per + (1 - r) * kd_rows * distill_temp ** 2).mean()
                    else:
                        loss = (1 - distill_alpha) * loss + distill_alpha * kd_rows.mean() * distill_temp ** 2
            opt.zero_grad(set_to_none=True)
            loss.backward()
            opt.step()
            if not in_swa:
                sched.step()
            c, n = _accuracy(logits.detach(), y, task_type)
            correct, total, seen = correct + c, total + n, seen + len(x)
        if in_swa:
            swa_model.update_parameters(model)
        test_acc, _ = evaluate(swa_model.module if in_swa else model, test, task_type, amp)
        if hard_mining:
            _, per = evaluate(model, train, task_type, amp)
            weights = per.clamp(min=1e-6)
        if self_distill and distill_ensemble and task_type == "classification" and not duo:
            logits_all, per = _logits_and_losses(model, train, amp)
            wrong = logits_all.argmax(-1) != train.y
            logit_hist.append(logits_all)
            loss_hist.append(per.masked_fill(wrong, float("inf")))
            table = ensemble_teacher_logits(logit_hist, loss_hist, distill_ensemble_k)
        elif self_distill:
            if teacher is not None and distill_merge:
                merged = merge_teacher_student(teacher.state_dict(), model.state_dict(), distill_merge_alpha, distill_merge)
                teacher.load_state_dict(merged)
            else:
                teacher = copy.deepcopy(model)
            teacher.eval()
        dt = time.perf_counter() - t0
        history.append(dict(epoch=epoch + 1, train_acc=correct / max(total, 1), test_acc=test_acc, samples_per_s=seen / dt, lr=opt.param_groups[0]["lr"]))
        if verbose:
            print(f"[{model_name}] epoch {epoch + 1:2d}: train_acc={history[-1]['train_acc']:.4f} test_acc={test_acc:.4f} "
                  f"lr={history[-1]['lr']:.2e} {history[-1]['samples_per_s']:.1f} samples/s{' [SWA]' if in_swa else ''}", flush=True)
        if checkpoint_dir:
            os.makedirs(checkpoint_dir, exist_ok=True)
            ckpt = {"epoch": epoch + 1, "model": model.state_dict(), "optimizer": opt.state_dict(), "scheduler": sched.state_dict(), "test_acc": test_acc}
            if in_swa:
                ckpt["swa_model"] = swa_model.state_dict()
            torch.save(ckpt, os.path.join(checkpoint_dir, f"{model_name}_epoch{epoch + 1:03d}.pt"))
    return history


def set_determinism(seed: int):
    torch.manual_seed(seed)
    np.random.seed(seed)
    torch.backends.cudnn.deterministic, torch.backends.cudnn.benchmark = True, False


def profile_one_batch(model, data: PreloadedDataset, task_type, amp, warmup: int = 10, out: str = "bench_scatter_trace.json"):
    from torch.profiler import ProfilerActivity, profile
    opt = torch.optim.AdamW(model.parameters(), lr=1e-4)
    it = data.batches()

    def step():
        _, x, y = next(it)
        with torch.autocast(x.device.type, dtype=torch.bfloat16, enabled=amp):
            loss = _loss_per_sample(model(x), y, task_type).mean()
        opt.zero_grad(set_to_none=True)
        loss.backward()
        opt.step()
    for _ in range(min(warmup, len(data) - 1)):
        step()
    acts = [ProfilerActivity.CPU] + ([ProfilerActivity.CUDA] if data.x.is_cuda else [])
    with profile(activities=acts) as prof:
        step()
    prof.export_chrome_trace(out)
    print(prof.key_averages().table(sort_by="self_cuda_time_total" if data.x.is_cuda else "self_cpu_time_total", row_limit=25))


def _train_with_ponder(model, train: PreloadedDataset, test: PreloadedDataset, a, dev, n_classes: int) -> float:
    """``--ponder``: the classifier is trained on cross entropy plus a learned score of (logits, target)."""
    from ..models.unified.ponder import PonderTrainConfig, PonderTrainer, PonderWrapper

    class _Loader:          # PreloadedDataset batches as (inputs, labels) pairs with a length, what the trainer iterates over
        def __init__(self, data):
            self.data = data

        def __len__(self):
            return len(self.data)

        def __iter__(self):
            return ((x, y) for _, x, y in self.data.batches())

    cfg = PonderTrainConfig(meta_lr=a.ponder_meta_lr, model_lr=a.lr, epochs=a.epochs, meta_warmup_epochs=a.ponder_meta_warmup,
                            meta_wean_epochs=a.ponder_meta_wean, reward_scale=a.ponder_reward_scale,
                            meta_min_supervised=a.ponder_min_supervised)
    trainer = PonderTrainer(PonderWrapper(model, n_classes=n_classes), _Loader(train), _Loader(test), dev, cfg, squeeze_channel=False)
    return trainer.train(a.epochs)


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", default="all", help=f"one of {MODEL_TYPES} or 'all' or a comma list")
    ap.add_argument("--dataset", default="random-image")
    ap.add_argument("--epochs", type=int, default=10)
    ap.add_argument("--layers", type=int, default=4)
    ap.add_argument("--runs", type=int, default=1)
    ap.add_argument("--device", default="auto", choices=["cpu", "cuda", "auto"])
    ap.add_argument("--lr", type=float, default=3e-4)
    ap.add_argument("--batch-size", type=int, default=128)
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--seq-len", type=int, default=None)
    ap.add_argument("--num-train", type=int, default=10000)
    ap.add_argument("--num-test", type=int, default=2000)
    ap.add_argument("--cosine-start", type=float, default=0.1)
    ap.add_argument("--swa", action="store_true")
    ap.add_argument("--swa-start", type=float, default=0.8)
    ap.add_argument("--swa-lr", type=float, default=1e-5)
    ap.add_argument("--checkpoint-dir", default=None)
    ap.add_argument("--channels", type=int, default=4)
    ap.add_argument("--kernel-size", type=int, default=17)
    ap.add_argument("--amp", action="store_true", help="bf16 autocast")
    ap.add_argument("--profile", action="store_true", help="profile one batch after 10 warm-up batches, then exit")
    ap.add_argument("--hard-mining", action="store_true")
    ap.add_argument("--attn-order", default="tele,conv,lowrank")
    ap.add_argument("--target-params", type=int, default=400_000)
    ap.add_argument("--label-smoothing", type=float, default=0.1)
    ap.add_argument("--cross-layer", action="store_true")
    ap.add_argument("--with-router", type=int, default=0)
    ap.add_argument("--self-distill", action="store_true")
    ap.add_argument("--distill-alpha", type=float, default=0.5)
    ap.add_argument("--distill-temp", type=float, default=2.0)
    ap.add_argument("--distill-merge", default=None, choices=["ema", "slerp", "lerp"])
    ap.add_argument("--distill-merge-alpha", type=float, default=0.5)
    ap.add_argument("--task-vocab-size", type=int, default=None)
    ap.add_argument("--siren-conv", action="store_true")
    ap.add_argument("--jacobi-iters", type=int, default=1)
    ap.add_argument("--hard-start", type=float, default=None, help="share of each batch back-propagated at the first epoch (hardest first)")
    ap.add_argument("--hard-end", type=float, default=None, help="the same at the last epoch (linear in between)")
    ap.add_argument("--first-epoch-pct", type=float, default=None, help="first epoch only: back-propagate the hardest share of each batch")
    ap.add_argument("--wtf-mode", action="store_true", help="descent on the harder half of each batch, ascent on the easier half")
    ap.add_argument("--duo", action="store_true", help="two models on complementary shares of each batch, merged at inference")
    ap.add_argument("--duo-merge", default="mean", choices=DuoModel.MERGE_STRATEGIES)
    ap.add_argument("--distill-adaptive", action="store_true", help="self-distillation with a per-sample teacher / label blend")
    ap.add_argument("--2d", dest="mode_2d", action="store_true", help="image-native models on an (H, W) grid (square images unless --grid is given)")
    ap.add_argument("--3d", dest="mode_3d", action="store_true", help="volume-native models: colour planes become the depth axis of an (H, W, 3) grid")
    ap.add_argument("--grid", default=None, help="H,W or H,W,D of the inputs for --2d / --3d when they are not square")
    ap.add_argument("--ssm", action="store_true", help="add a state-space mixer after every attention / local / hierarchical block")
    ap.add_argument("--conv-position", default="both", choices=["pre", "post", "both"], help="hierarchical block: convolution before / after the attention")
    ap.add_argument("--merge-mode", default="lowrank", choices=["gate", "learned", "lowrank"], help="hierarchical block: how levels are merged")
    ap.add_argument("--lowrank-hier", dest="lowrank_hier", action="store_true", default=True, help="hierarchical block: low-rank full attention per level (default)")
    ap.add_argument("--no-lowrank-hier", dest="lowrank_hier", action="store_false", help="hierarchical block: windowed attention per level")
    ap.add_argument("--no-attn-residual", action="store_true", help="hierarchical block: no residual around the attention")
    ap.add_argument("--ml-decoder", action="store_true", help="query-group classification head instead of mean pool + linear")
    ap.add_argument("--distill-from-merged", action="store_true", help="self-distillation teacher = weight merge of the previous teacher and the model")
    ap.add_argument("--distill-ensemble", action="store_true", help="self-distillation teacher = per-sample ensemble of the best epochs' logits")
    ap.add_argument("--distill-ensemble-k", type=int, default=3)
    ap.add_argument("--ponder", action="store_true", help="train through the learned auxiliary loss (models/unified/ponder.py)")
    ap.add_argument("--ponder-meta-lr", type=float, default=3e-4)
    ap.add_argument("--ponder-reward-scale", type=float, default=100.0)
    ap.add_argument("--ponder-min-supervised", type=float, default=0.0)
    ap.add_argument("--ponder-meta-warmup", type=int, default=1)
    ap.add_argument("--ponder-meta-wean", type=int, default=1)
    # accepted for command-line compatibility with the reference harness; they have no effect here: data is always
    # resident on the device (no loader workers, nothing to preload lazily) and nothing is traced or compiled
    ap.add_argument("--workers", type=int, default=0, help=argparse.SUPPRESS)
    ap.add_argument("--no-preload", dest="preload", action="store_false", help=argparse.SUPPRESS)
    ap.add_argument("--compile", action="store_true", help=argparse.SUPPRESS)
    a = ap.parse_args(argv)
    dev = torch.device("cuda" if (a.device == "auto" and torch.cuda.is_available()) or a.device == "cuda" else "cpu")
    xa, ya, xb, yb, n_out, task_type, vocab, L = load_dataset(a.dataset, a.seq_len, a.num_train, a.num_test, a.seed, a.task_vocab_size)
    hier_kw = dict(conv_position=a.conv_position, attn_residual=not a.no_attn_residual, merge_mode=a.merge_mode, lowrank_hier=a.lowrank_hier)
    grid = None
    if a.mode_2d or a.mode_3d:
        if task_type != "classification":
            raise SystemExit("--2d / --3d are for classification datasets")
        if a.grid:
            grid = tuple(int(v) for v in a.grid.split(","))
        else:
            cells = L // 3 if a.mode_3d else L
            side = int(round(cells ** 0.5))
            grid = (side, side, 3) if a.mode_3d else (side, side)
        if int(np.prod(grid)) != L or len(grid) != (3 if a.mode_3d else 2):
            raise SystemExit(f"inputs of {L} values do not fill a grid {grid}: pass --grid H,W{',D' if a.mode_3d else ''}")

    def make_model(kind: str):
        from .scatter_grid import GRID_MODEL_TYPES, build_grid_model
        if grid is not None and kind in GRID_MODEL_TYPES:
            return build_grid_model(kind, a.layers, n_out, grid, num_channels=a.channels, kernel_size=min(a.kernel_size, 7 if len(grid) == 2 else 5),
                                    use_ssm=a.ssm, ml_decoder=a.ml_decoder, **(hier_kw if kind == "hier" else {})).to(dev)
        if a.mode_3d:
            raise SystemExit(f"--3d has the model types {GRID_MODEL_TYPES}")
        as_image = grid is not None and kind in ("ripple", "ripple-channel")      # these embed (B, H, W) pixel grids themselves
        core = build_model(kind, a.layers, n_out, L, num_channels=a.channels, kernel_size=a.kernel_size, attn_order=a.attn_order,
                           target_params=a.target_params, cross_layer=a.cross_layer, router_top_k=a.with_router, jacobi_iters=a.jacobi_iters,
                           siren_conv=a.siren_conv, vocab_size=vocab, per_token=task_type == "lm", use_ssm=a.ssm, ml_decoder=a.ml_decoder,
                           hier_kw=hier_kw, embed_2d=grid if as_image else None)
        return (_AsImage(core, grid) if as_image else core).to(dev)

    kinds = MODEL_TYPES if a.model == "all" else a.model.split(",")
    if grid is not None and a.model == "all":
        from .scatter_grid import GRID_MODEL_TYPES
        kinds = GRID_MODEL_TYPES + ([k for k in ("ripple", "ripple-channel", "flat") if not a.mode_3d])
    results = {}
    for kind in kinds:
        accs = []
        for run in range(a.runs):
            set_determinism(a.seed + run)
            model = make_model(kind)
            train = PreloadedDataset(xa, ya, dev, a.batch_size, True, a.seed + run)
            test = PreloadedDataset(xb, yb, dev, a.batch_size, False)
            print(f"[{kind}] {count_params(model):,} parameters, sequence length {L}, {task_type}", flush=True)
            if a.profile:
                profile_one_batch(model, train, task_type, a.amp)
                return results
            if a.duo:
                set_determinism(a.seed + run + 1000)
                twin = make_model(kind)
                model = DuoModel(model, twin, a.duo_merge)
            if a.ponder and task_type != "lm":
                accs.append(_train_with_ponder(model, train, test, a, dev, n_out))
                continue
            hist = train_model(model, train, test, a.epochs, a.lr, task_type, cosine_start=a.cosine_start, swa=a.swa, swa_start=a.swa_start,
                               swa_lr=a.swa_lr, hard_mining=a.hard_mining, amp=a.amp, label_smoothing=a.label_smoothing, self_distill=a.self_distill,
                               distill_alpha=a.distill_alpha, distill_temp=a.distill_temp, distill_merge=a.distill_merge,
                               distill_merge_alpha=a.distill_merge_alpha, checkpoint_dir=a.checkpoint_dir, model_name=kind,
                               hard_start=a.hard_start, hard_end=a.hard_end, first_epoch_pct=a.first_epoch_pct, wtf_mode=a.wtf_mode,
                               distill_adaptive=a.distill_adaptive, distill_from_merged=a.distill_from_merged,
                               distill_ensemble=a.distill_ensemble, distill_ensemble_k=a.distill_ensemble_k)
            accs.append(hist[-1]["test_acc"])
        results[kind] = dict(mean=float(np.mean(accs)), std=float(np.std(accs)), runs=accs)
        print(f"[{kind}] final test accuracy {results[kind]['mean']:.4f} +- {results[kind]['std']:.4f}", flush=True)
    return results


if __name__ == "__main__":
    main()
