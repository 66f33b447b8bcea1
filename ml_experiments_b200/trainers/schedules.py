"""Schedules of the HEAD speedrun trainer: batch size, attention window, learning rate, Muon momentum, multi-token
prediction weights, YaRN window transitions (reference: modded-nanogpt/train_gpt.py:816-913,1500-1749)."""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch


@dataclass
class ScheduleArgs:
    num_scheduled_iterations: int = 1535
    num_extension_iterations: int = 40
    cooldown_frac: float = 0.55
    train_bs_schedule: tuple = (8 * 2048 * 8, 16 * 2048 * 8, 24 * 2048 * 8)
    train_bs_extension: int = 24 * 2048 * 8
    train_max_seq_len: int = 128 * 16
    ws_schedule: tuple = (3, 7, 11)
    ws_final: int = 13
    ws_validate_post_yarn_ext: int = 20
    block_size: int = 128

    @property
    def num_iterations(self) -> int:
        return self.num_scheduled_iterations + self.num_extension_iterations


def get_bs(step: int, a: ScheduleArgs) -> int:
    if step >= a.num_scheduled_iterations:
        return a.train_bs_extension
    return a.train_bs_schedule[int(len(a.train_bs_schedule) * step / a.num_scheduled_iterations)]


def get_ws(step: int, a: ScheduleArgs) -> tuple[int, int]:
    """``(short, long)`` window sizes in blocks."""
    if step >= a.num_scheduled_iterations:
        return a.ws_final // 2, a.ws_final
    w = a.ws_schedule[int(len(a.ws_schedule) * step / a.num_scheduled_iterations)]
    return w // 2, w


def get_lr(step: int, a: ScheduleArgs) -> float:
    if step > a.num_scheduled_iterations:
        return 0.1
    x = step / a.num_scheduled_iterations
    lr_max = 1.73 if x > 2 / 3 else (1.52 if x > 1 / 3 else 1.0)
    if x >= 1 - a.cooldown_frac:
        w = (1 - x) / a.cooldown_frac
        return lr_max * w + (1 - w) * 0.1
    return lr_max


def get_muon_momentum(step: int, a: ScheduleArgs, warmup: int = 300, cooldown: int = 50, lo: float = 0.85, hi: float = 0.95) -> float:
    cd_start = a.num_iterations - cooldown
    if step < warmup:
        return lo + step / warmup * (hi - lo)
    if step > cd_start:
        return hi - (step - cd_start) / cooldown * (hi - lo)
    return hi


def mtp_weights(step: int, a: ScheduleArgs) -> list[float]:
    """Multi-token-prediction weights: three targets early, two in the middle third, one at the end."""
    x = min(step / a.num_scheduled_iterations, 1.0)
    if x < 1 / 3:
        return [1.0, 0.5, 0.25 * (1 - 3 * x)]
    if x < 2 / 3:
        return [1.0, 0.5 * (1 - (3 * x - 1))]
    return [1.0]


class Yarn:
    """Rotary tables with half-truncated frequencies whose low frequencies are rescaled when the attention window
    grows (YaRN); ``attn_scale`` follows ``0.2 ln(new / old) + 1`` at every transition."""

    def __init__(self, head_dim: int, max_seq_len: int, base: float = 1024.0, device=None, alpha: int = 1, beta: int = 32):
        self.head_dim, self.max_seq_len, self.alpha, self.beta = head_dim, max_seq_len, alpha, beta
        freq = (1 / base) ** torch.linspace(0, 1, steps=head_dim // 4, dtype=torch.float32)
        self.angular_freq = torch.cat([freq, freq.new_zeros(head_dim // 4)]).to(device)
        self.attn_scale = 0.1
        self._rebuild(device)

    def _rebuild(self, device=None):
        t = torch.arange(2 * self.max_seq_len, dtype=torch.float32, device=self.angular_freq.device)
        theta = torch.outer(t, self.angular_freq)
        self.cos, self.sin = theta.cos().contiguous(), theta.sin().contiguous()

    def apply(self, old_window: int, new_window: int) -> None:
        if old_window == new_window:
            return
        rotations = 128 * old_window * self.angular_freq / (2 * math.pi)
        scale = old_window / new_window
        interp = torch.clamp((rotations - self.alpha) / (self.beta - self.alpha), 0, 1)
        self.angular_freq = self.angular_freq * (scale + (1 - scale) * interp)
        self.attn_scale *= 0.2 * math.log(new_window / old_window) + 1
        self._rebuild()


@dataclass
class TrainingManager:
    """Steps the schedules and reports what changed (batch size -> loader ``.send``; window -> ``Yarn.apply``)."""

    args: ScheduleArgs = field(default_factory=ScheduleArgs)
    yarn: Yarn | None = None
    _ws: tuple = (0, 0)
    _bs: int = 0

    def advance_schedule(self, step: int) -> dict:
        a = self.args
        out = {"lr_mul": get_lr(step, a), "muon_momentum": get_muon_momentum(step, a), "mtp_weights": mtp_weights(step, a),
               "do_adam": step % 2 == 1, "batch_changed": False, "window_changed": False}
        bs, ws = get_bs(step, a), get_ws(step, a)
        if bs != self._bs:
            out["batch_changed"], self._bs = True, bs
        if ws != self._ws:
            if self.yarn is not None and self._ws[1] > 0:
                self.yarn.apply(self._ws[1], ws[1])
            out["window_changed"], self._ws = True, ws
        out.update(batch_size=bs, ws_short=ws[0], ws_long=ws[1])
        return out
