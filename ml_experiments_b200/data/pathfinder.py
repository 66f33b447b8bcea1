"""Pathfinder / Path-X image generator: two circular markers and dashed "snakes" (chains of short oriented paddles);
the label says whether both markers sit on the ends of the same snake. The reference drives an external generator
(`snakes2` of drewlinsley/pathfinder, not shipped with it; scripts/generate_pathx.py:13-110) with: image 256 x 256,
contour length 14 paddles, distractor length 14 // 3, 30 // distractor_length distractor snakes, paddle length 5,
thickness 2, margin 3, marker radius 5, continuity 1.8. This module draws images of the same construction with numpy
(direction random walk whose step is bounded by ``pi / (2 * continuity)``), deterministic in the seed.
"""
from __future__ import annotations

import math

import numpy as np


def _draw_segment(img, x0, y0, x1, y1, thickness, value=1.0):
    H, W = img.shape
    pad = thickness + 1
    xa, xb = int(max(min(x0, x1) - pad, 0)), int(min(max(x0, x1) + pad + 1, W))
    ya, yb = int(max(min(y0, y1) - pad, 0)), int(min(max(y0, y1) + pad + 1, H))
    if xa >= xb or ya >= yb:
        return
    ys, xs = np.mgrid[ya:yb, xa:xb]
    dx, dy = x1 - x0, y1 - y0
    t = np.clip(((xs - x0) * dx + (ys - y0) * dy) / max(dx * dx + dy * dy, 1e-9), 0, 1)
    dist = np.hypot(xs - (x0 + t * dx), ys - (y0 + t * dy))
    img[ya:yb, xa:xb] = np.maximum(img[ya:yb, xa:xb], value * np.clip(thickness / 2 + 0.5 - dist, 0, 1))


def _draw_disc(img, x, y, radius, value=1.0):
    H, W = img.shape
    xa, xb = int(max(x - radius - 1, 0)), int(min(x + radius + 2, W))
    ya, yb = int(max(y - radius - 1, 0)), int(min(y + radius + 2, H))
    ys, xs = np.mgrid[ya:yb, xa:xb]
    img[ya:yb, xa:xb] = np.maximum(img[ya:yb, xa:xb], value * np.clip(radius + 0.5 - np.hypot(xs - x, ys - y), 0, 1))


def _snake(rng, size, n_paddles, paddle_length, margin, continuity, padding):
    """Centres and headings of a chain of paddles that stays inside the padded image (``None`` when it cannot)."""
    step = paddle_length + margin
    for _ in range(20):
        x, y = rng.uniform(padding, size - padding, 2)
        heading = rng.uniform(0, 2 * math.pi)
        pts = []
        for _ in range(n_paddles):
            pts.append((x, y, heading))
            heading += rng.uniform(-1, 1) * math.pi / (2 * continuity)
            x, y = x + step * math.cos(heading), y + step * math.sin(heading)
            if not (padding <= x <= size - padding and padding <= y <= size - padding):
                break
        else:
            return pts
    return None


def _draw_snake(img, pts, paddle_length, thickness, contrast=1.0):
    for x, y, h in pts:
        dx, dy = 0.5 * paddle_length * math.cos(h), 0.5 * paddle_length * math.sin(h)
        _draw_segment(img, x - dx, y - dy, x + dx, y + dy, thickness, contrast)


def pathfinder_image(rng, size: int = 256, contour_length: int = 14, marker_radius: int = 5, continuity: float = 1.8, paddle_length: int = 5,
                     paddle_thickness: int = 2, paddle_margin: int = 3, padding: int = 22, positive: bool | None = None):
    """-> ``(image float32 [size, size] in [0, 1], label)``."""
    positive = bool(rng.integers(0, 2)) if positive is None else positive
    scale = size / 256
    if scale < 1:  # smaller canvases keep the construction with proportionally smaller parts
        marker_radius = max(int(round(marker_radius * scale)), 1)
        paddle_length = max(int(round(paddle_length * max(scale, 0.4))), 2)
        paddle_margin = max(int(round(paddle_margin * max(scale, 0.4))), 1)
    padding = max(int(padding * scale), marker_radius + 1)
    img = np.zeros((size, size), dtype=np.float32)
    distractor_length = max(contour_length // 3, 1)

    def place(n):  # a chain that does not fit is retried one paddle shorter
        while True:
            pts = _snake(rng, size, n, paddle_length, paddle_margin, continuity, padding)
            if pts is not None:
                return pts
            n = max(n - 1, 2)

    target = place(contour_length)
    second = place(len(target))  # in a negative image the second marker sits on another snake of the same length
    _draw_snake(img, target, paddle_length, paddle_thickness)
    if not positive:
        _draw_snake(img, second, paddle_length, paddle_thickness)
    for _ in range(max(int(round((30 // distractor_length) * min(scale * scale * 4, 1.0))), 1)):
        d = _snake(rng, size, distractor_length, paddle_length, paddle_margin, continuity, padding)
        if d is not None:
            _draw_snake(img, d, paddle_length, paddle_thickness)
    ends = (target[0], target[-1]) if positive else (target[0], second[-1])
    for x, y, _ in ends:
        _draw_disc(img, x, y, marker_radius)
    return img, int(positive)


def generate(n: int, size: int = 256, seed: int = 0, **kw):
    """``n`` images, half positive: ``(uint8 [n, size, size], int64 [n])``."""
    rng = np.random.default_rng(seed)
    xs, ys = np.zeros((n, size, size), dtype=np.uint8), np.zeros(n, dtype=np.int64)
    for i in range(n):
        img, ys[i] = pathfinder_image(rng, size, positive=bool(i % 2), **kw)
        xs[i] = np.round(img * 255).astype(np.uint8)
    order = rng.permutation(n)
    return xs[order], ys[order]
