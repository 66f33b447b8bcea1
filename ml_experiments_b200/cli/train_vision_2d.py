"""Train ``Model2d`` as an image classifier on MNIST / Fashion-MNIST / CIFAR-10 / CIFAR-100 (roles of the reference's
``scripts/train_mnist_cifar.py`` and ``scripts/train_vision_2d.py``): adaptive-conv or fixed-kernel branches, optional
attention, OneCycle AdamW with gradient clipping, auxiliary regularisers, optional SWA with batch-norm refresh, resume,
best-accuracy checkpoint.

The data path is device-resident: the whole set sits on the GPU as one uint8 tensor (CIFAR-10 is 150 MB of 180 GB) and
every batch is cut, augmented (random affine for grey images, pad-crop + flip for colour) and normalised by batched
tensor ops on the device, so no loader workers or host copies run inside an epoch. Sources: torchvision files already
present under ``--data-dir`` (nothing is downloaded), ``npz:<path>`` with ``x_train y_train x_test y_test``, or
``synthetic`` (class-coded blobs of the named dataset's shape).

    python -m ml_experiments_b200.cli.train_vision_2d --dataset cifar10 --source synthetic --epochs 2 --width 32
"""
from __future__ import annotations

import argparse
import json
import math
import time
from dataclasses import dataclass
from pathlib import Path

import numpy as np
import torch
import torch.nn.functional as F
from torch.optim.swa_utils import SWALR, AveragedModel

from ..models.unified.two_d import HeadConfig2d, LayerConfig2d, Model2d, ModelConfig2d
from ..utils.checkpoint import load_checkpoint, save_checkpoint


@dataclass
class DatasetConfig:
    name: str
    n_classes: int
    channels: int
    height: int
    width: int


DATASET_CONFIGS = {
    "mnist": DatasetConfig("mnist", 10, 1, 28, 28),
    "fashion-mnist": DatasetConfig("fashion-mnist", 10, 1, 28, 28),
    "cifar10": DatasetConfig("cifar10", 10, 3, 32, 32),
    "cifar100": DatasetConfig("cifar100", 100, 3, 32, 32),
}


def synthetic_images(ds: DatasetConfig, n: int, seed: int):
    """uint8 ``[n, C, H, W]`` whose class decides the position and colour of a bright blob over noise."""
    g = torch.Generator().manual_seed(seed)
    y = torch.randint(0, ds.n_classes, (n,), generator=g)
    yy, xx = torch.meshgrid(torch.arange(ds.height).float(), torch.arange(ds.width).float(), indexing="ij")
    side = math.ceil(math.sqrt(ds.n_classes))
    cy = ((y // side).float() + 0.5) / side * ds.height
    cx = ((y % side).float() + 0.5) / side * ds.width
    blob = torch.exp(-((yy[None] - cy[:, None, None]) ** 2 + (xx[None] - cx[:, None, None]) ** 2) / (2 * (ds.height / (2.5 * side)) ** 2))
    x = blob[:, None].expand(-1, ds.channels, -1, -1) * 200 + torch.rand(n, ds.channels, ds.height, ds.width, generator=g) * 55
    return x.clamp(0, 255).to(torch.uint8), y


def load_arrays(ds: DatasetConfig, source: str, data_dir: str, n_train: int, n_val: int, seed: int):
    """-> ``x_train, y_train, x_val, y_val`` with x uint8 ``[N, C, H, W]``."""
    if source == "synthetic":
        return (*synthetic_images(ds, n_train, seed), *synthetic_images(ds, n_val, seed + 1))
    if source.startswith("npz:"):
        d = np.load(source[4:])
        def img(a):
            t = torch.from_numpy(a)
            t = t.unsqueeze(1) if t.dim() == 3 else (t.permute(0, 3, 1, 2) if t.shape[-1] in (1, 3) else t)
            return t.contiguous() if t.dtype == torch.uint8 else (t.float().clamp(0, 1) * 255).to(torch.uint8)
        return img(d["x_train"]), torch.from_numpy(d["y_train"]).long(), img(d["x_test"]), torch.from_numpy(d["y_test"]).long()
    from torchvision import datasets
    cls = {"mnist": datasets.MNIST, "fashion-mnist": datasets.FashionMNIST, "cifar10": datasets.CIFAR10, "cifar100": datasets.CIFAR100}[ds.name]
    out = []
    for train in (True, False):
        d = cls(data_dir, train=train, download=False)
        x = torch.as_tensor(np.asarray(d.data))
        x = x.unsqueeze(1) if x.dim() == 3 else x.permute(0, 3, 1, 2)
        out += [x.contiguous(), torch.as_tensor(np.asarray(d.targets)).long()]
    return tuple(out)


def to_gray(x: torch.Tensor) -> torch.Tensor:
    if x.shape[1] == 1:
        return x
    w = torch.tensor([0.299, 0.587, 0.114], device=x.device).view(1, 3, 1, 1)
    return (x.float() * w).sum(1, keepdim=True).round().to(torch.uint8)


def augment(x: torch.Tensor, gen: torch.Generator) -> torch.Tensor:
    """``x`` float ``[B, C, H, W]`` in [0, 1]. Grey: rotation <= 10 deg, shift <= 10 %, zoom 0.9-1.1 (one batched
    affine grid). Colour: 4-pixel reflect-free pad + random crop + horizontal flip."""
    B, C, H, W = x.shape
    r = lambda *s: torch.rand(*s, device=x.device, generator=gen)
    if C == 1:
        ang = (r(B) * 2 - 1) * math.radians(10)
        sc = 1.0 / (0.9 + 0.2 * r(B))
        theta = torch.zeros(B, 2, 3, device=x.device)
        theta[:, 0, 0], theta[:, 0, 1] = sc * torch.cos(ang), -sc * torch.sin(ang)
        theta[:, 1, 0], theta[:, 1, 1] = sc * torch.sin(ang), sc * torch.cos(ang)
        theta[:, :, 2] = (r(B, 2) * 2 - 1) * 0.2                      # 10 % of the size = 0.2 in [-1, 1] coordinates
        return F.grid_sample(x, F.affine_grid(theta, list(x.shape), align_corners=False), padding_mode="zeros", align_corners=False)
    pad = F.pad(x, (4, 4, 4, 4))
    dy, dx = (r(B) * 9).long().clamp(max=8), (r(B) * 9).long().clamp(max=8)
    rows = dy[:, None] + torch.arange(H, device=x.device)[None]
    cols = dx[:, None] + torch.arange(W, device=x.device)[None]
    flip = r(B) < 0.5
    cols = torch.where(flip[:, None], cols.flip(1), cols)
    return pad[torch.arange(B, device=x.device)[:, None, None, None], torch.arange(C, device=x.device)[None, :, None, None],
               rows[:, None, :, None], cols[:, None, None, :]]


def normalise(x: torch.Tensor) -> torch.Tensor:
    return (x - 0.5) / 0.5


def build_model(a, ds: DatasetConfig, in_channels: int):
    g = max(1, min(4, a.width // 4))
    layer = LayerConfig2d(
        embed_width=a.width, in_channels=in_channels, dropout=0.1, conv_groups=g, use_attention=not a.no_attention, attn_heads=g,
        attn_ffn_mult=4, attn_window_size=16, attn_use_rope=True, num_attn_features=4, ssm_state_size=32, ssm_n_heads=g,
        ssm_kernel_sizes=(3, 5, 7), ssm_expand=2, num_ssm_features=4, adaptive_conv=a.adaptive, n_adaptive_branches=a.n_branches,
        adaptive_kernel_size=7, adaptive_init_sigmas=tuple(0.1 + 0.15 * i for i in range(a.n_branches)) if a.adaptive else None,
        context_dim=16, num_embed_features=4, mlp_hidden_mult=4, mlp_output_dim=16)
    cfg = ModelConfig2d(n_layers=a.n_layers, layer=layer, head=HeadConfig2d(head_type="classifier", n_classes=ds.n_classes))
    return Model2d(cfg), cfg


def class_logits(model, x, n_classes):
    logits, aux = model(x)
    if n_classes == 2 and logits.dim() == 1:                              # two classes -> one logit per image
        logits = torch.stack([torch.zeros_like(logits), logits], -1)
    return logits, aux


@torch.no_grad()
def evaluate(model, x, y, batch_size, n_classes):
    model.eval()
    loss = correct = 0.0
    for i in range(0, len(x), batch_size):
        logits, _ = class_logits(model, normalise(x[i:i + batch_size].float() / 255), n_classes)
        loss += F.cross_entropy(logits.float(), y[i:i + batch_size], reduction="sum").item()
        correct += (logits.argmax(-1) == y[i:i + batch_size]).sum().item()
    return loss / len(x), correct / len(x)


def train_epoch(model, x, y, opt, sched, batch_size, n_classes, gen, aux_weight=0.01, use_augment=True):
    model.train()
    order = torch.randperm(len(x), device=x.device, generator=gen)
    n_full = len(x) // batch_size * batch_size or len(x)                  # drop the ragged last batch
    stats = torch.zeros(2, device=x.device)
    for i in range(0, n_full, batch_size):
        idx = order[i:i + batch_size]
        xb = x[idx].float() / 255
        xb = normalise(augment(xb, gen) if use_augment else xb)
        logits, aux = class_logits(model, xb, n_classes)
        loss = F.cross_entropy(logits.float(), y[idx])
        if aux:
            loss = loss + aux_weight * sum(v.mean() for v in aux.values() if torch.is_tensor(v) and v.numel() > 0)
        opt.zero_grad(set_to_none=True)
        loss.backward()
        torch.nn.utils.clip_grad_norm_(model.parameters(), 1.0)
        opt.step()
        if sched is not None:
            sched.step()
        stats += torch.stack([loss.detach() * len(idx), (logits.argmax(-1) == y[idx]).sum()])
    loss, correct = stats.tolist()                                       # one host read per epoch
    return loss / n_full, correct / n_full


@torch.no_grad()
def refresh_batch_norm(model, x, batch_size):
    """Recompute BatchNorm running statistics of an averaged model from the (unaugmented) training images."""
    bns = [m for m in model.modules() if isinstance(m, torch.nn.modules.batchnorm._BatchNorm)]
    if not bns:
        return
    for m in bns:
        m.reset_running_stats()
        m.momentum = None
    model.train()
    for i in range(0, len(x), batch_size):
        model(normalise(x[i:i + batch_size].float() / 255))


def main(argv=None):
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--dataset", default="mnist", choices=sorted(DATASET_CONFIGS))
    ap.add_argument("--source", default="torchvision", help="torchvision | synthetic | npz:<path>")
    ap.add_argument("--data-dir", default="data")
    ap.add_argument("--n-train", type=int, default=4096, help="synthetic source only")
    ap.add_argument("--n-val", type=int, default=1024, help="synthetic source only")
    ap.add_argument("--epochs", type=int, default=50)
    ap.add_argument("--lr", type=float, default=1e-3)
    ap.add_argument("--batch-size", type=int, default=128)
    ap.add_argument("--eval-batch-size", type=int, default=256)
    ap.add_argument("--seed", type=int, default=42)
    ap.add_argument("--output", default=None)
    ap.add_argument("--resume", default=None)
    ap.add_argument("--adaptive", action="store_true")
    ap.add_argument("--n-branches", type=int, default=3)
    ap.add_argument("--n-layers", type=int, default=2)
    ap.add_argument("--width", type=int, default=64)
    ap.add_argument("--grayscale", action="store_true")
    ap.add_argument("--no-attention", action="store_true")
    ap.add_argument("--no-augment", action="store_true")
    ap.add_argument("--swa", action="store_true")
    ap.add_argument("--swa-start", type=float, default=0.75, help="fraction of the epochs after which averaging starts")
    ap.add_argument("--swa-lr", type=float, default=None)
    ap.add_argument("--aux-weight", type=float, default=0.01)
    ap.add_argument("--device", default="cuda" if torch.cuda.is_available() else "cpu")
    a = ap.parse_args(argv)
    torch.manual_seed(a.seed)
    device = torch.device(a.device)
    ds = DATASET_CONFIGS[a.dataset]
    out = Path(a.output or f"models/{a.dataset}_2d_model.pt")
    xa, ya, xb, yb = load_arrays(ds, a.source, a.data_dir, a.n_train, a.n_val, a.seed)
    if a.grayscale:
        xa, xb = to_gray(xa), to_gray(xb)
    xa, ya, xb, yb = xa.to(device), ya.to(device), xb.to(device), yb.to(device)
    model, cfg = build_model(a, ds, xa.shape[1])
    model = model.to(device)
    opt = torch.optim.AdamW(model.parameters(), lr=a.lr, weight_decay=0.01, fused=device.type == "cuda")
    steps_per_epoch = max(len(xa) // a.batch_size, 1)
    swa_start = int(a.epochs * a.swa_start) if a.swa else a.epochs
    sched = torch.optim.lr_scheduler.OneCycleLR(opt, max_lr=a.lr, total_steps=max(swa_start * steps_per_epoch, 2), pct_start=0.1)
    swa_model = AveragedModel(model) if a.swa else None
    swa_sched = SWALR(opt, swa_lr=a.swa_lr or a.lr * 0.1, anneal_epochs=1) if a.swa else None
    start, best_acc, history = 0, 0.0, []
    if a.resume:
        ck = load_checkpoint(a.resume, map_location=device)
        model.load_state_dict(ck["state_dict"])
        opt.load_state_dict(ck["optimizer"])
        sched.load_state_dict(ck["scheduler"])
        if swa_model is not None and ck.get("swa_state") is not None:
            swa_model.load_state_dict(ck["swa_state"])
        start, best_acc, history = ck["epoch"], ck.get("best_acc", 0.0), ck.get("history", [])
    gen = torch.Generator(device=device).manual_seed(a.seed + start)
    t0 = time.perf_counter()
    for epoch in range(start, a.epochs):
        in_swa = a.swa and epoch >= swa_start
        tl, ta = train_epoch(model, xa, ya, opt, None if in_swa else sched, a.batch_size, ds.n_classes, gen, a.aux_weight, not a.no_augment)
        if in_swa:
            swa_model.update_parameters(model)
            swa_sched.step()
        vl, va = evaluate(model, xb, yb, a.eval_batch_size, ds.n_classes)
        history.append({"epoch": epoch + 1, "train_loss": tl, "train_acc": ta, "val_loss": vl, "val_acc": va, "swa": in_swa})
        print(f"epoch {epoch + 1}/{a.epochs} train loss={tl:.4f} acc={ta:.4f} | val loss={vl:.4f} acc={va:.4f}{' (swa)' if in_swa else ''}", flush=True)
        state = {"model_config": cfg.to_dict(), "state_dict": model.state_dict(), "optimizer": opt.state_dict(), "scheduler": sched.state_dict(),
                 "swa_state": swa_model.state_dict() if swa_model is not None else None, "epoch": epoch + 1, "best_acc": max(best_acc, va),
                 "history": history, "dataset": a.dataset}
        out.parent.mkdir(parents=True, exist_ok=True)
        save_checkpoint(state, out.with_suffix(".last.pt"))
        if va > best_acc:
            best_acc = va
            save_checkpoint(state, out)
    swa_acc = None
    if a.swa and a.epochs > swa_start:
        refresh_batch_norm(swa_model, xa, a.eval_batch_size)
        _, swa_acc = evaluate(swa_model.module, xb, yb, a.eval_batch_size, ds.n_classes)
        print(f"SWA val acc={swa_acc:.4f}", flush=True)
        if swa_acc >= best_acc:
            best_acc = swa_acc
            save_checkpoint({"model_config": cfg.to_dict(), "state_dict": swa_model.module.state_dict(), "epoch": a.epochs, "best_acc": best_acc,
                             "history": history, "dataset": a.dataset, "swa": True}, out)
    summary = {"dataset": a.dataset, "parameters": sum(p.numel() for p in model.parameters()), "best_acc": best_acc, "swa_acc": swa_acc,
               "epochs": a.epochs, "seconds": time.perf_counter() - t0, "images_per_s": len(xa) * (a.epochs - start) / max(time.perf_counter() - t0, 1e-9)}
    print(json.dumps(summary))
    return summary


if __name__ == "__main__":
    main()
