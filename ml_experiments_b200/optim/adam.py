"""Adam with one fused element-wise kernel per parameter (fp32 moments, fp32 or bf16 parameters and gradients).

Same update rule and constructor arguments as ``torch.optim.Adam`` (the reference trainers use
``torch.optim.Adam(..., betas=(0.8, 0.95), eps=1e-10, fused=True)``); ``weight_decay`` is decoupled (AdamW style).
On CPU tensors the identical math runs in plain torch.
"""
from __future__ import annotations

import torch

from ..ops.runtime import ops
from ..utils.shadow import mark_modified, set_shadow, shadow_entries


class FusedAdam(torch.optim.Optimizer):
    def __init__(self, params, lr: float = 1e-3, betas=(0.9, 0.999), eps: float = 1e-8, weight_decay: float = 0.0,
                 fused: bool = True):
        defaults = dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay)
        super().__init__(params, defaults)

    @torch.no_grad()
    def step(self, closure=None):
        loss = None
        if closure is not None:
            with torch.enable_grad():
                loss = closure()
        for group in self.param_groups:
            b1, b2 = group["betas"]
            for p in group["params"]:
                if p.grad is None:
                    continue
                st = self.state[p]
                if not st:
                    st["step"] = 0
                    st["exp_avg"] = torch.zeros(p.shape, dtype=torch.float32, device=p.device)
                    st["exp_avg_sq"] = torch.zeros(p.shape, dtype=torch.float32, device=p.device)
                st["step"] += 1
                t = st["step"]
                bias1, bias2 = 1 - b1 ** t, 1 - b2 ** t
                lr = float(group["lr"])
                g = p.grad
                if p.is_cuda and p.is_contiguous() and g.is_contiguous() and p.dtype in (torch.float32, torch.bfloat16) \
                        and g.dtype in (torch.float32, torch.bfloat16):
                    # the kernel updates p without bumping Tensor._version: tell the shadow cache. If the forward keeps a
                    # bf16 / e4m3 copy of this parameter (the fp8 lm_head), the same kernel pass refreshes it.
                    ents = [e for e in shadow_entries(p) if e[0] in (torch.bfloat16, torch.float8_e4m3fn)
                            and e[2].is_contiguous() and e[2].shape == p.shape]
                    sh = ents[0] if len(ents) == 1 else None
                    ops().adam_step(p, g, st["exp_avg"], st["exp_avg_sq"], lr, b1, b2, group["eps"],
                                    group["weight_decay"], bias1, bias2, 1.0, None if sh is None else sh[2],
                                    1.0 if sh is None else float(sh[1]))
                    mark_modified(p)
                    if sh is not None:
                        set_shadow(p, sh[2], sh[1])
                else:
                    gf = g.float()
                    m, v = st["exp_avg"], st["exp_avg_sq"]
                    m.mul_(b1).add_(gf, alpha=1 - b1)
                    v.mul_(b2).addcmul_(gf, gf, value=1 - b2)
                    pf = p.float()
                    pf.mul_(1 - lr * group["weight_decay"])
                    pf.addcdiv_(m, v.sqrt() / (bias2 ** 0.5) + group["eps"], value=-lr / bias1)
                    p.copy_(pf)
                    mark_modified(p)
        return loss
