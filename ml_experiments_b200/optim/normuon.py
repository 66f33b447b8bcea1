"""NorMuon + Adam in one optimizer with explicit communication scheduling (the HEAD modded-nanogpt optimizer), and
the medium-track ``NorMuon`` / ``DistAdam`` pair.

Reference: ``NorMuonAndAdam`` (modded-nanogpt/train_gpt.py:201-775): a ``param_table`` gives every labelled parameter
its optimizer (``normuon`` / ``adam``), its communication pattern (``none`` / ``replicated`` = all-reduce /
``sharded`` = reduce-scatter + all-gather), betas and lr / wd multipliers; ``step`` launches every reduction first
(``scatter_order``), then updates label by label (``work_order``) and launches the all-gathers, then waits. The update
rules restated here:

* Adam: fp32 moments, bias correction folded into the step size, *cautious* weight decay (decay only where update and
  parameter agree in sign);
* NorMuon: fp32 momentum ``lerp`` + Nesterov ``lerp``, Polar-Express orthogonalisation (5 GEMM triples), variance
  reduction with a low-rank second moment along the longer side, cautious weight decay, and for bf16 parameters an
  extra uint16 "mantissa" buffer so that the parameter effectively carries fp32 precision.

``DistAdam`` (modded-nanogpt/train_gpt_medium.py:715-834) registers post-accumulate-grad hooks that start the
gradient reduce-scatter (all-reduce for tiny tensors) while backward is still running.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field

import torch
import torch.distributed as dist

from ..ops.newton_schulz import POLAR_EXPRESS_COEFFS, newton_schulz_, newton_schulz_torch


# ---------------------------------------------------------------------------------------------------- update rules
def polar_express(G: torch.Tensor) -> torch.Tensor:
    """Orthogonalise the (batched) matrix ``G``; bf16 result. tcgen05 GEMMs on CUDA, plain torch elsewhere."""
    if G.is_cuda and G.dim() >= 2 and all(d % 8 == 0 for d in G.shape[-2:]):
        X = G.reshape(-1, *G.shape[-2:]).to(torch.bfloat16)
        X = X / (X.float().norm(dim=(-2, -1), keepdim=True) * 1.02 + 1e-6).to(torch.bfloat16)
        return newton_schulz_(X.contiguous(), POLAR_EXPRESS_COEFFS).reshape(G.shape)
    return newton_schulz_torch(G, POLAR_EXPRESS_COEFFS, eps=1e-6, norm_scale=1.02)


def _reshape_hint(p):
    """The bank's optimizer view: the reference hangs a tuple named ``reshape`` on the parameter (shadowing the tensor
    method of that name; modded-nanogpt/train_gpt.py:1125); ``reshape_to`` is accepted as well."""
    for name in ("reshape", "reshape_to"):
        hint = getattr(p, name, None)
        if isinstance(hint, (tuple, list)):
            return tuple(hint)
    return None


_vector_cache: dict = {}


def _device_vector(values: tuple, repeat: int, device) -> torch.Tensor:
    """Per-matrix multipliers as a device vector; the few distinct tuples of a schedule are uploaded once each."""
    key = (values, repeat, str(device))
    t = _vector_cache.get(key)
    if t is None:
        if len(_vector_cache) > 4096:
            _vector_cache.clear()
        t = torch.tensor(values, dtype=torch.float32).repeat_interleave(repeat).to(device)
        _vector_cache[key] = t
    return t


def _cuda_stack(t: torch.Tensor) -> bool:
    return t.is_cuda and t.dim() >= 2 and t.is_contiguous() and t.dtype in (torch.bfloat16, torch.float32)


def normuon_step_(p: torch.Tensor, mantissa, v: torch.Tensor, second_momentum: torch.Tensor, beta2: float, red_dim: int,
                  lr, wd_lr) -> None:
    """Variance reduction of ``v`` and the cautious update of ``p`` in one go. On CUDA this is three kernels
    (sums of squares, per-matrix scale, fused scale + decay + step: ``csrc/fused/normuon.cu``) and the rescaled update is
    never written to memory; elsewhere it is :func:`normuon_variance_reduction` + :func:`cautious_update_`.
    ``lr`` / ``wd_lr``: floats, or per-matrix lists for a stack whose matrices have different multipliers."""
    per_matrix = isinstance(lr, (list, tuple))
    if _cuda_stack(v) and _cuda_stack(p) and second_momentum.is_cuda and second_momentum.dtype == torch.float32:
        from ..ops.runtime import ops

        o = ops()
        v3 = v.reshape(-1, *v.shape[-2:])
        p3 = p.reshape(-1, *p.shape[-2:])
        red_cols = red_dim in (-1, v.dim() - 1)
        stat = torch.empty(second_momentum.shape, dtype=torch.float32, device=v.device)
        o.normuon_scales(v3, stat, second_momentum, red_cols, float(beta2))
        m16 = None if mantissa is None else mantissa.view(torch.int16) if mantissa.element_size() == 2 else None
        if mantissa is not None and m16 is None:
            raise TypeError("the mantissa buffer of a bf16 parameter must be a 16-bit integer tensor on CUDA")
        lr_t = wd_t = None
        if per_matrix:      # one value per leading index of p; a leading index may hold several matrices (4-D banks)
            rep = p3.shape[0] // len(lr)
            assert rep * len(lr) == p3.shape[0], (p.shape, len(lr))
            lr_t = _device_vector(tuple(lr), rep, v.device)
            wd_t = _device_vector(tuple(wd_lr), rep, v.device)
        o.normuon_update(p3, m16, v3, stat.reshape(-1), red_cols, 0.0 if per_matrix else float(lr),
                         0.0 if per_matrix else float(wd_lr), lr_t, wd_t)
        return
    v = normuon_variance_reduction(v, second_momentum, beta2, red_dim)
    if per_matrix:
        for i in range(p.shape[0]):
            cautious_update_(p[i], None if mantissa is None else mantissa[i], v[i], lr[i], wd_lr[i])
    else:
        cautious_update_(p, mantissa, v, lr, wd_lr)


def normuon_variance_reduction(v: torch.Tensor, second_momentum: torch.Tensor, beta2: float, red_dim: int) -> torch.Tensor:
    """Rescales rows (or columns) of the orthogonalised update by a running second moment while keeping its norm."""
    v_mean = v.float().square().mean(dim=red_dim, keepdim=True)
    n = v.size(red_dim)
    v_norm = (v_mean.sum(dim=(-2, -1), keepdim=True) * n).sqrt()
    second_momentum.lerp_(v_mean.to(second_momentum.dtype), 1 - beta2)
    step = second_momentum.clamp_min(1e-10).rsqrt()
    v_norm_new = ((v_mean * n) * step.float().square()).sum(dim=(-2, -1), keepdim=True).sqrt()
    return v * (step * (v_norm / v_norm_new.clamp_min(1e-10))).to(v.dtype)


def cautious_update_(p: torch.Tensor, mantissa: torch.Tensor | None, upd: torch.Tensor, lr: float, wd_lr: float) -> None:
    """``p -= wd_lr * p * [upd * p >= 0] + lr * upd`` in fp32. For bf16 ``p`` the low 16 bits live in ``mantissa``."""
    u = upd.float()
    if p.dtype == torch.bfloat16 and mantissa is not None:
        raw = (p.view(torch.int16).to(torch.int32) << 16) | (mantissa.to(torch.int32) & 0xFFFF)
        pf = raw.view(torch.float32)
        pf = pf - pf * ((u * pf) >= 0) * wd_lr - u * lr
        raw = pf.view(torch.int32)
        p.copy_((raw >> 16).to(torch.int16).view(torch.bfloat16))
        mantissa.copy_((raw & 0xFFFF).to(torch.int32).to(mantissa.dtype))
    else:
        pf = p.float()
        p.copy_((pf - pf * ((u * pf) >= 0) * wd_lr - u * lr).to(p.dtype))


def adam_cautious_(p, g, exp_avg, exp_avg_sq, beta1, beta2, eps, step_size, wd_lr) -> None:
    """Adam step with the decay applied only where it agrees in sign with the update. One kernel on CUDA
    (``csrc/fused/normuon.cu::adam_cautious_kernel``: p and g bf16 or fp32, fp32 moments), the operator chain elsewhere."""
    if (p.is_cuda and p.is_contiguous() and g.is_contiguous() and p.dtype in (torch.bfloat16, torch.float32)
            and g.dtype in (torch.bfloat16, torch.float32) and exp_avg.dtype == torch.float32 and exp_avg.is_contiguous()
            and exp_avg_sq.dtype == torch.float32 and exp_avg_sq.is_contiguous() and g.shape == p.shape):
        from ..ops.runtime import add_launches, ops
        ops().adam_cautious(p, g, exp_avg, exp_avg_sq, float(beta1), float(beta2), float(eps), float(step_size), float(wd_lr))
        add_launches(1)
        return
    g = g.float()
    exp_avg.mul_(beta1).add_(g, alpha=1 - beta1)
    exp_avg_sq.mul_(beta2).addcmul_(g, g, value=1 - beta2)
    upd = exp_avg / (exp_avg_sq.sqrt() + eps) * step_size
    pf = p.float()
    upd = upd + pf * ((upd * pf) > 0) * wd_lr
    p.copy_((pf - upd).to(p.dtype))


# ---------------------------------------------------------------------------------------------------- combined optimizer
@dataclass
class ParamConfig:
    label: str
    optim: str = "adam"              # "adam" | "normuon"
    comms: str = "none"              # "none" | "replicated" | "sharded"
    adam_betas: tuple = (0.9, 0.99)
    lr_mul: float = 1.0
    wd_mul: float = 1.0
    lr: float = 0.0
    weight_decay: float = 0.0
    eps: float = 1e-10
    momentum: float = 0.95
    beta2: float = 0.95
    reshape: tuple | None = None     # view used for sharding / batched orthogonalisation
    per_matrix_lr_mul: list | None = None
    chunk_size: int = 0
    extra: dict = field(default_factory=dict)


class NorMuonAndAdam:
    def __init__(self, named_params, param_table: dict, scatter_order: list[str] | None = None,
                 work_order: list[str] | None = None, adam_defaults: dict | None = None,
                 normuon_defaults: dict | None = None, rank: int | None = None, world_size: int | None = None, group=None):
        self.group = group
        self.world_size = world_size if world_size is not None else (dist.get_world_size(group) if dist.is_initialized() else 1)
        self.rank = rank if rank is not None else (dist.get_rank(group) if dist.is_initialized() else 0)
        adam_defaults = dict(lr=0.008, eps=1e-10, weight_decay=0.005, **(adam_defaults or {}))
        normuon_defaults = dict(lr=0.023, momentum=0.95, beta2=0.95, weight_decay=1.2, **(normuon_defaults or {}))
        self.params: dict[str, torch.Tensor] = {}
        self.cfgs: dict[str, ParamConfig] = {}
        self.param_states: dict[str, dict] = {}
        for name, p in named_params:
            label = getattr(p, "label", name)
            if label not in param_table:
                continue
            t = dict(param_table[label])
            base = normuon_defaults if t.get("optim", "adam") == "normuon" else adam_defaults
            cfg = ParamConfig(label=label, optim=t.get("optim", "adam"), comms=t.get("comms", "none"),
                              adam_betas=tuple(t.get("adam_betas", (0.9, 0.99))), lr_mul=t.get("lr_mul", 1.0),
                              wd_mul=t.get("wd_mul", 1.0), lr=t.get("lr", base["lr"]),
                              weight_decay=t.get("weight_decay", base["weight_decay"]), eps=t.get("eps", base.get("eps", 1e-10)),
                              momentum=t.get("momentum", base.get("momentum", 0.95)), beta2=t.get("beta2", base.get("beta2", 0.95)),
                              reshape=tuple(t["reshape"]) if t.get("reshape") else _reshape_hint(p),
                              per_matrix_lr_mul=t.get("per_matrix_lr_mul"))
            if self.world_size == 1:
                cfg.comms = "none"
            self.params[label], self.cfgs[label] = p, cfg
            self._init_state(label)
        self.scatter_order = [l for l in (scatter_order or list(self.params)) if l in self.params]
        self.work_order = [l for l in (work_order or list(self.params)) if l in self.params]
        self._step = 0

    # ------------------------------------------------------------------------------------------ state
    def _view(self, label: str) -> torch.Tensor:
        p, cfg = self.params[label], self.cfgs[label]
        return p.data.view(cfg.reshape) if cfg.reshape else p.data

    def _shard(self, label: str, t: torch.Tensor) -> torch.Tensor:
        cfg = self.cfgs[label]
        if cfg.comms != "sharded":
            return t
        return t[self.rank * cfg.chunk_size:(self.rank + 1) * cfg.chunk_size]

    def _init_state(self, label: str) -> None:
        cfg = self.cfgs[label]
        v = self._view(label)
        if cfg.comms == "sharded":
            assert v.shape[0] % self.world_size == 0, f"{label}: dim 0 ({v.shape[0]}) must divide by world size"
            cfg.chunk_size = v.shape[0] // self.world_size
        else:
            cfg.chunk_size = v.shape[0] if v.dim() > 0 else 1
        s = self._shard(label, v)
        st: dict = {}
        if cfg.optim == "adam":
            st["exp_avg"] = torch.zeros_like(s, dtype=torch.float32)
            st["exp_avg_sq"] = torch.zeros_like(s, dtype=torch.float32)
            st["step"] = 0
        else:
            st["momentum_buffer"] = torch.zeros_like(s, dtype=torch.float32)
            red = -1 if s.shape[-2] >= s.shape[-1] else -2
            shp = list(s.shape)
            shp[red] = 1
            st["second_momentum_buffer"] = torch.zeros(shp, dtype=torch.float32, device=s.device)
            st["red_dim"] = red
            if s.dtype == torch.bfloat16:
                st["mantissa"] = torch.zeros_like(s, dtype=torch.int16)
        self.param_states[label] = st

    # ------------------------------------------------------------------------------------------ communication
    def _launch_reduce(self, label: str):
        cfg, p = self.cfgs[label], self.params[label]
        g = p.grad
        if g is None or cfg.comms == "none":
            return None, (None if g is None else (g.view(cfg.reshape) if cfg.reshape else g))
        if cfg.comms == "replicated":
            return dist.all_reduce(g, op=dist.ReduceOp.AVG, group=self.group, async_op=True), g.view(cfg.reshape) if cfg.reshape else g
        gv = g.view(cfg.reshape) if cfg.reshape else g
        chunk = torch.empty_like(gv[: cfg.chunk_size])
        w = dist.reduce_scatter_tensor(chunk, gv.contiguous(), op=dist.ReduceOp.AVG, group=self.group, async_op=True)
        return w, chunk

    def _launch_gather(self, label: str):
        cfg = self.cfgs[label]
        if cfg.comms != "sharded":
            return None
        full = self._view(label)
        return dist.all_gather_into_tensor(full, self._shard(label, full).contiguous(), group=self.group, async_op=True)

    # ------------------------------------------------------------------------------------------ updates
    def _adam(self, label: str, g: torch.Tensor) -> None:
        cfg, st = self.cfgs[label], self.param_states[label]
        st["step"] += 1
        b1, b2 = cfg.adam_betas
        t = st["step"]
        lr = cfg.lr * cfg.lr_mul
        step_size = lr * math.sqrt(1 - b2 ** t) / (1 - b1 ** t)
        p_slice = self._shard(label, self._view(label))
        # the decay is scheduled by the learning rate twice: lr_eff**2 * weight_decay * wd_mul
        # (modded-nanogpt/train_gpt.py:658-672)
        adam_cautious_(p_slice, g, st["exp_avg"], st["exp_avg_sq"], b1, b2, cfg.eps, step_size,
                       lr * lr * cfg.weight_decay * cfg.wd_mul)

    def _normuon(self, label: str, g: torch.Tensor) -> None:
        cfg, st = self.cfgs[label], self.param_states[label]
        g = g.float()
        st["momentum_buffer"].lerp_(g, 1 - cfg.momentum)
        u = g.lerp(st["momentum_buffer"], cfg.momentum)
        v = polar_express(u)
        p_slice = self._shard(label, self._view(label))
        # p -= p * mask * (wd_mul * wd * lr) * lr_eff + v * lr_eff (modded-nanogpt/train_gpt.py:708-760): the decay
        # coefficient carries the effective learning rate of the matrix as well
        wd = cfg.wd_mul * cfg.weight_decay * cfg.lr
        if cfg.per_matrix_lr_mul is not None:
            first = self.rank * cfg.chunk_size if cfg.comms == "sharded" else 0
            lrs = [cfg.lr * cfg.lr_mul * cfg.per_matrix_lr_mul[first + i] for i in range(p_slice.shape[0])]
            normuon_step_(p_slice, st.get("mantissa"), v, st["second_momentum_buffer"], cfg.beta2, st["red_dim"], lrs,
                          [wd * l for l in lrs])
        else:
            lr_eff = cfg.lr * cfg.lr_mul
            normuon_step_(p_slice, st.get("mantissa"), v, st["second_momentum_buffer"], cfg.beta2, st["red_dim"], lr_eff,
                          wd * lr_eff)

    @torch.no_grad()
    def step(self, do_adam: bool = True) -> None:
        self._step += 1
        pending = {}
        for label in self.scatter_order:
            if self.cfgs[label].optim == "adam" and not do_adam:
                continue
            pending[label] = self._launch_reduce(label)
        gathers = []
        for label in self.work_order:
            if label not in pending:
                continue
            work, g = pending[label]
            if work is not None:
                work.wait()
            if g is None:
                continue
            (self._adam if self.cfgs[label].optim == "adam" else self._normuon)(label, g)
            w = self._launch_gather(label)
            if w is not None:
                gathers.append(w)
        for w in gathers:
            w.wait()
        for label in pending:
            self.params[label].grad = None

    def zero_grad(self, set_to_none: bool = True) -> None:
        for p in self.params.values():
            p.grad = None

    # ------------------------------------------------------------------------------------------ checkpoint
    def state_dict(self) -> dict:
        """Per-rank state: sharded entries hold this rank's slice only (save one file per rank, or gather)."""
        return {"param_states": {k: {n: (t.clone() if torch.is_tensor(t) else t) for n, t in st.items()}
                                 for k, st in self.param_states.items()},
                "param_cfgs": {k: vars(c).copy() for k, c in self.cfgs.items()}, "step": self._step,
                "rank": self.rank, "world_size": self.world_size}

    def load_state_dict(self, sd: dict) -> None:
        for k, st in sd["param_states"].items():
            if k in self.param_states:
                for n, t in st.items():
                    if torch.is_tensor(t):
                        self.param_states[k][n].copy_(t)
                    else:
                        self.param_states[k][n] = t
        self._step = sd.get("step", 0)

    def reset(self) -> None:
        for label in self.params:
            self._init_state(label)
        self._step = 0


# ---------------------------------------------------------------------------------------------------- medium-track pair
class NorMuon(torch.optim.Optimizer):
    """``torch.optim.Optimizer`` flavour: gradients of equally shaped parameters are stacked, reduce-scattered,
    orthogonalised on the owning rank and all-gathered (modded-nanogpt/train_gpt_medium.py:454-712)."""

    def __init__(self, params, lr=0.02, weight_decay=0.01, momentum=0.95, beta2=0.95, group=None):
        super().__init__([*params], dict(lr=lr, weight_decay=weight_decay, momentum=momentum, beta2=beta2))
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0

    @torch.no_grad()
    def step(self, closure=None):
        for hp in self.param_groups:
            by_shape: dict = {}
            for p in hp["params"]:
                if p.grad is not None:
                    by_shape.setdefault(tuple(p.shape), []).append(p)
            for shape, plist in by_shape.items():
                W = self.world
                pad = (-len(plist)) % W
                per = (len(plist) + pad) // W
                stack = torch.stack([p.grad.float() for p in plist] + [torch.zeros_like(plist[0].grad, dtype=torch.float32)] * pad)
                if W > 1:
                    mine = torch.empty_like(stack[:per])
                    dist.reduce_scatter_tensor(mine, stack, op=dist.ReduceOp.AVG, group=self.group)
                else:
                    mine = stack
                key = ("stack", shape)
                st = self.state.setdefault(key, {})
                if not st:
                    st["momentum_buffer"] = torch.zeros_like(mine)
                    red = -1 if shape[-2] >= shape[-1] else -2
                    shp = list(mine.shape)
                    shp[red] = 1
                    st["second"], st["red"] = torch.zeros(shp, device=mine.device), red
                st["momentum_buffer"].lerp_(mine, 1 - hp["momentum"])
                u = mine.lerp(st["momentum_buffer"], hp["momentum"])
                v = normuon_variance_reduction(polar_express(u), st["second"], hp["beta2"], st["red"]).float()
                if W > 1:
                    full = torch.empty_like(stack)
                    dist.all_gather_into_tensor(full, v.contiguous(), group=self.group)
                else:
                    full = v
                scale = max(1.0, shape[-2] / shape[-1]) ** 0.5
                for i, p in enumerate(plist):
                    # eff_lr = shape_mult * lr_mul * lr ; eff_wd = wd_mul * wd * lr ; decay coefficient eff_wd * eff_lr
                    # (modded-nanogpt/train_gpt_medium.py:428-433,626-647)
                    lr_eff = scale * getattr(p, "lr_mul", 1.0) * hp["lr"]
                    wd = getattr(p, "wd_mul", 1.0) * hp["weight_decay"] * hp["lr"]
                    cautious_update_(p, None, full[i], lr_eff, wd * lr_eff)


class DistAdam(torch.optim.Optimizer):
    """Sharded Adam whose gradient reduce-scatter (all-reduce below 1024 elements) starts from
    ``post_accumulate_grad`` hooks during backward; ``step`` waits, updates the owned slice and all-gathers."""

    def __init__(self, params, lr=1e-3, betas=(0.8, 0.95), eps=1e-10, weight_decay=0.0, group=None):
        super().__init__([*params], dict(lr=lr, betas=betas, eps=eps, weight_decay=weight_decay))
        self.group = group
        self.world = dist.get_world_size(group) if dist.is_initialized() else 1
        self.rank = dist.get_rank(group) if dist.is_initialized() else 0
        self.should_sync = True
        self._pending: dict = {}
        for hp in self.param_groups:
            for p in hp["params"]:
                p.register_post_accumulate_grad_hook(self._hook)

    def _sharded(self, p) -> bool:
        return self.world > 1 and p.numel() >= 1024 and p.shape[0] % self.world == 0

    def _hook(self, p):
        if not self.should_sync or self.world == 1 or p.grad is None:
            return
        if self._sharded(p):
            per = p.shape[0] // self.world
            chunk = torch.empty_like(p.grad[:per])
            w = dist.reduce_scatter_tensor(chunk, p.grad.contiguous(), op=dist.ReduceOp.AVG, group=self.group, async_op=True)
            self._pending[p] = (w, chunk)
        else:
            self._pending[p] = (dist.all_reduce(p.grad, op=dist.ReduceOp.AVG, group=self.group, async_op=True), p.grad)

    @torch.no_grad()
    def step(self, closure=None):
        gathers = []
        for hp in self.param_groups:
            b1, b2 = hp["betas"]
            for p in hp["params"]:
                if p.grad is None:
                    continue
                if p in self._pending:
                    w, g = self._pending.pop(p)
                    w.wait()
                else:
                    g = p.grad
                sharded = self._sharded(p) and g.shape != p.shape
                per = p.shape[0] // self.world if sharded else None
                p_slice = p[self.rank * per:(self.rank + 1) * per] if sharded else p
                st = self.state[p]
                if not st:
                    st["step"] = 0
                    st["exp_avg"] = torch.zeros_like(p_slice, dtype=torch.float32)
                    st["exp_avg_sq"] = torch.zeros_like(p_slice, dtype=torch.float32)
                st["step"] += 1
                t = st["step"]
                # lr = group lr * param.lr_mul ; decay = lr * wd * wd_mul * lr (modded-nanogpt/train_gpt_medium.py:805-826)
                lr = hp["lr"] * getattr(p, "lr_mul", 1.0)
                adam_cautious_(p_slice, g, st["exp_avg"], st["exp_avg_sq"], b1, b2, hp["eps"],
                               lr * math.sqrt(1 - b2 ** t) / (1 - b1 ** t),
                               lr * lr * hp["weight_decay"] * getattr(p, "wd_mul", 1.0))
                if sharded:
                    gathers.append(dist.all_gather_into_tensor(p.data, p_slice.contiguous(), group=self.group, async_op=True))
        for w in gathers:
            w.wait()
