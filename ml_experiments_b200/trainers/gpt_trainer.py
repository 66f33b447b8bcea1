"""Trainer of the "classic" modded-nanogpt configuration (GPT-2 124M, Muon + Adam, one 48x1024-token sequence per
rank per step) and of the same family at other sizes.

Follows the training section of records/track_1_short/2025-01-26_BatchSize/c44090cc-...txt:462-625: Adam
(betas 0.8/0.95, eps 1e-10) on head (lr 0.008), embeddings (0.6) and scalars (0.04); Muon (lr 0.05, momentum warm-up
0.85 -> 0.95 over 300 steps) on the hidden matrices; learning-rate multiplier 1 then linear to 0.1 over the last 40 % of
the run; sliding window growing 128 -> 1792 tokens in 128-token blocks; gradients averaged over ranks every step.
"""
from __future__ import annotations

import os
from dataclasses import dataclass

import torch
import torch.distributed as dist

from ..models.gpt import GPT, GPTConfig, next_multiple_of_n
from ..optim import FusedAdam, Muon


@dataclass
class Hyperparameters:
    train_files: str = "data/fineweb10B/fineweb_train_*.bin"
    val_files: str = "data/fineweb10B/fineweb_val_*.bin"
    val_tokens: int = 10485760
    num_iterations: int = 1770
    cooldown_frac: float = 0.4
    val_loss_every: int = 125
    seq_len: int = 48 * 1024
    val_seq_len: int = 4 * 64 * 1024
    save_checkpoint: bool = False
    head_lr: float = 0.008
    embed_lr: float = 0.6
    scalar_lr: float = 0.04
    muon_lr: float = 0.05
    muon_momentum: float = 0.95
    muon_momentum_warmup_steps: int = 300


def get_lr(step: int, hp: Hyperparameters) -> float:
    t = 1 - step / hp.num_iterations
    w = min(max(t, 0.0) / hp.cooldown_frac, 1.0)
    return w * 1.0 + (1 - w) * 0.1


def window_blocks(step: int, hp: Hyperparameters) -> int:
    """Sliding window (in 128-token blocks) at ``step``: 128 -> 1792 tokens, linear over the run."""
    return next_multiple_of_n(1728 * step / hp.num_iterations, n=128) // 128


class _NoSync:
    """Stands in for a gradient synchroniser when every parameter's averaging is fused into its optimizer kernel."""

    def sync_non_muon_grads(self):
        pass


class GPTTrainer:
    """Owns model, optimizers and (optionally) the process group; ``train_step`` runs one optimizer step."""

    def __init__(self, config: GPTConfig | None = None, hp: Hyperparameters | None = None, device="cuda",
                 rank: int = 0, world_size: int = 1, seed: int = 0, grad_sync: str = "auto", matrix_optimizer: str = "muon"):
        self.hp = hp or Hyperparameters()
        self.config = config or GPTConfig(max_seq_len=max(self.hp.seq_len, 65536))
        self.rank, self.world_size = rank, world_size
        self.device = torch.device(device)
        torch.manual_seed(seed)
        model = GPT(config=self.config).to(self.device)
        model.cast_embeddings_bf16()
        self.model = model
        if world_size > 1:
            for p in model.parameters():
                dist.broadcast(p.detach(), 0)
        hidden, embed, scalar, head = model.param_groups()
        hp_ = self.hp
        adam_groups = [dict(params=head, lr=hp_.head_lr), dict(params=embed, lr=hp_.embed_lr),
                       dict(params=scalar, lr=hp_.scalar_lr)]
        self.optimizer1 = None
        self.sharded_adam = False
        self._adam_stream = None
        self.grad_sync = grad_sync
        self.comm = None
        self.comm_mode = "single"
        if matrix_optimizer == "dion":
            from ..optim.dion import Dion

            sw = None
            if world_size > 1 and self.device.type == "cuda":
                from ..parallel import muon_dist as md
                from ..parallel.symm import SymmWorld

                try:
                    sw = SymmWorld.create(rank, world_size, self.device)
                    self.comm = md.FusedGradSync(model, hidden, sw)
                    self.comm_mode = "fused-p2p"
                except Exception:
                    self.comm = md.GradSync(model, hidden, rank, world_size)
                    self.comm_mode = "nccl"
            self.optimizer2 = Dion(hidden, lr=hp_.muon_lr * 0.2, mu=hp_.muon_momentum, rank_fraction=0.25, world=sw)
        elif world_size > 1 and self.device.type == "cuda":
            from ..parallel import muon_dist as md

            if grad_sync in ("auto", "fused"):
                try:
                    from ..parallel.symm import SymmWorld

                    sw = SymmWorld.create(rank, world_size, self.device)
                    self.optimizer2 = md.FusedDistMuon(hidden, sw, lr=hp_.muon_lr, momentum=hp_.muon_momentum)
                    if os.environ.get("B200_SHARDED_ADAM", "1") == "1":     # "0": bucket all-reduce + replicated Adam instead
                        # Adam state sharded over the ranks; reduce-scatter, update and all-gather are one kernel per
                        # table, the head's launched from backward as soon as its gradient exists
                        from ..parallel.adam_dist import ShardedAdam

                        self.optimizer1 = ShardedAdam(adam_groups, sw, betas=(0.8, 0.95), eps=1e-10,
                                                      max_blocks=int(os.environ.get("B200_ADAM_BLOCKS", "96")))
                        self.sharded_adam = True
                        model._grad_out = self.optimizer1.grad_views
                        self._head_seg = self.optimizer1.segment_of(model.lm_head.weight)
                        self._adam_stream = torch.cuda.Stream(self.device)
                        self.comm = _NoSync()
                    else:
                        self.comm = md.FusedGradSync(model, hidden, sw)
                    self.comm_mode = "fused-p2p"
                except Exception as e:  # symmetric memory unavailable: NCCL plumbing with the same work split
                    if grad_sync == "fused":
                        raise
                    if rank == 0:
                        print(f"[gpt_trainer] fused peer-memory path unavailable ({type(e).__name__}: {e}); using NCCL")
                    self.comm = None
            if self.comm is None:
                self.comm = md.GradSync(model, hidden, rank, world_size)
                self.optimizer2 = md.DistMuon(hidden, self.comm, lr=hp_.muon_lr, momentum=hp_.muon_momentum)
                self.comm_mode = "nccl"
        else:
            self.optimizer2 = Muon(hidden, lr=hp_.muon_lr, momentum=hp_.muon_momentum, rank=rank, world_size=world_size)
        if self.optimizer1 is None:
            self.optimizer1 = FusedAdam(adam_groups, betas=(0.8, 0.95), eps=1e-10)
        self.optimizers = [self.optimizer1, self.optimizer2]
        # the Muon forms that keep their gradients in stacks let the weight-gradient GEMMs write there directly
        if self.device.type == "cuda" and hasattr(self.optimizer2, "grad_views") and os.environ.get("B200_GRAD_IN_PLACE", "1") == "1":
            views = dict(getattr(model, "_grad_out", None) or {})
            views.update(self.optimizer2.grad_views())
            model._grad_out = views
        # B200_OVERLAP_SYNC=1 runs the bucket all-reduce on a side stream beside the Muon step (measured: no gain at 2 or 8 GPUs)
        # (only beside the fused Muon step: Dion's own all-reduces share the bucket all-reduce's flag channel and counter)
        self.overlap_sync = (self.comm_mode == "fused-p2p" and hasattr(self.comm, "start_async")
                             and type(self.optimizer2).__name__ == "FusedDistMuon"
                             and os.environ.get("B200_OVERLAP_SYNC", "0") == "1")
        for opt in self.optimizers:
            for g in opt.param_groups:
                g["initial_lr"] = g["lr"]
        self.step = 0

    # ------------------------------------------------------------------------------------------
    def _sync_grads(self):
        if self.world_size == 1:
            return
        if self.comm is not None:
            self.comm.sync_non_muon_grads()
            return
        for p in self.model.parameters():
            if p.grad is not None:
                dist.all_reduce(p.grad, op=dist.ReduceOp.AVG)

    def train_step(self, inputs, targets, window: int | None = None) -> torch.Tensor:
        """One optimizer step on a flat token sequence. Host tensors are copied to the device (non-blocking).

        ``inputs`` / ``targets`` may also be equally long lists of sequences: their gradients are accumulated and
        averaged before the one optimizer step (the reference's single-GPU runs reach the 8-GPU batch this way:
        records/track_1_short/2026-01-10_FusedLinearReLUSquare/single_gpu_run.txt, grad-accum 8)."""
        hp = self.hp
        w = window_blocks(self.step, hp) if window is None else window
        micro = list(zip(inputs, targets)) if isinstance(inputs, (list, tuple)) else [(inputs, targets)]
        # hyper-parameters of this step first: with the sharded Adam the head's update is launched from inside backward
        frac = min(self.step / hp.muon_momentum_warmup_steps, 1)
        for g in self.optimizer2.param_groups:
            g["momentum"] = (1 - frac) * 0.85 + frac * 0.95
        lr_mul = get_lr(min(self.step, hp.num_iterations), hp)
        for opt in self.optimizers:
            for g in opt.param_groups:
                g["lr"] = g["initial_lr"] * lr_mul
        if self.sharded_adam and len(micro) == 1 and os.environ.get("B200_ADAM_EARLY", "1") == "1":
            self.model._grad_hooks = {id(self.model.lm_head.weight): self._head_grad_ready}
        loss = None
        for x, y in micro:
            if x.device != self.device:
                x = x.to(self.device, non_blocking=True)
                y = y.to(self.device, non_blocking=True)
            if y.dtype != torch.int64:
                y = y.to(torch.int64)
            l = self.model.loss_and_grad(x, y, w)
            loss = l if loss is None else loss + l
        self.model._grad_hooks = None
        if len(micro) > 1:
            loss = loss / len(micro)
            torch._foreach_mul_([p.grad for p in self.model.parameters() if p.grad is not None], 1.0 / len(micro))
        if self.sharded_adam:
            # the remaining tables (embeddings, scalars) go out on the side stream beside the Muon step: link-bound
            # copies with a capped grid next to the GEMM-bound Newton-Schulz iterations
            cur = torch.cuda.current_stream(self.device)
            ready = torch.cuda.Event()
            ready.record(cur)
            with torch.cuda.stream(self._adam_stream):
                self._adam_stream.wait_event(ready)
                for i in range(len(self.optimizer1.segments)):
                    if i not in self.optimizer1._launched:
                        self.optimizer1.launch(i)
            self.optimizer2.step()
            cur.wait_stream(self._adam_stream)
            self.optimizer1.finish()
        elif self.overlap_sync:
            # the all-reduce of the embedding / head gradients (link-bound) runs beside the Muon step (GEMM-bound)
            self.comm.start_async()
            self.optimizer2.step()
            self.comm.join_async()
            self.optimizer1.step()
        else:
            self._sync_grads()
            for opt in self.optimizers:
                opt.step()
        self.model.zero_grad(set_to_none=True)
        self.step += 1
        return loss

    def _head_grad_ready(self, p, g):
        """Called from backward when the head's weight gradient is complete: its fused reduce-scatter + Adam +
        all-gather starts on the side stream right away and runs under the rest of backward."""
        opt = self.optimizer1
        view = opt.grad_views[id(p)]
        if g.data_ptr() != view.data_ptr():
            view.copy_(g.view_as(view))
        cur = torch.cuda.current_stream(self.device)
        ready = torch.cuda.Event()
        ready.record(cur)
        with torch.cuda.stream(self._adam_stream):
            self._adam_stream.wait_event(ready)
            opt.launch(self._head_seg, early=True)

    @torch.no_grad()
    def eval_loss(self, inputs: torch.Tensor, targets: torch.Tensor, window: int) -> torch.Tensor:
        self.model.eval()
        loss = self.model(inputs.to(self.device), targets.to(self.device).long(), window)
        self.model.train()
        if self.world_size > 1:
            dist.all_reduce(loss, op=dist.ReduceOp.AVG)
        return loss

    def state_dict(self):
        return dict(step=self.step, model=self.model.state_dict(),
                    optimizers=[opt.state_dict() for opt in self.optimizers])

    def load_state_dict(self, sd):
        self.step = sd["step"]
        with torch.no_grad():
            # copy into the existing storage: the distributed Muon keeps its matrices in banked buffers
            for n, p in self.model.state_dict().items():
                p.copy_(sd["model"][n])
        from ..utils.shadow import mark_modified

        for p in self.model.parameters():
            mark_modified(p)
        for opt, s in zip(self.optimizers, sd["optimizers"]):
            opt.load_state_dict(s)

    # -- checkpoints of a distributed run: the replicated part once, the sharded Muon momentum from every rank
    def save_checkpoint(self, path) -> None:
        """Every rank must call this. Rank 0 writes ``path`` (step, model, replicated optimizer state); each rank
        writes ``path.rank{r}`` with its slice of the Muon momentum (which lives outside ``Optimizer.state``)."""
        from ..utils.checkpoint import save_sharded

        shard, rows = {}, {}
        for opt in self.optimizers:
            if hasattr(opt, "sharded_state"):
                shard.update(opt.sharded_state())
                rows.update(opt.sharded_rows())
        sd = self.state_dict()
        if any(k.startswith("mom_") for k in shard):
            # the momentum is saved through the shards; drop per-parameter views of the same buffers
            sd["optimizers"][1] = dict(sd["optimizers"][1], state={})
        save_sharded(sd, {k: v.cpu() for k, v in shard.items()}, path, self.rank, self.world_size, rows)

    def load_checkpoint(self, path) -> None:
        """Counterpart of :meth:`save_checkpoint`; the world size may differ from the one that saved."""
        from ..utils.checkpoint import load_sharded

        rep, shard = load_sharded(path, self.rank, self.world_size)
        self.load_state_dict(rep)
        shard = {k: v.to(self.device) for k, v in shard.items()}
        for opt in self.optimizers:
            if shard and hasattr(opt, "load_sharded_state"):
                opt.load_sharded_state(shard)


def synthetic_batch(seq_len: int, vocab: int = 50257, doc_len: int = 1024, seed: int = 0, pin: bool = True):
    """Uniform random token ids with a BOS token every ``doc_len`` positions (host tensors, optionally pinned)."""
    g = torch.Generator().manual_seed(seed)
    toks = torch.randint(0, vocab, (seq_len + 1,), generator=g, dtype=torch.int32)
    toks[:-1][::doc_len] = 50256
    inputs = toks[:-1].clone()
    targets = toks[1:].to(torch.int64)
    if pin and torch.cuda.is_available():
        inputs, targets = inputs.pin_memory(), targets.pin_memory()
    return inputs, targets


def init_distributed():
    """Reads the torchrun environment; returns ``(rank, local_rank, world_size)`` after creating the NCCL group."""
    rank = int(os.environ.get("RANK", 0))
    world = int(os.environ.get("WORLD_SIZE", 1))
    local = int(os.environ.get("LOCAL_RANK", 0))
    if world > 1 and not dist.is_initialized():
        torch.cuda.set_device(local)
        dist.init_process_group(backend="nccl", device_id=torch.device("cuda", local))
    return rank, local, world
