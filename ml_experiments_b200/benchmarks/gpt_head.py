"""The current speedrun GPT (11 layers, d 768, 6 x 128 heads, parameter banks, paired heads, bigram hash embedding, fp8
transposed lm_head, multi-token loss) trained with ``NorMuonAndAdam`` on synthetic tokens.

    python -m ml_experiments_b200.benchmarks.gpt_head [--tokens 49152 --steps 10]
    torchrun --nproc-per-node N -m ml_experiments_b200.benchmarks.gpt_head ...

One step = forward + backward of one ``--tokens``-token sequence per rank (documents of 1024 tokens, windows 5 / 11
blocks as in the last phase of the reference schedule), then ``NorMuonAndAdam.step`` with the reference's parameter
table, scatter and work order (modded-nanogpt/train_gpt.py:1574-1622): NorMuon on the attention / MLP banks (Polar
Express on tcgen05 GEMMs, variance-reduction and cautious-update kernels), Adam with cautious weight decay on
everything else; with several ranks the sharded entries are reduce-scattered / all-gathered and the replicated ones
all-reduced.
"""
from __future__ import annotations

import argparse

import torch

from .common import emit, init_dist, timed_steps

PARAM_TABLE = {
    "attn": dict(optim="normuon", comms="sharded"),
    "mlp": dict(optim="normuon", comms="sharded", per_matrix_lr_mul=None),
    "scalars": dict(optim="adam", comms="replicated", adam_betas=(0.9, 0.99), lr_mul=5.0, wd_mul=0.0),
    **{f"ve{i}": dict(optim="adam", comms="sharded", adam_betas=(0.75, 0.95), lr_mul=75.0, wd_mul=5.0) for i in range(5)},
    "bigram_embed": dict(optim="adam", comms="sharded", adam_betas=(0.75, 0.95), lr_mul=75.0, wd_mul=5.0),
    "smear_gate": dict(optim="adam", comms="replicated", adam_betas=(0.9, 0.99), lr_mul=0.01, wd_mul=0.0),
    "skip_gate": dict(optim="adam", comms="replicated", adam_betas=(0.9, 0.99), lr_mul=0.05, wd_mul=0.0),
    "attn_gate_bank": dict(optim="adam", comms="replicated", adam_betas=(0.9, 0.99)),
    "ve_gate_bank": dict(optim="adam", comms="replicated", adam_betas=(0.9, 0.99)),
    "x0_lambdas": dict(optim="adam", comms="replicated", adam_betas=(0.65, 0.95), lr_mul=5.0, wd_mul=0.0),
    "lm_head": dict(optim="adam", comms="sharded", adam_betas=(0.5, 0.95), wd_mul=150.0),
    "embed": dict(optim="adam", comms="sharded", adam_betas=(0.5, 0.95), wd_mul=150.0),
}
WORK_ORDER = ["scalars", "smear_gate", "skip_gate", "attn_gate_bank", "ve_gate_bank", "x0_lambdas",
              "ve0", "ve1", "ve2", "ve3", "ve4", "bigram_embed", "lm_head", "embed", "attn", "mlp"]


def build(dev, tokens: int, world: int, vocab: int = 50304, bigram_vocab: int = 50304 * 5, fp8: bool = True):
    from ..models.gpt_head import GPT
    from ..optim.normuon import NorMuonAndAdam

    model = GPT(vocab_size=vocab, num_heads=6, head_dim=128, model_dim=768, max_seq_len=tokens, bigram_vocab_size=bigram_vocab,
                use_fp8=fp8, world_size=world).to(dev).bfloat16()
    table = {k: {a: b for a, b in v.items() if b is not None} for k, v in PARAM_TABLE.items()}
    n_mlp = model.mlp_bank.shape[0]
    table["mlp"]["per_matrix_lr_mul"] = [1.0, 2.0] * n_mlp          # the output projections take twice the rate
    opt = NorMuonAndAdam(model.named_parameters(), table, scatter_order=list(table), work_order=WORK_ORDER,
                         adam_defaults=None, normuon_defaults=None)
    return model, opt


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--tokens", type=int, default=48 * 1024)
    ap.add_argument("--steps", type=int, default=10)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--no-fp8", action="store_true")
    a = ap.parse_args()
    rank, world, local = init_dist()
    dev = torch.device("cuda", local)
    torch.manual_seed(0)
    from ..models.gpt_head import ForwardScheduleConfig

    model, opt = build(dev, a.tokens, world, fp8=not a.no_fp8)
    g = torch.Generator().manual_seed(1000 + rank)
    toks = torch.randint(0, 50257, (a.tokens + 1,), generator=g)
    toks[:-1][::1024] = 50256
    x, y = toks[:-1].to(dev), toks[1:].to(dev)
    bigram = ((x.roll(1) * 36313) ^ (x * 27191)) % model.bigram_embed.num_embeddings      # hash of (previous, current) token
    seqlens = torch.arange(0, a.tokens + 1, 1024, dtype=torch.int32, device=dev)
    cfg = ForwardScheduleConfig(mtp_weights=torch.tensor([1.0, 0.5, 0.25], device=dev), ws_short=5, ws_long=11)
    losses = []

    def step():
        loss = model(x, y, seqlens, bigram, cfg) / a.tokens
        loss.backward()
        opt.step()
        losses.append(loss.detach())

    ms = timed_steps(step, a.steps, a.warmup, world, dev)
    from ..ops.runtime import check_status

    check_status()
    first, last = float(losses[0]), float(losses[-1])
    emit(rank, impl="ours", metric="tokens/s HEAD speedrun GPT (NorMuon + Adam)", value=a.tokens * world / (ms / 1e3), unit="tokens/s",
         ms_per_step=ms, n_gpus=world, first_loss=first, final_loss=last,
         config=dict(layers=11, d_model=768, heads="6x128", tokens_per_rank=a.tokens, fp8_head=not a.no_fp8), dtype="bf16",
         data="synthetic uniform tokens, BOS every 1024")
    if not (last == last and last != first):
        raise SystemExit("the loss did not move or is not finite")


if __name__ == "__main__":
    main()
