"""Native sparse attention, DeepSeek style (zoology/mixers/deepseek_nsa.py:74-351): three causal branches per head —
attention over MLP-compressed key/value blocks (plus learned memory slots), fine attention over the ``num_selected_blocks``
blocks with the highest compressed-attention importance (plus the query's own block, causally), and an exact sliding
window — mixed by a learned per-head sigmoid gate. The fine branch is evaluated with a block-selection mask over the full
score matrix, which gives the same result as gathering the selected blocks; rotary embedding (interleaved pairs) is
applied after the compressed branch, as in the reference."""
from __future__ import annotations

from copy import deepcopy

import torch
import torch.nn as nn
import torch.nn.functional as F


def _rope_interleaved(t, base: float = 10000.0):
    """Rotates adjacent channel pairs of ``[B, H, L, D]`` by position."""
    L, D = t.shape[-2], t.shape[-1]
    inv = 1.0 / (base ** (torch.arange(0, D, 2, device=t.device, dtype=torch.float32) / D))
    ang = torch.arange(L, device=t.device, dtype=torch.float32)[:, None] * inv
    cos, sin = ang.cos().repeat_interleave(2, -1), ang.sin().repeat_interleave(2, -1)
    x1, x2 = t[..., 0::2], t[..., 1::2]
    rot = torch.stack((-x2, x1), dim=-1).flatten(-2)
    return (t.float() * cos + rot.float() * sin).to(t.dtype)


def _grouped_attend(q, k, v, mask, scale):
    """``q [B, H, L, D]``, ``k, v [B, Hkv, J, D]``; ``mask`` broadcastable to ``[B, Hkv, G, L, J]`` -> out, scores."""
    B, H, L, D = q.shape
    G = H // k.shape[1]
    qg = q.view(B, k.shape[1], G, L, D)
    sim = torch.einsum("bhgid,bhjd->bhgij", qg, k) * scale
    if mask is not None:
        sim = sim.masked_fill(~mask, -torch.finfo(sim.dtype).max)
    out = torch.einsum("bhgij,bhjd->bhgid", sim.softmax(dim=-1), v)
    return out.reshape(B, H, L, D), sim.reshape(B, H, L, -1)


class SparseAttention(nn.Module):
    def __init__(self, d_model, num_heads, sliding_window_size, compress_block_size, selection_block_size, num_selected_blocks,
                 kv_heads=None, num_compressed_mem_kv=1, causal=False, norm=True, use_triton_kernel=False,
                 interpolated_importance_score=False, query_heads_share_selected_kv=True, compress_mlp=None,
                 compress_mlp_expand_factor=1.0, layer_idx=-1):
        super().__init__()
        dim_head = d_model // num_heads
        kv_heads = num_heads if kv_heads is None else kv_heads
        assert kv_heads <= num_heads and num_heads % kv_heads == 0 and num_compressed_mem_kv > 0 and num_selected_blocks >= 0
        self.dim, self.heads, self.kv_heads, self.dim_head = d_model, num_heads, kv_heads, dim_head
        self.num_grouped_queries, self.scale = num_heads // kv_heads, dim_head ** -0.5
        self.norm = nn.RMSNorm(d_model) if norm else nn.Identity()
        self.qkv_split = (dim_head * num_heads, dim_head * kv_heads, dim_head * kv_heads)
        self.to_qkv = nn.Linear(d_model, sum(self.qkv_split), bias=False)
        self.sliding_window_size, self.compress_block_size = sliding_window_size, compress_block_size
        self.selection_block_size, self.num_selected_blocks = selection_block_size, num_selected_blocks
        self.query_heads_share_selected_kv = query_heads_share_selected_kv
        self.compress_mem_kv = nn.Parameter(torch.zeros(2, kv_heads, num_compressed_mem_kv, dim_head))
        self.k_intrablock_positions = nn.Parameter(torch.zeros(kv_heads, compress_block_size, dim_head))
        self.v_intrablock_positions = nn.Parameter(torch.zeros(kv_heads, compress_block_size, dim_head))
        cdim = compress_block_size * dim_head
        mlp = compress_mlp if compress_mlp is not None else nn.Sequential(
            nn.Flatten(-2), nn.Linear(cdim, int(compress_mlp_expand_factor * cdim)), nn.ReLU(), nn.Linear(int(compress_mlp_expand_factor * cdim), dim_head))
        self.k_compress, self.v_compress = deepcopy(mlp), deepcopy(mlp)
        combine = nn.Linear(d_model, 3 * num_heads)
        nn.init.zeros_(combine.weight)
        combine.bias.data.copy_(torch.tensor([-2.0, -2.0, 2.0] * num_heads))
        self.to_strategy_combine = nn.Sequential(combine, nn.Sigmoid())
        self.combine_heads = nn.Linear(dim_head * num_heads, d_model, bias=False)

    def forward(self, inp, **kwargs):
        B, L, _ = inp.shape
        H, Hk, D, cb, sb, dev = self.heads, self.kv_heads, self.dim_head, self.compress_block_size, self.selection_block_size, inp.device
        assert L % cb == 0, "sequence length must be divisible by compress block size"
        W = L // cb
        inp = self.norm(inp)
        q, k, v = self.to_qkv(inp).split(self.qkv_split, dim=-1)
        q, k, v = (t.view(B, L, -1, D).transpose(1, 2) for t in (q, k, v))
        # compressed branch
        ck = self.k_compress((k + self.k_intrablock_positions.repeat(1, W, 1)).view(B, Hk, W, cb, D))
        cv = self.v_compress((v + self.v_intrablock_positions.repeat(1, W, 1)).view(B, Hk, W, cb, D))
        mem_k, mem_v = self.compress_mem_kv.unsqueeze(1).expand(2, B, -1, -1, -1)
        M = mem_k.shape[-2]
        ck, cv = torch.cat((mem_k, ck), dim=-2), torch.cat((mem_v, cv), dim=-2)
        pos = torch.arange(L, device=dev)
        ck_end = F.pad((torch.arange(W, device=dev) + 1) * cb - 1, (M, 0), value=-1)
        cmask = ck_end[None, :] < pos[:, None]                                   # a block is visible once it is complete
        compressed_out, csim = _grouped_attend(q, ck, cv, cmask, self.scale)
        q, k = _rope_interleaved(q), _rope_interleaved(k)
        # fine branch
        imp = csim[..., M:]
        n_sel = min(self.num_selected_blocks, W)
        G = self.num_grouped_queries
        if self.query_heads_share_selected_kv:
            imp = imp.view(B, Hk, G, L, W).mean(2)
        causal = pos[None, :] <= pos[:, None]
        if n_sel > 0:
            assert cb == sb, "compress and selection block sizes must match"
            imp = F.pad(imp, (1, 0), value=-1e3).softmax(dim=-1)[..., 1:]
            val, idx = imp.topk(n_sel, dim=-1)
            sel = torch.zeros_like(imp, dtype=torch.bool).scatter(-1, idx, val > 1e-10)      # [B, h, L, W]
            own = (pos[:, None] // sb) == torch.arange(W, device=dev)[None, :]
            fmask = sel.repeat_interleave(sb, dim=-1) | (own.repeat_interleave(sb, dim=-1) & causal)
            fmask = fmask.unsqueeze(2) if self.query_heads_share_selected_kv else fmask.view(B, Hk, G, L, L)
        else:
            fmask = causal
        fine_out, _ = _grouped_attend(q, k, v, fmask, self.scale)
        # sliding window branch: keys j in [i - window, i]
        wmask = causal & (pos[None, :] >= pos[:, None] - self.sliding_window_size)
        window_out, _ = _grouped_attend(q, k, v, wmask, self.scale)
        gate = self.to_strategy_combine(inp).view(B, L, H, 3).permute(0, 2, 1, 3)    # [B, H, L, 3]
        out = gate[..., 0:1] * compressed_out + gate[..., 1:2] * fine_out + gate[..., 2:3] * window_out
        return self.combine_heads(out.transpose(1, 2).reshape(B, L, H * D))

    def state_size(self, sequence_length: int = 2048):
        n = sequence_length // self.compress_block_size
        return 2 * n * self.dim + 2 * self.sliding_window_size * self.dim + 2 * self.selection_block_size * self.dim * self.num_selected_blocks
