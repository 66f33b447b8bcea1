"""``RippleMixer``: the multi-operator Ripple attention as a sequence mixer for the recall harness
(zoology/mixers/ripple.py:18-86). The harness block already provides norm, MLP and residual, so only the operator
stack (telephone / adaptive conv / low-rank / attention / Jacobi SSM, in the order given) is exposed."""
from __future__ import annotations

import torch.nn as nn

from ...models.ripple import RippleAttention


class RippleMixer(nn.Module):
    def __init__(self, d_model: int, layer_idx: int = None, num_heads: int = 4, order: str = "tele,conv,lowrank",
                 max_kernel_size: int = None, max_seq_len: int = 8192, use_triton: bool = True, jacobi_iters: int = 2,
                 siren_conv: bool = False, dim_divisor: int = 1, differential: bool = True, embed_residual: bool = True,
                 plain_conv_size: int = 0, diffuse_se: bool = False, diff_inject: bool = False, diff_readout: bool = False,
                 bc_norm: bool = False, relu2: bool = False):
        super().__init__()
        channels = d_model // dim_divisor
        self.d_model, self.channels, self.layer_idx = d_model, channels, layer_idx
        self.proj_in = nn.Linear(d_model, channels) if dim_divisor > 1 else nn.Identity()
        self.proj_out = nn.Linear(channels, d_model) if dim_divisor > 1 else nn.Identity()
        self.attn = RippleAttention(channels=channels, num_heads=num_heads, max_kernel_size=max_kernel_size or 16, use_triton=use_triton,
                                    order=order, max_seq_len=max_seq_len, jacobi_iters=jacobi_iters, siren_conv=siren_conv,
                                    differential=differential, embed_residual=embed_residual, plain_conv_size=plain_conv_size,
                                    diffuse_se=diffuse_se, diff_inject=diff_inject, diff_readout=diff_readout, bc_norm=bc_norm, relu2=relu2)

    def forward(self, x):
        out = self.attn(self.proj_in(x))
        out = out[0] if isinstance(out, tuple) else out
        return self.proj_out(out)

    def state_size(self, sequence_length: int = 2048, **kwargs) -> int:
        return 0
