"""H3 (zoology/mixers/h3/h3.py:19-207): ``y = Q * SSM_diag(SSM_shift(K) * V)`` with both state-space maps applied as FFT
convolutions. The shift kernel (ss_kernel_shift.py:14-53) and the diagonal S4D kernel (ss_kernel_diag.py:33-185,
``diag-lin`` / ``diag-inv`` / ``diag-real`` initialisations of dplr.py:9-62, bilinear or zero-order-hold
discretisation, Vandermonde product evaluated densely) are restated here; the generic HiPPO/NPLR kernels of the S4
package are not."""
from __future__ import annotations

import math

import torch
import torch.nn as nn
import torch.nn.functional as F

from .hyena import OptimModule as _HyenaOptim


class OptimModule(_HyenaOptim):
    def register(self, name, tensor, lr=None):  # zero weight decay always (ssm_utils.py:9-20)
        super().register(name, tensor, lr=lr, wd=0.0)


def diag_init(scaling: str, N: int, H: int):
    half = N // 2
    real, imag = 0.5 * torch.ones(H, half), torch.arange(half).float().expand(H, half)
    if scaling in ("lin", "linear"):
        imag = math.pi * imag
    elif scaling in ("inv", "inverse"):
        imag = 1 / math.pi * N * (N / (1 + 2 * imag) - 1)
    elif scaling == "real":
        imag, real = 0 * imag, 1 + torch.arange(half).float().expand(H, half)
    else:
        raise NotImplementedError(scaling)
    return torch.complex(-real, imag), torch.ones(H, half, dtype=torch.cfloat)


def log_vandermonde(v, x, L):
    """``2 Re sum_n v_n exp(x_n l)`` for ``l < L``; ``v, x [..., N]`` complex."""
    l = torch.arange(L, device=x.device)
    return 2 * torch.einsum("...n,...nl->...l", v, torch.exp(x.unsqueeze(-1) * l)).real


class SSKernelDiag(OptimModule):
    def __init__(self, A, B, C, log_dt, L=None, disc="bilinear", real_type="exp", lr=None, **kwargs):
        super().__init__()
        self.L, self.disc, self.real_type = L, disc, real_type
        self.H, self.N, self.repeat, self.channels = log_dt.size(-1), A.size(-1), log_dt.size(-1) // A.size(0), C.shape[0]
        self.C = nn.Parameter(torch.view_as_real(C.conj().resolve_conj()))
        lr_dict, lr = ({}, lr) if lr is None or isinstance(lr, float) else (lr, None)
        self.register("log_dt", log_dt, lr_dict.get("dt", lr))
        self.register("B", torch.view_as_real(B), lr_dict.get("B", lr))
        self.register("inv_A_real", torch.log(-A.real.clamp(max=-1e-4)), lr_dict.get("A", lr))
        self.register("A_imag", A.imag, lr_dict.get("A", lr))

    def _A(self):
        return torch.complex(-torch.exp(self.inv_A_real), self.A_imag)

    def forward(self, L, state=None, rate=1.0):
        dt = torch.exp(self.log_dt) * rate
        C = torch.view_as_complex(self.C)
        A = self._A().repeat(self.repeat, 1)
        B = torch.view_as_complex(self.B).repeat(self.repeat, 1)
        dtA = A * dt.unsqueeze(-1)
        C = B[None] * C
        if self.disc == "zoh":
            K = log_vandermonde(C * (torch.exp(dtA) - 1.0) / A, dtA, L)
        else:
            C = C * (1.0 - dtA / 2).reciprocal() * dt.unsqueeze(-1)
            K = log_vandermonde(C, ((1.0 + dtA / 2) / (1.0 - dtA / 2)).log(), L)
        return K.view(self.channels, self.H, L), None

    def discrete(self):
        dt = torch.exp(self.log_dt)
        A = self._A().repeat(self.repeat, 1)
        B = torch.view_as_complex(self.B).repeat(self.repeat, 1)
        dtA = A * dt.unsqueeze(-1)
        if self.disc == "zoh":
            return torch.exp(dtA), B * (torch.exp(dtA) - 1.0) / A
        return (1.0 + dtA / 2) / (1.0 - dtA / 2), B * (1.0 - dtA / 2).reciprocal() * dt.unsqueeze(-1)

    def default_state(self, *batch_shape):
        return torch.zeros(*batch_shape, self.H, self.N, dtype=torch.cfloat, device=self.C.device)

    def step(self, u, state):
        dA, dB = self.discrete()
        state = dA * state + dB * u.unsqueeze(-1)
        return 2 * torch.einsum("chn,bhn->bch", torch.view_as_complex(self.C), state).real, state


class SSKernelShift(OptimModule):
    def __init__(self, B, C, L=None, lr=None, **kwargs):
        super().__init__()
        self.L, self.N, self.H = L, B.size(-1), B.shape[0]
        lr_dict, lr = ({}, lr) if lr is None or isinstance(lr, float) else (lr, None)
        self.register("B", B, lr_dict.get("B", lr))
        self.C = nn.Parameter(C)

    def forward(self, state=None, rate=1.0, L=None):
        L = self.L if L is None else L
        B_f = torch.fft.rfft(self.B.float(), n=2 * self.N)
        C_f = torch.fft.rfft(self.C.float(), n=2 * self.N)
        k = torch.fft.irfft(B_f.conj() * C_f, n=2 * self.N)[..., : min(self.N, L)]
        return (F.pad(k, (0, L - self.N)) if self.N < L else k).float(), None

    def default_state(self, *batch_shape):
        return torch.zeros(*batch_shape, self.H, self.N, dtype=self.C.dtype, device=self.C.device)

    def step(self, u, state):
        state = F.pad(state, (1, -1)) + self.B * u.unsqueeze(-1)
        return torch.einsum("chn,bhn->bch", self.C, state), state


class SSKernel(nn.Module):
    def __init__(self, H, N=64, L=None, measure="diag-lin", channels=1, dt_min=0.001, dt_max=0.1, deterministic=False, lr=None,
                 mode="diag", n_ssm=None, **kernel_args):
        super().__init__()
        self.N, self.H, self.channels, self.mode = N, H, channels, mode
        n_ssm = H if n_ssm is None else n_ssm
        if deterministic:
            log_dt = torch.linspace(math.log(dt_min), math.log(dt_max), H)
        else:
            log_dt = torch.rand(H) * (math.log(dt_max) - math.log(dt_min)) + math.log(dt_min)
        if mode == "shift":
            B = torch.zeros(H, N)
            B[..., 0] = 1.0
            C = torch.empty(H, channels, N)
            nn.init.kaiming_uniform_(C, a=math.sqrt(5))
            self.kernel = SSKernelShift(B, C.transpose(0, 1).contiguous(), L=L, lr=lr, **kernel_args)
        elif mode == "diag":
            measures = {"diag": ["diag-inv", "diag-lin"]}.get(measure, [measure])
            parts = [diag_init(m.split("-")[1], N, n_ssm // len(measures)) for m in measures]
            w, B = torch.cat([p[0] for p in parts]), torch.cat([p[1] for p in parts])
            C = torch.randn(channels, H, N // 2, dtype=torch.cfloat) * B.repeat(H // n_ssm, 1)
            self.kernel = SSKernelDiag(w, B, C, log_dt, L=L, lr=lr, **kernel_args)
        else:
            raise NotImplementedError(f"{mode=} is not valid")

    def forward(self, state=None, L=None, rate=1.0):
        return self.kernel(state=state, L=L, rate=rate)

    def step(self, u, state):
        return self.kernel.step(u, state)

    def default_state(self, *a):
        return self.kernel.default_state(*a)


class H3(nn.Module):
    def __init__(self, d_model: int, d_state: int = 64, l_max: int = None, head_dim: int = 1, use_fast_fftconv: bool = False,
                 dropout: float = 0.0, layer_idx: int = None, device=None, dtype=None, kernel_args: dict = {}, **kwargs):
        super().__init__()
        assert d_model % head_dim == 0
        d_state = int(d_state)
        self.d_model, self.head_dim, self.H, self.N, self.L, self.layer_idx = d_model, head_dim, d_model // head_dim, d_state, l_max, layer_idx
        self.q_proj, self.k_proj, self.v_proj = (nn.Linear(d_model, d_model) for _ in range(3))
        self.ssm_k_kernel = SSKernel(d_model, N=d_state, L=l_max, mode="shift", lr=kernel_args.get("lr", None))
        self.ssm_k_D = nn.Parameter(torch.randn(d_model))
        self.kernel = SSKernel(self.H, N=d_state, L=l_max, channels=1, **kernel_args)
        self.D = nn.Parameter(torch.randn(self.H))
        self.output_linear = nn.Linear(d_model, d_model)

    def forward(self, u, *args, **kwargs):
        B, L, _ = u.shape
        Lk = L if self.L is None else min(L, self.L)
        n = Lk + L
        q, k, v = (p(u).transpose(1, 2).float() for p in (self.q_proj, self.k_proj, self.v_proj))   # [B, d, L]
        kk = self.ssm_k_kernel(L=Lk)[0][0]
        k = torch.fft.irfft(torch.fft.rfft(kk, n=n) * torch.fft.rfft(k, n=n), n=n)[..., :L] + self.ssm_k_D[:, None] * k
        d = self.head_dim
        # (h d1) split: channel index = h * head_dim + d1
        k5 = k.view(B, self.H, d, L).permute(0, 2, 1, 3)[:, :, None]         # b d1 1 h l
        v5 = v.view(B, self.H, d, L).permute(0, 2, 1, 3)[:, None]            # b 1 d2 h l
        kv = k5 * v5
        sk = self.kernel(L=Lk)[0][0]                                         # [H, Lk]
        y = torch.fft.irfft(torch.fft.rfft(kv, n=n) / n * torch.fft.rfft(sk, n=n), n=n, norm="forward")[..., :L]
        y = y + kv * self.D.unsqueeze(-1)
        q5 = q.view(B, self.H, d, L).permute(0, 2, 1, 3)[:, :, None]         # b d1 1 h l
        y = (y * q5).sum(dim=1)                                              # b d2 h l
        y = y.reshape(B, d * self.H, L).transpose(1, 2)                      # channel = d2 * H + h, as the reference's '(d h)'
        return self.output_linear(y.to(self.output_linear.weight.dtype))

    def state_size(self, sequence_length: int = 2048):
        return self.d_model * self.N
