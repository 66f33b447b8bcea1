"""Low-precision shadows of master parameters.

The fused model consumes bf16 (or scaled fp8) copies of fp32 master weights. A shadow is rebuilt only when the
parameter changed (``Tensor._version`` or storage pointer differs), and an optimizer that produces the updated
low-precision values itself can hand them over with :func:`set_shadow` and skip the cast pass.
"""
from __future__ import annotations

import weakref

import torch

_cache: dict[tuple[int, torch.dtype], tuple] = {}


def _key(p: torch.Tensor, dtype: torch.dtype):
    return (id(p), dtype)


def shadow_of(p: torch.Tensor, dtype: torch.dtype, scale: float = 1.0) -> torch.Tensor:
    """Returns ``(p * scale).to(dtype)``, cached until ``p`` is modified in place or re-allocated."""
    if p.dtype == dtype and scale == 1.0:
        return p.detach()
    k = _key(p, dtype)
    ent = _cache.get(k)
    if ent is not None:
        ref, version, ptr, sc, t = ent
        if ref() is p and version == p._version and ptr == p.data_ptr() and sc == scale:
            return t
    src = p.detach()
    if dtype in (torch.float8_e4m3fn, torch.float8_e5m2) and src.is_cuda and src.dtype in (torch.float32, torch.bfloat16):
        from ..ops.fused import cast_fp8

        t = cast_fp8(src, scale, dtype)
    else:
        t = (src * scale).to(dtype) if scale != 1.0 else src.to(dtype)
    _cache[k] = (weakref.ref(p), p._version, p.data_ptr(), scale, t)
    return t


def set_shadow(p: torch.Tensor, t: torch.Tensor, scale: float = 1.0) -> None:
    """Registers ``t`` as the current shadow of ``p`` (call after the in-place update of ``p``)."""
    _cache[_key(p, t.dtype)] = (weakref.ref(p), p._version, p.data_ptr(), scale, t)


def get_shadow_buffer(p: torch.Tensor, dtype: torch.dtype):
    """The cached shadow tensor of ``p`` if one exists (possibly stale), for in-place refresh by an optimizer."""
    ent = _cache.get(_key(p, dtype))
    return None if ent is None or ent[0]() is not p else ent[4]


def clear() -> None:
    _cache.clear()
