"""Low-precision shadows of master parameters.

The fused model consumes bf16 (or scaled fp8) copies of fp32 master weights. A shadow is rebuilt only when the
parameter changed. "Changed" is decided by three things together: the storage pointer, ``Tensor._version`` (bumped
by every in-place *torch* operation) and an explicit generation number kept here. The generation exists because the
operators of ``torch.ops.b200`` update parameters in place WITHOUT touching ``Tensor._version`` (an operator
registered through ``TORCH_LIBRARY`` does not bump it, whatever its schema says): every optimizer of this package
therefore either calls :func:`mark_modified` after such an update, or hands over the low-precision values it produced
itself with :func:`set_shadow` and skips the cast pass.
"""
from __future__ import annotations

import weakref

import torch

_cache: dict[tuple[int, torch.dtype], tuple] = {}
_generation: dict[int, int] = {}


def _key(p: torch.Tensor, dtype: torch.dtype):
    return (id(p), dtype)


def generation(p: torch.Tensor) -> int:
    return _generation.get(id(p), 0)


def mark_modified(p: torch.Tensor) -> None:
    """Tells the cache that ``p`` was changed in place by something that does not bump ``Tensor._version``."""
    _generation[id(p)] = _generation.get(id(p), 0) + 1


def _stamp(p: torch.Tensor):
    return (p._version, generation(p), p.data_ptr())


def shadow_of(p: torch.Tensor, dtype: torch.dtype, scale: float = 1.0) -> torch.Tensor:
    """Returns ``(p * scale).to(dtype)``, cached until ``p`` is modified in place or re-allocated."""
    if p.dtype == dtype and scale == 1.0:
        return p.detach()
    k = _key(p, dtype)
    ent = _cache.get(k)
    if ent is not None:
        ref, stamp, sc, t = ent
        if ref() is p and stamp == _stamp(p) and sc == scale:
            return t
    src = p.detach()
    if dtype in (torch.float8_e4m3fn, torch.float8_e5m2) and src.is_cuda and src.dtype in (torch.float32, torch.bfloat16):
        from ..ops.fused import cast_fp8

        t = cast_fp8(src, scale, dtype)
    else:
        t = (src * scale).to(dtype) if scale != 1.0 else src.to(dtype)
    _cache[k] = (weakref.ref(p), _stamp(p), scale, t)
    return t


def set_shadow(p: torch.Tensor, t: torch.Tensor, scale: float = 1.0) -> None:
    """Registers ``t`` as the current shadow of ``p`` (call AFTER the in-place update of ``p`` and after
    :func:`mark_modified`, if that is called at all). Shadows of ``p`` in other dtypes are dropped: they are stale."""
    for k in [k for k in _cache if k[0] == id(p) and k[1] != t.dtype]:
        del _cache[k]
    _cache[_key(p, t.dtype)] = (weakref.ref(p), _stamp(p), scale, t)


def get_shadow_buffer(p: torch.Tensor, dtype: torch.dtype):
    """The cached shadow tensor of ``p`` if one exists (possibly stale), for in-place refresh by an optimizer."""
    ent = _cache.get(_key(p, dtype))
    return None if ent is None or ent[0]() is not p else ent[3]


def shadow_entries(p: torch.Tensor):
    """``[(dtype, scale, tensor)]`` of every cached shadow of ``p`` (possibly stale): an optimizer that can write the
    low-precision copy in its own update kernel refreshes these buffers in place."""
    out = []
    for (pid, dtype), ent in _cache.items():
        if pid == id(p) and ent[0]() is p:
            out.append((dtype, ent[2], ent[3]))
    return out


def clear() -> None:
    _cache.clear()
    _generation.clear()
