"""The allocation-free attention backward, called through its exported C symbol.

Some users of the library cannot let it allocate device memory (all memory already belongs to their own pool, or an
allocation would stall their loop). For them ``b200_attn_bwd_noalloc`` keeps its one temporary buffer in a fixed array
inside the library. This test loads the shared library with ctypes, calls the symbol twice in a row on different data
and checks both results against the regular backward, which allocates its temporary per call.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from ml_experiments_b200 import _ext

    _ext.load()
    lib = ctypes.CDLL(str(_ext.lib_path()))
    f = lib.b200_attn_bwd_noalloc
    vp, ll = ctypes.c_void_p, ctypes.c_longlong
    f.argtypes = [vp] * 11 + [ctypes.c_int] * 3 + [ll] * 8 + [ctypes.c_float, ctypes.c_int, vp, vp]
    f.restype = ctypes.c_int
    lib.b200_attn_bwd_noalloc_error.restype = ctypes.c_char_p
    return lib


def _case(seed, t, h, doc_len, window, d=128):
    from ml_experiments_b200.ops import attention as A

    torch.manual_seed(seed)
    qkv = torch.randn(t, 3, h, d, device="cuda", dtype=torch.bfloat16)
    q, k, v = qkv[:, 0], qkv[:, 1], qkv[:, 2]
    starts = torch.zeros(t, dtype=torch.bool, device="cuda")
    starts[::doc_len] = True
    ds, de = A.doc_bounds_from_starts(starts)
    d_o = torch.randn(t, h, d, device="cuda", dtype=torch.bfloat16)
    o, lse = A.flash_attention_forward(q, k, v, ds, de, 0.12, window)
    return q, k, v, o, lse, d_o, ds, de


def _call(lib, q, k, v, o, lse, d_o, ds, de, window):
    from ml_experiments_b200.ops.runtime import status

    t, h, d = q.shape
    dq = torch.zeros(t, h, d, dtype=torch.float32, device="cuda")
    dk = torch.zeros(t, h, d, dtype=torch.bfloat16, device="cuda")
    dv = torch.zeros(t, h, d, dtype=torch.bfloat16, device="cuda")
    stream = torch.cuda.current_stream().cuda_stream
    rc = lib.b200_attn_bwd_noalloc(q.data_ptr(), k.data_ptr(), v.data_ptr(), o.data_ptr(), d_o.data_ptr(), lse.data_ptr(),
                                   dq.data_ptr(), dk.data_ptr(), dv.data_ptr(), ds.data_ptr(), de.data_ptr(), t, h, d,
                                   q.stride(0), k.stride(0), v.stride(0), o.stride(0), d_o.stride(0), dq.stride(0),
                                   dk.stride(0), dv.stride(0), 0.12, window, status().data_ptr(), stream)
    assert rc == 0, lib.b200_attn_bwd_noalloc_error()
    return dq, dk, dv


def test_noalloc_matches_regular_backward_twice():
    from ml_experiments_b200.ops import attention as A
    from ml_experiments_b200.ops.runtime import check_status

    lib = _lib()
    for seed, t, h, doc_len, window in ((0, 1024, 2, 1024, 0), (1, 2048, 3, 640, 3)):
        q, k, v, o, lse, d_o, ds, de = _case(seed, t, h, doc_len, window)
        want = A.flash_attention_backward(q, k, v, o, d_o, lse, ds, de, 0.12, window)
        got = _call(lib, q, k, v, o, lse, d_o, ds, de, window)
        torch.cuda.synchronize()
        check_status()
        for name, g, w in zip(("dq", "dk", "dv"), got, want):
            rel = ((g.float() - w.float()).norm() / w.float().norm()).item()
            assert rel < 2e-2, (name, rel)


def test_noalloc_head_dim_64():
    """The entry point takes both head sizes of the kernel; any other is refused with an argument error."""
    from ml_experiments_b200.ops import attention as A
    from ml_experiments_b200.ops.runtime import check_status

    lib = _lib()
    q, k, v, o, lse, d_o, ds, de = _case(2, 1024, 4, 512, 0, d=64)
    want = A.flash_attention_backward(q, k, v, o, d_o, lse, ds, de, 0.12, 0)
    got = _call(lib, q, k, v, o, lse, d_o, ds, de, 0)
    torch.cuda.synchronize()
    check_status()
    for name, g, w in zip(("dq", "dk", "dv"), got, want):
        rel = ((g.float() - w.float()).norm() / w.float().norm()).item()
        assert rel < 2e-2, (name, rel)
    z = torch.zeros(8, device="cuda")
    p = z.data_ptr()
    rc = lib.b200_attn_bwd_noalloc(p, p, p, p, p, p, p, p, p, p, p, 128, 1, 96, 1, 1, 1, 1, 1, 1, 1, 1, 0.1, 0, None, None)
    assert rc == -1 and b"head_dim" in lib.b200_attn_bwd_noalloc_error()


def test_noalloc_rejects_oversized_problem():
    lib = _lib()
    z = torch.zeros(8, device="cuda")
    p = z.data_ptr()
    rc = lib.b200_attn_bwd_noalloc(p, p, p, p, p, p, p, p, p, p, p, 1 << 19, 4, 128, 1, 1, 1, 1, 1, 1, 1, 1, 0.1, 0, None, None)
    assert rc == -2 and b"scratch" in lib.b200_attn_bwd_noalloc_error()
