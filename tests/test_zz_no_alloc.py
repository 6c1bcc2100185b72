"""The allocation-free C entry point for split-KV decode attention, called through its exported symbol.

Some callers cannot allocate device memory when they need attention: code between the begin and end of a stream capture,
serving loops that must not hit cudaMalloc's implicit synchronisation, and hosts that only hand a plugin raw device
pointers. For them the library keeps the split-KV partials in a built-in device array; this test loads the shared object
with ctypes, calls ``dlv_decode_attention_noalloc`` twice in a row on raw pointers and compares both results with the
regular (allocating) op, and checks that oversize requests are refused without launching anything.
"""
import ctypes
import math

import pytest
import torch

pytestmark = pytest.mark.gpu


def _lib():
    from deliverance_b200.ops.build import so_path

    lib = ctypes.CDLL(so_path())
    fn = lib.dlv_decode_attention_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_longlong, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p,
                   ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_float, ctypes.c_float,
                   ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    lib.dlv_decode_attention_noalloc_scratch_floats.restype = ctypes.c_ulonglong
    lib.dlv_decode_attention_noalloc_scratch_floats.argtypes = [ctypes.c_int] * 4
    return lib


def test_noalloc_decode_attention_matches_allocating_op():
    from deliverance_b200 import ops

    lib = _lib()
    dev = torch.device("cuda", 0)
    H, KV, D, page = 32, 8, 128, 32
    ctx = [1, 33, 100, 257, 600]
    B = len(ctx)
    g = torch.Generator().manual_seed(0)
    n_pages = sum((c + page - 1) // page for c in ctx) + 1
    kc = (torch.randn(n_pages, KV, page, D, generator=g) * 0.5).to(torch.bfloat16).to(dev)
    vc = (torch.randn(n_pages, KV, page, D, generator=g) * 0.5).to(torch.bfloat16).to(dev)
    bt = torch.zeros(B, max((c + page - 1) // page for c in ctx), dtype=torch.int32)
    nxt = 1
    for i, c in enumerate(ctx):
        n = (c + page - 1) // page
        bt[i, :n] = torch.arange(nxt, nxt + n, dtype=torch.int32)
        nxt += n
    bt = bt.to(dev)
    cl = torch.tensor(ctx, dtype=torch.int32, device=dev)
    scale = 1.0 / math.sqrt(D)
    stream = torch.cuda.current_stream(dev).cuda_stream
    for call, splits in enumerate((4, 4, 7)):  # two calls in a row with the same shape, then a different split count
        q = (torch.randn(B, H * D, generator=g) * 0.5).to(torch.bfloat16).to(dev)
        ref = ops.decode_attention(q, kc, vc, bt, cl, H, scale, 0.0, 0, splits)
        out = torch.full_like(ref, float("nan"))
        rc = lib.dlv_decode_attention_noalloc(q.data_ptr(), q.stride(0), kc.data_ptr(), vc.data_ptr(), bt.data_ptr(), bt.stride(0), cl.data_ptr(),
                                              out.data_ptr(), B, H, KV, D, page, scale, 0.0, 0, splits, stream)
        assert rc == 0, (call, rc)
        torch.cuda.synchronize(dev)
        assert torch.isfinite(out.float()).all()
        rel = ((out.float() - ref.float()).norm() / ref.float().norm()).item()
        assert rel < 1e-2, (call, rel)
    # a request beyond the built-in scratch is refused (nothing launched, output untouched)
    need = lib.dlv_decode_attention_noalloc_scratch_floats(4096, H, D, 16)
    assert need > (1 << 20)
    sentinel = torch.zeros(4, dtype=torch.bfloat16, device=dev)
    rc = lib.dlv_decode_attention_noalloc(q.data_ptr(), q.stride(0), kc.data_ptr(), vc.data_ptr(), bt.data_ptr(), bt.stride(0), cl.data_ptr(),
                                          sentinel.data_ptr(), 4096, H, KV, D, page, scale, 0.0, 0, 16, stream)
    assert rc == 2
    rc = lib.dlv_decode_attention_noalloc(q.data_ptr(), q.stride(0), kc.data_ptr(), vc.data_ptr(), bt.data_ptr(), bt.stride(0), cl.data_ptr(),
                                          out.data_ptr(), B, H, KV, 96, page, scale, 0.0, 0, 2, stream)
    assert rc == 1  # unsupported head_dim
    # pointers or strides that the kernels' 16-byte loads could not take are refused on the host (nothing is launched on them)
    args = dict(q=q.data_ptr(), qs=q.stride(0), k=kc.data_ptr(), v=vc.data_ptr())
    for bad in (dict(q=q.data_ptr() + 4), dict(qs=q.stride(0) + 4), dict(k=kc.data_ptr() + 8), dict(v=vc.data_ptr() + 2)):
        a = dict(args, **bad)
        rc = lib.dlv_decode_attention_noalloc(a["q"], a["qs"], a["k"], a["v"], bt.data_ptr(), bt.stride(0), cl.data_ptr(), sentinel.data_ptr(),
                                              B, H, KV, D, page, scale, 0.0, 0, 2, stream)
        assert rc == 1, bad
    torch.cuda.synchronize(dev)
    assert sentinel.float().abs().sum().item() == 0.0
