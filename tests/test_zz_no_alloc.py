"""The allocation-free column-sum entry point, called through its exported C symbol.

Some callers cannot ask the driver for memory when they need a result: an allocator lock is held, the
thread must not stall on cudaMalloc's synchronisation, or their memory was budgeted once at start-up. ``oslo_colsum_noalloc`` serves them
from a workspace built into the library. This test compares it with the ordinary ``colsum`` op (which
allocates its workspace) on two consecutive calls, since the calls share the built-in workspace. The file
name sorts last so that a failure here never hides another test.
"""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

DT = {torch.bfloat16: 0, torch.float16: 1, torch.float32: 2}


def _lib():
    from oslo_b200 import ops
    assert ops.load_ext(required=True) is not None
    lib = ctypes.CDLL(ops.ext_path())
    fn = lib.oslo_colsum_noalloc
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    return fn


def _call(fn, x, out):
    stream = torch.cuda.current_stream().cuda_stream
    return fn(x.data_ptr(), out.data_ptr(), x.size(0), x.size(1), DT[x.dtype], stream)


def test_noalloc_colsum_matches_allocating_entry_point_twice_in_a_row():
    fn = _lib()
    ext = torch.ops.oslo_b200
    torch.manual_seed(0)
    torch.cuda.set_device(0)
    cases = [(1000, 4096, torch.bfloat16), (37, 520, torch.float32), (5000, 16384, torch.float16)]
    for rows, cols, dt in cases:
        x1 = torch.randn(rows, cols, device="cuda").to(dt)
        x2 = (torch.randn(rows, cols, device="cuda") * 3 + 1).to(dt)
        o1 = torch.full((cols,), float("nan"), device="cuda")
        o2 = torch.full((cols,), float("nan"), device="cuda")
        assert _call(fn, x1, o1) == 0          # two calls back to back share the built-in workspace:
        assert _call(fn, x2, o2) == 0          # the second must not see anything of the first
        torch.cuda.synchronize()
        w1, w2 = ext.colsum(x1), ext.colsum(x2)
        tol = 1e-3 * rows ** 0.5 if dt != torch.float32 else 1e-4 * rows ** 0.5
        assert torch.allclose(o1, w1, atol=tol, rtol=1e-4), (rows, cols, dt, (o1 - w1).abs().max().item())
        assert torch.allclose(o2, w2, atol=tol, rtol=1e-4), (rows, cols, dt, (o2 - w2).abs().max().item())
        assert torch.allclose(o1, x1.float().sum(0), atol=tol * 4, rtol=1e-3)


def test_noalloc_colsum_refuses_oversize_and_bad_arguments():
    fn = _lib()
    x = torch.zeros(4, 16384 + 8, device="cuda", dtype=torch.bfloat16)
    out = torch.full((16384 + 8,), 7.0, device="cuda")
    assert _call(fn, x, out) == -10            # wider than the built-in workspace: refused, nothing launched
    torch.cuda.synchronize()
    assert bool((out == 7.0).all())
    stream = torch.cuda.current_stream().cuda_stream
    assert fn(x.data_ptr(), out.data_ptr(), 4, 64, 9, stream) == -2
    assert fn(None, out.data_ptr(), 4, 64, 0, stream) == -3
    empty = torch.zeros(0, 64, device="cuda", dtype=torch.float32)
    o = torch.ones(64, device="cuda")
    assert fn(empty.data_ptr() or x.data_ptr(), o.data_ptr(), 0, 64, 2, stream) == 0
    torch.cuda.synchronize()
    assert bool((o == 0).all())
