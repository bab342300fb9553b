"""accb_reduce_mean_rank3_noalloc: the reduce_mean entry point for hosts that own all device memory.

Some users of this library may not let a library call allocate on the GPU: a server or framework that wraps a
HAT function as a custom operator gives it buffers from its own arena, and a cudaMalloc hidden inside the
call would escape that arena's budget, could fail once the arena holds nearly all of HBM, and would stall
every stream of the device.  The no-alloc entry point keeps the partial sums of a split reduction in a
256 KiB array built into the library instead.  This test calls it through the C ABI (ctypes) on device
buffers and checks it against the ordinary entry point, twice in a row with different shapes, because the
built-in array is shared by all calls and still holds the previous call's partial sums.

The file name sorts last on purpose: a run that stops at the first failure has then already run every
other test.
"""
import ctypes

import numpy as np
import pytest

from accera_b200 import runtime as rt

pytestmark = pytest.mark.gpu

RTOL = 1e-5      # the reduce_mean tolerance of the other GPU tests


def _both(shape, axes, seed):
    import torch
    dev = torch.device("cuda:0")
    g = torch.Generator(device="cpu").manual_seed(seed)
    x = torch.randn(shape, generator=g, dtype=torch.float32).to(dev)
    dims, mask = rt.reduce_mean_rank3_dims(*shape, axes, 0)
    n_out = int(np.prod(dims))
    want = torch.full((n_out,), float("nan"), device=dev)
    got = torch.full((n_out,), float("nan"), device=dev)
    rt.reduce_mean_rank3(x, want, axes)                                   # existing entry point
    rt.synchronize()
    lib = rt.lib()
    stream = torch.cuda.current_stream(dev).cuda_stream
    rc = lib.accb_reduce_mean_rank3_noalloc(ctypes.c_void_p(x.data_ptr()), shape[0], shape[1], shape[2],
                                            ctypes.c_void_p(got.data_ptr()), mask, ctypes.c_void_p(stream or None))
    assert rc == 0, lib.accb_last_error().decode()
    torch.cuda.synchronize(dev)
    scale = x.abs().mean(dim=tuple(axes)).reshape(-1).cpu().numpy()
    g_np, w_np = got.cpu().numpy(), want.cpu().numpy()
    assert np.isfinite(g_np).all()
    assert (np.abs(g_np - w_np) <= RTOL * np.maximum(np.abs(w_np), scale)).all(), (shape, axes)
    exact = x.double().mean(dim=tuple(axes)).reshape(-1).cpu().numpy()
    assert (np.abs(g_np - exact) <= RTOL * np.maximum(np.abs(exact), scale)).all(), (shape, axes)


def test_noalloc_matches_existing_entry_point_on_two_calls_in_a_row():
    # both shapes take the split path (few outputs, long reductions), so both use the built-in scratch;
    # the second is smaller and runs over the first call's leftovers
    _both((1, 4, 1 << 20), [2], seed=11)          # rows split
    _both((6000, 1, 192), [0], seed=12)           # cols split
    _both((1, 2, 300000), [2], seed=13)
    _both((2, 64, 4096), [2], seed=14)            # single pass: no scratch at all


def test_noalloc_rejects_shapes_beyond_the_builtin_scratch():
    import torch
    dev = torch.device("cuda:0")
    # 37000 outputs, each split in two: 296 000 B of partial sums > the 256 KiB built in
    x = torch.zeros(600, 1, 37000, device=dev)
    y = torch.full((37000,), 5.0, device=dev)
    lib = rt.lib()
    rc = lib.accb_reduce_mean_rank3_noalloc(ctypes.c_void_p(x.data_ptr()), 600, 1, 37000, ctypes.c_void_p(y.data_ptr()), 1, None)
    assert rc == rt.ERR_LIMIT
    msg = lib.accb_last_error().decode()
    assert "296000" in msg and "262144" in msg
    torch.cuda.synchronize(dev)
    assert bool((y == 5.0).all())                  # nothing was launched
    rt.reduce_mean_rank3(x, y, [0])                # the ordinary entry point takes the same shape
    rt.synchronize()
    assert bool((y == 0.0).all())


def test_noalloc_rejects_host_buffers_and_bad_arguments():
    lib = rt.lib()
    x = np.zeros((1, 2, 4096), np.float32)
    y = np.zeros(2, np.float32)
    rc = lib.accb_reduce_mean_rank3_noalloc(ctypes.c_void_p(x.ctypes.data), 1, 2, 4096, ctypes.c_void_p(y.ctypes.data), 4, None)
    assert rc == rt.ERR_ARG and b"device memory" in lib.accb_last_error()
    assert lib.accb_reduce_mean_rank3_noalloc(None, 1, 2, 3, None, 9, None) == rt.ERR_ARG
    assert lib.accb_reduce_mean_rank3_noalloc(None, -1, 2, 3, None, 4, None) == rt.ERR_ARG


def test_noalloc_leaves_free_device_memory_unchanged():
    """The contract in the name: once the first call on the device has resolved the built-in array's address, a call
    changes nothing about device memory - not the driver's free-memory figure, and not the cached scratch buffer of
    the ordinary entry point."""
    import torch
    dev = torch.device("cuda:0")
    x = torch.randn(1, 4, 1 << 20, device=dev)
    y = torch.empty(4, device=dev)
    y2 = torch.empty(1 << 14, device=dev)
    x2 = torch.randn(3000, 1, 1 << 14, device=dev)
    lib = rt.lib()
    stream = ctypes.c_void_p(torch.cuda.current_stream(dev).cuda_stream or None)

    def call(data, out, d, mask):
        rc = lib.accb_reduce_mean_rank3_noalloc(ctypes.c_void_p(data.data_ptr()), d[0], d[1], d[2], ctypes.c_void_p(out.data_ptr()), mask, stream)
        assert rc == 0, lib.accb_last_error().decode()
    call(x, y, (1, 4, 1 << 20), 4)                     # set-up call (first use on this device resolves the symbol)
    torch.cuda.synchronize(dev)
    rt.release_workspace()                             # the ordinary entry point's cached buffers are gone: nothing to lean on
    torch.cuda.synchronize(dev)
    free_before, _ = torch.cuda.mem_get_info(dev)
    call(x, y, (1, 4, 1 << 20), 4)                     # rows split: uses the built-in scratch
    call(x2, y2, (3000, 1, 1 << 14), 1)                # cols split: uses it again, over the leftovers
    torch.cuda.synchronize(dev)
    free_after, _ = torch.cuda.mem_get_info(dev)
    assert free_after == free_before
    assert (y - x.double().mean(dim=(0, 2)).float()).abs().max().item() <= 1e-5 * x.abs().mean().item()
    assert lib.accb_last_error() == b""                # a successful call leaves no stale error text behind


def test_noalloc_works_in_a_process_that_never_used_the_allocating_entry_point():
    """A fresh process calls only the no-alloc entry point (two shapes that take the split path) and checks the
    result itself: it cannot be borrowing scratch memory that accb_reduce_mean_rank3 allocated earlier."""
    import os
    import subprocess
    import sys
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    code = r'''
import ctypes, sys
sys.path.insert(0, %r)
import torch
from accera_b200 import runtime as rt
dev = torch.device("cuda:0")
lib = rt.lib()
torch.manual_seed(3)
for shape, mask, dims in (((1, 4, 1 << 20), 4, (0, 2)), ((6000, 1, 192), 1, (0,))):
    x = torch.randn(*shape, device=dev)
    n_out = 4 if mask == 4 else 192
    y = torch.full((n_out,), float("nan"), device=dev)
    rc = lib.accb_reduce_mean_rank3_noalloc(ctypes.c_void_p(x.data_ptr()), shape[0], shape[1], shape[2],
                                            ctypes.c_void_p(y.data_ptr()), mask, None)
    assert rc == 0, lib.accb_last_error()
    torch.cuda.synchronize()
    want = x.double().mean(dim=dims).reshape(-1).float()
    assert (y - want).abs().max().item() <= 1e-5 * x.abs().mean().item(), shape
print("fresh process ok")
''' % root
    r = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, timeout=600)
    assert r.returncode == 0 and "fresh process ok" in r.stdout, r.stdout + r.stderr
