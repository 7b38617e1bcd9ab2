"""The allocation-free RMSNorm backward (``b200_rmsnorm_bwd_noalloc``).

Some users of the library may not allocate device memory at the moment they call it — while a
stream is being captured, inside a host callback or a latency-critical loop where ``cudaMalloc``
would synchronise the device, or when an embedder forbids all allocators.  For them the library
exports one C symbol whose scratch memory is a fixed array inside the module.  This test calls that
symbol directly (ctypes, no torch binding in between) and checks it against the regular entry point
on two consecutive calls, because the shared scratch array keeps the first call's contents.
"""
import ctypes
import gc

import pytest
import torch

from archscale_b200.ops import backend
from archscale_b200.ops.norm import rms_norm_ref

pytestmark = pytest.mark.gpu


def _lib():
    path = backend.extension_path()
    assert path is not None, "archscale_b200/_C.so is not built"
    backend.require_extension()          # make sure torch's libraries are loaded first
    lib = ctypes.CDLL(path)
    f = lib.b200_rmsnorm_bwd_noalloc
    f.restype = ctypes.c_int
    f.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_int, ctypes.c_void_p, ctypes.c_int,
                  ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p]
    lib.b200_noalloc_last_error.restype = ctypes.c_char_p
    return lib


def _call(lib, dy, x, w, rstd, dx, dw):
    code = {torch.float32: 0, torch.bfloat16: 1}
    stream = torch.cuda.current_stream().cuda_stream
    return lib.b200_rmsnorm_bwd_noalloc(dy.data_ptr(), code[dy.dtype], x.data_ptr(), code[x.dtype], w.data_ptr(),
                                        code[w.dtype], rstd.data_ptr(), dx.data_ptr(), dw.data_ptr(), x.shape[0],
                                        x.shape[1], ctypes.c_void_p(stream))


def test_noalloc_matches_regular_entry_point_twice():
    lib = _lib()
    ext = backend.require_extension()
    torch.manual_seed(0)
    # The first call on a device resolves the address of the built-in array; with lazy module loading that is also when the
    # driver materialises the array (its 4.6 MiB come out of free memory once, there).  Make that call before measuring.
    x0 = torch.randn(8, 1024, device="cuda")
    assert _call(lib, x0.bfloat16(), x0, torch.ones(1024, device="cuda"), torch.ones(8, device="cuda"), torch.empty_like(x0),
                 torch.empty(1024, device="cuda")) == 0
    for rows, cols, xdt in [(1000, 2048, torch.float32), (333, 1024, torch.bfloat16)]:   # two calls in a row
        x = torch.randn(rows, cols, device="cuda").to(xdt)
        w = 1 + 0.1 * torch.randn(cols, device="cuda")
        dy = torch.randn(rows, cols, device="cuda").bfloat16()
        _, rstd = ext.rmsnorm_fwd(x, w, 1e-5, torch.bfloat16)
        dx_ref, dw_ref = ext.rmsnorm_bwd(dy, x, w, rstd)
        dx = torch.empty_like(x)
        dw = torch.empty(cols, device="cuda", dtype=torch.float32)
        gc.collect()                                     # unrelated garbage freed during the call would move the counters
        torch.cuda.synchronize()
        before = torch.cuda.memory_allocated()
        n_allocs = torch.cuda.memory_stats()["allocation.all.allocated"]
        free_before, _ = torch.cuda.mem_get_info()       # the driver's view: sees a raw cudaMalloc that torch's counter cannot
        rc = _call(lib, dy, x, w, rstd, dx, dw)
        torch.cuda.synchronize()
        assert rc == 0, lib.b200_noalloc_last_error()
        assert torch.cuda.memory_stats()["allocation.all.allocated"] == n_allocs     # no allocation event at all
        assert torch.cuda.memory_allocated() <= before
        assert torch.cuda.mem_get_info()[0] == free_before
        tol = 2e-2 if xdt == torch.bfloat16 else 1e-5
        assert (dx.float() - dx_ref.float()).norm() <= tol * dx_ref.float().norm()
        assert (dw - dw_ref).norm() <= 1e-5 * dw_ref.norm()
        # and against the plain PyTorch fp32 formula of the same op
        xo = x.float().detach().requires_grad_()
        wo = w.clone().requires_grad_()
        rms_norm_ref(xo, wo, 1e-5).backward(dy.float())
        assert (dx.float() - xo.grad).norm() <= (2e-2 if xdt == torch.bfloat16 else 2e-3) * xo.grad.norm()
        assert (dw - wo.grad).norm() <= 2e-3 * wo.grad.norm()


def test_noalloc_rejects_oversized_rows():
    lib = _lib()
    cols = 8192
    x = torch.randn(8, cols, device="cuda")
    w = torch.ones(cols, device="cuda")
    dy = torch.randn(8, cols, device="cuda")
    rstd = torch.ones(8, device="cuda")
    rc = _call(lib, dy, x, w, rstd, torch.empty_like(x), torch.empty(cols, device="cuda"))
    assert rc < 0
    assert b"exceeds" in lib.b200_noalloc_last_error()
