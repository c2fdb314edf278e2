"""The conv backward entry point that takes no workspace.

Some hosts of this library cannot allocate device memory at call time (their own
allocator owns the whole GPU, or an allocation would stall the device), so they
cannot give ``slx_cconv1d_bwd`` its scratch buffer.  ``slx_cconv1d_bwd_noalloc``
keeps that scratch inside the library image instead.  This test calls it through
the C ABI twice in a row and compares every output with the regular entry point.
It lives in a file collected last so that a failure here cannot hide other tests.
"""

from __future__ import annotations

from ctypes import byref

import pytest
import torch

pytestmark = pytest.mark.gpu


def _run(lib, _lib, fn_noalloc, shape, x, w, bias, st, dy, dn):
    dev = x.device
    b, T, C = x.shape
    W = w.shape[1]
    dx = torch.full((b, T, C), float("nan"), device=dev, dtype=x.dtype)
    dw = torch.full((C, W), float("nan"), device=dev, dtype=torch.float32)
    db = torch.full((C,), float("nan"), device=dev, dtype=torch.float32)
    dst = torch.full((b, C, W - 1), float("nan"), device=dev, dtype=torch.float32)
    stream = _lib.stream_ptr(dev)
    if fn_noalloc:
        rc = lib.slx_cconv1d_bwd_noalloc(byref(shape), x.data_ptr(), w.data_ptr(), bias.data_ptr(), st.data_ptr(),
                                         dy.data_ptr(), dn.data_ptr(), dx.data_ptr(), dw.data_ptr(), db.data_ptr(),
                                         dst.data_ptr(), stream)
    else:
        n = int(lib.slx_cconv1d_bwd_workspace_bytes(byref(shape)))
        ws = torch.empty((n,), device=dev, dtype=torch.uint8)
        rc = lib.slx_cconv1d_bwd(byref(shape), x.data_ptr(), w.data_ptr(), bias.data_ptr(), st.data_ptr(),
                                 dy.data_ptr(), dn.data_ptr(), dx.data_ptr(), dw.data_ptr(), db.data_ptr(),
                                 dst.data_ptr(), ws.data_ptr(), n, stream)
    _lib.check(rc, "cconv1d backward")
    torch.cuda.synchronize()
    return dx, dw, db, dst


def test_noalloc_backward_matches_workspace_backward_twice():
    from slinoss_b200 import _lib

    lib = _lib.lib()
    g = torch.Generator().manual_seed(0)
    for call, (b, T, C, W, silu) in enumerate([(2, 300, 768, 4, 0), (3, 130, 96, 3, 1)]):
        dt = torch.bfloat16
        mk = lambda *s: torch.randn(*s, generator=g).to(dt).cuda()
        x, w, bias, st = mk(b, T, C), mk(C, W), mk(C), mk(b, C, W - 1)
        dy, dn = mk(b, T, C), mk(b, C, W - 1)
        shape = _lib.ConvShape(b, T, C, W, _lib.dtype_code(dt), silu, C, T * C)
        ref = _run(lib, _lib, False, shape, x, w, bias, st, dy, dn)
        got = _run(lib, _lib, True, shape, x, w, bias, st, dy, dn)
        for name, r, o in zip(("dx", "dweight", "dbias", "dstate"), ref, got):
            assert torch.isfinite(o.float()).all(), (call, name)
            # same kernels, same reduction order: identical bits
            assert torch.equal(r, o), (call, name)


def test_noalloc_rejects_oversized_shapes_with_a_clear_message():
    from slinoss_b200 import _lib

    lib = _lib.lib()
    shape = _lib.ConvShape(64, 8192, 4096, 4, 1, 0, 4096, 8192 * 4096)  # far beyond 1 Mi floats of partials
    rc = lib.slx_cconv1d_bwd_noalloc(byref(shape), *([None] * 11))
    assert rc == -3
    msg = lib.slx_last_error_string().decode()
    assert "built-in buffer" in msg and "slx_cconv1d_bwd" in msg
