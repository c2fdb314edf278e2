"""tcgen05 tile engine self-test: every operand arrangement used by the scan
kernels against a plain fp32 product of the same bf16 values."""

from __future__ import annotations

import pytest
import torch

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("mode", [0, 1, 2, 3])
def test_umma_selftest(mode):
    from slinoss_b200 import _lib

    g = torch.Generator().manual_seed(mode)
    shapes = {0: ((128, 64), (128, 64), (128, 128)), 1: ((128, 128), (128, 64), (128, 64)),
              2: ((128, 128), (128, 64), (128, 64)), 3: ((128, 64), (64, 64), (128, 64))}[mode]
    A = torch.randn(shapes[0], generator=g).to(torch.bfloat16).cuda()
    B = torch.randn(shapes[1], generator=g).to(torch.bfloat16).cuda()
    C = torch.full(shapes[2], float("nan"), device="cuda", dtype=torch.float32)
    status = torch.zeros(1, device="cuda", dtype=torch.int32)
    rc = _lib.selftest_lib().slx_umma_selftest(mode, A.data_ptr(), B.data_ptr(), C.data_ptr(), status.data_ptr(),
                                               _lib.stream_ptr(A.device))
    assert rc == 0, _lib.selftest_lib().slx_selftest_last_error_string()
    torch.cuda.synchronize()
    assert int(status.item()) == 0, "bounded mbarrier wait ran out"
    a, b = A.float(), B.float()
    ref = {0: lambda: a @ b.T, 1: lambda: a @ b, 2: lambda: a.T @ b, 3: lambda: a @ b.T}[mode]()
    err = (C - ref).norm() / ref.norm()
    assert float(err) < 1e-5, f"mode {mode}: relative error {float(err):.3e}"
