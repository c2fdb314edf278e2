"""GPU parity of the v2x2ssd scan against the pinned CPU oracle and the golden
fixtures produced by the reference.  Everything goes through the C ABI.

Tolerances (relative L2 error): 1e-5 for fp32 inputs,
2e-2 for bf16/fp16 inputs with fp32 state.
"""

from __future__ import annotations

import numpy as np
import pytest
import torch

from gpu_util import SCAN_GRADS, make_scan_inputs, oracle_fwd_bwd, run_b200_fwd_bwd, to_np
from util import golden, rel_err

pytestmark = pytest.mark.gpu

TOL_F32 = 1e-5
TOL_HALF = 2e-2


def _cuda(x, dtype=None):
    t = torch.from_numpy(np.ascontiguousarray(x))
    if dtype is not None:
        t = t.to(dtype)
    return t.cuda()


def _golden_inputs(g, dtype):
    inp = dict(U=_cuda(g["U"], dtype), M=_cuda(g["M"], torch.float32), K=_cuda(g["K"], torch.float32),
               B=_cuda(g["B"], dtype), C=_cuda(g["C"], dtype), dY=_cuda(g["dY"], dtype),
               initial_states=None, B_prev=None, U_prev=None, d_final=None)
    if "initial_states" in g:
        inp["initial_states"] = _cuda(g["initial_states"], torch.float32)
    if "B_prev" in g:
        inp["B_prev"] = _cuda(g["B_prev"], dtype)
        inp["U_prev"] = _cuda(g["U_prev"], dtype)
    if "d_final" in g:
        inp["d_final"] = _cuda(g["d_final"], torch.float32)
    return inp


def test_golden_small_stages_and_gradients():
    import slinoss_b200 as sb

    g = golden("scan_small_f64.npz")
    L = int(g["chunk_size"])
    inp = _golden_inputs(g, torch.float32)
    inc, mch = sb.chunk_increment_b200(inp["U"], inp["M"], inp["K"], inp["B"], B_prev=inp["B_prev"],
                                       U_prev=inp["U_prev"], chunk_size=L)
    assert rel_err(to_np(inc), g["inc"]) < TOL_F32
    assert rel_err(to_np(mch), g["m_chunk"]) < TOL_F32
    starts, fin = sb.state_passing_b200(inc, mch, initial_states=inp["initial_states"])
    assert rel_err(to_np(starts), g["chunk_starts"]) < TOL_F32
    assert rel_err(to_np(fin), g["final_state"]) < TOL_F32
    Y3 = sb.chunk_scan_b200(inp["U"], inp["M"], inp["K"], inp["B"], inp["C"], starts,
                            B_prev=inp["B_prev"], U_prev=inp["U_prev"], chunk_size=L)
    assert rel_err(to_np(Y3), g["Y_stage3"]) < TOL_F32
    Y, fin2, grads = run_b200_fwd_bwd(inp, L)
    assert rel_err(to_np(Y), g["Y"]) < TOL_F32
    assert rel_err(to_np(fin2), g["final_state"]) < TOL_F32
    for name in SCAN_GRADS:
        assert rel_err(to_np(grads[name]), g[name]) < TOL_F32, name


def test_golden_cfg0_fp32():
    g = golden("scan_cfg0_f32.npz")
    inp = _golden_inputs(g, torch.float32)
    Y, fin, grads = run_b200_fwd_bwd(inp, int(g["chunk_size"]), with_final_grad=False)
    Yo, fino, go = oracle_fwd_bwd(inp, with_final_grad=False)
    assert rel_err(to_np(Y), Yo) < TOL_F32 and rel_err(to_np(fin), fino) < TOL_F32
    for name in ("dU", "dM", "dK", "dB", "dC"):
        assert rel_err(to_np(grads[name]), go[name]) < TOL_F32, name
        # against the reference's own fp32 numbers (which carry fp32 noise themselves)
        assert rel_err(to_np(grads[name]), g[name]) < 3e-5, name
    assert rel_err(to_np(Y), g["Y"]) < 1e-5


def test_golden_bf16():
    g = golden("scan_bf16.npz")
    inp = _golden_inputs(g, torch.bfloat16)
    Y, fin, grads = run_b200_fwd_bwd(inp, int(g["chunk_size"]))
    assert rel_err(to_np(Y), g["Y"]) < TOL_HALF
    assert rel_err(to_np(fin), g["final_state"]) < TOL_HALF
    for name in ("dU", "dM", "dK", "dB", "dC"):
        assert rel_err(to_np(grads[name]), g[name]) < TOL_HALF, name


CASES = [
    # b, h, T, N, P, L, dtype, streaming, with_init, dist
    (1, 2, 1, 4, 8, 16, torch.float32, True, True, "tests"),       # single token
    (2, 2, 50, 5, 7, 16, torch.float32, True, True, "tests"),      # odd sizes, ragged tail
    (1, 3, 100, 16, 32, 32, torch.float32, False, True, "tests"),
    (2, 2, 130, 24, 64, 64, torch.float32, True, False, "tests"),
    (1, 2, 256, 16, 32, 128, torch.float32, True, True, "tests"),
    (1, 2, 300, 64, 64, 64, torch.bfloat16, True, True, "tests"),
    (1, 2, 384, 128, 64, 128, torch.bfloat16, False, False, "cfg2"),
    (2, 2, 256, 128, 64, 64, torch.bfloat16, True, True, "cfg2"),
    (1, 2, 200, 32, 64, 64, torch.float16, True, True, "tests"),
]


@pytest.mark.parametrize("case", CASES, ids=lambda c: f"b{c[0]}h{c[1]}T{c[2]}N{c[3]}P{c[4]}L{c[5]}{str(c[6])[6:]}")
def test_seeded_parity_against_oracle(case):
    b, h, T, N, P, L, dtype, streaming, with_init, dist = case
    inp = make_scan_inputs(b, h, T, N, P, dtype, seed=T + N, streaming=streaming, with_init=with_init,
                           dist=dist)
    Y, fin, grads = run_b200_fwd_bwd(inp, L)
    Yo, fino, go = oracle_fwd_bwd(inp)
    tol = TOL_F32 if dtype == torch.float32 else TOL_HALF
    errs = {"Y": rel_err(to_np(Y), Yo), "final": rel_err(to_np(fin), fino)}
    for name in SCAN_GRADS:
        if grads[name] is not None:
            errs[name] = rel_err(to_np(grads[name]), go[name])
    bad = {k: v for k, v in errs.items() if not v < tol}
    assert not bad, f"tolerance {tol}: {errs}"


def test_segment_chaining_equals_single_pass():
    """Two chained calls through the carried state reproduce one call
    (reference tests/test_v2x2ssd_cute.py:818-929)."""
    import slinoss_b200 as sb

    inp = make_scan_inputs(1, 2, 192, 16, 32, torch.float32, seed=5, streaming=True, with_init=True)
    full = sb.v2x2ssd_b200(inp["U"], inp["M"], inp["K"], inp["B"], inp["C"], chunk_size=32,
                           initial_states=inp["initial_states"], B_prev=inp["B_prev"],
                           U_prev=inp["U_prev"], return_state=True)
    cut = 80  # not a multiple of the chunk
    sl = lambda t, a, b_: t[:, :, a:b_].contiguous()
    y1, s1, b1, u1 = sb.v2x2ssd_b200(*(sl(inp[k], 0, cut) for k in "UMKBC"), chunk_size=32,
                                     initial_states=inp["initial_states"], B_prev=inp["B_prev"],
                                     U_prev=inp["U_prev"], return_state=True)
    y2, s2, b2, u2 = sb.v2x2ssd_b200(*(sl(inp[k], cut, 192) for k in "UMKBC"), chunk_size=32,
                                     initial_states=s1, B_prev=b1, U_prev=u1, return_state=True)
    assert rel_err(to_np(torch.cat([y1, y2], dim=2)), to_np(full[0])) < TOL_F32
    assert rel_err(to_np(s2), to_np(full[1])) < TOL_F32
    assert torch.equal(b2, full[2]) and torch.equal(u2, full[3])


def test_bitwise_repeatable():
    inp = make_scan_inputs(1, 2, 256, 64, 64, torch.bfloat16, seed=9, streaming=True, with_init=True)
    a = run_b200_fwd_bwd(inp, 64)
    b = run_b200_fwd_bwd(inp, 64)
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1])
    for name in SCAN_GRADS:
        assert torch.equal(a[2][name], b[2][name]), name


def test_no_grad_and_empty_sequence():
    import slinoss_b200 as sb

    inp = make_scan_inputs(1, 2, 64, 8, 16, torch.float32, seed=3)
    with torch.no_grad():
        y = sb.v2x2ssd_b200(inp["U"], inp["M"], inp["K"], inp["B"], inp["C"], chunk_size=32)
    Yo, _, _ = oracle_fwd_bwd(inp)
    assert rel_err(to_np(y), Yo) < TOL_F32
    e = lambda t: t[:, :, :0].contiguous()
    out = sb.v2x2ssd_b200(e(inp["U"]), e(inp["M"]), e(inp["K"]), e(inp["B"]), e(inp["C"]), chunk_size=32,
                          return_state=True)
    assert out[0].shape == (1, 2, 0, 16) and float(out[1].abs().sum()) == 0.0


def test_backend_object_matches_op():
    import slinoss_b200 as sb

    inp = make_scan_inputs(1, 2, 96, 16, 32, torch.bfloat16, seed=4, streaming=True, with_init=True)
    be = sb.B200ScanBackend()
    st = sb.ScanState(state=inp["initial_states"], b_prev=inp["B_prev"], u_prev=inp["U_prev"])
    y, nxt = be(sb.ScanInputs(inp["U"], inp["M"], inp["K"], inp["B"], inp["C"]), chunk_size=32, state=st)
    ref = sb.v2x2ssd_b200(inp["U"], inp["M"], inp["K"], inp["B"], inp["C"], chunk_size=32,
                          initial_states=inp["initial_states"], B_prev=inp["B_prev"],
                          U_prev=inp["U_prev"], return_state=True)
    assert torch.equal(y, ref[0]) and torch.equal(nxt.state, ref[1])
    assert nxt.state.dtype == torch.bfloat16 and nxt.b_prev.shape == (1, 2, 32)


@pytest.mark.parametrize("dtype,T,N,P,L", [(torch.float32, 160, 16, 32, 32), (torch.bfloat16, 384, 64, 64, 128)])
def test_two_call_backward_and_final_only_state_pass(dtype, T, N, P, L):
    """slx_v2x2ssd_bwd_begin + _finish give the bits of the single call; the first half's
    d_initial is the single call's for a zero d_final; the final-only state pass gives the
    final state of the full one."""
    import slinoss_b200 as sb
    from slinoss_b200.ops.v2x2ssd import _bwd_begin, _bwd_impl, _fwd_impl

    inp = make_scan_inputs(2, 2, T, N, P, dtype, seed=77, streaming=True, with_init=True)
    U, M, K, B, C = (inp[k] for k in ("U", "M", "K", "B", "C"))
    init, bp, up = inp["initial_states"].float(), inp["B_prev"].float(), inp["U_prev"].float()
    Y, fin, starts, mch = _fwd_impl(U, M, K, B, C, init, bp, up, L)
    dY, dfin = inp["dY"], inp["d_final"].float()
    one = _bwd_impl(U, M, K, B, C, bp, up, starts, mch, fin, dY, dfin, L, want_initial=True, want_prev=True)
    g0, ws = _bwd_begin(M, C, mch, dY, L, P)
    two = _bwd_impl(U, M, K, B, C, bp, up, starts, mch, fin, dY, dfin, L, want_initial=True, want_prev=True,
                    workspace=ws)
    for a, b_ in zip(one, two):
        assert torch.equal(a, b_)
    zero = _bwd_impl(U, M, K, B, C, bp, up, starts, mch, fin, dY, None, L, want_initial=True, want_prev=True)
    assert torch.equal(g0, zero[5])
    # the fused forward stores its increments like its chunk starts
    inc, mch2 = sb.chunk_increment_b200(U, M, K, B, B_prev=bp, U_prev=up, chunk_size=L, inc_dtype=starts.dtype)
    st_full, fin_full = sb.state_passing_b200(inc, mch2, initial_states=init, starts_dtype=starts.dtype)
    none, fin_only = sb.state_passing_b200(inc, mch2, initial_states=init, want_starts=False)
    assert none is None and torch.equal(fin_only, fin_full) and torch.equal(fin_full, fin)
    assert torch.equal(st_full, starts)


def test_views_at_odd_storage_offsets_are_handled():
    """Contiguous views whose first element is not 16-byte aligned are copied by the op; the C
    ABI itself refuses such pointers instead of issuing misaligned vector accesses."""
    import ctypes

    import slinoss_b200 as sb
    from slinoss_b200 import _lib

    inp = make_scan_inputs(1, 2, 128, 64, 64, torch.bfloat16, seed=3, dist="cfg2")

    def shifted(t):  # same values, storage offset of one element
        flat = torch.empty(t.numel() + 1, dtype=t.dtype, device=t.device)
        flat[1:].copy_(t.reshape(-1))
        return flat[1:].view(t.shape)

    args = [inp[k] for k in ("U", "M", "K", "B", "C")]
    y_ref = sb.v2x2ssd_b200(*args, chunk_size=128)
    sh = [shifted(t) for t in args]
    assert any(t.data_ptr() % 16 for t in sh)
    assert torch.equal(sb.v2x2ssd_b200(*sh, chunk_size=128), y_ref)
    U, M, K, B, C = sh
    s = _lib.scan_shape(2, 128, 64, 64, 128, torch.bfloat16)
    inc = torch.empty(1, 2, 1, 64, 128, device="cuda")
    mch = torch.empty(1, 2, 1, 2, device="cuda")
    rc = _lib.lib().slx_chunk_increment_fwd(ctypes.byref(s), U.data_ptr(), M.data_ptr(), K.data_ptr(), B.data_ptr(),
                                            None, None, inc.data_ptr(), 0, mch.data_ptr(), _lib.stream_ptr(U.device))
    assert rc == -3 and b"16-byte aligned" in _lib.lib().slx_last_error_string()


@pytest.mark.parametrize("dtype,L", [(torch.float32, 32), (torch.bfloat16, 128)])
def test_zero_transition_is_flagged_not_silently_replaced(dtype, L):
    """abs(M) == 0 makes the reference raise (reference.py:480-485).  Here the outputs of the
    zero transition's token and everything after it are NaN, a status word is set, and strict=True
    raises."""
    import slinoss_b200 as sb

    inp = make_scan_inputs(1, 2, 384, 64, 64, dtype, seed=8)
    M = inp["M"].clone()
    M[0, 1, 200] = 0.0
    args = [inp["U"], M, inp["K"], inp["B"], inp["C"]]
    sb.read_scan_status()
    y = sb.v2x2ssd_b200(*args, chunk_size=L)
    assert sb.read_scan_status() == 1 and sb.read_scan_status() == 0
    c0 = (200 // L) * L
    assert bool(torch.isfinite(y[0, 0]).all()) and bool(torch.isfinite(y[0, 1, :c0]).all())
    assert bool(torch.isnan(y[0, 1, 200:]).all())   # from the zero transition on, through every later chunk
    with pytest.raises(ValueError, match="magnitude exactly 0"):
        sb.v2x2ssd_b200(*args, chunk_size=L, strict=True)
    y_ok = sb.v2x2ssd_b200(inp["U"], inp["M"], inp["K"], inp["B"], inp["C"], chunk_size=L, strict=True)
    assert bool(torch.isfinite(y_ok).all())
