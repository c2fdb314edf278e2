"""Tensor-core (tcgen05) scan kernels against the fp32-exact CUDA-core kernels and
the CPU oracle, stage by stage, at the shapes the tensor path covers
(chunk 128, P 64, 2N in {64..256}, half inputs)."""

from __future__ import annotations

import pytest
import torch

from gpu_util import SCAN_GRADS, make_scan_inputs, oracle_fwd_bwd, run_b200_fwd_bwd, to_np
from util import rel_err

pytestmark = pytest.mark.gpu


TC = 2  # tensor-core kernel family under test (set per test by the fixture)


@pytest.fixture(autouse=True, params=[(1, 0), (2, 0), (2, 3)], ids=["per-chunk", "persistent", "persistent-3-ctas"])
def _tensor_path_on(request):
    """Every test of this file runs with both tcgen05 kernel families; the persistent one also with
    three CTAs only, so that every CTA walks several chunks (ring and barrier phases wrap around,
    the staging buffers alternate) on these small inputs."""
    import slinoss_b200 as sb
    from slinoss_b200 import _lib

    global TC
    TC, ctas = request.param
    prev = sb.set_tensor_path(TC)
    prev_ctas = _lib.set_persistent_ctas(ctas)
    yield
    sb.set_tensor_path(prev)
    _lib.set_persistent_ctas(prev_ctas)
    assert sb.read_tc_status() == 0, "a bounded completion wait ran out"


@pytest.mark.parametrize("N,T,dtype,streaming", [
    (128, 384, torch.bfloat16, True),
    (128, 300, torch.bfloat16, False),   # ragged last chunk
    (64, 256, torch.float16, True),
    (32, 128, torch.bfloat16, True),
    (96, 200, torch.bfloat16, False),
])
def test_chunk_scan_stage_tc_vs_exact(N, T, dtype, streaming):
    import slinoss_b200 as sb

    inp = make_scan_inputs(2, 2, T, N, 64, dtype, seed=N + T, streaming=streaming, with_init=True, dist="cfg2")
    kw = dict(B_prev=inp["B_prev"], U_prev=inp["U_prev"], chunk_size=128)
    inc, mch = sb.chunk_increment_b200(inp["U"], inp["M"], inp["K"], inp["B"], **kw)
    starts, _ = sb.state_passing_b200(inc, mch, initial_states=inp["initial_states"])
    y_tc = sb.chunk_scan_b200(inp["U"], inp["M"], inp["K"], inp["B"], inp["C"], starts, **kw)
    sb.set_tensor_path(False)
    y_ex = sb.chunk_scan_b200(inp["U"], inp["M"], inp["K"], inp["B"], inp["C"], starts, **kw)
    sb.set_tensor_path(TC)
    # both round Y to the half dtype; the tensor path also rounds its operands
    assert rel_err(to_np(y_tc), to_np(y_ex)) < 1e-2
    Yo, _, _ = oracle_fwd_bwd(inp)
    assert rel_err(to_np(y_tc), Yo) < 2e-2


@pytest.mark.parametrize("N,T,dtype", [(128, 512, torch.bfloat16), (64, 384, torch.float16)])
def test_full_op_tc_vs_oracle(N, T, dtype):
    inp = make_scan_inputs(2, 2, T, N, 64, dtype, seed=7, streaming=True, with_init=True, dist="cfg2")
    Y, fin, grads = run_b200_fwd_bwd(inp, 128)
    Yo, fino, go = oracle_fwd_bwd(inp)
    errs = {"Y": rel_err(to_np(Y), Yo), "final": rel_err(to_np(fin), fino)}
    errs.update({k: rel_err(to_np(grads[k]), go[k]) for k in SCAN_GRADS})
    assert all(v < 2e-2 for v in errs.values()), errs


@pytest.mark.parametrize("N,T,streaming", [(64, 1, True), (32, 5, True), (128, 127, False), (128, 129, True)])
def test_short_and_one_past_a_chunk_tc_vs_oracle(N, T, streaming):
    """Sequences shorter than one 128-token chunk (row 127 of every tile is padding and doubles as the slot of
    the token in front of the chunk) and one token past a chunk, with and without streaming inputs."""
    inp = make_scan_inputs(2, 2, T, N, 64, torch.bfloat16, seed=T, streaming=streaming, with_init=True, dist="cfg2")
    Y, fin, grads = run_b200_fwd_bwd(inp, 128)
    Yo, fino, go = oracle_fwd_bwd(inp)
    errs = {"Y": rel_err(to_np(Y), Yo), "final": rel_err(to_np(fin), fino)}
    errs.update({k: rel_err(to_np(grads[k]), go[k]) for k in SCAN_GRADS if grads[k] is not None})
    assert all(v < 2e-2 for v in errs.values()), errs


@pytest.mark.parametrize("N,T,dtype", [(128, 300, torch.bfloat16), (32, 256, torch.float16), (96, 128, torch.bfloat16)])
def test_increment_stage_tc_vs_exact(N, T, dtype):
    import slinoss_b200 as sb

    inp = make_scan_inputs(2, 2, T, N, 64, dtype, seed=N, streaming=True, with_init=False, dist="cfg2")
    kw = dict(B_prev=inp["B_prev"], U_prev=inp["U_prev"], chunk_size=128)
    inc_tc, m_tc = sb.chunk_increment_b200(inp["U"], inp["M"], inp["K"], inp["B"], **kw)
    sb.set_tensor_path(False)
    inc_ex, m_ex = sb.chunk_increment_b200(inp["U"], inp["M"], inp["K"], inp["B"], **kw)
    sb.set_tensor_path(TC)
    assert rel_err(to_np(m_tc), to_np(m_ex)) < 1e-6
    assert rel_err(to_np(inc_tc), to_np(inc_ex)) < 5e-3


@pytest.mark.parametrize("N,T,dtype", [(128, 640, torch.bfloat16), (32, 300, torch.float16)])
def test_half_increments_are_the_rounded_fp32_ones(N, T, dtype):
    """The whole-op entry points keep the chunk increments in the activation dtype.  At stage level:
    ``inc_dtype`` = that dtype gives exactly the fp32 increments rounded once, and the state pass
    reads them as those values (its recurrence stays fp32)."""
    import slinoss_b200 as sb

    inp = make_scan_inputs(2, 2, T, N, 64, dtype, seed=N + 1, streaming=True, with_init=True, dist="cfg2")
    kw = dict(B_prev=inp["B_prev"], U_prev=inp["U_prev"], chunk_size=128)
    inc32, mch = sb.chunk_increment_b200(inp["U"], inp["M"], inp["K"], inp["B"], **kw)
    inc16, mch16 = sb.chunk_increment_b200(inp["U"], inp["M"], inp["K"], inp["B"], inc_dtype=dtype, **kw)
    assert inc16.dtype == dtype and torch.equal(inc16, inc32.to(dtype)) and torch.equal(mch, mch16)
    st_a, fin_a = sb.state_passing_b200(inc16, mch, initial_states=inp["initial_states"], starts_dtype=dtype)
    st_b, fin_b = sb.state_passing_b200(inc16.float(), mch, initial_states=inp["initial_states"], starts_dtype=dtype)
    assert torch.equal(st_a, st_b) and torch.equal(fin_a, fin_b)
    _, fin_c = sb.state_passing_b200(inc16, mch, initial_states=inp["initial_states"], want_starts=False)
    assert torch.equal(fin_c, fin_a)
    # against the fp32 increments the final state moves by the storage rounding only
    _, fin32 = sb.state_passing_b200(inc32, mch, initial_states=inp["initial_states"])
    assert rel_err(to_np(fin_a), to_np(fin32)) < (4e-3 if dtype == torch.bfloat16 else 6e-4)
    with pytest.raises(TypeError):
        sb.state_passing_b200(inc16, mch, starts_dtype=torch.float32)


@pytest.mark.parametrize("N,T,dtype,streaming", [
    (128, 384, torch.bfloat16, True),
    (128, 200, torch.bfloat16, False),   # ragged last chunk
    (32, 256, torch.float16, True),
    (96, 128, torch.bfloat16, True),
])
def test_backward_tc_vs_exact_and_oracle(N, T, dtype, streaming):
    """Tensor-core backward against the fp32-exact kernels (same half inputs) and the oracle."""
    import slinoss_b200 as sb

    inp = make_scan_inputs(2, 2, T, N, 64, dtype, seed=3 * N + T, streaming=streaming, with_init=True,
                           dist="cfg2")
    Y, fin, g_tc = run_b200_fwd_bwd(inp, 128)
    sb.set_tensor_path(False)
    Y2, fin2, g_ex = run_b200_fwd_bwd(inp, 128)
    sb.set_tensor_path(TC)
    Yo, fino, go = oracle_fwd_bwd(inp)
    errs_ex, errs_or = {}, {}
    for k in SCAN_GRADS:
        if g_tc[k] is None:
            continue
        errs_ex[k] = rel_err(to_np(g_tc[k]), to_np(g_ex[k]))
        errs_or[k] = rel_err(to_np(g_tc[k]), go[k])
    assert all(v < 2e-2 for v in errs_or.values()), ("oracle", errs_or, "exact", errs_ex)
    assert all(v < 2e-2 for v in errs_ex.values()), ("exact", errs_ex)


def test_strong_decay_takes_per_element_path():
    """Multipliers of magnitude < exp(-1.9) switch a chunk from the factored decay table to one
    exponential per score; both paths must agree with the oracle."""
    inp = make_scan_inputs(1, 2, 384, 64, 64, torch.bfloat16, seed=91, streaming=True, with_init=True,
                           dist="tests")
    M = inp["M"].clone()
    M[:, 0, ::7] *= 0.2          # head 0: every 7th token has |m| in [0.12, 0.19]; head 1 stays on the table path
    inp["M"] = M.contiguous()
    Y, fin, grads = run_b200_fwd_bwd(inp, 128)
    Yo, fino, go = oracle_fwd_bwd(inp)
    errs = {"Y": rel_err(to_np(Y), Yo), "final": rel_err(to_np(fin), fino)}
    errs.update({k: rel_err(to_np(grads[k]), go[k]) for k in SCAN_GRADS if grads[k] is not None})
    # dM is the accumulated sum divided by conj(m): small |m| amplifies the half-precision
    # rounding of that sum, so dM alone gets a wider band here
    tol = {k: 2e-2 for k in errs}
    tol["dM"] = 4e-2
    assert all(errs[k] < tol[k] for k in errs), errs


def test_requested_chunk_is_retiled_to_the_tensor_chunk():
    """chunk_size is a tiling hint: half inputs at P=64 run in 128-token chunks whatever is asked."""
    import slinoss_b200 as sb

    inp = make_scan_inputs(1, 2, 320, 64, 64, torch.bfloat16, seed=5, dist="cfg2")
    args = [inp[k] for k in ("U", "M", "K", "B", "C")]
    y64 = sb.v2x2ssd_b200(*args, chunk_size=64)
    y128 = sb.v2x2ssd_b200(*args, chunk_size=128)
    assert torch.equal(y64, y128)
    y_exact = sb.v2x2ssd_b200(*args, chunk_size=64, retile=False)
    assert not torch.equal(y_exact, y128)
    assert rel_err(to_np(y_exact), to_np(y128)) < 1e-2


def test_residual_formats():
    """What autograd keeps of the chunk-start states: 'recompute' gives the bits of the default."""
    import slinoss_b200 as sb

    inp = make_scan_inputs(2, 2, 512, 128, 64, torch.bfloat16, seed=17, streaming=True, with_init=True, dist="cfg2")

    def run(residual):
        lv = {k: inp[k].detach().clone().requires_grad_(True) for k in ("U", "M", "K", "B", "C", "initial_states",
                                                                       "B_prev", "U_prev")}
        Y, fin, _, _ = sb.v2x2ssd_b200(lv["U"], lv["M"], lv["K"], lv["B"], lv["C"], chunk_size=128,
                                       initial_states=lv["initial_states"], B_prev=lv["B_prev"],
                                       U_prev=lv["U_prev"], return_state=True, residual=residual)
        g = torch.autograd.grad([Y, fin], list(lv.values()), [inp["dY"], inp["d_final"].to(fin.dtype)])
        return Y, g

    y0, g0 = run("keep")
    y1, g1 = run("recompute")
    assert torch.equal(y0, y1) and all(torch.equal(a, b) for a, b in zip(g0, g1))
    with pytest.raises(ValueError, match="residual must be"):
        sb.v2x2ssd_b200(inp["U"], inp["M"], inp["K"], inp["B"], inp["C"], chunk_size=128, residual="fp16")


def test_chunk_starts_dtype_follows_the_kernel_path():
    """The stages exchange chunk_starts in the activation dtype where the tensor-core kernels run
    and in fp32 elsewhere; the stage-level functions accept either and convert."""
    import slinoss_b200 as sb
    from slinoss_b200 import _lib
    from slinoss_b200.ops.v2x2ssd import _fwd_impl, _shape

    inp = make_scan_inputs(1, 2, 256, 64, 64, torch.bfloat16, seed=4, dist="cfg2")
    U, M, K, B, C = (inp[k] for k in ("U", "M", "K", "B", "C"))
    assert _lib.starts_dtype(_shape(1, 2, 256, 64, 64, 128, torch.bfloat16)) == torch.bfloat16
    assert _lib.starts_dtype(_shape(1, 2, 256, 64, 64, 64, torch.bfloat16)) == torch.float32
    assert _lib.starts_dtype(_shape(1, 2, 256, 64, 64, 128, torch.float32)) == torch.float32
    Y, fin, starts, mch = _fwd_impl(U, M, K, B, C, None, None, None, 128)
    assert starts.dtype == torch.bfloat16
    # the fused op keeps its increments in the activation dtype too; fp32 starts from those increments
    inc, mch2 = sb.chunk_increment_b200(U, M, K, B, chunk_size=128, inc_dtype=torch.bfloat16)
    st32, fin2 = sb.state_passing_b200(inc.float(), mch2)
    assert st32.dtype == torch.float32 and torch.equal(fin2, fin)
    assert torch.equal(st32.to(torch.bfloat16), starts)          # same recurrence, one rounding
    y_stage = sb.chunk_scan_b200(U, M, K, B, C, st32, chunk_size=128)   # fp32 starts are converted
    assert torch.equal(y_stage, Y)
