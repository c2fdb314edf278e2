"""The headline workload itself (b4 H32 P64 N128 T8192, bf16 in / fp32 state, tensor-core path):
size-independent properties on the whole tensors, and (batch, head) slices against the oracle.

Every (batch, head) pair is an independent sequence, so a slice of the full-size result must
equal what the float64 oracle computes for that sequence alone."""

from __future__ import annotations

import numpy as np
import pytest
import torch

from gpu_util import SCAN_GRADS, make_scan_inputs, oracle_fwd_bwd, run_b200_fwd_bwd, to_np
from util import rel_err

pytestmark = pytest.mark.gpu

B, H, T, N, P, L = 4, 32, 8192, 128, 64, 128


@pytest.fixture(scope="module")
def headline():
    inp = make_scan_inputs(B, H, T, N, P, torch.bfloat16, seed=2024, streaming=True, with_init=True, dist="cfg2")
    Y, fin, grads = run_b200_fwd_bwd(inp, L)
    torch.cuda.synchronize()
    return inp, Y, fin, grads


def _slice(inp, b, h):
    out = {}
    for k, v in inp.items():
        out[k] = None if v is None else v[b:b + 1, h:h + 1].contiguous()
    return out


@pytest.mark.parametrize("b,h", [(0, 0), (2, 17), (3, 31)])
def test_slices_of_the_headline_run_match_the_oracle(headline, b, h):
    inp, Y, fin, grads = headline
    Yo, fino, go = oracle_fwd_bwd(_slice(inp, b, h))
    errs = {"Y": rel_err(to_np(Y[b:b + 1, h:h + 1]), Yo), "final": rel_err(to_np(fin[b:b + 1, h:h + 1]), fino)}
    for k in SCAN_GRADS:
        errs[k] = rel_err(to_np(grads[k][b:b + 1, h:h + 1]), go[k])
    assert all(np.isfinite(v) and v < 2e-2 for v in errs.values()), errs


def test_headline_run_is_finite_and_repeatable(headline):
    inp, Y, fin, grads = headline
    for name, t in [("Y", Y), ("final", fin)] + [(k, grads[k]) for k in SCAN_GRADS]:
        assert bool(torch.isfinite(t).all()), name
    Y2, fin2, grads2 = run_b200_fwd_bwd(inp, L)
    assert torch.equal(Y, Y2) and torch.equal(fin, fin2)
    for k in SCAN_GRADS:
        assert torch.equal(grads[k], grads2[k]), k


def test_headline_segment_chaining(headline):
    """[0, T/2) then [T/2, T) through the carried state reproduces the single pass."""
    import slinoss_b200 as sb

    inp, Y, fin, _ = headline
    cut = T // 2
    sl = lambda t, a, b_: t[:, :, a:b_].contiguous()
    with torch.no_grad():
        y1, s1, b1, u1 = sb.v2x2ssd_b200(*(sl(inp[k], 0, cut) for k in "UMKBC"), chunk_size=L,
                                         initial_states=inp["initial_states"], B_prev=inp["B_prev"],
                                         U_prev=inp["U_prev"], return_state=True, output_dtype=torch.float32)
        y2, s2, _, _ = sb.v2x2ssd_b200(*(sl(inp[k], cut, T) for k in "UMKBC"), chunk_size=L, initial_states=s1,
                                       B_prev=b1, U_prev=u1, return_state=True, output_dtype=torch.float32)
    # the first half is the same computation chunk for chunk; the second half differs only in how
    # its start state was rounded on the way through the carried tensors
    assert rel_err(to_np(y1), to_np(Y[:, :, :cut])) < 5e-3
    assert rel_err(to_np(y2), to_np(Y[:, :, cut:])) < 5e-3
    assert rel_err(to_np(s2), to_np(fin)) < 5e-3


def test_headline_forward_is_linear_in_u(headline):
    """Y is linear in (U, U_prev) for fixed M, K, B, C and a zero initial state: Y(2U) = 2 Y(U)
    exactly in binary floating point (a power-of-two scale commutes with every rounding)."""
    import slinoss_b200 as sb

    inp, _, _, _ = headline
    args = [inp[k] for k in ("M", "K", "B", "C")]
    with torch.no_grad():
        y1 = sb.v2x2ssd_b200(inp["U"], *args, chunk_size=L, B_prev=inp["B_prev"], U_prev=inp["U_prev"])
        y2 = sb.v2x2ssd_b200(inp["U"] * 2, *args, chunk_size=L, B_prev=inp["B_prev"], U_prev=inp["U_prev"] * 2)
    assert torch.equal(y2, y1 * 2)


def test_long_sequence_slice_matches_the_oracle():
    """The long-context length (262144 tokens = 2048 chunks of 128; batch 1, two heads, bf16 inputs,
    fp32 state): this is where rounding the chunk-start states and their gradients to bf16 between
    the stages, once per chunk boundary, would accumulate if it mattered.  One head of the run is
    compared with the float64 oracle of that head alone: Y, final state and the five gradients within
    the bf16 contract (relative L2 <= 2e-2)."""
    Tl = 262144
    inp = make_scan_inputs(1, 2, Tl, N, P, torch.bfloat16, seed=4096, streaming=False, with_init=False, dist="cfg2")
    Y, fin, grads = run_b200_fwd_bwd(inp, L)
    torch.cuda.synchronize()
    sl = _slice(inp, 0, 1)
    Yo, fino, go = oracle_fwd_bwd(sl)
    errs = {"Y": rel_err(to_np(Y[:, 1:2]), Yo), "final": rel_err(to_np(fin[:, 1:2]), fino)}
    for k in ("dU", "dM", "dK", "dB", "dC"):
        errs[k] = rel_err(to_np(grads[k][:, 1:2]), go[k])
    print("[long sequence]", {k: f"{v:.2e}" for k, v in errs.items()})
    assert all(np.isfinite(v) and v < 2e-2 for v in errs.values()), errs
