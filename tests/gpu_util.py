"""Helpers of the GPU parity tests (seeded inputs, oracle calls)."""

from __future__ import annotations

import math

import numpy as np
import torch

from oracle import scan as oscan

SCAN_GRADS = ("dU", "dM", "dK", "dB", "dC", "d_initial", "dB_prev", "dU_prev")


def make_scan_inputs(b, h, T, N, P, dtype, *, seed, streaming=False, with_init=False,
                     dist="tests", device="cuda"):
    """dist="tests": the reference tests' generator (tests/test_v2x2ssd_cute.py:25-67);
    dist="cfg2": radius sigmoid(N(2,1)), angle tanh(N(0,1))*pi/4, B,C ~ N(0,1/N)."""
    g = torch.Generator().manual_seed(seed)
    if dist == "tests":
        radius = 0.6 + 0.35 * torch.rand((b, h, T), generator=g)
        angle = (2.0 * math.pi) * torch.rand((b, h, T), generator=g) - math.pi
        bscale = 0.1
    else:
        radius = torch.sigmoid(2.0 + torch.randn((b, h, T), generator=g))
        angle = torch.tanh(torch.randn((b, h, T), generator=g)) * (math.pi / 4)
        bscale = 1.0 / math.sqrt(N)
    M = torch.view_as_real(torch.polar(radius, angle)).float().contiguous()
    K = (torch.randn((b, h, T, 2, 2), generator=g) * 0.1).float()
    U = torch.randn((b, h, T, P), generator=g).to(dtype)
    B = (torch.randn((b, h, T, 2 * N), generator=g) * bscale).to(dtype)
    C = (torch.randn((b, h, T, 2 * N), generator=g) * bscale).to(dtype)
    init = torch.randn((b, h, P, 2 * N), generator=g).float() if with_init else None
    Bp = (torch.randn((b, h, 2 * N), generator=g) * bscale).to(dtype) if streaming else None
    Up = torch.randn((b, h, P), generator=g).to(dtype) if streaming else None
    dY = torch.randn((b, h, T, P), generator=g).to(dtype)
    dfin = (torch.randn((b, h, P, 2 * N), generator=g) * 0.1).to(dtype).float()
    dev = torch.device(device)
    mv = lambda t: None if t is None else t.to(dev)
    return dict(U=mv(U), M=mv(M), K=mv(K), B=mv(B), C=mv(C), initial_states=mv(init),
                B_prev=mv(Bp), U_prev=mv(Up), dY=mv(dY), d_final=mv(dfin))


def to_np(t):
    return None if t is None else t.detach().float().cpu().numpy().astype(np.float64)


def oracle_fwd_bwd(inp, *, with_final_grad=True):
    kw = dict(initial_states=to_np(inp["initial_states"]), B_prev=to_np(inp["B_prev"]),
              U_prev=to_np(inp["U_prev"]))
    args = [to_np(inp[k]) for k in ("U", "M", "K", "B", "C")]
    Y, fin = oscan.v2x2ssm_fwd(*args, **kw)
    grads = oscan.v2x2ssm_bwd(*args, dY=to_np(inp["dY"]),
                              d_final=to_np(inp["d_final"]) if with_final_grad else None, **kw)
    return Y, fin, grads


def run_b200_fwd_bwd(inp, chunk_size, *, with_final_grad=True):
    import slinoss_b200 as sb

    leaves = {}
    for k in ("U", "M", "K", "B", "C", "initial_states", "B_prev", "U_prev"):
        t = inp[k]
        leaves[k] = None if t is None else t.detach().clone().requires_grad_(True)
    Y, fin, b_last, u_last = sb.v2x2ssd_b200(
        leaves["U"], leaves["M"], leaves["K"], leaves["B"], leaves["C"], chunk_size=chunk_size,
        initial_states=leaves["initial_states"], B_prev=leaves["B_prev"], U_prev=leaves["U_prev"],
        return_state=True)
    outs, gouts = [Y], [inp["dY"]]
    if with_final_grad:
        outs.append(fin)
        gouts.append(inp["d_final"].to(fin.dtype))
    names = [k for k in leaves if leaves[k] is not None]
    grads = torch.autograd.grad(outs, [leaves[k] for k in names], gouts)
    gmap = dict(zip(names, grads))
    out = dict(dU=gmap["U"], dM=gmap["M"], dK=gmap["K"], dB=gmap["B"], dC=gmap["C"],
               d_initial=gmap.get("initial_states"), dB_prev=gmap.get("B_prev"),
               dU_prev=gmap.get("U_prev"))
    return Y, fin, out
