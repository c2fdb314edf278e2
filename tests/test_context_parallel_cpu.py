"""Context-parallel scan: message pattern and chaining algebra on CPU ranks
(gloo, world sizes 2 and 3) with the CPU oracle as the local engine, against a
single-process run over the whole sequence."""

from __future__ import annotations

import os
import socket
import sys
from pathlib import Path

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

ROOT = Path(__file__).resolve().parents[1]


from slinoss_b200.context_parallel import TorchSegmentAlgebra


class OracleEngine(TorchSegmentAlgebra):
    """The engine calls of slinoss_b200.context_parallel, served by oracle/ (the segment algebra
    comes from the package's plain-torch mix-in)."""

    @staticmethod
    def _np(t):
        return None if t is None else t.detach().double().numpy()

    @staticmethod
    def _t(x):
        return torch.from_numpy(np.ascontiguousarray(x)).float()

    def forward_parts(self, U, M, K, B, Bp, Up, L):
        from oracle import scan as oscan

        inc, mch = oscan.chunk_increment(*map(self._np, (U, M, K, B)), B_prev=self._np(Bp), U_prev=self._np(Up),
                                         chunk_size=L)
        _, f0 = oscan.state_passing(inc, mch, initial_states=None)
        return self._t(inc), self._t(mch), self._t(f0)

    def forward_finish(self, U, M, K, B, C, inc, mch, z_in, Bp, Up, L):
        from oracle import scan as oscan

        starts, final = oscan.state_passing(self._np(inc), self._np(mch), initial_states=self._np(z_in))
        Y = oscan.chunk_scan(*map(self._np, (U, M, K, B, C)), starts, B_prev=self._np(Bp), U_prev=self._np(Up),
                             chunk_size=L)
        return self._t(Y), self._t(starts), self._t(final)

    def backward_zero(self, U, M, K, B, C, mch, starts, final, dY, L):
        from oracle import scan as oscan

        g = oscan.v2x2ssm_bwd(*map(self._np, (U, M, K, B, C)), dY=self._np(dY),
                              initial_states=np.zeros(tuple(final.shape)))
        return self._t(g["d_initial"])

    def backward_full(self, U, M, K, B, C, Bp, Up, mch, starts, final, dY, d_final, L):
        from oracle import scan as oscan

        g = oscan.v2x2ssm_bwd(*map(self._np, (U, M, K, B, C)), dY=self._np(dY), d_final=self._np(d_final),
                              initial_states=self._np(starts[:, :, 0]), B_prev=self._np(Bp), U_prev=self._np(Up))
        t = self._t
        return (t(g["dU"]), t(g["dM"]), t(g["dK"]), t(g["dB"]), t(g["dC"]), t(g["d_initial"]),
                t(g["dB_prev"]) if Bp is not None else None, t(g["dU_prev"]) if Bp is not None else None)


def _inputs(T, seed=0):
    g = torch.Generator().manual_seed(seed)
    b, h, P, N = 1, 2, 4, 3
    radius = 0.7 + 0.25 * torch.rand((b, h, T), generator=g)
    angle = 2.0 * torch.rand((b, h, T), generator=g) - 1.0
    M = torch.view_as_real(torch.polar(radius, angle)).contiguous()
    K = torch.randn((b, h, T, 2, 2), generator=g) * 0.3
    U = torch.randn((b, h, T, P), generator=g)
    B = torch.randn((b, h, T, 2 * N), generator=g) * 0.5
    C = torch.randn((b, h, T, 2 * N), generator=g) * 0.5
    init = torch.randn((b, h, P, 2 * N), generator=g)
    dY = torch.randn((b, h, T, P), generator=g)
    dfin = torch.randn((b, h, P, 2 * N), generator=g)
    return U, M, K, B, C, init, dY, dfin


def _mid_cotangent(shape, rank):
    return torch.randn(shape, generator=torch.Generator().manual_seed(100 + rank))


def _worker(rank, world, port, T, L, out_dir, mid_final_grad=False):
    sys.path.insert(0, str(ROOT))
    sys.path.insert(0, str(ROOT / "tests"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from slinoss_b200.context_parallel import v2x2ssd_context_parallel

        U, M, K, B, C, init, dY, dfin = _inputs(T)
        # slices: multiples of L on every rank but the last, which takes the ragged rest
        per = (T // world // L) * L
        lo = rank * per
        hi = T if rank == world - 1 else lo + per
        leaves = [t[:, :, lo:hi].contiguous().requires_grad_(True) for t in (U, M, K, B, C)]
        init_l = init.clone().requires_grad_(True) if rank == 0 else None
        Y, fin = v2x2ssd_context_parallel(*leaves, chunk_size=L, initial_states=init_l, engine=OracleEngine())
        outs, gouts = [Y], [dY[:, :, lo:hi]]
        if rank == world - 1:
            outs.append(fin)
            gouts.append(dfin)
        elif mid_final_grad:
            # a cotangent on an intermediate rank's end-of-segment state
            outs.append(fin)
            gouts.append(_mid_cotangent(fin.shape, rank))
        grads = torch.autograd.grad(outs, leaves + ([init_l] if rank == 0 else []), gouts, allow_unused=True)
        np.savez(Path(out_dir) / f"r{rank}.npz", Y=Y.detach().numpy(), fin=fin.detach().numpy(), lo=lo, hi=hi,
                 **{f"g{i}": g.numpy() for i, g in enumerate(grads)})
    finally:
        dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("world,T,L", [(2, 70, 16), (3, 100, 16), (4, 130, 16)])
def test_context_parallel_matches_single_pass(tmp_path, world, T, L):
    from oracle import scan as oscan
    from util import rel_err

    mp.spawn(_worker, args=(world, _free_port(), T, L, str(tmp_path)), nprocs=world, join=True)
    U, M, K, B, C, init, dY, dfin = _inputs(T)
    n = lambda t: t.double().numpy()
    Yo, fino = oscan.v2x2ssm_fwd(n(U), n(M), n(K), n(B), n(C), initial_states=n(init))
    go = oscan.v2x2ssm_bwd(n(U), n(M), n(K), n(B), n(C), dY=n(dY), d_final=n(dfin), initial_states=n(init))
    names = ["dU", "dM", "dK", "dB", "dC"]
    for r in range(world):
        z = np.load(tmp_path / f"r{r}.npz")
        lo, hi = int(z["lo"]), int(z["hi"])
        assert rel_err(z["Y"], Yo[:, :, lo:hi]) < 2e-6
        for i, name in enumerate(names):
            assert rel_err(z[f"g{i}"], go[name][:, :, lo:hi]) < 5e-6, (r, name)
        if r == world - 1:
            assert rel_err(z["fin"], fino) < 2e-6
        if r == 0:
            assert rel_err(z["g5"], go["d_initial"]) < 5e-6


def test_cotangent_on_an_intermediate_final_state_is_honoured(tmp_path):
    """Every rank returns its end-of-segment state as a differentiable output.  A loss on rank r's
    state (r < R-1) must reach the gradients of all tokens before the end of segment r: checked
    against one pass in which the same state is the final state of the prefix [0, hi_r)."""
    from oracle import scan as oscan
    from util import rel_err

    world, T, L = 3, 100, 16
    mp.spawn(_worker, args=(world, _free_port(), T, L, str(tmp_path), True), nprocs=world, join=True)
    U, M, K, B, C, init, dY, dfin = _inputs(T)
    n = lambda t: t.double().numpy()
    go = oscan.v2x2ssm_bwd(n(U), n(M), n(K), n(B), n(C), dY=n(dY), d_final=n(dfin), initial_states=n(init))
    names = ["dU", "dM", "dK", "dB", "dC"]
    total = {k: go[k].copy() for k in names}
    total["d_initial"] = go["d_initial"].copy()
    per = (T // world // L) * L
    for r in range(world - 1):  # add the gradient of <cotangent_r, state at the end of segment r>
        hi = (r + 1) * per
        cot = _mid_cotangent((1, 2, 4, 6), r).double().numpy()
        gp = oscan.v2x2ssm_bwd(*(n(t)[:, :, :hi] for t in (U, M, K, B, C)), dY=np.zeros_like(n(dY)[:, :, :hi]),
                               d_final=cot, initial_states=n(init))
        for k in names:
            total[k][:, :, :hi] += gp[k]
        total["d_initial"] += gp["d_initial"]
    for r in range(world):
        z = np.load(tmp_path / f"r{r}.npz")
        lo, hi = int(z["lo"]), int(z["hi"])
        for i, name in enumerate(names):
            assert rel_err(z[f"g{i}"], total[name][:, :, lo:hi]) < 5e-6, (r, name)
        if r == 0:
            assert rel_err(z["g5"], total["d_initial"]) < 5e-6


def _absent_peer_worker(rank, world, port, out_dir):
    import datetime

    sys.path.insert(0, str(ROOT))
    sys.path.insert(0, str(ROOT / "tests"))
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=4))
    import time

    from slinoss_b200.context_parallel import v2x2ssd_context_parallel

    U, M, K, B, C, init, dY, dfin = _inputs(64)
    lo, hi = rank * 32, (rank + 1) * 32
    leaves = [t[:, :, lo:hi].contiguous() for t in (U, M, K, B, C)]
    result = "no call"
    t0 = time.perf_counter()
    if rank == 0:
        try:
            v2x2ssd_context_parallel(*leaves, chunk_size=16, engine=OracleEngine())
            result = "returned"
        except RuntimeError as e:
            result = f"RuntimeError after {time.perf_counter() - t0:.1f}s: {str(e)[:120]}"
    else:
        time.sleep(8)  # the peer is alive but never makes the call
    (Path(out_dir) / f"r{rank}.txt").write_text(result)
    # no destroy_process_group: after a failed collective the group is not reusable; the process ends here
    os._exit(0)


def test_a_peer_that_never_joins_raises_instead_of_hanging(tmp_path):
    """Host-side failure handling: rank 1 never enters the exchange; rank 0 must get a Python
    exception within the process group's timeout (4 s here), not wait forever."""
    world = 2
    mp.spawn(_absent_peer_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    msg = (tmp_path / "r0.txt").read_text()
    assert msg.startswith("RuntimeError after"), msg
    assert "context-parallel exchange" in msg
    secs = float(msg.split("after ")[1].split("s")[0])
    assert secs < 8.0, msg
