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


class OracleEngine:
    """The four engine calls of slinoss_b200.context_parallel, served by oracle/."""

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


def _worker(rank, world, port, T, L, out_dir):
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
        grads = torch.autograd.grad(outs, leaves + ([init_l] if rank == 0 else []), gouts, allow_unused=True)
        np.savez(Path(out_dir) / f"r{rank}.npz", Y=Y.detach().numpy(), fin=fin.detach().numpy(), lo=lo, hi=hi,
                 **{f"g{i}": g.numpy() for i, g in enumerate(grads)})
    finally:
        dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


@pytest.mark.parametrize("world,T,L", [(2, 70, 16), (3, 100, 16)])
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
