"""Context-parallel v2x2ssd: one long sequence split over the ranks of a process
group, with only chunk-final states (and one-token halos) crossing ranks.

The reference has no distributed code; what it has is the segment-chaining
contract (running ``[0:t)`` then ``[t:T)`` through ``ScanState`` reproduces one
pass, reference tests/test_v2x2ssd_cute.py:818-929).  This module distributes
exactly that contract.  Rank ``r`` owns tokens ``[r*T/R, (r+1)*T/R)``.

Forward
  1. halo: the last token's ``(B, U)`` row goes to rank ``r+1`` (its ``B_prev, U_prev``).
  2. every rank, in parallel: chunk increments and a state pass from a ZERO start,
     giving ``f0`` (its segment's affine offset) and ``m_seg = prod m_chunk``.
  3. chain (R-1 hops of one (b,H,P,2N) fp32 state): ``z_out = m_seg * z_in + f0``.
  4. every rank: state pass from its true ``z_in``, then the chunk scan.
Backward mirrors it: every rank computes its reverse pass from a zero
``d_final`` (``g0``), the true ``d_final`` is chained from the last rank down with
``d_initial = g0 + conj(m_seg) * d_final``, every rank then runs its full
backward, and the halo gradients return to the previous rank's last row.

All arithmetic is done by an *engine* (the sm_100a kernels by default); the
message pattern is engine-independent and is tested on CPU ranks (gloo) with a
CPU engine.
"""

from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.distributed as dist


def _cmul(m: torch.Tensor, z: torch.Tensor) -> torch.Tensor:
    """(b,h,2) packed complex times (b,h,P,2N) interleaved complex state."""
    zc = torch.view_as_complex(z.reshape(*z.shape[:-1], z.shape[-1] // 2, 2).contiguous())
    mc = torch.view_as_complex(m.contiguous())[..., None, None]
    return torch.view_as_real(mc * zc).reshape(z.shape).contiguous()


def _segment_transition(m_chunk: torch.Tensor) -> torch.Tensor:
    """prod over chunks of the packed complex chunk transitions: (b,h,C,2) -> (b,h,2)."""
    return torch.view_as_real(torch.view_as_complex(m_chunk.contiguous()).prod(dim=2)).contiguous()


class B200Engine:
    """Local arithmetic on the sm_100a kernels (through the C ABI)."""

    def forward_parts(self, U, M, K, B, Bp, Up, L):
        from .ops.v2x2ssd import chunk_increment_b200, state_passing_b200

        inc, mch = chunk_increment_b200(U, M, K, B, B_prev=Bp, U_prev=Up, chunk_size=L)
        _, f0 = state_passing_b200(inc, mch, initial_states=None, want_starts=False)
        return inc, mch, f0

    def forward_finish(self, U, M, K, B, C, inc, mch, z_in, Bp, Up, L):
        from .ops.v2x2ssd import chunk_scan_b200, state_passing_b200

        from . import _lib
        from .ops.v2x2ssd import _shape

        b, h, T, P = map(int, U.shape)
        sdt = _lib.starts_dtype(_shape(b, h, T, P, int(B.shape[-1]) // 2, L, U.dtype))
        starts, final = state_passing_b200(inc, mch, initial_states=z_in, starts_dtype=sdt)
        Y = chunk_scan_b200(U, M, K, B, C, starts, B_prev=Bp, U_prev=Up, chunk_size=L)
        return Y, starts, final

    def backward_zero(self, U, M, K, B, C, mch, starts, final, dY, L):
        """d_initial of the segment for d_final = 0, plus the workspace that already holds dZ0
        (handed back to ``backward_full`` so that it is not computed twice)."""
        from .ops.v2x2ssd import _bwd_begin

        return _bwd_begin(M, C, mch, dY, L, int(U.shape[-1]))

    def backward_full(self, U, M, K, B, C, Bp, Up, mch, starts, final, dY, d_final, L, token=None):
        from .ops.v2x2ssd import _bwd_impl

        return _bwd_impl(U, M, K, B, C, Bp, Up, starts, mch, final, dY, d_final, L, want_initial=True,
                         want_prev=Bp is not None, workspace=token)


def _send(t, dst, group):
    dist.send(t.contiguous(), dst=dist.get_global_rank(group, dst) if group is not None else dst, group=group)


def _recv(t, src, group):
    dist.recv(t, src=dist.get_global_rank(group, src) if group is not None else src, group=group)
    return t


class _ContextParallelScanFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, U, M, K, B, C, initial_states, L, group, engine):
        R, r = dist.get_world_size(group), dist.get_rank(group)
        b, h, T, P = map(int, U.shape)
        D = int(B.shape[-1])
        dev = U.device
        U, M, K, B, C = (t.detach() for t in (U, M, K, B, C))
        # 1. halo
        Bp = Up = None
        if r + 1 < R:
            halo = torch.cat([B[:, :, -1, :].float(), U[:, :, -1, :].float()], dim=-1).contiguous()
            _send(halo, r + 1, group)
        if r > 0:
            halo_in = _recv(torch.empty((b, h, D + P), device=dev, dtype=torch.float32), r - 1, group)
            Bp, Up = halo_in[..., :D].contiguous(), halo_in[..., D:].contiguous()
        # 2. local parts from a zero start
        inc, mch, f0 = engine.forward_parts(U, M, K, B, Bp, Up, L)
        m_seg = _segment_transition(mch)
        # 3. chain of segment-final states
        if r == 0:
            z_in = None if initial_states is None else initial_states.detach().float().contiguous()
        else:
            z_in = _recv(torch.empty((b, h, P, D), device=dev, dtype=torch.float32), r - 1, group)
        z_out = f0 if z_in is None else _cmul(m_seg, z_in) + f0
        if r + 1 < R:
            _send(z_out, r + 1, group)
        # 4. finish locally
        Y, starts, final = engine.forward_finish(U, M, K, B, C, inc, mch, z_in, Bp, Up, L)
        ctx.L, ctx.group, ctx.engine = L, group, engine
        ctx.has_init = initial_states is not None
        ctx.has_prev = Bp is not None
        ctx.init_dtype = None if initial_states is None else initial_states.dtype
        saved = [U, M, K, B, C, mch, starts, final, m_seg]
        if Bp is not None:
            saved += [Bp, Up]
        ctx.save_for_backward(*saved)
        return Y, final

    @staticmethod
    def backward(ctx, dY, d_final_in):
        saved = ctx.saved_tensors
        U, M, K, B, C, mch, starts, final, m_seg = saved[:9]
        Bp, Up = (saved[9], saved[10]) if ctx.has_prev else (None, None)
        group, engine, L = ctx.group, ctx.engine, ctx.L
        R, r = dist.get_world_size(group), dist.get_rank(group)
        b, h, T, P = map(int, U.shape)
        D = int(B.shape[-1])
        dev = U.device
        dY = torch.zeros_like(U) if dY is None else dY.to(U.dtype).contiguous()
        # reverse chain of d_final: d_initial(r) = g0(r) + conj(m_seg(r)) d_final(r)
        res = engine.backward_zero(U, M, K, B, C, mch, starts, final, dY, L)
        g0, token = res if isinstance(res, tuple) else (res, None)  # an engine may hand over reusable work
        if r == R - 1:
            d_final = None if d_final_in is None else d_final_in.float().contiguous()
        else:
            d_final = _recv(torch.empty((b, h, P, D), device=dev, dtype=torch.float32), r + 1, group)
        if r > 0:
            m_conj = m_seg * torch.tensor([1.0, -1.0], device=dev, dtype=m_seg.dtype)
            d_init_chain = g0 if d_final is None else g0 + _cmul(m_conj, d_final)
            _send(d_init_chain, r - 1, group)
        extra = {} if token is None else {"token": token}
        dU, dM, dK, dB, dC, d_init, dBp, dUp = engine.backward_full(U, M, K, B, C, Bp, Up, mch, starts, final, dY,
                                                                    d_final, L, **extra)
        # halo gradients go back to the previous rank's last token
        if r > 0:
            _send(torch.cat([dBp, dUp], dim=-1).contiguous(), r - 1, group)
        if r + 1 < R:
            hg = _recv(torch.empty((b, h, D + P), device=dev, dtype=torch.float32), r + 1, group)
            dB[:, :, -1, :] += hg[..., :D].to(dB.dtype)
            dU[:, :, -1, :] += hg[..., D:].to(dU.dtype)
        d_init_out = d_init.to(ctx.init_dtype) if (ctx.has_init and r == 0) else None
        return dU, dM, dK, dB, dC, d_init_out, None, None, None


def v2x2ssd_context_parallel(U, M, K, B, C, *, chunk_size: int, group=None,
                             initial_states: Optional[torch.Tensor] = None,
                             engine=None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Scan of a sequence that is split over the ranks of ``group`` along time.

    Every rank passes its own contiguous slice (length a multiple of
    ``chunk_size`` except possibly on the last rank).  ``initial_states`` is used
    on rank 0 only.  Returns ``(Y_local, final_state_fp32)``; ``final_state`` is
    the true end-of-sequence state on the last rank (and the end-of-segment state
    elsewhere).  Differentiable in ``U, M, K, B, C`` and rank 0's ``initial_states``.
    """
    if engine is None:
        engine = B200Engine()
    R, r = dist.get_world_size(group), dist.get_rank(group)
    if r + 1 < R and int(U.shape[2]) % int(chunk_size) != 0:
        raise ValueError("every rank but the last needs a slice length that is a multiple of chunk_size")
    if int(U.shape[2]) == 0:
        raise ValueError("context-parallel scan needs a non-empty slice on every rank")
    return _ContextParallelScanFn.apply(U, M, K, B, C, initial_states, int(chunk_size), group, engine)


__all__ = ["v2x2ssd_context_parallel", "B200Engine"]
