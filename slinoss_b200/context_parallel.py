"""Context-parallel v2x2ssd: one long sequence split over the ranks of a process
group, with only chunk-final states (and one-token halos) crossing ranks.

The reference has no distributed code; what it has is the segment-chaining
contract (running ``[0:t)`` then ``[t:T)`` through ``ScanState`` reproduces one
pass, reference tests/test_v2x2ssd_cute.py:818-929).  This module distributes
exactly that contract.  Rank ``r`` owns tokens ``[r*T/R, (r+1)*T/R)``.

A segment acts on the state that enters it as an affine map ``z_out = m_seg z_in + f0``
(``m_seg`` = product of its chunk transitions, ``f0`` = its final state from a zero start).
Instead of handing the state from rank to rank (R-1 dependent hops), every rank contributes
its ``(m_seg, f0)`` pair to ONE all-gather and then folds the pairs of the ranks in front of
it locally (one small kernel, ``slx_segment_fold``).

Forward
  1. halo all-gather: every rank's last ``(B, U)`` row; rank ``r`` uses row ``r-1`` as its
     ``B_prev, U_prev``.
  2. every rank, in parallel: chunk increments and a state pass from a ZERO start -> ``f0``, ``m_seg``.
  3. state all-gather of ``(m_seg, f0)`` (rank 0 contributes ``m_seg z_init + f0``), local fold
     -> ``z_in``.
  4. every rank: state pass from its true ``z_in``, then the chunk scan.
Backward mirrors it: every rank computes its reverse pass from a zero ``d_final`` (``g0``),
contributes ``(m_seg, g0 + conj(m_seg) d_final_local)`` to one all-gather, folds the pairs of
the ranks behind it into its true ``d_final``, runs its full backward, and a last all-gather
returns the halo gradients to the previous rank's last row.

All arithmetic is done by an *engine* (the sm_100a kernels by default); the message pattern is
engine-independent and is tested on CPU ranks (gloo) with a CPU engine.  Every collective is
waited for with the process group's timeout: a rank that never joins makes the others raise
``RuntimeError`` instead of waiting forever.
"""

from __future__ import annotations

from ctypes import byref
from typing import Optional, Tuple

import torch
import torch.distributed as dist


class B200Engine:
    """Local arithmetic on the sm_100a kernels (through the C ABI)."""

    def forward_parts(self, U, M, K, B, Bp, Up, L):
        from . import _lib
        from .ops.v2x2ssd import _shape, chunk_increment_b200, state_passing_b200

        b, h, T, P = map(int, U.shape)
        # increments stored like the chunk starts (the activation dtype on the tensor-core path)
        sdt = _lib.starts_dtype(_shape(b, h, T, P, int(B.shape[-1]) // 2, L, U.dtype))
        inc, mch = chunk_increment_b200(U, M, K, B, B_prev=Bp, U_prev=Up, chunk_size=L, inc_dtype=sdt)
        _, f0 = state_passing_b200(inc, mch, initial_states=None, want_starts=False)
        return inc, mch, f0

    def forward_finish(self, U, M, K, B, C, inc, mch, z_in, Bp, Up, L):
        from . import _lib
        from .ops.v2x2ssd import _shape, chunk_scan_b200, state_passing_b200

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

    # ---- segment algebra (slx_segment_*) ------------------------------------------------------
    def segment_transition(self, mch):
        from . import _lib

        b, h, NC, _ = map(int, mch.shape)
        out = torch.empty((b, h, 2), device=mch.device, dtype=torch.float32)
        with _lib.guard(mch.device):
            _lib.check(_lib.lib().slx_segment_transition(b * h, NC, mch.data_ptr(), out.data_ptr(),
                                                         _lib.stream_ptr(mch.device)), "segment_transition")
        return out

    def axpy(self, m, z, f, conj: bool):
        from . import _lib

        b, h, P, D = map(int, f.shape)
        out = torch.empty_like(f)
        with _lib.guard(f.device):
            _lib.check(_lib.lib().slx_segment_axpy(b * h, P, D // 2, m.data_ptr(), z.data_ptr(), f.data_ptr(),
                                                   1 if conj else 0, out.data_ptr(), _lib.stream_ptr(f.device)),
                       "segment_axpy")
        return out

    def fold(self, states, ms, first: int, count: int, step: int, conj: bool):
        """``out = states[first]; for j = 1..count-1: out = m[first + j*step] * out + states[first + j*step]``
        over the gathered ``states (R,b,h,P,2N)`` and ``ms (R,b,h,2)``."""
        from . import _lib

        R, b, h, P, D = map(int, states.shape)
        out = torch.empty((b, h, P, D), device=states.device, dtype=torch.float32)
        with _lib.guard(states.device):
            _lib.check(_lib.lib().slx_segment_fold(
                b * h, P, D // 2, count, states[first].data_ptr(), step * b * h * P * D, ms[first].data_ptr(),
                step * b * h * 2, 1 if conj else 0, out.data_ptr(), _lib.stream_ptr(states.device)), "segment_fold")
        return out


class TorchSegmentAlgebra:
    """The segment algebra in plain torch complex arithmetic, for engines that run on the CPU
    (the gloo tests); mix into such an engine."""

    @staticmethod
    def _c(z):
        return torch.view_as_complex(z.reshape(*z.shape[:-1], z.shape[-1] // 2, 2).contiguous())

    def segment_transition(self, mch):
        return torch.view_as_real(torch.view_as_complex(mch.contiguous()).prod(dim=2)).contiguous()

    def axpy(self, m, z, f, conj: bool):
        mc = torch.view_as_complex(m.contiguous())[..., None, None]
        if conj:
            mc = mc.conj()
        return torch.view_as_real(mc * self._c(z) + self._c(f)).reshape(f.shape).contiguous()

    def fold(self, states, ms, first: int, count: int, step: int, conj: bool):
        out = states[first]
        for j in range(1, count):
            out = self.axpy(ms[first + j * step], out, states[first + j * step], conj)
        return out.contiguous()


def _all_gather(t: torch.Tensor, group, what: str) -> torch.Tensor:
    """``(R, *t.shape)`` gathered over the group; waits with the group's timeout and turns a
    timeout or a failed peer into ``RuntimeError`` naming the exchange."""
    R = dist.get_world_size(group)
    out = torch.empty((R,) + tuple(t.shape), device=t.device, dtype=t.dtype)
    try:
        work = dist.all_gather_into_tensor(out.view(-1), t.contiguous().view(-1), group=group, async_op=True)
        work.wait()
    except Exception as e:  # gloo raises RuntimeError, NCCL DistBackendError; name the step either way
        raise RuntimeError(f"context-parallel exchange '{what}' failed on rank {dist.get_rank(group)}: a peer did "
                           f"not join before the process group's timeout or the transport broke ({e})") from e
    return out


class _ContextParallelScanFn(torch.autograd.Function):
    @staticmethod
    def forward(ctx, U, M, K, B, C, initial_states, L, group, engine):
        R, r = dist.get_world_size(group), dist.get_rank(group)
        b, h, T, P = map(int, U.shape)
        D = int(B.shape[-1])
        U, M, K, B, C = (t.detach() for t in (U, M, K, B, C))
        # 1. halo: last (B, U) row of every rank
        Bp = Up = None
        if R > 1:
            halo = torch.cat([B[:, :, -1, :].float(), U[:, :, -1, :].float()], dim=-1).contiguous()
            halos = _all_gather(halo, group, "forward halo")
            if r > 0:
                Bp, Up = halos[r - 1][..., :D].contiguous(), halos[r - 1][..., D:].contiguous()
        # 2. local parts from a zero start
        inc, mch, f0 = engine.forward_parts(U, M, K, B, Bp, Up, L)
        m_seg = engine.segment_transition(mch)
        # 3. state entering this segment
        z_in = None
        if r == 0 and initial_states is not None:
            z_in = initial_states.detach().float().contiguous()
        if R > 1:
            mine = f0 if z_in is None else engine.axpy(m_seg, z_in, f0, False)  # rank 0 resolves its own start
            ms = _all_gather(m_seg, group, "forward transitions")
            zs = _all_gather(mine, group, "forward states")
            if r > 0:
                z_in = engine.fold(zs, ms, 0, r, 1, False)
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
        dY = torch.zeros_like(U) if dY is None else dY.to(U.dtype).contiguous()
        res = engine.backward_zero(U, M, K, B, C, mch, starts, final, dY, L)
        g0, token = res if isinstance(res, tuple) else (res, None)  # an engine may hand over reusable work
        # d_final of this segment = its own cotangent (any rank may have one) + d_initial of the next
        # segment; d_initial(r) = g0(r) + conj(m_seg(r)) d_final(r).  Every rank contributes the part
        # it knows, g0 + conj(m_seg) d_final_local, and folds the ranks behind it.
        d_final = None if d_final_in is None else d_final_in.float().contiguous()
        if R > 1:
            mine = g0 if d_final is None else engine.axpy(m_seg, d_final, g0, True)
            ms = _all_gather(m_seg, group, "backward transitions")
            gs = _all_gather(mine, group, "backward states")
            if r + 1 < R:
                tail = engine.fold(gs, ms, R - 1, R - 1 - r, -1, True)  # d_initial of rank r+1
                d_final = tail if d_final is None else d_final + tail
        extra = {} if token is None else {"token": token}
        dU, dM, dK, dB, dC, d_init, dBp, dUp = engine.backward_full(U, M, K, B, C, Bp, Up, mch, starts, final, dY,
                                                                    d_final, L, **extra)
        # halo gradients go back to the previous rank's last token
        if R > 1:
            dev = U.device
            hg = (torch.cat([dBp.float(), dUp.float()], dim=-1).contiguous() if r > 0
                  else torch.zeros((b, h, D + P), device=dev, dtype=torch.float32))
            hgs = _all_gather(hg, group, "halo gradients")
            if r + 1 < R:
                dB[:, :, -1, :] += hgs[r + 1][..., :D].to(dB.dtype)
                dU[:, :, -1, :] += hgs[r + 1][..., D:].to(dU.dtype)
        d_init_out = d_init.to(ctx.init_dtype) if (ctx.has_init and r == 0) else None
        return dU, dM, dK, dB, dC, d_init_out, None, None, None


def v2x2ssd_context_parallel(U, M, K, B, C, *, chunk_size: int, group=None,
                             initial_states: Optional[torch.Tensor] = None,
                             engine=None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Scan of a sequence that is split over the ranks of ``group`` along time.

    Every rank passes its own contiguous slice (length a multiple of
    ``chunk_size`` except possibly on the last rank).  ``initial_states`` is used
    on rank 0 only.  Returns ``(Y_local, final_state_fp32)``; ``final_state`` is
    the true end-of-sequence state on the last rank and the state at the end of the rank's
    segment elsewhere.  Differentiable in ``U, M, K, B, C`` and rank 0's ``initial_states``; a
    cotangent on any rank's ``final_state`` is honoured (it joins the chained ``d_final``).

    Every rank of the group must make the call: the exchanges are collectives.  A rank that
    does not join makes the others raise ``RuntimeError`` after the group's timeout
    (``dist.init_process_group(timeout=...)`` / ``dist.new_group(timeout=...)``).
    """
    if engine is None:
        engine = B200Engine()
    R, r = dist.get_world_size(group), dist.get_rank(group)
    if r + 1 < R and int(U.shape[2]) % int(chunk_size) != 0:
        raise ValueError("every rank but the last needs a slice length that is a multiple of chunk_size")
    if int(U.shape[2]) == 0:
        raise ValueError("context-parallel scan needs a non-empty slice on every rank")
    for name, t in (("U", U), ("M", M), ("K", K), ("B", B), ("C", C)):
        if not t.is_contiguous():
            raise ValueError(f"{name} must be contiguous; got strides {t.stride()} "
                             "(a time slice of a longer tensor needs .contiguous()).")
    return _ContextParallelScanFn.apply(U, M, K, B, C, initial_states, int(chunk_size), group, engine)


__all__ = ["v2x2ssd_context_parallel", "B200Engine", "TorchSegmentAlgebra"]
