"""Stage-level timings of the scan path on one GPU, with achieved bandwidth /
tensor throughput per kernel against the measured peaks.

    python -m slinoss_b200.bench_stages [--batch 4 --heads 32 --T 8192 --N 128 --chunk 128] [--prep] [--conv]

Prints one JSON line per stage: name, ms (CUDA events, median of reps after
warm-up), algorithmic bytes and dense flops per launch, GB/s, TFLOP/s and the
fraction of the measured HBM / bf16 peaks (MEASURED_PEAKS.json beside the
package root, else the pool's fallback figures).  Inputs are seeded synthetic
tensors larger than L2.
"""

from __future__ import annotations

import argparse
import json
import math
from ctypes import byref
from pathlib import Path

import torch

from . import _lib

ROOT = Path(__file__).resolve().parents[1]


def _peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return float(d["hbm_gbs"]), float(d["bf16_tflops_sustained"]), "measured"
    return 6650.0, 1400.0, "fallback"


REPS, WARM = 10, 3   # overridden by --reps / --warm (a profiler capture wants few launches)


def _time(fn, reps=None, warm=None):
    reps = REPS if reps is None else reps
    warm = WARM if warm is None else warm
    for _ in range(warm):
        fn()
    torch.cuda.synchronize()
    ts = []
    for _ in range(reps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        fn()
        e1.record()
        torch.cuda.synchronize()
        ts.append(e0.elapsed_time(e1))
    ts.sort()
    return ts[len(ts) // 2]


def _emit(name, ms, nbytes, flops, hbm, tfl, src, extra=None):
    gbs = nbytes / (ms * 1e-3) / 1e9
    tf = flops / (ms * 1e-3) / 1e12
    line = dict(stage=name, ms=round(ms, 4), bytes=int(nbytes), flops=int(flops), gbs=round(gbs, 1),
                tflops=round(tf, 2), frac_hbm=round(gbs / hbm, 4), frac_tensor=round(tf / tfl, 4), peaks=src)
    if extra:
        line.update(extra)
    print(json.dumps(line), flush=True)


def scan_stages(b, h, T, P, N, L, dtype):
    dev = torch.device("cuda")
    hbm, tfl, src = _peaks()
    g = torch.Generator().manual_seed(0)
    D, BH, NC = 2 * N, b * h, (T + L - 1) // L
    es = torch.empty((), dtype=dtype).element_size()
    radius = torch.sigmoid(2.0 + torch.randn((b, h, T), generator=g))
    angle = torch.tanh(torch.randn((b, h, T), generator=g)) * (math.pi / 4)
    M = torch.view_as_real(torch.polar(radius, angle)).float().contiguous().to(dev)
    K = (torch.randn((b, h, T, 2, 2), generator=g) * 0.1).float().to(dev)
    U = torch.randn((b, h, T, P), generator=g).to(dtype).to(dev)
    B = (torch.randn((b, h, T, D), generator=g) / math.sqrt(N)).to(dtype).to(dev)
    C = (torch.randn((b, h, T, D), generator=g) / math.sqrt(N)).to(dtype).to(dev)
    dY = torch.randn((b, h, T, P), generator=g).to(dtype).to(dev)
    lib, st = _lib.lib(), _lib.stream_ptr(dev)
    s = _lib.scan_shape(BH, T, P, N, L, dtype)
    f32 = dict(device=dev, dtype=torch.float32)
    inc = torch.empty((b, h, NC, P, D), **f32)
    starts = torch.empty(inc.shape, device=dev, dtype=_lib.starts_dtype(s))
    sdt = _lib.dtype_code(starts.dtype)
    mch = torch.empty((b, h, NC, 2), **f32)
    final = torch.empty((b, h, P, D), **f32)
    Y = torch.empty_like(U)
    dz0 = torch.empty_like(inc)
    d_inc = torch.empty_like(starts)
    zdot = torch.empty((b, h, NC, 2), **f32)
    part = torch.empty((BH * NC * 2 * 64,), **f32)
    dU, dB, dC = torch.empty_like(U), torch.empty_like(B), torch.empty_like(C)
    dM, dK = torch.empty_like(M), torch.empty_like(K)
    cB, cU = torch.empty((b, h, NC, D), **f32), torch.empty((b, h, NC, P), **f32)
    ck = _lib.check
    ht = BH * T
    state_bytes = BH * NC * P * D * 4

    def inc_fn():
        ck(lib.slx_chunk_increment_fwd(byref(s), U.data_ptr(), M.data_ptr(), K.data_ptr(), B.data_ptr(), None, None,
                                       inc.data_ptr(), mch.data_ptr(), st), "inc")

    _emit("chunk_increment_fwd", _time(inc_fn), ht * (es * (P + D) + 24) + state_bytes, 2 * ht * P * D, hbm, tfl, src)

    def sp_fn():
        ck(lib.slx_state_passing_fwd(BH, NC, P, N, inc.data_ptr(), mch.data_ptr(), None, starts.data_ptr(), sdt,
                                     final.data_ptr(), st), "sp")

    starts_bytes = starts.numel() * starts.element_size()
    _emit("state_passing_fwd", _time(sp_fn), state_bytes + starts_bytes, 0, hbm, tfl, src)

    def scan_fn():
        ck(lib.slx_chunk_scan_fwd(byref(s), U.data_ptr(), M.data_ptr(), K.data_ptr(), B.data_ptr(), C.data_ptr(),
                                  starts.data_ptr(), None, None, Y.data_ptr(), st), "scan")

    _emit("chunk_scan_fwd", _time(scan_fn), ht * (es * (2 * P + 2 * D) + 24) + starts_bytes,
          ht * (2 * L * (D + P) + 2 * P * D), hbm, tfl, src)

    def dz0_fn():
        ck(lib.slx_chunk_scan_bwd_dz0(byref(s), M.data_ptr(), C.data_ptr(), dY.data_ptr(), dz0.data_ptr(), st), "dz0")

    _emit("chunk_scan_bwd_dz0", _time(dz0_fn), ht * (es * (P + D) + 8) + state_bytes, 2 * ht * P * D, hbm, tfl, src)

    def spb_fn():
        ck(lib.slx_state_passing_bwd(BH, NC, P, N, dz0.data_ptr(), mch.data_ptr(), starts.data_ptr(), sdt,
                                     final.data_ptr(), None, d_inc.data_ptr(), None, zdot.data_ptr(),
                                     part.data_ptr(), st), "spb")

    _emit("state_passing_bwd", _time(spb_fn), state_bytes + 2 * starts_bytes, 0, hbm, tfl, src)

    def bwd_fn():
        ck(lib.slx_chunk_scan_bwd(byref(s), U.data_ptr(), M.data_ptr(), K.data_ptr(), B.data_ptr(), C.data_ptr(), None,
                                  None, starts.data_ptr(), d_inc.data_ptr(), zdot.data_ptr(), dY.data_ptr(),
                                  dU.data_ptr(), dM.data_ptr(), dK.data_ptr(), dB.data_ptr(), dC.data_ptr(),
                                  cB.data_ptr(), cU.data_ptr(), st), "bwd")

    _emit("chunk_scan_bwd", _time(bwd_fn), ht * (es * (3 * P + 4 * D) + 48) + 2 * starts_bytes,
          ht * 2 * (2 * L * P + 3 * L * D + 3 * P * D), hbm, tfl, src)


def prep_stage(b, T, H, P, N, dtype):
    """scanprep forward / backward through the C ABI with preallocated buffers (kernel time only)."""
    dev = torch.device("cuda")
    hbm, tfl, src = _peaks()
    g = torch.Generator().manual_seed(1)
    es = torch.empty((), dtype=dtype).element_size()
    value = torch.randn(b, T, H * P, generator=g).to(dtype).to(dev)
    params = torch.randn(b, T, H * 13, generator=g).to(dtype).to(dev)
    bc = torch.randn(b, T, H * 4 * N, generator=g).to(dtype).to(dev)
    bias = torch.zeros(H, 13, device=dev, dtype=torch.float32)
    scale = torch.ones(H, 4, N, device=dev, dtype=torch.float32)
    f32 = dict(device=dev, dtype=torch.float32)
    U = torch.empty((b, H, T, P), device=dev, dtype=dtype)
    Bo = torch.empty((b, H, T, 2 * N), device=dev, dtype=dtype)
    Co = torch.empty_like(Bo)
    M = torch.empty((b, H, T, 2), **f32)
    K = torch.empty((b, H, T, 2, 2), **f32)
    s = _lib.PrepShape(b, T, H, P, N, _lib.dtype_code(dtype), 1, 1e-4, 1e-1, 0.9, 1.0, math.pi, 0.5, 1e-8,
                       H * P, H * 13, H * 4 * N)
    lib, st, ck = _lib.lib(), _lib.stream_ptr(dev), _lib.check

    def fwd():
        ck(lib.slx_scanprep_fwd(byref(s), value.data_ptr(), params.data_ptr(), bc.data_ptr(), bias.data_ptr(),
                                scale.data_ptr(), U.data_ptr(), M.data_ptr(), K.data_ptr(), Bo.data_ptr(),
                                Co.data_ptr(), st), "scanprep fwd")

    rows = b * T * H
    per_row = es * (P + 13 + 4 * N) + es * (P + 4 * N) + 24
    _emit("scanprep_fwd", _time(fwd), rows * per_row, 0, hbm, tfl, src)
    dU, dB, dC = torch.randn_like(U), torch.randn_like(Bo), torch.randn_like(Co)
    dM, dK = torch.randn_like(M), torch.randn_like(K)
    d_value, d_params, d_bc = torch.empty_like(value), torch.empty_like(params), torch.empty_like(bc)
    d_bias, d_scale = torch.empty_like(bias), torch.empty_like(scale)
    nbytes = int(lib.slx_scanprep_bwd_workspace_bytes(byref(s)))
    ws = torch.empty((max(nbytes, 16),), device=dev, dtype=torch.uint8)

    def bwd():
        ck(lib.slx_scanprep_bwd(byref(s), params.data_ptr(), bc.data_ptr(), bias.data_ptr(), scale.data_ptr(),
                                dU.data_ptr(), dM.data_ptr(), dK.data_ptr(), dB.data_ptr(), dC.data_ptr(),
                                d_value.data_ptr(), d_params.data_ptr(), d_bc.data_ptr(), d_bias.data_ptr(),
                                d_scale.data_ptr(), ws.data_ptr(), nbytes, st), "scanprep bwd")

    _emit("scanprep_bwd", _time(bwd), rows * (per_row + es * (13 + 4 * N)), 0, hbm, tfl, src,
          dict(note="reads params, bc and all five gradients; writes d_value, d_params, d_bc"))


def conv_stage(b, T, Cn, dtype):
    """Depthwise causal conv (width 4, bias, no activation) through the C ABI, kernel time only."""
    dev = torch.device("cuda")
    hbm, tfl, src = _peaks()
    g = torch.Generator().manual_seed(2)
    es = torch.empty((), dtype=dtype).element_size()
    W = 4
    x = torch.randn(b, T, Cn, generator=g).to(dtype).to(dev)
    w = torch.randn(Cn, W, generator=g).to(dtype).to(dev)
    bias = torch.randn(Cn, generator=g).to(dtype).to(dev)
    y = torch.empty_like(x)
    nxt = torch.empty((b, Cn, W - 1), device=dev, dtype=dtype)
    s = _lib.ConvShape(b, T, Cn, W, _lib.dtype_code(dtype), 0, Cn, T * Cn)
    lib, st, ck = _lib.lib(), _lib.stream_ptr(dev), _lib.check

    def fwd():
        ck(lib.slx_cconv1d_fwd(byref(s), x.data_ptr(), w.data_ptr(), bias.data_ptr(), None, y.data_ptr(),
                               nxt.data_ptr(), st), "conv fwd")

    _emit("cconv1d_fwd", _time(fwd), b * T * Cn * 2 * es, 0, hbm, tfl, src)
    dy = torch.randn_like(y)
    dx = torch.empty_like(x)
    dw = torch.empty((Cn, W), device=dev, dtype=torch.float32)
    db = torch.empty((Cn,), device=dev, dtype=torch.float32)
    nbytes = int(lib.slx_cconv1d_bwd_workspace_bytes(byref(s)))
    ws = torch.empty((max(nbytes, 16),), device=dev, dtype=torch.uint8)

    def bwd():
        ck(lib.slx_cconv1d_bwd(byref(s), x.data_ptr(), w.data_ptr(), bias.data_ptr(), None, dy.data_ptr(), None,
                               dx.data_ptr(), dw.data_ptr(), db.data_ptr(), None, ws.data_ptr(), nbytes, st),
           "conv bwd")

    _emit("cconv1d_bwd", _time(bwd), b * T * Cn * 3 * es, 0, hbm, tfl, src)


def decode_stage(b, H, P, N, dtype):
    """One-token decode step at a serving batch, through the C ABI; state updated out of place
    and in place (what a ScanState carried between tokens does)."""
    dev = torch.device("cuda")
    hbm, tfl, src = _peaks()
    g = torch.Generator().manual_seed(3)
    r = lambda *sh: torch.randn(*sh, generator=g)
    value, gate = r(b, H, P).to(dtype).to(dev), r(b, H, P).to(dtype).to(dev)
    params, bc = r(b, H, 13).to(dtype).to(dev), r(b, H, 4, N).to(dtype).to(dev)
    skip = r(H, P).to(dtype).to(dev)
    bias = torch.zeros(H, 13, device=dev)
    scale = torch.ones(H, 4, N, device=dev)
    st_in, st_out = r(b, H, P, 2 * N).to(dev), torch.empty(b, H, P, 2 * N, device=dev)
    bp, up = r(b, H, 2 * N).to(dtype).to(dev), r(b, H, P).to(dtype).to(dev)
    bl, ul = torch.empty_like(bp), torch.empty_like(up)
    out = torch.empty(b, H * P, device=dev, dtype=dtype)
    s = _lib.DecodeShape(b, H, P, N, _lib.dtype_code(dtype), 1, 1e-4, 1e-1, 0.9, 1.0, math.pi, 0.5, 1e-8)
    lib, st, ck = _lib.lib(), _lib.stream_ptr(dev), _lib.check

    def call(zin, zout):
        ck(lib.slx_decode_step(byref(s), value.data_ptr(), params.data_ptr(), bc.data_ptr(), gate.data_ptr(),
                               skip.data_ptr(), bias.data_ptr(), scale.data_ptr(), zin.data_ptr(), bp.data_ptr(),
                               up.data_ptr(), out.data_ptr(), zout.data_ptr(), bl.data_ptr(), ul.data_ptr(), st),
           "decode")

    nbytes = b * H * 2 * P * 2 * N * 4
    _emit("decode_step", _time(lambda: call(st_in, st_out)), nbytes, 0, hbm, tfl, src,
          dict(note=f"b{b} H{H} P{P} N{N}, state read from one buffer and written to another"))
    _emit("decode_step_in_place", _time(lambda: call(st_in, st_in)), nbytes, 0, hbm, tfl, src,
          dict(note="state updated in place"))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--batch", type=int, default=4)
    ap.add_argument("--heads", type=int, default=32)
    ap.add_argument("--T", type=int, default=8192)
    ap.add_argument("--P", type=int, default=64)
    ap.add_argument("--N", type=int, default=128)
    ap.add_argument("--chunk", type=int, default=128)
    ap.add_argument("--dtype", default="bf16", choices=["bf16", "f16", "f32"])
    ap.add_argument("--no-scan", action="store_true")
    ap.add_argument("--prep", action="store_true")
    ap.add_argument("--conv", action="store_true")
    ap.add_argument("--decode", action="store_true", help="one-token decode step at batch --decode-batch")
    ap.add_argument("--decode-batch", type=int, default=256)
    ap.add_argument("--reps", type=int, default=10, help="timed launches per stage")
    ap.add_argument("--warm", type=int, default=3, help="untimed launches per stage")
    a = ap.parse_args()
    global REPS, WARM
    REPS, WARM = max(a.reps, 1), max(a.warm, 0)
    dt = dict(bf16=torch.bfloat16, f16=torch.float16, f32=torch.float32)[a.dtype]
    if not a.no_scan:
        scan_stages(a.batch, a.heads, a.T, a.P, a.N, a.chunk, dt)
    if a.prep:
        prep_stage(a.batch, a.T, a.heads, a.P, a.N, dt)
    if a.conv:
        conv_stage(a.batch, a.T, a.heads * a.P, dt)
    if a.decode:
        decode_stage(a.decode_batch, a.heads, a.P, a.N, dt)


if __name__ == "__main__":
    main()
