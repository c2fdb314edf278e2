"""Headline benchmark: v2x2ssd forward+backward tokens/s on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--chunk 64|128] [--impl reference]
    python bench.py --stages-only [--only NAME] [--reps R] [--warm W] [--T ..]   (per-kernel lines)

One "step" is one forward + one backward of the scan over one batch of seeded
synthetic inputs of the headline configuration (batch 4, heads 32, P 64, N 128,
T 8192, bf16 U/B/C/dY, fp32 M/K/state; radius = sigmoid(N(2,1)), angle =
tanh(N(0,1)) pi/4, taps 0.1 N(0,1), B, C ~ N(0,1/N)).  Rank 0 prints ONE JSON line:

  value      tokens/s (tokens = batch*T per call, all heads) with inputs resident
             in HBM, whole job (sum over ranks; every rank runs its own batch:
             weak scaling, no collective on the data path).  The timed region is
             K steps repeated `inner_repeats` times so that it lasts >= 1 s.
  e2e        the same metric through the public op with HOST buffers: pinned
             host -> device copies of every input and device -> host copies of
             every result inside the timed region; `host_link` beside it gives the
             copy rates of the same buffers with no kernels (upload, download, both)
  roofline   the dominant kernel (per-chunk backward), timed alone with CUDA
             events: dense-tile flops per launch / duration against the measured
             bf16 burst peak; `traffic` from the ncu capture recorded in
             profiles/dominant_kernel_traffic.json
  stages     every kernel of the path timed by itself through the C ABI
             (scan stages, scan prep, conv, gate/skip, conv update, decode step): ms,
             bound, achieved, frac
  cp         the context-parallel mode: one b1 H32 T262144 sequence split over the
             ranks along time (at N = 1 the same sequence on one GPU)
  config1 / config3   the reference's own SLinOSSMixer layer (fwd+bwd) and NextCharLM
             training step with every mixer on the B200 backends (needs the reference
             package under baseline/_ref); config1 also times the layer with unfused
             glue and on the reference's own torch backends on the same GPU
  cpu_baseline  the reference's CPU path timed on the host cores on a bounded
             sample of the same workload (rank 0, N=1)

``--impl reference`` times the reference's own ``v2x2ssd`` + ``torch.autograd.grad`` on the
host CPU in fp32 compute on (batch 1, head 1) slices of the same workload (the C port in
oracle/ when the reference package is not installed) and prints the same line shape.
"""

from __future__ import annotations

import argparse
import json
import math
import os
import subprocess
import sys
import tempfile
import time
from ctypes import byref
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))
REF_DIR = ROOT / "baseline" / "_ref"

HEADLINE = dict(batch=4, heads=32, T=8192, P=64, N=128)
METRIC = "v2x2ssd fwd+bwd tokens/sec (H32 P64 N128 T8192 b4, bf16 in / fp32 state)"


def workload_name(cfg, chunk):
    return (f"v2x2ssd fwd+bwd b{cfg['batch']} H{cfg['heads']} P{cfg['P']} N{cfg['N']} T{cfg['T']} "
            f"chunk {chunk} per GPU")


def _peaks():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        d = json.loads(p.read_text())
        return dict(hbm_gbs=float(d["hbm_gbs"]), tflops=float(d["bf16_tflops_sustained"]),
                    tflops_burst=float(d["bf16_tflops"]), source="measured")
    return dict(hbm_gbs=6650.0, tflops=1400.0, tflops_burst=1590.0, source="fallback")


def algorithmic_bytes_per_head_token(P, D):
    """Compulsory HBM traffic of fwd+bwd with bf16 activations: every operand read
    once, every result written once (U,B,C,M,K,Y fwd; U,B,C,M,K,dY -> dU,dB,dC,dM,dK
    bwd), chunk-state intermediates excluded: 10P + 12D + 72 bytes."""
    return 10 * P + 12 * D + 72


def dense_flops_bwd_chunk(L, P, D):
    """Dense-tile flops of the per-chunk backward in the merged-tap formulation with real
    (rotated) operands, i.e. the minimum a tile engine executes without skipping masked
    tiles: G=dY U^T, S=Q K^T, dq=dS K, X=dS^T Q, dU=S^T dY (L*L tiles) plus dY Z0, U Lambda,
    B^ Lambda^T (L*P*D tiles).  The complex-Gram kernels execute about twice this (two real
    products per complex one); the figure is kept as the common yardstick."""
    return 2 * (2 * L * L * P + 3 * L * L * D + 3 * L * P * D)


def make_inputs(cfg, device, seed, dtype):
    import torch

    b, h, T, P, N = cfg["batch"], cfg["heads"], cfg["T"], cfg["P"], cfg["N"]
    g = torch.Generator(device="cpu").manual_seed(seed)
    radius = torch.sigmoid(2.0 + torch.randn((b, h, T), generator=g))
    angle = torch.tanh(torch.randn((b, h, T), generator=g)) * (math.pi / 4)
    M = torch.view_as_real(torch.polar(radius, angle)).float().contiguous()
    K = (torch.randn((b, h, T, 2, 2), generator=g) * 0.1).float()
    U = torch.randn((b, h, T, P), generator=g).to(dtype)
    B = (torch.randn((b, h, T, 2 * N), generator=g) / math.sqrt(N)).to(dtype)
    C = (torch.randn((b, h, T, 2 * N), generator=g) / math.sqrt(N)).to(dtype)
    dY = torch.randn((b, h, T, P), generator=g).to(dtype)
    host = dict(U=U, M=M, K=K, B=B, C=C, dY=dY)
    if device is None:
        return host
    return {k: v.to(device) for k, v in host.items()}


class ClockSampler:
    """nvidia-smi clocks/throttle reasons sampled every 50 ms during a timed region."""

    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index = index
        self.proc = None
        self.path = None

    def start(self):
        try:
            f = tempfile.NamedTemporaryFile("w", suffix=".csv", delete=False)
            self.path = f.name
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                 "-lms", "50"], stdout=f, stderr=subprocess.DEVNULL)
            time.sleep(0.15)  # let the sampler come up before the timed region starts
        except Exception:
            self.proc = None
        return self

    def stop(self):
        out = dict(sm_mhz=None, sm_max_mhz=None, reasons=[], samples=0)
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        try:
            rows = [r.split(",") for r in Path(self.path).read_text().strip().splitlines() if r.strip()]
            rows = [r for r in rows if len(r) >= 9]
            sm = sorted(float(r[1]) for r in rows)
            if sm:
                out["sm_mhz"] = sm[len(sm) // 2]
                out["sm_max_mhz"] = float(rows[0][2])
                out["power_w_max"] = max(float(r[3]) for r in rows)
            names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
            seen = set()
            for r in rows:
                for name, val in zip(names, r[5:9]):
                    if val.strip().lower().startswith("active"):
                        seen.add(name)
            out["reasons"] = sorted(seen)
            out["samples"] = len(rows)
        except Exception:
            pass
        finally:
            try:
                os.unlink(self.path)
            except Exception:
                pass
        return out


# ----------------------------------------------------------------------------------------------
# CPU arms
# ----------------------------------------------------------------------------------------------

def _have_reference() -> bool:
    return (REF_DIR / "slinoss" / "__init__.py").exists()


def _import_reference():
    if str(REF_DIR) not in sys.path:
        sys.path.insert(0, str(REF_DIR))
    import slinoss  # noqa: F401


def cpu_reference_time(cfg, chunk, n_slices, T_sample, seed=0):
    """Seconds for fwd + autograd.grad of the reference's own ``v2x2ssd`` (fp32 compute, bf16
    inputs like the GPU arm) over ``n_slices`` (batch 1, head 1) slices of ``T_sample`` tokens."""
    import torch

    _import_reference()
    from slinoss.ops.v2x2ssd import v2x2ssd

    one = dict(cfg, batch=1, heads=1, T=T_sample)
    total = 0.0
    for i in range(n_slices):
        inp = make_inputs(one, None, seed + i, torch.bfloat16)
        leaves = [inp[k].requires_grad_(True) for k in ("U", "M", "K", "B", "C")]
        t0 = time.perf_counter()
        out = v2x2ssd(*leaves, chunk_size=chunk, compute_dtype=torch.float32, output_dtype=torch.bfloat16)
        Y = out[0] if isinstance(out, tuple) else out
        torch.autograd.grad(Y, leaves, inp["dY"])
        total += time.perf_counter() - t0
    return total


def cpu_port_time(cfg, chunk, bh_sample, T_sample, threads):
    """Seconds for fwd+bwd of the C oracle on (bh_sample, T_sample) head-sequences."""
    import numpy as np

    from oracle import scan as oscan

    os.environ["OMP_NUM_THREADS"] = str(threads)
    rng = np.random.default_rng(0)
    P, N = cfg["P"], cfg["N"]
    sh = (1, bh_sample, T_sample)
    r = 1.0 / (1.0 + np.exp(-(2.0 + rng.standard_normal(sh))))
    th = np.tanh(rng.standard_normal(sh)) * (math.pi / 4)
    M = np.stack([r * np.cos(th), r * np.sin(th)], -1)
    K = rng.standard_normal(sh + (2, 2)) * 0.1
    U = rng.standard_normal(sh + (P,))
    B = rng.standard_normal(sh + (2 * N,)) / math.sqrt(N)
    C = rng.standard_normal(sh + (2 * N,)) / math.sqrt(N)
    dY = rng.standard_normal(sh + (P,))
    t0 = time.perf_counter()
    oscan.v2x2ssd_fwd(U, M, K, B, C, chunk_size=chunk)
    oscan.v2x2ssm_bwd(U, M, K, B, C, dY=dY)
    return time.perf_counter() - t0


def cpu_tokens_per_s(cfg, seconds, bh_sample, T_sample):
    """Extrapolate the sample to the full workload: tokens = batch*T, all heads."""
    full_units = cfg["batch"] * cfg["heads"] * cfg["T"]
    t_full = seconds * full_units / (bh_sample * T_sample)
    return cfg["batch"] * cfg["T"] / t_full


def cpu_sample(cfg, chunk, n_slices, seed=0, warm=True):
    """One bounded sample of the workload on the host cores: (seconds, units, info).  The reference
    package when it is installed under baseline/_ref, else the C port of oracle/."""
    BH, T = cfg["batch"] * cfg["heads"], cfg["T"]
    if _have_reference():
        import torch

        if warm:
            cpu_reference_time(cfg, chunk, 1, 256)
        sec = cpu_reference_time(cfg, chunk, n_slices, T, seed=seed)
        info = dict(unit="tokens/s", cores=torch.get_num_threads(), kind="reference",
                    sample=f"{n_slices} (batch 1, head 1) slices x {T} tokens, fwd + autograd.grad of the reference's "
                           f"v2x2ssd (bf16 inputs, fp32 compute, torch CPU ops); "
                           + (f"extrapolated to {BH} slices" if n_slices < BH else "that is the whole workload"))
        return sec, n_slices, info
    threads = os.cpu_count() or 1
    bh_s = min(threads, BH)
    if warm:
        cpu_port_time(cfg, chunk, bh_s, 256, threads)
    sec = cpu_port_time(cfg, chunk, bh_s, T, threads)
    info = dict(unit="tokens/s", cores=threads, kind="port",
                sample=f"{bh_s} (batch,head) sequences x {T} tokens, fwd+bwd, float64 C port with OpenMP; "
                       f"extrapolated to {BH} sequences")
    return sec, bh_s, info


def run_reference_arm(args, cfg):
    """The reference's CPU path on this box's host cores, a bounded sample per step."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    # one slice timed first; then as many slices per step as keep the whole run within ~2 minutes
    t_one, _, _ = cpu_sample(cfg, args.chunk, 1, warm=True)
    BH = cfg["batch"] * cfg["heads"]
    n_slices = max(1, min(BH, int(120.0 / (max(args.steps, 1) * max(t_one, 1e-3)))))
    for i in range(max(args.warmup - 1, 0)):
        cpu_sample(dict(cfg, T=min(cfg["T"], 1024)), args.chunk, 1, seed=900 + i, warm=False)
    secs, units, info = [], n_slices, None
    for i in range(args.steps):
        sec, units, info = cpu_sample(cfg, args.chunk, n_slices, seed=10 * i, warm=False)
        secs.append(sec)
    sec = sum(secs) / len(secs)
    val = cpu_tokens_per_s(cfg, sec, units, cfg["T"])
    info = dict(info, value=val)
    line = dict(impl="reference", metric=METRIC, value=val, unit="tokens/s", n_gpus=args.gpus,
                steps=args.steps, warmup=args.warmup, ms_per_step=sec * 1e3, higher_is_better=True,
                scaling="weak", vs_baseline=None, dtype="bf16" if info["kind"] == "reference" else "f64",
                data="synthetic",
                config=dict(workload=workload_name(cfg, args.chunk), sample_per_step=info["sample"]),
                cpu_baseline=info,
                e2e=dict(value=val, unit="tokens/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0),
                gpu_launches=0)
    print(json.dumps(line))
    return 0


# ----------------------------------------------------------------------------------------------
# per-kernel timings through the C ABI
# ----------------------------------------------------------------------------------------------

def _time_kernel(fn, reps, warm):
    import torch

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


def _stage(name, ms, nbytes, flops, peaks, bound, note=None):
    gbs = nbytes / (ms * 1e-3) / 1e9
    tf = flops / (ms * 1e-3) / 1e12
    d = dict(stage=name, ms=round(ms, 4), bound=bound, bytes=int(nbytes), flops=int(flops))
    if bound == "hbm":
        d.update(achieved=round(gbs, 1), peak=peaks["hbm_gbs"], unit="GB/s", frac=round(gbs / peaks["hbm_gbs"], 4))
    else:
        d.update(achieved=round(tf, 2), peak=peaks["tflops_burst"], unit="TFLOP/s",
                 frac=round(tf / peaks["tflops_burst"], 4), gbs=round(gbs, 1),
                 frac_hbm=round(gbs / peaks["hbm_gbs"], 4))
    if note:
        d["note"] = note
    return d


def scan_stage_timings(inp, b, h, T, P, N, L, dtype, reps=10, warm=3, only=None):
    """Every scan kernel by itself, median of `reps` launches (CUDA events around the C-ABI call)."""
    import torch

    from slinoss_b200 import _lib

    dev = inp["U"].device
    peaks = _peaks()
    D, BH, NC = 2 * N, b * h, (T + L - 1) // L
    es = torch.empty((), dtype=dtype).element_size()
    U, M, K, B, C, dY = (inp[k].detach() for k in ("U", "M", "K", "B", "C", "dY"))
    lib, st = _lib.lib(), _lib.stream_ptr(dev)
    s = _lib.scan_shape(BH, T, P, N, L, dtype)
    f32 = dict(device=dev, dtype=torch.float32)
    # increments / dZ0 are stored like the chunk starts, as the whole-op entry points store them
    starts = torch.empty((b, h, NC, P, D), device=dev, dtype=_lib.starts_dtype(s))
    inc = torch.empty_like(starts)
    sdt = _lib.dtype_code(starts.dtype)
    mch = torch.empty((b, h, NC, 2), **f32)
    final = torch.empty((b, h, P, D), **f32)
    Y = torch.empty_like(U)
    dz0 = torch.empty_like(inc)
    d_inc = torch.empty_like(starts)
    zdot = torch.empty((b, h, NC, 2), **f32)
    part = torch.empty((int(lib.slx_state_passing_bwd_partials_bytes(BH, NC, P, N)) // 4,), **f32)
    dU, dB, dC = torch.empty_like(U), torch.empty_like(B), torch.empty_like(C)
    dM, dK = torch.empty_like(M), torch.empty_like(K)
    cB, cU = torch.empty((b, h, NC, D), **f32), torch.empty((b, h, NC, P), **f32)
    ck = _lib.check
    ht = BH * T
    state_bytes = inc.numel() * inc.element_size()
    starts_bytes = starts.numel() * starts.element_size()

    def inc_fn():
        ck(lib.slx_chunk_increment_fwd(byref(s), U.data_ptr(), M.data_ptr(), K.data_ptr(), B.data_ptr(), None, None,
                                       inc.data_ptr(), sdt, mch.data_ptr(), st), "inc")

    def sp_fn():
        ck(lib.slx_state_passing_fwd(BH, NC, P, N, inc.data_ptr(), sdt, mch.data_ptr(), None, starts.data_ptr(), sdt,
                                     final.data_ptr(), st), "sp")

    def scan_fn():
        ck(lib.slx_chunk_scan_fwd(byref(s), U.data_ptr(), M.data_ptr(), K.data_ptr(), B.data_ptr(), C.data_ptr(),
                                  starts.data_ptr(), None, None, Y.data_ptr(), st), "scan")

    def dz0_fn():
        ck(lib.slx_chunk_scan_bwd_dz0(byref(s), M.data_ptr(), C.data_ptr(), dY.data_ptr(), dz0.data_ptr(), sdt, st),
           "dz0")

    def spb_fn():
        ck(lib.slx_state_passing_bwd(BH, NC, P, N, dz0.data_ptr(), sdt, mch.data_ptr(), starts.data_ptr(), sdt,
                                     final.data_ptr(), None, d_inc.data_ptr(), None, zdot.data_ptr(),
                                     part.data_ptr(), st), "spb")

    def bwd_fn():
        ck(lib.slx_chunk_scan_bwd(byref(s), U.data_ptr(), M.data_ptr(), K.data_ptr(), B.data_ptr(), C.data_ptr(), None,
                                  None, starts.data_ptr(), d_inc.data_ptr(), zdot.data_ptr(), dY.data_ptr(),
                                  dU.data_ptr(), dM.data_ptr(), dK.data_ptr(), dB.data_ptr(), dC.data_ptr(),
                                  cB.data_ptr(), cU.data_ptr(), st), "bwd")

    # (name, fn, algorithmic bytes, dense flops, bound); each stage needs the outputs of the ones before it
    plan = [
        ("chunk_increment_fwd", inc_fn, ht * (es * (P + D) + 24) + state_bytes, 2 * ht * P * D, "hbm"),
        ("state_passing_fwd", sp_fn, state_bytes + starts_bytes, 0, "hbm"),
        ("chunk_scan_fwd", scan_fn, ht * (es * (2 * P + 2 * D) + 24) + starts_bytes,
         ht * (2 * L * (D + P) + 2 * P * D), "tensor"),
        ("chunk_scan_bwd_dz0", dz0_fn, ht * (es * (P + D) + 8) + state_bytes, 2 * ht * P * D, "hbm"),
        ("state_passing_bwd", spb_fn, state_bytes + 2 * starts_bytes, 0, "hbm"),
        ("chunk_scan_bwd", bwd_fn, ht * (es * (3 * P + 4 * D) + 48) + 2 * starts_bytes,
         dense_flops_bwd_chunk(L, P, D) * BH * NC, "tensor"),
    ]
    out = []
    for name, fn, nbytes, flops, bound in plan:
        if only is not None and name != only:
            fn()  # the stages before the chosen one produce its inputs
            continue
        out.append(_stage(name, _time_kernel(fn, reps, warm), nbytes, flops, peaks, bound))
        if only is not None:
            break
    torch.cuda.synchronize()
    return out


def prep_conv_decode_timings(b, T, H, P, N, dtype, reps=10, warm=3, only=None, decode_batch=256):
    """Scan prep, conv (width 4, bias) and the one-token decode step by themselves (C ABI, kernel time)."""
    import torch

    from slinoss_b200 import _lib

    dev = torch.device("cuda", torch.cuda.current_device())
    peaks = _peaks()
    lib, st, ck = _lib.lib(), _lib.stream_ptr(dev), _lib.check
    es = torch.empty((), dtype=dtype).element_size()
    out = []
    want = lambda n: only is None or only == n
    g = torch.Generator().manual_seed(1)
    if want("scanprep_fwd") or want("scanprep_bwd"):
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

        def fwd():
            ck(lib.slx_scanprep_fwd(byref(s), value.data_ptr(), params.data_ptr(), bc.data_ptr(), bias.data_ptr(),
                                    scale.data_ptr(), U.data_ptr(), M.data_ptr(), K.data_ptr(), Bo.data_ptr(),
                                    Co.data_ptr(), st), "scanprep fwd")

        rows = b * T * H
        per_row = es * (P + 13 + 4 * N) + es * (P + 4 * N) + 24
        if want("scanprep_fwd"):
            out.append(_stage("scanprep_fwd", _time_kernel(fwd, reps, warm), rows * per_row, 0, peaks, "hbm"))
        if want("scanprep_bwd"):
            fwd()
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

            out.append(_stage("scanprep_bwd", _time_kernel(bwd, reps, warm), rows * (per_row + es * (13 + 4 * N)), 0,
                              peaks, "hbm", "reads params, bc and all five gradients; writes d_value, d_params, d_bc"))
            del dU, dB, dC, dM, dK, d_value, d_params, d_bc, ws
        del value, params, bc, U, Bo, Co, M, K
    if want("cconv1d_fwd") or want("cconv1d_bwd"):
        Cn, W = H * P, 4
        x = torch.randn(b, T, Cn, generator=g).to(dtype).to(dev)
        w = torch.randn(Cn, W, generator=g).to(dtype).to(dev)
        bias = torch.randn(Cn, generator=g).to(dtype).to(dev)
        y = torch.empty_like(x)
        nxt = torch.empty((b, Cn, W - 1), device=dev, dtype=dtype)
        s = _lib.ConvShape(b, T, Cn, W, _lib.dtype_code(dtype), 0, Cn, T * Cn)

        def cfwd():
            ck(lib.slx_cconv1d_fwd(byref(s), x.data_ptr(), w.data_ptr(), bias.data_ptr(), None, y.data_ptr(),
                                   nxt.data_ptr(), st), "conv fwd")

        if want("cconv1d_fwd"):
            out.append(_stage("cconv1d_fwd", _time_kernel(cfwd, reps, warm), b * T * Cn * 2 * es, 0, peaks, "hbm"))
        if want("cconv1d_bwd"):
            dy = torch.randn_like(y)
            dx = torch.empty_like(x)
            dw = torch.empty((Cn, W), device=dev, dtype=torch.float32)
            db = torch.empty((Cn,), device=dev, dtype=torch.float32)
            nbytes = int(lib.slx_cconv1d_bwd_workspace_bytes(byref(s)))
            ws = torch.empty((max(nbytes, 16),), device=dev, dtype=torch.uint8)

            def cbwd():
                ck(lib.slx_cconv1d_bwd(byref(s), x.data_ptr(), w.data_ptr(), bias.data_ptr(), None, dy.data_ptr(),
                                       None, dx.data_ptr(), dw.data_ptr(), db.data_ptr(), None, ws.data_ptr(), nbytes,
                                       st), "conv bwd")

            out.append(_stage("cconv1d_bwd", _time_kernel(cbwd, reps, warm), b * T * Cn * 3 * es, 0, peaks, "hbm"))
        del x, y
    if want("gate_skip_fwd") or want("gate_skip_bwd"):
        # the mixer's skip + re-layout + SiLU gate (one pass each way); gate read as a contiguous (b,T,H*P) tensor
        yh = torch.randn((b, H, T, P), generator=g).to(dtype).to(dev)
        uh = torch.randn((b, H, T, P), generator=g).to(dtype).to(dev)
        gt = torch.randn((b, T, H * P), generator=g).to(dtype).to(dev)
        sk = torch.randn((H * P,), generator=g).to(dev)
        og = torch.empty((b, T, H * P), device=dev, dtype=dtype)
        gs = _lib.GlueShape(b, T, H, P, _lib.dtype_code(dtype), H * P, T * H * P)
        n_el = b * T * H * P

        def gfwd():
            ck(lib.slx_gate_skip_fwd(byref(gs), yh.data_ptr(), uh.data_ptr(), gt.data_ptr(), sk.data_ptr(), og.data_ptr(),
                                     st), "gate_skip fwd")

        if want("gate_skip_fwd"):
            out.append(_stage("gate_skip_fwd", _time_kernel(gfwd, reps, warm), n_el * 4 * es, 0, peaks, "hbm",
                              "reads y, u, gate; writes the gated token-major rows"))
        if want("gate_skip_bwd"):
            go = torch.randn_like(og)
            dyh, duh, dgt = torch.empty_like(yh), torch.empty_like(uh), torch.empty_like(gt)
            dsk = torch.empty((H * P,), device=dev, dtype=torch.float32)
            nbytes = int(lib.slx_gate_skip_bwd_workspace_bytes(byref(gs)))
            wsg = torch.empty((max(nbytes, 16),), device=dev, dtype=torch.uint8)

            def gbwd():
                ck(lib.slx_gate_skip_bwd(byref(gs), yh.data_ptr(), uh.data_ptr(), gt.data_ptr(), sk.data_ptr(),
                                         go.data_ptr(), dyh.data_ptr(), duh.data_ptr(), dgt.data_ptr(), dsk.data_ptr(),
                                         wsg.data_ptr(), nbytes, st), "gate_skip bwd")

            out.append(_stage("gate_skip_bwd", _time_kernel(gbwd, reps, warm), n_el * 7 * es, 0, peaks, "hbm",
                              "reads y, u, gate, d_out; writes dy, du, d_gate (+ d_skip partials)"))
        del yh, uh, gt, og
    if want("cconv1d_update"):
        # one decode token through the conv (state shifted in place), serving batch
        bd, Cn, W = decode_batch, H * P, 4
        xu = torch.randn((bd, Cn), generator=g).to(dtype).to(dev)
        wu = torch.randn((Cn, W), generator=g).to(dtype).to(dev)
        bu = torch.randn((Cn,), generator=g).to(dtype).to(dev)
        su = torch.randn((bd, Cn, W - 1), generator=g).to(dtype).to(dev)
        yu = torch.empty_like(xu)
        cs = _lib.ConvShape(bd, 1, Cn, W, _lib.dtype_code(dtype), 1, Cn, Cn)

        def cupd():
            ck(lib.slx_cconv1d_update(byref(cs), xu.data_ptr(), wu.data_ptr(), bu.data_ptr(), su.data_ptr(), yu.data_ptr(),
                                      su.data_ptr(), st), "conv update")

        out.append(_stage("cconv1d_update", _time_kernel(cupd, reps, warm), bd * Cn * (2 + 2 * (W - 1)) * es, 0, peaks,
                          "hbm", f"one token, batch {bd}, {Cn} channels, SiLU fused, state updated in place "
                                 "(3.7 MB: latency-bound, not bandwidth-bound)"))
    if want("decode_step"):
        bd = decode_batch
        r = lambda *sh: torch.randn(*sh, generator=g)
        value, gate = r(bd, H, P).to(dtype).to(dev), r(bd, H, P).to(dtype).to(dev)
        params, bc = r(bd, H, 13).to(dtype).to(dev), r(bd, H, 4, N).to(dtype).to(dev)
        skip = r(H, P).to(dtype).to(dev)
        bias = torch.zeros(H, 13, device=dev)
        scale = torch.ones(H, 4, N, device=dev)
        st_in, st_out = r(bd, H, P, 2 * N).to(dev), torch.empty(bd, H, P, 2 * N, device=dev)
        bp, up = r(bd, H, 2 * N).to(dtype).to(dev), r(bd, H, P).to(dtype).to(dev)
        bl, ul = torch.empty_like(bp), torch.empty_like(up)
        o = torch.empty(bd, H * P, device=dev, dtype=dtype)
        s = _lib.DecodeShape(bd, H, P, N, _lib.dtype_code(dtype), 1, 1e-4, 1e-1, 0.9, 1.0, math.pi, 0.5, 1e-8)

        def dec():
            ck(lib.slx_decode_step(byref(s), value.data_ptr(), params.data_ptr(), bc.data_ptr(), gate.data_ptr(),
                                   skip.data_ptr(), bias.data_ptr(), scale.data_ptr(), st_in.data_ptr(), bp.data_ptr(),
                                   up.data_ptr(), o.data_ptr(), st_out.data_ptr(), bl.data_ptr(), ul.data_ptr(), st),
               "decode")

        out.append(_stage("decode_step", _time_kernel(dec, reps, warm), bd * H * 2 * P * 2 * N * 4, 0, peaks, "hbm",
                          f"one token, batch {bd} H{H} P{P} N{N}, fp32 state read and written"))
    torch.cuda.synchronize()
    return out


# ----------------------------------------------------------------------------------------------
# context-parallel mode, model-level configurations
# ----------------------------------------------------------------------------------------------

def _timed_steps(step, warm, min_ms, dist_barrier, dev, sampler_index=None):
    """Warm up, then repeat `step` until the region lasts >= min_ms.  Returns
    (ms per step as the max over ranks, steps timed, clock record or None)."""
    import torch
    import torch.distributed as dist

    multi = dist.is_initialized() and dist.get_world_size() > 1
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(warm):
        step()
    dist_barrier()
    e0.record()
    step()
    e1.record()
    dist_barrier()
    est = max(e0.elapsed_time(e1), 1e-3)
    n = max(3, int(math.ceil(min_ms / est)))
    if multi:
        tn = torch.tensor([n], device=dev, dtype=torch.int64)
        dist.all_reduce(tn, op=dist.ReduceOp.MAX)
        n = int(tn.item())
    sampler = ClockSampler(sampler_index).start() if sampler_index is not None else None
    dist_barrier()
    e0.record()
    for _ in range(n):
        step()
    e1.record()
    dist_barrier()
    clocks = sampler.stop() if sampler is not None else None
    t = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
    if multi:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item()) / n, n, clocks


def cp_measure(args, world, rank, local_rank, dev, barrier):
    """One b1 H32 P64 N128 sequence of --cp-T tokens, bf16 / fp32 state, split over the ranks along
    time (strong scaling); at N > 1 rank 0 also times the plain op on the whole sequence so that the
    line carries its own single-GPU base."""
    import torch

    import slinoss_b200 as sb
    from slinoss_b200.context_parallel import v2x2ssd_context_parallel

    T, L = args.cp_T, args.chunk
    T_loc = T // world
    cfg = dict(batch=1, heads=32, T=T_loc, P=64, N=128)
    inp = make_inputs(cfg, dev, seed=77 + rank, dtype=torch.bfloat16)
    leaves = [inp[k].requires_grad_(True) for k in ("U", "M", "K", "B", "C")]

    def step():
        Y, _ = v2x2ssd_context_parallel(*leaves, chunk_size=L)
        torch.autograd.grad(Y, leaves, inp["dY"])

    ms, n, clocks = _timed_steps(step, 3, 1000.0, barrier, dev, local_rank if rank == 0 else None)
    del inp, leaves
    torch.cuda.empty_cache()
    base_ms = None
    if world > 1:
        if rank == 0:
            cfg1 = dict(batch=1, heads=32, T=T, P=64, N=128)
            inp1 = make_inputs(cfg1, dev, seed=77, dtype=torch.bfloat16)
            lv = [inp1[k].requires_grad_(True) for k in ("U", "M", "K", "B", "C")]

            def step1():
                Y = sb.v2x2ssd_b200(*lv, chunk_size=L)
                torch.autograd.grad(Y, lv, inp1["dY"])

            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            for _ in range(3):
                step1()
            torch.cuda.synchronize()
            e0.record()
            for _ in range(10):
                step1()
            e1.record()
            torch.cuda.synchronize()
            base_ms = e0.elapsed_time(e1) / 10
            del inp1, lv
            torch.cuda.empty_cache()
        barrier()
    peaks = _peaks()
    alg = algorithmic_bytes_per_head_token(64, 256) * 32 * T
    per_gpu_gbs = alg / world / (ms * 1e-3) / 1e9
    out = dict(workload=f"context-parallel v2x2ssd fwd+bwd b1 H32 P64 N128 T{T} chunk {L}, {T_loc} tokens per rank",
               exchange="one all-gather of (segment transition, segment state) per direction + one-token halos, NCCL",
               scaling="strong", n_gpus=world, ms_per_step=ms, steps_timed=n, tokens_per_s=T / (ms * 1e-3),
               hbm_frac_per_gpu=per_gpu_gbs / peaks["hbm_gbs"], clocks=clocks)
    if base_ms is not None:
        out.update(single_gpu_ms_per_step=base_ms, efficiency_vs_n1=base_ms / (ms * world),
                   what_is_left="per-rank launch gaps and four small all-gathers per step; the collectives move "
                                "2 MiB per rank and direction")
    return out


def model_configs(args, world, rank, local_rank, dev, barrier):
    """The reference's own model code with every mixer on the B200 backends: one SLinOSSMixer layer
    (d_model 768, 12 heads, d_state 64, conv 4, chunk 64, batch 8, 2048 tokens, bf16) forward+backward,
    and the 24-layer NextCharLM (d_model 1024, 16 heads, d_state 128, byte vocabulary, uniform random
    tokens, batch 16 per GPU, 4096 tokens, bf16) training step (zero_grad, forward, cross-entropy,
    backward, clip, fused AdamW), data-parallel over the ranks.  Needs baseline/_ref."""
    import torch

    if not _have_reference():
        return None, None
    _import_reference()
    from slinoss.layers import SLinOSSMixer
    from slinoss.models.nextchar import NextCharLM

    import slinoss_b200 as sb

    c1 = None
    if world == 1:
        x = torch.randn((8, 2048, 768), device=dev, dtype=torch.bfloat16, requires_grad=True)

        def time_layer(kind):
            torch.manual_seed(0)
            mixer = SLinOSSMixer(768, d_state=64, expand=1, d_head=64, d_conv=4, chunk_size=64, device=dev,
                                 dtype=torch.bfloat16).train()
            if kind == "reference":
                from slinoss.layers.backend import (ReferenceCConv1dBackend, ReferenceMixerDecodeBackend,
                                                    ReferenceScanBackend, ReferenceScanPrepBackend)
                mixer.backend = ReferenceScanBackend(compute_dtype=None)
                mixer.scanprep.backend = ReferenceScanPrepBackend()
                mixer.cconv_backend = ReferenceCConv1dBackend()
                mixer.decode_backend = ReferenceMixerDecodeBackend()
            else:
                sb.use_b200_backends(mixer, fuse_glue=(kind == "fused"))

            def layer_step():
                y = mixer(x)
                y.float().square().mean().backward()

            ms, n, _ = _timed_steps(layer_step, 3, 300.0 if kind != "reference" else 150.0, barrier, dev)
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            for _ in range(3):
                layer_step()
            torch.cuda.synchronize()
            wall = (time.perf_counter() - t0) / 3 * 1e3
            del mixer
            torch.cuda.empty_cache()
            return ms, n, wall

        ms_f, n_f, wall_f = time_layer("fused")
        ms_p, _, _ = time_layer("plain")
        try:  # the reference's own torch backends on the same GPU: the "before" of this drop-in
            ms_r, _, _ = time_layer("reference")
        except Exception as exc:  # e.g. out of memory in the reference's autograd graph
            ms_r = None
            print(f"[bench] reference backends on the GPU failed: {exc!r}"[:300], file=sys.stderr)
        # host cost of the scan op at this layer's shape (b8 H12 T2048 P64 N64): Python-level forward + backward
        # wall time against the sum of its kernels timed one by one through the C ABI
        ocfg = dict(batch=8, heads=12, T=2048, P=64, N=64)
        oin = make_inputs(ocfg, dev, 7, torch.bfloat16)
        olv = [oin[k].requires_grad_(True) for k in ("U", "M", "K", "B", "C")]

        def op_step():
            Yo = sb.v2x2ssd_b200(*olv, chunk_size=128)
            torch.autograd.grad(Yo, olv, oin["dY"])

        for _ in range(5):
            op_step()
        torch.cuda.synchronize()
        t0 = time.perf_counter()
        for _ in range(50):
            op_step()
        torch.cuda.synchronize()
        op_wall = (time.perf_counter() - t0) / 50 * 1e3
        op_kernels = sum(st["ms"] for st in scan_stage_timings(
            {k: v.detach() for k, v in oin.items()}, 8, 12, 2048, 64, 64, 128, torch.bfloat16, reps=10, warm=3))
        del oin, olv
        c1 = dict(workload="reference SLinOSSMixer layer fwd+bwd, d_model 768, 12 heads x 64, d_state 64, conv 4, "
                           "chunk 64, batch 8, 2048 tokens, bf16 / fp32 scan state, "
                           "use_b200_backends(mixer, fuse_glue=True)",
                  ms_per_step=ms_f, steps_timed=n_f, wall_ms_per_step=wall_f, tokens_per_s=8 * 2048 / (ms_f * 1e-3),
                  unfused_glue_ms_per_step=ms_p, reference_backends_same_gpu_ms_per_step=ms_r,
                  speedup_vs_reference_backends=(None if ms_r is None else ms_r / ms_f),
                  scan_op_wall_ms=op_wall, scan_op_kernel_ms_sum=op_kernels,
                  scan_op_wall_over_kernels=op_wall / op_kernels)
        del x
        torch.cuda.empty_cache()
    torch.manual_seed(1)
    model = NextCharLM(vocab_size=256, block_size=4096, d_model=1024, n_layers=24, d_state=128, expand=1,
                       d_head=64, d_conv=4, chunk_size=64).to(device=dev, dtype=torch.bfloat16)
    sb.use_b200_backends(model, fuse_glue=True)
    ddp = model
    if world > 1:
        ddp = torch.nn.parallel.DistributedDataParallel(model, device_ids=[local_rank])
    params = [p for p in model.parameters() if p.requires_grad]
    opt = torch.optim.AdamW(params, lr=3e-4, weight_decay=0.1, fused=True)
    g = torch.Generator(device=dev).manual_seed(2 + rank)
    xb = torch.randint(0, 256, (16, 4096), device=dev, generator=g)
    yb = torch.randint(0, 256, (16, 4096), device=dev, generator=g)

    def train_step():
        opt.zero_grad(set_to_none=True)
        logits = ddp(xb)
        loss = torch.nn.functional.cross_entropy(logits.float().view(-1, 256), yb.view(-1))
        loss.backward()
        torch.nn.utils.clip_grad_norm_(params, max_norm=1.0, foreach=True)
        opt.step()

    ms, n, _ = _timed_steps(train_step, 3, 1500.0, barrier, dev)
    c3 = dict(workload="reference NextCharLM training step, 24 layers, d_model 1024, 16 heads x 64, d_state 128, "
                       "vocab 256 (uniform random tokens), batch 16 per GPU, 4096 tokens, bf16, "
                       "use_b200_backends(model, fuse_glue=True), "
                       + (f"DDP over {world} GPUs" if world > 1 else "1 GPU"),
              ms_per_step=ms, steps_timed=n, tokens_per_s=16 * 4096 * world / (ms * 1e-3), n_gpus=world)
    del model, ddp, opt
    torch.cuda.empty_cache()
    return c1, c3


# ----------------------------------------------------------------------------------------------

def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--chunk", type=int, default=128)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--T", type=int, default=HEADLINE["T"])
    ap.add_argument("--batch", type=int, default=HEADLINE["batch"])
    ap.add_argument("--heads", type=int, default=HEADLINE["heads"])
    ap.add_argument("--N", type=int, default=HEADLINE["N"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-stages", action="store_true")
    ap.add_argument("--no-cp", action="store_true")
    ap.add_argument("--no-models", action="store_true")
    ap.add_argument("--cp-T", type=int, default=262144)
    ap.add_argument("--stages-only", action="store_true",
                    help="print one JSON line per kernel (C-ABI calls, CUDA events) and exit; for profiler captures")
    ap.add_argument("--only", default=None, help="with --stages-only: time this kernel alone")
    ap.add_argument("--reps", type=int, default=10)
    ap.add_argument("--warm", type=int, default=3)
    args = ap.parse_args()
    cfg = dict(HEADLINE, T=args.T, batch=args.batch, heads=args.heads, N=args.N)
    if args.impl == "reference":
        return run_reference_arm(args, cfg)

    import torch
    import torch.distributed as dist

    import slinoss_b200 as sb
    from slinoss_b200 import _lib

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    dtype = torch.bfloat16
    L = args.chunk
    b, h, T, P, N = cfg["batch"], cfg["heads"], cfg["T"], cfg["P"], cfg["N"]
    D, BH, NC = 2 * N, b * h, (T + L - 1) // L

    if args.stages_only:
        inp = make_inputs(cfg, dev, seed=1234, dtype=dtype)
        scan_names = ("chunk_increment_fwd", "state_passing_fwd", "chunk_scan_fwd", "chunk_scan_bwd_dz0",
                      "state_passing_bwd", "chunk_scan_bwd")
        lines = []
        if args.only is None or args.only in scan_names:
            lines += scan_stage_timings(inp, b, h, T, P, N, L, dtype, args.reps, args.warm, args.only)
        if args.only is None or args.only not in scan_names:
            lines += prep_conv_decode_timings(b, T, h, P, N, dtype, args.reps, args.warm, args.only)
        for ln in lines:
            print(json.dumps(ln), flush=True)
        return 0

    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    else:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29533")
        dist.init_process_group("nccl", rank=0, world_size=1, device_id=dev)
    W = max(args.warmup, 3)
    K = args.steps
    peaks = _peaks()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    inp = make_inputs(cfg, dev, seed=1234 + rank, dtype=dtype)
    leaves = {k: inp[k].requires_grad_(True) for k in ("U", "M", "K", "B", "C")}

    def step():
        Y = sb.v2x2ssd_b200(leaves["U"], leaves["M"], leaves["K"], leaves["B"], leaves["C"], chunk_size=L)
        return Y, torch.autograd.grad(Y, list(leaves.values()), inp["dY"])

    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for _ in range(W):
        step()
    barrier()
    e0.record()
    step()
    e1.record()
    barrier()
    est = torch.tensor([max(e0.elapsed_time(e1), 1e-3)], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(est, op=dist.ReduceOp.MIN)
    inner = max(1, int(math.ceil(1000.0 / (K * float(est.item())))))  # the timed region lasts >= 1 s
    sampler = ClockSampler(local_rank).start() if rank == 0 else None
    barrier()
    e0.record()
    for _ in range(K * inner):
        step()
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    clocks = sampler.stop() if rank == 0 else None
    t = torch.tensor([ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step = float(t.item()) / (K * inner)
    tokens_step = cfg["batch"] * cfg["T"] * world
    value = tokens_step / (ms_step * 1e-3)

    # ---- end to end: host buffers in, host buffers out --------------------------------
    # Every step copies its inputs from pinned host memory and its outputs (Y and the five
    # gradients) back to pinned host memory.  The copies run on their own streams with two
    # buffer slots, so that the upload of step i+1, the kernels of step i and the download of
    # step i-1 overlap (PCIe is full duplex); all copies of the timed steps lie inside the timed region.
    e2e = None
    if not args.no_e2e:
        host_in = {k: v.detach().cpu().pin_memory() for k, v in inp.items()}
        dev_in = [{k: torch.empty_like(v, device=dev) for k, v in host_in.items()} for _ in range(2)]
        host_out = [None, None]
        cur = torch.cuda.current_stream()
        s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()
        ev_in = [torch.cuda.Event() for _ in range(2)]
        ev_used = [torch.cuda.Event() for _ in range(2)]      # kernels that read slot's inputs are done
        ev_out = [torch.cuda.Event() for _ in range(2)]       # slot's host output buffers are free again
        for e in ev_used + ev_out:
            e.record(cur)

        def e2e_step(i):
            slot = i % 2
            with torch.cuda.stream(s_in):
                s_in.wait_event(ev_used[slot])
                for k in host_in:
                    dev_in[slot][k].copy_(host_in[k], non_blocking=True)
                ev_in[slot].record(s_in)
            cur.wait_event(ev_in[slot])
            lv = [dev_in[slot][k].requires_grad_(True) for k in ("U", "M", "K", "B", "C")]
            Y = sb.v2x2ssd_b200(*lv, chunk_size=L)
            gr = torch.autograd.grad(Y, lv, dev_in[slot]["dY"])
            outs = (Y.detach(),) + tuple(gr)
            ev_used[slot].record(cur)
            for k in ("U", "M", "K", "B", "C"):
                dev_in[slot][k].requires_grad_(False)
            if host_out[slot] is None:
                host_out[slot] = [torch.empty(o.shape, dtype=o.dtype).pin_memory() for o in outs]
            with torch.cuda.stream(s_out):
                s_out.wait_event(ev_used[slot])
                s_out.wait_event(ev_out[slot])
                for ho, o in zip(host_out[slot], outs):
                    o.record_stream(s_out)
                    ho.copy_(o, non_blocking=True)
                ev_out[slot].record(s_out)

        for i in range(2):
            e2e_step(i)
        cur.wait_stream(s_in)
        cur.wait_stream(s_out)
        barrier()
        Ke = max(4, min(K, 10))
        e0.record()
        for i in range(Ke):
            e2e_step(i)
        cur.wait_stream(s_in)
        cur.wait_stream(s_out)
        e1.record()
        barrier()
        te = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
        if world > 1:
            dist.all_reduce(te, op=dist.ReduceOp.MAX)
        h2d = sum(v.numel() * v.element_size() for v in host_in.values())
        d2h = sum(v.numel() * v.element_size() for v in host_out[0])
        e2e = dict(value=tokens_step / (float(te.item()) / Ke * 1e-3), unit="tokens/s",
                   h2d_bytes_per_step=h2d, d2h_bytes_per_step=d2h, steps=Ke,
                   overlap="upload, kernels and download of consecutive steps on three streams, two buffer slots")
        # what the host link gives for the same buffers with no kernels in between (this rank's copies while the
        # other ranks do the same): upload alone, download alone, both at once.  The end-to-end step cannot be
        # faster than its larger copy at the both-at-once rate.
        outs0 = [torch.empty(o.shape, dtype=o.dtype, device=dev) for o in host_out[0]]

        def up():
            with torch.cuda.stream(s_in):
                for k in host_in:
                    dev_in[0][k].copy_(host_in[k], non_blocking=True)

        def down():
            with torch.cuda.stream(s_out):
                for ho, o in zip(host_out[0], outs0):
                    ho.copy_(o, non_blocking=True)

        def timed(fns, reps=3):
            barrier()
            t0 = time.perf_counter()
            for _ in range(reps):
                for f in fns:
                    f()
            s_in.synchronize()
            s_out.synchronize()
            return (time.perf_counter() - t0) / reps

        up(), down()
        t_up, t_down, t_both = timed([up]), timed([down]), timed([up, down])
        step_s = float(te.item()) / Ke * 1e-3
        e2e["host_link"] = dict(h2d_gbs=round(h2d / t_up / 1e9, 1), d2h_gbs=round(d2h / t_down / 1e9, 1),
                                both_at_once_gbs_each_way=round(max(h2d, d2h) / t_both / 1e9, 1),
                                step_over_copy_floor=round(step_s / t_both, 3))
        del host_in, host_out, dev_in, outs0

    # ---- every kernel by itself; the dominant one gives the roofline object ----------------------
    stages = None
    roofline = None
    if rank == 0 and not args.no_stages:
        with torch.no_grad():
            stages = scan_stage_timings(inp, b, h, T, P, N, L, dtype)
            if world == 1:
                stages += prep_conv_decode_timings(b, T, h, P, N, dtype)
        dom = max((s for s in stages if s["stage"].startswith("chunk_scan")), key=lambda s: s["ms"])
        traffic, tsrc = None, None
        tfile = ROOT / "profiles" / "dominant_kernel_traffic.json"
        if tfile.exists():
            rec = json.loads(tfile.read_text()).get(dom["stage"])
            if rec and rec.get("P") == P and rec.get("N") == N and rec.get("chunk") == L:
                traffic = rec["dram_bytes"] / rec["chunks"] * BH * NC
                tsrc = (f"ncu capture of {rec['chunks']} chunks ({rec['kernel']}) scaled by the chunk count, "
                        "profiles/dominant_kernel_traffic.json")
        roofline = dict(kernel=dom["stage"], bound="tensor", achieved=dom["achieved"], peak=peaks["tflops_burst"],
                        unit="TFLOP/s", frac=dom["achieved"] / peaks["tflops_burst"], traffic=traffic,
                        traffic_source=tsrc, ms_per_launch=dom["ms"], flops_per_launch=dom["flops"],
                        algorithmic_gbs=dom["gbs"], frac_hbm=dom["frac_hbm"],
                        peak_source=peaks["source"] + " (bf16 burst: the kernel is timed alone)")
    alg_bytes = algorithmic_bytes_per_head_token(P, D) * BH * T
    hbm = alg_bytes / (ms_step * 1e-3) / 1e9
    roofline_op = dict(bound="hbm", achieved=hbm, peak=peaks["hbm_gbs"], unit="GB/s", frac=hbm / peaks["hbm_gbs"],
                       algorithmic_bytes_per_step=alg_bytes, peak_source=peaks["source"])
    del inp, leaves
    torch.cuda.empty_cache()

    cp = None
    if not args.no_cp:
        cp = cp_measure(args, world, rank, local_rank, dev, barrier)
    c1 = c3 = None
    if not args.no_models:
        c1, c3 = model_configs(args, world, rank, local_rank, dev, barrier)

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        t_one, _, _ = cpu_sample(cfg, L, 1)
        # ~15 s of host work: the whole workload when it fits, else as many slices as do
        sec, units, info = cpu_sample(cfg, L, max(1, min(cfg["batch"] * cfg["heads"], int(15.0 / max(t_one, 1e-3)))),
                                      warm=False)
        cpu = dict(info, value=cpu_tokens_per_s(cfg, sec, units, T), seconds=round(sec, 2))

    if rank == 0:
        n_kernels = 8  # increment, state pass, scan | dZ0, reverse state pass, zdot reduce, per-chunk backward, carry fix-up
        line = dict(metric=METRIC, value=value, unit="tokens/s", n_gpus=world, steps=K, inner_repeats=inner, warmup=W,
                    ms_per_step=ms_step, higher_is_better=True, scaling="weak", vs_baseline=None, dtype="bf16",
                    data="synthetic",
                    config=dict(workload=workload_name(cfg, L), l2="inputs larger than L2 (1.4 GB per step)",
                                sharding="batch x heads per rank"),
                    clocks=clocks, e2e=e2e, gpu_launches=n_kernels * K * inner, roofline=roofline,
                    roofline_whole_op=roofline_op, stages=stages, cp=cp, config1=c1, config3=c3, cpu_baseline=cpu)
        print(json.dumps(line))
    dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
