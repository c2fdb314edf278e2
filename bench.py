"""Headline benchmark: v2x2ssd forward+backward tokens/s on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--chunk 64|128] [--impl reference]

One "step" is one forward + one backward of the scan over one batch of seeded
synthetic inputs of the headline configuration (batch 4, heads 32, P 64, N 128,
T 8192, bf16 U/B/C/dY, fp32 M/K/state; parameter distributions of BASELINE
config 2).  Rank 0 prints ONE JSON line:

  value      tokens/s (tokens = batch*T per call, all heads) with inputs resident
             in HBM, whole job (sum over ranks; every rank runs its own batch:
             weak scaling, no collective on the data path)
  e2e        the same metric through the public op with HOST buffers: pinned
             host -> device copies of every input and device -> host copies of
             every result inside the timed region
  roofline   the dominant kernel (per-chunk backward), timed alone with CUDA
             events: algorithmic dense-tile flops per launch / duration against
             the measured bf16 tensor peak; plus the whole-op HBM figure
  cpu_baseline  the CPU oracle (a C port of the reference algorithm) timed on the
             host cores on a bounded sample of the same workload (rank 0, N=1)

``--impl reference`` times the reference algorithm on the host CPU (the C port in
oracle/; the Python reference itself cannot travel to the GPU box) on a bounded
sample per step and prints the same line shape.
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

HEADLINE = dict(batch=4, heads=32, T=8192, P=64, N=128)
METRIC = "v2x2ssd fwd+bwd tokens/sec (H32 P64 N128 T8192 b4, bf16 in / fp32 state)"


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
    """Dense-tile flops of the per-chunk backward kernel (what a tile engine
    executes without skipping masked tiles), merged-tap formulation:
    G=dY U^T, S=Q K^T, dq=dS K, X=dS^T Q, dU=S^T dY (L*L tiles) plus
    dY Z0, U Lambda, B^ Lambda^T (L*P*D tiles)."""
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
    """nvidia-smi clocks/throttle reasons sampled every 50 ms during the timed region."""

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
        except Exception:
            self.proc = None

    def stop(self):
        out = dict(sm_mhz=None, sm_max_mhz=None, reasons=[])
        if self.proc is None:
            return out
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        try:
            rows = [r.split(",") for r in Path(self.path).read_text().strip().splitlines() if r.strip()]
            sm = sorted(float(r[1]) for r in rows if len(r) >= 9)
            if sm:
                out["sm_mhz"] = sm[len(sm) // 2]
                out["sm_max_mhz"] = float(rows[0][2])
            names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
            seen = set()
            for r in rows:
                if len(r) < 9:
                    continue
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


def run_reference_arm(args, cfg):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return 0
    threads = os.cpu_count() or 1
    bh_s, T_s = min(threads, cfg["batch"] * cfg["heads"]), min(4096, cfg["T"])
    for _ in range(max(args.warmup, 1)):
        cpu_port_time(cfg, args.chunk, bh_s, 256, threads)
    times = [cpu_port_time(cfg, args.chunk, bh_s, T_s, threads) for _ in range(args.steps)]
    sec = sum(times) / len(times)
    val = cpu_tokens_per_s(cfg, sec, bh_s, T_s)
    sample = (f"{bh_s} (batch,head) sequences x {T_s} tokens per step, fwd+bwd, float64, OpenMP; "
              f"extrapolated to {cfg['batch'] * cfg['heads']} sequences x {cfg['T']} tokens")
    line = dict(impl="reference", metric=METRIC, value=val, unit="tokens/s", n_gpus=args.gpus,
                steps=args.steps, warmup=args.warmup, ms_per_step=sec * 1e3, higher_is_better=True,
                scaling="weak", vs_baseline=None, dtype="f64", data="synthetic",
                config=dict(workload=f"v2x2ssd fwd+bwd b{cfg['batch']} H{cfg['heads']} P{cfg['P']} N{cfg['N']} "
                                     f"T{cfg['T']} chunk {args.chunk}"),
                cpu_baseline=dict(value=val, unit="tokens/s", cores=threads, kind="port", sample=sample),
                e2e=dict(value=val, unit="tokens/s", h2d_bytes_per_step=0, d2h_bytes_per_step=0),
                gpu_launches=0)
    print(json.dumps(line))
    return 0


def run_context_parallel(args) -> int:
    """BASELINE config 4: batch 1, heads 32, P 64, N 128, T 262144, bf16 / fp32 state, the
    sequence split over the ranks; only chunk-final states and one-token halos cross ranks
    (NCCL send/recv over NVLink).  Strong scaling: total work fixed."""
    import torch
    import torch.distributed as dist

    from slinoss_b200.context_parallel import v2x2ssd_context_parallel

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world == 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        os.environ.setdefault("MASTER_PORT", "29533")
        dist.init_process_group("nccl", rank=0, world_size=1, device_id=dev)
    else:
        dist.init_process_group("nccl", device_id=dev)
    T, L = args.cp_T, args.chunk
    T_loc = T // world
    cfg = dict(batch=1, heads=32, T=T_loc, P=64, N=128)
    inp = make_inputs(cfg, dev, seed=77 + rank, dtype=torch.bfloat16)
    leaves = [inp[k].requires_grad_(True) for k in ("U", "M", "K", "B", "C")]

    def step():
        Y, _ = v2x2ssd_context_parallel(*leaves, chunk_size=L)
        torch.autograd.grad(Y, leaves, inp["dY"])

    W, K = max(args.warmup, 3), args.steps
    for _ in range(W):
        step()
    dist.barrier()
    torch.cuda.synchronize()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(K):
        step()
    e1.record()
    dist.barrier()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1)], device=dev, dtype=torch.float64)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    clocks = sampler.stop() if rank == 0 else None
    ms_step = float(t.item()) / K
    peaks = _peaks()
    alg = algorithmic_bytes_per_head_token(64, 256) * 32 * T
    if rank == 0:
        per_gpu_gbs = alg / world / (ms_step * 1e-3) / 1e9
        print(json.dumps(dict(
            metric="v2x2ssd fwd+bwd tokens/sec, context-parallel (b1 H32 P64 N128, bf16 in / fp32 state)",
            value=T / (ms_step * 1e-3), unit="tokens/s", n_gpus=world, steps=K, warmup=W, ms_per_step=ms_step,
            higher_is_better=True, scaling="strong", vs_baseline=None, dtype="bf16", data="synthetic",
            config=dict(workload=f"context-parallel v2x2ssd fwd+bwd b1 H32 P64 N128 T{T} chunk {L}, "
                                 f"{T_loc} tokens per rank", exchange="chunk-final state + 1-token halo per hop, "
                                 "NCCL send/recv", l2="inputs larger than L2"),
            clocks=clocks, gpu_launches=(8 + 3) * K,
            roofline_whole_op=dict(bound="hbm", achieved=per_gpu_gbs, peak=peaks["hbm_gbs"], unit="GB/s per GPU",
                                   frac=per_gpu_gbs / peaks["hbm_gbs"], peak_source=peaks["source"]))))
    dist.destroy_process_group()
    return 0


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--chunk", type=int, default=128)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--T", type=int, default=HEADLINE["T"])
    ap.add_argument("--batch", type=int, default=HEADLINE["batch"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--mode", default="batch", choices=["batch", "cp"],
                    help="batch: every rank runs its own (batch x heads) shard (headline, weak scaling); "
                         "cp: one b1 H32 T262144 sequence split over the ranks along time (strong scaling)")
    ap.add_argument("--cp-T", type=int, default=262144)
    args = ap.parse_args()
    cfg = dict(HEADLINE, T=args.T, batch=args.batch)
    if args.impl == "reference":
        return run_reference_arm(args, cfg)
    if args.mode == "cp":
        return run_context_parallel(args)

    import torch
    import torch.distributed as dist

    import slinoss_b200 as sb
    from slinoss_b200 import _lib

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=dev)
    dtype = torch.bfloat16
    L = args.chunk
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

    for _ in range(W):
        step()
    barrier()
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    e0.record()
    for _ in range(K):
        step()
    e1.record()
    barrier()
    ms = e0.elapsed_time(e1)
    clocks = sampler.stop() if rank == 0 else None
    t = torch.tensor([ms], device=dev, dtype=torch.float64)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_step = float(t.item()) / K
    tokens_step = cfg["batch"] * cfg["T"] * world
    value = tokens_step / (ms_step * 1e-3)

    # ---- end to end: host buffers in, host buffers out --------------------------------
    # Every step copies its inputs from pinned host memory and its outputs (Y and the five
    # gradients) back to pinned host memory.  The copies run on their own streams with two
    # buffer slots, so that the upload of step i+1, the kernels of step i and the download of
    # step i-1 overlap (PCIe is full duplex); all copies of the K steps lie inside the timed region.
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
        del host_in, host_out, dev_in

    # ---- dominant kernel alone: per-chunk backward -------------------------------------
    b, h, T, P, N = cfg["batch"], cfg["heads"], cfg["T"], cfg["P"], cfg["N"]
    D, BH, NC = 2 * N, b * h, (T + L - 1) // L
    lib = _lib.lib()
    shape = _lib.scan_shape(BH, T, P, N, L, dtype)
    st = _lib.stream_ptr(dev)
    f32 = dict(device=dev, dtype=torch.float32)
    with torch.no_grad():
        U, M, Kt, B, C, dY = (inp[k].detach() for k in ("U", "M", "K", "B", "C", "dY"))
        Y = torch.empty_like(U)
        final = torch.empty((b, h, P, D), **f32)
        starts = torch.empty((b, h, NC, P, D), device=dev, dtype=_lib.starts_dtype(shape))
        inc_buf = torch.empty((b, h, NC, P, D), **f32)
        mch = torch.empty((b, h, NC, 2), **f32)
        _lib.check(lib.slx_v2x2ssd_fwd(byref(shape), U.data_ptr(), M.data_ptr(), Kt.data_ptr(), B.data_ptr(),
                                       C.data_ptr(), None, None, None, Y.data_ptr(), final.data_ptr(),
                                       starts.data_ptr(), mch.data_ptr(), inc_buf.data_ptr(), st), "fwd")
        del inc_buf
        dz0 = torch.empty((b, h, NC, P, D), **f32)
        d_inc = torch.empty((b, h, NC, P, D), device=dev, dtype=starts.dtype)
        zdot = torch.empty((b, h, NC, 2), **f32)
        part = torch.empty((BH * NC * 2 * 64,), **f32)
        _lib.check(lib.slx_chunk_scan_bwd_dz0(byref(shape), M.data_ptr(), C.data_ptr(), dY.data_ptr(),
                                              dz0.data_ptr(), st), "dz0")
        _lib.check(lib.slx_state_passing_bwd(BH, NC, P, N, dz0.data_ptr(), mch.data_ptr(), starts.data_ptr(),
                                             _lib.dtype_code(starts.dtype), final.data_ptr(), None,
                                             d_inc.data_ptr(), None, zdot.data_ptr(),
                                             part.data_ptr(), st), "state bwd")
        del dz0
        dU, dB, dC = torch.empty_like(U), torch.empty_like(B), torch.empty_like(C)
        dM, dK = torch.empty_like(M), torch.empty_like(Kt)
        cB, cU = torch.empty((b, h, NC, D), **f32), torch.empty((b, h, NC, P), **f32)

        def bwd_kernel():
            _lib.check(lib.slx_chunk_scan_bwd(byref(shape), U.data_ptr(), M.data_ptr(), Kt.data_ptr(), B.data_ptr(),
                                              C.data_ptr(), None, None, starts.data_ptr(), d_inc.data_ptr(),
                                              zdot.data_ptr(), dY.data_ptr(), dU.data_ptr(), dM.data_ptr(),
                                              dK.data_ptr(), dB.data_ptr(), dC.data_ptr(), cB.data_ptr(),
                                              cU.data_ptr(), st), "chunk_scan_bwd")

        for _ in range(3):
            bwd_kernel()
        torch.cuda.synchronize()
        reps = max(3, min(K, 10))
        e0.record()
        for _ in range(reps):
            bwd_kernel()
        e1.record()
        torch.cuda.synchronize()
        k_ms = e0.elapsed_time(e1) / reps
    flops = dense_flops_bwd_chunk(L, P, D) * BH * NC
    achieved = flops / (k_ms * 1e-3) / 1e12
    # DRAM bytes of one launch: ncu measured 355.9 MB for 1024 chunks of this kernel at P64 N128
    # (the capture's summary is committed under profiles/); the kernel's traffic is per chunk
    traffic = None
    if L == 128 and P == 64 and N == 128:
        traffic = 355.9e6 / 1024 * BH * NC
    roofline = dict(kernel="chunk_scan_bwd_tc_kernel" if L == 128 else "chunk_scan_bwd_kernel", bound="tensor",
                    achieved=achieved, peak=peaks["tflops"], unit="TFLOP/s", frac=achieved / peaks["tflops"],
                    traffic=traffic, traffic_source="ncu capture of 1024 chunks scaled by the chunk count",
                    ms_per_launch=k_ms, flops_per_launch=flops,
                    peak_source=peaks["source"] + " (bf16 sustained)")
    alg_bytes = algorithmic_bytes_per_head_token(P, D) * BH * T
    per_rank_ms = ms_step
    hbm = alg_bytes / (per_rank_ms * 1e-3) / 1e9
    roofline_op = dict(bound="hbm", achieved=hbm, peak=peaks["hbm_gbs"], unit="GB/s", frac=hbm / peaks["hbm_gbs"],
                       algorithmic_bytes_per_step=alg_bytes, peak_source=peaks["source"])

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        threads = os.cpu_count() or 1
        bh_s, T_s = min(2 * threads, BH), T
        cpu_port_time(cfg, L, min(threads, bh_s), 256, threads)
        sec = cpu_port_time(cfg, L, bh_s, T_s, threads)
        cpu = dict(value=cpu_tokens_per_s(cfg, sec, bh_s, T_s), unit="tokens/s", cores=threads, kind="port",
                   sample=f"{bh_s} (batch,head) sequences x {T_s} tokens, fwd+bwd, float64 C port with OpenMP, "
                          f"{sec:.2f} s; extrapolated to {BH} sequences x {T} tokens")

    if rank == 0:
        line = dict(metric=METRIC, value=value, unit="tokens/s", n_gpus=world, steps=K, warmup=W,
                    ms_per_step=ms_step, higher_is_better=True, scaling="weak", vs_baseline=None, dtype="bf16",
                    data="synthetic",
                    config=dict(workload=f"v2x2ssd fwd+bwd b{b} H{h} P{P} N{N} T{T} chunk {L} per GPU",
                                l2="inputs larger than L2 (1.4 GB per step)", sharding="batch x heads per rank"),
                    clocks=clocks, e2e=e2e, gpu_launches=8 * K, roofline=roofline, roofline_whole_op=roofline_op,
                    cpu_baseline=cpu)
        print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()
    return 0


if __name__ == "__main__":
    sys.exit(main())
