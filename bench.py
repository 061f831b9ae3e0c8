"""Benchmark of the SPH perception hot path: binning + perception forward + backward.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference] [--workload NAME]

One "step" is one pass of the hot path over one batch of synthetic particle systems of the
headline configuration (3D, B=4 systems of N=65,536 particles, C=32 features, ~40 neighbours):
grid build, reorder into cell order, density sweep, blur+gradient sweep, blur+gradient backward
sweep, density backward sweep.  The metric is particles/s through forward+backward (binning
included).  Prints ONE JSON line on rank 0.

* ``value``: inputs resident in HBM, CUDA-event time per step, L2 flushed between steps.
* ``e2e``: the same step driven through the public ``sphops`` API from pinned HOST buffers, with
  the host->device copy of positions and features and the device->host copy of both gradients
  inside the timed region.
* ``roofline``: the dominant kernel (blur+gradient backward) timed by its own event pair inside
  the timed steps, against the measured HBM copy bandwidth.
* ``cpu_baseline``: the CPU oracle (a port of the reference's operators) on the host cores, on a
  bounded sample of the same workload; ``cpu_baseline_reference``: the reference's own
  ``sphops/torch_sph.py`` on its CPU-runnable configuration (when a copy of the reference is
  present under ``baseline/_ref``).  ``--impl reference`` prints the CPU arm as its own line.
* ``gpu_reference``: the reference's own CUDA kernels (compiled for this GPU by
  ``baseline/gpu_ref``) on the same inputs, when that library is present: a same-GPU comparator.
* ``strong_scaling``: the many-small-systems step (256 systems) and the 64-step periodic rollout
  (64 systems of 262,144 particles) with their systems sharded over the ranks.

For N > 1 (torchrun) every rank runs the full headline workload on its own GPU (independent
systems, weak scaling) plus one NCCL all-reduce of an MLP-gradient-sized buffer per step on a side
stream; time is the max over ranks.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
if str(ROOT) not in sys.path:
    sys.path.insert(0, str(ROOT))

METRIC = "perception_fwd_bwd_particles_per_s"
UNIT = "particles/s"
MLP_GRAD_FLOATS = 10880  # parameters of the reference's 66->128->18 update MLP


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=10)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--workload", default=None)
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extras", action="store_true",
                    help="skip the strong-scaling shards and the reference-kernel comparator")
    ap.add_argument("--tile-forward", default=None, metavar="ROWS,PARTICLES,STAGES,WARPS,CELLS",
                    help="run the blur+gradient forward sweep on the cell-tile streaming engine with this tuning "
                         "(0 = automatic), e.g. 448,32,2,24,2")
    ap.add_argument("--tile-backward", default=None, metavar="ROWS,PARTICLES,STAGES,WARPS,CELLS",
                    help="same for the backward sweep, e.g. 128,32,2,8,2")
    return ap.parse_args()


def measured_peak_gbs():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


def workload_config(w):
    """The workload both arms are timed on (identical in the GPU line and the reference line)."""
    return {"workload": w.name, "dim": w.dim, "systems": w.B, "particles_per_system": w.N, "features": w.C,
            "eps": w.eps, "grid": list(w.grid_size), "boundary": w.boundary,
            "max_particles_per_block": w.max_particles_per_block,
            "upstream_gradients": "N(0,1)", "l2": "256 MB buffer written between timed GPU steps (L2 flush)"}


# ----------------------------------------------------------------------------------------------
# CPU arm: the oracle port on the host cores
# ----------------------------------------------------------------------------------------------
def cpu_oracle_step(w, x, s, ups, systems):
    """Forward + chained backward of `systems` systems with the C oracle; returns seconds."""
    import numpy as np
    import oracle

    xs, ss = x[:systems].numpy(), s[:systems].numpy()
    u = {k: v[:systems].numpy() for k, v in ups.items()}
    t0 = time.perf_counter()
    fw = oracle.forward(xs, w.eps, w.dim, s=ss, want=("rho",))
    rho = fw["rho"].astype(np.float32)
    oracle.forward(xs, w.eps, w.dim, s=ss, rho_in=rho, want=("blur", "grad"))
    dx1, ds, drho = oracle.backward(xs, w.eps, w.dim, s=ss, rho_in=rho, g_blur=u["g_blur"], g_grad=u["g_grad"])
    g_total = (u["g_rho"].astype(np.float64) + drho).astype(np.float32)
    oracle.backward(xs, w.eps, w.dim, g_rho=g_total)
    return time.perf_counter() - t0


REF_ROOT = ROOT / "baseline" / "_ref"


def cpu_baseline(w, x, s, ups, repeats=3):
    import oracle

    oracle.set_threads(os.cpu_count() or 1)
    systems = 1
    cpu_oracle_step(w, x, s, ups, systems)  # warm-up (page-in, thread pool)
    times = [cpu_oracle_step(w, x, s, ups, systems) for _ in range(repeats)]
    t = statistics.median(times)
    return {"value": systems * w.N / t, "unit": UNIT, "cores": oracle.num_threads(), "kind": "port",
            "sample": f"{systems} of {w.B} systems ({systems * w.N} particles), forward+backward, "
                      f"median of {repeats} after 1 warm-up, {t:.3f} s per pass"}


def load_torch_sph():
    """The reference's pure-torch operators, imported unmodified from the copy under baseline/_ref
    (None when the copy is absent)."""
    path = REF_ROOT / "sphops" / "torch_sph.py"
    if not path.exists():
        return None
    import importlib.util
    spec = importlib.util.spec_from_file_location("reference_torch_sph", path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


def torch_sph_step(ts, w, x, s, ups):
    """Density, blur and gradient forward, then backward with the seeded upstream gradients, with the
    reference's brute-force torch operators on the CPU (the protocol of sphops/test.py:236-285).
    x [B, n, P], s [B, n, C] CPU tensors; returns seconds."""
    import torch

    box = [g * w.eps for g in w.grid_size[: w.dim]] if w.boundary == "periodic" else None
    per = w.boundary == "periodic"
    xr = x[..., : w.dim].clone().requires_grad_(True)
    sr = s.clone().requires_grad_(True)
    t0 = time.perf_counter()
    rho = ts.density(xr, w.eps, None, per, box)
    blur = ts.blur(xr, rho, sr, w.eps, None, per, box)
    grad = ts.gradient(xr, rho, sr, w.eps, None, per, box)
    torch.autograd.backward([rho.reshape(ups["g_rho"].shape), blur, grad], [ups["g_rho"], ups["g_blur"], ups["g_grad"]])
    return time.perf_counter() - t0


def sub_box_sample(w, x, s, ups, target):
    """About `target` particles of system 0 around its densest region, with their features and upstream
    gradients: a sample of the workload at its own density that the O(n^2) reference operators can hold."""
    import torch

    d = w.dim
    x0 = x[0, :, :d]
    centre = x0.median(dim=0).values
    dist = (x0 - centre).abs().max(dim=1).values          # Chebyshev distance: a cube around the centre
    idx = torch.argsort(dist)[:target]
    pick = lambda t: t[0:1, idx].contiguous()
    return pick(x), pick(s), {k: pick(v) for k, v in ups.items()}


def cpu_reference_cfg1(repeats=3):
    """The reference's own torch_sph.py on its CPU-runnable configuration (2D, 4,096 particles, C=16),
    in full: forward + backward, all host cores, median of `repeats` after one warm-up."""
    ts = load_torch_sph()
    if ts is None:
        return None
    import torch
    from npa_b200.workloads import CONFIGS, make_inputs

    w = CONFIGS["cfg1_2d_growing"]
    x, s, ups = make_inputs(w, seed=0)
    torch.set_num_threads(os.cpu_count() or 1)
    torch_sph_step(ts, w, x, s, ups)
    times = [torch_sph_step(ts, w, x, s, ups) for _ in range(repeats)]
    t = statistics.median(times)
    return {"value": w.B * w.N / t, "unit": UNIT, "cores": torch.get_num_threads(), "kind": "reference",
            "workload": w.name,
            "sample": f"sphops/torch_sph.py unmodified, whole configuration ({w.B * w.N} particles), density + blur + "
                      f"gradient forward and backward, median of {repeats} after 1 warm-up, {t:.3f} s per pass"}


def run_reference_arm(args, w):
    """--impl reference: the reference's CPU implementation of the path on the host cores.

    With a copy of the reference under baseline/_ref this is its own sphops/torch_sph.py (brute
    force, O(n^2) memory), timed per step on a sub-box sample of the workload that it can hold;
    otherwise the C port of the same operators (the oracle) on one system per step."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    from npa_b200.workloads import make_inputs

    x, s, ups = make_inputs(w, seed=0)
    ts = load_torch_sph()
    if ts is not None:
        import torch
        torch.set_num_threads(os.cpu_count() or 1)
        # size the sample so that warm-up + K timed steps take about 2.5 minutes: the cost of the brute-force
        # operators grows with n^2, calibrated on a 512-particle probe
        n0 = min(w.N, 512)
        probe = sub_box_sample(w, x, s, ups, n0)
        torch_sph_step(ts, w, *probe)
        t0 = torch_sph_step(ts, w, *probe)
        n = int(n0 * (150.0 / (t0 * (args.steps + 2))) ** 0.5)
        n = max(256, min(n, 2048, w.N))
        xs, ss, us = sub_box_sample(w, x, s, ups, n)
        step = lambda: torch_sph_step(ts, w, xs, ss, us)
        particles, cores, kind = n, torch.get_num_threads(), "reference"
        sample = (f"each step = sphops/torch_sph.py (unmodified, float32) on the {n} particles of system 0 nearest "
                  "its centre (same density as the workload), density + blur + gradient forward and backward")
        dtype = "f32"
    else:
        import oracle
        oracle.set_threads(os.cpu_count() or 1)  # torchrun exports OMP_NUM_THREADS=1; use every host core
        step = lambda: cpu_oracle_step(w, x, s, ups, 1)
        particles, cores, kind = w.N, oracle.num_threads(), "port"
        sample = (f"each step = 1 of {w.B} systems ({w.N} particles), forward+backward with the C port of the "
                  "reference's operators (OpenMP over particles, double accumulation)")
        dtype = "f64"
    for _ in range(max(1, min(args.warmup, 2))):
        step()
    times = [step() for _ in range(args.steps)]
    total = sum(times)
    value = particles * args.steps / total
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": dtype,
        "data": "synthetic", "config": workload_config(w),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": kind, "sample": sample},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# ----------------------------------------------------------------------------------------------
# GPU arm
# ----------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.rows = []
        self.proc = None
        self.index = index

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "50",
                 "-i", str(self.index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        self.thread = threading.Thread(target=self._read, daemon=True)
        self.thread.start()

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) < 7:
                continue
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except ValueError:
                continue
            for name, flag in zip(names, r[3:7]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def bytes_per_particle(w):
    """Algorithmic (compulsory) bytes per particle of each stage: every input read once, every
    output written once, neighbour re-reads assumed to hit on-chip memory."""
    P, C, D = w.P, w.C, w.dim
    return {
        "grid_build": 4 * P + 4,                                   # read x, write permutation
        "reorder": 8 * (P + C) + 4,                                # read x, s, perm; write x_bin, s_bin
        "density_sweep": 4 * P + 4,                                # read x; write rho
        "blur_gradient_sweep": 4 * (P + 1 + C) + 4 * (C + C * D),  # read x, rho, s; write blur, grad
        "blur_gradient_backward": 4 * (P + 1 + C + C + C * D) + 4 * (P + C + 1),
        "density_backward": 4 * (P + 2 + P) + 4 * P,               # read x, 2 rho upstreams, grad_x; write grad_x
    }


def backward_flops_per_pair(w):
    """fp32 operations the fused blur+gradient backward spends on one accepted pair (a multiply-add
    counts 2): per feature 3 multiply-adds of the blur terms and, per axis, 5 of the gradient terms
    (h = v_j gG_i + v_i gG_j, K.h, df h, gG_j.K) plus 3 adds; per pair ~60 for the kernel scalars
    (r^2, poly6 and spiky factors, v_j = m_j / rho_j) and the position terms."""
    C, D = w.C, w.dim
    return C * (2 * 3 + 2 * 5 * D + 3) + 60


def fp32_roofline(w, accepted_pairs, launch_ms, clocks):
    sm_mhz = (clocks or {}).get("sm_max_mhz") or 1965.0
    peak = 148 * 128 * 2 * sm_mhz * 1e6 / 1e12
    achieved = accepted_pairs * backward_flops_per_pair(w) / (launch_ms * 1e-3) / 1e12
    return {"bound": "fp32", "kernel": "feature_backward_kernel", "achieved": achieved, "peak": peak,
            "unit": "TFLOP/s", "frac": achieved / peak, "accepted_pairs": accepted_pairs,
            "flops_per_pair": backward_flops_per_pair(w)}


HEADLINE_NAME = "cfg4_3d_splat"


def _max_over_ranks(ms, world, dev):
    import torch
    import torch.distributed as dist

    t = torch.tensor([ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def strong_scaling(rank, world, dev):
    """Fixed total work, systems sharded over the ranks (no collective on the data path):

    * the many-small-systems configuration (256 systems of 512 particles): one forward + backward step;
    * the scale-out rollout (64 periodic systems of 262,144 particles, C=16): 64 steps of re-bin ->
      perception forward -> move by a seeded smooth velocity field with periodic wrap, backward through
      the final step (npa_b200.rollout).
    Times are CUDA-event times, max over ranks, barrier-aligned."""
    import torch
    import torch.distributed as dist

    from npa_b200 import sphops as sph
    from npa_b200.rollout import PerceptionRollout, VelocityField
    from npa_b200.sharding import shard_range
    from npa_b200.workloads import CONFIGS, make_inputs, scaled

    out = {}

    def timed(fn, reps):
        fn()
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(reps):
            fn()
        e1.record()
        torch.cuda.synchronize()
        return _max_over_ranks(e0.elapsed_time(e1) / reps, world, dev)

    # ---- many small systems: one step -----------------------------------------------------
    w3 = CONFIGS["cfg3_2d_pointmnist_strokes"]
    lo, hi = shard_range(w3.B, rank, world)
    ws = scaled(w3, B=hi - lo)
    x, s, ups = make_inputs(w3, seed=3)
    x, s = x[lo:hi].contiguous().to(dev), s[lo:hi].contiguous().to(dev)
    ups = {k: v[lo:hi].contiguous().to(dev) for k, v in ups.items()}
    grid = sph.HashGrid(dim=ws.dim, boundary=ws.boundary, mode=ws.mode, grid_size=ws.grid_size, eps=ws.eps,
                        num_particles=ws.N, batch_size=ws.B, max_particles_per_block=ws.max_particles_per_block)
    roll = PerceptionRollout(grid, ws.C, steps=1, dt=0.0, velocity=VelocityField(ws.dim, dev))
    ms_eager = timed(lambda: roll.run(x, s, ups), 20)
    # the step is a chain of 13 small dependent launches: recorded once in a CUDA graph and replayed
    ms = ms_eager
    mode = "eager"
    try:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            roll.run(x, s, ups)
        ms = timed(graph.replay, 20)
        mode = "cuda graph replay"
        del graph
    except Exception as exc:  # capture not possible on this stack: keep the eager time
        print(f"[bench] cfg3 step not captured: {exc}", file=sys.stderr)
    out["cfg3_2d_pointmnist_strokes"] = {"systems_total": w3.B, "systems_per_rank": hi - lo, "ms_per_step": ms,
                                         "ms_per_step_eager": ms_eager, "launch": mode,
                                         "particles_per_s": w3.B * w3.N / (ms * 1e-3)}
    del roll, grid, x, s, ups

    # ---- scale-out rollout ------------------------------------------------------------------
    w5 = CONFIGS["cfg5_3d_rollout"]
    lo, hi = shard_range(w5.B, rank, world)
    ws = scaled(w5, B=hi - lo)
    steps, dt = int(w5.extra["steps"]), float(w5.extra["dt"])
    from npa_b200.workloads import make_positions
    x0 = make_positions(ws, seed=500 + rank).to(dev)   # every rank draws its own shard of the 64 systems
    gen = torch.Generator(device=dev).manual_seed(900 + rank)
    s0 = torch.randn(ws.B, ws.N, ws.C, generator=gen, device=dev)
    ups = {"g_rho": torch.randn(ws.B, ws.N, generator=gen, device=dev),
           "g_blur": torch.randn(ws.B, ws.N, ws.C, generator=gen, device=dev),
           "g_grad": torch.randn(ws.B, ws.N, ws.C, ws.dim, generator=gen, device=dev)}
    grid = sph.HashGrid(dim=ws.dim, boundary=ws.boundary, mode=ws.mode, grid_size=ws.grid_size, eps=ws.eps,
                        num_particles=ws.N, batch_size=ws.B, max_particles_per_block=ws.max_particles_per_block)
    # the velocity field gathers the particles into clumps over the 64 steps (at the end three particles in four have
    # more than 63 neighbours, one in four more than 255, one in seventeen more than 383): long lists keep them out of
    # the cell search (-23 % per rollout against 63 slots)
    roll = PerceptionRollout(grid, ws.C, steps=steps, dt=dt, velocity=VelocityField(ws.dim, dev, seed=5), list_slots=384)
    x, s = x0.clone(), s0.clone()

    def rollout():
        x.copy_(x0)
        s.copy_(s0)
        roll.run(x, s, ups)

    ms = timed(rollout, 1)
    out["cfg5_3d_rollout"] = {"systems_total": w5.B, "systems_per_rank": hi - lo, "steps": steps,
                              "ms_per_rollout": ms, "particle_steps_per_s": w5.B * w5.N * steps / (ms * 1e-3),
                              "gpu_launches_per_rollout": roll.launches}
    del roll, grid, x, s, x0, s0, ups
    torch.cuda.empty_cache()
    return out


def gpu_reference(w, x_d, s_d, ups, dev, our_step_ms):
    """The reference's own CUDA kernels (sphops/sph_cuda.cu compiled for this GPU by baseline/gpu_ref)
    on the same inputs: initialize, bin_particles, density / blur / gradient forward, blur / gradient /
    density backward (eight launches groups per step, its per-operator API has no fused call)."""
    try:
        from baseline.gpu_ref import refgrid
    except Exception:
        return None
    if not refgrid.available():
        return None
    import torch

    B, N, C, D = w.B, w.N, w.C, w.dim
    i32 = dict(dtype=torch.int32, device=dev)
    f32 = dict(dtype=torch.float32, device=dev)
    g = refgrid.ReferenceGrid(D, w.boundary, w.grid_size, w.eps, N, B, w.max_particles_per_block)
    cells = 1
    for n in w.grid_size[:D]:
        cells *= n
    perm, offs = torch.empty(B, N, **i32), torch.empty(B * cells + 1, **i32)
    info = torch.empty(g.max_blocks, 4, **i32)
    mass = torch.ones(B, N, **f32)
    xb, sb, mb = torch.empty_like(x_d), torch.empty_like(s_d), torch.empty_like(mass)
    rho, blur, grad = torch.empty(B, N, **f32), torch.empty(B, N, C, **f32), torch.empty(B, N, C, D, **f32)
    gx, gs, gr = torch.empty_like(x_d), torch.empty_like(s_d), torch.empty(B, N, **f32)
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)

    def step():
        g.initialize(x_d, perm, offs, info)
        g.bin_particles(x_d, s_d, mass, perm, xb, sb, mb)
        g.density_forward(xb, mb, rho, offs, info)
        g.blur_forward(xb, rho, mb, sb, blur, offs, info)
        g.gradient_forward(xb, rho, mb, sb, grad, offs, info)
        g.blur_backward(xb, rho, mb, sb, ups["g_blur"], gx, gs, gr, offs, info)
        g.gradient_backward(xb, rho, mb, sb, ups["g_grad"], gx, gs, gr, offs, info)
        g.density_backward(xb, mb, ups["g_rho"], gx, offs, info)

    # the reference launches on the legacy default stream, which synchronises with torch's streams
    torch.cuda.synchronize()
    for _ in range(3):
        step()
    torch.cuda.synchronize()
    times = []
    for _ in range(10):
        flush.zero_()
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        step()
        e1.record()
        torch.cuda.synchronize()
        times.append(e0.elapsed_time(e1))
    ms = statistics.median(times)
    return {"what": "sphops/sph_cuda.cu of the reference, unmodified, nvcc -O3 --use_fast_math for sm_100a, float32",
            "ms_per_step": ms, "value": B * N / (ms * 1e-3), "unit": UNIT,
            "ratio_this_over_reference": ms / our_step_ms,
            "note": "per-operator calls as the reference's sph.py makes them (no fused sweep exists there); median of 10"}


def run_gpu_arm(args, w):
    import torch
    import torch.distributed as dist

    from npa_b200 import sphops as sph
    from npa_b200.workloads import make_inputs

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise RuntimeError("bench.py needs a CUDA device: the npa_b200 kernels have no CPU fallback")
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    from npa_b200 import _native
    for backward, spec in ((False, args.tile_forward), (True, args.tile_backward)):
        if spec:
            _native.tile_tuning(backward, True, *[int(v) for v in spec.split(",")])
    if world > 1:
        from npa_b200.sharding import bind_to_gpu_cpus
        bound = bind_to_gpu_cpus(local_rank)  # pinned buffers below land on the GPU's NUMA node
        print(f"[bench] rank {rank}: bound to {len(bound) if bound else 'no'} cores near GPU {local_rank}", file=sys.stderr)
        dist.init_process_group("nccl", device_id=dev)

    # every rank owns its own B independent systems (batch sharded over ranks, weak scaling)
    x_h, s_h, ups_h = make_inputs(w, seed=rank)
    x_h, s_h = x_h.pin_memory(), s_h.pin_memory()
    x_d, s_d = x_h.to(dev), s_h.to(dev)
    ups = {k: v.to(dev) for k, v in ups_h.items()}
    B, N, C, D, P = w.B, w.N, w.C, w.dim, w.P

    grid = sph.HashGrid(dim=D, boundary=w.boundary, mode=w.mode, grid_size=w.grid_size, eps=w.eps,
                        num_particles=N, batch_size=B, max_particles_per_block=w.max_particles_per_block)
    hg = grid.hashgrid
    i32 = dict(dtype=torch.int32, device=dev)
    f32 = dict(dtype=torch.float32, device=dev)
    perm = torch.empty(B, N, **i32)
    offs = torch.empty(B * grid.num_cells + 1, **i32)
    info = torch.empty(hg.max_blocks, 4, **i32)
    x_bin, s_bin = torch.empty_like(x_d), torch.empty_like(s_d)
    rho = torch.empty(B, N, **f32)
    blur = torch.empty(B, N, C, **f32)
    grad = torch.empty(B, N, C, D, **f32)
    grad_x, grad_s, grad_rho = torch.empty_like(x_d), torch.empty_like(s_d), torch.empty(B, N, **f32)
    # neighbour lists: written by the density sweep, read by the other three.  127 slots: with 63, one particle in 600
    # of this workload overflows, and in the density backward (eight particles per warp pass) every pass that holds
    # such a particle walks the cells for all of its lanes: 108 -> 82 us
    pairs = torch.empty(B, N, 128, **i32)
    mlp_grad = torch.zeros(MLP_GRAD_FLOATS, **f32)
    comm = torch.cuda.Stream(dev) if world > 1 else None      # the gradient all-reduce runs beside the sweeps
    step_done = torch.cuda.Event()
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)  # > 126 MB of L2
    phases = ["grid_build", "reorder", "density_sweep", "blur_gradient_sweep", "blur_gradient_backward",
              "density_backward"]
    launches_per_step = 7 + 1 + 1 + 1 + 1 + 1  # grid build (7 kernels), reorder, four sweeps

    def step(ev=None):
        mark = (lambda k: ev[k].record()) if ev is not None else (lambda k: None)
        mark(0)
        hg.initialize(x_d, perm, offs, info)
        mark(1)
        hg.bin_particles(x_d, s_d, None, perm, x_bin, s_bin, None)
        mark(2)
        hg.perception_forward(x_bin, None, None, rho, None, None, None, None, None, offs, info, pair_cache=pairs)
        mark(3)
        hg.blur_gradient_forward(x_bin, rho, None, s_bin, blur, grad, offs, info, pair_cache=pairs,
                                 pair_cache_valid=True)
        mark(4)
        hg.blur_gradient_backward(x_bin, rho, None, s_bin, ups["g_blur"], ups["g_grad"], grad_x, grad_s,
                                  grad_rho, offs, info, pair_cache=pairs)
        mark(5)
        hg.density_chain_backward(x_bin, None, ups["g_rho"], grad_rho, None, grad_x, True, offs, info, pair_cache=pairs)
        mark(6)
        if world > 1:
            # the only exchange of data-parallel training: the MLP gradients, reduced on a side stream once this
            # step's backward is done; the next step's sweeps do not depend on it (the optimizer step does)
            step_done.record()
            comm.wait_event(step_done)
            with torch.cuda.stream(comm):
                dist.all_reduce(mlp_grad)

    sampler = ClockSampler(torch.cuda.current_device() if "CUDA_VISIBLE_DEVICES" not in os.environ
                           else os.environ["CUDA_VISIBLE_DEVICES"].split(",")[local_rank])
    if rank == 0:
        sampler.start()  # nvidia-smi needs a moment to start: launched before the warm-up steps
    for _ in range(max(args.warmup, 3)):
        flush.zero_()
        step()
    torch.cuda.synchronize()

    events = [[torch.cuda.Event(enable_timing=True) for _ in range(7)] for _ in range(args.steps)]
    if world > 1:
        dist.barrier()
    torch.cuda.synchronize()
    t_begin, t_end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t_begin.record()
    for k in range(args.steps):
        flush.zero_()  # L2 flush between timed steps, outside the per-step event pair
        step(events[k])
    if world > 1:
        torch.cuda.current_stream().wait_stream(comm)  # the timed region ends when the last all-reduce has
    t_end.record()
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    clocks = sampler.stop() if rank == 0 else None

    phase_ms = {p: sum(e[i].elapsed_time(e[i + 1]) for e in events) / args.steps for i, p in enumerate(phases)}
    # accepted pairs (r < h, self pair included) of this rank's systems, for the arithmetic model below
    cnt = torch.empty(B, N, **f32)
    hg.count_forward(x_bin, cnt, offs, info)
    accepted_pairs = float(cnt.sum(dtype=torch.float64).item())
    step_ms_local = sum(e[0].elapsed_time(e[6]) for e in events) / args.steps
    if world > 1:
        # whole timed region (flushes included) minus the flushes, so that an all-reduce that did not hide
        # behind the next step shows up; never less than the sum of the per-step event pairs
        flush_ms = sum(events[k][6].elapsed_time(events[k + 1][0]) for k in range(args.steps - 1)) if args.steps > 1 else 0.0
        first_flush = t_begin.elapsed_time(events[0][0])
        region = (t_begin.elapsed_time(t_end) - flush_ms - first_flush) / args.steps
        step_ms_local = max(step_ms_local, region)
    t = torch.tensor([step_ms_local], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    step_ms = float(t.item())
    value = world * B * N / (step_ms * 1e-3)

    # ---- end to end through the public API from pinned host buffers --------------------------
    # Every step copies positions and features host -> device, runs binning + forward + backward
    # through the public sphops API and copies both gradients device -> host.  The three stages of
    # consecutive steps overlap on three streams (npa_b200.pipeline), as a host-fed loop would run.
    from npa_b200.pipeline import HostStepPipeline

    def api_step(inp):
        xi, si = inp[0].detach().requires_grad_(True), inp[1].detach().requires_grad_(True)
        snap = grid.instantiate(xi.detach())
        xb, sb = sph.bin_particles(xi, si, snap)
        r, bl, gr = sph.perceive(xb, sb, snap, with_density_gradient=False)
        torch.autograd.backward([r, bl, gr], [ups["g_rho"], ups["g_blur"], ups["g_grad"]])
        if world > 1:
            dist.all_reduce(mlp_grad)
        return xi.grad, si.grad

    pipe = HostStepPipeline(api_step, (x_h, s_h), (x_h, s_h), device=dev, depth=2)
    pipe.run([(x_h, s_h)] * 3)
    torch.cuda.synchronize()
    if world > 1:
        dist.barrier()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    pipe.run([(x_h, s_h)] * args.steps)   # returns once the last gradients are in host memory
    e1.record()
    torch.cuda.synchronize()
    t = torch.tensor([e0.elapsed_time(e1) / args.steps], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    e2e_ms = float(t.item())
    h2d = x_h.numel() * 4 + s_h.numel() * 4
    d2h = h2d

    extras = {}
    if not args.no_extras and w.name == HEADLINE_NAME:
        del pipe
        torch.cuda.empty_cache()
        extras["strong_scaling"] = strong_scaling(rank, world, dev)
        if rank == 0 and world == 1:
            cmp_line = gpu_reference(w, x_d, s_d, ups, dev, step_ms)
            if cmp_line is not None:
                extras["gpu_reference"] = cmp_line

    if rank == 0:
        peak, peak_kind = measured_peak_gbs()
        bpp = bytes_per_particle(w)
        dom = "blur_gradient_backward"
        achieved = B * N * bpp[dom] / (phase_ms[dom] * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": step_ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_config(w),
            "tile_engine": {"forward": args.tile_forward, "backward": args.tile_backward},
            "parallelism": f"{world} x independent batches of {B} systems (weak scaling)",
            "phase_ms": phase_ms,
            "binning_mpoints_per_s": B * N / ((phase_ms["grid_build"] + phase_ms["reorder"]) * 1e-3) / 1e6,
            "roofline": {"bound": "hbm", "kernel": "feature_backward_kernel (blur+gradient backward)",
                         "achieved": achieved, "peak": peak, "peak_kind": peak_kind, "unit": "GB/s",
                         "frac": achieved / peak, "traffic": TRAFFIC_BYTES_PER_LAUNCH.get(w.name),
                         "algorithmic_bytes_per_launch": B * N * bpp[dom], "launch_ms": phase_ms[dom]},
            # secondary ceiling: fp32 multiply-adds of the dominant kernel against the FMA pipes
            # (148 SMs x 128 lanes x 2 flop x max SM clock); the count of operations per accepted
            # pair is the kernel's own arithmetic (see backward_flops_per_pair)
            "fp32_roofline": fp32_roofline(w, accepted_pairs, phase_ms[dom], clocks),
            "step_roofline": {"algorithmic_bytes_per_particle": sum(bpp.values()),
                              "achieved": B * N * sum(bpp.values()) / (step_ms_local * 1e-3) / 1e9,
                              "frac": B * N * sum(bpp.values()) / (step_ms_local * 1e-3) / 1e9 / peak},
            "e2e": {"value": world * B * N / (e2e_ms * 1e-3), "unit": UNIT, "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    # what the host side of this machine delivers to all ranks together
                    "host_gb_per_s_all_ranks": world * (h2d + d2h) / (e2e_ms * 1e-3) / 1e9},
            "gpu_launches": launches_per_step * args.steps,
            "clocks": clocks,
        }
        if extras:
            line.update(extras)
        if not args.no_cpu_baseline and world == 1:
            line["cpu_baseline"] = cpu_baseline(w, x_h, s_h, ups_h)
            ref = cpu_reference_cfg1()
            if ref is not None:
                line["cpu_baseline_reference"] = ref
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the dominant kernel, from an ncu capture of a
# full launch of the same workload (profiles/ncu_feature_kernels_cfg4_3d_splat.md); other workloads: not captured.
TRAFFIC_BYTES_PER_LAUNCH = {"cfg4_3d_splat": 273.1e6}


def main():
    args = parse_args()
    from npa_b200.workloads import CONFIGS, HEADLINE

    w = CONFIGS[args.workload or HEADLINE]
    if args.impl == "reference":
        run_reference_arm(args, w)
    else:
        run_gpu_arm(args, w)


if __name__ == "__main__":
    main()
