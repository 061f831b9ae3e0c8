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
  bounded sample of the same workload.  ``--impl reference`` prints that arm as its own line.

For N > 1 (torchrun) every rank runs the full workload on its own GPU (independent systems
sharded over ranks, weak scaling) plus one NCCL all-reduce of an MLP-gradient-sized buffer per
step; time is the max over ranks.
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
    return ap.parse_args()


def measured_peak_gbs():
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


def workload_config(w, extra=None):
    cfg = {"workload": w.name, "dim": w.dim, "systems": w.B, "particles_per_system": w.N, "features": w.C,
           "eps": w.eps, "grid": list(w.grid_size), "boundary": w.boundary,
           "max_particles_per_block": w.max_particles_per_block}
    if extra:
        cfg.update(extra)
    return cfg


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


def cpu_baseline(w, x, s, ups, repeats=1):
    import oracle

    oracle.set_threads(os.cpu_count() or 1)
    systems = 1
    cpu_oracle_step(w, x, s, ups, systems)  # warm-up (page-in, thread pool)
    times = [cpu_oracle_step(w, x, s, ups, systems) for _ in range(repeats)]
    t = statistics.median(times)
    return {"value": systems * w.N / t, "unit": UNIT, "cores": oracle.num_threads(), "kind": "port",
            "sample": f"{systems} of {w.B} systems ({systems * w.N} particles), forward+backward, "
                      f"median of {repeats} after 1 warm-up, {t:.3f} s per pass"}


def run_reference_arm(args, w):
    """--impl reference: the CPU port of the reference's operators, timed step by step."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    import oracle
    from npa_b200.workloads import make_inputs

    oracle.set_threads(os.cpu_count() or 1)  # torchrun exports OMP_NUM_THREADS=1; use every host core
    x, s, ups = make_inputs(w, seed=0)
    systems = 1
    for _ in range(max(1, min(args.warmup, 2))):
        cpu_oracle_step(w, x, s, ups, systems)
    times = [cpu_oracle_step(w, x, s, ups, systems) for _ in range(args.steps)]
    total = sum(times)
    value = systems * w.N * args.steps / total
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": 1e3 * total / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f64",
        "data": "synthetic", "config": workload_config(w, {"sample": f"{systems} system per step"}),
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": oracle.num_threads(), "kind": "port",
                         "sample": f"each step = {systems} of {w.B} systems ({systems * w.N} particles), "
                                   "forward+backward with the C oracle (OpenMP over particles)"},
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
    pairs = torch.empty(B, N, 64, **i32)  # neighbour lists: written by the density sweep, read by the other three
    mlp_grad = torch.zeros(MLP_GRAD_FLOATS, **f32)
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
        if world > 1:
            dist.all_reduce(mlp_grad)  # the only exchange of data-parallel training: the MLP gradients
        mark(6)

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
    for k in range(args.steps):
        flush.zero_()  # L2 flush between timed steps, outside the per-step event pair
        step(events[k])
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

    if rank == 0:
        peak, peak_kind = measured_peak_gbs()
        bpp = bytes_per_particle(w)
        dom = "blur_gradient_backward"
        achieved = B * N * bpp[dom] / (phase_ms[dom] * 1e-3) / 1e9
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": max(args.warmup, 3), "ms_per_step": step_ms, "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": workload_config(w, {"l2": "256 MB buffer written between timed steps (L2 flush)",
                                          "parallelism": f"{world} x independent batches of {B} systems",
                                          "upstream_gradients": "N(0,1), device resident"}),
            "phase_ms": phase_ms,
            "binning_mpoints_per_s": B * N / ((phase_ms["grid_build"] + phase_ms["reorder"]) * 1e-3) / 1e6,
            "roofline": {"bound": "hbm", "kernel": "feature_backward_kernel (blur+gradient backward)",
                         "achieved": achieved, "peak": peak, "peak_kind": peak_kind, "unit": "GB/s",
                         "frac": achieved / peak, "traffic": TRAFFIC_BYTES_PER_LAUNCH,
                         "algorithmic_bytes_per_launch": B * N * bpp[dom], "launch_ms": phase_ms[dom]},
            # secondary ceiling: fp32 multiply-adds of the dominant kernel against the FMA pipes
            # (148 SMs x 128 lanes x 2 flop x max SM clock); the count of operations per accepted
            # pair is the kernel's own arithmetic (see backward_flops_per_pair)
            "fp32_roofline": fp32_roofline(w, accepted_pairs, phase_ms[dom], clocks),
            "step_roofline": {"algorithmic_bytes_per_particle": sum(bpp.values()),
                              "achieved": B * N * sum(bpp.values()) / (step_ms_local * 1e-3) / 1e9,
                              "frac": B * N * sum(bpp.values()) / (step_ms_local * 1e-3) / 1e9 / peak},
            "e2e": {"value": world * B * N / (e2e_ms * 1e-3), "unit": UNIT, "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            "gpu_launches": launches_per_step * args.steps,
            "clocks": clocks,
        }
        if not args.no_cpu_baseline and world == 1:
            line["cpu_baseline"] = cpu_baseline(w, x_h, s_h, ups_h)
        print(json.dumps(line), flush=True)
    if world > 1:
        dist.destroy_process_group()


# dram__bytes_read.sum + dram__bytes_write.sum of one launch of the dominant kernel on the
# headline workload, from an ncu capture (profiles/); None until measured.
TRAFFIC_BYTES_PER_LAUNCH = 273.1e6  # profiles/ncu_feature_kernels_cfg4_3d_splat.md, same workload, full launch


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
