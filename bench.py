#!/usr/bin/env python
"""Benchmark of the TACE energy + force + stress path on B200.

One "step" = one evaluation of energy, conservative forces and stress for the whole batch of the
workload (the headline configuration: 64 random periodic crystals, fp32, L = 3, 128 channels, 89 elements).
With N GPUs a pool of 64 N crystals is split over the ranks with the longest-processing-time rule on
estimated edge counts (``tace_b200.shard``); every rank evaluates its share with replicated weights (weak
scaling, no collective on the data path) and the per-structure energies and stresses are gathered with one
all_gather in the end-to-end loop.  `value` is timed with the batch and its neighbour list resident in HBM;
`e2e` goes through the public API from pinned host buffers (upload, GPU neighbour list, evaluation,
download of energy / forces / stress).  Unless --no-domain-md is given, the line also carries `domain_md`:
a short velocity-Verlet run of the 1 048 576-atom Cu-Al system of configuration 5, domain-decomposed
over the same N GPUs (strong scaling, halo exchange per interaction layer).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl native|reference] [--workload NAME]
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

ROOT = os.path.dirname(os.path.abspath(__file__))
for p in (ROOT, os.path.join(ROOT, "tests")):
    if p not in sys.path:
        sys.path.insert(0, p)

import numpy as np
import torch

METRIC = "atom-steps/s (E+F)"
UNIT = "atom-steps/s"


def peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as fh:
            d = json.load(fh)
        return {"hbm_gbs": d["hbm_gbs"], "bf16_tflops": d["bf16_tflops"], "source": "measured"}
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "source": "fallback"}


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
              "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.index, self.proc, self.lines = index, None, []

    def start(self):
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--id={self.index}", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "250"],
                stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.lines.append(line.strip())

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        self.thread.join(timeout=2)
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 6:
                continue
            try:
                sm.append(float(parts[0])); mx.append(float(parts[1]))
            except ValueError:
                continue
            for n, v in zip(names, parts[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def dist_setup(n_gpus: int):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        torch.cuda.set_device(local)
        # every rank reports the same CPU affinity on these hosts: give each its own slice of the cores so that the
        # host sides of the ranks (Python, pinned staging, launches) do not migrate onto each other
        try:
            cores = sorted(os.sched_getaffinity(0))
            per = max(1, len(cores) // world)
            mine = cores[local * per:(local + 1) * per] or cores
            os.sched_setaffinity(0, mine)
            torch.set_num_threads(max(1, min(len(mine), 8)))
        except (AttributeError, OSError):
            pass
        dist.init_process_group("nccl", device_id=torch.device("cuda", local))
    return rank, world, local


def barrier(world: int):
    if world > 1:
        import torch.distributed as dist
        dist.barrier()
    torch.cuda.synchronize()


def max_over_ranks(x: float, world: int, device) -> float:
    if world == 1:
        return x
    import torch.distributed as dist
    t = torch.tensor([x], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    return float(t.item())


def gather_floats(xs, world: int, device):
    """Every rank's list of floats, as a list of lists (rank-major)."""
    t = torch.tensor(xs, dtype=torch.float64, device=device)
    if world == 1:
        return [t.tolist()]
    import torch.distributed as dist
    out = [torch.zeros_like(t) for _ in range(world)]
    dist.all_gather(out, t)
    return [o.tolist() for o in out]


def sum_over_ranks(x: float, world: int, device) -> float:
    if world == 1:
        return x
    import torch.distributed as dist
    t = torch.tensor([x], dtype=torch.float64, device=device)
    dist.all_reduce(t, op=dist.ReduceOp.SUM)
    return float(t.item())


def build_model(wl: dict, dtype):
    import tace_b200
    from tace_b200 import synth
    cfg = synth.model_config(wl["L"], wl["channels"], wl["cutoff"], wl["elements"], wl["avg_num_neighbors"], **wl.get("model", {}))
    prev = torch.get_default_dtype()
    torch.set_default_dtype(dtype)
    try:
        torch.manual_seed(0)
        model = tace_b200.TensorModel(tace_b200.e3nnTACE(**cfg))
    finally:
        torch.set_default_dtype(prev)
    return model, cfg


def algorithmic_bytes(phase: str, dims: dict):
    """Bytes the phase's kernel must move if every per-edge tensor is recomputed on chip: one gather of
    the source features per edge, one pass over the per-atom messages (or their gradient), the edge list."""
    s, E, N, C = dims["s"], dims["E"], dims["N"], dims["C"]
    layer = int(phase[1]) if phase.startswith("t") and phase[1].isdigit() else 0
    NX = 1 if layer == 0 else dims["D"]
    NM = dims["NM"][layer]
    if ".tp" in phase:
        return s * (E * NX * C + N * NM * C) + 4 * E
    return None


def gemm_flops(phase: str, dims: dict):
    layer = int(phase[1])
    return 2.0 * dims["E"] * 64 * dims["NP"][layer] * dims["C"]


def cpu_sample_structures(structures, wl):
    """The fixed sample both CPU legs time: for a batch of crystals, the four crystals at the octile midpoints of the
    size-sorted batch (12.5 %, 37.5 %, 62.5 %, 87.5 %; about 140 atoms for configuration 2), chosen by index; for a
    single large structure, a smaller cell of the same material named by the workload."""
    from tace_b200 import synth
    if wl.get("cpu_sample"):
        return synth.workload_structures(wl["cpu_sample"]), f"a smaller cell of the same material ({wl['cpu_sample']})"
    if len(structures) < 8:
        return list(structures), "the whole workload"
    order = sorted(range(len(structures)), key=lambda i: (len(structures[i]["positions"]), i))
    picks = sorted(order[int(q * len(order))] for q in (0.125, 0.375, 0.625, 0.875))
    return [structures[i] for i in picks], f"crystals {picks} of the batch (size octile midpoints)"


def cpu_sample(structures, wl, dtype, state_dict):
    """The CPU oracle (PyTorch, autograd forces, all host threads) on the fixed sample."""
    from helpers import oracle_batch
    from oracle.model import build_oracle
    from tace_b200 import synth
    cores = len(os.sched_getaffinity(0)) if hasattr(os, "sched_getaffinity") else (os.cpu_count() or 1)
    torch.set_num_threads(cores)
    cfg = synth.model_config(wl["L"], wl["channels"], wl["cutoff"], wl["elements"], wl["avg_num_neighbors"], **wl.get("model", {}))
    oracle = build_oracle(cfg, state_dict, dtype)
    chosen, what = cpu_sample_structures(structures, wl)
    data = oracle_batch(chosen, wl["elements"], wl["cutoff"], dtype)
    n_atoms = data["positions"].shape[0]
    sample = f"{what}: {len(chosen)} structure(s), {n_atoms} atoms, {data['edge_index'].shape[1]} edges"
    return oracle, data, n_atoms, sample, cores, chosen


def run_reference(args, rank, world):
    """--impl reference: the CPU restatement of the reference path (the reference itself needs e3nn /
    matscipy / ase, which cannot be installed offline), all host threads, the same fixed sample per step as the
    `cpu_baseline` leg of the native arm."""
    if rank != 0:
        return
    from tace_b200 import synth
    wl = synth.WORKLOADS[args.workload]
    dtype = torch.float64 if wl["dtype"] == "float64" else torch.float32
    structures = synth.workload_structures(args.workload)
    model, cfg = build_model(wl, dtype)
    oracle, data, n_atoms, sample, cores, _ = cpu_sample(structures, wl, dtype, model.state_dict())
    for _ in range(args.warmup):
        oracle(data)
    times = []
    for _ in range(args.steps):
        t0 = time.perf_counter()
        oracle(data)
        times.append(time.perf_counter() - t0)
    dt = sum(times)
    value = n_atoms * args.steps / dt
    plan = model.readout_fn.plan
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": 1e3 * dt / args.steps, "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32" if dtype == torch.float32 else "f64", "data": "synthetic",
        "config": {"workload": args.workload, "L": plan.L, "channels": plan.C, "cutoff": wl["cutoff"],
                   "elements": len(wl["elements"]), "parallelism": f"cpu, {cores} threads", "sample": sample + " per step"},
        "step_ms": {"min": 1e3 * min(times), "median": 1e3 * statistics.median(times), "max": 1e3 * max(times)},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": cores, "kind": "port", "sample": sample + " per step"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }))


def md_measure(workload, wl, dtype, rank, world, device, steps, warmup):
    """Molecular-dynamics workloads: ONE periodic Cu/Al system, velocity Verlet, dt = 1 fs,
    Maxwell-Boltzmann start at 300 K.  A step = half kick + drift, ghost positions, neighbour list (reused while no
    atom has moved more than half the 1.0 A skin), energy and forces with halo exchanges between layers, ghost forces
    returned, half kick.  With N GPUs the box is cut into N blocks (strong scaling: the system is the same at every
    N).  Collective: every rank calls it; rank 0 gets the result dictionary, the others None."""
    from tace_b200 import synth
    from tace_b200.md import DomainMD, masses_for, maxwell_boltzmann
    s = synth.workload_structures(workload)[0]
    model, cfg = build_model(wl, dtype)
    masses = masses_for(s["atomic_numbers"])
    vel = maxwell_boltzmann(masses, 300.0, seed=5)
    n_atoms = len(masses)
    t_setup = time.perf_counter()
    md = DomainMD(model.to(device), s["cell"], s["positions"], s["atomic_numbers"], velocities=vel, masses=masses, dt=1.0, skin=1.0,
                  rank=rank, world_size=world, device=device)
    torch.cuda.synchronize()
    t_setup = time.perf_counter() - t_setup
    e_start = md.potential() + md.kinetic_energy()
    md.step(warmup)
    torch.cuda.synchronize()
    launches0 = model.launch_count()
    md.timings.clear()
    md.domain.set_time_exchanges(True)
    md.domain.halo_stats(reset=True)
    rebuilds0 = getattr(md, "n_list_builds", 0)
    sampler = ClockSampler(device.index or 0)
    if rank == 0:
        sampler.start()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier(world)
    t0 = time.perf_counter()
    start.record()
    md.step(steps)
    stop.record()
    torch.cuda.synchronize()
    wall = max_over_ranks(time.perf_counter() - t0, world, device)
    barrier(world)
    total_ms = max_over_ranks(start.elapsed_time(stop), world, device)
    clocks = sampler.stop() if rank == 0 else None
    launches = model.launch_count() - launches0
    halo_ms, halo_bytes = md.domain.halo_stats()
    md.domain.set_time_exchanges(False)
    halo_ms = max_over_ranks(halo_ms, world, device)
    halo_bytes = sum_over_ranks(float(halo_bytes), world, device)
    e_end = md.potential() + md.kinetic_energy()
    temperature = md.temperature()
    host_split = {k: round(1e3 * v / steps, 3) for k, v in md.timings.items()}
    edges = sum_over_ranks(float(md.n_edges), world, device)
    ghosts = sum_over_ranks(float(md.domain.n_ghost), world, device)
    per_rank = gather_floats([float(md.domain.n_owned), float(md.domain.n_ghost), float(md.n_edges)], world, device)
    # per-phase device times of one more evaluation
    model.enable_profile(True)
    md._evaluate()
    phases = model.read_profile()
    model.enable_profile(False)
    result = None
    if rank == 0:
        pk = peaks()
        plan = model.readout_fn.plan
        L, C = plan.L, plan.C
        dims = {"s": 4 if dtype == torch.float32 else 8, "E": int(md.n_edges), "N": md.domain.n_owned + md.domain.n_ghost, "C": C,
                "D": (L + 1) ** 2, "NM": [sum((2 * l + 1) * lp.k[l] for l in range(L + 1)) for lp in plan.layers],
                "NP": [len(lp.tp_paths) for lp in plan.layers]}
        kernel_phases = {k: v for k, v in phases.items() if ".tp" in k}
        top = max(kernel_phases, key=kernel_phases.get)
        ab = algorithmic_bytes(top, dims)
        achieved = ab / (phases[top] * 1e-3) / 1e9
        roofline = {"bound": "hbm", "kernel": top, "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                    "frac": achieved / pk["hbm_gbs"], "traffic": None, "peak_source": pk["source"],
                    "algorithmic_bytes_per_launch": ab, "ms_per_launch": phases[top],
                    "note": "all chunk launches of the phase on rank 0 taken together"}
        value = n_atoms * steps / (total_ms * 1e-3)
        result = {
            "metric": "atom-steps/s (MD step)", "value": value, "unit": UNIT, "n_gpus": world, "steps": steps, "warmup": warmup,
            "ms_per_step": total_ms / steps, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
            "dtype": "f32" if dtype == torch.float32 else "f64", "data": "synthetic",
            "config": {"workload": workload, "L": L, "channels": C, "cutoff": wl["cutoff"], "elements": len(wl["elements"]),
                       "atoms": n_atoms, "edges": int(edges), "ghost_atoms": int(ghosts), "grid": list(md.domain.grid.grid),
                       "parallelism": f"spatial domain decomposition over {world} GPU(s), halo exchange per interaction layer",
                       "l2": "per-step working set (> 1 GB) exceeds L2", "partitions": md.domain.n_partitions,
                       "neighbour_list_builds": getattr(md, "n_list_builds", 0) - rebuilds0, "setup_s": round(t_setup, 2),
                       "radial_table": bool(model.uses_radial_table)},
            "e2e": {"value": n_atoms * steps / wall, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 8,
                    "note": "state lives on the device; wall clock of the same steps including host-side scheduling"},
            "gpu_launches": launches, "clocks": clocks, "roofline": roofline, "cpu_baseline": None,
            "md": {"energy_start_eV": e_start, "energy_end_eV": e_end, "temperature_K": temperature,
                   "host_ms_per_step": host_split, "exchange_ms_per_step": round(halo_ms / steps, 3),
                   "halo_bytes_per_step": int(halo_bytes / steps),
                   "ranks": [{"owned": int(r[0]), "ghosts": int(r[1]), "edges": int(r[2])} for r in per_rank]},
            "phases_ms": {k: round(v, 4) for k, v in sorted(phases.items(), key=lambda kv: -kv[1])},
        }
    model.release()
    del md, model
    torch.cuda.empty_cache()
    return result


def run_md(args, wl, dtype, rank, world, device):
    result = md_measure(args.workload, wl, dtype, rank, world, device, args.steps, args.warmup)
    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()
    if rank == 0:
        print(json.dumps(result))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None, help="timed steps (default: 300 native, 10 reference)")
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="native", choices=["native", "reference"])
    ap.add_argument("--workload", default="crystals64_fp32")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-domain-md", action="store_true", help="skip the domain-decomposed MD measurement added to the default line")
    ap.add_argument("--md-steps", type=int, default=5)
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.steps is None:  # a timed region of a second or two for the GPU arm; a few minutes at most for the CPU arm
        args.steps = 300 if args.impl == "native" else 10

    if args.impl == "reference":
        run_reference(args, int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1")))
        return

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: tace_b200 has no CPU path")
    rank, world, local = dist_setup(args.gpus)
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)

    from tace_b200 import shard, synth
    from tace_b200.graph import build_batch, z_to_index
    wl = synth.WORKLOADS[args.workload]
    dtype = torch.float64 if wl["dtype"] == "float64" else torch.float32
    if args.workload in synth.MD_WORKLOADS:
        run_md(args, wl, dtype, rank, world, device)
        return
    pool = None
    if args.workload == "crystals64_fp32":
        # one pool of 64 crystals per GPU (the first 64 are the single-GPU batch), split by estimated edge count
        pool = synth.random_crystals(64 * world, seed=1)
        parts = shard.partition_lpt([shard.estimate_edges(c, wl["cutoff"]) for c in pool], world)
        structures = [pool[i] for i in parts[rank]]
    else:
        structures = synth.workload_structures(args.workload)
    model, cfg = build_model(wl, dtype)
    host = synth.collate(structures)
    host["species"] = z_to_index(host["atomic_numbers"], wl["elements"])
    pinned = {k: torch.as_tensor(v).pin_memory() for k, v in host.items()}
    n_atoms = int(host["positions"].shape[0])

    data = build_batch(pinned, wl["elements"], wl["cutoff"], dtype, device)
    n_edges = int(data["edge_index"].shape[1])
    flush = torch.empty(256 << 20, dtype=torch.uint8, device=device)  # larger than the 126 MB L2

    for _ in range(args.warmup):
        out = model(data)
    torch.cuda.synchronize()
    launches0 = model.launch_count()

    sampler = ClockSampler(local)
    if rank == 0:
        sampler.start()
    starts = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    stops = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps)]
    barrier(world)
    # untimed device work ahead of the first start event, so the host gets a few steps ahead of the GPU and a
    # scheduling hiccup of the (shared) host does not leave the GPU idle inside a timed step
    for _ in range(200):
        flush.fill_(0)
    host_s = 0.0
    for k in range(args.steps):
        flush.fill_(k & 0xFF)  # evict L2 between timed steps (outside the per-step event pair)
        starts[k].record()
        t_host = time.perf_counter()
        out = model(data)
        host_s += time.perf_counter() - t_host
        stops[k].record()
    barrier(world)
    step_ms = [a.elapsed_time(b) for a, b in zip(starts, stops)]
    total_ms = max_over_ranks(sum(step_ms), world, device)
    per_rank = gather_floats([sum(step_ms) / args.steps, 1e3 * host_s / args.steps, float(n_atoms), float(n_edges),
                              min(step_ms), statistics.median(step_ms), max(step_ms)], world, device)
    clocks = sampler.stop() if rank == 0 else None
    launches = model.launch_count() - launches0
    total_atoms = sum_over_ranks(float(n_atoms), world, device)
    value = total_atoms * args.steps / (total_ms * 1e-3)

    # per-phase device times (separate, untimed passes with event recording switched on)
    model.enable_profile(True)
    phases = {}
    reps = 3
    for _ in range(reps):
        flush.fill_(1)
        model(data)
        for name, ms in model.read_profile().items():
            phases[name] = phases.get(name, 0.0) + ms / reps
    model.enable_profile(False)

    # end to end through the public API: pinned host buffers -> upload -> neighbour list -> evaluation -> download
    # The loop is software-pipelined the way a throughput-oriented caller would write it: upload + neighbour list of
    # step k+1 run on a second stream while step k is evaluated, and the host waits for the downloaded results of step
    # k only after it has enqueued step k+1 (two sets of pinned result buffers), so the GPU never waits for the host.
    # Every step still uploads its own inputs from pinned memory and downloads its own results inside the timed
    # region.  With several GPUs every step ends with one all_gather of the per-structure energies and stresses of all
    # ranks (shares padded to the largest share).
    e2e_split = {"upload_and_neighbour_list": 0.0, "evaluation_call": 0.0, "download_enqueue": 0.0, "gather": 0.0, "wait_previous": 0.0}
    # high priority: the neighbour-list kernels of step k+1 are short and the host waits for their edge count, so they
    # must not queue behind the long evaluation kernels of step k
    side = torch.cuda.Stream(device, priority=-1)
    n_graphs = len(structures)
    share_max = int(max_over_ranks(float(n_graphs), world, device))
    gather_in = torch.zeros(share_max, 10, dtype=dtype, device=device)
    gather_out = torch.zeros(world * share_max, 10, dtype=dtype, device=device)
    host_out = [{"energy": torch.empty(n_graphs, dtype=dtype).pin_memory(), "forces": torch.empty(n_atoms, 3, dtype=dtype).pin_memory(),
                 "stress": torch.empty(n_graphs, 3, 3, dtype=dtype).pin_memory()} for _ in range(2)]

    def prepare():
        t_a = time.perf_counter()
        with torch.cuda.stream(side):
            d = build_batch(pinned, wl["elements"], wl["cutoff"], dtype, device)
            ready = torch.cuda.Event()
            ready.record(side)
        e2e_split["upload_and_neighbour_list"] += time.perf_counter() - t_a
        return d, ready

    e2e_step_s = []

    def e2e_loop(n):
        nxt = prepare()
        pending = None  # (event, inputs, outputs) of the step whose results are still on their way to the host
        t_prev = time.perf_counter()
        for k in range(n):
            d, ready = nxt
            torch.cuda.current_stream(device).wait_event(ready)
            t_b = time.perf_counter()
            o = model(d)
            t_c = time.perf_counter()
            if world > 1:
                import torch.distributed as dist
                gather_in[:n_graphs, 0] = o["energy"]
                gather_in[:n_graphs, 1:] = o["stress"].reshape(n_graphs, 9)
                dist.all_gather_into_tensor(gather_out, gather_in)
            t_d = time.perf_counter()
            for key, buf in host_out[k % 2].items():  # one asynchronous copy per result into pinned memory
                buf.copy_(o[key], non_blocking=True)
            done = torch.cuda.Event()
            done.record()
            t_e = time.perf_counter()
            if k + 1 < n:
                nxt = prepare()  # overlaps the evaluation of step k
            t_f = time.perf_counter()
            if pending is not None:  # the results of step k-1 are in host memory after this
                pending[0].synchronize()
                e2e_step_s.append(time.perf_counter() - t_prev)
                t_prev = time.perf_counter()
            pending = (done, d, o)  # inputs and outputs stay referenced until their step has finished on the device
            e2e_split["evaluation_call"] += t_c - t_b
            e2e_split["gather"] += t_d - t_c
            e2e_split["download_enqueue"] += t_e - t_d
            e2e_split["wait_previous"] += time.perf_counter() - t_f
        pending[0].synchronize()
        e2e_step_s.append(time.perf_counter() - t_prev)
        return host_out[(n - 1) % 2]

    e2e_steps = min(args.steps, 100)
    e2e_loop(args.warmup)
    barrier(world)
    for key in e2e_split:
        e2e_split[key] = 0.0
    e2e_step_s.clear()
    t0 = time.perf_counter()
    res = e2e_loop(e2e_steps)
    torch.cuda.synchronize()
    e2e_s = max_over_ranks(time.perf_counter() - t0, world, device)
    barrier(world)
    h2d = sum(int(pinned[k].numel() * pinned[k].element_size()) for k in ("positions", "lattice", "pbc", "ptr", "species", "batch"))
    d2h = sum(int(t.numel() * t.element_size()) for t in res.values())
    e2e_value = total_atoms * e2e_steps / e2e_s

    # CPU leg on rank 0 (N = 1 only): the oracle on the fixed sample, timed, and compared with the GPU result for the
    # very same crystals (the sample's crystals evaluated by the GPU as a batch of their own)
    cpu = None
    if world == 1 and not args.no_cpu_baseline:
        oracle, cdata, c_atoms, sample, cores, chosen = cpu_sample(structures, wl, dtype, model.state_dict())
        ref = oracle(cdata)
        t0 = time.perf_counter()
        for _ in range(2):
            oracle(cdata)
        dt = (time.perf_counter() - t0) / 2
        gpu = model({k: v.to(device) for k, v in cdata.items()})
        n_per = (cdata["ptr"][1:] - cdata["ptr"][:-1]).to(torch.float64)
        cpu = {"value": c_atoms / dt, "unit": UNIT, "cores": cores, "kind": "port",
               "sample": sample + ", 2 timed evaluations of the PyTorch CPU restatement with autograd forces",
               "max_abs_dE_per_atom": float(((gpu["energy"].cpu().double() - ref["energy"].double()).abs() / n_per).max()),
               "max_abs_dF": float((gpu["forces"].cpu().double() - ref["forces"].double()).abs().max())}

    plan = model.readout_fn.plan
    L, C = plan.L, plan.C
    uses_table = bool(model.uses_radial_table)
    graph_replays = model.graph_replays()
    # the domain-decomposed MD measurement of configuration 5 on the same GPUs (strong scaling)
    domain_md = None
    if args.workload == "crystals64_fp32" and not args.no_domain_md:
        del out, data
        model.release()
        torch.cuda.empty_cache()
        md_wl = synth.WORKLOADS["cual1m_fp32"]
        domain_md = md_measure("cual1m_fp32", md_wl, torch.float32, rank, world, device, args.md_steps, 3)
        if domain_md is not None:
            for key in ("roofline", "cpu_baseline", "higher_is_better", "vs_baseline", "data", "unit"):
                domain_md.pop(key, None)

    if world > 1:
        import torch.distributed as dist
        dist.destroy_process_group()
    if rank != 0:
        return

    pk = peaks()
    dims = {"s": 4 if dtype == torch.float32 else 8, "E": n_edges, "N": n_atoms, "C": C, "D": (L + 1) ** 2,
            "NM": [sum((2 * l + 1) * lp.k[l] for l in range(L + 1)) for lp in plan.layers],
            "NP": [len(lp.tp_paths) for lp in plan.layers]}
    # the dominant kernel: tensor-product passes and the radial-MLP GEMMs are single-kernel phases
    kernel_phases = {k: v for k, v in phases.items() if ".tp" in k or "radial_gemm" in k}
    top = max(kernel_phases, key=kernel_phases.get)
    traffic = None
    tpath = os.path.join(ROOT, "profiles", "traffic.json")
    if os.path.exists(tpath):
        with open(tpath) as fh:
            traffic = json.load(fh).get(f"{args.workload}:{top}" + (":table" if uses_table else ""))
    ab = algorithmic_bytes(top, dims)
    layer = int(top[1]) if top[1].isdigit() else 0
    if ".tp" in top and layer in plan.tece_layers:
        # the TECE edge block is bound by its SO(2) linears: 2 * rows * K * N per order block and edge, the same count
        # again for the input gradients of the backward pass; fp32 models run them as three TF32 products each
        fl = 0.0
        for _ref, _name, ci, co, n_in, n_out in plan.so2_linears():
            fl += sum(2.0 * (1 if m == 0 else 2) * n_in[m] * ci * n_out[m] * co for m in range(len(n_in)))
        fl *= n_edges
        achieved = fl / (phases[top] * 1e-3) / 1e12
        roofline = {"bound": "tensor", "kernel": top + " (edge block: SO(2) GEMMs and their element-wise kernels)", "achieved": achieved,
                    "peak": pk["bf16_tflops"], "unit": "TFLOP/s", "frac": achieved / pk["bf16_tflops"], "traffic": None,
                    "peak_source": pk["source"], "flops_per_launch": fl, "ms_per_launch": phases[top],
                    "note": "useful FP32 FLOPs of the SO(2) linears over the whole phase; every one costs three TF32 tensor-core FLOPs"}
    elif ab is not None:
        achieved = ab / (phases[top] * 1e-3) / 1e9
        roofline = {"bound": "hbm", "kernel": top, "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                    "frac": achieved / pk["hbm_gbs"], "traffic": traffic, "peak_source": pk["source"],
                    "algorithmic_bytes_per_launch": ab, "ms_per_launch": phases[top]}
    else:
        fl = gemm_flops(top, dims)
        achieved = fl / (phases[top] * 1e-3) / 1e12
        roofline = {"bound": "tensor", "kernel": top, "achieved": achieved, "peak": pk["bf16_tflops"], "unit": "TFLOP/s",
                    "frac": achieved / pk["bf16_tflops"], "traffic": traffic, "peak_source": pk["source"],
                    "flops_per_launch": fl, "ms_per_launch": phases[top]}

    sharding = (f"dp{world}: one pool of {64 * world} crystals split by estimated edge count (longest-processing-time rule), "
                "replicated weights, no data-path collective; per-structure results gathered with one all_gather per step in e2e"
                if pool is not None else f"dp{world}")
    print(json.dumps({
        "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": total_ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32" if dtype == torch.float32 else "f64", "data": "synthetic",
        "config": {"workload": args.workload, "L": L, "channels": C, "cutoff": wl["cutoff"], "elements": len(wl["elements"]),
                   "atoms_per_gpu": n_atoms, "edges_per_gpu": n_edges, "graphs_per_gpu": len(structures),
                   "atoms_total": int(total_atoms), "parallelism": sharding,
                   "radial_weights": "tabulated (cubic Hermite, 512 intervals)" if uses_table else "radial MLP per edge",
                   "l2": "flushed between timed steps (256 MiB write outside the per-step CUDA-event pair)"},
        "step_ms": {"min": min(r[4] for r in per_rank), "median": statistics.median(step_ms), "max": max(r[6] for r in per_rank)},
        "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h, "steps": e2e_steps,
                "step_ms": {"min": round(1e3 * min(e2e_step_s), 3), "median": round(1e3 * statistics.median(e2e_step_s), 3),
                            "max": round(1e3 * max(e2e_step_s), 3)},
                "pipelining": "upload + neighbour list of step k+1 on a second stream during the evaluation of step k; the host "
                              "reads the downloaded results of step k after enqueueing step k+1"},
        "gpu_launches": launches, "clocks": clocks, "roofline": roofline, "cpu_baseline": cpu,
        "phases_ms": {k: round(v, 4) for k, v in sorted(phases.items(), key=lambda kv: -kv[1])},
        "ranks": [{"device_ms_per_step": round(r[0], 3), "host_ms_per_call": round(r[1], 3), "atoms": int(r[2]), "edges": int(r[3]),
                   "step_ms_min": round(r[4], 3), "step_ms_median": round(r[5], 3), "step_ms_max": round(r[6], 3)} for r in per_rank],
        "graph_replays": graph_replays,
        "e2e_host_ms_per_step": {k: round(1e3 * v / e2e_steps, 3) for k, v in e2e_split.items()},
        "domain_md": domain_md,
    }))


if __name__ == "__main__":
    main()
