"""Benchmark of the MACE energy+force path: atom-steps/s on synthetic structures with random-init
weights of the benchmark configurations.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME] [--dtype float64|float32]

One JSON line on stdout (rank 0). A "step" is one full evaluation of one structure: edge arrays
in, index building, all forward and reverse stages, per-atom force / virial / energy reduction.
``value`` is measured with the edge arrays already resident in HBM, ``e2e`` with host (pinned)
arrays in and host results out through the public Python/C-ABI call. ``--impl reference`` times the
reference's own CPU evaluator (``oracle/_ref``) on the host cores instead.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import tempfile
import time
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "mace_energy_force_atom_steps_per_s"
UNIT = "atom-steps/s"

WORKLOADS = {
    # name: (model spec name, structure builder, description)
    "fcc4000": ("fcc128", lambda st, z, seed: st.fcc_box(10, 3.6, z, seed=seed),
                "configs[1]: 4000-atom FCC (10x10x10 cells, a=3.6 A, 5 species, 0.1 A jitter), model 128x0e+128x1o, "
                "l_max 3, correlation 3, r_cut 6 A, 10 radial functions, 89-element model exported for the 5 species present"),
    "fcc1372": ("fcc128", lambda st, z, seed: st.fcc_box(7, 3.6, z, seed=seed),
                "profiling case: 1372-atom FCC box (7x7x7 cells) of the configs[1] construction and model"),
    "fcc6912": ("fcc128", lambda st, z, seed: st.fcc_box(12, 3.6, z, seed=seed),
                "profiling case for the float64 GEMMs: 6,912-atom FCC box (12x12x12 cells) of the configs[1] construction and model, "
                "110,592 rows per operand of the tensor-product output GEMM, about 3 GB on the device"),
    "fcc32k": ("fcc128", lambda st, z, seed: st.fcc_box(20, 3.6, z, seed=seed),
               "profiling case for the channel-mixing GEMMs: 32,000-atom FCC box (20x20x20 cells) of the configs[1] construction and "
               "model, 1.28 M rows of 128 channels per GEMM operand"),
    "fcc256k": ("fcc128", lambda st, z, seed: st.fcc_box((10, 80, 80), 3.6, z, seed=seed),
                "configs[3] per-GPU share: 256,000-atom FCC slab (10x80x80 cells) of the configs[1] construction and model; "
                "8 of these side by side are the 2,048,000-atom box"),
    "water98304": ("organic128_HO", lambda st, z, seed: st.water_box_density(32, 1.0, seed=seed),
                   "configs[2]: 98,304-atom water box (32,768 H2O, 1.0 g/cm^3), organic-liquid model 128x0e+128x1o, r_cut 5 A, "
                   "10-element model exported for the species present (H, O)"),
    "liquid500k": ("deep256", lambda st, z, seed: st.molecular_liquid(55556, 0.79, seed=seed),
                   "configs[4]: 500,004-atom liquid (55,556 rigid 9-atom C2H5OH-like molecules, 0.79 g/cm^3), model 256x0e+256x1o+256x2e, "
                   "three interaction blocks, r_cut 5 A; needs several GPUs (about 300 GB of per-atom arrays in float32)"),
    "liquid62k": ("deep256", lambda st, z, seed: st.molecular_liquid(6945, 0.79, seed=seed),
                  "configs[4] per-GPU share: 62,505-atom liquid (6,945 molecules) of the same construction and three-block model"),
    "water192": ("water64", lambda st, z, seed: st.water_box(4, 12.42, seed=seed),
                 "configs[0]: 64 H2O (192 atoms) in a 12.42 A cell, model 64x0e, r_cut 5 A"),
}
CPU_SAMPLE_CELLS = 4   # the CPU baseline evaluates a 4x4x4-cell (256-atom) box of the same construction


_REAL_STDOUT = None


def emit(obj):
    stream = _REAL_STDOUT or sys.stdout
    stream.write(json.dumps(obj) + "\n")
    stream.flush()


def log(*a):
    print(*a, file=sys.stderr, flush=True)


def model_path(spec_name: str) -> tuple[Path, list[int]]:
    """Model JSON regenerated from its seed into the temp directory (cached across runs on one machine)."""
    from symmetrix_b200.modelgen.generate import generate_model, named_spec, write_json
    cache = Path(os.environ.get("SMX_MODEL_CACHE", tempfile.gettempdir())) / f"smx_bench_{spec_name}.json"
    spec = named_spec("organic128", atomic_numbers=[1, 8]) if spec_name == "organic128_HO" else named_spec(spec_name)
    if not cache.exists():
        t0 = time.time()
        model = generate_model(spec)
        tmp = cache.with_suffix(f".{os.getpid()}.tmp")
        write_json(model, tmp)
        os.replace(tmp, cache)
        log(f"[bench] generated {cache} in {time.time() - t0:.1f} s")
    return cache, sorted(spec.atomic_numbers), spec


def build_inputs(workload: str, seed: int):
    from symmetrix_b200 import structures as st
    spec_name, builder, _ = WORKLOADS[workload]
    path, numbers, spec = model_path(spec_name)
    s = builder(st, numbers, seed)
    nl = st.neighbor_list(s, spec.r_cut)
    return path, spec, s, nl, st.evaluator_inputs(s, nl, numbers)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""
    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.proc = None
        self.path = Path(tempfile.gettempdir()) / f"smx_clocks_{os.getpid()}.csv"
        try:
            self.fh = open(self.path, "w")
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-i", str(gpu_index), "-lms", "100"], stdout=self.fh, stderr=subprocess.DEVNULL)
        except Exception:
            self.proc = None

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except Exception:
            self.proc.kill()
        self.fh.close()
        sm, mx, reasons = [], [], set()
        for line in self.path.read_text().splitlines():
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1])); mx.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"], parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        try:
            self.path.unlink()
        except OSError:
            pass
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["no samples"]}
        # median of the upper half: samples between steps (host-side gaps) idle the clocks
        busy = sorted(sm)[len(sm) // 2:]
        return {"sm_mhz": float(np.median(busy)), "sm_max_mhz": float(max(mx)), "reasons": sorted(reasons), "samples": len(sm)}


def measured_peaks() -> tuple[float, str]:
    p = ROOT / "MEASURED_PEAKS.json"
    if p.exists():
        try:
            return float(json.loads(p.read_text())["hbm_gbs"]), "measured"
        except Exception:
            pass
    return 6650.0, "fallback"


def roofline_for(stage: str, ms: float, n_atoms: int, n_edges: int, K: int, L_max: int, dtype_bytes: int) -> dict:
    """Algorithmic bytes and flops of the stage's dominant kernel for one launch (one full structure).

    Per edge: xyz 24 B + sender index 4 B + sender type 4 B + r 8 B, one gathered sender feature row
    nLM*K*s B, 24 B of partial force written (reverse). Per node: Q*K*s B of tensor-product output written
    (forward) or of its adjoint read (reverse). Scratch the implementation adds (the per-edge adjoint
    message buffer) and table reads served by L2 are not counted. Flops are the operation counts of the
    generated straight-line code per (edge, channel), an FMA counting 2.
    """
    from symmetrix_b200.modelgen.gen_tp_code import tables
    paths, nz, _ = tables(L_max)
    P, Q, nLM = len(paths), sum(2 * p[0] + 1 for p in paths), (L_max + 1) ** 2
    T1, T2 = sum(2 * p[1] + 1 for p in paths), sum(2 * p[2] + 1 for p in paths)
    nnz = len(nz)
    n_yh = len({(a, b) for (_, _, a, b, _) in nz})
    # operation counts of the generated straight-line code, per (edge, channel); an FMA counts 2
    fwd_flops = n_yh + 2 * nnz + 2 * Q + 6 * P
    rev_flops = nnz + 2 * nnz + 2 * nnz + 2 * T1 + 2 * T2 + 2 * T2 + 2 * P + 11 * P
    s = dtype_bytes
    if stage in ("reverse_Phi1", "reverse_Phim"):
        byts = n_edges * (40 + nLM * K * s + 24) + n_atoms * Q * K * s
        flops = n_edges * K * rev_flops
        kernel = "tp_reverse_tmem_kernel" if dtype_bytes == 8 else "tp_reverse_kernel"
    elif stage in ("compute_Phi1", "compute_Phim"):
        byts = n_edges * (40 + nLM * K * s) + n_atoms * Q * K * s
        flops = n_edges * K * fwd_flops
        kernel = "tp_forward_kernel"
    elif stage == "reverse_A0":
        byts = n_edges * (40 + 24) + n_atoms * 16 * K * s
        flops = n_edges * K * (8 * 16 + 14 * 4)
        kernel = "layer0_reverse_kernel"
    else:
        byts = n_edges * 40 + n_atoms * 16 * K * s
        flops = n_edges * K * (2 * 16 + 9 * 4)
        kernel = "layer0_forward_kernel"
    peak, how = measured_peaks()
    achieved = byts / (ms * 1e-3) / 1e9
    # dram__bytes_read.sum + dram__bytes_write.sum per edge from the ncu captures summarised in
    # profiles/tp_reverse_tmem_fcc1372_fp64.md and profiles/edge_kernels_fcc1372_fp64.md (a smaller box of the same
    # construction; traffic grows with the edge count)
    per_edge = {("tp_reverse_tmem_kernel", 8): 6527.0, ("tp_forward_kernel", 8): 2985.0,
                ("layer0_reverse_kernel", 8): 654.0, ("layer0_forward_kernel", 8): 405.0}.get((kernel, dtype_bytes))
    traffic = per_edge * n_edges if per_edge and K == 128 and L_max == 1 else None
    return {"bound": "hbm", "kernel": kernel, "stage": stage, "achieved": achieved, "peak": peak, "unit": "GB/s",
            "frac": achieved / peak, "peak_source": f"of {how}", "traffic": traffic, "launch_ms": ms,
            "algorithmic_bytes": byts, "algorithmic_flops": flops, "achieved_tflops": flops / (ms * 1e-3) / 1e12}


# ------------------------------------------------------------------------------------------- ours
def run_ours(args):
    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if world != args.gpus:
        log(f"[bench] WORLD_SIZE={world} differs from --gpus {args.gpus}; using WORLD_SIZE")
    torch.cuda.set_device(local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=torch.device("cuda", local_rank))

    from symmetrix_b200 import MACE, _lib

    if world > 1:
        return run_decomposed(args, rank, world, local_rank, dist)
    path, spec, s, nl, inputs = build_inputs(args.workload, seed=1 + rank)
    n_atoms, n_edges = s.num_atoms, int(inputs["r"].size)
    ev = MACE(path, dtype=args.dtype, device=local_rank)
    dtype_bytes = 8 if args.dtype == "float64" else 4

    keys = ["node_types", "num_neigh", "neigh_indices", "neigh_types", "xyz", "r"]
    dev = {k: torch.as_tensor(np.ascontiguousarray(inputs[k])).cuda(local_rank) for k in keys}
    pinned = {k: torch.as_tensor(np.ascontiguousarray(inputs[k])).pin_memory() for k in keys}
    host = {k: pinned[k].numpy() for k in keys}
    flush = torch.empty(256 * 1024 * 1024 // 4, dtype=torch.float32, device=f"cuda:{local_rank}")   # 256 MB > 126 MB L2
    f_out = np.zeros((n_atoms, 3)); v_out = np.zeros(6)

    def step_device():
        ev.compute_node_energies_forces(n_atoms, *[dev[k] for k in keys])
        return ev.reduce_forces()

    def step_host():
        ev.compute_node_energies_forces(n_atoms, *[host[k] for k in keys])
        return ev.reduce_forces()

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(step_fn, steps, warmup):
        for _ in range(warmup):
            step_fn()
        barrier()
        dev_ms, wall = 0.0, 0.0
        for _ in range(steps):
            flush.zero_()                      # L2 flush between timed iterations
            torch.cuda.synchronize()
            t0 = time.perf_counter()
            ev.timer_start()
            step_fn()
            dev_ms += ev.timer_stop()
            wall += time.perf_counter() - t0
        barrier()
        return dev_ms, wall

    launches0 = ev.launch_count
    sampler = ClockSampler(local_rank) if rank == 0 else None
    dev_ms, wall_s = timed(step_device, args.steps, args.warmup)
    clocks = sampler.stop() if sampler else None
    launches = ev.launch_count - launches0
    launches_per_step = launches // (args.steps + args.warmup)
    e2e_ms, e2e_wall = timed(step_host, args.steps, max(1, args.warmup // 2))

    # per-stage device time -> dominant kernel and its roofline
    ev.set_profiling(True)
    stage_acc: dict = {}
    for _ in range(max(2, min(args.steps, 5))):
        flush.zero_(); torch.cuda.synchronize()
        ev.compute_node_energies_forces(n_atoms, *[dev[k] for k in keys])
        for name, ms in ev.stage_times().items():
            stage_acc.setdefault(name, []).append(ms)
    ev.set_profiling(False)
    stage_ms = {k: float(np.mean(v)) for k, v in stage_acc.items()}
    dominant = max(stage_ms, key=stage_ms.get)
    roof = roofline_for(dominant, stage_ms[dominant], n_atoms, n_edges, ev.num_channels, ev.L_max, dtype_bytes)
    fma = ctypes_fma_peak(_lib, 32 if args.dtype == "float32" else 64, local_rank)
    roof["fma_peak_tflops"] = fma
    roof["fma_frac"] = roof["achieved_tflops"] / fma if fma else None
    roof["l2_stream"] = l2_stream_floor(ev, dominant, roof["launch_ms"])

    def reduce_max(x):
        if world == 1:
            return x
        t = torch.tensor([x], dtype=torch.float64, device=f"cuda:{local_rank}")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    dev_ms_max = reduce_max(dev_ms)
    e2e_ms_max = reduce_max(e2e_wall * 1e3)
    total_atoms = n_atoms * world
    value = total_atoms * args.steps / (dev_ms_max * 1e-3)
    e2e_value = total_atoms * args.steps / (e2e_ms_max * 1e-3)
    h2d = sum(host[k].nbytes for k in keys)
    d2h = f_out.nbytes + v_out.nbytes + 8

    out = None
    if rank == 0:
        out = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": dev_ms_max / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f64" if args.dtype == "float64" else "f32", "data": "synthetic",
            "config": {"workload": args.workload, "description": WORKLOADS[args.workload][2], "atoms_per_gpu": n_atoms,
                       "edges_per_gpu": n_edges, "parallelism": "single GPU" if world == 1 else f"{world} independent boxes (one per GPU, no halo exchange)",
                       "l2": "256 MB buffer written between timed steps (L2 flush); per-step working set exceeds 126 MB",
                       "timing": "CUDA events on the evaluator's stream around each step, summed over steps, max over ranks"},
            "e2e": {"value": e2e_value, "unit": UNIT, "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h,
                    "ms_per_step": e2e_ms_max / args.steps, "timing": "wall clock around the public call with pinned host arrays in, host forces/virial/energy out"},
            "gpu_launches": launches, "gpu_launches_per_step": launches_per_step,
            "clocks": clocks, "roofline": roof, "stage_ms": stage_ms,
            "wall_ms_per_step": wall_s * 1e3 / args.steps,
        }
        if "compute_A1" in stage_ms and fma:
            # the channel-mixing GEMM of the tensor-product output (tensor cores: DMMA in float64, tcgen05 3xTF32 in float32):
            # Phi1 [N, Q, K] in, A1 [N, 16, K] out; its flop rate beside the measured FMA peak of the same precision
            K, Q = ev.num_channels, ev.num_lme
            a1_ms = stage_ms["compute_A1"]
            a1_bytes = n_atoms * (Q + 16) * K * dtype_bytes
            a1_flops = 2.0 * n_atoms * Q * K * K
            peak_gbs, how = measured_peaks()
            out["gemm_A1"] = {"kernel": "gemm_rows_f64_async_kernel" if dtype_bytes == 8 else "gemm_rows_tcgen05_kernel",
                              "launch_ms": a1_ms, "algorithmic_bytes": a1_bytes, "achieved_gbs": a1_bytes / (a1_ms * 1e-3) / 1e9,
                              "hbm_frac": a1_bytes / (a1_ms * 1e-3) / 1e9 / peak_gbs, "peak_source": f"of {how}",
                              "achieved_tflops": a1_flops / (a1_ms * 1e-3) / 1e12,
                              "tflops_over_fma_peak": a1_flops / (a1_ms * 1e-3) / 1e12 / fma}
        sample = None
        if world == 1 and not args.no_cpu_baseline:
            out["cpu_baseline"], sample = cpu_baseline(args.workload)
        ev2 = None
        if world == 1 and not args.no_extra:
            other = "float32" if args.dtype == "float64" else "float64"
            ev2 = MACE(path, dtype=other, device=local_rank)
            ev_saved = ev

            def step2():
                ev2.compute_node_energies_forces(n_atoms, *[dev[k] for k in keys])
                return ev2.reduce_forces()
            for _ in range(max(3, args.warmup)):
                step2()
            ms2 = 0.0
            for _ in range(args.steps):
                flush.zero_(); torch.cuda.synchronize()
                ev2.timer_start(); step2(); ms2 += ev2.timer_stop()
            e64 = ev_saved.reduce_forces()[2] if args.dtype == "float64" else ev2.reduce_forces()[2]
            e32 = ev2.reduce_forces()[2] if args.dtype == "float64" else ev_saved.reduce_forces()[2]
            out["extra"] = {other: {"value": n_atoms * args.steps / (ms2 * 1e-3), "ms_per_step": ms2 / args.steps},
                            "fp32_vs_fp64_rel_energy_diff": abs(e32 - e64) / abs(e64)}
        if sample is not None:
            # the GPU path on the CPU baseline's own inputs, against the reference's results (outside every timed region)
            evs = {("f64" if args.dtype == "float64" else "f32"): ev}
            if ev2 is not None:
                evs["f32" if args.dtype == "float64" else "f64"] = ev2
            out["parity"] = parity_on_sample(evs, sample)
            out["parity"]["against"] = out["cpu_baseline"]["kind"] + " CPU evaluator on the cpu_baseline sample"
        if world == 1 and not args.no_extra:
            out.setdefault("extra", {})["radial_mlp"] = radial_mode_comparison(path, n_atoms, dev, keys, flush, torch, local_rank)
        if world == 1 and not args.no_extra and args.workload == "fcc4000":
            del ev2
            out.setdefault("extra", {})["config3"] = config3_single(local_rank, torch)
        emit(out)
    if world > 1:
        dist.barrier()
        dist.destroy_process_group()
    return out


def radial_mode_comparison(path, n_atoms, dev, keys, flush, torch, local_rank) -> dict:
    """float32 stage times of the tensor product with the radial functions (a) from the spline tables, (b) from the
    un-splined network at run time (SMX_RADIAL=mlp: Bessel x cutoff and hidden layers per edge, last layer on the tensor
    cores inside the tensor-product kernels) and (c) from the low-rank form of the tables (SMX_RADIAL=lowrank: tabulated
    last hidden layer, last layer on the tensor cores inside the kernels), for model files that carry the extra keys."""
    from symmetrix_b200 import MACE
    out = {}
    for mode in ("spline", "mlp", "lowrank"):
        os.environ["SMX_RADIAL"] = mode
        try:
            ev = MACE(path, dtype="float32", device=local_rank)
        except Exception as exc:            # model without x_radial_* keys
            out[mode] = {"unavailable": str(exc)}
            continue
        finally:
            os.environ.pop("SMX_RADIAL", None)
        ev.set_profiling(True)
        acc: dict = {}
        total = 0.0
        for it in range(4):
            flush.zero_(); torch.cuda.synchronize()
            ev.timer_start()
            ev.compute_node_energies_forces(n_atoms, *[dev[k] for k in keys])
            t = ev.timer_stop()
            if it > 0:
                total += t
                for name, ms in ev.stage_times().items():
                    acc[name] = acc.get(name, 0.0) + ms / 3
        energy = ev.reduce_forces(want_forces=False)[2]
        out[mode] = {"compute_Phi1_ms": acc.get("compute_Phi1"), "reverse_Phi1_ms": acc.get("reverse_Phi1"), "step_ms": total / 3,
                     "energy": energy}
        del ev
    for mode in ("mlp", "lowrank"):
        if "energy" in out.get("spline", {}) and "energy" in out.get(mode, {}):
            out[mode]["rel_energy_diff_vs_spline"] = abs(out[mode]["energy"] - out["spline"]["energy"]) / abs(out["spline"]["energy"])
    return out


def config3_single(local_rank, torch) -> dict:
    """configs[3] at one GPU: its per-GPU share, a 256,000-atom slab (10x80x80 cells) of the configs[1] model in float32."""
    from symmetrix_b200 import MACE
    path, spec, s, nl, inputs = build_inputs("fcc256k", seed=1)
    ev = MACE(path, dtype="float32", device=local_rank)
    keys = ["node_types", "num_neigh", "neigh_indices", "neigh_types", "xyz", "r"]
    dev = {k: torch.as_tensor(np.ascontiguousarray(inputs[k])).cuda(local_rank) for k in keys}
    steps, ms = 3, 0.0
    for it in range(1 + steps):
        ev.timer_start()
        ev.compute_node_energies_forces(s.num_atoms, *[dev[k] for k in keys])
        ev.reduce_forces(want_forces=True)
        t = ev.timer_stop()
        if it > 0:
            ms += t
    # per-stage device times of one more evaluation, and the channel-mixing GEMM of the tensor-product output (compute_A1,
    # tcgen05 kernel) against the HBM roofline: it reads Phi1 [N, Q, K] and writes A1 [N, 16, K] once each
    ev.set_profiling(True)
    ev.compute_node_energies_forces(s.num_atoms, *[dev[k] for k in keys])
    stage_ms = ev.stage_times()
    ev.set_profiling(False)
    peak, how = measured_peaks()
    K, Q = ev.num_channels, ev.num_lme
    a1_bytes = s.num_atoms * (Q + 16) * K * 4
    a1_flops = 2.0 * s.num_atoms * Q * K * K
    a1 = {"kernel": "gemm_rows_tcgen05_kernel", "stage": "compute_A1", "launch_ms": stage_ms.get("compute_A1"),
          "algorithmic_bytes": a1_bytes, "achieved_gbs": a1_bytes / (stage_ms["compute_A1"] * 1e-3) / 1e9,
          "hbm_frac": a1_bytes / (stage_ms["compute_A1"] * 1e-3) / 1e9 / peak, "peak_source": f"of {how}",
          "achieved_tflops_3xtf32_counted_once": a1_flops / (stage_ms["compute_A1"] * 1e-3) / 1e12}
    return {"workload": "fcc256k", "dtype": "f32", "atoms": s.num_atoms, "edges": int(inputs["r"].size), "steps": steps,
            "ms_per_step": ms / steps, "value": s.num_atoms * steps / (ms * 1e-3), "unit": UNIT, "stage_ms": stage_ms, "gemm_A1": a1,
            "note": "inputs larger than L2; one warm-up step; efficiency at N GPUs = value(N) / (N x this value)"}


def config3_decomposed(args, rank, world, local_rank, dist, torch) -> dict:
    """configs[3] at N GPUs: N slabs of 256,000 atoms (10x80x80 cells each; at N = 8 the 2,048,000-atom box, 80x80x80
    cells), configs[1] model in float32, ghost shell and halo exchange as in the main run."""
    from symmetrix_b200 import MACE, structures as st
    from symmetrix_b200.domain import SlabRank, evaluate_decomposed, make_slab_plan
    path, numbers, spec = model_path("fcc128")
    s = st.fcc_box((10 * world, 80, 80), 3.6, numbers, seed=1)
    ev = MACE(path, dtype="float32", device=local_rank)
    if args.dd_transport == "library":
        ev.comm_init(dist)
    rk = SlabRank(make_slab_plan(s, spec.r_cut, rank, world, mode=args.dd_mode), ev, spec.r_cut, numbers)
    rk.build_edges()
    steps, total = 3, 0.0
    for it in range(1 + steps):
        dist.barrier(); torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        evaluate_decomposed([rk], dist=dist)
        torch.cuda.synchronize()
        e1.record(); e1.synchronize()
        if it > 0:
            total += e0.elapsed_time(e1)
    t = torch.tensor([total], dtype=torch.float64, device=f"cuda:{local_rank}")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms = float(t.item())
    return {"workload": f"fcc256k x {world} along x", "dtype": "f32", "atoms": s.num_atoms, "steps": steps, "ms_per_step": ms / steps,
            "value": s.num_atoms * steps / (ms * 1e-3), "unit": UNIT, "ghost_rows_this_rank": rk.plan.n_ghost,
            "note": "weak scaling of configs[3]; efficiency = value / (N x the single-GPU extra.config3.value); "
                    "timed with CUDA events, barrier + synchronize on both sides, max over ranks"}


def run_decomposed(args, rank, world, local_rank, dist):
    """N > 1: one structure, N times longer along x than the single-GPU workload (weak scaling), cut into N slabs
    with a ghost shell of r_cut; H1 rows forward, H1_adj and force rows back between slab neighbours (NCCL
    send/recv), energy + virial all-reduced."""
    import torch
    from symmetrix_b200 import MACE, structures as st
    from symmetrix_b200.domain import SlabRank, evaluate_decomposed, make_slab_plan

    spec_name = WORKLOADS[args.workload][0]
    path, numbers, spec = model_path(spec_name) if rank == 0 else (None, None, None)
    dist.barrier()
    path, numbers, spec = model_path(spec_name)
    cells = {"fcc4000": (10, 10, 10), "fcc1372": (7, 7, 7), "fcc6912": (12, 12, 12), "fcc32k": (20, 20, 20), "fcc256k": (10, 80, 80)}.get(args.workload)
    if cells is not None:
        # weak scaling: the box grows along x with the number of GPUs
        s = st.fcc_box((cells[0] * world, cells[1], cells[2]), 3.6, numbers, seed=1)
        scaling, label = "weak", f"{args.workload} x {world} along x"
    else:
        # strong scaling: the same box (configs[2]: the 98,304-atom water box) cut into `world` slabs
        s = WORKLOADS[args.workload][1](st, numbers, 1)
        scaling, label = "strong", f"{args.workload} in {world} slabs along x"
    ev = MACE(path, dtype=args.dtype, device=local_rank)
    if args.dd_transport == "library":
        ev.comm_init(dist)            # halo rows by ncclSend / ncclRecv issued inside the library, on the evaluator's stream
    rk = SlabRank(make_slab_plan(s, spec.r_cut, rank, world, mode=args.dd_mode, num_interactions=ev.num_interactions), ev, spec.r_cut, numbers)
    rk.build_edges()
    flush = torch.empty(256 * 1024 * 1024 // 4, dtype=torch.float32, device=f"cuda:{local_rank}")

    def barrier():
        dist.barrier()
        torch.cuda.synchronize()

    def step_device():
        return evaluate_decomposed([rk], dist=dist)

    def step_host():
        rk.build_edges()                       # positions from host memory, neighbour list rebuilt on the device
        e, v, f = evaluate_decomposed([rk], dist=dist)
        return e, v, f[0].cpu()

    def timed(fn, steps, warmup):
        for _ in range(warmup):
            fn()
        barrier()
        total = 0.0
        for _ in range(steps):
            flush.zero_()
            barrier()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            e0.record()
            fn()
            torch.cuda.synchronize()
            e1.record()
            e1.synchronize()
            total += e0.elapsed_time(e1)
        barrier()
        return total

    launches0 = ev.launch_count
    sampler = ClockSampler(local_rank) if rank == 0 else None
    ms = timed(step_device, args.steps, args.warmup)
    clocks = sampler.stop() if sampler else None
    launches = ev.launch_count - launches0
    e2e_ms = timed(step_host, max(2, args.steps // 4), 1)
    e2e_steps = max(2, args.steps // 4)

    # per-stage device time on this rank (separate passes) -> roofline of the dominant kernel
    rk.stage_ms = {}
    prof_steps = 3
    for _ in range(prof_steps):
        step_device()
    stage_ms = {k: v / prof_steps for k, v in rk.stage_ms.items()}
    rk.stage_ms = None
    dominant = max(stage_ms, key=stage_ms.get)
    roof = roofline_for(dominant, stage_ms[dominant], rk.plan.n_own, rk.num_edges, ev.num_channels, ev.L_max,
                        8 if args.dtype == "float64" else 4)
    roof["scope"] = "rank 0's slab"

    # Correctness of the decomposed run, outside the timed region: rank 0 evaluates the whole box as one domain and every
    # rank compares its owned forces (and the reduced energy) with it.
    dd_check = None
    if s.num_atoms <= 300_000:
        energy_dd, _, owned = evaluate_decomposed([rk], dist=dist)
        ref_f = torch.zeros((s.num_atoms, 3), dtype=torch.float64, device=f"cuda:{local_rank}")
        ref_e = torch.zeros(1, dtype=torch.float64, device=f"cuda:{local_rank}")
        if rank == 0:
            single = MACE(path, dtype=args.dtype, device=local_rank)
            zmap = {int(z): t_ for t_, z in enumerate(single.atomic_numbers)}
            single.build_neighbors(s.positions, np.array([zmap[int(z)] for z in s.numbers], dtype=np.int32), s.cell, s.pbc, r_cut=spec.r_cut)
            single.compute_current()
            f1, _, e1 = single.reduce_forces()
            ref_f.copy_(torch.as_tensor(f1)); ref_e[0] = e1
            del single
        dist.broadcast(ref_f, 0); dist.broadcast(ref_e, 0)
        own = torch.as_tensor(rk.plan.own_global, device=ref_f.device)
        err = torch.stack([(owned[0] - ref_f[own]).abs().max(), ref_f.abs().max()])
        dist.all_reduce(err, op=dist.ReduceOp.MAX)
        e1 = float(ref_e.item())
        dd_check = {"rel_dE": abs(energy_dd - e1) / abs(e1), "max_abs_dF": float(err[0].item()), "rel_dF": float((err[0] / err[1]).item()),
                    "against": "the whole box evaluated as one domain on rank 0 (same precision), outside the timed region",
                    "gate": "1e-10 relative" if args.dtype == "float64" else "1e-4 relative, 1e-3 eV/A"}
    else:
        dd_check = {"skipped": "the whole box does not fit one GPU's evaluation; checked on smaller boxes by tests/test_gpu_domain.py"}

    t = torch.tensor([ms, e2e_ms], dtype=torch.float64, device=f"cuda:{local_rank}")
    dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_max, e2e_max = (float(x) for x in t.cpu())
    counts = torch.tensor([rk.plan.n_own, rk.plan.n_ghost, rk.num_edges], dtype=torch.float64, device=f"cuda:{local_rank}")
    dist.all_reduce(counts)
    width = ev.num_LM * ev.num_channels * (8 if args.dtype == "float64" else 4)
    h2d_bytes = int((rk.plan.n_own + rk.plan.n_ghost) * 28 * world)
    config3 = None
    if args.workload == "fcc4000" and not args.no_extra:
        del ev, rk                       # the evaluator's arrays make room for the larger workload
        torch.cuda.empty_cache()
        config3 = config3_decomposed(args, rank, world, local_rank, dist, torch)
    if rank == 0:
        n_total = s.num_atoms
        out = {
            "metric": METRIC, "value": n_total * args.steps / (ms_max * 1e-3), "unit": UNIT, "n_gpus": world, "steps": args.steps,
            "warmup": args.warmup, "ms_per_step": ms_max / args.steps, "higher_is_better": True, "scaling": scaling, "vs_baseline": None,
            "dtype": "f64" if args.dtype == "float64" else "f32", "data": "synthetic",
            "config": {"workload": label, "description": WORKLOADS[args.workload][2],
                       "atoms_total": n_total, "atoms_per_gpu": n_total // world, "ghost_rows_total": int(counts[1].item()),
                       "edges_total": int(counts[2].item()),
                       "parallelism": (f"{world} slabs along x, ghost shell r_cut, halo exchange of H1 / H1_adj / force rows by NCCL send/recv"
                                       if args.dd_mode == "message_passing" else
                                       f"{world} slabs along x, ghost shell 2 r_cut, layer 0 recomputed on ghosts, force rows by NCCL send/recv"),
                       "transport": args.dd_transport,
                       "halo_bytes_per_rank_per_exchange": int(counts[1].item() / world * width),
                       "l2": "256 MB buffer written between timed steps (L2 flush)",
                       "timing": "CUDA events around each step with a barrier + synchronize on both sides, summed, max over ranks"},
            "e2e": {"value": n_total * e2e_steps / (e2e_max * 1e-3), "unit": UNIT,
                    "h2d_bytes_per_step": h2d_bytes,
                    "d2h_bytes_per_step": int(n_total * 24 + 56 * world), "ms_per_step": e2e_max / e2e_steps,
                    "timing": "per step: local positions/types from host, neighbour list rebuilt on the device, evaluation, owned forces to host"},
            "gpu_launches": launches * world, "gpu_launches_per_step": launches // (args.steps + args.warmup),
            "clocks": clocks, "roofline": roof, "stage_ms": stage_ms, "dd_check": dd_check,
        }
        if config3 is not None:
            out["extra"] = {"config3": config3}
        emit(out)
    dist.barrier()
    dist.destroy_process_group()
    return None


def l2_stream_floor(ev, stage: str, launch_ms: float) -> dict:
    """The edge kernels read one spline row per edge (4 * P * K values) out of a table larger than L2 that no
    SM reuses from L1; this measures, on the evaluator's current edge set, a kernel that does only those reads.
    `frac` = probe time / kernel time: how close the kernel is to the floor the L2 -> SM path sets."""
    layer = 0 if stage.endswith("A0") else 1
    ms, nbytes = ev.measure_row_stream(layer)
    return {"bytes": nbytes, "probe_ms": ms, "probe_gbs": nbytes / (ms * 1e-3) / 1e9 if ms > 0 else None,
            "kernel_gbs": nbytes / (launch_ms * 1e-3) / 1e9, "frac": ms / launch_ms if launch_ms > 0 else None}


def ctypes_fma_peak(_lib, precision: int, device: int) -> float | None:
    import ctypes
    lib = _lib.load()
    t = ctypes.c_double(0.0)
    if lib.smx_measure_fma_peak(precision, device, ctypes.byref(t)) != 0:
        return None
    return t.value


# ------------------------------------------------------------------------------------------- CPU arms
def _cpu_sample_inputs(workload: str, seed: int):
    from symmetrix_b200 import structures as st
    spec_name, _, _ = WORKLOADS[workload]
    path, numbers, spec = model_path(spec_name)
    if workload in ("fcc4000", "fcc1372", "fcc6912", "fcc32k", "fcc256k"):
        s = st.fcc_box(CPU_SAMPLE_CELLS, 3.6, numbers, seed=seed)
        sample = f"{CPU_SAMPLE_CELLS}x{CPU_SAMPLE_CELLS}x{CPU_SAMPLE_CELLS}-cell FCC box ({s.num_atoms} atoms) of the same construction and model"
    else:
        s = st.water_box(4, 12.42, seed=seed)
        sample = "the full 192-atom structure"
    nl = st.neighbor_list(s, spec.r_cut)
    return path, s, st.evaluator_inputs(s, nl, numbers), sample


def _timed_variant():
    """The timed build of the reference: with OpenBLAS (one thread) when that build is here and loads, else with the
    plain-loop BLAS; (None, None) when the reference was never compiled."""
    from oracle import ref as ref_driver
    os.environ.setdefault("OPENBLAS_NUM_THREADS", "1")
    if ref_driver.available("timed_openblas"):
        try:
            ref_driver._load("timed_openblas")
            return "timed_openblas", "OpenBLAS 0.3.15 (one thread)"
        except OSError:
            pass
    if ref_driver.available("timed"):
        return "timed", "plain-loop BLAS"
    return None, None


def cpu_baseline(workload: str):
    """The reference CPU evaluator (serial, one core) on a bounded sample of the workload."""
    from oracle import ref as ref_driver
    path, s, inputs, sample = _cpu_sample_inputs(workload, seed=1)
    variant, blas = _timed_variant()
    if variant:
        r = ref_driver.ReferenceMACE(path, variant)
        kind = "reference"
        fn = lambda: r.compute_node_energies_forces(inputs)   # noqa: E731
    else:
        from oracle.mace_numpy import MaceOracle
        o = MaceOracle(path)
        kind, blas = "port", "numpy"
        fn = lambda: o.compute_node_energies_forces(inputs)   # noqa: E731
    e_ref, f_ref = fn()                    # first call sizes the evaluator's internal arrays
    reps, t0 = 0, time.perf_counter()
    while reps < 3 and (time.perf_counter() - t0) < 20.0:
        fn(); reps += 1
    dt = (time.perf_counter() - t0) / reps
    out = {"value": s.num_atoms / dt, "unit": UNIT, "cores": 1, "kind": kind,
           "sample": f"{sample}; {reps} evaluations after one warm-up; -O3 -ffast-math -march=x86-64-v3, {blas}",
           "seconds_per_step": dt,
           "note": "a lower bound on the reference's CPU speed when the BLAS is the plain-loop one"}
    return out, (path, inputs, e_ref, f_ref)


def parity_on_sample(evaluators: dict, sample) -> dict:
    """The GPU path on exactly the inputs the CPU baseline evaluated, against the reference's energies and forces."""
    path, inputs, e_ref, f_ref = sample
    out = {}
    for name, ev in evaluators.items():
        ev.compute_node_energies_forces(int(inputs["num_nodes"]), inputs["node_types"], inputs["num_neigh"], inputs["neigh_indices"],
                                        inputs["neigh_types"], inputs["xyz"], inputs["r"])
        e, f = ev.node_energies, ev.node_forces
        out[name] = {"rel_dE": float(abs(e.sum() - e_ref.sum()) / abs(e_ref.sum())), "max_abs_dF": float(np.abs(f - f_ref).max()),
                     "rel_dF": float(np.abs(f - f_ref).max() / np.abs(f_ref).max()), "atoms": int(inputs["num_nodes"]),
                     "gate": "1e-10 relative" if name == "f64" else "1e-4 relative, 1e-3 eV/A"}
    return out


def _replica_main(idx, workload, steps, warmup, barrier, times):
    from oracle import ref as ref_driver
    path, s, inputs, _ = _cpu_sample_inputs(workload, seed=100 + idx)
    variant, _ = _timed_variant()
    r = ref_driver.ReferenceMACE(path, variant) if variant else None
    if r is None:
        from oracle.mace_numpy import MaceOracle
        o = MaceOracle(path)
        fn = lambda: o.compute_node_energies_forces(inputs)   # noqa: E731
    else:
        fn = lambda: r.compute_node_energies_forces(inputs)   # noqa: E731
    for _ in range(warmup):
        fn()
    barrier.wait()
    t0 = time.perf_counter()
    for _ in range(steps):
        fn()
    times[idx] = time.perf_counter() - t0
    barrier.wait()


def run_reference(args):
    """The reference's own CPU implementation on all usable host cores: the evaluator is serial, so the host
    is filled with independent replicas, each evaluating its own sample box per step."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return None
    import multiprocessing as mp
    from oracle import ref as ref_driver
    try:
        import psutil
        mem_gb = psutil.virtual_memory().available / 2 ** 30
    except Exception:
        mem_gb = 64.0
    cores = os.cpu_count() or 1
    try:
        cores = len(os.sched_getaffinity(0))
    except Exception:
        pass
    replicas = int(max(1, min(cores, mem_gb // 4, 64)))
    model_path(WORKLOADS[args.workload][0])            # generate once, before the replicas start
    path, s, inputs, sample = _cpu_sample_inputs(args.workload, seed=100)
    ctx = mp.get_context("spawn")
    barrier = ctx.Barrier(replicas)
    times = ctx.Array("d", replicas)
    warmup = max(1, min(args.warmup, 2))
    steps = max(1, min(args.steps, 5))
    procs = [ctx.Process(target=_replica_main, args=(i, args.workload, steps, warmup, barrier, times)) for i in range(replicas)]
    for p in procs:
        p.start()
    for p in procs:
        p.join()
    if any(p.exitcode != 0 for p in procs):
        emit({"impl": "reference", "unavailable": "a CPU replica of the reference evaluator exited with an error"})
        return None
    t = max(times)
    value = replicas * s.num_atoms * steps / t
    variant, blas = _timed_variant()
    kind = "reference" if variant else "port"
    out = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": steps, "warmup": warmup,
        "ms_per_step": t * 1e3 / steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f64",
        "data": "synthetic",
        "config": {"workload": args.workload, "description": WORKLOADS[args.workload][2],
                   "parallelism": f"{replicas} independent serial replicas on the host cores (the reference CPU path has no threading)"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": replicas, "kind": kind,
                         "sample": f"each replica evaluates a {sample} per step; requested steps/warmup {args.steps}/{args.warmup} "
                                   f"bounded to {steps}/{warmup}; BLAS: {blas}"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    emit(out)
    return out


def main():
    # Libraries (NCCL among them) may print to stdout; the one JSON line goes to the real stdout, everything else to stderr.
    global _REAL_STDOUT
    _REAL_STDOUT = os.fdopen(os.dup(1), "w")
    os.dup2(2, 1)
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=40)
    ap.add_argument("--warmup", type=int, default=3)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="fcc4000", choices=sorted(WORKLOADS))
    ap.add_argument("--dtype", default=None, choices=["float64", "float32"])
    ap.add_argument("--dd-mode", default="message_passing", choices=["message_passing", "recompute"],
                    help="N > 1: exchange H1 / H1_adj rows (ghost shell r_cut) or recompute layer 0 on a 2 r_cut shell")
    ap.add_argument("--dd-transport", default="torch", choices=["torch", "library"],
                    help="N > 1: halo buffers through torch.distributed, or NCCL send / recv issued inside the library")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-extra", action="store_true")
    args = ap.parse_args()
    if args.dtype is None:   # configs[0] and [1] are quoted in float64 (the reference CPU precision), the larger ones in float32
        args.dtype = "float32" if args.workload in ("fcc256k", "water98304", "liquid500k", "liquid62k") else "float64"
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
