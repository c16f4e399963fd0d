"""Slab decomposition on GPUs: all ranks emulated in one process on one GPU, and real ranks over NCCL when the
machine has at least two GPUs."""
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

from symmetrix_b200 import MACE, structures as st
from symmetrix_b200.domain import SlabRank, evaluate_decomposed, make_slab_plan

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]


def _single(path, s, dtype="float64"):
    ev = MACE(path, dtype=dtype)
    nl = st.neighbor_list(s, ev.r_cut)
    inp = st.evaluator_inputs(s, nl, ev.atomic_numbers)
    ev.compute_node_energies_forces(inp["num_nodes"], inp["node_types"], inp["num_neigh"], inp["neigh_indices"], inp["neigh_types"],
                                    inp["xyz"], inp["r"])
    return ev.reduce_forces()


@pytest.mark.parametrize("dtype,world,mode", [("float64", 2, "message_passing"), ("float64", 3, "message_passing"),
                                              ("float32", 2, "message_passing"), ("float64", 2, "recompute"),
                                              ("float64", 3, "recompute"), ("float32", 3, "recompute")])
def test_emulated_ranks_on_one_gpu_match_single_domain(model_file, dtype, world, mode):
    path, model, spec = model_file("fcc128", num_channels=32, num_spline_points=32)
    s = st.fcc_box((4 * world, 3, 3), 3.6, model["atomic_numbers"], seed=17, jitter=0.12)
    f_ref, v_ref, e_ref = _single(path, s)
    ranks = []
    for r in range(world):
        ev = MACE(path, dtype=dtype)
        rk = SlabRank(make_slab_plan(s, spec.r_cut, r, world, mode=mode), ev, spec.r_cut, ev.atomic_numbers)
        rk.build_edges()
        ranks.append(rk)
    rel, fabs = (1e-10, 1e-9) if dtype == "float64" else (1e-4, 1e-3)
    for _ in range(2):
        energy, virial, owned = evaluate_decomposed(ranks)
        forces = np.zeros_like(f_ref)
        for rk, f in zip(ranks, owned):
            forces[rk.plan.own_global] = f.cpu().numpy()
        assert abs(energy - e_ref) <= rel * abs(e_ref)
        assert np.abs(forces - f_ref).max() <= fabs
        assert np.abs(virial - v_ref).max() <= 100 * rel * max(1.0, np.abs(v_ref).max())


@pytest.mark.parametrize("dtype,mode", [("float64", "message_passing"), ("float64", "recompute"), ("float32", "message_passing")])
def test_zbl_and_density_normalised_model_decomposes_on_gpu(model_file, dtype, mode):
    """compute_ZBL and the *_scaled stages in a decomposed run (pair_symmetrix_mace.cpp:449-494, 667-697)."""
    world = 2
    path, model, spec = model_file("fcc128", num_channels=32, num_spline_points=32, zbl=True, density=True)
    s = st.fcc_box((4 * world, 3, 3), 3.2, model["atomic_numbers"], seed=9, jitter=0.25)
    f_ref, v_ref, e_ref = _single(path, s)
    ranks = []
    for r in range(world):
        ev = MACE(path, dtype=dtype)
        assert ev.has_zbl
        rk = SlabRank(make_slab_plan(s, spec.r_cut, r, world, mode=mode), ev, spec.r_cut, ev.atomic_numbers)
        rk.build_edges()
        ranks.append(rk)
    rel, fabs = (1e-10, 1e-8) if dtype == "float64" else (1e-4, 1e-3)
    energy, virial, owned = evaluate_decomposed(ranks)
    forces = np.zeros_like(f_ref)
    for rk, f in zip(ranks, owned):
        forces[rk.plan.own_global] = f.cpu().numpy()
    assert abs(energy - e_ref) <= rel * abs(e_ref)
    assert np.abs(forces - f_ref).max() <= fabs * max(1.0, np.abs(f_ref).max())


def test_decomposed_float64_evaluations_are_bitwise_reproducible(model_file):
    """The fold-back of H1_adj and force rows on the owner adds in a fixed order (no atomics): two evaluations give the
    same bits. Thin slabs make atoms ghosts of the same peer twice, so rows repeat inside one unpack list."""
    world = 2
    path, model, spec = model_file("fcc128", num_channels=32, num_spline_points=32)
    s = st.fcc_box((4, 3, 3), 3.6, model["atomic_numbers"], seed=23, jitter=0.12)      # 7.2 A slabs, r_cut 6 A
    ranks = []
    for r in range(world):
        ev = MACE(path, dtype="float64")
        rk = SlabRank(make_slab_plan(s, spec.r_cut, r, world), ev, spec.r_cut, ev.atomic_numbers)
        rk.build_edges()
        ranks.append(rk)
    assert any(np.unique(rows).size < rows.size for rk in ranks for rows in rk.plan.send_rows.values())
    f_ref, v_ref, e_ref = _single(path, s)
    results = []
    for _ in range(3):
        energy, virial, owned = evaluate_decomposed(ranks)
        results.append((energy, np.asarray(virial).copy(), [f.cpu().numpy().copy() for f in owned]))
    assert abs(results[0][0] - e_ref) <= 1e-10 * abs(e_ref)
    for energy, virial, owned in results[1:]:
        assert energy == results[0][0]
        assert np.array_equal(virial, results[0][1])
        for a, b in zip(owned, results[0][2]):
            assert np.array_equal(a, b)


def _gpu_count():
    import torch
    return torch.cuda.device_count()


@pytest.mark.parametrize("dtype,mode", [("float64", "message_passing"), ("float32", "message_passing"), ("float64", "recompute")])
def test_ranks_over_nccl_match_single_domain(model_file, dtype, mode, tmp_path):
    world = min(_gpu_count(), 4)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    path, model, spec = model_file("fcc128", num_channels=32, num_spline_points=32)
    out = tmp_path / "dd.npz"
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(29400 + os.getpid() % 500), str(ROOT / "tests" / "dd_nccl_worker.py"), str(path), dtype, str(out), mode]
    subprocess.run(cmd, check=True, env=env, timeout=600)
    d = np.load(out)
    rel, fabs = (1e-10, 1e-9) if dtype == "float64" else (1e-4, 1e-3)
    assert abs(float(d["energy"]) - float(d["e_ref"])) <= rel * abs(float(d["e_ref"]))
    assert np.abs(d["forces"] - d["f_ref"]).max() <= fabs
    assert np.abs(d["virial"] - d["v_ref"]).max() <= 100 * rel * max(1.0, np.abs(d["v_ref"]).max())


@pytest.mark.parametrize("dtype,mode", [("float64", "message_passing"), ("float64", "recompute"), ("float32", "message_passing")])
def test_three_block_model_emulated_ranks_match_single_domain(model_file, dtype, mode):
    """Three interaction blocks: H1 and Hm rows travel forward, Hm_adj and H1_adj back (message passing), or a 3 r_cut
    shell with three receiver sets (recompute)."""
    world = 2
    path, model, spec = model_file("deep256", num_channels=32, num_spline_points=32, radial_mlp=(8, 8))
    s = st.fcc_box((10, 2, 2), 3.6, model["atomic_numbers"], seed=21, jitter=0.12)      # 36 A along x, r_cut 5 A
    f_ref, v_ref, e_ref = _single(path, s)
    ranks = []
    for r in range(world):
        ev = MACE(path, dtype=dtype)
        rk = SlabRank(make_slab_plan(s, spec.r_cut, r, world, mode=mode, num_interactions=3), ev, spec.r_cut, ev.atomic_numbers)
        rk.build_edges()
        ranks.append(rk)
    rel, fabs = (1e-10, 1e-9) if dtype == "float64" else (1e-4, 1e-3)
    for _ in range(2):
        energy, virial, owned = evaluate_decomposed(ranks)
        forces = np.zeros_like(f_ref)
        for rk, f in zip(ranks, owned):
            forces[rk.plan.own_global] = f.cpu().numpy()
        assert abs(energy - e_ref) <= rel * abs(e_ref)
        assert np.abs(forces - f_ref).max() <= fabs
        assert np.abs(virial - v_ref).max() <= 100 * rel * max(1.0, np.abs(v_ref).max())
