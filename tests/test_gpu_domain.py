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
def test_emulated_ranks_on_one_gpu_match_single_domain(model_file, dtype, world, mode, extra=None):
    path, model, spec = model_file("fcc128", num_channels=32, num_spline_points=32, **(extra or {}))
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


@pytest.mark.parametrize("mode", ["message_passing", "recompute"])
def test_degree_three_features_decompose_on_gpu(model_file, mode):
    """Halo rows of 16 feature components (L_max = 3)."""
    test_emulated_ranks_on_one_gpu_match_single_domain(model_file, "float64", 2, mode, extra={"L_max": 3})


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


def test_kept_groupings_of_unpack_add_lists(model_file):
    """smx_halo_cache_lists: the grouping of an unpack-add index list is reused while the list stays at its address, gives
    the same bits as a fresh grouping, and is dropped on request (here: before the list is rewritten in place)."""
    import torch
    path, model, spec = model_file("fcc128", num_channels=32, num_spline_points=32)
    s = st.fcc_box(3, 3.6, model["atomic_numbers"], seed=4)
    ev = MACE(path, dtype="float64")
    nl = st.neighbor_list(s, ev.r_cut)
    inp = st.evaluator_inputs(s, nl, ev.atomic_numbers)
    ev.compute_node_energies_forces(inp["num_nodes"], inp["node_types"], inp["num_neigh"], inp["neigh_indices"], inp["neigh_types"],
                                    inp["xyz"], inp["r"])
    ev.atom_forces(s.num_atoms)
    ev.use_torch_stream(True)          # the tensor operations below and the evaluator's kernels in one stream order
    rng = np.random.default_rng(0)
    dev = f"cuda:{ev.info.device}"
    rows = torch.as_tensor(rng.integers(0, s.num_atoms, size=500).astype(np.int32), device=dev)      # rows repeat
    buf = torch.as_tensor(rng.normal(size=(500, 3)), device=dev)

    def apply(n_times):
        base = ev.device_view("atom_forces").view(-1, 3)[: s.num_atoms]
        start = base.clone()
        for _ in range(n_times):
            ev.halo_unpack("atom_forces", rows, buf, add=True)
        out = base.clone()
        base.copy_(start)
        return start.cpu().numpy(), out.cpu().numpy()

    launches0 = ev.launch_count
    start, plain = apply(2)
    per_call = (ev.launch_count - launches0) // 2
    ev.halo_cache_lists(True)
    launches0 = ev.launch_count
    _, kept = apply(2)
    assert np.array_equal(kept, plain)
    assert ev.launch_count - launches0 < 2 * per_call            # the second call skipped the sort
    expect = start.copy()
    for _ in range(2):
        np.add.at(expect, rows.cpu().numpy(), buf.cpu().numpy())
    np.testing.assert_allclose(kept, expect, rtol=0, atol=1e-12)
    # rewrite the list in place: drop the kept grouping first
    ev.halo_cache_lists(False)
    rows.copy_(torch.as_tensor(rng.integers(0, s.num_atoms, size=500).astype(np.int32), device=dev))
    ev.halo_cache_lists(True)
    start, again = apply(1)
    expect = start.copy()
    np.add.at(expect, rows.cpu().numpy(), buf.cpu().numpy())
    np.testing.assert_allclose(again, expect, rtol=0, atol=1e-12)


def _write_vec(f, a, dt):
    a = np.ascontiguousarray(a, dtype=dt).reshape(-1)
    f.write(np.int64(a.size).tobytes()); f.write(a.tobytes())


@pytest.mark.parametrize("mode", ["message_passing", "recompute"])
@pytest.mark.parametrize("flags", [dict(), dict(zbl=True, density=True)])
def test_cpp_pair_style_harness_replays_both_decomposed_modes(model_file, tmp_path, mode, flags):
    """tests/pair_harness.cpp: the stage sequences of the reference pair style's two decomposed compute() modes
    (pair_symmetrix_mace.cpp:436-495 and :551-748), with the reference's argument lists, against the C++ facade, for all
    ranks of a 3-slab decomposition; forward_comm / reverse_comm are played on the host vectors. Energy and forces must
    equal the single-domain evaluation."""
    root = Path(__file__).resolve().parents[1]
    pkg = root / "symmetrix_b200"
    exe = tmp_path / "pair_harness"
    subprocess.run(["g++", "-std=c++20", "-O1", f"-I{root / 'include'}", str(root / "tests" / "pair_harness.cpp"), "-o", str(exe),
                    f"-L{pkg}", "-lsymmetrix_b200", f"-Wl,-rpath,{pkg}"], check=True)
    world = 3
    path, model, spec = model_file("fcc128", num_channels=32, num_spline_points=32, **flags)
    a0 = 3.2 if flags else 3.6
    s = st.fcc_box((4 * world, 3, 3), a0, model["atomic_numbers"], seed=13, jitter=0.2 if flags else 0.12)
    f_ref, v_ref, e_ref = _single(path, s)
    zmap = {int(z): t for t, z in enumerate(model["atomic_numbers"])}
    plans = [make_slab_plan(s, spec.r_cut, r, world, mode=mode) for r in range(world)]
    for plan in plans:
        local = st.Structure(plan.positions, plan.cell, plan.numbers, plan.pbc)
        nl = st.neighbor_list(local, spec.r_cut)
        n_recv = plan.n_own + (plan.n_inner if mode == "recompute" else 0)
        types = np.array([zmap[int(z)] for z in plan.numbers], dtype=np.int32)
        num_neigh = np.bincount(nl["i"], minlength=local.num_atoms).astype(np.int32)[:n_recv]
        e_cnt = int(num_neigh.sum())
        with open(tmp_path / f"case{plan.rank}.bin", "wb") as f:
            _write_vec(f, [plan.n_own, plan.n_own + plan.n_ghost, n_recv, len(plan.peers)], np.int32)
            _write_vec(f, types[:n_recv], np.int32); _write_vec(f, num_neigh, np.int32)
            _write_vec(f, nl["j"][:e_cnt], np.int32); _write_vec(f, types[nl["j"][:e_cnt]], np.int32)
            _write_vec(f, nl["D"][:e_cnt], np.float64); _write_vec(f, nl["d"][:e_cnt], np.float64)
            for q in plan.peers:
                _write_vec(f, [q], np.int32); _write_vec(f, plan.send_rows[q], np.int32); _write_vec(f, plan.recv_rows[q], np.int32)
    subprocess.run([str(exe), str(path), "0" if mode == "message_passing" else "1", str(world), str(tmp_path / "case"),
                    str(tmp_path / "out")], check=True)
    energy, forces = 0.0, np.zeros_like(f_ref)
    for plan in plans:
        out = np.fromfile(tmp_path / f"out{plan.rank}.bin", dtype=np.float64)
        energy += out[0]
        forces[plan.own_global] = out[1:].reshape(-1, 3)
    assert abs(energy - e_ref) <= 1e-10 * abs(e_ref)
    assert np.abs(forces - f_ref).max() <= 1e-8 * max(1.0, np.abs(f_ref).max())


def _gpu_count():
    import torch
    return torch.cuda.device_count()


@pytest.mark.parametrize("dtype,mode,transport", [("float64", "message_passing", "torch"), ("float32", "message_passing", "torch"),
                                                  ("float64", "recompute", "torch"), ("float64", "message_passing", "library"),
                                                  ("float32", "message_passing", "library"), ("float64", "recompute", "library")])
def test_ranks_over_nccl_match_single_domain(model_file, dtype, mode, transport, tmp_path):
    world = min(_gpu_count(), 4)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    path, model, spec = model_file("fcc128", num_channels=32, num_spline_points=32)
    out = tmp_path / "dd.npz"
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={world}", "--master-addr", "127.0.0.1",
           "--master-port", str(29400 + os.getpid() % 500), str(ROOT / "tests" / "dd_nccl_worker.py"), str(path), dtype, str(out), mode, transport]
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
