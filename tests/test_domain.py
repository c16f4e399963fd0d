"""Slab decomposition: plans, halo exchanges and multi-process runs, on CPU (numpy oracle as the per-rank
evaluator, gloo as the transport). The GPU/NCCL counterpart is in test_gpu_domain.py."""
import os
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

from symmetrix_b200 import structures as st
from symmetrix_b200.domain import SlabRank, evaluate_decomposed, make_slab_plan
from tests.oracle_backend import OracleBackend

GOLDEN = Path(__file__).resolve().parent / "golden"
R_CUT = 4.0   # cutoff of the tiny golden model


def _structure():
    return st.fcc_box((7, 2, 2), 3.6, [1, 8], seed=3, jitter=0.15)      # 25.2 A along the slab axis


def _single_domain():
    s = _structure()
    b = OracleBackend(GOLDEN / "tiny_model.json")
    nl = st.neighbor_list(s, R_CUT)
    inputs = st.evaluator_inputs(s, nl, b.atomic_numbers)
    e, f = b.o.compute_node_energies_forces(inputs)
    forces, virial = st.atom_forces_and_virial(inputs, nl, f)
    return s, e.sum(), forces, virial


@pytest.mark.parametrize("mode", ["message_passing", "recompute"])
def test_plans_are_consistent_between_ranks(mode):
    s = _structure()
    shell = R_CUT if mode == "message_passing" else 2 * R_CUT
    for world in (2, 3, 4, 6):
        plans = [make_slab_plan(s, R_CUT, r, world, mode=mode) for r in range(world)]
        assert sum(p.n_own for p in plans) == s.num_atoms
        assert np.array_equal(np.sort(np.concatenate([p.own_global for p in plans])), np.arange(s.num_atoms))
        for p in plans:
            for q in p.peers:
                # what q sends me is exactly my ghost rows owned by q, in the same order
                sent_global = plans[q].own_global[plans[q].send_rows[p.rank]]
                mine = p.ghost_global[p.recv_rows[q] - p.n_own]
                assert np.array_equal(sent_global, mine)
            # ghost images sit inside the shell around the slab
            x = p.positions[p.n_own:, 0]
            w = s.cell[0, 0] / world
            assert np.all((x >= 0) & (x < w + 2 * shell))
            assert np.all((p.positions[:p.n_own, 0] >= shell - 1e-9) & (p.positions[:p.n_own, 0] < shell + w + 1e-9))
            if mode == "recompute":
                # the ghosts within r_cut of the slab come first: they are receivers of layer 0
                near = (x >= shell - R_CUT) & (x < shell + w + R_CUT)
                assert np.all(near[:p.n_inner]) and not np.any(near[p.n_inner:])


def test_plan_rejects_slabs_thinner_than_the_cutoff():
    s = _structure()
    with pytest.raises(ValueError):
        make_slab_plan(s, R_CUT, 0, 7)


@pytest.mark.parametrize("mode", ["message_passing", "recompute"])
@pytest.mark.parametrize("world", [1, 2, 3, 5])
def test_decomposed_evaluation_equals_single_domain(world, mode):
    s, e_ref, f_ref, v_ref = _single_domain()
    ranks = []
    for r in range(world):
        b = OracleBackend(GOLDEN / "tiny_model.json")
        rk = SlabRank(make_slab_plan(s, R_CUT, r, world, mode=mode), b, R_CUT, b.atomic_numbers)
        rk.build_edges()
        ranks.append(rk)
    for _ in range(2):   # a second evaluation on the same edge sets must give the same answer
        energy, virial, owned = evaluate_decomposed(ranks)
        forces = np.zeros_like(f_ref)
        for rk, f in zip(ranks, owned):
            forces[rk.plan.own_global] = f.numpy()
        assert abs(energy - e_ref) < 1e-11 * abs(e_ref)
        np.testing.assert_allclose(forces, f_ref, atol=1e-11)
        np.testing.assert_allclose(virial, v_ref, atol=1e-10)


@pytest.mark.parametrize("mode", ["message_passing", "recompute"])
@pytest.mark.parametrize("world", [2, 3])
def test_zbl_and_density_normalised_model_decomposes(model_file, world, mode):
    """Pair repulsion and density-normalised blocks in a decomposed run: compute_ZBL on the owned atoms and the
    *_scaled stages where the pair style has them (pair_symmetrix_mace.cpp:449-494, 667-697)."""
    path, model, spec = model_file("tiny", zbl=True, density=True)
    s = st.fcc_box((7, 2, 2), 3.2, model["atomic_numbers"], seed=5, jitter=0.25)      # some pairs inside the ZBL envelope
    b0 = OracleBackend(model)
    assert b0.has_zbl
    nl = st.neighbor_list(s, spec.r_cut)
    inputs = st.evaluator_inputs(s, nl, b0.atomic_numbers)
    e, f = b0.o.compute_node_energies_forces(inputs)
    f_ref, v_ref = st.atom_forces_and_virial(inputs, nl, f)
    ranks = []
    for r in range(world):
        b = OracleBackend(model)
        rk = SlabRank(make_slab_plan(s, spec.r_cut, r, world, mode=mode), b, spec.r_cut, b.atomic_numbers)
        rk.build_edges()
        ranks.append(rk)
    energy, virial, owned = evaluate_decomposed(ranks)
    forces = np.zeros_like(f_ref)
    for rk, fo in zip(ranks, owned):
        forces[rk.plan.own_global] = fo.numpy()
    assert abs(energy - e.sum()) < 1e-11 * abs(e.sum())
    np.testing.assert_allclose(forces, f_ref, atol=1e-10)
    np.testing.assert_allclose(virial, v_ref, atol=1e-9)


def _gloo_worker(rank, world, port, out_dir, mode="message_passing"):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    import torch.distributed as dist
    dist.init_process_group("gloo", rank=rank, world_size=world)
    s = _structure()
    b = OracleBackend(GOLDEN / "tiny_model.json")
    rk = SlabRank(make_slab_plan(s, R_CUT, rank, world, mode=mode), b, R_CUT, b.atomic_numbers)
    rk.build_edges()
    energy, virial, owned = evaluate_decomposed([rk], dist=dist)
    np.savez(Path(out_dir) / f"rank{rank}.npz", energy=energy, virial=virial, forces=owned[0].numpy(), own=rk.plan.own_global)
    dist.barrier()
    dist.destroy_process_group()


@pytest.mark.parametrize("world,mode", [(2, "message_passing"), (3, "message_passing"), (2, "recompute")])
def test_decomposed_evaluation_over_gloo(world, mode, tmp_path):
    import torch.multiprocessing as mp
    s, e_ref, f_ref, v_ref = _single_domain()
    port = 29500 + (os.getpid() % 2000) + world + (10 if mode == "recompute" else 0)
    mp.spawn(_gloo_worker, args=(world, port, str(tmp_path), mode), nprocs=world, join=True)
    forces = np.zeros_like(f_ref)
    for r in range(world):
        d = np.load(tmp_path / f"rank{r}.npz")
        forces[d["own"]] = d["forces"]
        assert abs(float(d["energy"]) - e_ref) < 1e-11 * abs(e_ref)      # every rank holds the reduced total
        np.testing.assert_allclose(d["virial"], v_ref, atol=1e-10)
    np.testing.assert_allclose(forces, f_ref, atol=1e-11)


# ------------------------------------------------------------------------------------------------ three blocks
def _deep_structure(numbers):
    return st.fcc_box((10, 2, 2), 3.6, numbers, seed=4, jitter=0.15)      # 36 A along the slab axis, r_cut 5 A


@pytest.mark.parametrize("mode", ["message_passing", "recompute"])
@pytest.mark.parametrize("world", [2, 3])
def test_three_block_model_decomposes_in_both_modes(model_file, world, mode):
    """Two feature exchanges each way (H1, Hm) in message-passing mode; a 3 r_cut shell with three receiver sets in
    recompute mode. Checked against the single-domain evaluation of the same (numpy) evaluator."""
    if mode == "recompute" and world == 3:
        pytest.skip("a 15 A shell on both sides needs slabs the 36 A box cannot give three ranks")
    path, model, spec = model_file("deep256", num_channels=4, num_spline_points=24, radial_mlp=(8, 8))
    s = _deep_structure(model["atomic_numbers"])
    b0 = OracleBackend(model)
    nl = st.neighbor_list(s, spec.r_cut)
    inputs = st.evaluator_inputs(s, nl, b0.atomic_numbers)
    e, f = b0.o.compute_node_energies_forces(inputs)
    f_ref, v_ref = st.atom_forces_and_virial(inputs, nl, f)
    ranks = []
    for r in range(world):
        b = OracleBackend(model)
        rk = SlabRank(make_slab_plan(s, spec.r_cut, r, world, mode=mode, num_interactions=3), b, spec.r_cut, b.atomic_numbers)
        rk.build_edges()
        ranks.append(rk)
    energy, virial, owned = evaluate_decomposed(ranks)
    forces = np.zeros_like(f_ref)
    for rk, fo in zip(ranks, owned):
        forces[rk.plan.own_global] = fo.numpy()
    assert abs(energy - e.sum()) < 1e-11 * abs(e.sum())
    np.testing.assert_allclose(forces, f_ref, atol=1e-11)
    np.testing.assert_allclose(virial, v_ref, atol=1e-10)


# ------------------------------------------------------------------------------------------------ a rank that leaves
def _leaving_worker(rank, world, port, out_dir):
    """Rank 1 leaves between two steps (no exchange in flight); rank 0 must learn of it as an error from its next halo
    exchange within the process-group timeout, not hang."""
    import datetime
    import time
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), RANK=str(rank), WORLD_SIZE=str(world))
    import torch.distributed as dist
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=8))
    s = _structure()
    b = OracleBackend(GOLDEN / "tiny_model.json")
    rk = SlabRank(make_slab_plan(s, R_CUT, rank, world), b, R_CUT, b.atomic_numbers)
    rk.build_edges()
    evaluate_decomposed([rk], dist=dist)          # one complete step with both ranks
    if rank == 1:
        os._exit(0)                               # gone before the next step starts
    t0 = time.time()
    outcome = "no error"
    try:
        evaluate_decomposed([rk], dist=dist)
    except Exception as exc:                      # gloo reports the closed connection or the timeout
        outcome = type(exc).__name__
    (Path(out_dir) / "rank0.txt").write_text(f"{outcome} {time.time() - t0:.1f}")
    os._exit(0)


def test_a_rank_leaving_between_steps_ends_the_next_exchange_with_an_error(tmp_path):
    import torch.multiprocessing as mp
    port = 29500 + (os.getpid() % 2000) + 37
    mp.spawn(_leaving_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    outcome, seconds = (tmp_path / "rank0.txt").read_text().split()
    assert outcome != "no" and float(seconds) < 60.0, (outcome, seconds)
