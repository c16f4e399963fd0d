"""The oracle against the committed golden vectors (which came from the reference's own CPU
evaluator, see tests/golden/make_golden.py) and, where present, against that evaluator itself."""
import json
from pathlib import Path

import numpy as np
import pytest

from oracle import ref as ref_driver
from oracle.mace_numpy import MaceOracle, real_sh_with_grad
from symmetrix_b200 import structures as st
from symmetrix_b200.modelgen.harmonics import random_rotation

GOLDEN = Path(__file__).resolve().parent / "golden"
INPUT_KEYS = ["num_nodes", "node_types", "num_neigh", "neigh_indices", "neigh_types", "xyz", "r"]
STAGES = ["Y", "Y_grad", "A0", "M0", "H1", "Phi1", "A1", "M1", "H2", "H2_adj", "M1_adj", "A1_adj", "H1_adj", "M0_adj", "A0_adj"]


@pytest.fixture(scope="module")
def tiny():
    case = np.load(GOLDEN / "tiny_case.npz")
    return case, {k: case[k] for k in INPUT_KEYS}


def test_port_matches_golden_tiny_stagewise(tiny):
    case, inputs = tiny
    o = MaceOracle(GOLDEN / "tiny_model.json")
    e, f = o.compute_node_energies_forces(inputs)
    np.testing.assert_allclose(e, case["node_energies"], rtol=1e-12, atol=1e-13)
    np.testing.assert_allclose(f, case["node_forces"], rtol=1e-11, atol=1e-13)
    for name in STAGES:
        got = getattr(o, name).reshape(-1)
        want = case["stage_" + name]
        assert got.size == want.size, name
        np.testing.assert_allclose(got, want, rtol=1e-11, atol=1e-12, err_msg=name)
    np.testing.assert_allclose(o.dPhi1.reshape(-1), case["stage_Phi1_adj"], rtol=1e-11, atol=1e-12)


def test_port_matches_golden_water64(model_file):
    from tests.golden.make_golden import model_checksum

    path, model, spec = model_file("water64")
    gold = np.load(GOLDEN / "water64_case.npz")
    assert model_checksum(model) == str(gold["model_sha256"]), "model generator drifted from the golden fixture"
    s = st.water_box(4, 12.42, seed=0)
    np.testing.assert_array_equal(s.positions, gold["positions"])
    nl = st.neighbor_list(s, spec.r_cut)
    assert nl["i"].size == int(gold["num_edges"])
    inputs = st.evaluator_inputs(s, nl, model["atomic_numbers"])
    o = MaceOracle(model)
    e, f = o.compute_node_energies_forces(inputs)
    forces, virial = st.atom_forces_and_virial(inputs, nl, f)
    np.testing.assert_allclose(e, gold["node_energies"], rtol=1e-11)
    np.testing.assert_allclose(forces, gold["atom_forces"], rtol=1e-9, atol=1e-11)
    np.testing.assert_allclose(virial, gold["virial"], rtol=1e-9, atol=1e-10)
    sums = np.array([getattr(o, n).sum() for n in ["A0", "M0", "H1", "Phi1", "A1", "M1", "H2"]])
    np.testing.assert_allclose(sums, gold["stage_sums"], rtol=1e-9, atol=1e-9)


@pytest.mark.skipif(not ref_driver.available(), reason="oracle/_ref not built (needs the reference checkout)")
def test_compiled_reference_matches_golden(tiny):
    case, inputs = tiny
    r = ref_driver.ReferenceMACE(GOLDEN / "tiny_model.json")
    e, f = r.compute_node_energies_forces(inputs)
    np.testing.assert_array_equal(e, case["node_energies"])
    np.testing.assert_array_equal(f, case["node_forces"])


@pytest.mark.skipif(not ref_driver.available(), reason="oracle/_ref not built (needs the reference checkout)")
def test_harmonics_match_reference_closed_form():
    """Pins the sphericart restatement to the reference's own closed form (spherical_harmonic.cpp:28-43)."""
    rng = np.random.default_rng(3)
    v = rng.standard_normal((5, 3))
    y, _ = real_sh_with_grad(3, v)
    for p in range(5):
        for l in range(4):
            for m in range(-l, l + 1):
                # evaluator convention: 2 sqrt(pi) * S_lm of the shuffled vector (z, x, y)
                want = 2 * np.sqrt(np.pi) * ref_driver.real_sph_harm_xyz(l, m, v[p, 2], v[p, 0], v[p, 1])
                assert abs(want - y[p, l * l + l + m]) < 1e-13


def test_harmonic_gradients_by_finite_differences():
    rng = np.random.default_rng(4)
    v = rng.standard_normal((4, 3)) * 2.0
    _, g = real_sh_with_grad(3, v)
    h = 1e-6
    for c in range(3):
        dv = np.zeros_like(v); dv[:, c] = h
        yp, _ = real_sh_with_grad(3, v + dv)
        ym, _ = real_sh_with_grad(3, v - dv)
        np.testing.assert_allclose(g[:, c, :], (yp - ym) / (2 * h), atol=1e-8)


def test_port_forces_are_energy_gradients(tiny):
    """Central differences on edge vectors, as the reference tests do (test_mace.py:73-84, 682-704)."""
    _, inputs = tiny
    o = MaceOracle(GOLDEN / "tiny_model.json")
    _, f = o.compute_node_energies_forces(inputs)
    f = f.reshape(-1, 3)
    xyz = inputs["xyz"].reshape(-1, 3).copy()
    h = 1e-5
    rng = np.random.default_rng(0)
    for e in rng.choice(xyz.shape[0], size=6, replace=False):
        for c in range(3):
            vals = []
            for sgn in (+1, -1):
                x2 = xyz.copy(); x2[e, c] += sgn * h
                inp = dict(inputs); inp["xyz"] = x2.reshape(-1); inp["r"] = np.linalg.norm(x2, axis=1)
                en, _ = o.compute_node_energies_forces(inp)
                vals.append(en.sum())
            assert abs(-(vals[0] - vals[1]) / (2 * h) - f[e, c]) < 1e-6 * max(1.0, abs(f[e, c]))


def test_energy_is_rotation_invariant(tiny):
    _, inputs = tiny
    o = MaceOracle(GOLDEN / "tiny_model.json")
    e0, f0 = o.compute_node_energies_forces(inputs)
    rot = random_rotation(np.random.default_rng(9))
    inp = dict(inputs); inp["xyz"] = (inputs["xyz"].reshape(-1, 3) @ rot.T).reshape(-1)
    e1, f1 = o.compute_node_energies_forces(inp)
    np.testing.assert_allclose(e1, e0, rtol=1e-11, atol=1e-12)
    np.testing.assert_allclose(f1.reshape(-1, 3), f0.reshape(-1, 3) @ rot.T, atol=1e-11)


def test_periodic_copies_repeat_the_cell_answer():
    """The property the full-size GPU tests rest on, here with the CPU restatement: a structure made of periodic copies
    of a cell has the cell's per-atom energies and forces, copy by copy (`structures.replicate`)."""
    o = MaceOracle(GOLDEN / "tiny_model.json")
    numbers = json.loads((GOLDEN / "tiny_model.json").read_text())["atomic_numbers"]
    cell = st.water_box(2, 7.0, seed=3)

    def run(s):
        nl = st.neighbor_list(s, o.r_cut)
        inputs = st.evaluator_inputs(s, nl, numbers)
        e, nf = o.compute_node_energies_forces(inputs)
        return e, st.atom_forces_and_virial(inputs, nl, nf)[0]

    e0, f0 = run(cell)
    e1, f1 = run(st.replicate(cell, (2, 1, 3)))
    np.testing.assert_allclose(e1.reshape(6, -1), np.broadcast_to(e0, (6, e0.size)), rtol=1e-11, atol=1e-12)
    np.testing.assert_allclose(f1.reshape(6, -1, 3), np.broadcast_to(f0, (6,) + f0.shape), atol=1e-10)


@pytest.mark.skipif(not ref_driver.available(), reason="oracle/_ref not built (needs the reference checkout)")
def test_port_matches_compiled_reference_with_zbl_and_density_normalisation(model_file):
    path, model, spec = model_file("tiny", zbl=True, density=True)
    s = st.water_box(2, 8.0, seed=3)
    nl = st.neighbor_list(s, spec.r_cut)
    inputs = st.evaluator_inputs(s, nl, model["atomic_numbers"])
    e_ref, f_ref = ref_driver.ReferenceMACE(path).compute_node_energies_forces(inputs)
    e, f = MaceOracle(model).compute_node_energies_forces(inputs)
    np.testing.assert_allclose(e, e_ref, rtol=1e-12, atol=1e-13)
    np.testing.assert_allclose(f, f_ref, rtol=1e-10, atol=1e-12)
    plain_path, plain_model, _ = model_file("tiny")
    e_plain, _ = MaceOracle(plain_model).compute_node_energies_forces(inputs)
    assert abs(e.sum() - e_plain.sum()) > 1.0      # the two extra terms are not negligible in this test


def test_port_forces_with_zbl_and_density_are_energy_gradients(model_file):
    path, model, spec = model_file("tiny", zbl=True, density=True)
    s = st.water_box(2, 8.0, seed=3)
    nl = st.neighbor_list(s, spec.r_cut)
    inputs = st.evaluator_inputs(s, nl, model["atomic_numbers"])
    o = MaceOracle(model)
    _, f = o.compute_node_energies_forces(inputs)
    f = f.reshape(-1, 3)
    xyz = inputs["xyz"].reshape(-1, 3).copy()
    h = 1e-5
    for e in (3, 40, 77):
        for c in range(3):
            vals = []
            for sgn in (+1, -1):
                x2 = xyz.copy(); x2[e, c] += sgn * h
                inp = dict(inputs); inp["xyz"] = x2.reshape(-1); inp["r"] = np.linalg.norm(x2, axis=1)
                vals.append(o.compute_node_energies_forces(inp)[0].sum())
            assert abs(-(vals[0] - vals[1]) / (2 * h) - f[e, c]) < 2e-6 * max(1.0, abs(f[e, c]))


# ------------------------------------------------------------------------------------------------
# Three interaction blocks: no reference implementation exists (parity unpinned by the reference); the generalised
# restatement is checked by finite differences, rotation invariance and reduction to the two-block oracle.
# ------------------------------------------------------------------------------------------------
def _deep_case(model_file, channels=6):
    import copy
    from oracle.mace_numpy_deep import DeepMaceOracle
    path, model, spec = model_file("deep256", num_channels=channels, num_spline_points=32, radial_mlp=(8, 8))
    s = st.molecular_liquid(4, seed=3)
    nl = st.neighbor_list(s, spec.r_cut)
    inputs = st.evaluator_inputs(s, nl, model["atomic_numbers"])
    return copy, DeepMaceOracle, model, spec, s, nl, inputs


def test_three_block_oracle_forces_are_energy_gradients(model_file):
    copy, DeepMaceOracle, model, spec, s, nl, inputs = _deep_case(model_file)
    e, f = DeepMaceOracle(model).compute_node_energies_forces(inputs)
    forces, _ = st.atom_forces_and_virial(inputs, nl, f)
    h = 1e-5
    for atom, comp in [(0, 0), (5, 2), (11, 1)]:
        es = []
        for sign in (+1, -1):
            s2 = copy.deepcopy(s)
            s2.positions[atom, comp] += sign * h
            nl2 = st.neighbor_list(s2, spec.r_cut)
            es.append(DeepMaceOracle(model).compute_node_energies_forces(st.evaluator_inputs(s2, nl2, model["atomic_numbers"]))[0].sum())
        assert abs(-(es[0] - es[1]) / (2 * h) - forces[atom, comp]) < 1e-6 * max(1.0, np.abs(forces).max())


def test_three_block_oracle_is_rotation_invariant(model_file):
    copy, DeepMaceOracle, model, spec, s, nl, inputs = _deep_case(model_file)
    e, f = DeepMaceOracle(model).compute_node_energies_forces(inputs)
    rot = random_rotation(np.random.default_rng(1))
    s2 = copy.deepcopy(s)
    s2.positions = s.positions @ rot.T
    s2.cell = s.cell @ rot.T
    nl2 = st.neighbor_list(s2, spec.r_cut)
    e2, _ = DeepMaceOracle(model).compute_node_energies_forces(st.evaluator_inputs(s2, nl2, model["atomic_numbers"]))
    assert abs(e2.sum() - e.sum()) < 1e-11 * abs(e.sum())


def test_three_block_oracle_reduces_to_the_two_block_oracle(model_file):
    """With the middle block made the identity (no contraction term, residual = 1, no readout) the features that
    reach the last block are H1 and the model is the two-block model, which is pinned against the reference."""
    copy, DeepMaceOracle, model, spec, s, nl, inputs = _deep_case(model_file)
    K, nL, n_el = spec.num_channels, spec.L_max + 1, len(model["atomic_numbers"])
    ident = dict(model)
    ident["Hm_weights"] = np.zeros(nL * K * K)
    ident["Hm_weights_for_H1"] = np.tile(np.eye(K)[None, None], (n_el, nL, 1, 1)).ravel()
    ident["readout_m_weights"] = np.zeros(K)
    e3, f3 = DeepMaceOracle(ident).compute_node_energies_forces(inputs)
    two = dict(ident)
    two["num_interactions"] = 2
    e2, f2 = MaceOracle(two).compute_node_energies_forces(inputs)
    assert abs(e3.sum() - e2.sum()) < 1e-12 * abs(e2.sum())
    np.testing.assert_allclose(f3, f2, atol=1e-12)
