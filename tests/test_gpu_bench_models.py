"""The model files and structures the benchmark runs, against the reference's own CPU evaluator (class MACE compiled
unmodified into oracle/_ref): configs[1] at its stated size (4,000-atom FCC box, the K = 128, 256-point model that bench.py
times) against the answer that evaluator gave for the same inputs (tests/golden/fcc4000_case.npz, made by
tests/golden/make_golden_bench.py: minutes and 20 GB on one core, so not repeated here), and the configs[2] / configs[3] /
L_max = 2 models at benchmark width on boxes the CPU evaluator finishes in seconds, run live. float64: 1e-10 relative;
float32: 1e-4 relative and 1e-3 eV/A. All tests need a GPU."""
import hashlib
from pathlib import Path

import numpy as np
import pytest

import bench
from oracle import ref as ref_driver
from symmetrix_b200 import MACE, structures as st

pytestmark = pytest.mark.gpu

TOL = {"float64": dict(rel=1e-10, f_abs=1e-9), "float32": dict(rel=1e-4, f_abs=1e-3)}


def _reference(path, inputs):
    if not ref_driver.available():
        pytest.skip("the compiled reference (oracle/_ref/libref_parity.so) is not here")
    r = ref_driver.ReferenceMACE(path)
    return r.compute_node_energies_forces(inputs)


def _check(dtype, path, inputs, e_ref, f_ref):
    ev = MACE(path, dtype=dtype)
    ev.compute_node_energies_forces(int(inputs["num_nodes"]), inputs["node_types"], inputs["num_neigh"], inputs["neigh_indices"],
                                    inputs["neigh_types"], inputs["xyz"], inputs["r"])
    e, f = ev.node_energies, ev.node_forces
    tol = TOL[dtype]
    assert abs(e.sum() - e_ref.sum()) <= tol["rel"] * abs(e_ref.sum())
    assert np.abs(e - e_ref).max() <= 10 * tol["rel"] * np.abs(e_ref).max()
    assert np.abs(f - f_ref).max() <= max(tol["f_abs"], 10 * tol["rel"] * np.abs(f_ref).max()) if dtype == "float64" else \
        np.abs(f - f_ref).max() <= tol["f_abs"]
    return ev


@pytest.fixture(scope="module")
def fcc4000():
    path, spec, s, nl, inputs = bench.build_inputs("fcc4000", seed=1)
    gold = np.load(Path(__file__).resolve().parent / "golden" / "fcc4000_case.npz")
    h = hashlib.sha256()
    for key in ["node_types", "num_neigh", "neigh_indices", "neigh_types", "xyz", "r"]:
        h.update(np.ascontiguousarray(inputs[key]).tobytes())
    assert h.hexdigest() == str(gold["inputs_sha256"]), "the benchmark structure is not the one the golden answer was made for"
    return path, s, inputs, gold


@pytest.mark.parametrize("dtype", ["float64", "float32"])
def test_configs1_benchmark_case_at_full_size(fcc4000, dtype):
    """Exactly what `bench.py` (default workload) evaluates: same model file, same 4,000-atom structure, same seed."""
    path, s, inputs, gold = fcc4000
    ev = MACE(path, dtype=dtype)
    ev.compute_node_energies_forces(int(inputs["num_nodes"]), inputs["node_types"], inputs["num_neigh"], inputs["neigh_indices"],
                                    inputs["neigh_types"], inputs["xyz"], inputs["r"])
    e = ev.node_energies
    forces, virial, energy = ev.reduce_forces()
    tol = TOL[dtype]
    e_ref, f_ref, v_ref = gold["node_energies"], gold["atom_forces"], gold["virial"]
    assert abs(energy - e_ref.sum()) <= tol["rel"] * abs(e_ref.sum())
    assert np.abs(e - e_ref).max() <= 10 * tol["rel"] * np.abs(e_ref).max()
    if dtype == "float64":
        assert np.abs(forces - f_ref).max() <= 10 * tol["rel"] * np.abs(f_ref).max()
    else:
        assert np.abs(forces - f_ref).max() <= tol["f_abs"]
    assert np.abs(virial - v_ref).max() <= 100 * tol["rel"] * max(1.0, np.abs(v_ref).max())


@pytest.mark.parametrize("dtype", ["float64", "float32"])
def test_configs2_benchmark_model_on_a_648_atom_water_box(dtype):
    """The organic-liquid model file of the 98,304-atom water benchmark (K = 128, r_cut 5 A, exported for H and O) on a
    box of the same construction and density that the CPU evaluator handles: 216 molecules."""
    path, numbers, spec = bench.model_path("organic128_HO")
    s = st.water_box_density(6, 1.0, seed=3)
    assert s.num_atoms == 648
    nl = st.neighbor_list(s, spec.r_cut)
    inputs = st.evaluator_inputs(s, nl, numbers)
    e_ref, f_ref = _reference(path, inputs)
    _check(dtype, path, inputs, e_ref, f_ref)


@pytest.mark.parametrize("dtype", ["float64", "float32"])
def test_lmax2_model_at_benchmark_width(model_file, dtype):
    """The 256x0e+256x1o+256x2e feature set (configs[4]'s irreps) as a two-block model, which the reference can run,
    at full channel width."""
    path, model, spec = model_file("large256", num_spline_points=64)
    s = st.molecular_liquid(30, seed=6)
    nl = st.neighbor_list(s, spec.r_cut)
    inputs = st.evaluator_inputs(s, nl, model["atomic_numbers"])
    e_ref, f_ref = _reference(path, inputs)
    _check(dtype, path, inputs, e_ref, f_ref)


@pytest.mark.parametrize("workload,builder", [
    ("water64", lambda z: st.water_box(4, 12.42, seed=0)),                   # configs[0] as stated: 192 atoms, 64x0e
    ("fcc128", lambda z: st.fcc_box(4, 3.6, z, seed=2)),                     # configs[1] model on a 256-atom box
])
@pytest.mark.parametrize("mode", ["mlp", "lowrank"])
def test_runtime_radial_network_mode_meets_the_float32_gates(monkeypatch, workload, builder, mode):
    """SMX_RADIAL=mlp: the radial functions of block 1 evaluated at run time from the un-splined network (Bessel functions
    x polynomial cutoff, hidden layers per edge, last layer as a tensor-core GEMM) instead of the spline tables that the
    reference's exporter makes of the same network (extract_mace_data.py:144-172). The two differ by the interpolation
    error of the 256-point splines and float32 rounding; gate: 1e-4 relative energy, 1e-3 eV/A, against the float64 spline
    path (which is pinned to the reference). SMX_RADIAL=lowrank uses the tabulated last hidden layer instead of the network's
    first layers: spline construction and the last layer are linear, so that form equals the spline tables to rounding."""
    path, numbers, spec = bench.model_path(workload)
    s = builder(numbers)
    nl = st.neighbor_list(s, spec.r_cut)
    inputs = st.evaluator_inputs(s, nl, numbers)

    def evaluate(dtype):
        ev = MACE(path, dtype=dtype)
        ev.compute_node_energies_forces(int(inputs["num_nodes"]), inputs["node_types"], inputs["num_neigh"], inputs["neigh_indices"],
                                        inputs["neigh_types"], inputs["xyz"], inputs["r"])
        return ev.node_energies, ev.node_forces

    e64, f64 = evaluate("float64")
    monkeypatch.setenv("SMX_RADIAL", mode)
    e_mlp, f_mlp = evaluate("float32")
    monkeypatch.delenv("SMX_RADIAL")
    assert abs(e_mlp.sum() - e64.sum()) <= 1e-4 * abs(e64.sum())
    assert np.abs(f_mlp - f64).max() <= 1e-3
    # and the mode is refused where it does not apply
    monkeypatch.setenv("SMX_RADIAL", mode)
    with pytest.raises(Exception):
        MACE(path, dtype="float64")
