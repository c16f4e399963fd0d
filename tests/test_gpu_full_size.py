"""The benchmark configurations at their stated sizes, through a property that does not depend on the size: a periodic
structure made of copies of a small cell has, atom by atom, the energies and forces of that cell. The small cell is one
the reference's CPU evaluator (class MACE compiled unmodified into oracle/_ref) has answered -- the committed answers under
tests/golden/ -- so the large evaluation is compared with the reference's own numbers:

* configs[3], per-GPU share: 256,000 atoms (10 x 80 x 80 FCC cells), float32, copies of the 4,000-atom case;
* configs[1] model in float64 on 32,000 atoms (1e-10);
* configs[2]: 98,304-atom water box at 1.0 g/cm^3, float32, copies of a 1,536-atom box of the same construction;
* configs[4], per-GPU share: 62,784 atoms of the molecular liquid, three-block 256x0e+256x1o+256x2e model, float32, against
  the float64 evaluation of the 981-atom cell by this library (the reference has no three-block evaluator).

Neighbour lists are built on the GPU (`smx_build_neighbors`). All tests need a GPU."""
import hashlib
from pathlib import Path

import numpy as np
import pytest

import bench
from symmetrix_b200 import Symmetrix, structures as st

pytestmark = pytest.mark.gpu


def _evaluate(path, s, dtype):
    calc = Symmetrix(path, dtype=dtype)
    res = calc.calculate(s.positions, s.cell, s.numbers, s.pbc)
    out = {k: np.array(v, copy=True) for k, v in res.items()}
    del calc
    return out


def _compare(res, copies, e_cell, f_cell, rel, f_abs):
    n = e_cell.size
    e = res["energies"].reshape(copies, n)
    f = res["forces"].reshape(copies, n, 3)
    assert abs(res["energy"] - copies * e_cell.sum()) <= rel * abs(copies * e_cell.sum())
    assert np.abs(e - e_cell[None]).max() <= 10 * rel * np.abs(e_cell).max()
    assert np.abs(f - f_cell[None]).max() <= f_abs
    # the copies must also agree with one another far better than with the cell (same arithmetic, other rows)
    assert np.abs(f - f[0][None]).max() <= f_abs


@pytest.fixture(scope="module")
def fcc4000_gold():
    path, spec, s, nl, inputs = bench.build_inputs("fcc4000", seed=1)
    gold = np.load(Path(__file__).resolve().parent / "golden" / "fcc4000_case.npz")
    return path, s, gold


def test_configs3_share_of_256000_atoms_repeats_the_reference_answer(fcc4000_gold):
    path, s, gold = fcc4000_gold
    big = st.replicate(s, (1, 8, 8))
    assert big.num_atoms == 256_000 and np.allclose(np.diag(big.cell), [36.0, 288.0, 288.0])
    res = _evaluate(path, big, "float32")
    _compare(res, 64, gold["node_energies"], gold["atom_forces"], rel=1e-4, f_abs=1e-3)


def test_configs1_model_float64_on_32000_atoms_repeats_the_reference_answer(fcc4000_gold):
    path, s, gold = fcc4000_gold
    big = st.replicate(s, (2, 2, 2))
    res = _evaluate(path, big, "float64")
    f_ref = gold["atom_forces"]
    _compare(res, 8, gold["node_energies"], f_ref, rel=1e-10, f_abs=1e-9 * max(1.0, np.abs(f_ref).max()))


def test_configs2_water_box_of_98304_atoms_repeats_the_reference_answer():
    """The cell's reference answer is committed (tests/golden/water1536_case.npz, made by make_golden_bench.py)."""
    path, numbers, spec = bench.model_path("organic128_HO")
    cell = st.water_box_density(8, 1.0, seed=5)
    assert cell.num_atoms == 1536
    nl = st.neighbor_list(cell, spec.r_cut)
    inputs = st.evaluator_inputs(cell, nl, numbers)
    gold = np.load(Path(__file__).resolve().parent / "golden" / "water1536_case.npz")
    h = hashlib.sha256()
    for key in ["node_types", "num_neigh", "neigh_indices", "neigh_types", "xyz", "r"]:
        h.update(np.ascontiguousarray(inputs[key]).tobytes())
    assert h.hexdigest() == str(gold["inputs_sha256"]), "the water cell is not the one the golden answer was made for"
    e_ref, f_ref = gold["node_energies"], gold["atom_forces"]
    big = st.replicate(cell, (4, 4, 4))
    assert big.num_atoms == 98_304
    res = _evaluate(path, big, "float32")
    _compare(res, 64, e_ref, f_ref, rel=1e-4, f_abs=1e-3)
    small = _evaluate(path, cell, "float64")
    _compare(small, 1, e_ref, f_ref, rel=1e-10, f_abs=1e-9 * max(1.0, np.abs(f_ref).max()))


def test_configs4_share_of_62784_atoms_repeats_its_cell():
    path, numbers, spec = bench.model_path("deep256")
    cell = st.molecular_liquid(109, 0.79, seed=4)
    assert cell.num_atoms == 981
    small = _evaluate(path, cell, "float64")
    big = st.replicate(cell, (4, 4, 4))
    assert big.num_atoms == 62_784
    res = _evaluate(path, big, "float32")
    _compare(res, 64, small["energies"], small["forces"], rel=1e-4, f_abs=1e-3)
