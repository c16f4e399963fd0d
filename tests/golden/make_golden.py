"""Regenerates the committed golden vectors from the reference's own CPU evaluator.

Run in a container that holds the reference checkout (it needs ``oracle/_ref``, built by
``oracle/build_ref.py``):  ``python tests/golden/make_golden.py``

Outputs (all small, committed):
* ``tiny_model.json``   a complete model file in the reference's schema (8 channels, 24 spline nodes)
* ``tiny_case.npz``     evaluator inputs for a 24-atom periodic water cell and the reference's outputs
                        for them: node energies, per-edge partial forces and every stage array
* ``water64_case.npz``  reference outputs for benchmark configuration 0 (192 atoms, 64x0e model); model and
                        structure are regenerated from their seeds, a checksum guards against generator drift
"""
import hashlib
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

from oracle.ref import ReferenceMACE  # noqa: E402
from symmetrix_b200 import structures as st  # noqa: E402
from symmetrix_b200.modelgen.generate import generate_model, named_spec, write_json  # noqa: E402

HERE = Path(__file__).resolve().parent
STAGES = ["Y", "Y_grad", "A0", "M0", "H1", "Phi1", "A1", "M1", "H2", "H2_adj", "M1_adj", "A1_adj",
          "Phi1_adj", "H1_adj", "M0_adj", "A0_adj"]


def model_checksum(model: dict) -> str:
    h = hashlib.sha256()
    for key in ["radial_spline_values_1", "A0_weights", "H1_weights", "Phi1_clebsch_gordan", "readout_2_weights_1"]:
        h.update(np.ascontiguousarray(np.asarray(model[key], dtype=np.float64)).tobytes())
    for a in sorted(model["M1_weights"]):
        h.update(np.ascontiguousarray(model["M1_weights"][a]).tobytes())
    return h.hexdigest()


def main():
    # --- tiny
    spec = named_spec("tiny")
    model = generate_model(spec)
    write_json(model, HERE / "tiny_model.json")
    s = st.water_box(2, 8.0, seed=3)
    nl = st.neighbor_list(s, spec.r_cut)
    inp = st.evaluator_inputs(s, nl, model["atomic_numbers"])
    ref = ReferenceMACE(HERE / "tiny_model.json")
    e, f = ref.compute_node_energies_forces(inp)
    out = {k: np.asarray(v) for k, v in inp.items()}
    out["node_energies"] = e
    out["node_forces"] = f
    for name in STAGES:
        out["stage_" + name] = ref.get(name)
    np.savez_compressed(HERE / "tiny_case.npz", **out)
    print("tiny: E =", e.sum(), "edges =", inp["r"].size)

    # --- configuration 0
    spec = named_spec("water64")
    model = generate_model(spec)
    path = Path("/tmp/water64_golden.json")
    write_json(model, path)
    s = st.water_box(4, 12.42, seed=0)
    nl = st.neighbor_list(s, spec.r_cut)
    inp = st.evaluator_inputs(s, nl, model["atomic_numbers"])
    ref = ReferenceMACE(path)
    e, f = ref.compute_node_energies_forces(inp)
    forces, virial = st.atom_forces_and_virial(inp, nl, f)
    np.savez_compressed(
        HERE / "water64_case.npz", node_energies=e, atom_forces=forces, virial=virial,
        num_edges=np.int64(inp["r"].size), positions=s.positions,
        model_sha256=np.array(model_checksum(model)),
        stage_sums=np.array([ref.get(n).sum() for n in ["A0", "M0", "H1", "Phi1", "A1", "M1", "H2"]]))
    print("water64: E =", e.sum(), "edges =", inp["r"].size, "|F|max =", np.abs(forces).max())


if __name__ == "__main__":
    main()
