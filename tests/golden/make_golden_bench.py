"""Generates ``fcc4000_case.npz`` and ``water1536_case.npz``: the reference's answers for the exact inputs ``bench.py``
times by default and for the 1,536-atom water cell whose 64 copies make the 98,304-atom box of configs[2].

The reference's own CPU evaluator (``oracle/_ref/libref_parity.so``: class MACE compiled unmodified, -O2, no fast-math)
is run here on the configs[1] benchmark case -- model file of ``bench.model_path("fcc128")`` (K = 128, 256 spline points,
5 species), structure of ``bench.build_inputs("fcc4000", seed=1)`` (4,000 atoms, 311,946 edges) -- which takes minutes
and about 20 GB on one core, too long to repeat inside the GPU test run. Stored: per-node energies, per-atom forces,
virial, and SHA-256 digests of the input arrays so that the test can tell whether it evaluates the same inputs.

``water1536_case.npz``: model file of ``bench.model_path("organic128_HO")``, structure ``water_box_density(8, 1.0, seed=5)``
(82,984 edges; 45 s and 6 GB).

    python tests/golden/make_golden_bench.py [fcc4000] [water1536]
"""
import hashlib
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[2]
sys.path.insert(0, str(ROOT))

import bench  # noqa: E402
from oracle import ref  # noqa: E402
from symmetrix_b200 import structures as st  # noqa: E402


def digest(inputs) -> str:
    h = hashlib.sha256()
    for key in ["node_types", "num_neigh", "neigh_indices", "neigh_types", "xyz", "r"]:
        h.update(np.ascontiguousarray(inputs[key]).tobytes())
    return h.hexdigest()


def water1536_inputs():
    path, numbers, spec = bench.model_path("organic128_HO")
    s = st.water_box_density(8, 1.0, seed=5)
    nl = st.neighbor_list(s, spec.r_cut)
    return path, s, nl, st.evaluator_inputs(s, nl, numbers)


def main(cases):
    for case in cases:
        if case == "fcc4000":
            path, spec, s, nl, inputs = bench.build_inputs("fcc4000", seed=1)
        else:
            path, s, nl, inputs = water1536_inputs()
        r = ref.ReferenceMACE(path, "parity")
        e, f = r.compute_node_energies_forces(inputs)
        forces, virial = st.atom_forces_and_virial(inputs, nl, f)
        out = Path(__file__).resolve().parent / f"{case}_case.npz"
        np.savez_compressed(out, node_energies=e, atom_forces=forces, virial=virial, energy=e.sum(),
                            inputs_sha256=np.array(digest(inputs)), num_edges=np.array(inputs["r"].size))
        print(f"wrote {out}: E = {e.sum():.12f}, {s.num_atoms} atoms, {inputs['r'].size} edges")


if __name__ == "__main__":
    main(sys.argv[1:] or ["fcc4000", "water1536"])
