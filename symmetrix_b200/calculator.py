"""Calculator with the behaviour of the reference's ASE calculator ``Symmetrix``
(symmetrix/source/symmetrix/symmetrix_calc.py:23-102), without depending on ASE: it takes
positions, cell, atomic numbers and periodicity directly and returns the same results
dictionary (``energy``, ``free_energy``, ``energies``, ``forces``, ``stress`` in Voigt order
xx, yy, zz, yz, xz, xy). Neighbour list, evaluation and force/virial reduction all run on the GPU.
"""
from __future__ import annotations

import numpy as np

from .mace import MACE


class Symmetrix:
    implemented_properties = ["energy", "free_energy", "energies", "forces", "stress"]

    def __init__(self, model_file, dtype: str = "float64", device: int = 0):
        if dtype not in ["float32", "float64"]:
            raise ValueError(f"Unsupported dtype '{dtype}'. Supported dtypes are 'float64' and 'float32'.")
        self.evaluator = MACE(str(model_file), dtype=dtype, device=device)
        self.cutoff = self.evaluator.r_cut
        self.results: dict = {}
        # atomic number -> node type of the model (-1: the model has no such element)
        self._type_of = np.full(128, -1, dtype=np.int32)
        for t, z in enumerate(self.evaluator.atomic_numbers):
            self._type_of[int(z)] = t

    def calculate(self, positions, cell, numbers, pbc=(True, True, True)) -> dict:
        z = np.asarray(numbers, dtype=np.int64)
        if z.size and (z.min() < 0 or z.max() >= self._type_of.size):
            raise ValueError("structure contains an element the model has no type for")
        types = self._type_of[z]
        if (types < 0).any():
            raise ValueError("structure contains an element the model has no type for")
        cell = np.asarray(cell, dtype=np.float64).reshape(3, 3)
        self.evaluator.build_neighbors(positions, types, cell, pbc)
        self.evaluator.compute_current()
        forces, virial, energy = self.evaluator.reduce_forces()
        volume = abs(np.linalg.det(cell))
        vxx, vyy, vzz, vxy, vxz, vyz = virial
        self.results = {
            "energy": energy, "free_energy": energy,
            "energies": self.evaluator.node_energies[: len(types)],
            "forces": forces,
            # stress = -(pair_forces^T xyz) / V in Voigt order (symmetrix_calc.py:100-102)
            "stress": -np.array([vxx, vyy, vzz, vyz, vxz, vxy]) / volume,
        }
        return self.results
