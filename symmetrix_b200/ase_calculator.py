"""ASE calculator with the constructor and results of the reference's ``symmetrix.Symmetrix``
(symmetrix/source/symmetrix/symmetrix_calc.py:23-102), for installations that have ASE.

    from symmetrix_b200.ase_calculator import Symmetrix
    atoms.calc = Symmetrix("model.json", dtype="float64")

Differences from the reference class: the neighbour list is built on the GPU from the positions, cell and periodicity of
the ``Atoms`` object (``smx_build_neighbors``; the reference calls matscipy / ``ase.neighborlist``), the per-atom forces and
the virial are reduced on the GPU (the reference uses ``numpy.bincount`` on the pair forces), ``use_kokkos`` is accepted
and ignored (there is one, GPU, evaluator), and a model file that is not symmetrix JSON raises instead of being converted
(the converter needs mace-torch). ASE is imported when this module is; the package itself does not depend on it
(``symmetrix_b200.Symmetrix`` in ``calculator.py`` is the same calculator without the ASE base class).
"""
from __future__ import annotations

import numpy as np
from ase.calculators.calculator import Calculator, all_changes

from .calculator import Symmetrix as _ArrayCalculator


class Symmetrix(Calculator):
    implemented_properties = ["energy", "free_energy", "energies", "forces", "stress"]

    def __init__(self, model_file, dtype="float64", use_kokkos=True, device: int = 0, **kwargs):
        Calculator.__init__(self, **kwargs)
        self._impl = _ArrayCalculator(model_file, dtype=dtype, device=device)      # raises ValueError for an unsupported dtype
        self.use_kokkos = use_kokkos
        self.evaluator = self._impl.evaluator
        self.cutoff = self._impl.cutoff

    def calculate(self, atoms=None, properties=("energy",), system_changes=all_changes):
        Calculator.calculate(self, atoms, properties, system_changes)
        a = self.atoms
        out = self._impl.calculate(np.asarray(a.get_positions(), dtype=np.float64), np.asarray(a.get_cell(), dtype=np.float64),
                                   a.get_atomic_numbers(), tuple(bool(p) for p in a.get_pbc()))
        self.results.update(out)
