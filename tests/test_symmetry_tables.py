"""Independent check of the symmetry tables the evaluator compiles in (CPU).

The coupling constants in csrc/generated/ (tensor-product code and cg_canon.hpp) come from
symmetrix_b200/modelgen/harmonics.py, which derives them numerically as the null space of the equivariance
constraint. Here the same tensors are built from an unrelated source -- the Clebsch-Gordan coefficients of
``sympy.physics.quantum.cg`` (complex spherical basis, Condon-Shortley phase) -- and carried into the real basis with
the relations the reference uses between its real and complex harmonics (libsymmetrix/source/spherical_harmonic.cpp:
45-55, 84-98):  S_l0 = Y_l^0,  S_{l,m>0} = sqrt2 (-1)^m Re Y_l^m,  S_{l,-m} = sqrt2 (-1)^m Im Y_l^m, i.e.
    S_{l, m} = ((-1)^m Y_l^m + Y_l^{-m}) / sqrt2,      S_{l,-m} = ((-1)^m Y_l^m - Y_l^{-m}) / (i sqrt2).
A model file may scale each path's coupling block freely (the loader folds the scale into the radial functions), so the
comparison is up to one factor per path."""
import numpy as np
import pytest

from symmetrix_b200.modelgen.gen_tp_code import tables
from symmetrix_b200.modelgen.generate import tp_paths
from symmetrix_b200.modelgen.harmonics import coupling


def real_from_complex(l: int) -> np.ndarray:
    """U with S_l = U Y_l; rows m = -l..l of the real harmonics, columns mu = -l..l of the complex ones."""
    u = np.zeros((2 * l + 1, 2 * l + 1), dtype=complex)
    u[l, l] = 1.0
    for m in range(1, l + 1):
        s = (-1.0) ** m
        u[l + m, l + m] = s / np.sqrt(2); u[l + m, l - m] = 1 / np.sqrt(2)
        u[l - m, l + m] = s / (1j * np.sqrt(2)); u[l - m, l - m] = -1 / (1j * np.sqrt(2))
    return u


def sympy_real_coupling(l1: int, l2: int, l: int) -> np.ndarray:
    from sympy import S
    from sympy.physics.quantum.cg import CG
    c = np.zeros((2 * l + 1, 2 * l1 + 1, 2 * l2 + 1))
    for mu1 in range(-l1, l1 + 1):
        for mu2 in range(-l2, l2 + 1):
            mu = mu1 + mu2
            if abs(mu) <= l:
                c[l + mu, l1 + mu1, l2 + mu2] = float(CG(S(l1), S(mu1), S(l2), S(mu2), S(l), S(mu)).doit())
    u, u1, u2 = real_from_complex(l), real_from_complex(l1), real_from_complex(l2)
    # T_real[m] = sum U[m,mu] <l1 mu1 l2 mu2 | l mu> conj(U1[m1,mu1]) conj(U2[m2,mu2]) A_real[m1] B_real[m2]
    real = np.einsum("mu,uvw,av,bw->mab", u, c.astype(complex), u1.conj(), u2.conj())
    assert np.abs(real.imag).max() < 1e-12 or np.abs(real.real).max() < 1e-12      # one global phase: 1 or i
    return real.real if np.abs(real.real).max() > np.abs(real.imag).max() else real.imag


@pytest.mark.parametrize("L", [0, 1, 2])
def test_coupling_tables_match_sympy_clebsch_gordan(L):
    for (l, l1, l2) in tp_paths(3, L):
        ours = coupling(l1, l2, l)
        theirs = sympy_real_coupling(l1, l2, l)
        cos = np.sum(ours * theirs) / np.sqrt(np.sum(ours * ours) * np.sum(theirs * theirs))
        assert abs(abs(cos) - 1.0) < 1e-12, (l, l1, l2, cos)
        scale = np.sum(ours * theirs) / np.sum(theirs * theirs)
        assert np.abs(ours - scale * theirs).max() < 1e-12, (l, l1, l2)


@pytest.mark.parametrize("L", [0, 1, 2])
def test_compiled_nonzero_table_is_the_sympy_pattern(L):
    """The (path, m, lm1, lm2, value) list that the kernels' straight-line code and cg_canon.hpp are written from."""
    paths, nz, _ = tables(L)
    for p, (l, l1, l2) in enumerate(paths):
        theirs = sympy_real_coupling(l1, l2, l)
        mine = np.zeros_like(theirs)
        for (pp, m, lm1, lm2, c) in nz:
            if pp == p:
                mine[m, lm1 - l1 * l1, lm2 - l2 * l2] = c
        scale = np.sum(mine * theirs) / np.sum(theirs * theirs)
        assert np.abs(mine - scale * theirs).max() < 1e-12, (l, l1, l2)
        assert np.count_nonzero(np.abs(theirs) > 1e-12) == sum(1 for e in nz if e[0] == p)
