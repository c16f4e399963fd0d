"""Real spherical harmonics and the invariant coupling tensors built from them.

Everything here is derived numerically from one definition -- the real harmonics ``Y_lm`` in
the convention the MACE evaluator feeds its tensor products with (reference
libsymmetrix/source/mace.cpp:118-148: orthonormal real harmonics of the direction of the
axis-shuffled vector (z, x, y), times 2 sqrt(pi), index lm = l*l + l + m). Rotation matrices
are obtained by fitting ``Y_l(R x) = D_l(R) Y_l(x)`` and coupling (Clebsch-Gordan) tensors as
the null space of the equivariance constraint, so every table is consistent with that
definition by construction and no external convention has to be transcribed.
"""
from __future__ import annotations

import functools
import math

import numpy as np


def real_sh(l_max: int, xyz: np.ndarray) -> np.ndarray:
    """``Y[n, (l_max+1)^2]`` for vectors ``xyz[n, 3]`` (any non-zero length)."""
    xyz = np.asarray(xyz, dtype=np.float64)
    r = np.linalg.norm(xyz, axis=1)
    # axis shuffle (x, y, z) -> (z, x, y), reference mace.cpp:127-131
    ux, uy, uz = xyz[:, 2] / r, xyz[:, 0] / r, xyz[:, 1] / r
    n = xyz.shape[0]
    c = np.zeros((l_max + 1, n))
    s = np.zeros((l_max + 1, n))
    c[0] = 1.0
    for m in range(1, l_max + 1):
        c[m] = c[m - 1] * ux - s[m - 1] * uy
        s[m] = s[m - 1] * ux + c[m - 1] * uy
    q = np.zeros((l_max + 1, l_max + 1, n))  # q[l, m] = d^m P_l / dz^m
    for m in range(l_max + 1):
        dfact = 1.0
        for k in range(2 * m - 1, 1, -2):
            dfact *= k
        q[m, m] = dfact
        if m + 1 <= l_max:
            q[m + 1, m] = (2 * m + 1) * uz * dfact
        for l in range(m + 2, l_max + 1):
            q[l, m] = ((2 * l - 1) * uz * q[l - 1, m] - (l + m - 1) * q[l - 2, m]) / (l - m)
    out = np.zeros((n, (l_max + 1) ** 2))
    scale = 2.0 * math.sqrt(math.pi)  # reference mace.cpp:135-138
    for l in range(l_max + 1):
        for m in range(l + 1):
            norm = math.sqrt((2 * l + 1) / (4 * math.pi) * math.factorial(l - m) / math.factorial(l + m))
            if m == 0:
                out[:, l * l + l] = scale * norm * q[l, 0]
            else:
                f = scale * math.sqrt(2.0) * norm
                out[:, l * l + l + m] = f * q[l, m] * c[m]
                out[:, l * l + l - m] = f * q[l, m] * s[m]
    return out


def random_rotation(rng: np.random.Generator) -> np.ndarray:
    a = rng.standard_normal((3, 3))
    qm, rm = np.linalg.qr(a)
    qm = qm * np.sign(np.diag(rm))
    if np.linalg.det(qm) < 0:
        qm[:, 0] = -qm[:, 0]
    return qm


def rotation_matrix_l(l: int, rot: np.ndarray, rng: np.random.Generator | None = None) -> np.ndarray:
    """``D`` with ``Y_l(rot @ x) = D @ Y_l(x)`` for the harmonics of :func:`real_sh`."""
    rng = rng or np.random.default_rng(12345)
    pts = rng.standard_normal((8 * (2 * l + 1) + 8, 3))
    sl = slice(l * l, (l + 1) * (l + 1))
    a = real_sh(l, pts)[:, sl]
    b = real_sh(l, pts @ rot.T)[:, sl]
    dt, *_ = np.linalg.lstsq(a, b, rcond=None)
    return dt.T


@functools.lru_cache(maxsize=None)
def _rotations(count: int = 4):
    rng = np.random.default_rng(20240607)
    return tuple(random_rotation(rng) for _ in range(count))


@functools.lru_cache(maxsize=None)
def _dmat(l: int, which: int) -> np.ndarray:
    return rotation_matrix_l(l, _rotations()[which])


@functools.lru_cache(maxsize=None)
def coupling(l1: int, l2: int, l3: int) -> np.ndarray | None:
    """Real Clebsch-Gordan tensor ``C[m3, m1, m2]`` coupling ``l1 (x) l2 -> l3``.

    The unique (up to scale) tensor with ``D3 C = C (D1 (x) D2)`` for every proper rotation.
    Normalised so that ``sum_{m1 m2} C[m3, m1, m2]^2 = 1`` for every ``m3``; the sign is fixed
    by making the first entry of largest magnitude positive. ``None`` if the triangle rule fails.
    """
    if l3 < abs(l1 - l2) or l3 > l1 + l2:
        return None
    n1, n2, n3 = 2 * l1 + 1, 2 * l2 + 1, 2 * l3 + 1
    rows = []
    for w in range(len(_rotations())):
        d1, d2, d3 = _dmat(l1, w), _dmat(l2, w), _dmat(l3, w)
        # constraint: (D3 (x) I - I (x) (D1 (x) D2)^T) vec(C) = 0 with C as [n3, n1*n2]
        k12 = np.kron(d1, d2)
        rows.append(np.kron(d3, np.eye(n1 * n2)) - np.kron(np.eye(n3), k12.T))
    a = np.concatenate(rows, axis=0)
    _, sv, vt = np.linalg.svd(a)
    null = vt[sv.size - 1] if sv[-1] < 1e-9 else None
    if null is None:
        return None
    if sv.size >= 2 and sv[-2] < 1e-9:
        raise RuntimeError(f"coupling ({l1},{l2},{l3}): null space is not one-dimensional")
    c = null.reshape(n3, n1, n2)
    c = c / math.sqrt(np.sum(c * c) / n3)
    c[np.abs(c) < 1e-12] = 0.0
    flat = c.ravel()
    lead = flat[np.argmax(np.abs(flat) > 0.5 * np.max(np.abs(flat)))]
    if lead < 0:
        c = -c
    return c
