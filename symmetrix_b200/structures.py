"""Seeded synthetic structures and a host neighbour-list builder.

The structures follow the constructions named for the benchmark configurations (rigid water
molecules on a jittered grid, a jittered multi-species FCC lattice, a molecular liquid built
from a rigid 9-atom template). The neighbour builder is the host-side statement of the edge
rule the callers of the evaluator use (pair_symmetrix/pair_symmetrix_mace.cpp:249-265,286-315:
``dx = x_j - x_i`` with ``x_j`` a periodic image position, edge kept iff
``dx*dx + dy*dy + dz*dz < r_cut*r_cut``; ASE path symmetrix/source/symmetrix/symmetrix_calc.py:77).
"""
from __future__ import annotations

import math
from dataclasses import dataclass

import numpy as np


@dataclass
class Structure:
    positions: np.ndarray        # [N, 3] float64, inside the cell
    cell: np.ndarray             # [3, 3] float64, rows are lattice vectors
    numbers: np.ndarray          # [N] atomic numbers
    pbc: tuple[bool, bool, bool] = (True, True, True)

    @property
    def num_atoms(self) -> int:
        return int(self.positions.shape[0])


def _random_rotations(rng: np.random.Generator, n: int) -> np.ndarray:
    q = rng.standard_normal((n, 4))
    q /= np.linalg.norm(q, axis=1, keepdims=True)
    w, x, y, z = q.T
    return np.stack([
        np.stack([1 - 2 * (y * y + z * z), 2 * (x * y - z * w), 2 * (x * z + y * w)], axis=1),
        np.stack([2 * (x * y + z * w), 1 - 2 * (x * x + z * z), 2 * (y * z - x * w)], axis=1),
        np.stack([2 * (x * z - y * w), 2 * (y * z + x * w), 1 - 2 * (x * x + y * y)], axis=1),
    ], axis=1)


def water_box(n_side: int = 4, box: float = 12.42, seed: int = 0, noise: float = 0.05) -> Structure:
    """``n_side^3`` rigid H2O (O-H 0.96 A, H-O-H 104.5 deg) on a jittered grid, random orientations."""
    rng = np.random.default_rng(seed)
    n_mol = n_side ** 3
    spacing = box / n_side
    grid = np.stack(np.meshgrid(*[np.arange(n_side)] * 3, indexing="ij"), axis=-1).reshape(-1, 3)
    centres = (grid + 0.5) * spacing + rng.uniform(-0.2, 0.2, size=(n_mol, 3)) * spacing * 0.5
    half = math.radians(104.5) / 2
    template = np.array([[0.0, 0.0, 0.0],
                         [0.96 * math.sin(half), 0.0, 0.96 * math.cos(half)],
                         [-0.96 * math.sin(half), 0.0, 0.96 * math.cos(half)]])
    rots = _random_rotations(rng, n_mol)
    pos = centres[:, None, :] + np.einsum("nij,aj->nai", rots, template)
    pos = pos.reshape(-1, 3) + rng.normal(0.0, noise, size=(3 * n_mol, 3))
    pos = np.mod(pos, box)
    numbers = np.tile(np.array([8, 1, 1]), n_mol)
    return Structure(pos, np.eye(3) * box, numbers)


def water_box_density(n_mol_side: int, density_g_cm3: float = 1.0, seed: int = 0) -> Structure:
    """Water box of ``n_mol_side^3`` molecules at the given density (same construction)."""
    n_mol = n_mol_side ** 3
    volume = n_mol * 18.01528 / (density_g_cm3 * 0.602214076)  # A^3
    return water_box(n_mol_side, volume ** (1.0 / 3.0), seed)


def fcc_box(n_cells: int | tuple[int, int, int] = 10, a: float = 3.6, species: list[int] | None = None,
            jitter: float = 0.1, seed: int = 0) -> Structure:
    """FCC lattice of ``n_cells`` conventional cells per axis, species drawn uniformly, Gaussian jitter."""
    rng = np.random.default_rng(seed)
    nc = (n_cells,) * 3 if isinstance(n_cells, int) else tuple(n_cells)
    basis = np.array([[0, 0, 0], [0.5, 0.5, 0], [0.5, 0, 0.5], [0, 0.5, 0.5]])
    grid = np.stack(np.meshgrid(np.arange(nc[0]), np.arange(nc[1]), np.arange(nc[2]), indexing="ij"), axis=-1).reshape(-1, 3)
    pos = ((grid[:, None, :] + basis[None, :, :]) * a).reshape(-1, 3)
    pos = pos + rng.normal(0.0, jitter, size=pos.shape)
    box = np.array(nc, dtype=np.float64) * a
    pos = np.mod(pos, box)
    species = species or [29]
    numbers = rng.choice(np.asarray(species), size=pos.shape[0])
    return Structure(pos, np.diag(box), numbers)


def molecular_liquid(n_mol: int, density_g_cm3: float = 0.79, seed: int = 0, min_dist: float = 0.8) -> Structure:
    """Random copies of a rigid 9-atom C2H5OH-like template, random orientations, overlap rejection."""
    rng = np.random.default_rng(seed)
    template = np.array([
        [0.000, 0.000, 0.000], [1.520, 0.000, 0.000], [2.050, 1.320, 0.000],      # C C O
        [-0.390, 1.020, 0.000], [-0.390, -0.510, 0.890], [-0.390, -0.510, -0.890],  # H3
        [1.900, -0.520, 0.890], [1.900, -0.520, -0.890], [3.010, 1.280, 0.000],     # H2, HO
    ])
    z = np.array([6, 6, 8, 1, 1, 1, 1, 1, 1])
    template = template - template.mean(axis=0)
    mass = 46.068
    volume = n_mol * mass / (density_g_cm3 * 0.602214076)
    box = volume ** (1.0 / 3.0)
    # molecules on a jittered grid (keeps construction O(N)), then reject/redo close contacts
    n_side = int(math.ceil(n_mol ** (1.0 / 3.0)))
    grid = np.stack(np.meshgrid(*[np.arange(n_side)] * 3, indexing="ij"), axis=-1).reshape(-1, 3)
    pick = rng.permutation(grid.shape[0])[:n_mol]
    spacing = box / n_side
    centres = (grid[pick] + 0.5) * spacing + rng.uniform(-0.15, 0.15, size=(n_mol, 3)) * spacing
    rots = _random_rotations(rng, n_mol)
    pos = centres[:, None, :] + np.einsum("nij,aj->nai", rots, template)
    pos = np.mod(pos.reshape(-1, 3), box)
    numbers = np.tile(z, n_mol)
    s = Structure(pos, np.eye(3) * box, numbers)
    for _ in range(20):
        nl = neighbor_list(s, min_dist)
        bad_atoms = np.unique(nl["i"])
        bad_mol = np.unique(bad_atoms // 9)
        # contacts inside one rigid molecule are part of the template, not overlaps
        inter = (nl["i"] // 9) != (nl["j"] // 9)
        bad_mol = np.unique(nl["i"][inter] // 9)
        if bad_mol.size == 0:
            break
        new_rots = _random_rotations(rng, bad_mol.size)
        new_centres = centres[bad_mol] + rng.uniform(-0.1, 0.1, size=(bad_mol.size, 3)) * spacing
        newpos = new_centres[:, None, :] + np.einsum("nij,aj->nai", new_rots, template)
        pos = s.positions.reshape(n_mol, 9, 3)
        pos[bad_mol] = np.mod(newpos, box)
        s = Structure(pos.reshape(-1, 3), s.cell, numbers)
    return s


def replicate(s: Structure, reps: tuple[int, int, int]) -> Structure:
    """``reps`` periodic copies of the cell along its three lattice vectors; copy (a, b, c) holds atoms
    ``((a * reps[1] + b) * reps[2] + c) * N ... + N`` in the order of ``s``. Every atom of the result has the environment of
    its original, so energies and forces of a periodic evaluation repeat copy by copy."""
    ra, rb, rc = (int(x) for x in reps)
    shifts = np.stack(np.meshgrid(np.arange(ra), np.arange(rb), np.arange(rc), indexing="ij"), axis=-1).reshape(-1, 3)
    offsets = shifts.astype(np.float64) @ s.cell
    pos = (offsets[:, None, :] + s.positions[None, :, :]).reshape(-1, 3)
    cell = s.cell * np.array([ra, rb, rc], dtype=np.float64)[:, None]
    return Structure(pos, cell, np.tile(s.numbers, shifts.shape[0]), s.pbc)


# --------------------------------------------------------------------------- neighbour list

def _image_range(cell: np.ndarray, pbc, r_cut: float) -> list[int]:
    vol = abs(np.linalg.det(cell))
    out = []
    for a in range(3):
        if not pbc[a]:
            out.append(0)
            continue
        cross = np.cross(cell[(a + 1) % 3], cell[(a + 2) % 3])
        height = vol / np.linalg.norm(cross)
        out.append(int(math.ceil(r_cut / height)))
    return out


def neighbor_list(s: Structure, r_cut: float, chunk: int = 512) -> dict:
    """Full neighbour list, edges grouped by receiver ``i`` (CSR), rows ordered by (sender, image).

    Edge rule and arithmetic (all float64, no fused multiply-add): the image position is
    ``p = x_j + (n0*a0 + n1*a1 + n2*a2)`` with the shift accumulated in that order,
    ``d = p - x_i`` and the edge is kept iff ``d0*d0 + d1*d1 + d2*d2 < r_cut*r_cut`` with the
    three products summed left to right; self-pairs with a zero shift are excluded.
    Returns ``i, j`` (int32), ``S`` (integer shifts), ``D`` (= d) and ``d`` (= sqrt of the sum).
    """
    pos = np.ascontiguousarray(s.positions, dtype=np.float64)
    cell = np.asarray(s.cell, dtype=np.float64)
    n = pos.shape[0]
    rng_img = _image_range(cell, s.pbc, r_cut)
    shifts = [(a, b, c) for a in range(-rng_img[0], rng_img[0] + 1)
              for b in range(-rng_img[1], rng_img[1] + 1) for c in range(-rng_img[2], rng_img[2] + 1)]
    rc2 = r_cut * r_cut
    use_tree = n > 3000 and all(r == 1 for r, p in zip(rng_img, s.pbc) if p) and np.allclose(cell, np.diag(np.diag(cell)))
    out_i, out_j, out_s, out_d = [], [], [], []
    if use_tree:
        from scipy.spatial import cKDTree
        box = np.diag(cell).copy()
        wrapped = np.mod(pos, box)
        tree = cKDTree(wrapped, boxsize=box)
        pairs = tree.query_pairs(r_cut * (1 + 1e-9) + 1e-9, output_type="ndarray")
        ci = np.concatenate([pairs[:, 0], pairs[:, 1]])
        cj = np.concatenate([pairs[:, 1], pairs[:, 0]])
        # minimum-image shift of each candidate (box > 2 r_cut so at most one image is in range)
        raw = pos[cj] - pos[ci]
        nshift = -np.round(raw / box).astype(np.int64)
        for extra in ([0, 0, 0],):
            sh = nshift + np.asarray(extra)
            svec = (sh[:, 0:1] * cell[0][None, :] + sh[:, 1:2] * cell[1][None, :]) + sh[:, 2:3] * cell[2][None, :]
            p = pos[cj] + svec
            d = p - pos[ci]
            r2 = (d[:, 0] * d[:, 0] + d[:, 1] * d[:, 1]) + d[:, 2] * d[:, 2]
            keep = r2 < rc2
            out_i.append(ci[keep]); out_j.append(cj[keep]); out_s.append(sh[keep]); out_d.append(d[keep])
    else:
        svecs = np.array([(sh[0] * cell[0] + sh[1] * cell[1]) + sh[2] * cell[2] for sh in shifts])
        sh_arr = np.array(shifts, dtype=np.int64)
        for i0 in range(0, n, chunk):
            i1 = min(n, i0 + chunk)
            xi = pos[i0:i1]
            for si in range(len(shifts)):
                p = pos + svecs[si][None, :]
                d = p[None, :, :] - xi[:, None, :]
                r2 = (d[..., 0] * d[..., 0] + d[..., 1] * d[..., 1]) + d[..., 2] * d[..., 2]
                keep = r2 < rc2
                if shifts[si] == (0, 0, 0):
                    idx = np.arange(i0, i1)
                    keep[idx - i0, idx] = False
                ii, jj = np.nonzero(keep)
                out_i.append(ii + i0); out_j.append(jj)
                out_s.append(np.broadcast_to(sh_arr[si], (ii.size, 3)).copy()); out_d.append(d[ii, jj])
    i = np.concatenate(out_i); j = np.concatenate(out_j)
    S = np.concatenate(out_s); D = np.concatenate(out_d)
    code = ((S[:, 0] + 64) * 128 + (S[:, 1] + 64)) * 128 + (S[:, 2] + 64)
    order = np.lexsort((code, j, i))
    i, j, S, D = i[order], j[order], S[order], D[order]
    r2 = (D[:, 0] * D[:, 0] + D[:, 1] * D[:, 1]) + D[:, 2] * D[:, 2]
    return {"i": i.astype(np.int32), "j": j.astype(np.int32), "S": S.astype(np.int32), "D": D, "d": np.sqrt(r2),
            "num_atoms": n}


def evaluator_inputs(s: Structure, nl: dict, atomic_numbers: list[int]) -> dict:
    """The six arrays the evaluator takes (libsymmetrix/source/mace.hpp:28-36), from a neighbour list.

    Built as the ASE calculator does (symmetrix_calc.py:78-83), except that ``num_neigh`` counts
    receivers (identical for a full list) and every atom is a node even if it has no neighbours.
    """
    n = s.num_atoms
    zmap = {z: t for t, z in enumerate(atomic_numbers)}
    types = np.array([zmap[int(z)] for z in s.numbers], dtype=np.int32)
    num_neigh = np.bincount(nl["i"], minlength=n).astype(np.int32)
    return {
        "num_nodes": n,
        "node_types": types,
        "num_neigh": num_neigh,
        "neigh_indices": nl["j"].astype(np.int32),
        "neigh_types": types[nl["j"]].astype(np.int32),
        "xyz": np.ascontiguousarray(nl["D"], dtype=np.float64).reshape(-1),
        "r": np.ascontiguousarray(nl["d"], dtype=np.float64),
    }


def atom_forces_and_virial(inputs: dict, nl: dict, node_forces: np.ndarray):
    """Per-atom forces and the 6-component virial from per-edge partial forces.

    ``f[i] -= nf_ij``, ``f[j] += nf_ij`` and ``virial += sym(xyz_ij (x) nf_ij)``
    (pair_symmetrix/pair_symmetrix_mace.cpp:334-368; symmetrix_calc.py:93-102).
    """
    n = inputs["num_nodes"]
    nf = np.asarray(node_forces, dtype=np.float64).reshape(-1, 3)[: nl["i"].size]
    f = np.zeros((n, 3))
    for c in range(3):
        f[:, c] = np.bincount(nl["j"], weights=nf[:, c], minlength=n) - np.bincount(nl["i"], weights=nf[:, c], minlength=n)
    x = inputs["xyz"].reshape(-1, 3)
    v = np.array([
        np.sum(x[:, 0] * nf[:, 0]), np.sum(x[:, 1] * nf[:, 1]), np.sum(x[:, 2] * nf[:, 2]),
        0.5 * np.sum(x[:, 0] * nf[:, 1] + x[:, 1] * nf[:, 0]),
        0.5 * np.sum(x[:, 0] * nf[:, 2] + x[:, 2] * nf[:, 0]),
        0.5 * np.sum(x[:, 1] * nf[:, 2] + x[:, 2] * nf[:, 1]),
    ])
    return f, v
