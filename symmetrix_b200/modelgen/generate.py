"""Seeded synthetic MACE models in the JSON schema the evaluator loads.

The schema is the one written by the reference's exporter
(symmetrix/source/symmetrix/extract_mace_data.py:107-519) and read by its loaders
(libsymmetrix/source/mace.cpp:905-1030). Pretrained models cannot be downloaded or converted
here, so benchmark and test models carry random weights of the right shapes, while every
symmetry-determined table (Clebsch-Gordan COO for the tensor product, generalized couplings
for the symmetric contraction) is computed from first principles in :mod:`.harmonics`, and the
radial tables are what the exporter would tabulate: an MLP applied to a Bessel x polynomial-
cutoff basis, sampled on ``num_spline_points`` nodes and re-splined
(extract_mace_data.py:145-178).
"""
from __future__ import annotations

import json
import math
from dataclasses import dataclass, field

import numpy as np
from scipy.interpolate import CubicSpline

from .harmonics import coupling

SILU_CST = 1.6790  # second-moment normalisation constant of SiLU used by e3nn-style gates


@dataclass
class ModelSpec:
    atomic_numbers: list[int]
    num_channels: int
    L_max: int = 0            # highest degree of the hidden node features (0: 64x0e, 1: +1o, 2: +2e)
    l_max: int = 3            # spherical-harmonic degree (the reference supports exactly 3)
    r_cut: float = 5.0
    num_bessel: int = 8
    poly_p: int = 5
    radial_mlp: tuple[int, ...] = (64, 64, 64)
    num_spline_points: int = 256
    avg_num_neighbors: float = 40.0
    seed: int = 0
    correlation: int = 3
    zbl: bool = False          # add a ZBL pair repulsion (MACE "pair_repulsion")
    density: bool = False      # density-normalised interaction blocks (A0_scaled / A1_scaled)
    num_interactions: int = 2  # 3 adds a middle block (full-L output) between the reference's two; file keys "*m*"
    extra: dict = field(default_factory=dict)


# --------------------------------------------------------------------------- tensor product

def tp_paths(l_max: int, L_max: int) -> list[tuple[int, int, int]]:
    """Paths ``(l, l1, l2)``: harmonics degree ``l1`` (x) feature degree ``l2`` -> output ``l``.

    Natural parity (-1)^l everywhere, outputs limited to ``l <= l_max``; enumerated feature-
    major, then harmonic, then output degree, and stably sorted by output degree, which
    groups paths by non-decreasing ``l`` as the loader requires (mace.cpp:613-641).
    """
    paths = []
    for l2 in range(L_max + 1):
        for l1 in range(l_max + 1):
            for l in range(abs(l1 - l2), min(l1 + l2, l_max) + 1):
                if (l1 + l2 + l) % 2 == 0:
                    paths.append((l, l1, l2))
    paths.sort(key=lambda p: p[0])
    return paths


def tp_tables(l_max: int, L_max: int):
    """``Phi1_l, Phi1_l1, Phi1_l2`` and the COO triple of the real Clebsch-Gordan map."""
    paths = tp_paths(l_max, L_max)
    ls = [p[0] for p in paths]
    num_e = [sum(1 for x in ls if x == l) for l in range(l_max + 1)]
    t_off = np.concatenate([[0], np.cumsum([(2 * p[1] + 1) * (2 * p[2] + 1) for p in paths])])
    lme_list, t_list, c_list = [], [], []
    for l1 in range(l_max + 1):
        for m1 in range(-l1, l1 + 1):
            for l2 in range(L_max + 1):
                for m2 in range(-l2, l2 + 1):
                    for le, (l, pl1, pl2) in enumerate(paths):
                        if (pl1, pl2) != (l1, l2):
                            continue
                        cg = coupling(l1, l2, l)
                        e = le - sum(1 for x in ls if x < l)
                        for m in range(-l, l + 1):
                            v = cg[l + m, l1 + m1, l2 + m2]
                            if abs(v) > 1e-12:
                                lme = sum((2 * ll + 1) * num_e[ll] for ll in range(l)) + (l + m) * num_e[l] + e
                                t = int(t_off[le]) + (l1 + m1) * (2 * l2 + 1) + (l2 + m2)
                                lme_list.append(lme)
                                t_list.append(t)
                                c_list.append(float(v))
    return paths, lme_list, t_list, c_list


# --------------------------------------------------------------------------- symmetric contraction

def contraction_basis(l_max: int, L: int, correlation: int):
    """Equivariant polynomial maps of degree <= correlation from ``A[(l_max+1)^2]`` to degree ``L``.

    Returns, per ``M`` in ``-L..L``: ``(monomials, blocks)`` where ``monomials`` is a list of
    sorted index tuples and ``blocks`` a list (one per correlation order) of arrays
    ``U[eta, mu]`` padded to the common monomial list; ``poly_M = sum_eta w[eta] U[eta] . monomials``
    is equivariant for any weights ``w`` shared across ``M``.
    """
    nlm = (l_max + 1) ** 2
    per_order = []  # per order: list of dicts[M] -> {tuple: coef}
    # order 1
    order1 = []
    if L <= l_max:
        order1.append([{(L * L + L + M,): 1.0} for M in range(-L, L + 1)])
    per_order.append(order1)
    # order 2
    order2 = []
    if correlation >= 2:
        for l1 in range(l_max + 1):
            for l2 in range(l1, l_max + 1):
                if (l1 + l2 + L) % 2:
                    continue
                cg = coupling(l1, l2, L)
                if cg is None:
                    continue
                dicts = []
                for M in range(2 * L + 1):
                    d = {}
                    for a, b in zip(*np.nonzero(cg[M])):
                        key = tuple(sorted((l1 * l1 + int(a), l2 * l2 + int(b))))
                        d[key] = d.get(key, 0.0) + float(cg[M, a, b])
                    dicts.append(d)
                order2.append(dicts)
    per_order.append(order2)
    # order 3
    order3 = []
    if correlation >= 3:
        for l1 in range(l_max + 1):
            for l2 in range(l1, l_max + 1):
                for l12 in range(abs(l1 - l2), l1 + l2 + 1):
                    c12 = coupling(l1, l2, l12)
                    for l3 in range(l_max + 1):
                        if (l1 + l2 + l3 + L) % 2:
                            continue
                        c3 = coupling(l12, l3, L)
                        if c12 is None or c3 is None:
                            continue
                        u = np.einsum("Mqc,qab->Mabc", c3, c12)
                        dicts = []
                        for M in range(2 * L + 1):
                            d = {}
                            for a, b, c in zip(*np.nonzero(np.abs(u[M]) > 1e-14)):
                                key = tuple(sorted((l1 * l1 + int(a), l2 * l2 + int(b), l3 * l3 + int(c))))
                                d[key] = d.get(key, 0.0) + float(u[M, a, b, c])
                            dicts.append({k: v for k, v in d.items() if abs(v) > 1e-12})
                        if any(len(d) for d in dicts):
                            order3.append(dicts)
    per_order.append(order3)
    assert nlm > 0
    out = []
    for M in range(2 * L + 1):
        monomials: list[tuple[int, ...]] = []
        index: dict[tuple[int, ...], int] = {}
        for paths in per_order:
            for dicts in paths:
                for key in dicts[M]:
                    if key not in index:
                        index[key] = len(monomials)
                        monomials.append(key)
        blocks = []
        for paths in per_order:
            u = np.zeros((len(paths), len(monomials)))
            for eta, dicts in enumerate(paths):
                for key, v in dicts[M].items():
                    u[eta, index[key]] = v
            blocks.append(u)
        out.append((monomials, blocks))
    # normalise each path jointly over M so that random weights give O(1) outputs
    for order in range(len(per_order)):
        n_eta = len(per_order[order])
        for eta in range(n_eta):
            tot = sum(float(np.sum(out[M][1][order][eta] ** 2)) for M in range(2 * L + 1))
            if tot > 0:
                s = math.sqrt((2 * L + 1) / tot)
                for M in range(2 * L + 1):
                    out[M][1][order][eta] *= s
    return out


# --------------------------------------------------------------------------- radial tables

def bessel_cutoff_basis(r: np.ndarray, r_cut: float, num_bessel: int, p: int) -> np.ndarray:
    n = np.arange(1, num_bessel + 1)
    x = r[:, None] / r_cut
    bessel = math.sqrt(2.0 / r_cut) * np.sin(n[None, :] * math.pi * x) / r[:, None]
    cutoff = (1.0 - (p + 1) * (p + 2) / 2.0 * x ** p + p * (p + 2) * x ** (p + 1) - p * (p + 1) / 2.0 * x ** (p + 2))
    cutoff = np.where(x < 1.0, cutoff, 0.0)
    return bessel * cutoff


def silu(x):
    return SILU_CST * x / (1.0 + np.exp(-x))


def radial_mlp_tables(spec: ModelSpec, rng: np.random.Generator, num_out: int, gain: float):
    """Nodal values/derivatives ``[Pu][num_out][G]`` and the MLP weights that produced them."""
    g = spec.num_spline_points
    r, h = np.linspace(1e-12, spec.r_cut, g, retstep=True)
    dims = [spec.num_bessel, *spec.radial_mlp, num_out]
    weights = [rng.standard_normal((dims[i], dims[i + 1])) / math.sqrt(dims[i]) for i in range(len(dims) - 1)]
    weights[0] *= 3.0
    weights[-1] *= gain
    n_el = len(spec.atomic_numbers)
    pair_scale = {}
    values, derivs = [], []
    hidden_values, hidden_derivs = [], []
    basis = bessel_cutoff_basis(r, spec.r_cut, spec.num_bessel, spec.poly_p)
    for a in range(n_el):
        for b in range(a, n_el):
            # element-pair dependence: a fixed per-pair rescaling of the basis amplitudes
            sc = 1.0 + 0.25 * rng.uniform(-1.0, 1.0, size=spec.num_bessel)
            pair_scale[(a, b)] = sc
            x = basis * sc[None, :]
            for w in weights[:-1]:
                x = silu(x @ w)
            y = x @ weights[-1]                                     # [G, num_out]
            spl = CubicSpline(r, y, axis=0, bc_type=("not-a-knot", "clamped"))
            values.append(np.ascontiguousarray(spl(r).T))            # [num_out, G]
            derivs.append(np.ascontiguousarray(spl.derivative()(r).T))
            # The same tabulation of the last hidden layer. Spline construction is linear in the nodal data and the last
            # layer is linear, so the tables above are, to rounding, these times weights[-1]: the radial tables have the
            # rank of the hidden width, whatever the number of output functions.
            hspl = CubicSpline(r, x, axis=0, bc_type=("not-a-knot", "clamped"))
            hidden_values.append(np.ascontiguousarray(hspl(r).T))    # [hidden, G]
            hidden_derivs.append(np.ascontiguousarray(hspl.derivative()(r).T))
    radial_mlp_tables.last_hidden = (np.stack(hidden_values), np.stack(hidden_derivs))
    return float(h), np.stack(values), np.stack(derivs), weights, pair_scale


# --------------------------------------------------------------------------- the model

def generate_model(spec: ModelSpec) -> dict:
    """Model dictionary; arrays are numpy, convert with :func:`to_jsonable` / :func:`write_json`."""
    if spec.l_max != 3:
        raise ValueError("the evaluator (like the reference) supports l_max == 3 only")
    rng = np.random.default_rng(spec.seed)
    k = spec.num_channels
    n_el = len(spec.atomic_numbers)
    l_max, L_max = spec.l_max, spec.L_max
    nlm, nLM = (l_max + 1) ** 2, (L_max + 1) ** 2
    out: dict = {}
    out["num_channels"] = k
    out["r_cut"] = float(spec.r_cut)
    out["l_max"] = l_max
    out["L_max"] = L_max
    out["atomic_numbers"] = sorted(int(z) for z in spec.atomic_numbers)
    out["num_elements"] = n_el
    out["atomic_energies"] = rng.uniform(-5.0, -1.0, size=n_el)
    out["has_zbl"] = bool(spec.zbl)
    if spec.zbl:
        # universal ZBL screening coefficients; synthetic covalent radii (the envelope vanishes at r_u + r_v)
        out["zbl_a_exp"] = 0.3
        out["zbl_a_prefactor"] = 0.4543
        out["zbl_c"] = [0.1818, 0.5099, 0.2802, 0.02817]
        out["zbl_covalent_radii"] = [0.2] + [0.6 + 0.35 * math.sqrt(z) / (1.0 + 0.02 * z) for z in range(1, 119)]
        out["zbl_p"] = 6

    paths, lme, t_idx, cg = tp_tables(l_max, L_max)
    h, v0, d0, mlp0, _ = radial_mlp_tables(spec, rng, (l_max + 1) * k, gain=1.0)
    h1, v1, d1, mlp1, pair_scale1 = radial_mlp_tables(spec, rng, len(paths) * k, gain=1.0)
    # The un-splined radial network of interaction block 1 (what the reference's exporter feeds to its cubic splines,
    # extract_mace_data.py:144-172): Bessel functions times the polynomial cutoff, a per-pair rescaling of the basis, and
    # the MLP. Keys with the "x_" prefix are extras that the reference loader ignores; the evaluator's run-time radial
    # mode (SMX_RADIAL=mlp) evaluates R(r) from them instead of reading the spline tables.
    out["x_radial_num_bessel"] = int(spec.num_bessel)
    out["x_radial_poly_p"] = int(spec.poly_p)
    out["x_radial_silu_scale"] = SILU_CST
    out["x_radial_mlp_dims_1"] = [int(w.shape[0]) for w in mlp1] + [int(mlp1[-1].shape[1])]
    out["x_radial_mlp_weights_1"] = [np.ascontiguousarray(w).ravel() for w in mlp1]          # each [in][out], row-major
    out["x_radial_pair_scale_1"] = [pair_scale1[(a, b)] for a in range(n_el) for b in range(a, n_el)]
    # Low-rank form of the block-1 radial tables: the last hidden layer tabulated exactly like the radial functions
    # ([pair][hidden][G] nodal values and derivatives); radial_spline_*_1 = these x x_radial_mlp_weights_1[-1] to rounding.
    out["x_radial_basis_values_1"], out["x_radial_basis_derivs_1"] = radial_mlp_tables.last_hidden
    out["radial_spline_h"] = h
    out["radial_spline_values_0"] = v0
    out["radial_spline_derivs_0"] = d0
    out["radial_spline_values_1"] = v1
    out["radial_spline_derivs_1"] = d1

    out["H0_weights"] = rng.standard_normal(n_el * k)
    def density_tables():
        """tanh(f(r)^2) per element pair, f a random combination of the radial basis, tabulated like the radial functions."""
        g = spec.num_spline_points
        rr, hh = np.linspace(1e-12, spec.r_cut, g, retstep=True)
        basis = bessel_cutoff_basis(rr, spec.r_cut, spec.num_bessel, spec.poly_p)
        vals, ders = [], []
        for a in range(n_el):
            for b in range(a, n_el):
                w = rng.standard_normal(spec.num_bessel)
                y = np.tanh((basis @ w) ** 2)
                spl = CubicSpline(rr, y, bc_type=("not-a-knot", "clamped"))
                vals.append(spl(rr)); ders.append(spl.derivative()(rr))
        return float(hh), np.stack(vals), np.stack(ders)

    out["A0_scaled"] = bool(spec.density)
    if spec.density:
        out["A0_spline_h"], out["A0_spline_values"], out["A0_spline_derivs"] = density_tables()
    out["A0_weights"] = rng.standard_normal((n_el, l_max + 1, k * k)) / (math.sqrt(k) * math.sqrt(spec.avg_num_neighbors))

    def contraction_weights(L_list):
        weights = {a: {} for a in range(n_el)}
        monos = {}
        stats = {}
        for L in L_list:
            basis = contraction_basis(l_max, L, spec.correlation)
            n_eta = [b.shape[0] for b in basis[0][1]]
            # higher orders are damped so that features stay O(1) through both layers
            w = [rng.standard_normal((n_el, n, k)) / math.sqrt(max(n, 1)) * (0.5 ** o) for o, n in enumerate(n_eta)]
            for M in range(2 * L + 1):
                lm = L * L + M
                monomials, blocks = basis[M]
                coef = sum(np.einsum("aek,em->akm", w[o], blocks[o]) for o in range(len(blocks)))
                monos[lm] = [list(m) for m in monomials]
                for a in range(n_el):
                    weights[a][lm] = coef[a]          # [k, n_mono]
                stats[lm] = len(monomials)
        return weights, monos, stats

    m0_w, m0_m, m0_stats = contraction_weights(range(L_max + 1))
    out["M0_weights"] = m0_w
    out["M0_monomials"] = m0_m

    out["H1_weights"] = (rng.standard_normal((L_max + 1, k, k)) / math.sqrt(k)).ravel()

    if spec.num_interactions == 3:
        # Middle interaction block, an extension of the reference's two-block file format (its exporter stops at two,
        # extract_mace_data.py:70-71). Same tensor-product tables as the last block; the contraction keeps every (L, M)
        # like M0; the new features are a per-L linear of it plus a per-element, per-L residual of the previous
        # features; a linear readout on its scalar part.
        if spec.density or spec.zbl:
            raise ValueError("density normalisation / ZBL are not defined for the three-block extension")
        out["num_interactions"] = 3
        _, vm, dm, _, _ = radial_mlp_tables(spec, rng, len(paths) * k, gain=1.0)
        out["radial_spline_values_m"] = vm
        out["radial_spline_derivs_m"] = dm
        num_e_m = [sum(1 for p in paths if p[0] == l) for l in range(l_max + 1)]
        out["Am_weights"] = [
            (rng.standard_normal(num_e_m[l] * k * k) / (math.sqrt(num_e_m[l] * k) * math.sqrt(spec.avg_num_neighbors)))
            for l in range(l_max + 1)
        ]
        mm_w, mm_m, mm_stats = contraction_weights(range(L_max + 1))
        out["Mm_weights"] = mm_w
        out["Mm_monomials"] = mm_m
        out["Hm_weights"] = (rng.standard_normal((L_max + 1, k, k)) / math.sqrt(k)).ravel()
        out["Hm_weights_for_H1"] = (rng.standard_normal((n_el, L_max + 1, k, k)) / math.sqrt(k)).ravel()
        out["readout_m_weights"] = 0.25 * rng.standard_normal(k) / math.sqrt(k)
    elif spec.num_interactions != 2:
        raise ValueError("num_interactions must be 2 or 3")

    out["Phi1_l"] = [p[0] for p in paths]
    out["Phi1_l1"] = [p[1] for p in paths]
    out["Phi1_l2"] = [p[2] for p in paths]
    out["Phi1_lme"] = lme
    out["Phi1_clebsch_gordan"] = cg
    out["Phi1_lelm1lm2"] = t_idx

    out["A1_scaled"] = bool(spec.density)
    if spec.density:
        out["A1_spline_h"], out["A1_spline_values"], out["A1_spline_derivs"] = density_tables()
    num_e = [sum(1 for p in paths if p[0] == l) for l in range(l_max + 1)]
    out["A1_weights"] = [
        (rng.standard_normal(num_e[l] * k * k) / (math.sqrt(num_e[l] * k) * math.sqrt(spec.avg_num_neighbors)))
        for l in range(l_max + 1)
    ]

    m1_w, m1_m, m1_stats = contraction_weights([0])
    out["M1_weights"] = {a: m1_w[a][0] for a in range(n_el)}
    out["M1_monomials"] = m1_m[0]

    out["H2_weights_for_H1"] = rng.standard_normal((n_el, k * k)) / math.sqrt(k)
    out["H2_weights_for_M1"] = rng.standard_normal(k * k) / math.sqrt(k)
    out["readout_1_weights"] = 0.25 * rng.standard_normal(k) / math.sqrt(k)
    out["readout_2_weights_1"] = rng.standard_normal(16 * k) / math.sqrt(k)
    out["readout_2_weights_2"] = 0.25 * rng.standard_normal(16) / 4.0
    out["readout_2_scale_factor"] = SILU_CST

    # Extra keys (ignored by the reference loader): provenance and the un-splined radial MLPs.
    out["x_generator"] = {
        "seed": spec.seed, "num_bessel": spec.num_bessel, "poly_p": spec.poly_p,
        "radial_mlp": list(spec.radial_mlp), "avg_num_neighbors": spec.avg_num_neighbors,
        "num_monomials_M0": {str(kk): int(vv) for kk, vv in m0_stats.items()},
        "num_monomials_M1": int(m1_stats[0]), "nnz_clebsch_gordan": len(cg),
        **spec.extra,
    }
    return out


def to_jsonable(obj):
    if isinstance(obj, np.ndarray):
        return obj.tolist()
    if isinstance(obj, (np.floating,)):
        return float(obj)
    if isinstance(obj, (np.integer,)):
        return int(obj)
    if isinstance(obj, dict):
        return {str(k): to_jsonable(v) for k, v in obj.items()}
    if isinstance(obj, (list, tuple)):
        return [to_jsonable(v) for v in obj]
    return obj


def expand_contraction_weights(model: dict) -> dict:
    """Nested ``{a: {lm: {k: [...]}}}`` / ``{a: {k: [...]}}`` maps as the exporter writes them
    (extract_mace_data.py:273-304,427-474), from the dense arrays kept in memory."""
    m = dict(model)
    m["M0_weights"] = {
        a: {lm: {kk: row for kk, row in enumerate(np.asarray(arr))} for lm, arr in per_lm.items()}
        for a, per_lm in model["M0_weights"].items()
    }
    m["M1_weights"] = {a: {kk: row for kk, row in enumerate(np.asarray(arr))} for a, arr in model["M1_weights"].items()}
    if "Mm_weights" in model:
        m["Mm_weights"] = {
            a: {lm: {kk: row for kk, row in enumerate(np.asarray(arr))} for lm, arr in per_lm.items()}
            for a, per_lm in model["Mm_weights"].items()
        }
    return m


def write_json(model: dict, path) -> None:
    with open(path, "w") as f:
        json.dump(to_jsonable(expand_contraction_weights(model)), f)


# --------------------------------------------------------------------------- named configurations

ELEMENT_POOL_89 = list(range(1, 90))


def named_spec(name: str, **over) -> ModelSpec:
    """Model specifications of the benchmark configurations (sizes per configuration index)."""
    if name == "water64":      # configuration 0: 64x0e, H/O, r_cut 5, 8 Bessel functions
        spec = ModelSpec([1, 8], 64, L_max=0, r_cut=5.0, num_bessel=8, avg_num_neighbors=50.0, seed=11)
    elif name == "fcc128":     # configurations 1 and 3: 128x0e+128x1o, r_cut 6, 10 radial functions
        rng = np.random.default_rng(101)
        five = sorted(int(z) for z in rng.choice(ELEMENT_POOL_89, size=5, replace=False))
        spec = ModelSpec(five, 128, L_max=1, r_cut=6.0, num_bessel=10, avg_num_neighbors=78.0, seed=12,
                         extra={"element_pool": 89})
    elif name == "organic128":  # configuration 2: ten organic elements, r_cut 5
        spec = ModelSpec([1, 6, 7, 8, 9, 15, 16, 17, 35, 53], 128, L_max=1, r_cut=5.0, num_bessel=8,
                         avg_num_neighbors=50.0, seed=13)
    elif name == "large256":   # configuration 4: 256x0e+256x1o+256x2e
        spec = ModelSpec([1, 6, 7, 8], 256, L_max=2, r_cut=5.0, num_bessel=8, avg_num_neighbors=48.0, seed=14)
    elif name == "deep256":    # configuration 4 as asked: three interaction blocks (no reference implementation exists)
        spec = ModelSpec([1, 6, 7, 8], 256, L_max=2, r_cut=5.0, num_bessel=8, avg_num_neighbors=48.0, seed=15, num_interactions=3)
    elif name == "tiny":       # committed golden fixture: a few channels, coarse spline grid
        spec = ModelSpec([1, 8], 8, L_max=1, r_cut=4.0, num_bessel=4, radial_mlp=(8, 8), num_spline_points=24,
                         avg_num_neighbors=30.0, seed=5)
    else:
        raise KeyError(name)
    for key, val in over.items():
        setattr(spec, key, val)
    return spec
