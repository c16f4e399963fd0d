"""Test infrastructure: CPU restatement (numpy, float64) of the reference's MACE energy+force
evaluation. It is the oracle the CUDA path is checked against where the compiled reference
(``oracle/_ref``) is not at hand, and it is itself pinned against that compiled reference and
the committed golden vectors by ``tests/test_oracle.py``. Only tests, the smoke check and the
CPU-baseline leg of the benchmark may import it; the product never does.

Each method restates one stage of ``class MACE`` (libsymmetrix/source/mace.cpp); the cited
lines are the loops being restated. Array layouts are the reference's (row-major, channel
index fastest).
"""
from __future__ import annotations

import json
import math

import numpy as np


def load_model(path_or_dict) -> dict:
    if isinstance(path_or_dict, dict):
        return path_or_dict
    with open(path_or_dict) as f:
        return json.load(f)


def real_sh_with_grad(l_max: int, xyz: np.ndarray):
    """Stage ``compute_Y`` (mace.cpp:118-148): harmonics of the direction of the shuffled vector
    (z, x, y), scaled by 2 sqrt(pi), with Cartesian gradients in the original axis order.
    The harmonics follow the convention of spherical_harmonic.cpp:28-36 (see the sphericart
    restatement in ref_shims/include/sphericart.hpp). Returns ``Y[E, nlm]``, ``dY[E, 3, nlm]``."""
    xyz = np.asarray(xyz, dtype=np.float64).reshape(-1, 3)
    n = xyz.shape[0]
    nlm = (l_max + 1) ** 2
    r = np.sqrt(np.sum(xyz * xyz, axis=1))
    u = np.stack([xyz[:, 2], xyz[:, 0], xyz[:, 1]], axis=1) / r[:, None]   # shuffled unit vector
    ux, uy, uz = u.T
    c = np.zeros((l_max + 2, n)); s = np.zeros((l_max + 2, n)); c[0] = 1.0
    for m in range(1, l_max + 2):
        c[m] = c[m - 1] * ux - s[m - 1] * uy
        s[m] = s[m - 1] * ux + c[m - 1] * uy
    q = np.zeros((l_max + 1, l_max + 2, n))
    for m in range(l_max + 1):
        dfact = 1.0
        for k in range(2 * m - 1, 1, -2):
            dfact *= k
        q[m, m] = dfact
        if m + 1 <= l_max:
            q[m + 1, m] = (2 * m + 1) * uz * dfact
        for l in range(m + 2, l_max + 1):
            q[l, m] = ((2 * l - 1) * uz * q[l - 1, m] - (l + m - 1) * q[l - 2, m]) / (l - m)
    y = np.zeros((n, nlm)); g = np.zeros((n, 3, nlm))   # g: gradient w.r.t. the shuffled unit vector
    scale = 2.0 * math.sqrt(math.pi)
    for l in range(l_max + 1):
        for m in range(l + 1):
            nrm = scale * math.sqrt((2 * l + 1) / (4 * math.pi) * math.factorial(l - m) / math.factorial(l + m))
            dq = q[l, m + 1]
            if m == 0:
                lm = l * l + l
                y[:, lm] = nrm * q[l, 0]
                g[:, 2, lm] = nrm * dq
            else:
                f = math.sqrt(2.0) * nrm
                lp, ln = l * l + l + m, l * l + l - m
                y[:, lp] = f * q[l, m] * c[m]; y[:, ln] = f * q[l, m] * s[m]
                g[:, 0, lp] = f * q[l, m] * m * c[m - 1]; g[:, 1, lp] = -f * q[l, m] * m * s[m - 1]
                g[:, 2, lp] = f * dq * c[m]
                g[:, 0, ln] = f * q[l, m] * m * s[m - 1]; g[:, 1, ln] = f * q[l, m] * m * c[m - 1]
                g[:, 2, ln] = f * dq * s[m]
    radial = np.einsum("ecl,ec->el", g, u)
    gs = (g - radial[:, None, :] * u[:, :, None]) / r[:, None, None]
    # un-shuffle: d/dx = shuffled component 1, d/dy = 2, d/dz = 0 (mace.cpp:141-147)
    dy = np.stack([gs[:, 1], gs[:, 2], gs[:, 0]], axis=1)
    return y, dy


class SplineSet:
    """``CubicSplineSet`` (cubic_spline_set.cpp:5-84): vector-valued cubic Hermite spline."""

    def __init__(self, h, values, derivs):
        v = np.asarray(values, dtype=np.float64)   # [num_splines, G]
        d = np.asarray(derivs, dtype=np.float64)
        self.h = float(h)
        h = self.h
        self.c0 = v[:, :-1].T.copy()               # [G-1, num_splines]
        self.c1 = d[:, :-1].T.copy()
        self.c2 = ((-3 * v[:, :-1] - 2 * h * d[:, :-1] + 3 * v[:, 1:] - h * d[:, 1:]) / (h * h)).T.copy()
        self.c3 = ((2 * v[:, :-1] + h * d[:, :-1] - 2 * v[:, 1:] + h * d[:, 1:]) / (h * h * h)).T.copy()

    def evaluate_derivs(self, r):
        r = np.asarray(r, dtype=np.float64)
        i = (r / self.h).astype(np.int64)           # static_cast<int>(r / h), cubic_spline_set.cpp:55
        x = (r - self.h * i)[:, None]
        xx = x * x
        val = self.c0[i] + x * self.c1[i] + xx * self.c2[i] + (xx * x) * self.c3[i]
        der = self.c1[i] + (2 * x) * self.c2[i] + (3 * xx) * self.c3[i]
        return val, der


class MaceOracle:
    """Restatement of ``class MACE`` (mace.hpp:12-169), including ZBL and density normalisation."""

    def __init__(self, model):
        m = load_model(model)
        self.model = m
        self.has_zbl = bool(m.get("has_zbl"))
        self.A0_scaled, self.A1_scaled = bool(m.get("A0_scaled")), bool(m.get("A1_scaled"))
        if self.has_zbl:
            self.zbl = dict(a_exp=float(m["zbl_a_exp"]), a_prefactor=float(m["zbl_a_prefactor"]), c=np.asarray(m["zbl_c"], dtype=np.float64),
                            radii=np.asarray(m["zbl_covalent_radii"], dtype=np.float64), p=int(m["zbl_p"]))
        if self.A0_scaled:
            self.A0_spl = [SplineSet(m["A0_spline_h"], [v], [d]) for v, d in zip(m["A0_spline_values"], m["A0_spline_derivs"])]
        if self.A1_scaled:
            self.A1_spl = [SplineSet(m["A1_spline_h"], [v], [d]) for v, d in zip(m["A1_spline_values"], m["A1_spline_derivs"])]
        self.num_elements = int(m["num_elements"]); self.K = int(m["num_channels"])
        self.r_cut = float(m["r_cut"]); self.l_max = int(m["l_max"]); self.L_max = int(m["L_max"])
        self.nlm = (self.l_max + 1) ** 2; self.nLM = (self.L_max + 1) ** 2
        self.atomic_numbers = list(m["atomic_numbers"])
        self.atomic_energies = np.asarray(m["atomic_energies"], dtype=np.float64)
        h = m["radial_spline_h"]
        self.spl0 = [SplineSet(h, v, d) for v, d in zip(m["radial_spline_values_0"], m["radial_spline_derivs_0"])]
        self.spl1 = [SplineSet(h, v, d) for v, d in zip(m["radial_spline_values_1"], m["radial_spline_derivs_1"])]
        K, E = self.K, self.num_elements
        self.H0_w = np.asarray(m["H0_weights"], dtype=np.float64).reshape(E, K)
        self.A0_w = np.asarray(m["A0_weights"], dtype=np.float64).reshape(E, self.l_max + 1, K, K)
        self.H1_w = np.asarray(m["H1_weights"], dtype=np.float64).reshape(self.L_max + 1, K, K)
        self.Phi1_l = list(m["Phi1_l"]); self.Phi1_l1 = list(m["Phi1_l1"]); self.Phi1_l2 = list(m["Phi1_l2"])
        self.cg_lme = np.asarray(m["Phi1_lme"], dtype=np.int64)
        self.cg_t = np.asarray(m["Phi1_lelm1lm2"], dtype=np.int64)
        self.cg_c = np.asarray(m["Phi1_clebsch_gordan"], dtype=np.float64)
        self.num_e = [sum(1 for l in self.Phi1_l if l == ll) for ll in range(self.l_max + 1)]
        self.num_lme = sum(2 * l + 1 for l in self.Phi1_l)
        self.num_t = sum((2 * a + 1) * (2 * b + 1) for a, b in zip(self.Phi1_l1, self.Phi1_l2))
        self.A1_w = [np.asarray(w, dtype=np.float64).reshape(self.num_e[l] * K, K) for l, w in enumerate(m["A1_weights"])]
        self.M0_mono = {int(lm): [tuple(t) for t in v] for lm, v in m["M0_monomials"].items()}
        self.M0_coef = {}
        for a, per_lm in m["M0_weights"].items():
            for lm, per_k in per_lm.items():
                self.M0_coef[(int(a), int(lm))] = self._dense_coef(per_k)
        self.M1_mono = [tuple(t) for t in m["M1_monomials"]]
        self.M1_coef = {int(a): self._dense_coef(per_k) for a, per_k in m["M1_weights"].items()}
        self.H2_w_H1 = np.asarray(m["H2_weights_for_H1"], dtype=np.float64).reshape(E, K, K)
        self.H2_w_M1 = np.asarray(m["H2_weights_for_M1"], dtype=np.float64).reshape(K, K)
        self.ro1 = np.asarray(m["readout_1_weights"], dtype=np.float64).reshape(K)
        self.ro2_w1 = np.asarray(m["readout_2_weights_1"], dtype=np.float64).reshape(16, K)
        self.ro2_w2 = np.asarray(m["readout_2_weights_2"], dtype=np.float64).reshape(16)
        self.ro2_scale = float(m["readout_2_scale_factor"])

    def _dense_coef(self, per_k):
        if isinstance(per_k, np.ndarray):
            return np.asarray(per_k, dtype=np.float64)
        if isinstance(per_k, dict):
            return np.array([per_k[k] for k in sorted(per_k, key=lambda s: int(s))], dtype=np.float64)
        return np.asarray(per_k, dtype=np.float64)

    # ---------------------------------------------------------------- helpers
    def _edges(self, inp):
        self.N = int(inp["num_nodes"])
        self.node_types = np.asarray(inp["node_types"], dtype=np.int64)
        self.num_neigh = np.asarray(inp["num_neigh"], dtype=np.int64)
        self.neigh_indices = np.asarray(inp["neigh_indices"], dtype=np.int64)
        self.neigh_types = np.asarray(inp["neigh_types"], dtype=np.int64)
        self.xyz = np.asarray(inp["xyz"], dtype=np.float64).reshape(-1, 3)
        self.r = np.asarray(inp["r"], dtype=np.float64)
        self.recv = np.repeat(np.arange(self.N), self.num_neigh)
        ti = self.node_types[self.recv]; tj = self.neigh_types
        lo, hi = np.minimum(ti, tj), np.maximum(ti, tj)
        # unordered pair index, mace.cpp:81-83
        self.pair = lo * (2 * self.num_elements - lo - 1) // 2 + hi

    def _radial(self, splines, width):
        val = np.zeros((self.r.size, width)); der = np.zeros((self.r.size, width))
        for p, spl in enumerate(splines):
            sel = np.nonzero(self.pair == p)[0]
            if sel.size:
                val[sel], der[sel] = spl.evaluate_derivs(self.r[sel])
        return val, der

    def _segment_sum(self, per_edge):
        out = np.zeros((self.N,) + per_edge.shape[1:])
        np.add.at(out, self.recv, per_edge)
        return out

    # ---------------------------------------------------------------- forward stages
    def compute_Y(self):                                            # mace.cpp:118-148
        self.Y, self.Y_grad = real_sh_with_grad(self.l_max, self.xyz)

    def compute_R0(self):                                           # mace.cpp:66-90
        self.R0, self.R0_deriv = self._radial(self.spl0, (self.l_max + 1) * self.K)

    def compute_R1(self):                                           # mace.cpp:92-116
        self.R1, self.R1_deriv = self._radial(self.spl1, len(self.Phi1_l) * self.K)

    def _l_of_lm(self):
        return np.array([l for l in range(self.l_max + 1) for _ in range(2 * l + 1)])

    def compute_A0(self):                                           # mace.cpp:150-201
        K = self.K
        lof = self._l_of_lm()
        R0 = self.R0.reshape(-1, self.l_max + 1, K)
        H0 = self.H0_w[self.neigh_types]                            # [E, K]
        per_edge = R0[:, lof, :] * self.Y[:, :, None] * H0[:, None, :]
        self.Phi0 = self._segment_sum(per_edge)                     # [N, nlm, K]
        W = self.A0_w[self.node_types][:, lof]                      # [N, nlm, K, K]
        self.A0 = np.einsum("nmk,nmkj->nmj", self.Phi0, W)

    def _poly(self, A, mono, coef_of_node):
        """Value and gradient of the per-(node, channel) sparse polynomial
        (multivariate_polynomial.cpp:246-289, the direct evaluation the DAG is tested against)."""
        f = np.zeros((A.shape[0], self.K)); g = np.zeros_like(A)
        for mu, idx in enumerate(mono):
            c = coef_of_node[:, :, mu]
            prod = np.ones((A.shape[0], self.K))
            for q in idx:
                prod = prod * A[:, q, :]
            f += c * prod
            for pos, q in enumerate(idx):
                d = np.ones((A.shape[0], self.K))
                for pos2, q2 in enumerate(idx):
                    if pos2 != pos:
                        d = d * A[:, q2, :]
                g[:, q, :] += c * d
        return f, g

    def compute_M0(self):                                           # mace.cpp:348-370
        self.M0 = np.zeros((self.N, self.nLM, self.K))
        self.M0_grad = np.zeros((self.N, self.nLM, self.nlm, self.K))
        for lm in range(self.nLM):
            coef = np.stack([self.M0_coef[(a, lm)] for a in range(self.num_elements)])[self.node_types]
            self.M0[:, lm], self.M0_grad[:, lm] = self._poly(self.A0, self.M0_mono[lm], coef)

    def compute_H1(self):                                           # mace.cpp:397-423
        lof = np.array([l for l in range(self.L_max + 1) for _ in range(2 * l + 1)])
        self.H1 = np.einsum("nmk,mkj->nmj", self.M0, self.H1_w[lof])

    def _t_table(self):
        rows = []
        for p, (l1, l2) in enumerate(zip(self.Phi1_l1, self.Phi1_l2)):
            for lm1 in range(l1 * l1, l1 * (l1 + 2) + 1):
                for lm2 in range(l2 * l2, l2 * (l2 + 2) + 1):
                    rows.append((p, lm1, lm2))
        return np.array(rows, dtype=np.int64)

    def _cg_matrix(self):
        c = np.zeros((self.num_lme, self.num_t))
        np.add.at(c, (self.cg_lme, self.cg_t), self.cg_c)
        return c

    def compute_Phi1(self, H1=None):                                # mace.cpp:453-502
        K = self.K
        H1 = self.H1 if H1 is None else H1
        tt = self._t_table()
        R1 = self.R1.reshape(-1, len(self.Phi1_l), K)
        Hj = H1[self.neigh_indices]                                 # [E, nLM, K]
        self.Phi1r = np.zeros((self.N, self.num_t, K))
        for t, (p, lm1, lm2) in enumerate(tt):
            np.add.at(self.Phi1r[:, t], self.recv, R1[:, p] * self.Y[:, lm1, None] * Hj[:, lm2])
        self.Phi1 = np.einsum("qt,ntk->nqk", self._cg_matrix(), self.Phi1r)

    def compute_A1(self):                                           # mace.cpp:607-642
        K = self.K
        self.A1 = np.zeros((self.N, self.nlm, K))
        off = 0
        for l in range(self.l_max + 1):
            ne = self.num_e[l]
            blk = self.Phi1[:, off:off + (2 * l + 1) * ne].reshape(self.N, 2 * l + 1, ne * K)
            self.A1[:, l * l:(l + 1) ** 2] = blk @ self.A1_w[l]
            off += (2 * l + 1) * ne

    def compute_M1(self):                                           # mace.cpp:759-777
        coef = np.stack([self.M1_coef[a] for a in range(self.num_elements)])[self.node_types]
        self.M1, self.M1_grad = self._poly(self.A1, self.M1_mono, coef)

    def compute_H2(self):                                           # mace.cpp:796-832
        self.H2 = (np.einsum("nk,nkj->nj", self.H1[:self.N, 0], self.H2_w_H1[self.node_types])
                   + self.M1 @ self.H2_w_M1)

    def compute_readouts(self):                                     # mace.cpp:876-903, multilayer_perceptron.cpp:76-150
        # adds into node_energies, which the caller zero-fills (mace.cpp:27-28, 880-890)
        if getattr(self, "node_energies", None) is None or self.node_energies.shape[0] != self.N:
            self.node_energies = np.zeros(self.N)
        self.node_energies += self.atomic_energies[self.node_types]
        self.node_energies += self.H1[:self.N, 0] @ self.ro1
        self.H1_adj = np.zeros_like(self.H1)
        self.H1_adj[:self.N, 0] = self.ro1[None, :]
        z = self.H2 @ self.ro2_w1.T                                 # [N, 16]
        sig = 1.0 / (1.0 + np.exp(-z))
        act = self.ro2_scale * z * sig
        dact = self.ro2_scale * sig + self.ro2_scale * z * sig * (1 - sig)
        self.node_energies += act @ self.ro2_w2
        self.H2_adj = (dact * self.ro2_w2[None, :]) @ self.ro2_w1

    # ---------------------------------------------------------------- ZBL and density normalisation
    def compute_ZBL(self):                                          # zbl.cpp:22-125
        if not self.has_zbl:
            return
        z = self.zbl
        Z = np.asarray(self.atomic_numbers)
        Zu = Z[self.node_types[self.recv]].astype(np.float64); Zv = Z[self.neigh_types].astype(np.float64)
        r = self.r
        r_max = z["radii"][Zu.astype(int)] + z["radii"][Zv.astype(int)]
        a = z["a_prefactor"] * 0.529 / (Zu ** z["a_exp"] + Zv ** z["a_exp"])
        ce = np.array([-3.2, -0.9423, -0.4028, -0.2016])
        terms = z["c"][None, :] * np.exp(ce[None, :] * (r / a)[:, None])
        phi = terms.sum(axis=1); dphi = (terms * ce[None, :]).sum(axis=1) / a
        v = 14.3996 * Zu * Zv / r * phi
        dv = 14.3996 * Zu * Zv * (r * dphi - phi) / (r * r)
        p = z["p"]; x = r / r_max
        env = 1.0 - ((p + 1.0) * (p + 2.0) / 2.0) * x ** p + p * (p + 2.0) * x ** (p + 1) - (p * (p + 1.0) / 2.0) * x ** (p + 2)
        denv = (-((p + 1.0) * (p + 2.0) / 2.0) * p * x ** (p - 1) + p * (p + 2.0) * (p + 1.0) * x ** p
                - (p * (p + 1.0) / 2.0) * (p + 2.0) * x ** (p + 1)) / r_max
        inside = r < r_max
        env = np.where(inside, env, 0.0); denv = np.where(inside, denv, 0.0)
        np.add.at(self.node_energies, self.recv, 0.5 * v * env)
        g = 0.5 * (v * denv + dv * env)
        self.node_forces -= self.xyz / r[:, None] * g[:, None]

    def _density(self, splines):
        f = np.zeros(self.r.size); d = np.zeros(self.r.size)
        for p, spl in enumerate(splines):
            sel = np.nonzero(self.pair == p)[0]
            if sel.size:
                v, dv = spl.evaluate_derivs(self.r[sel])
                f[sel], d[sel] = v[:, 0], dv[:, 0]
        factor = 1.0 + np.bincount(self.recv, weights=f, minlength=self.N)
        return factor, d

    def compute_A0_scaled(self):                                    # mace.cpp:273-298
        if self.A0_scaled:
            factor, _ = self._density(self.A0_spl)
            self.A0 = self.A0 / factor[:, None, None]

    def compute_A1_scaled(self):                                    # mace.cpp:681-706
        if self.A1_scaled:
            factor, _ = self._density(self.A1_spl)
            self.A1 = self.A1 / factor[:, None, None]

    def _reverse_scaled(self, splines, A, A_adj):                   # mace.cpp:300-346, 708-757
        factor, d = self._density(splines)
        dot = np.einsum("nqk,nqk->n", A_adj, A)
        g = (dot / factor)[self.recv] * d / self.r
        self.node_forces += self.xyz * g[:, None]
        return A_adj / factor[:, None, None]

    def reverse_A0_scaled(self):
        if self.A0_scaled:
            self.A0_adj = self._reverse_scaled(self.A0_spl, self.A0, self.A0_adj)

    def reverse_A1_scaled(self):
        if self.A1_scaled:
            self.A1_adj = self._reverse_scaled(self.A1_spl, self.A1, self.A1_adj)

    # ---------------------------------------------------------------- reverse stages
    def reverse_H2(self):                                           # mace.cpp:834-874
        self.H1_adj[:self.N, 0] += np.einsum("nkj,nj->nk", self.H2_w_H1[self.node_types], self.H2_adj)
        self.M1_adj = self.H2_adj @ self.H2_w_M1.T

    def reverse_M1(self):                                           # mace.cpp:779-794
        self.A1_adj = self.M1_grad * self.M1_adj[:, None, :]

    def reverse_A1(self):                                           # mace.cpp:644-679
        K = self.K
        self.dPhi1 = np.zeros((self.N, self.num_lme, K))
        off = 0
        for l in range(self.l_max + 1):
            ne = self.num_e[l]
            blk = self.A1_adj[:, l * l:(l + 1) ** 2] @ self.A1_w[l].T
            self.dPhi1[:, off:off + (2 * l + 1) * ne] = blk.reshape(self.N, (2 * l + 1) * ne, K)
            off += (2 * l + 1) * ne

    def reverse_Phi1(self, H1=None):                                # mace.cpp:504-605
        K = self.K
        H1 = self.H1 if H1 is None else H1
        tt = self._t_table()
        dPhi1r = np.einsum("qt,nqk->ntk", self._cg_matrix(), self.dPhi1)
        R1 = self.R1.reshape(-1, len(self.Phi1_l), K); R1d = self.R1_deriv.reshape(-1, len(self.Phi1_l), K)
        Hj = H1[self.neigh_indices]
        xhat = self.xyz / self.r[:, None]
        for t, (p, lm1, lm2) in enumerate(tt):
            d = dPhi1r[self.recv, t]                                 # [E, K]
            rad = np.sum(d * R1d[:, p] * Hj[:, lm2], axis=1) * self.Y[:, lm1]
            ang = np.sum(d * R1[:, p] * Hj[:, lm2], axis=1)
            self.node_forces -= xhat * rad[:, None] + self.Y_grad[:, :, lm1] * ang[:, None]
            np.add.at(self.H1_adj[:, lm2], self.neigh_indices, R1[:, p] * self.Y[:, lm1, None] * d)

    def reverse_H1(self):                                           # mace.cpp:425-451
        lof = np.array([l for l in range(self.L_max + 1) for _ in range(2 * l + 1)])
        self.M0_adj = np.einsum("nmj,mkj->nmk", self.H1_adj[:self.N], self.H1_w[lof])

    def reverse_M0(self):                                           # mace.cpp:372-395
        self.A0_adj = np.einsum("nLqk,nLk->nqk", self.M0_grad, self.M0_adj)

    def reverse_A0(self):                                           # mace.cpp:203-271
        K = self.K
        lof = self._l_of_lm()
        W = self.A0_w[self.node_types][:, lof]
        Phi0_adj = np.einsum("nmj,nmkj->nmk", self.A0_adj, W)[self.recv]      # [E, nlm, K]
        R0 = self.R0.reshape(-1, self.l_max + 1, K)[:, lof]; R0d = self.R0_deriv.reshape(-1, self.l_max + 1, K)[:, lof]
        H0 = self.H0_w[self.neigh_types][:, None, :]
        rad = np.einsum("emk,emk,em->e", Phi0_adj, R0d * H0, self.Y)
        ang = np.einsum("emk,emk->em", Phi0_adj, R0 * H0)
        xhat = self.xyz / self.r[:, None]
        self.node_forces -= xhat * rad[:, None] + np.einsum("ecm,em->ec", self.Y_grad, ang)

    # ---------------------------------------------------------------- driver
    def compute_node_energies_forces(self, inp):                    # mace.cpp:17-64
        self._edges(inp)
        self.node_forces = np.zeros((self.r.size, 3))
        self.node_energies = np.zeros(self.N)
        self.compute_Y(); self.compute_R0(); self.compute_A0(); self.compute_A0_scaled(); self.compute_M0(); self.compute_H1()
        self.compute_R1(); self.compute_Phi1(); self.compute_A1(); self.compute_A1_scaled(); self.compute_M1(); self.compute_H2()
        self.compute_readouts()
        self.compute_ZBL()        # the reference adds it first (mace.cpp:32-35); the sums commute
        self.reverse_H2(); self.reverse_M1(); self.reverse_A1_scaled(); self.reverse_A1(); self.reverse_Phi1()
        self.reverse_H1(); self.reverse_M0(); self.reverse_A0_scaled(); self.reverse_A0()
        return self.node_energies.copy(), self.node_forces.reshape(-1).copy()
