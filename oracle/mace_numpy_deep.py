"""Test infrastructure: CPU restatement (numpy, float64) of a MACE evaluation with THREE interaction blocks.

PARITY UNPINNED BY THE REFERENCE: the reference implements exactly two interaction blocks (its exporter refuses
other depths, symmetrix/source/symmetrix/extract_mace_data.py:70-71, and ``class MACE`` has one fixed stage list,
libsymmetrix/source/mace.cpp:36-63), so no reference output exists for this model family. This file generalises the
layer-1 stages of ``mace.cpp`` (``compute_Phi1 ... compute_H2``, mace.cpp:453-832) to a middle block whose
contraction keeps every (L, M) exactly like ``compute_M0`` (mace.cpp:348-370) and whose new node features are a per-L
linear map of that contraction (as ``compute_H1``, mace.cpp:397-423) plus a per-element, per-L linear map of the previous
features (the residual that ``compute_H2`` applies to L = 0 only, mace.cpp:796-832). It is checked by finite differences,
rotation invariance, and by reducing to the two-block oracle (which IS pinned against the compiled reference) when the
middle block is made the identity. Only tests may import it; the product never does.
"""
from __future__ import annotations

import numpy as np

from .mace_numpy import MaceOracle, SplineSet


class DeepMaceOracle(MaceOracle):
    """Blocks: 0 (A0, M0, H1) -> m (Phim, Am, Mm, Hm) -> 1 (Phi1, A1, M1, H2) -> readouts on H1, Hm, H2."""

    def __init__(self, model):
        super().__init__(model)
        m = self.model
        if int(m.get("num_interactions", 2)) != 3:
            raise ValueError("DeepMaceOracle needs a model file with num_interactions == 3")
        K, E = self.K, self.num_elements
        h = m["radial_spline_h"]
        self.splm = [SplineSet(h, v, d) for v, d in zip(m["radial_spline_values_m"], m["radial_spline_derivs_m"])]
        self.Am_w = [np.asarray(w, dtype=np.float64).reshape(self.num_e[l] * K, K) for l, w in enumerate(m["Am_weights"])]
        self.Mm_mono = {int(lm): [tuple(t) for t in v] for lm, v in m["Mm_monomials"].items()}
        self.Mm_coef = {}
        for a, per_lm in m["Mm_weights"].items():
            for lm, per_k in per_lm.items():
                self.Mm_coef[(int(a), int(lm))] = self._dense_coef(per_k)
        self.Hm_w = np.asarray(m["Hm_weights"], dtype=np.float64).reshape(self.L_max + 1, K, K)
        self.Hm_res = np.asarray(m["Hm_weights_for_H1"], dtype=np.float64).reshape(E, self.L_max + 1, K, K)
        self.ro_m = np.asarray(m["readout_m_weights"], dtype=np.float64).reshape(K)
        self._lof = np.array([l for l in range(self.L_max + 1) for _ in range(2 * l + 1)])

    # ------------------------------------------------------------ tensor product with explicit operands
    def _tp_forward(self, R, H):                                    # as compute_Phi1, mace.cpp:453-502
        K = self.K
        tt = self._t_table()
        Rp = R.reshape(-1, len(self.Phi1_l), K)
        Hj = H[self.neigh_indices]
        Phir = np.zeros((self.N, self.num_t, K))
        for t, (p, lm1, lm2) in enumerate(tt):
            np.add.at(Phir[:, t], self.recv, Rp[:, p] * self.Y[:, lm1, None] * Hj[:, lm2])
        return np.einsum("qt,ntk->nqk", self._cg_matrix(), Phir)

    def _tp_reverse(self, R, Rd, H, dPhi, H_adj):                   # as reverse_Phi1, mace.cpp:504-605
        K = self.K
        tt = self._t_table()
        dPhir = np.einsum("qt,nqk->ntk", self._cg_matrix(), dPhi)
        Rp = R.reshape(-1, len(self.Phi1_l), K); Rdp = Rd.reshape(-1, len(self.Phi1_l), K)
        Hj = H[self.neigh_indices]
        xhat = self.xyz / self.r[:, None]
        for t, (p, lm1, lm2) in enumerate(tt):
            d = dPhir[self.recv, t]
            rad = np.sum(d * Rdp[:, p] * Hj[:, lm2], axis=1) * self.Y[:, lm1]
            ang = np.sum(d * Rp[:, p] * Hj[:, lm2], axis=1)
            self.node_forces -= xhat * rad[:, None] + self.Y_grad[:, :, lm1] * ang[:, None]
            np.add.at(H_adj[:, lm2], self.neigh_indices, Rp[:, p] * self.Y[:, lm1, None] * d)

    def _linear_A(self, Phi, W):                                    # as compute_A1, mace.cpp:607-642
        K = self.K
        A = np.zeros((self.N, self.nlm, K))
        off = 0
        for l in range(self.l_max + 1):
            ne = self.num_e[l]
            blk = Phi[:, off:off + (2 * l + 1) * ne].reshape(self.N, 2 * l + 1, ne * K)
            A[:, l * l:(l + 1) ** 2] = blk @ W[l]
            off += (2 * l + 1) * ne
        return A

    def _linear_A_reverse(self, A_adj, W):                          # as reverse_A1, mace.cpp:644-679
        K = self.K
        dPhi = np.zeros((self.N, self.num_lme, K))
        off = 0
        for l in range(self.l_max + 1):
            ne = self.num_e[l]
            blk = A_adj[:, l * l:(l + 1) ** 2] @ W[l].T
            dPhi[:, off:off + (2 * l + 1) * ne] = blk.reshape(self.N, (2 * l + 1) * ne, K)
            off += (2 * l + 1) * ne
        return dPhi

    # ------------------------------------------------------------ middle block, forward
    def compute_Rm(self):
        self.Rm, self.Rm_deriv = self._radial(self.splm, len(self.Phi1_l) * self.K)

    def compute_Phim(self):
        self.Phim = self._tp_forward(self.Rm, self.H1)

    def compute_Am(self):
        self.Am = self._linear_A(self.Phim, self.Am_w)

    def compute_Mm(self):                                           # as compute_M0, mace.cpp:348-370
        self.Mm = np.zeros((self.N, self.nLM, self.K))
        self.Mm_grad = np.zeros((self.N, self.nLM, self.nlm, self.K))
        for lm in range(self.nLM):
            coef = np.stack([self.Mm_coef[(a, lm)] for a in range(self.num_elements)])[self.node_types]
            self.Mm[:, lm], self.Mm_grad[:, lm] = self._poly(self.Am, self.Mm_mono[lm], coef)

    def compute_Hm(self):                                           # compute_H1 + the residual of compute_H2, for every L
        res = self.Hm_res[self.node_types][:, self._lof]            # [N, nLM, K, K]
        self.Hm = (np.einsum("nmk,mkj->nmj", self.Mm, self.Hm_w[self._lof])
                   + np.einsum("nmk,nmkj->nmj", self.H1[:self.N], res))

    # ------------------------------------------------------------ last block on the middle block's features
    def compute_Phi1(self, H1=None):
        self.Phi1 = self._tp_forward(self.R1, self.Hm if H1 is None else H1)

    def compute_H2(self):
        self.H2 = (np.einsum("nk,nkj->nj", self.Hm[:self.N, 0], self.H2_w_H1[self.node_types]) + self.M1 @ self.H2_w_M1)

    def compute_readouts(self):
        super().compute_readouts()                                  # E0 + ro1 . H1[:, 0] + MLP(H2); H1_adj, H2_adj
        self.node_energies += self.Hm[:self.N, 0] @ self.ro_m
        self.Hm_adj = np.zeros_like(self.Hm)
        self.Hm_adj[:self.N, 0] = self.ro_m[None, :]

    # ------------------------------------------------------------ reverse
    def reverse_H2(self):
        self.Hm_adj[:self.N, 0] += np.einsum("nkj,nj->nk", self.H2_w_H1[self.node_types], self.H2_adj)
        self.M1_adj = self.H2_adj @ self.H2_w_M1.T

    def reverse_Phi1(self, H1=None):
        self._tp_reverse(self.R1, self.R1_deriv, self.Hm if H1 is None else H1, self.dPhi1, self.Hm_adj)

    def reverse_Hm(self):
        res = self.Hm_res[self.node_types][:, self._lof]
        self.Mm_adj = np.einsum("nmj,mkj->nmk", self.Hm_adj[:self.N], self.Hm_w[self._lof])
        self.H1_adj[:self.N] += np.einsum("nmj,nmkj->nmk", self.Hm_adj[:self.N], res)

    def reverse_Mm(self):
        self.Am_adj = np.einsum("nLqk,nLk->nqk", self.Mm_grad, self.Mm_adj)

    def reverse_Am(self):
        self.dPhim = self._linear_A_reverse(self.Am_adj, self.Am_w)

    def reverse_Phim(self):
        self._tp_reverse(self.Rm, self.Rm_deriv, self.H1, self.dPhim, self.H1_adj)

    # ------------------------------------------------------------ driver
    def compute_node_energies_forces(self, inp):
        self._edges(inp)
        self.node_forces = np.zeros((self.r.size, 3))
        self.node_energies = np.zeros(self.N)
        self.compute_Y(); self.compute_R0(); self.compute_A0(); self.compute_M0(); self.compute_H1()
        self.compute_Rm(); self.compute_Phim(); self.compute_Am(); self.compute_Mm(); self.compute_Hm()
        self.compute_R1(); self.compute_Phi1(); self.compute_A1(); self.compute_M1(); self.compute_H2()
        self.compute_readouts()
        self.reverse_H2(); self.reverse_M1(); self.reverse_A1(); self.reverse_Phi1()
        self.reverse_Hm(); self.reverse_Mm(); self.reverse_Am(); self.reverse_Phim()
        self.reverse_H1(); self.reverse_M0(); self.reverse_A0()
        return self.node_energies.copy(), self.node_forces.reshape(-1).copy()
