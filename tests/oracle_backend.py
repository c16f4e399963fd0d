"""Test infrastructure: the numpy oracle dressed as an evaluator backend for ``symmetrix_b200.domain``,
so that the decomposition logic (plans, halo exchanges, multi-process runs over gloo) can be tested
without a GPU. Never used by the product."""
import numpy as np
import torch

from oracle.mace_numpy import MaceOracle, load_model
from oracle.mace_numpy_deep import DeepMaceOracle
from symmetrix_b200 import structures as st


class OracleBackend:
    def __init__(self, model):
        model = load_model(model)
        self.num_interactions = int(model.get("num_interactions", 2))
        self.o = DeepMaceOracle(model) if self.num_interactions == 3 else MaceOracle(model)
        self.num_LM = self.o.nLM
        self.num_channels = self.o.K
        self.atomic_numbers = self.o.atomic_numbers
        self.inputs = None

    def build_neighbors(self, positions, types, cell, pbc, r_cut):
        s = st.Structure(np.asarray(positions), np.asarray(cell), np.asarray(types), tuple(pbc))
        nl = st.neighbor_list(s, r_cut)
        self.nl = nl
        n = s.num_atoms
        self.inputs = {"num_nodes": n, "node_types": np.asarray(types, np.int32),
                       "num_neigh": np.bincount(nl["i"], minlength=n).astype(np.int32), "neigh_indices": nl["j"],
                       "neigh_types": np.asarray(types, np.int32)[nl["j"]], "xyz": nl["D"].reshape(-1), "r": nl["d"]}
        self.full_inputs = self.inputs
        return nl["i"].size

    def _activate(self, n):
        inp = self.full_inputs
        e = int(np.sum(inp["num_neigh"][:n]))
        self.inputs = {"num_nodes": n, "node_types": inp["node_types"][:n], "num_neigh": inp["num_neigh"][:n],
                       "neigh_indices": inp["neigh_indices"][:e], "neigh_types": inp["neigh_types"][:e],
                       "xyz": inp["xyz"][:3 * e], "r": inp["r"][:e]}
        self.o._edges(self.inputs)
        self.o.compute_Y(); self.o.compute_R0(); self.o.compute_R1()
        if self.num_interactions == 3:
            self.o.compute_Rm()
        return e

    def restrict_nodes(self, n_own):
        """New evaluation on the first n_own receivers: outputs zero-filled."""
        self._nf_full = np.zeros((self.full_inputs["r"].size, 3))
        self._en_full = np.zeros(self.full_inputs["num_nodes"])
        e = self._activate(n_own)
        self.o.node_forces = np.zeros((e, 3))
        self.o.node_energies = np.zeros(n_own)
        return e

    def set_active_nodes(self, n):
        """Other receiver set, same evaluation: partial forces and node energies are carried over."""
        nf, en = self.o.node_forces, self.o.node_energies
        self._nf_full[: nf.shape[0]] = nf
        self._en_full[: en.shape[0]] = en
        e = self._activate(n)
        self.o.node_forces = self._nf_full[:e].copy()
        self.o.node_energies = self._en_full[:n].copy()
        return e

    def _stage(self, name, zero_dxyz=True, zero_H1_adj=True):
        getattr(self.o, name)()

    def resize_rows(self, name, rows):
        arr = getattr(self.o, name)
        extra = rows - arr.shape[0]
        setattr(self.o, name, np.ascontiguousarray(np.concatenate([arr, np.zeros((extra,) + arr.shape[1:])])))

    def device_view(self, name):
        arr = self._atom_forces if name == "atom_forces" else getattr(self.o, name)
        assert arr.flags["C_CONTIGUOUS"]
        return torch.from_numpy(arr.reshape(-1))

    def sync(self):
        pass

    @property
    def has_zbl(self):
        return bool(getattr(self.o, "has_zbl", False))

    # halo rows: the numpy statement of smx_halo_pack / _unpack / _unpack_add
    def _halo_array(self, name):
        if name == "atom_forces":
            return self._atom_forces
        arr = getattr(self.o, name)
        return arr.reshape(arr.shape[0], -1)

    def halo_pack(self, name, rows):
        return torch.from_numpy(self._halo_array(name)[rows.numpy()].copy())

    def halo_unpack(self, name, rows, buf, add=False):
        arr = self._halo_array(name)
        if add:
            np.add.at(arr, rows.numpy(), buf.numpy())      # sequential: contributions are added in list order
        else:
            arr[rows.numpy()] = buf.numpy()

    def atom_forces(self, num_rows):
        self._atom_forces = self.reduce_forces(num_rows)[0]

    def reduce_forces(self, num_rows, want_forces=True, device=False):
        inp = self.inputs
        nf = self.o.node_forces
        recv = np.repeat(np.arange(inp["num_nodes"]), inp["num_neigh"])
        f = np.zeros((num_rows, 3))
        np.add.at(f, recv, -nf)
        np.add.at(f, inp["neigh_indices"], nf)
        x = inp["xyz"].reshape(-1, 3)
        v = np.array([np.sum(x[:, 0] * nf[:, 0]), np.sum(x[:, 1] * nf[:, 1]), np.sum(x[:, 2] * nf[:, 2]),
                      0.5 * np.sum(x[:, 0] * nf[:, 1] + x[:, 1] * nf[:, 0]), 0.5 * np.sum(x[:, 0] * nf[:, 2] + x[:, 2] * nf[:, 0]),
                      0.5 * np.sum(x[:, 1] * nf[:, 2] + x[:, 2] * nf[:, 1])])
        return f, v, float(self.o.node_energies.sum())
