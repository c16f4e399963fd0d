"""Slab domain decomposition of the MACE evaluation across ranks (one GPU per rank).

The scheme is the reference pair style's message-passing mode (pair_symmetrix/pair_symmetrix_mace.cpp:
376-547): every rank owns the atoms of one slab, sees ghost copies of the atoms within ``r_cut`` of its
faces, evaluates layer 0 on its own atoms, receives ``H1`` rows for its ghosts, evaluates layer 1 and the
reverse pass down to ``reverse_Phi1``, returns the ``H1_adj`` rows of its ghosts to their owners (who add
them), finishes the reverse pass, and finally returns the force rows of its ghosts. What LAMMPS ``Comm``
does there over MPI (``forward_comm`` / ``reverse_comm``, pack/unpack at pair_symmetrix_mace.cpp:194-238)
is done here with point-to-point sends between slab neighbours (NCCL over NVLink on GPUs, gloo on CPU).

A second mode, "recompute" (the pair style's ``no_mpi_message_passing`` branch, pair_symmetrix_mace.cpp:551-748),
trades the two feature exchanges for redundant work: the ghost shell is ``2 r_cut`` wide, layer 0 and its reverse run
on the owned atoms and on the ghosts within ``r_cut`` (whose neighbourhoods the wider shell completes), layer 1 on the
owned atoms, and only the force rows of the ghosts travel. Both modes give the same energies and forces.

The decomposition is 1-D along one cell axis; periodic images along the other two axes map to the same
row (as the single-domain mode does with ``atom->map``, pair_symmetrix_mace.cpp:304-306), images along the
slab axis are explicit ghost rows. Every rank derives the full plan from the same global structure, so no
metadata has to be exchanged.
"""
from __future__ import annotations

from dataclasses import dataclass, field

import numpy as np

from .structures import Structure


@dataclass
class SlabPlan:
    rank: int
    world: int
    axis: int
    n_own: int
    n_ghost: int
    own_global: np.ndarray            # [n_own] global atom ids, ascending
    ghost_global: np.ndarray          # [n_ghost]
    ghost_owner: np.ndarray           # [n_ghost] owning rank
    ghost_image: np.ndarray           # [n_ghost] cell shift along the slab axis (-1, 0, +1)
    positions: np.ndarray             # [n_own + n_ghost, 3] local coordinates (ghosts at their image position)
    numbers: np.ndarray               # [n_own + n_ghost]
    cell: np.ndarray                  # [3, 3] cell used for the local neighbour list
    pbc: tuple
    peers: list = field(default_factory=list)        # ranks exchanged with, ascending
    send_rows: dict = field(default_factory=dict)    # peer -> local owned rows, in the peer's ghost order
    recv_rows: dict = field(default_factory=dict)    # peer -> local ghost rows (ascending)
    mode: str = "message_passing"                    # or "recompute"
    n_inner: int = 0                                 # recompute mode: ghosts within r_cut of the slab (they come first)
    n_within: list = field(default_factory=list)     # recompute mode: ghosts within 1, 2, ... r_cut (cumulative counts)


def _ghost_list(frac: np.ndarray, owner: np.ndarray, rank: int, world: int, shell: float, inner: float = None):
    """Ghost images of `rank`: (global id, image shift) of atoms whose image lies in the shell around its slab.

    `frac` is the fractional coordinate along the slab axis, `shell` the ghost width in the same units. With `inner`
    (the width of one sub-shell, `shell` being a multiple of it) the images are ordered by sub-shell, nearest first,
    and the cumulative counts per sub-shell are returned as well."""
    lo, hi = rank / world, (rank + 1) / world
    out_g, out_n, out_cls = [], [], []
    for n in (-1, 0, 1):
        x = frac + n
        sel = ((x >= lo - shell) & (x < lo)) | ((x >= hi) & (x < hi + shell))
        if n == 0:
            sel &= owner != rank
        idx = np.nonzero(sel)[0]
        out_g.append(idx)
        out_n.append(np.full(idx.size, n, dtype=np.int64))
        if inner is not None:
            xi = x[idx]
            # sub-shell c holds the images within (c + 1) * inner of the slab, decided with the same comparisons as `sel`
            num = max(1, int(round(shell / inner)))
            cls = np.full(idx.size, num - 1, dtype=np.int64)
            for c in range(num - 2, -1, -1):
                w = shell * (c + 1) / num if c + 1 < num else shell
                cls[((xi >= lo - w) & (xi < lo)) | ((xi >= hi) & (xi < hi + w))] = c
            out_cls.append(cls)
    g = np.concatenate(out_g)
    n = np.concatenate(out_n)
    if inner is None:
        order = np.lexsort((g, n, owner[g]))
        return g[order], n[order]
    cls = np.concatenate(out_cls)
    order = np.lexsort((g, n, owner[g], cls))
    num = max(1, int(round(shell / inner)))
    within = [int(np.count_nonzero(cls <= c)) for c in range(num)]
    return g[order], n[order], within


def make_slab_plan(s: Structure, r_cut: float, rank: int, world: int, axis: int = 0, mode: str = "message_passing",
                   num_interactions: int = 2) -> SlabPlan:
    """Plan of rank `rank` of `world` for structure `s` (positions inside the cell, orthogonal slab axis).

    `num_interactions` (2 or 3) only matters in recompute mode, whose ghost shell is one r_cut per interaction block."""
    if mode not in ("message_passing", "recompute"):
        raise ValueError(f"unknown decomposition mode {mode!r}")
    cell = np.asarray(s.cell, dtype=np.float64)
    other = [a for a in range(3) if a != axis]
    if any(abs(cell[axis, o]) > 1e-12 or abs(cell[o, axis]) > 1e-12 for o in other):
        raise ValueError("the slab axis must be orthogonal to the other two cell vectors")
    if not s.pbc[axis]:
        raise ValueError("the slab axis must be periodic")
    length = cell[axis, axis]
    if world > 1 and length / world < r_cut:
        raise ValueError(f"slabs of {length / world:.2f} A are thinner than r_cut = {r_cut} A")
    pos = np.asarray(s.positions, dtype=np.float64)
    frac = pos[:, axis] / length
    owner = np.clip(np.floor(frac * world).astype(np.int64), 0, world - 1)
    own = np.nonzero(owner == rank)[0]
    if world == 1:
        return SlabPlan(rank, world, axis, own.size, 0, own, np.zeros(0, np.int64), np.zeros(0, np.int64), np.zeros(0, np.int64),
                        pos[own].copy(), np.asarray(s.numbers)[own], cell.copy(), tuple(s.pbc))
    width = r_cut if mode == "message_passing" else float(num_interactions) * r_cut
    if 2.0 * width > length + 1e-9 and mode == "recompute":
        raise ValueError(f"a {width:.2f} A ghost shell on both sides does not fit into a cell of {length:.2f} A")
    shell = width / length
    n_inner, within = 0, []
    if mode == "recompute":
        g, n, within = _ghost_list(frac, owner, rank, world, shell, inner=r_cut / length)
        n_inner = within[0]
    else:
        g, n = _ghost_list(frac, owner, rank, world, shell)
    gpos = pos[g].copy()
    gpos[:, axis] += n * length
    positions = np.concatenate([pos[own], gpos])
    # local cell: open along the slab axis (ghost images are explicit), periodic as given along the others
    lcell = cell.copy()
    lo = rank * length / world - width
    positions[:, axis] -= lo
    lcell[axis, axis] = length / world + 2 * width
    pbc = tuple(False if a == axis else bool(s.pbc[a]) for a in range(3))
    plan = SlabPlan(rank, world, axis, own.size, g.size, own, g, owner[g], n, positions,
                    np.concatenate([np.asarray(s.numbers)[own], np.asarray(s.numbers)[g]]), lcell, pbc)
    plan.mode, plan.n_inner, plan.n_within = mode, n_inner, within
    plan.peers = sorted(set(int(q) for q in owner[g]))
    for q in plan.peers:
        plan.recv_rows[q] = own.size + np.nonzero(owner[g] == q)[0]
        # what I must send to q: q's ghost list restricted to atoms I own, in q's order
        gq = _ghost_list(frac, owner, q, world, shell, inner=r_cut / length if mode == "recompute" else None)[0]
        mine = gq[owner[gq] == rank]
        plan.send_rows[q] = np.searchsorted(own, mine)
    return plan


class SlabRank:
    """One rank's share of a decomposed evaluation, split into phases between which halos are exchanged.

    `backend` is the evaluator of this rank (``symmetrix_b200.MACE`` on a GPU); `xp` is the array module
    used for the halo buffers (torch).
    """

    def __init__(self, plan: SlabPlan, backend, r_cut: float, atomic_numbers):
        import torch
        self.torch = torch
        self.plan = plan
        self.ev = backend
        self.rows = plan.n_own + plan.n_ghost
        self.recompute = plan.mode == "recompute"
        self.blocks = int(getattr(backend, "num_interactions", 2))
        if self.recompute and len(plan.n_within) != self.blocks:
            raise ValueError("the plan's ghost shell does not match the model's number of interaction blocks")
        # receivers of block b: owned atoms, plus (recompute mode) the ghosts within (blocks - 1 - b) r_cut of the slab
        self.n_block = [plan.n_own + (plan.n_within[self.blocks - 2 - b] if self.recompute and b < self.blocks - 1 else 0)
                        for b in range(self.blocks)]
        self.n_layer0 = self.n_block[0]
        self.width = backend.num_LM * backend.num_channels
        zmap = {int(z): t for t, z in enumerate(atomic_numbers)}
        self.types = np.array([zmap[int(z)] for z in plan.numbers], dtype=np.int32)
        self.r_cut = r_cut
        self.device = self._device()
        self.send_idx = {q: torch.as_tensor(np.ascontiguousarray(r), dtype=torch.int32, device=self.device) for q, r in plan.send_rows.items()}
        self.recv_idx = {q: torch.as_tensor(np.ascontiguousarray(r), dtype=torch.int32, device=self.device) for q, r in plan.recv_rows.items()}
        self.has_zbl = bool(getattr(backend, "has_zbl", False))
        self.num_edges = 0
        # on a GPU the evaluator shares torch's current stream: pack / unpack kernels, NCCL and the evaluator's kernels are
        # then ordered by the stream and no host synchronisation is needed between phases
        self.shared_stream = self.device != "cpu" and hasattr(self.ev, "use_torch_stream")
        if self.shared_stream:
            self.ev.use_torch_stream(True)
        if hasattr(self.ev, "halo_cache_lists"):
            self.ev.halo_cache_lists(False)     # groupings kept for an earlier plan's lists (their addresses may come again)
            self.ev.halo_cache_lists(True)      # send_idx / recv_idx live as long as this object and are never rewritten
        self.stage_ms = None          # set to {} to collect per-stage device times (adds a stream sync per stage)

    def _run(self, stage, *flags):
        if self.stage_ms is None:
            self.ev._stage(stage, *flags)
        else:
            self.ev.timer_start()
            self.ev._stage(stage, *flags)
            self.stage_ms[stage] = self.stage_ms.get(stage, 0.0) + self.ev.timer_stop()

    def _device(self):
        dev = getattr(self.ev, "info", None)
        return f"cuda:{dev.device}" if dev is not None else "cpu"

    # ---------------------------------------------------------------- phases
    def build_edges(self):
        """Neighbour list of the local atoms (owned + ghosts); receivers are the owned atoms only."""
        p = self.plan
        self.ev.build_neighbors(p.positions, self.types, p.cell, p.pbc, r_cut=self.r_cut)
        self.num_edges = self.ev.restrict_nodes(self.n_layer0)

    def begin_step(self):
        """Re-arm the current edge set (zero node energies / partial forces) for another evaluation, then the pair
        repulsion on the owned atoms (pair_symmetrix_mace.cpp:449-452; owned atoms only in recompute mode, :667-670)."""
        self.ev.restrict_nodes(self.n_layer0)
        if self.has_zbl:
            if self.n_layer0 != self.plan.n_own:
                self.ev.set_active_nodes(self.plan.n_own)
                self._run("compute_ZBL")
                self.ev.set_active_nodes(self.n_layer0)
            else:
                self._run("compute_ZBL")

    # The density-normalisation stages (compute/reverse_A0_scaled, _A1_scaled) sit where the reference has them
    # (pair_symmetrix_mace.cpp:458,476,486,494 and :674,682,691,697); they do nothing for models without them.
    def forward_layer0(self):
        for stage in ("compute_A0", "compute_A0_scaled", "compute_M0", "compute_H1"):
            self._run(stage)
        if self.recompute:
            self.ev.set_active_nodes(self.n_block[1])      # next block on fewer receivers; H1 keeps its ghost rows
        else:
            self.ev.resize_rows("H1", self.rows)

    def forward_middle(self):
        """Middle block of a three-block model (features Hm from H1)."""
        self._sync_torch()
        for stage in ("compute_Phim", "compute_Am", "compute_Mm", "compute_Hm"):
            self._run(stage)
        if self.recompute:
            self.ev.set_active_nodes(self.n_block[2])
        else:
            self.ev.resize_rows("Hm", self.rows)

    # Halo rows are packed and unpacked by the evaluator's own kernels on its stream (smx_halo_pack / _unpack /
    # _unpack_add); what travels between the ranks are the packed buffers.
    def pack_forward(self, peer, name="H1"):
        return self.ev.halo_pack(name, self.send_idx[peer])

    def unpack_forward(self, peer, buf, name="H1"):
        self.ev.halo_unpack(name, self.recv_idx[peer], buf)

    def layer1_and_reverse(self):
        self._sync_torch()
        for stage in ("compute_Phi1", "compute_A1", "compute_A1_scaled", "compute_M1", "compute_H2", "compute_readouts"):
            self._run(stage)
        self._run("reverse_H2", True, False)
        self._run("reverse_M1")
        self._run("reverse_A1_scaled", False, True)
        self._run("reverse_A1")
        self._run("reverse_Phi1", False, False)

    def pack_reverse(self, peer, name="H1_adj"):
        return self.ev.halo_pack(name, self.recv_idx[peer])

    def unpack_reverse(self, peer, buf, name="H1_adj"):
        self.ev.halo_unpack(name, self.send_idx[peer], buf, add=True)     # fixed order of additions: reproducible bits

    def reverse_middle(self):
        self._sync_torch()
        if self.recompute:
            self.ev.set_active_nodes(self.n_block[1])      # the partial Hm_adj of the ghosts goes through the middle block here
        self._run("reverse_Hm")
        self._run("reverse_Mm")
        self._run("reverse_Am")
        self._run("reverse_Phim", False, False)

    def reverse_layer0(self):
        self._sync_torch()
        if self.recompute:
            self.ev.set_active_nodes(self.n_layer0)        # the partial H1_adj of the ghosts goes through layer 0 here
        for stage in ("reverse_H1", "reverse_M0", "reverse_A0_scaled", "reverse_A0"):
            self._run(stage)
        # per-atom forces stay in the evaluator's "atom_forces" array; on a GPU energy and virial stay on the device too,
        # so there is no host synchronisation before the force-row exchange
        self.ev.atom_forces(self.rows)
        _, self.virial, self.energy = self.ev.reduce_forces(num_rows=self.rows, want_forces=False, device=self.shared_stream)

    def pack_forces(self, peer):
        return self.ev.halo_pack("atom_forces", self.recv_idx[peer])

    def unpack_forces(self, peer, buf):
        self.ev.halo_unpack("atom_forces", self.send_idx[peer], buf, add=True)

    def owned_forces(self):
        return self.ev.device_view("atom_forces").view(-1, 3)[: self.plan.n_own].clone()

    def _sync_torch(self):
        if self.device != "cpu" and not self.shared_stream:
            self.torch.cuda.synchronize()


def _exchange(ranks, transport_fn, pack, unpack, dist=None, native=None):
    """One halo exchange. With `dist` (torch.distributed) there is exactly one local rank and messages go
    point to point; without it `ranks` holds every rank and messages are handed over in memory. `native` =
    (array name, add, forward?) lets an evaluator that holds its own NCCL communicator (``MACE.comm_init``) do the whole
    exchange inside the library; otherwise the packed buffers travel through ``torch.distributed``."""
    if dist is None:
        box = {}
        for r in ranks:
            for q in r.plan.peers:
                box[(r.plan.rank, q)] = pack(r, q)
        for r in ranks:
            for q in r.plan.peers:
                unpack(r, q, box[(q, r.plan.rank)])
        return
    import torch
    r = ranks[0]
    if native is not None and getattr(r.ev, "comm_ready", False):
        # the library's own transport: pack kernels, grouped ncclSend / ncclRecv and unpack kernels on the evaluator's stream
        name, add, forward = native
        r.ev.halo_exchange(name, add, r.plan.peers, r.send_idx if forward else r.recv_idx, r.recv_idx if forward else r.send_idx)
        return
    ops, recvs = [], {}
    sends = {q: pack(r, q) for q in r.plan.peers}
    for q in r.plan.peers:
        # the peer sends me what I unpack: shape = [rows I receive for this exchange, width of what I send]
        n_recv = transport_fn(r, q)
        recvs[q] = torch.empty((n_recv,) + tuple(sends[q].shape[1:]), dtype=sends[q].dtype, device=sends[q].device)
        ops.append(dist.P2POp(dist.isend, sends[q], q))
        ops.append(dist.P2POp(dist.irecv, recvs[q], q))
    for req in dist.batch_isend_irecv(ops) if ops else []:
        req.wait()
    for q in r.plan.peers:
        unpack(r, q, recvs[q])


def evaluate_decomposed(ranks, dist=None):
    """One energy+force evaluation over all slabs.

    `ranks` is a list of :class:`SlabRank` -- all ranks of the decomposition when `dist` is None (single-
    process emulation), or the single local rank when `dist` is an initialised ``torch.distributed``.
    Returns (total energy, virial[6], list of owned-force tensors per local rank).
    """
    recompute, deep = ranks[0].recompute, ranks[0].blocks == 3

    def forward_halo(name):
        if not recompute:
            _exchange(ranks, lambda r, q: r.recv_idx[q].numel(), lambda r, q: r.pack_forward(q, name),
                      lambda r, q, b: r.unpack_forward(q, b, name), dist, native=(name, False, True))

    def reverse_halo(name):
        if not recompute:
            _exchange(ranks, lambda r, q: r.send_idx[q].numel(), lambda r, q: r.pack_reverse(q, name),
                      lambda r, q, b: r.unpack_reverse(q, b, name), dist, native=(name, True, False))

    for r in ranks:
        r.begin_step()
        r.forward_layer0()
    forward_halo("H1")
    if deep:
        for r in ranks:
            r.forward_middle()
        forward_halo("Hm")
    for r in ranks:
        r.layer1_and_reverse()
    if deep:
        reverse_halo("Hm_adj")
        for r in ranks:
            r.reverse_middle()
    reverse_halo("H1_adj")
    for r in ranks:
        r.reverse_layer0()
    _exchange(ranks, lambda r, q: r.send_idx[q].numel(), lambda r, q: r.pack_forces(q), lambda r, q, b: r.unpack_forces(q, b), dist,
              native=("atom_forces", True, False))
    if ranks[0].shared_stream:
        import torch
        t = sum(torch.cat([r.energy, r.virial]) for r in ranks)      # seven float64 values on the device
        if dist is not None:
            if getattr(ranks[0].ev, "comm_ready", False):
                ranks[0].ev.allreduce_sum(t)
            else:
                dist.all_reduce(t)
        owned = [r.owned_forces() for r in ranks]
        vals = t.cpu().numpy()                                      # the only host synchronisation of the step
        for r in ranks:
            r.ev.sync()                                             # reports a device-side wait that ran out during the step
        return float(vals[0]), vals[1:], owned
    energy = sum(r.energy for r in ranks)
    virial = sum(np.asarray(r.virial) for r in ranks)
    if dist is not None:
        import torch
        t = torch.tensor([energy, *virial], dtype=torch.float64, device=ranks[0].device)
        dist.all_reduce(t)
        vals = t.cpu().numpy()
        energy, virial = float(vals[0]), vals[1:]
    return energy, virial, [r.owned_forces() for r in ranks]
