"""Python face of the evaluator, with the names of the reference's pybind11 classes.

``MACE`` mirrors ``symmetrix.MACE`` / ``symmetrix.MACEKokkos`` / ``symmetrix.MACEKokkosFloat``
(reference symmetrix/source/cpp/mace.cpp:10-243, mace_kokkos.cpp:11-420): same constructor
argument, same attribute names (``atomic_numbers``, ``r_cut``, ``node_energies``, ``node_forces``,
``A0`` ... ``H2_adj``, readable and writable) and the same ``compute_*`` / ``reverse_*`` methods.
Everything runs on the GPU through the C ABI; there is no CPU path.
"""
from __future__ import annotations

import ctypes

import numpy as np

from . import _lib

_ARRAYS = ["node_energies", "node_forces", "A0", "A0_adj", "M0", "M0_adj", "H1", "H1_adj", "Phi1", "Phi1_adj",
           "A1", "A1_adj", "M1", "M1_adj", "H2", "H2_adj",
           # middle interaction block of models with three blocks (no counterpart in the reference)
           "Phim", "Phim_adj", "Am", "Am_adj", "Mm", "Mm_adj", "Hm", "Hm_adj"]


class SymmetrixError(RuntimeError):
    def __init__(self, status: int, message: str):
        super().__init__(f"[symmetrix_b200 status {status}] {message}")
        self.status = status


def _is_device_tensor(x) -> bool:
    return hasattr(x, "data_ptr") and getattr(x, "is_cuda", False)


class _Arg:
    """A host numpy array or a CUDA tensor, normalised to (pointer, keep-alive object)."""

    def __init__(self, x, dtype, device_ok: bool):
        if _is_device_tensor(x):
            if not device_ok:
                raise ValueError("cannot mix host and device arrays in one call")
            import torch
            want = {np.int32: torch.int32, np.float64: torch.float64}[dtype]
            if x.dtype != want or not x.is_contiguous():
                x = x.to(want).contiguous()
            self.obj, self.ptr, self.size, self.device = x, ctypes.c_void_p(x.data_ptr()), x.numel(), True
        else:
            a = np.ascontiguousarray(x, dtype=dtype).reshape(-1)
            self.obj, self.ptr, self.size, self.device = a, ctypes.c_void_p(a.ctypes.data), a.size, False


class MACE:
    """B200 evaluator with the interface of the reference's ``MACE`` class (mace.hpp:12-169)."""

    def __init__(self, filename, dtype: str = "float64", device: int = 0):
        if dtype not in ("float32", "float64"):
            raise ValueError(f"Unsupported dtype '{dtype}'. Supported dtypes are 'float64' and 'float32'.")
        self._lib = _lib.load()
        self._h = ctypes.c_void_p()
        prec = _lib.SMX_FP64 if dtype == "float64" else _lib.SMX_FP32
        status = self._lib.smx_create(str(filename).encode(), prec, int(device), ctypes.byref(self._h))
        if status != _lib.SMX_OK:
            msg = self._lib.smx_last_error(None).decode()
            self._h = ctypes.c_void_p()
            raise SymmetrixError(status, msg)
        info = _lib.ModelInfo()
        self._check(self._lib.smx_info(self._h, ctypes.byref(info)))
        self.info = info
        self.dtype = dtype
        self.num_elements, self.num_channels, self.r_cut = info.num_elements, info.num_channels, info.r_cut
        self.l_max, self.num_lm, self.L_max, self.num_LM = info.l_max, info.num_lm, info.L_max, info.num_LM
        self.num_lme, self.num_lelm1lm2, self.has_zbl = info.num_lme, info.num_lelm1lm2, bool(info.has_zbl)
        self.num_interactions = info.num_interactions
        buf = (ctypes.c_int * info.num_elements)()
        self._lib.smx_atomic_numbers(self._h, ctypes.cast(buf, ctypes.c_void_p), info.num_elements)
        self.atomic_numbers = list(buf)
        ebuf = (ctypes.c_double * info.num_elements)()
        self._lib.smx_atomic_energies(self._h, ctypes.cast(ebuf, ctypes.c_void_p), info.num_elements)
        self.atomic_energies = list(ebuf)
        self._num_nodes = 0
        self._num_edges = 0
        self.comm_ready = False

    # ------------------------------------------------------------------ plumbing
    def close(self):
        if getattr(self, "_h", None) and self._h.value:
            self._lib.smx_destroy(self._h)
            self._h = ctypes.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _check(self, status: int):
        if status != _lib.SMX_OK:
            raise SymmetrixError(status, self._lib.smx_last_error(self._h).decode())

    def _edge_call(self, fn, num_nodes, node_types, num_neigh, neigh_indices, neigh_types, xyz, r):
        dev = _is_device_tensor(xyz)
        args = [_Arg(node_types, np.int32, dev), _Arg(num_neigh, np.int32, dev), _Arg(neigh_indices, np.int32, dev),
                _Arg(neigh_types, np.int32, dev), _Arg(xyz, np.float64, dev), _Arg(r, np.float64, dev)]
        if any(a.device != dev for a in args):
            raise ValueError("all edge arrays must live in the same memory space")
        num_edges = args[5].size
        if args[4].size != 3 * num_edges or args[2].size != num_edges or args[3].size != num_edges:
            raise ValueError("edge arrays have inconsistent lengths")
        if args[0].size < num_nodes or args[1].size < num_nodes:
            raise ValueError("node arrays are shorter than num_nodes")
        self._keep = args   # device inputs are used in place: keep them alive until the next call
        self._check(fn(self._h, int(num_nodes), args[0].ptr, args[1].ptr, args[2].ptr, args[3].ptr, args[4].ptr, args[5].ptr,
                       int(num_edges), _lib.SMX_DEVICE if dev else _lib.SMX_HOST))
        self._num_nodes, self._num_edges = int(num_nodes), int(num_edges)

    # ------------------------------------------------------------------ whole evaluation
    def compute_node_energies_forces(self, num_nodes, node_types, num_neigh, neigh_indices, neigh_types, xyz, r):
        """``MACE::compute_node_energies_forces`` (mace.cpp:17-64)."""
        self._edge_call(self._lib.smx_compute, num_nodes, node_types, num_neigh, neigh_indices, neigh_types, xyz, r)

    def begin(self, num_nodes, node_types, num_neigh, neigh_indices, neigh_types, xyz, r):
        """Set the edge set for a sequence of stage calls and zero ``node_energies`` / ``node_forces``
        (what the message-passing pair style does by hand, pair_symmetrix_mace.cpp:437-440)."""
        self._edge_call(self._lib.smx_begin, num_nodes, node_types, num_neigh, neigh_indices, neigh_types, xyz, r)

    def _stage(self, name, zero_dxyz=True, zero_H1_adj=True):
        self._check(self._lib.smx_stage(self._h, name.encode(), int(zero_dxyz), int(zero_H1_adj)))

    # Stage methods. They take the reference's argument lists for source compatibility, but the
    # edge arrays in effect are those of the last begin() / compute_node_energies_forces().
    def compute_ZBL(self, *a): self._stage("compute_ZBL")
    def compute_Y(self, *a): self._stage("compute_Y")
    def compute_R0(self, *a): self._stage("compute_R0")
    def compute_R1(self, *a): self._stage("compute_R1")
    def compute_A0(self, *a): self._stage("compute_A0")
    def compute_A0_scaled(self, *a): self._stage("compute_A0_scaled")
    def compute_M0(self, *a): self._stage("compute_M0")
    def compute_H1(self, *a): self._stage("compute_H1")
    def compute_Phi1(self, *a): self._stage("compute_Phi1")
    def compute_A1(self, *a): self._stage("compute_A1")
    def compute_A1_scaled(self, *a): self._stage("compute_A1_scaled")
    def compute_M1(self, *a): self._stage("compute_M1")
    def compute_H2(self, *a): self._stage("compute_H2")
    def compute_readouts(self, *a): self._stage("compute_readouts")
    def reverse_M1(self, *a): self._stage("reverse_M1")
    def reverse_A1(self, *a): self._stage("reverse_A1")
    def reverse_A1_scaled(self, *a, zero_dxyz=True): self._stage("reverse_A1_scaled", zero_dxyz, True)
    def reverse_H1(self, *a): self._stage("reverse_H1")
    def reverse_M0(self, *a): self._stage("reverse_M0")
    def reverse_A0_scaled(self, *a): self._stage("reverse_A0_scaled")
    def reverse_A0(self, *a): self._stage("reverse_A0")

    # Middle interaction block (models whose file says "num_interactions": 3; the reference stops at two blocks)
    def compute_Rm(self, *a): self._stage("compute_Rm")
    def compute_Phim(self, *a): self._stage("compute_Phim")
    def compute_Am(self, *a): self._stage("compute_Am")
    def compute_Mm(self, *a): self._stage("compute_Mm")
    def compute_Hm(self, *a): self._stage("compute_Hm")
    def reverse_Hm(self, *a): self._stage("reverse_Hm")
    def reverse_Mm(self, *a): self._stage("reverse_Mm")
    def reverse_Am(self, *a): self._stage("reverse_Am")

    def reverse_Phim(self, *a, zero_dxyz=True, zero_H1_adj=True):
        self._stage("reverse_Phim", zero_dxyz, zero_H1_adj)

    def reverse_H2(self, *a, zero_H1_adj=True):
        self._stage("reverse_H2", True, zero_H1_adj)

    def reverse_Phi1(self, *a, zero_dxyz=True, zero_H1_adj=True):
        self._stage("reverse_Phi1", zero_dxyz, zero_H1_adj)

    # ------------------------------------------------------------------ arrays
    def get(self, name: str) -> np.ndarray:
        n = ctypes.c_long(0)
        self._check(self._lib.smx_get_array(self._h, name.encode(), None, 0, ctypes.byref(n), _lib.SMX_HOST))
        out = np.empty(n.value, dtype=np.float64)
        if n.value:
            self._check(self._lib.smx_get_array(self._h, name.encode(), ctypes.c_void_p(out.ctypes.data), n.value,
                                                ctypes.byref(n), _lib.SMX_HOST))
        return out

    def set(self, name: str, values) -> None:
        a = np.ascontiguousarray(values, dtype=np.float64).reshape(-1)
        self._check(self._lib.smx_set_array(self._h, name.encode(), ctypes.c_void_p(a.ctypes.data), a.size, _lib.SMX_HOST))

    def reduce_forces(self, num_rows=None, want_forces=True, want_virial=True, device=False):
        """Per-atom forces ``[num_rows, 3]``, virial ``[6]`` (xx, yy, zz, xy, xz, yz) and total energy.

        With ``device=True`` the three results are float64 torch tensors on the evaluator's GPU (the energy has
        shape ``[1]``), written asynchronously on the evaluator's stream: no host synchronisation happens."""
        rows = self._num_nodes if num_rows is None else int(num_rows)
        if device:
            import torch
            dev = f"cuda:{self.info.device}"
            f = torch.zeros((rows, 3), dtype=torch.float64, device=dev) if want_forces else None
            v = torch.zeros(6, dtype=torch.float64, device=dev) if want_virial else None
            e = torch.zeros(1, dtype=torch.float64, device=dev)
            self._check(self._lib.smx_reduce_forces(
                self._h, rows, ctypes.c_void_p(f.data_ptr()) if want_forces else None,
                ctypes.c_void_p(v.data_ptr()) if want_virial else None, ctypes.c_void_p(e.data_ptr()), _lib.SMX_DEVICE))
            return f, v, e
        f = np.zeros((rows, 3)) if want_forces else None
        v = np.zeros(6) if want_virial else None
        e = ctypes.c_double(0.0)
        self._check(self._lib.smx_reduce_forces(
            self._h, rows, ctypes.c_void_p(f.ctypes.data) if want_forces else None,
            ctypes.c_void_p(v.ctypes.data) if want_virial else None, ctypes.cast(ctypes.byref(e), ctypes.c_void_p),
            _lib.SMX_HOST))
        return f, v, e.value

    @property
    def last_device_ms(self) -> float:
        ms = ctypes.c_double(0.0)
        self._check(self._lib.smx_last_device_ms(self._h, ctypes.byref(ms)))
        return ms.value

    def timer_start(self) -> None:
        self._check(self._lib.smx_timer_start(self._h))

    def timer_stop(self) -> float:
        ms = ctypes.c_double(0.0)
        self._check(self._lib.smx_timer_stop(self._h, ctypes.byref(ms)))
        return ms.value

    def measure_row_stream(self, layer: int):
        """(device ms, bytes) of a kernel that only streams the spline row of every current edge from the table of
        interaction layer `layer`: the floor the L2 -> SM path sets for one pass of an edge kernel."""
        ms, nbytes = ctypes.c_double(0.0), ctypes.c_double(0.0)
        self._check(self._lib.smx_measure_row_stream(self._h, int(layer), ctypes.byref(ms), ctypes.byref(nbytes)))
        return ms.value, nbytes.value

    def validate_inputs(self, feature_rows=None):
        """Counts per kind of the out-of-range or inconsistent entries of the current edge set (all zero for good inputs):
        node type, negative neighbour count, counts not adding up, sender index, sender type, r out of range, r vs |xyz|."""
        rows = self._num_nodes if feature_rows is None else int(feature_rows)
        counts = (ctypes.c_long * 7)()
        total = ctypes.c_long(0)
        status = self._lib.smx_validate_inputs(self._h, rows, counts, ctypes.byref(total))
        if status not in (_lib.SMX_OK, _lib.SMX_ERR_INVALID_ARGUMENT):
            self._check(status)
        return list(counts)

    def set_profiling(self, enabled: bool) -> None:
        self._check(self._lib.smx_set_profiling(self._h, int(bool(enabled))))

    def stage_times(self) -> dict:
        """Device milliseconds of each stage of the last whole evaluation (profiling must be on)."""
        out = {}
        buf = ctypes.create_string_buffer(64)
        ms = ctypes.c_double(0.0)
        for idx in range(23 if self.num_interactions == 3 else 15):
            if self._lib.smx_stage_time(self._h, idx, buf, 64, ctypes.byref(ms)) != _lib.SMX_OK:
                break
            out[buf.value.decode()] = ms.value
        return out

    @property
    def launch_count(self) -> int:
        return int(self._lib.smx_launch_count(self._h))

    # ------------------------------------------------------------------ neighbour list
    def build_neighbors(self, positions, types, cell, pbc=(True, True, True), r_cut=None) -> int:
        """Build the edge set on the device (``smx_build_neighbors``); returns the number of edges."""
        pos = np.ascontiguousarray(positions, dtype=np.float64).reshape(-1, 3)
        ty = np.ascontiguousarray(types, dtype=np.int32).reshape(-1)
        c = np.ascontiguousarray(cell, dtype=np.float64).reshape(9)
        pb = np.ascontiguousarray([1 if b else 0 for b in pbc], dtype=np.int32)
        n = ctypes.c_long(0)
        self._check(self._lib.smx_build_neighbors(
            self._h, pos.shape[0], ctypes.c_void_p(pos.ctypes.data), ctypes.c_void_p(ty.ctypes.data),
            ctypes.c_void_p(c.ctypes.data), ctypes.c_void_p(pb.ctypes.data), float(self.r_cut if r_cut is None else r_cut),
            ctypes.byref(n), _lib.SMX_HOST))
        self._num_nodes, self._num_edges = pos.shape[0], n.value
        return n.value

    def get_edges(self) -> dict:
        n, e = self._num_nodes, self._num_edges
        out = {"num_neigh": np.zeros(n, np.int32), "neigh_indices": np.zeros(e, np.int32), "neigh_types": np.zeros(e, np.int32),
               "shifts": np.zeros((e, 3), np.int32), "xyz": np.zeros((e, 3)), "r": np.zeros(e)}
        p = lambda a: ctypes.c_void_p(a.ctypes.data)  # noqa: E731
        self._check(self._lib.smx_get_edges(self._h, p(out["num_neigh"]), p(out["neigh_indices"]), p(out["neigh_types"]),
                                            p(out["shifts"]), p(out["xyz"]), p(out["r"]), _lib.SMX_HOST))
        return out

    def compute_current(self) -> None:
        self._check(self._lib.smx_compute_current(self._h))

    # ------------------------------------------------------------------ helpers for decomposed drivers
    def sync(self) -> None:
        self._check(self._lib.smx_sync(self._h))

    def use_torch_stream(self, enable: bool = True) -> None:
        """Issue the evaluator's work on torch's current CUDA stream, so torch kernels and NCCL calls are ordered with it."""
        import torch
        ptr = torch.cuda.current_stream(self.info.device).cuda_stream if enable else None
        self._check(self._lib.smx_set_stream(self._h, ctypes.c_void_p(ptr), 1 if enable else 0))

    def restrict_nodes(self, num_nodes: int) -> int:
        """Keep the first ``num_nodes`` receivers of the current edge set (owned atoms first); returns the edge count."""
        n = ctypes.c_long(0)
        self._check(self._lib.smx_restrict_nodes(self._h, int(num_nodes), ctypes.byref(n)))
        self._num_nodes, self._num_edges = int(num_nodes), n.value
        return n.value

    def set_active_nodes(self, num_nodes: int) -> int:
        """Like :meth:`restrict_nodes`, but in the middle of an evaluation: the outputs accumulated so far and the feature
        rows beyond the active nodes are kept (recompute mode of the pair style: layer 0 on owned + ghost atoms, layer 1 on
        owned atoms)."""
        n = ctypes.c_long(0)
        self._check(self._lib.smx_set_active_nodes(self._h, int(num_nodes), ctypes.byref(n)))
        self._num_nodes, self._num_edges = int(num_nodes), n.value
        return n.value

    def resize_rows(self, name: str, rows: int) -> None:
        self._check(self._lib.smx_resize_rows(self._h, name.encode(), int(rows)))

    # Halo rows of a decomposed run, as kernels on the evaluator's stream (smx_halo_pack / _unpack / _unpack_add).
    # `rows` is an int32 CUDA tensor of row indices; buffers are CUDA tensors of the array's own element type.
    def _halo_dtype(self, name: str):
        import torch
        return torch.float64 if name == "atom_forces" or self.dtype == "float64" else torch.float32

    def halo_pack(self, name: str, rows):
        """``buf[m] = array[rows[m]]`` for the named array ("H1", "H1_adj", "Hm", "Hm_adj" or "atom_forces")."""
        import torch
        width = 3 if name == "atom_forces" else self.num_LM * self.num_channels
        buf = torch.empty((rows.numel(), width), dtype=self._halo_dtype(name), device=rows.device)
        self._check(self._lib.smx_halo_pack(self._h, name.encode(), ctypes.c_void_p(rows.data_ptr()), rows.numel(),
                                            ctypes.c_void_p(buf.data_ptr())))
        return buf

    def halo_unpack(self, name: str, rows, buf, add: bool = False) -> None:
        """``array[rows[m]] = buf[m]`` or, with ``add``, ``+=`` with each row's contributions added in list order
        (bitwise reproducible, also when a row occurs several times)."""
        if buf.dtype != self._halo_dtype(name) or not buf.is_contiguous():
            buf = buf.to(self._halo_dtype(name)).contiguous()
        fn = self._lib.smx_halo_unpack_add if add else self._lib.smx_halo_unpack
        self._check(fn(self._h, name.encode(), ctypes.c_void_p(rows.data_ptr()), rows.numel(), ctypes.c_void_p(buf.data_ptr())))

    def atom_forces(self, num_rows: int) -> None:
        """Per-atom forces of the current edge set into the device array "atom_forces" (no copy, no synchronisation)."""
        self._check(self._lib.smx_atom_forces(self._h, int(num_rows)))

    def active_counts(self):
        """(active receivers, their edges, receivers the edge set was built with)."""
        n, e, b = ctypes.c_int(0), ctypes.c_long(0), ctypes.c_int(0)
        self._check(self._lib.smx_active_counts(self._h, ctypes.byref(n), ctypes.byref(e), ctypes.byref(b)))
        return n.value, e.value, b.value

    def halo_cache_lists(self, enable: bool) -> None:
        """Keep (True) or drop (False) the per-list groupings of ``halo_unpack(add=True)`` / ``halo_exchange(add=True)``;
        only for index lists that are not changed in place."""
        self._check(self._lib.smx_halo_cache_lists(self._h, 1 if enable else 0))

    def debug_expire_waits(self, polls: int) -> None:
        """Test switch: make the first bounded wait of every float32 tensor-core GEMM CTA run out after `polls` polls."""
        self._check(self._lib.smx_debug_expire_waits(self._h, int(polls)))

    # NCCL transport inside the library (smx_comm_init / smx_halo_exchange / smx_allreduce_sum)
    def comm_init(self, dist) -> None:
        """Create the library's own NCCL communicator over the ranks of an initialised ``torch.distributed`` group; the
        128-byte id made by rank 0 travels through ``dist.broadcast_object_list``. Collective."""
        rank, world = dist.get_rank(), dist.get_world_size()
        box = [None]
        if rank == 0:
            buf = ctypes.create_string_buffer(128)
            status = self._lib.smx_comm_unique_id(buf, 128)
            if status != _lib.SMX_OK:
                raise SymmetrixError(status, self._lib.smx_last_error(None).decode())
            box[0] = buf.raw
        dist.broadcast_object_list(box, src=0)
        self._check(self._lib.smx_comm_init(self._h, box[0], 128, world, rank))
        self.comm_ready = True

    def halo_exchange(self, name: str, add: bool, peers, send_rows, recv_rows) -> None:
        """One exchange with the ranks `peers`: rows ``send_rows[q]`` of the named array go to peer q, the rows received
        from it are written (or, with `add`, added in a fixed order) to ``recv_rows[q]``. Index lists are int32 CUDA tensors."""
        n = len(peers)
        c_peers = (ctypes.c_int * n)(*[int(q) for q in peers])
        c_send = (ctypes.c_void_p * n)(*[send_rows[q].data_ptr() for q in peers])
        c_recv = (ctypes.c_void_p * n)(*[recv_rows[q].data_ptr() for q in peers])
        c_ns = (ctypes.c_int * n)(*[send_rows[q].numel() for q in peers])
        c_nr = (ctypes.c_int * n)(*[recv_rows[q].numel() for q in peers])
        self._check(self._lib.smx_halo_exchange(self._h, name.encode(), int(bool(add)), n, c_peers, c_send, c_ns, c_recv, c_nr))

    def allreduce_sum(self, values) -> None:
        """In-place sum of a float64 CUDA tensor over the ranks of the library's communicator."""
        self._check(self._lib.smx_allreduce_sum(self._h, ctypes.c_void_p(values.data_ptr()), values.numel()))

    def device_view(self, name: str):
        """Zero-copy torch view (1-D, float32 or float64) of a named device array; valid until that array is resized."""
        import torch
        ptr, n, eb = ctypes.c_void_p(), ctypes.c_long(0), ctypes.c_int(0)
        self._check(self._lib.smx_device_ptr(self._h, name.encode(), ctypes.byref(ptr), ctypes.byref(n), ctypes.byref(eb)))
        if n.value == 0:
            return torch.empty(0, dtype=torch.float64 if eb.value == 8 else torch.float32, device=f"cuda:{self.info.device}")

        class _View:
            __cuda_array_interface__ = {"shape": (n.value,), "typestr": "<f8" if eb.value == 8 else "<f4",
                                        "data": (ptr.value, False), "version": 2}
        return torch.as_tensor(_View(), device=f"cuda:{self.info.device}")


def _array_property(name):
    def getter(self):
        return self.get(name)

    def setter(self, values):
        self.set(name, values)

    return property(getter, setter)


for _name in _ARRAYS:
    setattr(MACE, _name, _array_property(_name))


class MACEKokkos(MACE):
    """Name kept for callers of the reference's device class (float64)."""

    def __init__(self, filename, device: int = 0):
        super().__init__(filename, "float64", device)


class MACEKokkosFloat(MACE):
    """Name kept for callers of the reference's float32 device class."""

    def __init__(self, filename, device: int = 0):
        super().__init__(filename, "float32", device)
