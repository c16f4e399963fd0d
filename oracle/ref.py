"""Test infrastructure: ctypes driver for ``oracle/_ref`` (the reference's own CPU evaluator,
compiled by ``oracle/build_ref.py``). Only tests, the smoke check and the CPU-baseline leg of
the benchmark may import this module; the product never does.
"""
from __future__ import annotations

import ctypes
from pathlib import Path

import numpy as np

_HERE = Path(__file__).resolve().parent
_c_int_p = ctypes.POINTER(ctypes.c_int)
_c_dbl_p = ctypes.POINTER(ctypes.c_double)


def available(variant: str = "parity") -> bool:
    return (_HERE / "_ref" / f"libref_{variant}.so").is_file()


def _load(variant: str):
    lib = ctypes.CDLL(str(_HERE / "_ref" / f"libref_{variant}.so"))
    lib.ref_create.restype = ctypes.c_void_p
    lib.ref_create.argtypes = [ctypes.c_char_p]
    lib.ref_destroy.argtypes = [ctypes.c_void_p]
    lib.ref_last_error.restype = ctypes.c_char_p
    lib.ref_info.argtypes = [ctypes.c_void_p, _c_int_p, _c_dbl_p]
    lib.ref_atomic_numbers.argtypes = [ctypes.c_void_p, _c_int_p, ctypes.c_int]
    lib.ref_atomic_numbers.restype = ctypes.c_int
    lib.ref_compute.argtypes = [ctypes.c_void_p, ctypes.c_int, _c_int_p, _c_int_p, _c_int_p, _c_int_p,
                                _c_dbl_p, _c_dbl_p, ctypes.c_long]
    lib.ref_stage.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.c_int, _c_int_p, _c_int_p, _c_int_p,
                              _c_int_p, _c_dbl_p, _c_dbl_p, ctypes.c_long, ctypes.c_int, ctypes.c_int]
    lib.ref_get.argtypes = [ctypes.c_void_p, ctypes.c_char_p, ctypes.POINTER(_c_dbl_p)]
    lib.ref_get.restype = ctypes.c_long
    lib.ref_set.argtypes = [ctypes.c_void_p, ctypes.c_char_p, _c_dbl_p, ctypes.c_long]
    lib.ref_real_sph_harm_xyz.restype = ctypes.c_double
    lib.ref_real_sph_harm_xyz.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.c_double, ctypes.c_double, ctypes.c_double]
    return lib


def _ip(a):
    return a.ctypes.data_as(_c_int_p)


def _dp(a):
    return a.ctypes.data_as(_c_dbl_p)


class ReferenceMACE:
    """The reference ``MACE`` class (libsymmetrix/source/mace.hpp:12-169) behind ctypes."""

    def __init__(self, json_path, variant: str = "parity"):
        self._lib = _load(variant)
        self._h = self._lib.ref_create(str(json_path).encode())
        if not self._h:
            raise RuntimeError(self._lib.ref_last_error().decode())
        info = (ctypes.c_int * 7)()
        rc = ctypes.c_double()
        self._lib.ref_info(self._h, info, ctypes.byref(rc))
        (self.num_elements, self.num_channels, self.l_max, self.L_max,
         self.num_lelm1lm2, self.num_lme, zbl) = list(info)
        self.has_zbl = bool(zbl)
        self.r_cut = rc.value
        buf = (ctypes.c_int * 128)()
        n = self._lib.ref_atomic_numbers(self._h, buf, 128)
        self.atomic_numbers = list(buf[:n])

    def __del__(self):
        if getattr(self, "_h", None):
            self._lib.ref_destroy(self._h)
            self._h = None

    @staticmethod
    def _prep(inputs):
        return (int(inputs["num_nodes"]),
                np.ascontiguousarray(inputs["node_types"], dtype=np.int32),
                np.ascontiguousarray(inputs["num_neigh"], dtype=np.int32),
                np.ascontiguousarray(inputs["neigh_indices"], dtype=np.int32),
                np.ascontiguousarray(inputs["neigh_types"], dtype=np.int32),
                np.ascontiguousarray(inputs["xyz"], dtype=np.float64).reshape(-1),
                np.ascontiguousarray(inputs["r"], dtype=np.float64))

    def compute_node_energies_forces(self, inputs):
        n, nt, nn, ni, et, xyz, r = self._prep(inputs)
        rc = self._lib.ref_compute(self._h, n, _ip(nt), _ip(nn), _ip(ni), _ip(et), _dp(xyz), _dp(r), r.size)
        if rc:
            raise RuntimeError(self._lib.ref_last_error().decode())
        return self.get("node_energies")[:n].copy(), self.get("node_forces")[: 3 * r.size].copy()

    def stage(self, name: str, inputs, flag0: bool = True, flag1: bool = True):
        n, nt, nn, ni, et, xyz, r = self._prep(inputs)
        rc = self._lib.ref_stage(self._h, name.encode(), n, _ip(nt), _ip(nn), _ip(ni), _ip(et), _dp(xyz), _dp(r),
                                 r.size, int(flag0), int(flag1))
        if rc:
            raise RuntimeError(self._lib.ref_last_error().decode())

    def get(self, name: str) -> np.ndarray:
        p = _c_dbl_p()
        n = self._lib.ref_get(self._h, name.encode(), ctypes.byref(p))
        if n < 0:
            raise KeyError(name)
        if n == 0:
            return np.zeros(0)
        return np.ctypeslib.as_array(p, shape=(n,)).copy()

    def set(self, name: str, values):
        v = np.ascontiguousarray(values, dtype=np.float64).reshape(-1)
        if self._lib.ref_set(self._h, name.encode(), _dp(v), v.size):
            raise KeyError(name)


def real_sph_harm_xyz(l, m, x, y, z, variant: str = "parity") -> float:
    return _load(variant).ref_real_sph_harm_xyz(l, m, x, y, z)
