"""ctypes binding of ``libsymmetrix_b200.so`` (the C ABI declared in ``include/symmetrix_b200.h``).

There is deliberately no fallback: if the shared library is missing, or no CUDA device is
usable, creating an evaluator raises.
"""
from __future__ import annotations

import ctypes
from pathlib import Path

PKG = Path(__file__).resolve().parent
LIB_PATH = PKG / "libsymmetrix_b200.so"

SMX_HOST, SMX_DEVICE = 0, 1
SMX_FP32, SMX_FP64 = 32, 64
SMX_OK, SMX_ERR_INVALID_ARGUMENT, SMX_ERR_MODEL, SMX_ERR_CUDA, SMX_ERR_UNSUPPORTED, SMX_ERR_NO_DEVICE = range(6)

# every symbol the header declares (checked by the CPU test-suite against the built library)
EXPORTED_SYMBOLS = [
    "smx_create", "smx_destroy", "smx_last_error", "smx_info", "smx_atomic_numbers", "smx_atomic_energies",
    "smx_compute", "smx_begin", "smx_stage", "smx_get_array", "smx_set_array", "smx_reduce_forces",
    "smx_last_device_ms", "smx_launch_count", "smx_build_neighbors", "smx_get_edges", "smx_compute_current",
    "smx_timer_start", "smx_timer_stop", "smx_set_profiling", "smx_stage_time", "smx_measure_fma_peak", "smx_measure_row_stream", "smx_validate_inputs",
    "smx_energy_virial_noalloc", "smx_sync", "smx_set_stream", "smx_restrict_nodes", "smx_set_active_nodes", "smx_resize_rows", "smx_device_ptr",
    "smx_halo_pack", "smx_halo_unpack", "smx_halo_unpack_add", "smx_halo_cache_lists", "smx_atom_forces", "smx_active_counts", "smx_debug_expire_waits",
    "smx_comm_unique_id", "smx_comm_init", "smx_comm_destroy", "smx_halo_exchange", "smx_allreduce_sum", "smx_model_digest",
]


class ModelInfo(ctypes.Structure):
    _fields_ = [
        ("num_elements", ctypes.c_int), ("num_channels", ctypes.c_int), ("r_cut", ctypes.c_double),
        ("l_max", ctypes.c_int), ("num_lm", ctypes.c_int), ("L_max", ctypes.c_int), ("num_LM", ctypes.c_int),
        ("num_paths", ctypes.c_int), ("num_lelm1lm2", ctypes.c_int), ("num_lme", ctypes.c_int),
        ("has_zbl", ctypes.c_int), ("precision", ctypes.c_int), ("device", ctypes.c_int),
        ("num_interactions", ctypes.c_int),
    ]


_lib = None


def load():
    """Load the shared library (once) and declare the argument types of every entry point."""
    global _lib
    if _lib is not None:
        return _lib
    if not LIB_PATH.is_file():
        raise RuntimeError(
            f"{LIB_PATH} is missing: build it with `python -m symmetrix_b200.build` (there is no CPU fallback)")
    lib = ctypes.CDLL(str(LIB_PATH))
    vp, ip, dp, lp = ctypes.c_void_p, ctypes.c_void_p, ctypes.c_void_p, ctypes.POINTER(ctypes.c_long)
    lib.smx_create.argtypes = [ctypes.c_char_p, ctypes.c_int, ctypes.c_int, ctypes.POINTER(vp)]
    lib.smx_destroy.argtypes = [vp]
    lib.smx_destroy.restype = None
    lib.smx_last_error.argtypes = [vp]
    lib.smx_last_error.restype = ctypes.c_char_p
    lib.smx_info.argtypes = [vp, ctypes.POINTER(ModelInfo)]
    lib.smx_atomic_numbers.argtypes = [vp, ip, ctypes.c_int]
    lib.smx_atomic_energies.argtypes = [vp, dp, ctypes.c_int]
    edge_args = [vp, ctypes.c_int, ip, ip, ip, ip, dp, dp, ctypes.c_long, ctypes.c_int]
    lib.smx_compute.argtypes = edge_args
    lib.smx_begin.argtypes = edge_args
    lib.smx_stage.argtypes = [vp, ctypes.c_char_p, ctypes.c_int, ctypes.c_int]
    lib.smx_get_array.argtypes = [vp, ctypes.c_char_p, dp, ctypes.c_long, lp, ctypes.c_int]
    lib.smx_set_array.argtypes = [vp, ctypes.c_char_p, dp, ctypes.c_long, ctypes.c_int]
    lib.smx_reduce_forces.argtypes = [vp, ctypes.c_int, dp, dp, dp, ctypes.c_int]
    lib.smx_last_device_ms.argtypes = [vp, ctypes.POINTER(ctypes.c_double)]
    lib.smx_launch_count.argtypes = [vp]
    lib.smx_launch_count.restype = ctypes.c_long
    lib.smx_build_neighbors.argtypes = [vp, ctypes.c_int, dp, ip, dp, ip, ctypes.c_double, lp, ctypes.c_int]
    lib.smx_get_edges.argtypes = [vp, ip, ip, ip, ip, dp, dp, ctypes.c_int]
    lib.smx_compute_current.argtypes = [vp]
    lib.smx_timer_start.argtypes = [vp]
    lib.smx_timer_stop.argtypes = [vp, ctypes.POINTER(ctypes.c_double)]
    lib.smx_set_profiling.argtypes = [vp, ctypes.c_int]
    lib.smx_stage_time.argtypes = [vp, ctypes.c_int, ctypes.c_char_p, ctypes.c_int, ctypes.POINTER(ctypes.c_double)]
    lib.smx_measure_fma_peak.argtypes = [ctypes.c_int, ctypes.c_int, ctypes.POINTER(ctypes.c_double)]
    lib.smx_measure_row_stream.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.POINTER(ctypes.c_double), ctypes.POINTER(ctypes.c_double)]
    lib.smx_validate_inputs.argtypes = [vp, ctypes.c_int, lp, lp]
    lib.smx_sync.argtypes = [vp]
    lib.smx_set_stream.argtypes = [vp, vp, ctypes.c_int]
    lib.smx_restrict_nodes.argtypes = [vp, ctypes.c_int, lp]
    lib.smx_set_active_nodes.argtypes = [vp, ctypes.c_int, lp]
    lib.smx_resize_rows.argtypes = [vp, ctypes.c_char_p, ctypes.c_int]
    lib.smx_device_ptr.argtypes = [vp, ctypes.c_char_p, ctypes.POINTER(ctypes.c_void_p), lp, ctypes.POINTER(ctypes.c_int)]
    lib.smx_halo_pack.argtypes = [vp, ctypes.c_char_p, ip, ctypes.c_int, vp]
    lib.smx_halo_unpack.argtypes = [vp, ctypes.c_char_p, ip, ctypes.c_int, vp]
    lib.smx_halo_unpack_add.argtypes = [vp, ctypes.c_char_p, ip, ctypes.c_int, vp]
    lib.smx_atom_forces.argtypes = [vp, ctypes.c_int]
    lib.smx_active_counts.argtypes = [vp, ctypes.POINTER(ctypes.c_int), lp, ctypes.POINTER(ctypes.c_int)]
    lib.smx_debug_expire_waits.argtypes = [vp, ctypes.c_int]
    lib.smx_halo_cache_lists.argtypes = [vp, ctypes.c_int]
    lib.smx_comm_unique_id.argtypes = [vp, ctypes.c_int]
    lib.smx_comm_init.argtypes = [vp, vp, ctypes.c_int, ctypes.c_int, ctypes.c_int]
    lib.smx_comm_destroy.argtypes = [vp]
    lib.smx_halo_exchange.argtypes = [vp, ctypes.c_char_p, ctypes.c_int, ctypes.c_int, ip, vp, ip, vp, ip]
    lib.smx_allreduce_sum.argtypes = [vp, dp, ctypes.c_int]
    lib.smx_model_digest.argtypes = [ctypes.c_char_p, ctypes.c_int, ctypes.POINTER(ctypes.c_ulonglong), ctypes.POINTER(ctypes.c_int)]
    lib.smx_energy_virial_noalloc.argtypes = [dp, ctypes.c_int, dp, dp, ctypes.c_long, dp, vp, ctypes.c_char_p, ctypes.c_int]
    _lib = lib
    return lib
