"""The allocation-free energy/virial entry point against the allocating one.

Some callers of this library cannot let it allocate device memory while they run (a host code that
owns the whole GPU through its own memory pool, a job with a fixed memory budget, a step loop that
cannot afford the device-wide synchronisation of cudaMalloc). ``smx_energy_virial_noalloc`` serves
them with a scratch array compiled into the library. This test calls it through the C ABI twice in
a row on device arrays and compares with ``smx_reduce_forces``. It lives in its own file, collected
last, and passes both alone in a fresh process and after the other tests.
"""
import ctypes
from pathlib import Path

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

GOLDEN = Path(__file__).resolve().parent / "golden"
INPUT_KEYS = ["num_nodes", "node_types", "num_neigh", "neigh_indices", "neigh_types", "xyz", "r"]


def _call(lib, e_dev, n, xyz_dev, nf_dev, n_edges, out_dev):
    err = ctypes.create_string_buffer(256)
    status = lib.smx_energy_virial_noalloc(ctypes.c_void_p(e_dev.data_ptr() if e_dev is not None else 0), n,
                                           ctypes.c_void_p(xyz_dev.data_ptr() if xyz_dev is not None else 0),
                                           ctypes.c_void_p(nf_dev.data_ptr() if nf_dev is not None else 0), n_edges,
                                           ctypes.c_void_p(out_dev.data_ptr()), None, err, 256)
    return status, err.value.decode()


def test_noalloc_energy_virial_matches_reduce_forces_twice():
    import torch
    from symmetrix_b200 import MACE, _lib

    lib = _lib.load()
    case = np.load(GOLDEN / "tiny_case.npz")
    inputs = {k: case[k] for k in INPUT_KEYS}
    ev = MACE(GOLDEN / "tiny_model.json", dtype="float64")
    torch.cuda.set_device(0)
    out = torch.full((7,), float("nan"), dtype=torch.float64, device="cuda")
    for scale in (1.0, -0.5):          # two calls in a row on different data: the shared scratch keeps nothing over
        inp = dict(inputs)
        inp["xyz"] = inputs["xyz"] * (1.0 if scale > 0 else 1.02)
        inp["r"] = np.linalg.norm(inp["xyz"].reshape(-1, 3), axis=1)
        ev.compute_node_energies_forces(int(inp["num_nodes"]), inp["node_types"], inp["num_neigh"], inp["neigh_indices"],
                                        inp["neigh_types"], inp["xyz"], inp["r"])
        _, virial, energy = ev.reduce_forces(want_forces=False)
        e_dev = torch.as_tensor(ev.node_energies).cuda()
        nf_dev = torch.as_tensor(ev.node_forces).cuda()
        xyz_dev = torch.as_tensor(np.ascontiguousarray(inp["xyz"])).cuda()
        torch.cuda.synchronize()
        status, msg = _call(lib, e_dev, e_dev.numel(), xyz_dev, nf_dev, nf_dev.numel() // 3, out)
        assert status == _lib.SMX_OK, msg
        torch.cuda.synchronize()
        got = out.cpu().numpy()
        # same tolerance as the other reduction checks: summation order differs between the two kernels
        assert abs(got[0] - energy) <= 1e-12 * abs(energy)
        np.testing.assert_allclose(got[1:], virial, rtol=1e-11, atol=1e-10)


def _numpy_sums(e, xyz, nf):
    x, f = xyz.reshape(-1, 3), nf.reshape(-1, 3)
    return np.array([e.sum(), (x[:, 0] * f[:, 0]).sum(), (x[:, 1] * f[:, 1]).sum(), (x[:, 2] * f[:, 2]).sum(),
                     0.5 * (x[:, 0] * f[:, 1] + x[:, 1] * f[:, 0]).sum(), 0.5 * (x[:, 0] * f[:, 2] + x[:, 2] * f[:, 0]).sum(),
                     0.5 * (x[:, 1] * f[:, 2] + x[:, 2] * f[:, 1]).sum()])


def test_noalloc_uses_several_scratch_rows_and_ignores_stale_ones():
    """Inputs that span several 4096-item chunks (one scratch row each), first with more edges than nodes, then a smaller
    call with more nodes than edges: the second call must not read the rows the first one left behind."""
    import torch
    from symmetrix_b200 import _lib

    lib = _lib.load()
    rng = np.random.default_rng(5)
    out = torch.full((7,), float("nan"), dtype=torch.float64, device="cuda")
    for n_nodes, n_edges in ((3000, 10000), (6000, 5000), (1, 4097)):
        e = rng.normal(size=n_nodes); xyz = rng.normal(size=3 * n_edges); nf = rng.normal(size=3 * n_edges)
        status, msg = _call(lib, torch.as_tensor(e).cuda(), n_nodes, torch.as_tensor(xyz).cuda(), torch.as_tensor(nf).cuda(), n_edges, out)
        assert status == _lib.SMX_OK, msg
        torch.cuda.synchronize()
        np.testing.assert_allclose(out.cpu().numpy(), _numpy_sums(e, xyz, nf), rtol=1e-12, atol=1e-10)


def test_noalloc_rejects_oversized_and_null_inputs():
    import torch
    from symmetrix_b200 import _lib

    lib = _lib.load()
    out = torch.zeros(7, dtype=torch.float64, device="cuda")
    dummy = torch.zeros(8, dtype=torch.float64, device="cuda")
    status, msg = _call(lib, dummy, 1, dummy, dummy, 16_777_217, out)
    assert status == _lib.SMX_ERR_INVALID_ARGUMENT and "16777216" in msg
    status, msg = _call(lib, None, 4, dummy, dummy, 1, out)
    assert status == _lib.SMX_ERR_INVALID_ARGUMENT and "null" in msg
    # empty input is fine and gives zeros
    status, msg = _call(lib, None, 0, None, None, 0, out)
    assert status == _lib.SMX_OK, msg
    torch.cuda.synchronize()
    assert float(out.abs().sum()) == 0.0
