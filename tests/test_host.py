"""Host-side logic and the C-ABI library, without a GPU: generators, neighbour rule, model
validation inside the loader, exported symbols."""
import ctypes
import json
import re
from pathlib import Path

import numpy as np
import pytest

from symmetrix_b200 import _lib, structures as st
from symmetrix_b200.modelgen import generate as gen
from symmetrix_b200.modelgen.harmonics import coupling, random_rotation, real_sh, rotation_matrix_l

ROOT = Path(__file__).resolve().parents[1]
GOLDEN = ROOT / "tests" / "golden"


def _has_gpu():
    try:
        import torch
        return torch.cuda.is_available()
    except Exception:
        return False


def test_library_exports_every_declared_symbol():
    header = (ROOT / "include" / "symmetrix_b200.h").read_text()
    declared = set(re.findall(r"\b(smx_[a-z_0-9]+)\s*\(", header))
    declared -= {"smx_handle"}
    assert declared == set(_lib.EXPORTED_SYMBOLS)
    lib = _lib.load()
    for name in declared:
        assert hasattr(lib, name), name


def test_header_cites_reference_for_each_entry_point():
    header = (ROOT / "include" / "symmetrix_b200.h").read_text()
    assert header.count("eplaces") >= 9
    assert "mace.cpp:17-64" in header and "pair_symmetrix_mace.cpp" in header


def _create(path, precision=64):
    lib = _lib.load()
    h = ctypes.c_void_p()
    status = lib.smx_create(str(path).encode(), precision, 0, ctypes.byref(h))
    msg = lib.smx_last_error(h if h.value else None).decode()
    if h.value:
        lib.smx_destroy(h)
    return status, msg


def test_create_reports_missing_and_malformed_files(tmp_path):
    status, msg = _create(tmp_path / "nope.json")
    assert status == _lib.SMX_ERR_MODEL and "cannot open" in msg
    bad = tmp_path / "bad.json"
    bad.write_text("this is not json")
    status, msg = _create(bad)
    assert status == _lib.SMX_ERR_MODEL and "parse error" in msg   # analogue of nlohmann's parse_error
    status, msg = _create(GOLDEN / "tiny_model.json", precision=16)
    assert status == _lib.SMX_ERR_INVALID_ARGUMENT


def test_create_rejects_models_outside_the_supported_set(tmp_path):
    model = json.loads((GOLDEN / "tiny_model.json").read_text())
    for key, val, expect in [("l_max", 2, "l_max"), ("L_max", 4, "L_max")]:
        m = dict(model); m[key] = val
        p = tmp_path / f"{key}.json"
        p.write_text(json.dumps(m))
        status, msg = _create(p)
        assert status == _lib.SMX_ERR_UNSUPPORTED and expect in msg, (key, status, msg)
    for key, expect in [("has_zbl", "zbl_a_exp"), ("A0_scaled", "A0_spline_h")]:    # switched on without their tables
        m = dict(model); m[key] = True
        p = tmp_path / f"{key}.json"
        p.write_text(json.dumps(m))
        status, msg = _create(p)
        assert status == _lib.SMX_ERR_MODEL and expect in msg, (key, status, msg)
    m = dict(model); m["H1_weights"] = model["H1_weights"][:-1]
    p = tmp_path / "short.json"; p.write_text(json.dumps(m))
    status, msg = _create(p)
    assert status == _lib.SMX_ERR_MODEL and "H1_weights" in msg
    m = dict(model); del m["Phi1_l"]
    p = tmp_path / "missing.json"; p.write_text(json.dumps(m))
    status, msg = _create(p)
    assert status == _lib.SMX_ERR_MODEL and "Phi1_l" in msg


@pytest.mark.skipif(_has_gpu(), reason="only meaningful on a machine without a GPU")
def test_no_cpu_fallback():
    status, msg = _create(GOLDEN / "tiny_model.json")
    assert status == _lib.SMX_ERR_NO_DEVICE and "no CPU path" in msg
    from symmetrix_b200 import MACE, SymmetrixError
    with pytest.raises(SymmetrixError):
        MACE(GOLDEN / "tiny_model.json")


# ------------------------------------------------------------------ generators
def test_rotation_matrices_are_orthogonal_representations():
    rng = np.random.default_rng(0)
    r1, r2 = random_rotation(rng), random_rotation(rng)
    for l in range(4):
        d1, d2, d12 = rotation_matrix_l(l, r1), rotation_matrix_l(l, r2), rotation_matrix_l(l, r1 @ r2)
        np.testing.assert_allclose(d1 @ d1.T, np.eye(2 * l + 1), atol=1e-12)
        np.testing.assert_allclose(d1 @ d2, d12, atol=1e-11)


def test_coupling_tensors_are_equivariant_and_follow_the_triangle_rule():
    rot = random_rotation(np.random.default_rng(1))
    assert coupling(1, 1, 3) is None and coupling(0, 2, 1) is None
    for (l1, l2, l3) in [(1, 1, 0), (1, 1, 1), (1, 2, 3), (3, 2, 1), (2, 2, 2), (3, 1, 3)]:
        c = coupling(l1, l2, l3)
        d1, d2, d3 = (rotation_matrix_l(l, rot) for l in (l1, l2, l3))
        lhs = np.einsum("Mm,mab->Mab", d3, c)
        rhs = np.einsum("Mab,ax,by->Mxy", c, d1, d2)
        np.testing.assert_allclose(lhs, rhs, atol=1e-11)
        np.testing.assert_allclose(np.sum(c * c, axis=(1, 2)), 1.0, atol=1e-12)


def test_tensor_product_path_table_matches_expected_counts():
    for L_max, (P, T, Q) in {0: (4, 16, 16), 1: (10, 88, 40), 2: (17, 243, 71)}.items():
        paths = gen.tp_paths(3, L_max)
        assert len(paths) == P
        assert sum((2 * a + 1) * (2 * b + 1) for _, a, b in paths) == T
        assert sum(2 * l + 1 for l, _, _ in paths) == Q
        assert [p[0] for p in paths] == sorted(p[0] for p in paths)


def test_contraction_basis_is_equivariant():
    rng = np.random.default_rng(2)
    rot = random_rotation(rng)
    a = rng.standard_normal(16)
    big_d = np.zeros((16, 16))
    for l in range(4):
        big_d[l * l:(l + 1) ** 2, l * l:(l + 1) ** 2] = rotation_matrix_l(l, rot)
    for L in range(3):
        basis = gen.contraction_basis(3, L, 3)
        n_eta = [b.shape[0] for b in basis[0][1]]
        w = [rng.standard_normal(n) for n in n_eta]

        def evaluate(vec):
            out = np.zeros(2 * L + 1)
            for M, (monos, blocks) in enumerate(basis):
                prods = np.array([np.prod(vec[list(mn)]) for mn in monos])
                out[M] = sum(w[o] @ blocks[o] @ prods for o in range(3))
            return out

        np.testing.assert_allclose(evaluate(big_d @ a), rotation_matrix_l(L, rot) @ evaluate(a), atol=1e-10)


def test_harmonics_follow_the_reference_l1_convention():
    v = np.array([[0.3, -0.5, 0.8]])
    np.testing.assert_allclose(real_sh(3, v)[0, 1:4], np.sqrt(3) * v[0] / np.linalg.norm(v), atol=1e-14)


# ------------------------------------------------------------------ structures and neighbour rule
def test_neighbor_list_is_symmetric_and_strict():
    s = st.water_box(2, 8.0, seed=1)
    nl = st.neighbor_list(s, 4.0)
    fwd = {(int(i), int(j), tuple(int(x) for x in sh)) for i, j, sh in zip(nl["i"], nl["j"], nl["S"])}
    assert all((j, i, (-a, -b, -c)) in fwd for (i, j, (a, b, c)) in fwd)
    assert np.all(nl["d"] < 4.0) and np.all(np.diff(nl["i"]) >= 0)
    np.testing.assert_array_equal(nl["d"], np.sqrt((nl["D"][:, 0] ** 2 + nl["D"][:, 1] ** 2) + nl["D"][:, 2] ** 2))


def test_neighbor_list_small_cell_has_multiple_images():
    s = st.Structure(np.array([[0.1, 0.2, 0.3], [1.0, 1.1, 0.9]]), np.eye(3) * 1.9, np.array([1, 8]))
    nl = st.neighbor_list(s, 4.0)
    assert np.abs(nl["S"]).max() >= 2
    same = nl["i"] == nl["j"]
    assert same.any() and not np.any(same & np.all(nl["S"] == 0, axis=1))


def test_neighbor_list_tree_path_equals_brute_force():
    s = st.fcc_box(9, 3.6, [29, 47], seed=2)          # 2916 atoms: brute force
    big = st.fcc_box((9, 9, 10), 3.6, [29, 47], seed=2)  # 3240 atoms: tree path
    nl_b = st.neighbor_list(big, 5.0)
    import symmetrix_b200.structures as mod
    # force the brute-force path on the same structure by chunking through a smaller threshold
    pos, cell = big.positions, big.cell
    small_copy = st.Structure(pos, cell, big.numbers)
    orig = mod.neighbor_list.__defaults__
    nl_a = _brute(small_copy, 5.0)
    for k in ["i", "j", "S"]:
        np.testing.assert_array_equal(nl_a[k], nl_b[k])
    np.testing.assert_array_equal(nl_a["D"], nl_b["D"])
    assert s.num_atoms == 2916


def _brute(s, rc):
    """Direct double loop over images, vectorised per receiver chunk (independent of the KD-tree path)."""
    pos, cell = s.positions, s.cell
    n = pos.shape[0]
    out = {"i": [], "j": [], "S": [], "D": []}
    shifts = [(a, b, c) for a in (-1, 0, 1) for b in (-1, 0, 1) for c in (-1, 0, 1)]
    for i0 in range(0, n, 256):
        xi = pos[i0:i0 + 256]
        for sh in shifts:
            sv = (sh[0] * cell[0] + sh[1] * cell[1]) + sh[2] * cell[2]
            d = (pos + sv)[None] - xi[:, None]
            r2 = (d[..., 0] * d[..., 0] + d[..., 1] * d[..., 1]) + d[..., 2] * d[..., 2]
            keep = r2 < rc * rc
            if sh == (0, 0, 0):
                idx = np.arange(xi.shape[0]); keep[idx, idx + i0] = False
            ii, jj = np.nonzero(keep)
            out["i"].append(ii + i0); out["j"].append(jj); out["S"].append(np.tile(sh, (ii.size, 1))); out["D"].append(d[ii, jj])
    i = np.concatenate(out["i"]); j = np.concatenate(out["j"]); S = np.concatenate(out["S"]); D = np.concatenate(out["D"])
    code = ((S[:, 0] + 64) * 128 + (S[:, 1] + 64)) * 128 + (S[:, 2] + 64)
    order = np.lexsort((code, j, i))
    return {"i": i[order].astype(np.int32), "j": j[order].astype(np.int32), "S": S[order].astype(np.int32), "D": D[order]}


def test_structures_have_the_requested_shape():
    w = st.water_box(4, 12.42, seed=0)
    assert w.num_atoms == 192 and sorted(set(w.numbers)) == [1, 8]
    oh = np.linalg.norm(w.positions[1] - w.positions[0])
    assert 0.7 < min(oh, abs(oh - 12.42)) < 1.3 or 0.7 < oh < 1.3
    f = st.fcc_box(3, 3.6, [13, 29, 47], seed=0)
    assert f.num_atoms == 108 and np.all(f.positions >= 0) and np.all(f.positions < 3 * 3.6)
    liq = st.molecular_liquid(27, seed=0)
    assert liq.num_atoms == 243
    nl = st.neighbor_list(liq, 0.8)
    assert np.all((nl["i"] // 9) == (nl["j"] // 9))   # no inter-molecular contact below 0.8 A


def test_cpp_facade_compiles_and_reports_missing_device(tmp_path):
    """The C++ mirror of the reference class compiles with g++ alone and links against the library."""
    import subprocess
    exe = tmp_path / "facade_harness"
    pkg = ROOT / "symmetrix_b200"
    subprocess.run(["g++", "-std=c++20", f"-I{ROOT / 'include'}", str(ROOT / "tests" / "facade_harness.cpp"), "-o", str(exe),
                    f"-L{pkg}", "-lsymmetrix_b200", f"-Wl,-rpath,{pkg}"], check=True)
    if not _has_gpu():
        r = subprocess.run([str(exe), str(GOLDEN / "tiny_model.json"), "/dev/null", str(tmp_path / "o.bin")], capture_output=True, text=True)
        assert r.returncode == 1 and "no CPU path" in r.stderr


def test_model_side_car_gives_the_same_model_and_follows_the_source_file(tmp_path, monkeypatch):
    """`<file>.smxcache`: written at the first load, read at the next, identical content (digest over everything the loader
    produces), invalidated when the source file changes, switched off by SMX_MODEL_CACHE=0. Runs without a GPU."""
    import ctypes
    import json
    import os
    import shutil
    from symmetrix_b200 import _lib
    lib = _lib.load()
    path = tmp_path / "model.json"
    shutil.copy(GOLDEN / "tiny_model.json", path)

    def digest(use_cache):
        d, hit = ctypes.c_ulonglong(0), ctypes.c_int(-1)
        assert lib.smx_model_digest(str(path).encode(), int(use_cache), ctypes.byref(d), ctypes.byref(hit)) == _lib.SMX_OK
        return d.value, hit.value

    plain, _ = digest(False)
    first, hit1 = digest(True)
    second, hit2 = digest(True)
    assert (hit1, hit2) == (0, 1) and plain == first == second
    assert (tmp_path / "model.json.smxcache").is_file()
    # a changed source file is parsed again (and gives another digest)
    model = json.loads(path.read_text())
    model["atomic_energies"][0] += 1.0
    path.write_text(json.dumps(model))
    os.utime(path, ns=(path.stat().st_atime_ns, path.stat().st_mtime_ns + 5_000_000_000))
    changed, hit3 = digest(True)
    assert hit3 == 0 and changed != plain
    assert digest(True) == (changed, 1)
    # a damaged side-car is ignored
    side = tmp_path / "model.json.smxcache"
    side.write_bytes(side.read_bytes()[: side.stat().st_size // 2])
    assert digest(True) == (changed, 0)
    monkeypatch.setenv("SMX_MODEL_CACHE", "0")
    assert digest(True) == (changed, 0)
