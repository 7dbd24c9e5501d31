"""CPU: the C-ABI library loads, exports every symbol the header declares, and its
validation returns the documented status codes without touching a GPU."""
import ctypes
import os
import re

import pytest
import torch

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib(built_library):
    from moda_b200 import _cabi
    return _cabi.load()


def _declared_symbols():
    names = set()
    inc = os.path.join(ROOT, "include")
    for fn in os.listdir(inc):
        if fn.endswith(".h"):
            text = open(os.path.join(inc, fn)).read()
            text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
            names |= set(re.findall(r"\b(moda_b200_\w+)\s*\(", text))
    return sorted(names)


def test_every_declared_symbol_is_exported(lib):
    from moda_b200 import _cabi
    declared = _declared_symbols()
    assert set(_cabi.EXPORTED_SYMBOLS) <= set(declared)
    assert len(declared) >= 9
    for name in declared:
        assert hasattr(lib, name), name


def _prob(**kw):
    from moda_b200._cabi import Problem
    base = dict(B=1, T_kv=64, H=2, D=64, G=1, L=2, mode=0, chunk_rows=64, dtype=0, path=0,
                scale=0.125, device=0)
    base.update(kw)
    return Problem(**base)


@pytest.mark.parametrize("kw,code", [
    ({}, 0),
    ({"B": 0}, 2), ({"T_kv": 0}, 2), ({"L": -1}, 2), ({"G": 0}, 2),
    ({"D": 96}, 3), ({"D": 256}, 3),
    ({"dtype": 2}, 4),
    ({"mode": 7}, 6), ({"mode": 3, "L": 0}, 6), ({"path": 6}, 6), ({"path": 5}, 0),
    ({"mode": 2, "chunk_rows": 0}, 7), ({"mode": 2, "chunk_rows": 64, "G": 3}, 7),
    ({"mode": 2, "chunk_rows": 64, "G": 4}, 0),
])
def test_check_problem_codes(lib, kw, code):
    p = _prob(**kw)
    assert lib.moda_b200_check_problem(ctypes.byref(p)) == code


def test_null_and_alignment_are_rejected_before_any_launch(lib):
    from moda_b200._cabi import Tensor4
    p = _prob()
    good = Tensor4(0x1000, 64 * 2 * 64, 2 * 64, 64)
    null = Tensor4(0, 0, 0, 0)
    odd = Tensor4(0x1008, 64 * 2 * 64, 2 * 64, 64)
    bad_stride = Tensor4(0x1000, 64 * 2 * 64, 2 * 64 + 4, 64)
    r = ctypes.byref
    f = lib.moda_b200_fwd
    assert f(r(p), r(null), r(good), r(good), r(good), r(good), r(good), 0x2000, None) == 1
    assert f(r(p), r(good), r(good), r(good), None, r(good), r(good), 0x2000, None) == 1      # L>0 needs depth
    assert f(r(p), r(good), r(good), r(good), r(good), r(good), r(good), None, None) == 1     # lse NULL
    assert f(r(p), r(odd), r(good), r(good), r(good), r(good), r(good), 0x2000, None) == 5
    assert f(r(p), r(good), r(bad_stride), r(good), r(good), r(good), r(good), 0x2000, None) == 5
    # a zero or negative stride on a dimension of extent > 1 (expanded / flipped view) is refused;
    # on a dimension of extent 1 (here the batch) the stride is irrelevant
    zero_h = Tensor4(0x1000, 64 * 2 * 64, 2 * 64, 0)
    neg_t = Tensor4(0x1000, 64 * 2 * 64, -2 * 64, 64)
    any_b = Tensor4(0x1000, 0, 2 * 64, 64)
    assert f(r(p), r(good), r(zero_h), r(good), r(good), r(good), r(good), 0x2000, None) == 5
    assert f(r(p), r(good), r(good), r(neg_t), r(good), r(good), r(good), 0x2000, None) == 5
    p2 = _prob(B=2)
    assert f(r(p2), r(good), r(any_b), r(good), r(good), r(good), r(good), 0x2000, None) == 5
    assert lib.moda_b200_resolve_path(r(_prob(path=2, D=64)), 0) == 2          # tcgen05 kernels take D = 64 and 128
    assert lib.moda_b200_resolve_path(r(_prob(path=4, D=128)), 1) == 2
    assert lib.moda_b200_resolve_path(r(_prob(path=2, scale=-1.0)), 0) == -10  # ... but only a positive scale
    assert lib.moda_b200_resolve_path(r(_prob(path=0, scale=-1.0)), 0) == 1


def test_workspace_size_and_bwd_rejects_small_workspace(lib):
    from moda_b200._cabi import Tensor4
    p = _prob(B=2, T_kv=100, H=3, G=2)
    n = ctypes.c_size_t(0)
    assert lib.moda_b200_bwd_workspace_bytes(ctypes.byref(p), ctypes.byref(n)) == 0
    assert n.value >= 2 * 200 * 3 * 4 and n.value % 256 == 0
    g = Tensor4(0x1000, 8192, 64, 64)
    r = ctypes.byref
    rc = lib.moda_b200_bwd(r(p), r(g), r(g), r(g), r(g), r(g), r(g), 0x2000, r(g), r(g), r(g), r(g),
                           r(g), r(g), 0x4000, 16, None)
    assert rc == 8


def test_status_strings(lib):
    assert lib.moda_b200_status_string(0) == b"ok"
    assert b"head dim" in lib.moda_b200_status_string(3)
    assert lib.moda_b200_version() >= 100


def test_python_wrappers_mirror_reference_assertions(built_library):
    import moda_b200 as M
    q = torch.zeros(1, 8, 2, 64, dtype=torch.bfloat16)
    k = torch.zeros(1, 8, 3, 64, dtype=torch.bfloat16)
    with pytest.raises(AssertionError, match="head-dimension GQA"):
        M.parallel_moda(q, k, k, warn_shape=False)
    k = torch.zeros(1, 4, 2, 64, dtype=torch.bfloat16)
    with pytest.raises(AssertionError, match="T_q must equal T_kv"):
        M.parallel_moda(q, k, k, warn_shape=False)
    with pytest.raises(AssertionError, match="legacy k/v"):
        M.parallel_fda(q, k, k)
    with pytest.raises(AssertionError):
        M.parallel_moda(q, q, q, g=torch.zeros(1, 8, 2), warn_shape=False)
    # no CPU path: a CPU tensor is refused loudly, never computed some other way
    with pytest.raises(RuntimeError, match="CUDA tensors only"):
        M.parallel_moda(q, q, q, warn_shape=False)
    with pytest.warns(UserWarning, match="head_first"):
        with pytest.raises(RuntimeError):
            M.parallel_moda(torch.zeros(1, 2, 4, 64, dtype=torch.bfloat16),
                            torch.zeros(1, 2, 4, 64, dtype=torch.bfloat16),
                            torch.zeros(1, 2, 4, 64, dtype=torch.bfloat16))


def test_fold_qkv_returns_views_of_the_projection_outputs(built_library):
    """The projection outputs are consumed in place: q is a reshape, k and v are strided views of
    the fused key/value projection (the layout vision_tasks/deit/models.py:244-253 builds), and the
    library's layout rule accepts all three without a copy."""
    import moda_b200 as M
    from moda_b200 import ops
    B, N, Hkv, G, D = 2, 197, 6, 1, 64
    qp = torch.randn(B, N, G * Hkv * D).to(torch.bfloat16)
    kvp = torch.randn(B, N, 2 * Hkv * D).to(torch.bfloat16)
    q, k, v = M.fold_qkv(qp, kvp, Hkv, G)
    assert q.shape == (B, N * G, Hkv, D) and k.shape == v.shape == (B, N, Hkv, D)
    assert q.data_ptr() == qp.data_ptr() and k.data_ptr() == kvp.data_ptr()
    assert v.data_ptr() == kvp.data_ptr() + Hkv * D * 2 and not k.is_contiguous()
    for x in (q, k, v):
        assert ops._usable(x) is x
    assert torch.equal(k, kvp.view(B, N, 2, Hkv, D)[:, :, 0])
    # G > 1: query head g*Hkv + h sits at folded row n*G + g of KV head h
    qp2 = torch.randn(1, 5, 3 * 2 * D)
    q2, _, _ = M.fold_qkv(qp2, torch.randn(1, 5, 2 * 2 * D), 2, 3)
    assert torch.equal(q2[0, 4 * 3 + 1, 1], qp2[0, 4].view(3, 2, D)[1, 1])
    # an expanded view is not usable in place
    e = torch.zeros(1, 8, 2, 64).expand(3, -1, -1, -1)
    assert ops._usable(e) is not e


def test_depth_cache_copy_accounting(built_library):
    """Bytes of K/V copied per forward: once per layer in place, against the stack-and-make-contiguous
    rebuild before every layer of the reference's caller (vision_tasks/deit/models.py:361-375)."""
    import moda_b200 as M
    c = M.DepthKVCache(2, 10, 11, 6, 64, torch.bfloat16, "cpu")
    per_layer = 2 * 2 * 10 * 6 * 64 * 2
    assert c.bytes_copied_per_forward(12) == 11 * per_layer
    assert c.bytes_copied_by_rebuilding(12) == 2 * sum(range(12)) * per_layer


def test_depth_cache_layout_fields_are_validated(lib):
    r = ctypes.byref
    assert lib.moda_b200_check_problem(r(_prob(L=2, depth_rows_per_pos=0))) == 0
    assert lib.moda_b200_check_problem(r(_prob(L=2, depth_rows_per_pos=2))) == 0
    assert lib.moda_b200_check_problem(r(_prob(L=2, depth_rows_per_pos=11))) == 0
    assert lib.moda_b200_check_problem(r(_prob(L=3, depth_rows_per_pos=2))) == 2     # fewer rows than layers
    assert lib.moda_b200_check_problem(r(_prob(L=2, depth_rows_per_pos=-1))) == 2
    # the tcgen05 kernels read an in-place cache through 5-D maps only when L divides their 32-row boxes
    assert lib.moda_b200_resolve_path(r(_prob(L=4, depth_rows_per_pos=11, G=2, T_kv=64)), 0) == 2
    assert lib.moda_b200_resolve_path(r(_prob(L=3, depth_rows_per_pos=11, G=2, T_kv=64)), 0) == 1
    assert lib.moda_b200_resolve_path(r(_prob(L=3, depth_rows_per_pos=11, G=2, T_kv=64, path=2)), 0) == -10
    # depth_append: layer index and capacity are checked before anything is launched
    from moda_b200._cabi import Tensor4
    t4 = Tensor4(0x1000, 64 * 2 * 64 * 11, 2 * 64, 64)
    assert lib.moda_b200_depth_append(r(_prob(depth_rows_per_pos=11)), r(t4), r(t4), r(t4), r(t4), 11, None) == 2
    assert lib.moda_b200_depth_append(r(_prob(depth_rows_per_pos=0)), r(t4), r(t4), r(t4), r(t4), 0, None) == 2
    assert lib.moda_b200_depth_append(r(_prob(depth_rows_per_pos=11)), None, r(t4), r(t4), r(t4), 0, None) == 1


def test_product_package_does_not_import_the_oracle():
    pkg = os.path.join(ROOT, "moda_b200")
    for dirpath, _, files in os.walk(pkg):
        for fn in files:
            if fn.endswith((".py", ".cu", ".cuh", ".h")):
                text = open(os.path.join(dirpath, fn)).read()
                assert not re.search(r"^\s*(from|import)\s+oracle\b", text, flags=re.M), fn
                assert "moda_oracle" not in text, fn


def test_build_is_keyed_by_content_not_by_file_times(built_library):
    """A checkout or a copy of the tree changes file times without changing a byte: the library must
    not be taken for stale then (the ranks of a multi-GPU launch would all start rebuilding it)."""
    import glob
    import time
    from moda_b200 import build
    assert not build._stale(build.OUT)
    src = sorted(glob.glob(os.path.join(build.CSRC, "*.cuh")))[0]
    st = os.stat(src)
    try:
        os.utime(src, (time.time() + 100, time.time() + 100))      # "newer" than the library
        assert not build._stale(build.OUT)
        assert build.build() == build.OUT                           # returns without compiling
    finally:
        os.utime(src, (st.st_atime, st.st_mtime))
    assert build._digest(()) != build._digest(("-DMODA_WAIT_TEST",))   # the flags are part of the key


def test_concurrent_build_calls_leave_one_whole_library(built_library):
    """Every rank of a multi-GPU launch calls build(): with an up-to-date stamp none of them writes,
    and all of them can load the library."""
    import subprocess
    import sys
    from moda_b200 import build
    before = os.stat(build.OUT).st_mtime_ns
    code = ("import ctypes; from moda_b200 import build; p = build.build(); "
            "ctypes.CDLL(p); print('ok')")
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    procs = [subprocess.Popen([sys.executable, "-c", code], cwd=root, stdout=subprocess.PIPE, text=True) for _ in range(6)]
    outs = [p.communicate(timeout=300)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs) and all("ok" in o for o in outs)
    assert os.stat(build.OUT).st_mtime_ns == before
