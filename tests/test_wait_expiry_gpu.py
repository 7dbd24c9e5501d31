"""GPU: a bounded wait that runs out is reported and leaves the context usable.

Every mbarrier wait of the tcgen05 kernels has a limit; when it expires the CTA records
``(1 << 8) | barrier id`` in a sticky status word, waits for its own TMA loads, frees its TMEM
and returns.  In the product nothing makes a wait expire, so this test loads a test-only build
of the same sources (``libmoda_b200_waittest.so``, ``-DMODA_WAIT_TEST``): its forwards (the
one-tile and the two-tile kernel) withhold the softmax warps' "P ready" arrival - an mbarrier only
threads arrive on, never a TMA load - and its waits give up after about a millisecond.  One
launch of one CTA with one key tile: the loads it issues have landed (they fed the score matmul,
and the one-tile kernel's TMA warp waits for them) before the wait times out.  Nothing traps,
faults or spins without bound.

Checked: the call returns, the status word names the P-ready barrier, reading it resets it, and
the ordinary library then runs a normal forward + backward in the same process with status 0.
"""
import ctypes

import pytest
import torch

from oracle import moda_oracle as mo
from tests.helpers import TOL_LSE_MAX_ABS, TOL_O_MAX_ABS, max_abs

pytestmark = pytest.mark.gpu

BAR_P = {"one_tile": 4,     # tc::BarId::kBarP of the one-tile forward
         "two_tiles": 14}   # tc::F3Bars::p0 (first part of P, query tile 0) of the two-tile forward


@pytest.mark.parametrize("fwd", ["one_tile", "two_tiles"])
def test_expired_wait_is_reported_and_context_survives(built_library, fwd):
    import moda_b200 as M
    from moda_b200 import _cabi, build
    wt = ctypes.CDLL(build.build_wait_test())
    P, T4 = ctypes.POINTER(_cabi.Problem), ctypes.POINTER(_cabi.Tensor4)
    wt.moda_b200_fwd.argtypes = [P, T4, T4, T4, T4, T4, T4, ctypes.c_void_p, ctypes.c_void_p]
    wt.moda_b200_fwd.restype = ctypes.c_int
    wt.moda_b200_device_status.argtypes = [ctypes.POINTER(ctypes.c_int)]
    wt.moda_b200_device_status.restype = ctypes.c_int

    dev = torch.device("cuda", 0)
    B, T, H, D, G = 1, 64, 1, 128, 1
    q, k, v, _, _, _ = [None if x is None else x.to(dev) for x in mo.make_inputs(1, B, T, H, D, 0, G, dtype=torch.bfloat16)]
    o = torch.zeros_like(q)
    lse = torch.zeros(B, T, H, dtype=torch.float32, device=dev)
    path = _cabi.PATH_TCGEN05_ONE_TILE if fwd == "one_tile" else _cabi.PATH_TCGEN05_TWO_TILES
    prob = _cabi.Problem(B, T, H, D, G, 0, _cabi.MODE_CAUSAL, 64, _cabi.DTYPE_BF16, path, D ** -0.5, 0)
    t4 = lambda x: ctypes.byref(_cabi.Tensor4(x.data_ptr(), x.stride(0), x.stride(1), x.stride(2)))
    st = ctypes.c_int(-1)
    assert wt.moda_b200_device_status(ctypes.byref(st)) == 0 and st.value == 0
    rc = wt.moda_b200_fwd(ctypes.byref(prob), t4(q), t4(k), t4(v), None, None, t4(o), lse.data_ptr(),
                          torch.cuda.current_stream().cuda_stream)
    assert rc == 0                                   # the launch itself is fine; the kernel gives up inside
    torch.cuda.synchronize()                         # returns: the kernel ended by itself
    assert wt.moda_b200_device_status(ctypes.byref(st)) == 0
    # (the softmax warps' own bounded wait for the end of the matmuls starts a few microseconds
    # later and may, in principle, run out first: barrier 13 of the two-tile forward)
    expected = {(1 << 8) | BAR_P[fwd]} | ({(1 << 8) | 13} if fwd == "two_tiles" else set())
    assert st.value in expected, hex(st.value)
    assert wt.moda_b200_device_status(ctypes.byref(st)) == 0 and st.value == 0      # reading reset it
    assert float(o.abs().max()) == 0.0               # the abandoned launch wrote no output

    # the context is intact: the ordinary library computes the same problem correctly
    ref_o, ref_lse = mo.moda_attention_ref(q.cpu(), k.cpu(), v.cpu(), None, None, None, G, mo.MODE_CAUSAL, 1)
    old = M.set_kernel_path(M.PATH_TCGEN05_ONE_TILE if fwd == "one_tile" else M.PATH_TCGEN05_TWO_TILES)
    try:
        o2, lse2 = M.parallel_moda_fwd(q, k, v, moda_group_num=G)
    finally:
        M.set_kernel_path(old)
    assert max_abs(o2.float().cpu(), ref_o) <= TOL_O_MAX_ABS and max_abs(lse2.cpu(), ref_lse) <= TOL_LSE_MAX_ABS
    assert _cabi.device_status() == 0


def test_expired_wait_in_the_backward_is_reported_and_context_survives(built_library):
    """The same for the backward: the test build's dq kernel withholds the softmax warps' "dS tile
    ready" arrival, the update-MMA warp's bounded wait runs out after about a millisecond, the CTA
    frees its TMEM and returns, the dk/dv launch behind it sees the status word and returns at
    once; no gradient is written, the status names the barrier, and the ordinary library then runs
    the same backward correctly."""
    import moda_b200 as M
    from moda_b200 import _cabi, build
    wt = ctypes.CDLL(build.build_wait_test())
    P, T4, V = ctypes.POINTER(_cabi.Problem), ctypes.POINTER(_cabi.Tensor4), ctypes.c_void_p
    wt.moda_b200_bwd_workspace_bytes.argtypes = [P, ctypes.POINTER(ctypes.c_size_t)]
    wt.moda_b200_bwd_workspace_bytes.restype = ctypes.c_int
    wt.moda_b200_bwd.argtypes = [P] + [T4] * 6 + [V] + [T4] * 6 + [V, ctypes.c_size_t, V]
    wt.moda_b200_bwd.restype = ctypes.c_int
    wt.moda_b200_device_status.argtypes = [ctypes.POINTER(ctypes.c_int)]
    wt.moda_b200_device_status.restype = ctypes.c_int

    dev = torch.device("cuda", 0)
    B, T, H, D, G = 1, 64, 1, 128, 1
    q, k, v, _, _, dout = [None if x is None else x.to(dev) for x in mo.make_inputs(2, B, T, H, D, 0, G, dtype=torch.bfloat16)]
    old = M.set_kernel_path(M.PATH_TCGEN05)
    try:
        o, lse = M.parallel_moda_fwd(q, k, v, moda_group_num=G)
        good = M.parallel_moda_bwd(q, k, v, o, None, lse, dout, moda_group_num=G)
    finally:
        M.set_kernel_path(old)
    assert _cabi.device_status() == 0

    prob = _cabi.Problem(B, T, H, D, G, 0, _cabi.MODE_CAUSAL, 64, _cabi.DTYPE_BF16, _cabi.PATH_TCGEN05, D ** -0.5, 0)
    need = ctypes.c_size_t(0)
    assert wt.moda_b200_bwd_workspace_bytes(ctypes.byref(prob), ctypes.byref(need)) == 0
    ws = torch.empty(max(need.value, 16), dtype=torch.uint8, device=dev)
    dq, dk, dv = torch.zeros_like(q), torch.zeros_like(k), torch.zeros_like(v)
    t4 = lambda x: ctypes.byref(_cabi.Tensor4(x.data_ptr(), x.stride(0), x.stride(1), x.stride(2)))
    st = ctypes.c_int(-1)
    assert wt.moda_b200_device_status(ctypes.byref(st)) == 0 and st.value == 0
    rc = wt.moda_b200_bwd(ctypes.byref(prob), t4(q), t4(k), t4(v), None, None, t4(o), lse.data_ptr(), t4(dout),
                          t4(dq), t4(dk), t4(dv), None, None, ws.data_ptr(), ws.numel(),
                          torch.cuda.current_stream().cuda_stream)
    assert rc == 0
    torch.cuda.synchronize()                         # returns: the kernels ended by themselves
    assert wt.moda_b200_device_status(ctypes.byref(st)) == 0
    # dq's "tiles ready" barrier (3 + 2 * ring of 6 = 15), or the softmax warps' own wait for the
    # end of the matmuls (17), whichever bounded wait ran out first
    assert st.value in {(1 << 8) | 15, (1 << 8) | 17}, hex(st.value)
    assert wt.moda_b200_device_status(ctypes.byref(st)) == 0 and st.value == 0
    assert float(dq.abs().max()) == 0.0 and float(dk.abs().max()) == 0.0 and float(dv.abs().max()) == 0.0

    old = M.set_kernel_path(M.PATH_TCGEN05)
    try:
        again = M.parallel_moda_bwd(q, k, v, o, None, lse, dout, moda_group_num=G)
    finally:
        M.set_kernel_path(old)
    for a, b in zip(good, again):
        if a is not None:
            assert torch.equal(a, b)
    assert _cabi.device_status() == 0
