"""GPU: a bounded wait that runs out is reported and leaves the context usable.

Every mbarrier wait of the tcgen05 kernels has a limit; when it expires the CTA records
``(1 << 8) | barrier id`` in a sticky status word, waits for its own TMA loads, frees its TMEM
and returns.  In the product nothing makes a wait expire, so this test loads a test-only build
of the same sources (``libmoda_b200_waittest.so``, ``-DMODA_WAIT_TEST``): its one-tile forward
withholds the softmax warps' "P ready" arrival - an mbarrier only threads arrive on, never a TMA
load - and its waits give up after about a millisecond.  One launch of one CTA with one key tile:
the three loads it issues have landed (the TMA warp waits for them) before the wait times out.
Nothing traps, faults or spins without bound.

Checked: the call returns, the status word names the P-ready barrier, reading it resets it, and
the ordinary library then runs a normal forward + backward in the same process with status 0.
"""
import ctypes

import pytest
import torch

from oracle import moda_oracle as mo
from tests.helpers import TOL_LSE_MAX_ABS, TOL_O_MAX_ABS, max_abs

pytestmark = pytest.mark.gpu

BAR_P = 4        # tc::BarId::kBarP of the one-tile forward


def test_expired_wait_is_reported_and_context_survives(built_library):
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
    prob = _cabi.Problem(B, T, H, D, G, 0, _cabi.MODE_CAUSAL, 64, _cabi.DTYPE_BF16, _cabi.PATH_TCGEN05_ONE_TILE,
                         D ** -0.5, 0)
    t4 = lambda x: ctypes.byref(_cabi.Tensor4(x.data_ptr(), x.stride(0), x.stride(1), x.stride(2)))
    st = ctypes.c_int(-1)
    assert wt.moda_b200_device_status(ctypes.byref(st)) == 0 and st.value == 0
    rc = wt.moda_b200_fwd(ctypes.byref(prob), t4(q), t4(k), t4(v), None, None, t4(o), lse.data_ptr(),
                          torch.cuda.current_stream().cuda_stream)
    assert rc == 0                                   # the launch itself is fine; the kernel gives up inside
    torch.cuda.synchronize()                         # returns: the kernel ended by itself
    assert wt.moda_b200_device_status(ctypes.byref(st)) == 0
    assert st.value == (1 << 8) | BAR_P, hex(st.value)
    assert wt.moda_b200_device_status(ctypes.byref(st)) == 0 and st.value == 0      # reading reset it
    assert float(o.abs().max()) == 0.0               # the abandoned launch wrote no output

    # the context is intact: the ordinary library computes the same problem correctly
    ref_o, ref_lse = mo.moda_attention_ref(q.cpu(), k.cpu(), v.cpu(), None, None, None, G, mo.MODE_CAUSAL, 1)
    old = M.set_kernel_path(M.PATH_TCGEN05_ONE_TILE)
    try:
        o2, lse2 = M.parallel_moda_fwd(q, k, v, moda_group_num=G)
    finally:
        M.set_kernel_path(old)
    assert max_abs(o2.float().cpu(), ref_o) <= TOL_O_MAX_ABS and max_abs(lse2.cpu(), ref_lse) <= TOL_LSE_MAX_ABS
    assert _cabi.device_status() == 0
