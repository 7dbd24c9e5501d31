"""GPU: the allocation-free backward entry point (``moda_b200_bwd_static_scratch``).

Who needs it: a caller that is not allowed to allocate device memory where the backward
runs — for example code that must not call ``cudaMalloc`` because that call synchronises
the device, or a callback that is handed only its input and output buffers.  The entry
point keeps the kernels' scratch in a fixed array inside the library, so the caller
passes inputs and outputs and nothing else.

The test drives it through the C ABI (ctypes) on tensors allocated up front, twice in a
row (the array is shared and keeps the previous call's contents), and checks every
gradient against the ordinary entry point ``moda_b200_bwd``, which takes a caller
workspace.  Both run the same deterministic kernels, so the comparison is exact; the
oracle tolerance of the other GPU tests is checked on top.  Collected last (file name)
so that a run stopping at the first failure has already run everything else; it passes
alone in a fresh process and after the other tests.
"""
import ctypes

import pytest
import torch

from oracle import moda_oracle as mo
from tests.helpers import check_grad

pytestmark = pytest.mark.gpu


def _t4(x):
    from moda_b200._cabi import Tensor4
    return None if x is None else ctypes.byref(Tensor4(x.data_ptr(), x.stride(0), x.stride(1), x.stride(2)))


@pytest.mark.parametrize("mode,D,T,L,G,path", [
    (mo.MODE_CHUNK_VISIBLE, 128, 640, 8, 4, "tcgen05"),
    (mo.MODE_CAUSAL, 128, 300, 3, 2, "auto"),
    (mo.MODE_NONCAUSAL, 64, 197, 11, 1, "auto"),
    (mo.MODE_DEPTH_ONLY, 128, 256, 16, 1, "auto"),
])
def test_static_scratch_backward_matches_workspace_backward(built_library, mode, D, T, L, G, path):
    import moda_b200 as M
    from moda_b200 import _cabi
    lib = _cabi.load()
    dev = torch.device("cuda", 0)
    B, H = 2, 2
    q, k, v, kd, vd, dout = mo.make_inputs(900 + T, B, T, H, D, L, G, dtype=torch.bfloat16,
                                           with_seq=(mode != mo.MODE_DEPTH_ONLY))
    ref = mo.moda_attention_ref_grads(q, k, v, kd, vd, dout, None, G, mode, max(64 // G, 1))
    q, k, v, kd, vd, dout = [None if x is None else x.to(dev) for x in (q, k, v, kd, vd, dout)]
    scale = D ** -0.5
    kernel_path = {"auto": M.PATH_AUTO, "tcgen05": M.PATH_TCGEN05}[path]
    old = M.set_kernel_path(kernel_path)
    try:
        if mode == mo.MODE_DEPTH_ONLY:
            o, lse = M.parallel_fda_fwd(q, scale=scale, cached_k=kd, cached_v=vd, moda_group_num=G)
        elif mode == mo.MODE_CHUNK_VISIBLE:
            o, lse = M.parallel_moda_chunk_visible_fwd(q, k, v, scale=scale, cached_k=kd, cached_v=vd, moda_group_num=G)
        else:
            o, lse = M.parallel_moda_fwd(q, k, v, scale=scale, cached_k=kd, cached_v=vd, moda_group_num=G,
                                         is_causal=(mode == mo.MODE_CAUSAL))
    finally:
        M.set_kernel_path(old)

    prob = _cabi.Problem(B, T, H, D, G, L, mode, 64, _cabi.DTYPE_BF16, kernel_path, scale, 0)
    need = ctypes.c_size_t(0)
    assert lib.moda_b200_bwd_workspace_bytes(ctypes.byref(prob), ctypes.byref(need)) == 0
    assert need.value <= _cabi.STATIC_SCRATCH_BYTES

    def grads_like():
        return [None if x is None else torch.full_like(x, float("nan")) for x in (q, k, v, kd, vd)]

    # everything the calls need exists before the first one: nothing is allocated in between
    ws = torch.empty(max(need.value, 256), dtype=torch.uint8, device=dev)
    g_ws = grads_like()
    g_a, g_b = grads_like(), grads_like()
    stream = torch.cuda.current_stream().cuda_stream
    ins = [_t4(x) for x in (q, k, v, kd, vd, o)]
    rc = lib.moda_b200_bwd(ctypes.byref(prob), *ins, lse.data_ptr(), _t4(dout), *[_t4(g) for g in g_ws],
                           ws.data_ptr(), ws.numel(), stream)
    assert rc == 0, _cabi.status_string(rc)
    # a first static-scratch call outside the measured window: it resolves the array's address and
    # lets the driver finish any lazy loading of the kernels involved
    rc = lib.moda_b200_bwd_static_scratch(ctypes.byref(prob), *ins, lse.data_ptr(), _t4(dout),
                                          *[_t4(g) for g in g_b], stream)
    assert rc == 0, _cabi.status_string(rc)
    torch.cuda.synchronize()
    # torch's counter sees only torch's caching allocator; the driver's free-memory figure also sees
    # a cudaMalloc made inside the library
    mem_before = torch.cuda.memory_allocated()
    free_before = torch.cuda.mem_get_info()[0]
    for dst in (g_a, g_b):   # two calls in a row share the static array
        rc = lib.moda_b200_bwd_static_scratch(ctypes.byref(prob), *ins, lse.data_ptr(), _t4(dout),
                                              *[_t4(g) for g in dst], stream)
        assert rc == 0, _cabi.status_string(rc)
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == mem_before
    assert torch.cuda.mem_get_info()[0] >= free_before, "device memory was allocated during the static-scratch calls"
    assert _cabi.device_status() == 0

    for name, gw, ga, gb, gr in zip(("dq", "dk", "dv", "d_depth_k", "d_depth_v"), g_ws, g_a, g_b, ref[2:]):
        if gw is None:
            continue
        assert not torch.isnan(ga.float()).any() and not torch.isnan(gb.float()).any(), name
        assert torch.equal(ga, gw), f"{name}: first static-scratch call differs from the workspace call"
        assert torch.equal(gb, gw), f"{name}: second static-scratch call differs from the workspace call"
        check_grad(name, ga.float().cpu(), gr)


def test_static_scratch_rejects_oversized_problem(built_library):
    """A problem whose scratch does not fit the fixed array is refused before any launch."""
    from moda_b200 import _cabi
    lib = _cabi.load()
    # benchmark config 4: 2.1 M query rows x 8 heads of fp32 statistics is far beyond 8 MiB
    prob = _cabi.Problem(1, 65536, 8, 128, 4, 32, 2, 64, _cabi.DTYPE_BF16, _cabi.PATH_AUTO, 0.088, 0)
    need = ctypes.c_size_t(0)
    assert lib.moda_b200_bwd_workspace_bytes(ctypes.byref(prob), ctypes.byref(need)) == 0
    assert need.value > _cabi.STATIC_SCRATCH_BYTES
    fake = _cabi.Tensor4(0x1000, 1 << 20, 1024, 128)
    r = ctypes.byref(fake)
    rc = lib.moda_b200_bwd_static_scratch(ctypes.byref(prob), r, r, r, r, r, r, 0x2000, r, r, r, r, r, r, None)
    assert rc == 11
    assert b"capacity" in lib.moda_b200_status_string(rc)


def test_python_helper_allocates_nothing(built_library):
    import moda_b200 as M
    from moda_b200 import ops
    dev = torch.device("cuda", 0)
    q, k, v, kd, vd, dout = [x.to(dev) for x in mo.make_inputs(5, 1, 200, 2, 128, 4, 2, dtype=torch.bfloat16)]
    o, lse = M.parallel_moda_fwd(q, k, v, cached_k=kd, cached_v=vd, moda_group_num=2)
    want = M.parallel_moda_bwd(q, k, v, o, None, lse, dout, cached_k=kd, cached_v=vd, moda_group_num=2)
    outs = [torch.empty_like(x) for x in (q, k, v, kd, vd)]
    torch.cuda.synchronize()
    before = torch.cuda.memory_allocated()
    ops.backward_into_static_scratch(q, k, v, kd, vd, o, lse, dout, *outs, 128 ** -0.5, 2, M.MODE_CAUSAL)
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == before
    for a, b in zip(outs, [g for g in want if g is not None]):
        assert torch.equal(a, b)
