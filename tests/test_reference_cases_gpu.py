"""GPU: every parameter tuple of the reference's own operator test, run through this library.

The tuples (B, T_kv, H, K, V, L, group, dtype, scale) come from
``tests/golden/reference_test_cases.json``, extracted from the reference's
``tests/ops/test_moda.py:95-198`` by ``tests/golden/make_reference_cases.py``; the seed (2025)
and the draw order q, k, v, depth_k, depth_v, dO are the reference test's (``:233-252``).  The
reference compares its Triton kernels with an in-file torch loop; here the CUDA path (through the
Python mirror, i.e. the C ABI) is compared with the CPU oracle on the same rounded inputs at the
tolerances of the other parity tests, which are tighter than the reference's own rule
(max-abs <= 1e-2 OR rel-L2 <= 0.1, ``:84-92``).  All tuples are causal own-position MoDA with
K = V = 64; they run on the default kernel path.
"""
import json
import os

import pytest
import torch

from oracle import moda_oracle as mo
from tests.helpers import GOLDEN_DIR, TOL_LSE_MAX_ABS, TOL_O_MAX_ABS, check_grad, max_abs

pytestmark = pytest.mark.gpu

with open(os.path.join(GOLDEN_DIR, "reference_test_cases.json")) as _f:
    _FIX = json.load(_f)
_DT = {"float16": torch.float16, "bfloat16": torch.bfloat16}


def test_fixture_is_the_full_list():
    assert len(_FIX["cases"]) == 102 and _FIX["seed"] == 2025


@pytest.mark.parametrize("idx", range(len(_FIX["cases"])))
def test_reference_case(built_library, idx):
    import moda_b200 as M
    B, T, H, K, V, L, G, dt, scale = _FIX["cases"][idx]
    assert K == V
    dtype = _DT[dt]
    dev = torch.device("cuda", 0)
    q, k, v, kd, vd, dout = mo.make_inputs(_FIX["seed"], B, T, H, K, L, G, dtype=dtype)
    ref = mo.moda_attention_ref_grads(q, k, v, kd, vd, dout, scale, G, mo.MODE_CAUSAL, 1)
    leaves = [None if x is None else x.to(dev).requires_grad_(True) for x in (q, k, v, kd, vd)]
    o, lse = M.parallel_moda(leaves[0], leaves[1], leaves[2], g=None, cached_k=leaves[3], cached_v=leaves[4],
                             scale=scale, cu_seqlens=None, moda_group_num=G, head_first=False, need_lse=True)
    assert max_abs(o.float().cpu(), ref[0]) <= TOL_O_MAX_ABS
    assert max_abs(lse.cpu(), ref[1]) <= TOL_LSE_MAX_ABS
    (o * dout.to(dev)).sum().backward()
    for name, leaf, g_ref in zip(("dq", "dk", "dv", "d_depth_k", "d_depth_v"), leaves, ref[2:]):
        if leaf is not None:
            check_grad(name, leaf.grad.float().cpu(), g_ref)
