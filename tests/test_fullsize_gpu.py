"""GPU: parity at benchmark config 4's full sequence length (T = 65536, G = 4, L = 32, D = 128;
chunk-visible as in the config, and the causal own-position operator at the same size) through
properties that do not need the full O(T^2) oracle:

* sampled query rows (o, lse, dq), sampled depth rows (d_depth_k/v) and the last sequence keys
  (dk, dv) against the oracle's single-row forms, at the tolerances of the small-case tests;
* causal prefix invariance: the first 4096 positions of the long run equal, bit for bit, a run
  on the problem truncated to 4096 positions (o, lse, dq);
* run-to-run bitwise reproducibility of every output;
* no bounded wait of the tcgen05 kernels expired.

Heads are independent problems, so two KV heads stand in for the eight of the config.
"""
import pytest
import torch

from oracle import moda_oracle as mo
from tests.helpers import TOL_GRAD_REL_L2, TOL_LSE_MAX_ABS, TOL_O_MAX_ABS, max_abs, rel_l2

pytestmark = pytest.mark.gpu

T, G, L, D, H = 65536, 4, 32, 128, 2
CP = 64 // G


@pytest.mark.parametrize("mode", [mo.MODE_CHUNK_VISIBLE, mo.MODE_CAUSAL], ids=["chunk_visible", "causal_own_position"])
def test_config4_full_length_properties(built_library, mode):
    import moda_b200 as M
    from moda_b200 import _cabi
    dev = torch.device("cuda", 0)
    gen = torch.Generator(device=dev).manual_seed(3)
    mk = lambda rows: torch.randn(1, rows, H, D, generator=gen, device=dev, dtype=torch.float32).to(torch.bfloat16)
    q, k, v, kd, vd, dout = mk(T * G), mk(T), mk(T), mk(T * L), mk(T * L), mk(T * G)
    scale = D ** -0.5

    def run(q, k, v, kd, vd, dout):
        if mode == mo.MODE_CHUNK_VISIBLE:
            o, lse = M.parallel_moda_chunk_visible_fwd(q, k, v, cached_k=kd, cached_v=vd, moda_group_num=G)
            dq, dk, dv, _, dkd, dvd = M.parallel_moda_chunk_visible_bwd(q, k, v, o, None, lse, dout, cached_k=kd,
                                                                        cached_v=vd, moda_group_num=G)
        else:
            o, lse = M.parallel_moda_fwd(q, k, v, cached_k=kd, cached_v=vd, moda_group_num=G, is_causal=True)
            dq, dk, dv, _, dkd, dvd = M.parallel_moda_bwd(q, k, v, o, None, lse, dout, cached_k=kd, cached_v=vd,
                                                          moda_group_num=G, is_causal=True)
        return o, lse, dq, dk, dv, dkd, dvd

    first = run(q, k, v, kd, vd, dout)
    assert _cabi.device_status() == 0
    o, lse, dq, dk, dv, dkd, dvd = first

    # run-to-run reproducibility
    second = run(q, k, v, kd, vd, dout)
    for a, b in zip(first, second):
        assert torch.equal(a, b)
    del second

    # causal prefix invariance
    Tp = 4096
    po, plse, pdq, *_ = run(q[:, :Tp * G], k[:, :Tp], v[:, :Tp], kd[:, :Tp * L], vd[:, :Tp * L], dout[:, :Tp * G])
    assert torch.equal(po, o[:, :Tp * G]) and torch.equal(plse, lse[:, :Tp * G]) and torch.equal(pdq, dq[:, :Tp * G])

    # sampled rows against the oracle's single-row forms (CPU, fp32)
    cq, ck, cv, ckd, cvd, cdo = [x.cpu() for x in (q, k, v, kd, vd, dout)]
    co, clse, cdq, cdk, cdv, cdkd, cdvd = [x.cpu() for x in first]
    rows = [0, 5, 63, 64, 4097, 131071, 131072, 200001, T * G - 65, T * G - 1]
    for i, r in enumerate(rows):
        h = i % H
        tm = mo.row_terms(cq, ck, cv, ckd, cvd, cdo, 0, h, r, scale, G, mode, CP)
        assert max_abs(co[0, r, h].float(), tm["o"]) <= TOL_O_MAX_ABS, f"o row {r}"
        assert abs(clse[0, r, h].item() - tm["lse"].item()) <= TOL_LSE_MAX_ABS, f"lse row {r}"
        assert rel_l2(cdq[0, r, h].float(), tm["dq"]) <= TOL_GRAD_REL_L2, f"dq row {r}"
    for i, c in enumerate([0, 31, 32 * 15 + 7, 32 * 16, 1000003, T * L - 1]):
        h = i % H
        rk, rv = mo.depth_row_grads(cq, ck, cv, ckd, cvd, cdo, 0, h, c, scale, G, mode, CP)
        assert rel_l2(cdkd[0, c, h].float(), rk) <= TOL_GRAD_REL_L2, f"d_depth_k row {c}"
        assert rel_l2(cdvd[0, c, h].float(), rv) <= TOL_GRAD_REL_L2, f"d_depth_v row {c}"
    for i, j in enumerate([T - 1, T - 3]):
        h = i % H
        rk, rv = mo.seq_key_grads(cq, ck, cv, ckd, cvd, cdo, 0, h, j, scale, G, mode, CP)
        assert rel_l2(cdk[0, j, h].float(), rk) <= TOL_GRAD_REL_L2, f"dk key {j}"
        assert rel_l2(cdv[0, j, h].float(), rv) <= TOL_GRAD_REL_L2, f"dv key {j}"
