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
from tests.helpers import TOL_GRAD_REL_L2, TOL_LSE_MAX_ABS, TOL_O_MAX_ABS, check_grad, max_abs, rel_l2

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


def test_config2_full_size_sampled_rows(built_library):
    """Benchmark config 2 in full (causal own-position MoDA, B=2, T=4096, Hkv=4, G=4, D=128, L=24,
    seed 1): sampled query rows (o, lse, dq), depth rows (d_depth_k/v) and sequence keys (dk, dv)
    against the oracle's single-row forms, plus run-to-run reproducibility."""
    import moda_b200 as M
    from moda_b200 import _cabi
    dev = torch.device("cuda", 0)
    B, T2, H2, G2, D2, L2 = 2, 4096, 4, 4, 128, 24
    gen = torch.Generator(device=dev).manual_seed(1)
    mk = lambda rows: torch.randn(B, rows, H2, D2, generator=gen, device=dev, dtype=torch.float32).to(torch.bfloat16)
    q, k, v, kd, vd, dout = mk(T2 * G2), mk(T2), mk(T2), mk(T2 * L2), mk(T2 * L2), mk(T2 * G2)
    scale = D2 ** -0.5

    def run():
        o, lse = M.parallel_moda_fwd(q, k, v, cached_k=kd, cached_v=vd, moda_group_num=G2, is_causal=True)
        dq, dk, dv, _, dkd, dvd = M.parallel_moda_bwd(q, k, v, o, None, lse, dout, cached_k=kd, cached_v=vd,
                                                      moda_group_num=G2, is_causal=True)
        return o, lse, dq, dk, dv, dkd, dvd

    first = run()
    assert _cabi.device_status() == 0
    for a, b in zip(first, run()):
        assert torch.equal(a, b)
    cq, ck, cv, ckd, cvd, cdo = [x.cpu() for x in (q, k, v, kd, vd, dout)]
    co, clse, cdq, cdk, cdv, cdkd, cdvd = [x.cpu() for x in first]
    for i, r in enumerate([0, 3, 4, 127, 128, 511, 4097, 9999, T2 * G2 - 129, T2 * G2 - 1]):
        b, h = i % B, i % H2
        tm = mo.row_terms(cq, ck, cv, ckd, cvd, cdo, b, h, r, scale, G2, mo.MODE_CAUSAL, 1)
        assert max_abs(co[b, r, h].float(), tm["o"]) <= TOL_O_MAX_ABS, f"o row {r}"
        assert abs(clse[b, r, h].item() - tm["lse"].item()) <= TOL_LSE_MAX_ABS, f"lse row {r}"
        assert rel_l2(cdq[b, r, h].float(), tm["dq"]) <= TOL_GRAD_REL_L2, f"dq row {r}"
    for i, c in enumerate([0, 23, 24, 24 * 31 + 5, 24 * 32, 50001, T2 * L2 - 1]):
        b, h = i % B, (i + 1) % H2
        rk, rv = mo.depth_row_grads(cq, ck, cv, ckd, cvd, cdo, b, h, c, scale, G2, mo.MODE_CAUSAL, 1)
        assert rel_l2(cdkd[b, c, h].float(), rk) <= TOL_GRAD_REL_L2, f"d_depth_k row {c}"
        assert rel_l2(cdvd[b, c, h].float(), rv) <= TOL_GRAD_REL_L2, f"d_depth_v row {c}"
    for i, j in enumerate([T2 - 1, T2 - 2, 2047, 0]):
        b, h = i % B, i % H2
        rk, rv = mo.seq_key_grads(cq, ck, cv, ckd, cvd, cdo, b, h, j, scale, G2, mo.MODE_CAUSAL, 1)
        assert rel_l2(cdk[b, j, h].float(), rk) <= TOL_GRAD_REL_L2, f"dk key {j}"
        assert rel_l2(cdv[b, j, h].float(), rv) <= TOL_GRAD_REL_L2, f"dv key {j}"


def test_config3_full_size_sampled_positions(built_library):
    """Benchmark config 3 in full (depth-only attention, B=8, T=8192, H=16, D=128, L=32, seed 2),
    forward and backward.  Every (batch, position, head) is an independent problem of one query and
    L keys, so sampled positions are checked exactly as small problems of the oracle (o, lse, dq and
    the position's L rows of d_depth_k/v); run-to-run reproducibility of every output on top."""
    import moda_b200 as M
    dev = torch.device("cuda", 0)
    B, T3, H3, D3, L3 = 8, 8192, 16, 128, 32
    gen = torch.Generator(device=dev).manual_seed(2)

    def mk(rows):     # drawn per batch row to bound the fp32 staging buffer
        out = torch.empty(B, rows, H3, D3, device=dev, dtype=torch.bfloat16)
        for b in range(B):
            out[b] = torch.randn(rows, H3, D3, generator=gen, device=dev, dtype=torch.float32).to(torch.bfloat16)
        return out

    q, kd, vd, dout = mk(T3), mk(T3 * L3), mk(T3 * L3), mk(T3)

    def run():
        o, lse = M.parallel_fda_fwd(q, cached_k=kd, cached_v=vd, moda_group_num=1)
        dq, _, dkd, dvd = M.parallel_fda_bwd(q, o, None, lse, dout, cached_k=kd, cached_v=vd, moda_group_num=1)
        return o, lse, dq, dkd, dvd

    first = run()
    second = run()
    for a, b in zip(first, second):
        assert torch.equal(a, b)
    del second
    o, lse, dq, dkd, dvd = first
    for i, (b, t, h) in enumerate([(0, 0, 0), (1, 1, 3), (2, 4095, 7), (3, 4096, 8), (5, 8000, 15), (7, T3 - 1, 15),
                                   (4, 77, 1), (6, 6001, 11)]):
        sl = slice(t * L3, (t + 1) * L3)
        tiny = [x.cpu() for x in (q[b:b + 1, t:t + 1, h:h + 1], kd[b:b + 1, sl, h:h + 1], vd[b:b + 1, sl, h:h + 1],
                                  dout[b:b + 1, t:t + 1, h:h + 1])]
        ro, rl, rdq, _, _, rdk, rdv = mo.moda_attention_ref_grads(tiny[0], None, None, tiny[1], tiny[2], tiny[3], None, 1,
                                                                   mo.MODE_DEPTH_ONLY, 1)
        assert max_abs(o[b, t, h].float().cpu(), ro[0, 0, 0]) <= TOL_O_MAX_ABS
        assert abs(lse[b, t, h].item() - rl[0, 0, 0].item()) <= TOL_LSE_MAX_ABS
        check_grad(f"dq ({b},{t},{h})", dq[b, t, h].float().cpu(), rdq[0, 0, 0])
        check_grad(f"d_depth_k ({b},{t},{h})", dkd[b, sl, h].float().cpu(), rdk[0, :, 0])
        check_grad(f"d_depth_v ({b},{t},{h})", dvd[b, sl, h].float().cpu(), rdv[0, :, 0])


def test_published_shape_d64_full_length(built_library):
    """The one shape the reference publishes a kernel time for (README.md:94: T = 65536, G = 8,
    d = 64, L = 64, causal own-position depth; one of the 8 KV heads) through the D = 64 tcgen05
    kernels at full length: sampled query rows, depth rows and the last sequence keys against the
    oracle's single-row forms, causal prefix invariance and run-to-run reproducibility."""
    import moda_b200 as M
    from moda_b200 import _cabi
    dev = torch.device("cuda", 0)
    Tp_, Gp, Lp, Dp = 65536, 8, 64, 64
    gen = torch.Generator(device=dev).manual_seed(7)
    mk = lambda rows: torch.randn(1, rows, 1, Dp, generator=gen, device=dev, dtype=torch.float32).to(torch.bfloat16)
    q, k, v, kd, vd, dout = mk(Tp_ * Gp), mk(Tp_), mk(Tp_), mk(Tp_ * Lp), mk(Tp_ * Lp), mk(Tp_ * Gp)
    scale = Dp ** -0.5

    def run(q, k, v, kd, vd, dout):
        o, lse = M.parallel_moda_fwd(q, k, v, cached_k=kd, cached_v=vd, moda_group_num=Gp, is_causal=True)
        dq, dk, dv, _, dkd, dvd = M.parallel_moda_bwd(q, k, v, o, None, lse, dout, cached_k=kd, cached_v=vd,
                                                      moda_group_num=Gp, is_causal=True)
        return o, lse, dq, dk, dv, dkd, dvd

    first = run(q, k, v, kd, vd, dout)
    assert _cabi.device_status() == 0
    for a, b in zip(first, run(q, k, v, kd, vd, dout)):
        assert torch.equal(a, b)
    o, lse, dq, dk, dv, dkd, dvd = first
    Tc = 2048
    po, plse, pdq, *_ = run(q[:, :Tc * Gp], k[:, :Tc], v[:, :Tc], kd[:, :Tc * Lp], vd[:, :Tc * Lp], dout[:, :Tc * Gp])
    assert torch.equal(po, o[:, :Tc * Gp]) and torch.equal(plse, lse[:, :Tc * Gp]) and torch.equal(pdq, dq[:, :Tc * Gp])

    cq, ck, cv, ckd, cvd, cdo = [x.cpu() for x in (q, k, v, kd, vd, dout)]
    co, clse, cdq, cdk, cdv, cdkd, cdvd = [x.cpu() for x in first]
    for r in [0, 7, 8, 1023, 1024, 262145, Tp_ * Gp - 257, Tp_ * Gp - 1]:
        tm = mo.row_terms(cq, ck, cv, ckd, cvd, cdo, 0, 0, r, scale, Gp, mo.MODE_CAUSAL, 1)
        assert max_abs(co[0, r, 0].float(), tm["o"]) <= TOL_O_MAX_ABS, f"o row {r}"
        assert abs(clse[0, r, 0].item() - tm["lse"].item()) <= TOL_LSE_MAX_ABS, f"lse row {r}"
        assert rel_l2(cdq[0, r, 0].float(), tm["dq"]) <= TOL_GRAD_REL_L2, f"dq row {r}"
    for c in [0, 63, 64, 64 * 1000 + 17, Tp_ * Lp - 1]:
        rk, rv = mo.depth_row_grads(cq, ck, cv, ckd, cvd, cdo, 0, 0, c, scale, Gp, mo.MODE_CAUSAL, 1)
        assert rel_l2(cdkd[0, c, 0].float(), rk) <= TOL_GRAD_REL_L2, f"d_depth_k row {c}"
        assert rel_l2(cdvd[0, c, 0].float(), rv) <= TOL_GRAD_REL_L2, f"d_depth_v row {c}"
    for j in [Tp_ - 1, Tp_ - 2]:
        rk, rv = mo.seq_key_grads(cq, ck, cv, ckd, cvd, cdo, 0, 0, j, scale, Gp, mo.MODE_CAUSAL, 1)
        assert rel_l2(cdk[0, j, 0].float(), rk) <= TOL_GRAD_REL_L2, f"dk key {j}"
        assert rel_l2(cdv[0, j, 0].float(), rv) <= TOL_GRAD_REL_L2, f"dv key {j}"
