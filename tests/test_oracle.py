"""CPU: the oracle restatement against fixtures produced by the reference's own
torch oracles (tests/golden/make_golden.py), and against its loop form."""
import math

import pytest
import torch

from oracle import moda_oracle as mo
from tests.helpers import golden_names, load_golden, max_abs, t


def _inputs(rec):
    c = rec["cfg"]
    q, k, v, kd, vd, dout = mo.make_inputs(c["seed"], c["B"], c["T_kv"], c["H"], c["D"], c["L"], c["G"],
                                           with_seq=(c["mode"] != mo.MODE_DEPTH_ONLY))
    return q, k, v, kd, vd, dout


@pytest.mark.parametrize("name", golden_names())
def test_seeded_inputs_reproduce(name):
    rec = load_golden(name)
    xs = [x for x in _inputs(rec) if x is not None]
    sums = [float(x.double().sum()) for x in xs]
    assert len(sums) == len(rec["input_checksum"])
    for a, b in zip(sums, rec["input_checksum"]):
        assert abs(a - b) <= 1e-6 * max(1.0, abs(b))
    if "in_q" in rec:
        assert torch.equal(xs[0], t(rec["in_q"]))


@pytest.mark.parametrize("name", golden_names())
def test_oracle_matches_reference_forward(name):
    rec = load_golden(name)
    c = rec["cfg"]
    q, k, v, kd, vd, _ = _inputs(rec)
    o, lse = mo.moda_attention_ref(q, k, v, kd, vd, c["scale"], c["G"], c["mode"], max(c["chunk_positions"], 1),
                                   row_block=37)
    assert max_abs(o, t(rec["o"])) <= 2e-5
    assert max_abs(lse, t(rec["lse"])) <= 2e-5


@pytest.mark.parametrize("name", [n for n in golden_names() if n != "config1"])
def test_oracle_matches_reference_gradients(name):
    rec = load_golden(name)
    c = rec["cfg"]
    q, k, v, kd, vd, dout = _inputs(rec)
    res = mo.moda_attention_ref_grads(q, k, v, kd, vd, dout, c["scale"], c["G"], c["mode"],
                                      max(c["chunk_positions"], 1))
    for key, got in zip(("dq", "dk", "dv", "dkd", "dvd"), res[2:]):
        if key in rec:
            assert got is not None
            assert max_abs(got, t(rec[key])) <= 5e-5, key
        else:
            assert got is None


def test_config1_sanity_values():
    # benchmark config 1 (B=1,T=256,H=4,D=64,L=4,G=1, seed 0): values recorded from the
    # reference's naive_mixture_of_depth_causal_ref in the build container.
    rec = load_golden("config1")
    assert abs(float(abs(rec["o"]).mean()) - 0.13568142) < 1e-7
    assert abs(float(rec["lse"].mean()) - 7.40047932) < 1e-6


@pytest.mark.parametrize("mode,G,L,cp", [
    (mo.MODE_CAUSAL, 1, 0, 1), (mo.MODE_CAUSAL, 2, 3, 1), (mo.MODE_NONCAUSAL, 1, 2, 1),
    (mo.MODE_CHUNK_VISIBLE, 4, 2, 16), (mo.MODE_CHUNK_VISIBLE, 2, 1, 32), (mo.MODE_DEPTH_ONLY, 2, 4, 1),
])
def test_vectorised_equals_loop(mode, G, L, cp):
    q, k, v, kd, vd, _ = mo.make_inputs(5, 2, 45, 2, 32, L, G, with_seq=(mode != mo.MODE_DEPTH_ONLY))
    o1, l1 = mo.moda_attention_ref(q, k, v, kd, vd, None, G, mode, cp, row_block=16)
    o2, l2 = mo.moda_attention_ref_loop(q, k, v, kd, vd, None, G, mode, cp)
    assert max_abs(o1, o2) <= 1e-5 and max_abs(l1, l2) <= 1e-5


def test_lse_is_base2_and_rows_normalised():
    q, k, v, kd, vd, _ = mo.make_inputs(9, 1, 8, 1, 16, 2, 1)
    o, lse = mo.moda_attention_ref(q, k, v, kd, vd, 0.25, 1, mo.MODE_CAUSAL)
    # row 0 sees key 0 and its own 2 depth rows
    logits = torch.cat([(q[0, 0, 0] @ k[0, :1, 0].T), (kd[0, :2, 0] @ q[0, 0, 0])]) * 0.25
    assert abs(lse[0, 0, 0].item() - torch.logsumexp(logits, 0).item() / math.log(2.0)) < 1e-5


@pytest.mark.parametrize("mode,G,L,cp", [(mo.MODE_CAUSAL, 2, 3, 1), (mo.MODE_CHUNK_VISIBLE, 4, 2, 16),
                                         (mo.MODE_NONCAUSAL, 1, 2, 1)])
def test_single_row_forms_match_full_restatement(mode, G, L, cp):
    """The per-row helpers used to sample full-size problems agree with the full oracle."""
    q, k, v, kd, vd, dout = mo.make_inputs(8, 1, 40, 2, 32, L, G)
    o, lse, dq, dk, dv, dkd, dvd = mo.moda_attention_ref_grads(q, k, v, kd, vd, dout, None, G, mode, cp)
    scale = 32 ** -0.5
    for r in (0, 7, 40 * G - 1):
        tm = mo.row_terms(q, k, v, kd, vd, dout, 0, 1, r, scale, G, mode, cp)
        assert max_abs(tm["o"], o[0, r, 1]) <= 1e-5 and abs(tm["lse"].item() - lse[0, r, 1].item()) <= 1e-5
        assert max_abs(tm["dq"], dq[0, r, 1]) <= 1e-5
    for c in (0, 17, 40 * L - 1):
        a, b_ = mo.depth_row_grads(q, k, v, kd, vd, dout, 0, 0, c, scale, G, mode, cp)
        assert max_abs(a, dkd[0, c, 0]) <= 1e-5 and max_abs(b_, dvd[0, c, 0]) <= 1e-5
    for j in (36, 39):
        a, b_ = mo.seq_key_grads(q, k, v, kd, vd, dout, 0, 0, j, scale, G, mode, cp)
        assert max_abs(a, dk[0, j, 0]) <= 1e-5 and max_abs(b_, dv[0, j, 0]) <= 1e-5
