"""GPU parity: the CUDA path (called through the Python mirror, i.e. through the
C-ABI) against the CPU oracle on the same seeded inputs.

Tolerances (bf16/fp16 inputs, fp32 oracle on the same rounded inputs):
  max|o - o_ref| <= 2e-2, max|lse - lse_ref| <= 1e-3 (base-2 units),
  every gradient rel-L2 <= 5e-2 (a gradient the oracle gives as numerically zero - rms below
  1e-3, e.g. a query with a single visible key - has no relative error and is held to
  max-abs <= 1e-2 instead; tests/helpers.py: check_grad).
The case grid covers the ranges of the reference's operator test
(tests/ops/test_moda.py:95-198: T_kv 1..256 incl. odd, H 1..8, L 0..16,
G in {1,2,4,8}, fp16/bf16, scales 0.0156..2.0) and adds what that test lacks:
non-causal, chunk-visible, depth-only, lse, D=128, strided inputs.
"""
import itertools

import pytest
import torch

from oracle import moda_oracle as mo
from tests.helpers import (TOL_LSE_MAX_ABS, TOL_O_MAX_ABS, check_grad, golden_names, load_golden, max_abs, t)

pytestmark = pytest.mark.gpu

DT = {"bf16": torch.bfloat16, "fp16": torch.float16}


def _run_case(M, mode, B, T, H, D, L, G, dtype, scale, seed, path=None, check_bwd=True, inputs=None):
    dev = torch.device("cuda", 0)
    if inputs is None:
        inputs = mo.make_inputs(seed, B, T, H, D, L, G, dtype=dtype, with_seq=(mode != mo.MODE_DEPTH_ONLY))
    q, k, v, kd, vd, dout = inputs
    cp = max(64 // G, 1)
    ref = mo.moda_attention_ref_grads(q, k, v, kd, vd, dout, scale, G, mode, cp)
    leaves = [None if x is None else x.to(dev).requires_grad_(True) for x in (q, k, v, kd, vd)]
    old = M.set_kernel_path(path if path is not None else M.PATH_AUTO)
    try:
        if mode == mo.MODE_DEPTH_ONLY:
            o, lse = M.parallel_fda(leaves[0], cached_k=leaves[3], cached_v=leaves[4], scale=scale,
                                    moda_group_num=G, need_lse=True, warn_shape=False)
        elif mode == mo.MODE_CHUNK_VISIBLE:
            o, lse = M.parallel_moda_chunk_visible(leaves[0], leaves[1], leaves[2], cached_k=leaves[3],
                                                   cached_v=leaves[4], scale=scale, moda_group_num=G,
                                                   need_lse=True, warn_shape=False)
        else:
            o, lse = M.parallel_moda(leaves[0], leaves[1], leaves[2], cached_k=leaves[3], cached_v=leaves[4],
                                     scale=scale, moda_group_num=G, is_causal=(mode == mo.MODE_CAUSAL),
                                     need_lse=True, warn_shape=False)
        assert M.last_launch_count() >= 1
        assert o.dtype == dtype and lse.dtype == torch.float32
        eo, el = max_abs(o.float().cpu(), ref[0]), max_abs(lse.cpu(), ref[1])
        assert eo <= TOL_O_MAX_ABS, f"o max-abs {eo}"
        assert el <= TOL_LSE_MAX_ABS, f"lse max-abs {el}"
        if check_bwd:
            (o.float() * dout.to(dev).float()).sum().backward()
            for name, leaf, g_ref in zip(("dq", "dk", "dv", "d_depth_k", "d_depth_v"), leaves, ref[2:]):
                if leaf is None:
                    continue
                assert leaf.grad is not None and leaf.grad.dtype == dtype, name
                check_grad(name, leaf.grad.float().cpu(), g_ref)
    finally:
        M.set_kernel_path(old)
    return o, lse


@pytest.fixture(scope="module")
def M(built_library):
    import moda_b200
    assert torch.cuda.is_available()
    return moda_b200


# (B, T_kv, H, L, G, dtype, scale) — causal own-position MoDA, D = 64
CAUSAL_CASES = [
    (1, 1, 1, 0, 1, "fp16", None), (1, 2, 2, 0, 2, "fp16", None), (2, 3, 2, 1, 2, "fp16", 1.0),
    (1, 63, 1, 0, 1, "fp16", 1.0), (1, 64, 2, 1, 1, "fp16", None), (1, 65, 2, 0, 4, "fp16", None),
    (2, 47, 3, 2, 2, "fp16", 0.5), (2, 95, 4, 4, 1, "fp16", None), (3, 80, 3, 0, 2, "fp16", None),
    (2, 111, 5, 4, 1, "fp16", 1.0), (1, 32, 2, 8, 2, "fp16", None), (1, 40, 2, 8, 4, "fp16", 0.25),
    (1, 129, 6, 3, 2, "fp16", 0.0156), (1, 191, 7, 5, 1, "fp16", 2.0), (1, 193, 2, 16, 1, "fp16", None),
    (2, 256, 4, 4, 2, "fp16", 1.0), (1, 128, 8, 12, 8, "fp16", None), (2, 192, 4, 0, 4, "fp16", 0.1),
    (1, 160, 2, 8, 2, "bf16", 0.1), (1, 128, 2, 8, 4, "bf16", 0.1), (1, 63, 2, 4, 2, "bf16", None),
    (2, 80, 3, 4, 4, "bf16", 0.1), (1, 255, 1, 7, 8, "bf16", None), (1, 64, 2, 0, 2, "bf16", None),
    (1, 33, 2, 1, 8, "bf16", 0.5), (1, 200, 3, 16, 1, "bf16", None),
]


@pytest.mark.parametrize("B,T,H,L,G,dt,scale", CAUSAL_CASES)
def test_causal_moda_d64(M, B, T, H, L, G, dt, scale):
    _run_case(M, mo.MODE_CAUSAL, B, T, H, 64, L, G, DT[dt], scale, seed=2025 + T + L)


@pytest.mark.parametrize("mode", [mo.MODE_CAUSAL, mo.MODE_NONCAUSAL, mo.MODE_CHUNK_VISIBLE, mo.MODE_DEPTH_ONLY])
@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("T,L,G", [(1, 1, 1), (70, 3, 1), (197, 11, 1), (128, 4, 4), (130, 2, 2), (96, 5, 8)])
@pytest.mark.parametrize("forced", [False, True], ids=["auto", "mma_sync"])
def test_all_modes(M, mode, D, T, L, G, forced):
    # "auto" evaluates own-position depth rows in the bandwidth kernels and merges the sequence
    # part in the attention kernels' epilogue; "mma_sync" keeps everything in one attention kernel
    _run_case(M, mode, 2, T, 2, D, L, G, torch.bfloat16, None, seed=7 + T + D,
              path=(M.PATH_SIMT_MMA if forced else None))


@pytest.mark.parametrize("mode", [mo.MODE_CAUSAL, mo.MODE_NONCAUSAL, mo.MODE_CHUNK_VISIBLE])
def test_no_depth(M, mode):
    _run_case(M, mode, 1, 150, 2, 128, 0, 2, torch.bfloat16, None, seed=3)


@pytest.mark.parametrize("mode,T,L,G", [
    (mo.MODE_CAUSAL, 1024, 24, 4),          # benchmark config 2 shape at reduced T, B, H
    (mo.MODE_CHUNK_VISIBLE, 1024, 32, 4),   # benchmark config 4 shape at reduced T, H
    (mo.MODE_CHUNK_VISIBLE, 512, 8, 1),
    (mo.MODE_DEPTH_ONLY, 512, 32, 1),       # benchmark config 3 shape at reduced B, T, H
    (mo.MODE_CAUSAL, 640, 0, 1),
])
def test_config_shapes_reduced_d128(M, mode, T, L, G):
    _run_case(M, mode, 1, T, 2, 128, L, G, torch.bfloat16, None, seed=11 + T)


def test_deit_shape_noncausal(M):
    # benchmark config 5 at reduced batch: T=197, H=6, D=64, L=11, non-causal
    _run_case(M, mo.MODE_NONCAUSAL, 3, 197, 6, 64, 11, 1, torch.bfloat16, None, seed=4)


@pytest.mark.parametrize("name", golden_names())
def test_against_reference_golden_fixtures(M, name):
    """Kernel vs outputs of the reference's own torch oracle (fp32 inputs rounded to
    bf16 for the kernel, so the fixture is compared at bf16-input tolerance)."""
    rec = load_golden(name)
    c = rec["cfg"]
    dev = torch.device("cuda", 0)
    q, k, v, kd, vd, dout = mo.make_inputs(c["seed"], c["B"], c["T_kv"], c["H"], c["D"], c["L"], c["G"],
                                           with_seq=(c["mode"] != mo.MODE_DEPTH_ONLY))
    if c["mode"] == mo.MODE_CHUNK_VISIBLE and c["chunk_positions"] * c["G"] != 64:
        pytest.skip("operator defines 64 query rows per chunk")
    xs = [None if x is None else x.to(dev).to(torch.bfloat16) for x in (q, k, v, kd, vd)]
    if c["mode"] == mo.MODE_DEPTH_ONLY:
        o, lse = M.parallel_fda_fwd(xs[0], scale=c["scale"], cached_k=xs[3], cached_v=xs[4],
                                    moda_group_num=c["G"])
    elif c["mode"] == mo.MODE_CHUNK_VISIBLE:
        o, lse = M.parallel_moda_chunk_visible_fwd(xs[0], xs[1], xs[2], scale=c["scale"], cached_k=xs[3],
                                                   cached_v=xs[4], moda_group_num=c["G"])
    else:
        o, lse = M.parallel_moda_fwd(xs[0], xs[1], xs[2], scale=c["scale"], cached_k=xs[3], cached_v=xs[4],
                                     moda_group_num=c["G"], is_causal=(c["mode"] == mo.MODE_CAUSAL))
    # inputs were rounded to bf16 (rel 2^-9) before the kernel: allow that on top
    assert max_abs(o.float().cpu(), t(rec["o"])) <= 6e-2
    assert max_abs(lse.cpu(), t(rec["lse"])) <= 6e-2
    # and exactly at kernel tolerance against the oracle on the rounded inputs
    ro, rl = mo.moda_attention_ref(*[None if x is None else x.cpu() for x in xs], c["scale"], c["G"],
                                   c["mode"], max(c["chunk_positions"], 1))
    assert max_abs(o.float().cpu(), ro) <= TOL_O_MAX_ABS
    assert max_abs(lse.cpu(), rl) <= TOL_LSE_MAX_ABS


def test_bitwise_reproducible(M):
    dev = torch.device("cuda", 0)
    q, k, v, kd, vd, dout = [x.to(dev) for x in mo.make_inputs(21, 2, 300, 2, 128, 6, 4, dtype=torch.bfloat16)]
    outs = []
    for _ in range(2):
        o, lse = M.parallel_moda_fwd(q, k, v, cached_k=kd, cached_v=vd, moda_group_num=4)
        grads = M.parallel_moda_bwd(q, k, v, o, None, lse, dout, cached_k=kd, cached_v=vd, moda_group_num=4)
        outs.append([o, lse] + [g for g in grads if g is not None])
    for a, b in zip(*outs):
        assert torch.equal(a, b)


def test_strided_head_slice_inputs_are_consumed_in_place(M):
    """A KV-head shard of a [B,T,H,D] tensor is a non-contiguous view; the library takes
    element strides, so no copy is needed and the result equals the contiguous call."""
    dev = torch.device("cuda", 0)
    q, k, v, kd, vd, _ = [x.to(dev) for x in mo.make_inputs(31, 2, 100, 4, 64, 3, 2, dtype=torch.bfloat16)]
    o_full, lse_full = M.parallel_moda_fwd(q, k, v, cached_k=kd, cached_v=vd, moda_group_num=2)
    sl = slice(1, 3)
    o_s, lse_s = M.parallel_moda_fwd(q[:, :, sl], k[:, :, sl], v[:, :, sl], cached_k=kd[:, :, sl],
                                     cached_v=vd[:, :, sl], moda_group_num=2)
    assert torch.equal(o_s, o_full[:, :, sl]) and torch.equal(lse_s, lse_full[:, :, sl])


def test_unfolded_convenience_form(M):
    dev = torch.device("cuda", 0)
    B, T, Hkv, G, D, L = 2, 90, 2, 4, 64, 3
    gen = torch.Generator().manual_seed(5)
    q = torch.randn(B, T, G * Hkv, D, generator=gen).to(torch.bfloat16)
    k = torch.randn(B, T, Hkv, D, generator=gen).to(torch.bfloat16)
    v = torch.randn(B, T, Hkv, D, generator=gen).to(torch.bfloat16)
    dk_ = torch.randn(B, T, L, Hkv, D, generator=gen).to(torch.bfloat16)
    dv_ = torch.randn(B, T, L, Hkv, D, generator=gen).to(torch.bfloat16)
    o, lse = M.moda_attention(q.to(dev), k.to(dev), v.to(dev), dk_.to(dev), dv_.to(dev), is_causal=True)
    assert o.shape == (B, T, G * Hkv, D) and lse.shape == (B, T, G * Hkv)
    # direct per-head formulation: query head hq = g*Hkv + h uses KV head h
    for hq in (0, 3, 5):
        h = hq % Hkv
        ro, rl = mo.moda_attention_ref(q[:, :, hq:hq + 1], k[:, :, h:h + 1], v[:, :, h:h + 1],
                                       dk_[:, :, :, h:h + 1].reshape(B, T * L, 1, D),
                                       dv_[:, :, :, h:h + 1].reshape(B, T * L, 1, D), None, 1, mo.MODE_CAUSAL)
        assert max_abs(o[:, :, hq:hq + 1].float().cpu(), ro) <= TOL_O_MAX_ABS
        assert max_abs(lse[:, :, hq:hq + 1].cpu(), rl) <= TOL_LSE_MAX_ABS


def test_errors_surface_as_exceptions(M):
    dev = torch.device("cuda", 0)
    q = torch.zeros(1, 8, 1, 96, dtype=torch.bfloat16, device=dev)
    with pytest.raises(M.ModaLibraryError, match="head dim"):
        M.parallel_moda(q, q, q, warn_shape=False)


# ------------------------------------------------------------------ tcgen05 kernels
@pytest.mark.parametrize("mode", [mo.MODE_CAUSAL, mo.MODE_NONCAUSAL, mo.MODE_CHUNK_VISIBLE])
@pytest.mark.parametrize("T,L,G,dt", [
    (1, 1, 1, "bf16"), (127, 0, 1, "bf16"), (128, 2, 1, "fp16"), (129, 3, 2, "bf16"), (300, 5, 4, "bf16"),
    (1000, 3, 4, "fp16"), (513, 16, 8, "bf16"), (2048, 24, 4, "bf16"),
])
@pytest.mark.parametrize("D", [64, 128])
def test_tcgen05_forward(M, mode, T, L, G, dt, D):
    """The tcgen05/TMEM/TMA forward, forced; its bounded waits must not have expired."""
    from moda_b200 import _cabi
    _run_case(M, mode, 1, T, 2, D, L, G, DT[dt], None, seed=100 + T, path=M.PATH_TCGEN05, check_bwd=False)
    assert _cabi.device_status() == 0


def test_tcgen05_forward_matches_mma_sync_path(M):
    """Two independent implementations of the same forward agree closely (both round P to bf16)."""
    dev = torch.device("cuda", 0)
    q, k, v, kd, vd, _ = [x.to(dev) for x in mo.make_inputs(77, 2, 777, 3, 128, 7, 2, dtype=torch.bfloat16)]
    res = {}
    for path in (M.PATH_SIMT_MMA, M.PATH_TCGEN05):
        old = M.set_kernel_path(path)
        try:
            res[path] = M.parallel_moda_fwd(q, k, v, cached_k=kd, cached_v=vd, moda_group_num=2)
        finally:
            M.set_kernel_path(old)
    (o1, l1), (o2, l2) = res[M.PATH_SIMT_MMA], res[M.PATH_TCGEN05]
    assert max_abs(o1.float(), o2.float()) <= 1e-2 and max_abs(l1, l2) <= 1e-4


def test_tcgen05_path_refuses_what_it_cannot_run(M):
    """A non-positive scale is served by the mma.sync kernels only (the tcgen05 softmax takes the row
    maximum before scaling); forcing the tcgen05 path on it is refused, the auto path computes it."""
    dev = torch.device("cuda", 0)
    q = torch.zeros(1, 64, 1, 64, dtype=torch.bfloat16, device=dev)
    old = M.set_kernel_path(M.PATH_TCGEN05)
    try:
        with pytest.raises(M.ModaLibraryError, match="does not support"):
            M.parallel_moda_fwd(q, q, q, scale=-0.5)
    finally:
        M.set_kernel_path(old)
    _run_case(M, mo.MODE_CAUSAL, 1, 100, 2, 64, 3, 2, torch.bfloat16, -0.25, seed=5)


@pytest.mark.parametrize("mode", [mo.MODE_CAUSAL, mo.MODE_NONCAUSAL, mo.MODE_CHUNK_VISIBLE])
@pytest.mark.parametrize("T,L,G,dt", [
    (1, 1, 1, "bf16"), (64, 0, 1, "bf16"), (127, 2, 1, "fp16"), (129, 3, 2, "bf16"), (300, 5, 4, "bf16"),
    (1000, 3, 4, "fp16"), (513, 16, 8, "bf16"), (1536, 24, 4, "bf16"),
])
@pytest.mark.parametrize("D,bwd", [(64, "two_kernel"), (128, "fused"), (128, "two_kernel")])
def test_tcgen05_forward_and_backward(M, mode, T, L, G, dt, D, bwd):
    """tcgen05 forward + backward, forced: the two-kernel backward (dq kernel + dk/dv kernel, the
    default) and the fused key-stationary backward (D = 128: five matmuls, dq summed in fixed
    point), each with the statistics pass and the depth-gradient kernel."""
    from moda_b200 import _cabi
    path = M.PATH_TCGEN05_FUSED_BWD if bwd == "fused" else M.PATH_TCGEN05
    _run_case(M, mode, 2 if T < 600 else 1, T, 2, D, L, G, DT[dt], None, seed=200 + T, path=path, check_bwd=True)
    assert _cabi.device_status() == 0


@pytest.mark.parametrize("scale_dout", [1.0, 3.0e4, 1.0e-6])
def test_fused_backward_fixed_point_scale_follows_the_gradient_magnitude(M, scale_dout):
    """dq of the fused backward is summed as scaled integers; the scale comes from a bound on each
    64-row block's |dQ|, so upstream gradients of any magnitude (loss scaling, vanishing gradients)
    keep the same relative accuracy.  Rows of very different magnitude in one call included."""
    dev = torch.device("cuda", 0)
    B, T, H, D, L, G = 1, 700, 2, 128, 4, 2
    q, k, v, kd, vd, dout = mo.make_inputs(321, B, T, H, D, L, G, dtype=torch.bfloat16)
    dout = (dout.float() * scale_dout)
    dout[:, : T * G // 2] *= 1.0e-3                      # half of the rows a thousand times smaller
    dout = dout.to(torch.bfloat16)
    ref = mo.moda_attention_ref_grads(q, k, v, kd, vd, dout, None, G, mo.MODE_CAUSAL, 1)
    q, k, v, kd, vd, dout = [x.to(dev) for x in (q, k, v, kd, vd, dout)]
    old = M.set_kernel_path(M.PATH_TCGEN05_FUSED_BWD)
    try:
        o, lse = M.parallel_moda_fwd(q, k, v, cached_k=kd, cached_v=vd, moda_group_num=G)
        g1 = M.parallel_moda_bwd(q, k, v, o, None, lse, dout, cached_k=kd, cached_v=vd, moda_group_num=G)
        g2 = M.parallel_moda_bwd(q, k, v, o, None, lse, dout, cached_k=kd, cached_v=vd, moda_group_num=G)
    finally:
        M.set_kernel_path(old)
    for a, b in zip(g1, g2):
        assert (a is None and b is None) or torch.equal(a, b)          # integer sums: order cannot matter
    dq = g1[0].float().cpu()
    half = T * G // 2
    for name, got, want in (("dq small rows", dq[:, :half], ref[2][:, :half]), ("dq large rows", dq[:, half:], ref[2][:, half:])):
        e = ((got - want).pow(2).sum().sqrt() / want.pow(2).sum().sqrt()).item()
        assert e <= 5e-2, f"{name}: rel-L2 {e}"


def test_tcgen05_backward_bitwise_reproducible_and_batched(M):
    dev = torch.device("cuda", 0)
    q, k, v, kd, vd, dout = [x.to(dev) for x in mo.make_inputs(23, 3, 333, 2, 128, 4, 4, dtype=torch.bfloat16)]
    old = M.set_kernel_path(M.PATH_TCGEN05)
    try:
        outs = []
        for _ in range(2):
            o, lse = M.parallel_moda_chunk_visible_fwd(q, k, v, cached_k=kd, cached_v=vd, moda_group_num=4)
            grads = M.parallel_moda_chunk_visible_bwd(q, k, v, o, None, lse, dout, cached_k=kd, cached_v=vd,
                                                      moda_group_num=4)
            outs.append([o, lse] + [g for g in grads if g is not None])
        for a, b in zip(*outs):
            assert torch.equal(a, b)
    finally:
        M.set_kernel_path(old)


# ------------------------------------------------------------------ depth-only bandwidth kernels
@pytest.mark.parametrize("D,T,L,G,dt", [
    (128, 1, 1, 1, "bf16"), (128, 33, 5, 2, "bf16"), (128, 100, 32, 1, "bf16"), (128, 64, 40, 1, "fp16"),
    (128, 50, 7, 4, "bf16"), (64, 197, 11, 1, "bf16"), (64, 60, 33, 4, "fp16"), (64, 17, 3, 8, "bf16"),
])
def test_depth_only_bandwidth_kernels(M, D, T, L, G, dt):
    """parallel_fda on the default path: one warp per (batch, position, head), fp32 registers.
    (G values the backward kernel does not hold in registers fall back to the mma.sync path.)"""
    _run_case(M, mo.MODE_DEPTH_ONLY, 2, T, 3, D, L, G, DT[dt], None, seed=300 + T + L)


def test_depth_only_paths_agree(M):
    dev = torch.device("cuda", 0)
    q, _, _, kd, vd, dout = mo.make_inputs(55, 2, 77, 2, 128, 9, 2, dtype=torch.bfloat16, with_seq=False)
    q, kd, vd, dout = [x.to(dev) for x in (q, kd, vd, dout)]
    outs = {}
    for path in (M.PATH_AUTO, M.PATH_SIMT_MMA):
        old = M.set_kernel_path(path)
        try:
            o, lse = M.parallel_fda_fwd(q, cached_k=kd, cached_v=vd, moda_group_num=2)
            g = M.parallel_fda_bwd(q, o, None, lse, dout, cached_k=kd, cached_v=vd, moda_group_num=2)
            outs[path] = [o, lse] + [x for x in g if x is not None]
        finally:
            M.set_kernel_path(old)
    for a, b in zip(outs[M.PATH_AUTO], outs[M.PATH_SIMT_MMA]):
        assert max_abs(a.float(), b.float()) <= 2e-2


@pytest.mark.parametrize("fwd", ["one_tile", "two_tiles"])
@pytest.mark.parametrize("D", [64, 128])
@pytest.mark.parametrize("mode,T,L,G", [(mo.MODE_CAUSAL, 300, 5, 4), (mo.MODE_CHUNK_VISIBLE, 1000, 3, 4),
                                        (mo.MODE_NONCAUSAL, 129, 2, 1), (mo.MODE_CAUSAL, 2048, 24, 4),
                                        (mo.MODE_CHUNK_VISIBLE, 96, 32, 4), (mo.MODE_CAUSAL, 1, 1, 1)])
def test_tcgen05_forward_variants(M, mode, T, L, G, D, fwd):
    """Each tcgen05 forward forced (the default picks by grid size): one query tile per CTA with
    two CTAs per SM, or two query tiles per CTA with one softmax warpgroup each."""
    from moda_b200 import _cabi
    path = M.PATH_TCGEN05_ONE_TILE if fwd == "one_tile" else M.PATH_TCGEN05_TWO_TILES
    _run_case(M, mode, 1, T, 2, D, L, G, torch.bfloat16, None, seed=400 + T, path=path, check_bwd=False)
    assert _cabi.device_status() == 0


def test_tcgen05_forwards_are_bit_identical(M):
    """The two forwards share one softmax arithmetic: which of them ran cannot be told from o, lse."""
    dev = torch.device("cuda", 0)
    for D in (64, 128):
        q, k, v, kd, vd, _ = [x.to(dev) for x in mo.make_inputs(91, 2, 700, 2, D, 6, 2, dtype=torch.bfloat16)]
        res = []
        for path in (M.PATH_TCGEN05_ONE_TILE, M.PATH_TCGEN05_TWO_TILES):
            old = M.set_kernel_path(path)
            try:
                res.append(M.parallel_moda_chunk_visible_fwd(q, k, v, cached_k=kd, cached_v=vd, moda_group_num=2))
            finally:
                M.set_kernel_path(old)
        assert torch.equal(res[0][0], res[1][0]) and torch.equal(res[0][1], res[1][1])


@pytest.mark.parametrize("B,H,T,D", [(1, 2, 700, 128), (8, 10, 600, 128), (1, 2, 300, 64), (8, 10, 520, 64)],
                         ids=["one_tile_d128", "two_tiles_d128", "one_tile_d64", "two_tiles_d64"])
@pytest.mark.parametrize("mode,L", [(mo.MODE_CAUSAL, 6), (mo.MODE_NONCAUSAL, 11)])
def test_split_depth_merges_into_each_tcgen05_forward(M, mode, L, B, H, T, D):
    """G = 1 on the auto path: the bandwidth kernels write the own-position depth partial and the
    tcgen05 forward / dq kernels fold the sequence part into it.  The small grids take the
    one-tile forward, the large ones (at least one 256-row CTA per SM) the two-tile forward."""
    from moda_b200 import _cabi
    _run_case(M, mode, B, T, H, D, L, 1, torch.bfloat16, None, seed=900 + T)
    assert _cabi.device_status() == 0


def test_expanded_views_are_copied_not_misread(M):
    """Zero-stride (expanded) tensors - a gradient broadcast over batch, depth KV shared by the
    batch - must give the results of their materialised copies: the library refuses non-positive
    strides and the wrapper falls back to a contiguous copy like the reference's @contiguous."""
    dev = torch.device("cuda", 0)
    B, T, H, D, L, G = 3, 200, 2, 128, 4, 2
    q, k, v, kd, vd, dout = [x.to(dev) for x in mo.make_inputs(61, B, T, H, D, L, G, dtype=torch.bfloat16)]
    k_e, kd_e, vd_e = k[:1].expand(B, -1, -1, -1), kd[:1].expand(B, -1, -1, -1), vd[:1].expand(B, -1, -1, -1)
    dout_e = dout[:1].expand(B, -1, -1, -1)
    assert k_e.stride(0) == 0 and dout_e.stride(0) == 0
    o1, lse1 = M.parallel_moda_fwd(q, k_e, v, cached_k=kd_e, cached_v=vd_e, moda_group_num=G)
    o2, lse2 = M.parallel_moda_fwd(q, k_e.contiguous(), v, cached_k=kd_e.contiguous(), cached_v=vd_e.contiguous(),
                                   moda_group_num=G)
    assert torch.equal(o1, o2) and torch.equal(lse1, lse2)
    g1 = M.parallel_moda_bwd(q, k_e, v, o1, None, lse1, dout_e, cached_k=kd_e, cached_v=vd_e, moda_group_num=G)
    g2 = M.parallel_moda_bwd(q, k_e.contiguous(), v, o1, None, lse1, dout_e.contiguous(),
                             cached_k=kd_e.contiguous(), cached_v=vd_e.contiguous(), moda_group_num=G)
    for a, b in zip(g1, g2):
        assert (a is None and b is None) or torch.equal(a, b)
    # the C ABI itself refuses such a view instead of reading batch b at a made-up offset
    from moda_b200 import _cabi
    import ctypes
    lib = _cabi.load()
    prob = _cabi.Problem(B, T, H, D, G, 0, M.MODE_CAUSAL, 64, _cabi.DTYPE_BF16, M.PATH_AUTO, D ** -0.5, 0)
    t4 = lambda x: ctypes.byref(_cabi.Tensor4(x.data_ptr(), x.stride(0), x.stride(1), x.stride(2)))
    rc = lib.moda_b200_fwd(ctypes.byref(prob), t4(q), t4(k_e), t4(v), None, None, t4(o1), lse1.data_ptr(),
                           torch.cuda.current_stream().cuda_stream)
    assert rc == 5
    # and autograd through a broadcast gradient: sum over batch gives every batch row the same dO
    leaves = [x.clone().requires_grad_(True) for x in (q, k, v, kd, vd)]
    w = torch.randn(T * G, H, D, device=dev, dtype=torch.bfloat16)
    o = M.parallel_moda(*leaves[:3], cached_k=leaves[3], cached_v=leaves[4], moda_group_num=G, warn_shape=False)
    (o.sum(0) * w).sum().backward()
    ref = mo.moda_attention_ref_grads(*[x.cpu() for x in (q, k, v, kd, vd)], w.cpu()[None].expand(B, -1, -1, -1).contiguous(),
                                      None, G, mo.MODE_CAUSAL, 32)
    for name, leaf, g_ref in zip(("dq", "dk", "dv", "d_depth_k", "d_depth_v"), leaves, ref[2:]):
        check_grad(name, leaf.grad.float().cpu(), g_ref)


def _random_cases(seed, n):
    import random
    rng = random.Random(seed)
    cases = []
    for _ in range(n):
        mode = rng.choice([mo.MODE_CAUSAL, mo.MODE_NONCAUSAL, mo.MODE_CHUNK_VISIBLE])
        G = rng.choice([1, 2, 4, 8])
        T = rng.choice([1, 5, 17, 63, 64, 65, 100, 128, 191, 200, 256, 300, 511, 513, 777, 1024, 1500])
        T = min(T, max(1, 4200 // G))
        L = rng.choice([0, 1, 2, 3, 5, 8, 11, 16, 24, 32, 33])
        cases.append((mode, rng.choice([1, 2]), T, rng.choice([1, 2, 3]), L, G, rng.choice(["bf16", "fp16"]),
                      rng.choice([64, 128]), rng.choice(["auto", "tcgen05", "one_tile", "two_tiles", "fused_bwd"]),
                      rng.randrange(1 << 30)))
    return cases


@pytest.mark.parametrize("mode,B,T,H,L,G,dt,D,path,seed", _random_cases(20251, 48))
def test_randomised_shapes(M, mode, B, T, H, L, G, dt, D, path, seed):
    """Seeded random draws over mode, batch, length, heads, depth layers, group size, dtype, head
    dim and kernel path (auto / tcgen05 / each forward forced); forward and backward."""
    from moda_b200 import _cabi
    paths = {"auto": None, "tcgen05": M.PATH_TCGEN05, "one_tile": M.PATH_TCGEN05_ONE_TILE,
             "two_tiles": M.PATH_TCGEN05_TWO_TILES, "fused_bwd": M.PATH_TCGEN05_FUSED_BWD}
    _run_case(M, mode, B, T, H, D, L, G, DT[dt], None, seed=seed, path=paths[path])
    assert _cabi.device_status() == 0


@pytest.mark.gpu
def test_tensor_pipe_rate_probe(M):
    """The measurement aid returns one finite rate per instruction shape, no faster than the
    nominal N/2 clocks and ordered as the shapes are (larger N and an A operand in shared memory
    cost more), and leaves the status word clean."""
    r = M.tensor_pipe_rates()
    assert set(r) == {"ss_n64", "ss_n128", "ss_n256", "ts_n64", "ts_n128", "ts_n256"}
    for name, v in r.items():
        n = int(name.split("_n")[1])
        assert n / 2 * 0.95 <= v < 4 * n, (name, v)
    assert r["ts_n64"] < r["ts_n128"] < r["ts_n256"]
    assert r["ss_n64"] < r["ss_n128"] < r["ss_n256"]
    for n in (64, 128, 256):
        assert r[f"ts_n{n}"] < r[f"ss_n{n}"]
    assert M.device_status() == 0
