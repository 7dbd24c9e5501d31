"""CPU: the sequence-sharded MoDA operator's host logic under a world_size-2 gloo group.

The kernels need a GPU, so here ``ops._forward`` / ``ops._backward`` are replaced by a dense fp32
torch evaluation of the same block problems (scores with the visibility mask, probabilities from
the GIVEN lse in the backward, as the kernels do).  What is tested is everything around them:
the block decomposition (earlier chunks non-causal, own chunk causal + depth), the exact merge of
the partial softmaxes, the all-gather of K/V, the reduce-scatter of dk/dv to the owning ranks and
the autograd wiring - against the CPU oracle on the unsharded sequence.
"""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import moda_oracle as mo

LOG2E = 1.4426950408889634


def _mask(Tq, Tk, G, mode, L=0, is_depth=False, cp=1):
    r = torch.arange(Tq)[:, None] // G
    if not is_depth:
        j = torch.arange(Tk)[None, :]
        return torch.ones(Tq, Tk, dtype=torch.bool) if mode == mo.MODE_NONCAUSAL else (j <= r)
    c = torch.arange(Tk)[None, :] // L
    if mode == mo.MODE_CHUNK_VISIBLE:
        return (c <= r) & (c // cp == r // cp)
    return c == r


def _scores(q, k, v, kd, vd, scale, G, mode):
    """logits (base 2) [B,H,Tq,K_all], values [B,H,K_all,D], keys [B,H,K_all,D], mask."""
    B, Tq, H, D = q.shape
    ks, vs, ms = [k], [v], [_mask(Tq, k.shape[1], G, mode)]
    if kd is not None:
        L = kd.shape[1] // k.shape[1]
        ks.append(kd); vs.append(vd); ms.append(_mask(Tq, kd.shape[1], G, mode, L, True, max(64 // G, 1)))
    K = torch.cat(ks, 1).float().permute(0, 2, 1, 3)
    V = torch.cat(vs, 1).float().permute(0, 2, 1, 3)
    m = torch.cat(ms, 1)
    s = torch.einsum("bthd,bhkd->bhtk", q.float(), K) * (scale * LOG2E)
    return s.masked_fill(~m, float("-inf")), K, V


def fake_forward(q, k, v, cached_k, cached_v, scale, G, mode, *a, **kw):
    s, K, V = _scores(q, k, v, cached_k, cached_v, scale, G, mode)
    lse = torch.logsumexp(s * 0.6931471805599453, dim=-1) * LOG2E
    p = torch.exp2(s - lse[..., None])
    o = torch.einsum("bhtk,bhkd->bthd", p, V)
    return o.to(q.dtype), lse.permute(0, 2, 1).contiguous()


def fake_backward(q, k, v, cached_k, cached_v, o, lse, do, scale, G, mode, *a, **kw):
    s, K, V = _scores(q, k, v, cached_k, cached_v, scale, G, mode)
    p = torch.exp2(s - lse.permute(0, 2, 1)[..., None])                    # the GIVEN (merged) lse
    delta = (o.float() * do.float()).sum(-1).permute(0, 2, 1)              # [B,H,Tq]
    dp = torch.einsum("bthd,bhkd->bhtk", do.float(), V)
    ds = p * (dp - delta[..., None])
    dq = scale * torch.einsum("bhtk,bhkd->bthd", ds, K)
    dK = scale * torch.einsum("bhtk,bthd->bkhd", ds, q.float())
    dV = torch.einsum("bhtk,bthd->bkhd", p, do.float())
    Tk = k.shape[1]
    dkd = dvd = None
    if cached_k is not None:
        dkd, dvd = dK[:, Tk:].to(q.dtype), dV[:, Tk:].to(q.dtype)
    return dq.to(q.dtype), dK[:, :Tk].to(q.dtype), dV[:, :Tk].to(q.dtype), dkd, dvd


def test_merge_of_partial_softmaxes_is_exact():
    from moda_b200.seq_parallel import merge_partials
    torch.manual_seed(0)
    B, T, H, D, n = 2, 7, 3, 8, 4
    s = torch.randn(B, H, T, 5 * n) * 3
    v = torch.randn(B, H, 5 * n, D)
    lse_all = torch.logsumexp(s, -1)
    o_all = torch.einsum("bhtk,bhkd->bthd", torch.softmax(s, -1), v)
    parts = []
    for j in range(n):
        sj, vj = s[..., 5 * j:5 * j + 5], v[:, :, 5 * j:5 * j + 5]
        parts.append((torch.einsum("bhtk,bhkd->bthd", torch.softmax(sj, -1), vj),
                      (torch.logsumexp(sj, -1) * LOG2E).permute(0, 2, 1)))
    o, lse = merge_partials(parts, torch.float32)
    assert torch.allclose(o, o_all, atol=1e-5) and torch.allclose(lse, (lse_all * LOG2E).permute(0, 2, 1), atol=1e-5)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, mode, G, L, ret):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from moda_b200 import ops, seq_parallel
        ops._forward, ops._backward = fake_forward, fake_backward         # this process only
        B, Tc, H, D = 1, 64 // G * 2, 2, 16
        T = Tc * world
        q, k, v, kd, vd, dout = mo.make_inputs(9, B, T, H, D, L, G)
        sl = lambda x, rows: None if x is None else x[:, rank * Tc * rows:(rank + 1) * Tc * rows].clone().requires_grad_(True)  # noqa: E731
        ql, kl, vl, kdl, vdl = sl(q, G), sl(k, 1), sl(v, 1), sl(kd, L), sl(vd, L)
        o, lse = seq_parallel.sequence_parallel_moda(ql, kl, vl, kdl, vdl, moda_group_num=G,
                                                     chunk_visible=(mode == mo.MODE_CHUNK_VISIBLE), need_lse=True)
        (o * dout[:, rank * Tc * G:(rank + 1) * Tc * G]).sum().backward()
        ret[rank] = [x.detach() if x is not None else None for x in
                     (o, lse, ql.grad, kl.grad, vl.grad, None if kdl is None else kdl.grad, None if vdl is None else vdl.grad)]
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("mode,G,L", [(mo.MODE_CAUSAL, 2, 3), (mo.MODE_CHUNK_VISIBLE, 4, 2), (mo.MODE_CAUSAL, 1, 0)])
def test_sequence_parallel_world2_matches_the_unsharded_oracle(mode, G, L):
    world = 2
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), mode, G, L, ret), nprocs=world, join=True)
    B, Tc, H, D = 1, 64 // G * 2, 2, 16
    q, k, v, kd, vd, dout = mo.make_inputs(9, B, Tc * world, H, D, L, G)
    ref = mo.moda_attention_ref_grads(q, k, v, kd, vd, dout, None, G, mode, max(64 // G, 1))
    rows = [G, G, G, 1, 1, L, L]
    for i, (want, per) in enumerate(zip(ref, rows)):
        if want is None:
            continue
        got = torch.cat([ret[r][i] for r in range(world)], dim=1)
        assert got.shape == want.shape, i
        assert torch.allclose(got, want, atol=2e-4, rtol=1e-4), (i, (got - want).abs().max())
