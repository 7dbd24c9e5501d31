"""GPU: the sequence-sharded MoDA operator with the real kernels.

One GPU suffices for the numerics: every rank's share (``rank_forward`` / ``rank_backward`` over
explicit lists of K/V blocks) is run in turn in this process - nothing waits on another rank, the
"collectives" are list indexing - and compared with the unsharded operator and the CPU oracle.
With two or more GPUs visible the same comparison also runs through ``sequence_parallel_moda``
under NCCL (one process per GPU)."""
import os
import socket

import pytest
import torch

from oracle import moda_oracle as mo
from tests.helpers import TOL_LSE_MAX_ABS, TOL_O_MAX_ABS, check_grad, max_abs

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("mode,D,G,L,Tc,W", [
    (mo.MODE_CAUSAL, 128, 4, 4, 256, 3),
    (mo.MODE_CHUNK_VISIBLE, 128, 4, 8, 128, 4),
    (mo.MODE_CAUSAL, 64, 1, 3, 192, 2),
    (mo.MODE_CAUSAL, 128, 2, 0, 320, 2),
])
def test_every_rank_share_on_one_gpu(built_library, mode, D, G, L, Tc, W):
    import moda_b200 as M
    from moda_b200 import _cabi
    from moda_b200.seq_parallel import rank_backward, rank_forward
    dev = torch.device("cuda", 0)
    B, H, T = 1, 2, Tc * W
    q, k, v, kd, vd, dout = mo.make_inputs(70 + Tc, B, T, H, D, L, G, dtype=torch.bfloat16)
    ref = mo.moda_attention_ref_grads(q, k, v, kd, vd, dout, None, G, mode, max(64 // G, 1))
    q, k, v, kd, vd, dout = [None if x is None else x.to(dev) for x in (q, k, v, kd, vd, dout)]
    scale = D ** -0.5
    cut = lambda x, r, rows: None if x is None else x[:, r * Tc * rows:(r + 1) * Tc * rows]   # noqa: E731 - views, consumed in place
    blocks = [(cut(k, j, 1), cut(v, j, 1)) for j in range(W)]
    os_, lses, dqs, dkds, dvds = [], [], [], [], []
    dk = [torch.zeros(B, Tc, H, D, device=dev) for _ in range(W)]
    dv = [torch.zeros(B, Tc, H, D, device=dev) for _ in range(W)]
    for r in range(W):
        qr, kdr, vdr, dor = cut(q, r, G), cut(kd, r, L), cut(vd, r, L), cut(dout, r, G)
        o, lse = rank_forward(qr, blocks[:r + 1], kdr, vdr, scale, G, mode)
        dq, dkv, dkd, dvd = rank_backward(qr, blocks[:r + 1], kdr, vdr, o, lse, dor, scale, G, mode)
        for j, (a, b) in enumerate(dkv):          # what the reduce-scatter would deliver to rank j
            dk[j] += a
            dv[j] += b
        os_.append(o); lses.append(lse); dqs.append(dq); dkds.append(dkd); dvds.append(dvd)
    assert _cabi.device_status() == 0
    o, lse = torch.cat(os_, 1), torch.cat(lses, 1)
    assert max_abs(o.float().cpu(), ref[0]) <= TOL_O_MAX_ABS and max_abs(lse.cpu(), ref[1]) <= TOL_LSE_MAX_ABS
    check_grad("dq", torch.cat(dqs, 1).float().cpu(), ref[2])
    check_grad("dk", torch.cat(dk, 1).cpu(), ref[3])
    check_grad("dv", torch.cat(dv, 1).cpu(), ref[4])
    if L > 0:
        check_grad("d_depth_k", torch.cat(dkds, 1).float().cpu(), ref[5])
        check_grad("d_depth_v", torch.cat(dvds, 1).float().cpu(), ref[6])
    # rank 0's share is the unsharded operator on the first chunk, bit for bit
    o0, lse0 = M.parallel_moda_fwd(cut(q, 0, G), *blocks[0], cached_k=cut(kd, 0, L), cached_v=cut(vd, 0, L),
                                   moda_group_num=G) if mode == mo.MODE_CAUSAL else \
        M.parallel_moda_chunk_visible_fwd(cut(q, 0, G), *blocks[0], cached_k=cut(kd, 0, L), cached_v=cut(vd, 0, L), moda_group_num=G)
    assert torch.equal(o0, os_[0]) and torch.equal(lse0, lses[0])


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _nccl_worker(rank, world, port, ret):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from moda_b200.seq_parallel import sequence_parallel_moda
        B, Tc, H, D, G, L = 1, 256, 2, 128, 4, 4
        q, k, v, kd, vd, dout = mo.make_inputs(5, B, Tc * world, H, D, L, G, dtype=torch.bfloat16)
        sl = lambda x, rows: x[:, rank * Tc * rows:(rank + 1) * Tc * rows].to(dev).requires_grad_(True)   # noqa: E731
        ql, kl, vl, kdl, vdl = sl(q, G), sl(k, 1), sl(v, 1), sl(kd, L), sl(vd, L)
        o, lse = sequence_parallel_moda(ql, kl, vl, kdl, vdl, moda_group_num=G, need_lse=True)
        (o.float() * dout[:, rank * Tc * G:(rank + 1) * Tc * G].to(dev).float()).sum().backward()
        torch.cuda.synchronize()
        ret[rank] = [x.detach().float().cpu() for x in (o, lse, ql.grad, kl.grad, vl.grad, kdl.grad, vdl.grad)]
    finally:
        dist.destroy_process_group()


def test_two_ranks_over_nccl(built_library):
    if torch.cuda.device_count() < 2:
        pytest.skip("needs two GPUs")
    import torch.multiprocessing as mp
    world = 2
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_nccl_worker, args=(world, _free_port(), ret), nprocs=world, join=True)
    B, Tc, H, D, G, L = 1, 256, 2, 128, 4, 4
    q, k, v, kd, vd, dout = mo.make_inputs(5, B, Tc * world, H, D, L, G, dtype=torch.bfloat16)
    ref = mo.moda_attention_ref_grads(q, k, v, kd, vd, dout, None, G, mo.MODE_CAUSAL, 1)
    got = [torch.cat([ret[r][i] for r in range(world)], dim=1) for i in range(7)]
    assert max_abs(got[0], ref[0]) <= TOL_O_MAX_ABS and max_abs(got[1], ref[1]) <= TOL_LSE_MAX_ABS
    for name, a, b in zip(("dq", "dk", "dv", "d_depth_k", "d_depth_v"), got[2:], ref[2:]):
        check_grad(name, a, b)
