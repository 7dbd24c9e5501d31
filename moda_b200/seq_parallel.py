"""Sequence-sharded (context-parallel) causal MoDA over the ranks of a process group.

The reference has no sequence parallelism: it scales sequence length only by tiling inside one
GPU (its paper names the sharded variant as future work), and the multi-GPU path of this library
shards by (batch x KV-head) without communication (``moda_b200.sharding``).  This module is the
other axis, for sequences whose K/V or activations do not fit one GPU: rank ``r`` of ``W`` holds
the contiguous chunk ``r`` of the sequence - ``q [B, Tc*G, H, D]``, ``k, v [B, Tc, H, D]`` and its
own depth K/V ``[B, Tc*L, H, D]`` (depth rows belong to positions, so they never cross ranks).

Forward, rank ``r``:
  1. the K/V chunks are exchanged with ONE all-gather into this GPU's own memory (NCCL over
     NVLink; the kernels then read ordinary local tensors through their own tensor maps);
  2. the local block (keys of chunk ``r``) runs the causal / chunk-visible operator with the depth
     K/V; every earlier block ``j < r`` runs the non-causal operator (all of its keys are visible to
     all local queries), no depth;
  3. the partial ``(o_j, lse_j)`` are merged exactly: ``lse = log2 sum_j 2^lse_j``,
     ``o = sum_j 2^(lse_j - lse) o_j`` (fp32).
Backward: every block's backward runs with the MERGED ``o`` and ``lse`` (then ``delta`` and the
probabilities are the global ones), ``dq`` is the sum over blocks, and the ``dk, dv`` a rank computes
for the chunks of earlier ranks are returned to their owners with one reduce-scatter (fp32).

Causal attention gives rank ``r`` ``r + 1`` blocks of work, so contiguous chunks are imbalanced
(the last rank works ``W`` times as long as the first); ``interleaved=True`` is not provided - a
caller that needs balance assigns two chunks per rank (``r`` and ``2W - 1 - r``) and calls this
twice.  ``chunk_visible`` needs ``Tc * G`` to be a multiple of 64 so that no 64-row chunk straddles
two ranks.

The algorithm is written over explicit lists of K/V blocks (``rank_forward`` / ``rank_backward``),
so a single process can run every rank's share in turn (that is how the single-GPU test checks it
against the unsharded operator); ``sequence_parallel_moda`` adds the collectives and autograd.
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple

import torch

from . import ops
from ._cabi import MODE_CAUSAL, MODE_CHUNK_VISIBLE, MODE_NONCAUSAL


def merge_partials(parts: Sequence[Tuple[torch.Tensor, torch.Tensor]], out_dtype) -> Tuple[torch.Tensor, torch.Tensor]:
    """Exact merge of softmax partials over disjoint key sets: ``parts`` = [(o_j, lse_j)] with
    lse in base-2 units.  Returns (o, lse)."""
    lse_all = torch.stack([l for _, l in parts], dim=0)                       # [n, B, T, H]
    lse = torch.logsumexp(lse_all * 0.6931471805599453, dim=0) * 1.4426950408889634
    o = torch.zeros_like(parts[0][0], dtype=torch.float32)
    for o_j, l_j in parts:
        o += torch.exp2(l_j - lse).unsqueeze(-1) * o_j.float()
    return o.to(out_dtype), lse


def rank_forward(q, kv_blocks: Sequence[Tuple[torch.Tensor, torch.Tensor]], depth_k, depth_v, scale, G, mode):
    """The share of one rank: ``kv_blocks[j]`` = (K, V) of chunk ``j`` for ``j = 0..r`` (the last one
    is the rank's own chunk).  Returns merged (o, lse)."""
    assert mode in (MODE_CAUSAL, MODE_CHUNK_VISIBLE)
    if mode == MODE_CHUNK_VISIBLE:
        assert q.shape[1] % ops.CHUNK_VISIBLE_QUERY_ROWS == 0, "a 64-row chunk must not straddle two ranks"
    parts = []
    for j, (kj, vj) in enumerate(kv_blocks):
        if j == len(kv_blocks) - 1:
            parts.append(ops._forward(q, kj, vj, depth_k, depth_v, scale, G, mode))
        else:
            parts.append(ops._forward(q, kj, vj, None, None, scale, G, MODE_NONCAUSAL))
    if len(parts) == 1:
        return parts[0]
    return merge_partials(parts, q.dtype)


def rank_backward(q, kv_blocks, depth_k, depth_v, o, lse, do, scale, G, mode):
    """Gradients of one rank's share: (dq, [(dk_j, dv_j) for j = 0..r] in fp32, d_depth_k, d_depth_v).
    ``o`` and ``lse`` are the MERGED forward results."""
    dq = None
    dkv: List[Tuple[torch.Tensor, torch.Tensor]] = []
    dkd = dvd = None
    for j, (kj, vj) in enumerate(kv_blocks):
        if j == len(kv_blocks) - 1:
            g = ops._backward(q, kj, vj, depth_k, depth_v, o, lse, do, scale, G, mode)
            dkd, dvd = g[3], g[4]
        else:
            g = ops._backward(q, kj, vj, None, None, o, lse, do, scale, G, MODE_NONCAUSAL)
        dq = g[0].float() if dq is None else dq + g[0].float()
        dkv.append((g[1].float(), g[2].float()))
    return dq.to(q.dtype), dkv, dkd, dvd


class _Comm:
    """The two collectives the operator needs, over ``torch.distributed``."""

    def __init__(self, group=None):
        import torch.distributed as dist
        self.dist, self.group = dist, group
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)

    def all_gather(self, x: torch.Tensor) -> List[torch.Tensor]:
        out = [torch.empty_like(x) for _ in range(self.world)]
        self.dist.all_gather(out, x.contiguous(), group=self.group)
        return out

    def reduce_scatter(self, xs: Sequence[torch.Tensor]) -> torch.Tensor:
        """Sum over ranks of ``xs[j]`` delivered to rank ``j``."""
        stacked = torch.stack(list(xs), dim=0).contiguous()
        if self.dist.get_backend(self.group) == "nccl":
            out = torch.empty_like(stacked[0])
            self.dist.reduce_scatter_tensor(out, stacked, group=self.group)
            return out
        self.dist.all_reduce(stacked, group=self.group)          # gloo has no reduce-scatter
        return stacked[self.rank].clone()


class _SeqParallelFunction(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, depth_k, depth_v, scale, G, mode, comm: _Comm):
        ks, vs = comm.all_gather(k), comm.all_gather(v)
        blocks = [(ks[j], vs[j]) for j in range(comm.rank)] + [(k, v)]
        o, lse = rank_forward(q, blocks, depth_k, depth_v, scale, G, mode)
        ctx.save_for_backward(q, k, v, depth_k, depth_v, o, lse, *[t for j in range(comm.rank) for t in (ks[j], vs[j])])
        ctx.scale, ctx.G, ctx.mode, ctx.comm = scale, G, mode, comm
        ctx.mark_non_differentiable(lse)
        return o, lse

    @staticmethod
    def backward(ctx, do, _dlse):
        q, k, v, depth_k, depth_v, o, lse, *rest = ctx.saved_tensors
        comm = ctx.comm
        blocks = [(rest[2 * j], rest[2 * j + 1]) for j in range(comm.rank)] + [(k, v)]
        dq, dkv, dkd, dvd = rank_backward(q, blocks, depth_k, depth_v, o, lse, do.to(q.dtype), ctx.scale, ctx.G, ctx.mode)
        zero = torch.zeros_like(k, dtype=torch.float32)
        dks = [dkv[j][0] if j <= comm.rank else zero for j in range(comm.world)]
        dvs = [dkv[j][1] if j <= comm.rank else zero for j in range(comm.world)]
        dk = comm.reduce_scatter(dks).to(k.dtype)
        dv = comm.reduce_scatter(dvs).to(v.dtype)
        return dq, dk, dv, dkd, dvd, None, None, None, None


def sequence_parallel_moda(q, k, v, cached_k=None, cached_v=None, scale: Optional[float] = None,
                           moda_group_num: int = 1, chunk_visible: bool = False, need_lse: bool = False,
                           group=None):
    """Causal MoDA (own-position depth, or chunk-visible) with the sequence sharded in contiguous
    chunks over the ranks of ``group`` (default: the world).  Arguments are this rank's chunk, in
    the operators' folded layout; every rank must call it.  Differentiable."""
    comm = _Comm(group)
    scale = q.shape[-1] ** -0.5 if scale is None else float(scale)
    mode = MODE_CHUNK_VISIBLE if chunk_visible else MODE_CAUSAL
    assert q.shape[1] == k.shape[1] * moda_group_num and q.shape[2] == k.shape[2]
    if cached_k is None or cached_v is None or cached_k.shape[1] == 0:
        cached_k = cached_v = None
    o, lse = _SeqParallelFunction.apply(q, k, v, cached_k, cached_v, scale, moda_group_num, mode, comm)
    return (o, lse) if need_lse else o
