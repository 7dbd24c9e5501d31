"""In-place depth-KV cache for a stack of MoDA layers.

The reference's only in-tree caller rebuilds the depth cache before EVERY layer from the list of
all earlier layers' K/V (``torch.stack(..., dim=2)`` + ``reshape`` + ``contiguous``:
vision_tasks/deit/models.py:361-390), so a model of N layers copies O(N^2) K/V tensors per forward,
and autograd un-stacks as many gradients in the backward.  ``DepthKVCache`` keeps one persistent
``[B, T, Lmax, H, D]`` buffer per K and V instead: each layer's K/V is copied into its slot once
(``moda_b200_depth_append``), the attention kernels read the first ``L`` layers of the buffer in
place (``moda_problem.depth_rows_per_pos``), and in the backward every layer ADDS its depth
gradients into one gradient cache of the same layout, from which each producing layer takes its
slice.

    cache = DepthKVCache(B, T, n_layers - 1, Hkv, D, dtype, device)
    for blk in blocks:
        q, k, v = ...                                   # this layer's projections
        o = cache.attend(q, k, v, moda_group_num=G, is_causal=False)
        cache.append(k, v)                              # visible to the layers after this one

Autograd: ``append`` returns nothing to the caller but keeps a scalar token per layer, which every
later ``attend`` takes as an input; the engine therefore runs an ``append``'s backward only after
all later layers have added their depth gradients, and that backward hands the slot's slice of
the gradient cache to the layer's ``k`` and ``v``.
"""
from __future__ import annotations

import ctypes
from typing import List, Optional

import torch

from . import _cabi
from . import ops
from ._cabi import MODE_CAUSAL, MODE_CHUNK_VISIBLE, MODE_NONCAUSAL


class DepthKVCache:
    """K/V of the preceding layers at every position, written in place layer by layer."""

    def __init__(self, batch: int, seq_len: int, max_layers: int, num_kv_heads: int, head_dim: int,
                 dtype: torch.dtype = torch.bfloat16, device=None):
        assert max_layers >= 1
        self.B, self.T, self.capacity, self.H, self.D = batch, seq_len, max_layers, num_kv_heads, head_dim
        self.k = torch.empty(batch, seq_len * max_layers, num_kv_heads, head_dim, dtype=dtype, device=device)
        self.v = torch.empty_like(self.k)
        self.grad_k: Optional[torch.Tensor] = None     # allocated (zeroed) by the first backward that needs it
        self.grad_v: Optional[torch.Tensor] = None
        self.L = 0
        self._tokens: List[torch.Tensor] = []

    def reset(self) -> None:
        """Start a new forward pass: no layers cached, gradient cache dropped."""
        self.L = 0
        self._tokens = []
        self.grad_k = self.grad_v = None

    def bytes_copied_per_forward(self, n_layers: int) -> int:
        """Bytes of K/V this cache copies for a model of ``n_layers`` attention layers (each of the
        first n_layers - 1 layers once)."""
        per_layer = 2 * self.B * self.T * self.H * self.D * self.k.element_size()
        return (n_layers - 1) * per_layer

    def bytes_copied_by_rebuilding(self, n_layers: int) -> int:
        """The same for the rebuild-before-every-layer scheme of the reference caller: layer i
        stacks i earlier layers and makes the result contiguous."""
        per_layer = 2 * self.B * self.T * self.H * self.D * self.k.element_size()
        return sum(2 * i for i in range(n_layers)) * per_layer      # stack copy + contiguous copy

    # ------------------------------------------------------------------ forward API
    def append(self, k: torch.Tensor, v: torch.Tensor) -> None:
        """Copy this layer's ``k, v [B, T, H, D]`` into the next free slot."""
        assert self.L < self.capacity, "DepthKVCache is full"
        assert k.shape == (self.B, self.T, self.H, self.D) and v.shape == k.shape
        token = _Append.apply(k, v, self, self.L)
        self.L += 1
        self._tokens.append(token)

    def attend(self, q, k, v, scale=None, moda_group_num: int = 1, is_causal: bool = True,
               chunk_visible: bool = False, need_lse: bool = False):
        """MoDA attention of this layer over its own ``k, v`` and the cached layers (same results
        as ``parallel_moda`` / ``parallel_moda_chunk_visible`` on the stacked cache)."""
        scale = q.shape[-1] ** -0.5 if scale is None else float(scale)
        mode = MODE_CHUNK_VISIBLE if chunk_visible else (MODE_CAUSAL if is_causal else MODE_NONCAUSAL)
        assert q.shape[1] == k.shape[1] * moda_group_num and q.shape[2] == k.shape[2]
        o, lse = _CachedAttention.apply(q, k, v, scale, moda_group_num, mode, self, self.L, *self._tokens)
        return (o, lse) if need_lse else o

    # ------------------------------------------------------------------ used by the backward
    def _grad_caches(self):
        if self.grad_k is None:
            self.grad_k = torch.zeros_like(self.k)
            self.grad_v = torch.zeros_like(self.v)
        return self.grad_k, self.grad_v

    def _slot(self, x: torch.Tensor, slot: int) -> torch.Tensor:
        return x.view(self.B, self.T, self.capacity, self.H, self.D)[:, :, slot]


class _Append(torch.autograd.Function):
    @staticmethod
    def forward(ctx, k, v, cache: DepthKVCache, slot: int):
        k_, v_ = ops._usable(k), ops._usable(v)
        prob = ops._problem(k_, cache.T, 0, 1, MODE_CAUSAL, 1.0, ops.CHUNK_VISIBLE_QUERY_ROWS, cache.capacity)
        lib = _cabi.load()
        ts = [ops._t4(x) for x in (k_, v_, cache.k, cache.v)]
        with torch.cuda.device(k.device):
            rc = lib.moda_b200_depth_append(ctypes.byref(prob), *[ctypes.byref(t) for t in ts], slot,
                                            torch.cuda.current_stream().cuda_stream)
        _cabi.check(rc, "moda_b200_depth_append")
        ctx.cache, ctx.slot = cache, slot
        return torch.zeros((), dtype=torch.float32, device=k.device)

    @staticmethod
    def backward(ctx, _grad_token):
        cache = ctx.cache
        if cache.grad_k is None:         # no later layer's backward ran: the slot received nothing
            return None, None, None, None
        return cache._slot(cache.grad_k, ctx.slot).clone(), cache._slot(cache.grad_v, ctx.slot).clone(), None, None


class _CachedAttention(torch.autograd.Function):
    @staticmethod
    def forward(ctx, q, k, v, scale, G, mode, cache: DepthKVCache, L: int, *tokens):
        if L == 0:
            o, lse = ops._forward(q, k, v, None, None, scale, G, mode)
        else:
            o, lse = ops._forward(q, k, v, cache.k, cache.v, scale, G, mode, cache_layers=L,
                                  cache_capacity=cache.capacity)
        # the cache is append-only, so rows of the first L layers never change after this point; it is
        # kept by reference (saving it with save_for_backward would trip autograd's version check on
        # the later in-place appends)
        ctx.save_for_backward(q, k, v, o, lse)
        ctx.scale, ctx.G, ctx.mode, ctx.cache, ctx.L, ctx.n_tokens = scale, G, mode, cache, L, len(tokens)
        ctx.mark_non_differentiable(lse)
        return o, lse

    @staticmethod
    def backward(ctx, do, _dlse):
        q, k, v, o, lse = ctx.saved_tensors
        cache, L = ctx.cache, ctx.L
        if L == 0:
            dq, dk, dv, _, _ = ops._backward(q, k, v, None, None, o, lse, do.to(q.dtype), ctx.scale, ctx.G, ctx.mode)
        else:
            dq, dk, dv, _, _ = ops._backward(q, k, v, cache.k, cache.v, o, lse, do.to(q.dtype), ctx.scale, ctx.G,
                                             ctx.mode, cache_layers=L, cache_capacity=cache.capacity,
                                             grad_cache=cache._grad_caches())
        zeros = [torch.zeros((), dtype=torch.float32, device=q.device) for _ in range(ctx.n_tokens)]
        return (dq, dk, dv, None, None, None, None, None, *zeros)
