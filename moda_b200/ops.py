"""Python mirror of the reference's MoDA operator interface, backed by libmoda_b200.so.

Same names, argument meaning and error behaviour as ``fla.ops.moda`` of hustvl/MoDA:

* ``parallel_moda``                     moda_v14.py:2792-2893
* ``parallel_moda_fwd`` / ``_bwd``      moda_v14.py:381-522 / 1470-1842
* ``parallel_moda_chunk_visible``       moda_v16.py:3614-3651 (``_fwd`` 498-633, ``_bwd`` 2099-2343)
* ``parallel_fda`` (+ ``_fwd``/``_bwd``) fda_v12.py:1346-1449 / 261-400 / 881-1135

plus ``moda_attention``, the unfolded ``[B,T,Hq,D]`` / ``[B,T,L,Hkv,D]`` convenience
form, which is a view of the folded call (query head ``hq = g*Hkv + h`` uses KV head
``h``: vision_tasks/deit/models.py:248-250).

Tensors must live on a CUDA device; every call launches on the current stream of
``q.device`` and does not synchronise.  Unlike the reference, strided (e.g.
head-sliced) inputs are consumed in place when their innermost stride is 1 and the
stride of every other dimension of size > 1 is a positive multiple of 8 elements;
otherwise (odd strides, expanded or flipped views) they are copied like the
reference's ``@contiguous`` (fla/utils.py:130-161).  The tile-tuning arguments
(``customized_*``, ``group_bs`` ...) sit in the reference's positions and are ignored:
the library has one fixed sm_100a configuration per kernel.

The tcgen05 kernels bound every wait; a wait that expires makes its launch return early
with outputs unwritten and records the fact in a sticky device word.  Nothing here
synchronises to look at it: a caller that needs the guarantee reads
``moda_b200.device_status()`` (0 = fine; resets on read) at its next synchronisation point.
"""
from __future__ import annotations

import ctypes
import warnings
from typing import Optional, Tuple

import torch

from . import _cabi
from ._cabi import (MODE_CAUSAL, MODE_CHUNK_VISIBLE, MODE_DEPTH_ONLY, MODE_NONCAUSAL,
                    PATH_AUTO, Problem, Tensor4)

# The reference's chunk-visible launchers hard-code 64 query rows per tile
# (moda_v16.py:581-585, 2183-2187), which makes it a semantic constant of that operator.
CHUNK_VISIBLE_QUERY_ROWS = 64

_DTYPES = {torch.bfloat16: _cabi.DTYPE_BF16, torch.float16: _cabi.DTYPE_FP16}

# kernel path override for tests and benchmarks (PATH_AUTO in normal use)
_forced_path = PATH_AUTO


def set_kernel_path(path: int) -> int:
    """Force PATH_AUTO / PATH_SIMT_MMA / PATH_TCGEN05 for subsequent calls; returns the old value."""
    global _forced_path
    old, _forced_path = _forced_path, int(path)
    return old


def _usable(x: torch.Tensor) -> torch.Tensor:
    """``x`` itself when the library can consume its layout in place, else a contiguous copy."""
    ok = x.stride(-1) == 1 and x.data_ptr() % 16 == 0
    for size, stride in zip(x.shape[:-1], x.stride()[:-1]):
        if size > 1 and (stride <= 0 or stride % 8 != 0):   # expanded (0) and odd strides are copied
            ok = False
    return x if ok else x.contiguous()


def _t4(x: Optional[torch.Tensor]) -> Optional[Tensor4]:
    if x is None:
        return None
    return Tensor4(x.data_ptr(), x.stride(0), x.stride(1), x.stride(2))


def _ref(t: Optional[Tensor4]):
    return ctypes.byref(t) if t is not None else None


def _problem(q, T_kv, L, G, mode, scale, chunk_rows, depth_rows_per_pos=0, accumulate_depth_grads=0) -> Problem:
    if not q.is_cuda:
        raise RuntimeError("moda_b200 runs on CUDA tensors only (there is no CPU path)")
    if q.dtype not in _DTYPES:
        raise TypeError(f"moda_b200 supports bf16/fp16 inputs, got {q.dtype}")
    B, T_q, H, D = q.shape
    return Problem(B, T_kv, H, D, G, L, mode, chunk_rows, _DTYPES[q.dtype], _forced_path,
                   float(scale), q.device.index if q.device.index is not None else torch.cuda.current_device(),
                   int(depth_rows_per_pos), int(accumulate_depth_grads))


def _check_same(q, *others):
    for x in others:
        if x is not None:
            assert x.dtype == q.dtype and x.device == q.device, "all tensors must share dtype and device"


def _forward(q, k, v, cached_k, cached_v, scale, G, mode, chunk_rows=CHUNK_VISIBLE_QUERY_ROWS,
             cache_layers=None, cache_capacity=0):
    """``cache_layers`` / ``cache_capacity``: cached_k / cached_v are an in-place layer cache
    ``[B, T_kv*capacity, H, D]`` of which the first ``cache_layers`` layers are valid."""
    B, T_q, H, D = q.shape
    assert T_q % G == 0, "T_q must be divisible by moda_group_num"
    T_kv = T_q // G
    use_depth = cached_k is not None and cached_v is not None
    L = (cached_k.shape[1] // T_kv if cache_layers is None else cache_layers) if use_depth else 0
    _check_same(q, k, v, cached_k, cached_v)
    q, k, v, cached_k, cached_v = [None if x is None else _usable(x) for x in (q, k, v, cached_k, cached_v)]
    if not use_depth:
        cached_k = cached_v = None
    prob = _problem(q, T_kv, L, G, mode, scale, chunk_rows, cache_capacity)
    o = torch.empty(B, T_q, H, D, dtype=q.dtype, device=q.device)
    lse = torch.empty(B, T_q, H, dtype=torch.float32, device=q.device)
    lib = _cabi.load()
    tq, tk, tv, tkd, tvd, to = map(_t4, (q, k, v, cached_k, cached_v, o))
    with torch.cuda.device(q.device):
        stream = torch.cuda.current_stream().cuda_stream
        rc = lib.moda_b200_fwd(ctypes.byref(prob), _ref(tq), _ref(tk), _ref(tv), _ref(tkd), _ref(tvd),
                               _ref(to), lse.data_ptr(), stream)
    _cabi.check(rc, "moda_b200_fwd")
    return o, lse


def _backward(q, k, v, cached_k, cached_v, o, lse, do, scale, G, mode,
              chunk_rows=CHUNK_VISIBLE_QUERY_ROWS, cache_layers=None, cache_capacity=0, grad_cache=None):
    """``cache_layers`` / ``cache_capacity`` as in ``_forward``; ``grad_cache = (gk, gv)``: gradient
    caches of the same layout to which the depth gradients are ADDED (the returned depth gradients
    are then those tensors)."""
    B, T_q, H, D = q.shape
    T_kv = T_q // G
    use_depth = cached_k is not None and cached_v is not None
    L = (cached_k.shape[1] // T_kv if cache_layers is None else cache_layers) if use_depth else 0
    _check_same(q, k, v, cached_k, cached_v, o, do)
    q, k, v, cached_k, cached_v, o, do = [
        None if x is None else _usable(x) for x in (q, k, v, cached_k, cached_v, o, do)]
    if not use_depth:
        cached_k = cached_v = None
    lse = lse.contiguous()
    assert lse.dtype == torch.float32
    prob = _problem(q, T_kv, L, G, mode, scale, chunk_rows, cache_capacity, 1 if grad_cache is not None else 0)
    dq = torch.empty_like(q, memory_format=torch.contiguous_format)
    dk = torch.empty_like(k, memory_format=torch.contiguous_format) if k is not None else None
    dv = torch.empty_like(v, memory_format=torch.contiguous_format) if v is not None else None
    if grad_cache is not None:
        dkd, dvd = grad_cache
        assert use_depth and dkd.shape == cached_k.shape and dvd.shape == cached_v.shape
        assert _usable(dkd) is dkd and _usable(dvd) is dvd
    else:
        dkd = torch.empty_like(cached_k, memory_format=torch.contiguous_format) if use_depth else None
        dvd = torch.empty_like(cached_v, memory_format=torch.contiguous_format) if use_depth else None
    lib = _cabi.load()
    nbytes = ctypes.c_size_t(0)
    _cabi.check(lib.moda_b200_bwd_workspace_bytes(ctypes.byref(prob), ctypes.byref(nbytes)),
                "moda_b200_bwd_workspace_bytes")
    ws = torch.empty(max(int(nbytes.value), 256), dtype=torch.uint8, device=q.device)
    ts = list(map(_t4, (q, k, v, cached_k, cached_v, o)))
    gs = list(map(_t4, (do, dq, dk, dv, dkd, dvd)))
    with torch.cuda.device(q.device):
        stream = torch.cuda.current_stream().cuda_stream
        rc = lib.moda_b200_bwd(ctypes.byref(prob), *[_ref(t) for t in ts], lse.data_ptr(),
                               *[_ref(t) for t in gs], ws.data_ptr(), ws.numel(), stream)
    _cabi.check(rc, "moda_b200_bwd")
    return dq, dk, dv, dkd, dvd


def last_launch_count() -> int:
    """Kernel launches issued by the most recent library call on this thread."""
    return int(_cabi.load().moda_b200_last_launch_count())


def tensor_pipe_rates(device=None) -> dict:
    """Measured clocks per ``tcgen05.mma`` instruction (M = 128, K = 16, bf16) for the shapes the
    attention kernels use: ``{"ss_n64": .., "ss_n128": .., "ss_n256": .., "ts_n64": .., "ts_n128": ..,
    "ts_n256": ..}`` (SS: both operands in shared memory, TS: A in TMEM; nominal would be N/2).
    Measurement aid with no reference counterpart; synchronises the current stream."""
    dev = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    out = torch.zeros(6, dtype=torch.float32, device=dev)
    with torch.cuda.device(dev):
        _cabi.tensor_pipe_rates(out.data_ptr(), dev.index or 0, torch.cuda.current_stream().cuda_stream)
        vals = out.cpu().tolist()
    return dict(zip(_cabi.TENSOR_PIPE_SHAPES, vals))


# --------------------------------------------------------------------------- autograd
class _ModaFunction(torch.autograd.Function):
    """Autograd glue (reference: moda_v14.py:2649-2789, moda_v16.py:3320-3493,
    fda_v12.py:1207-1338).  Saves inputs, o and lse; ``dlse`` is ignored like the
    reference (moda_v14.py:2727)."""

    @staticmethod
    def forward(ctx, q, k, v, cached_k, cached_v, scale, G, mode):
        o, lse = _forward(q, k, v, cached_k, cached_v, scale, G, mode)
        ctx.save_for_backward(q, k, v, cached_k, cached_v, o, lse)
        ctx.scale, ctx.G, ctx.mode = scale, G, mode
        ctx.mark_non_differentiable(lse)
        return o, lse

    @staticmethod
    def backward(ctx, do, dlse_unused):
        q, k, v, cached_k, cached_v, o, lse = ctx.saved_tensors
        dq, dk, dv, dkd, dvd = _backward(q, k, v, cached_k, cached_v, o, lse, do.to(q.dtype),
                                         ctx.scale, ctx.G, ctx.mode)
        return dq, dk, dv, dkd, dvd, None, None, None


# --------------------------------------------------------------------------- wrappers
def _prepare(api, q, k, v, g, cached_k, cached_v, scale, G, head_first, return_depth_grads,
             warn_shape, cu_seqlens, need_kv=True):
    assert g is None, f"{api}: gating (g) is not supported on the MoDA path"            # moda_v14.py:2672
    assert cu_seqlens is None, f"{api}: variable-length input is not supported"          # moda_v14.py:2673
    if head_first:
        q = q.transpose(1, 2)
        k = k.transpose(1, 2) if k is not None else None
        v = v.transpose(1, 2) if v is not None else None
        if cached_k is not None and cached_v is not None:
            cached_k, cached_v = cached_k.transpose(1, 2), cached_v.transpose(1, 2)
    elif warn_shape and q.shape[1] < q.shape[2]:
        warnings.warn(f"[{api}] detected seq_len({q.shape[1]}) < num_heads({q.shape[2]}). "
                      "input may be in head_first format while head_first=True is not set.")
    B, T_q, HQ, Kdim = q.shape
    assert G > 0
    if need_kv:
        T_kv, H = k.shape[1], k.shape[2]
    else:
        assert cached_k is not None and cached_v is not None, f"{api} requires cached_k/cached_v"
        assert T_q % G == 0, "T_q must be divisible by moda_group_num"
        T_kv, H = T_q // G, cached_k.shape[2]
    assert HQ == H, (
        "Implicit head-dimension GQA is not allowed. Please fold grouping only into "
        "`moda_group_num`: use q.shape[2] == k.shape[2] and set T_q = T_kv * moda_group_num.")
    if scale is None:
        scale = Kdim ** -0.5
    if G > 1:
        assert T_q == T_kv * G, "When moda_group_num > 1, T_q must equal T_kv * moda_group_num"
    else:
        assert T_q == T_kv, "When moda_group_num=1, T_q must equal T_kv"
    if need_kv:
        assert v.shape[1] == T_kv and v.shape[2] == H and k.shape[0] == B and v.shape[0] == B
        assert k.shape[3] == Kdim and v.shape[3] == Kdim, "head dims of q, k and v must match"
    if cached_k is not None and cached_v is not None:
        assert cached_k.shape[0] == B and cached_v.shape[0] == B
        assert cached_k.shape[2] == H and cached_v.shape[2] == H, "cached_k/v head count mismatch"
        assert cached_k.shape[1] % T_kv == 0, "cached_k time dimension must be T_kv * L"
        assert cached_v.shape[1] == cached_k.shape[1], "cached_v shape mismatch"
        assert cached_k.shape[3] == Kdim and cached_v.shape[3] == Kdim
        if cached_k.shape[1] == 0:
            cached_k = cached_v = None
        elif (cached_k.requires_grad or cached_v.requires_grad) and not return_depth_grads:
            warnings.warn("cached_k/v requires gradients, but return_depth_grads=False. "
                          "Gradients are still computed and returned.")
    else:
        cached_k = cached_v = None
    return q, k, v, cached_k, cached_v, float(scale)


def parallel_moda(q, k, v, g=None, cached_k=None, cached_v=None, scale=None, cu_seqlens=None,
                  moda_group_num=1, is_causal=True, head_first=False, need_lse=False,
                  return_depth_grads=True, warn_shape=True, customized_BT=None, customized_BS=None,
                  customized_BT_backward=None, customized_BS_backward=None, group_bs=None,
                  group_warps=None, depth_bs=None, depth_warps=None):
    """MoDA attention, own-position depth KV (reference: moda_v14.py:2792-2893).

    Returns ``o`` ([B,T_q,H,D], q.dtype) or ``(o, lse)`` (lse fp32, base-2) when
    ``need_lse``.  Outputs stay in the reference's layout (also for ``head_first``:
    the reference does not transpose back)."""
    q, k, v, cached_k, cached_v, scale = _prepare(
        "parallel_moda", q, k, v, g, cached_k, cached_v, scale, moda_group_num, head_first,
        return_depth_grads, warn_shape, cu_seqlens)
    mode = MODE_CAUSAL if is_causal else MODE_NONCAUSAL
    o, lse = _ModaFunction.apply(q, k, v, cached_k, cached_v, scale, moda_group_num, mode)
    return (o, lse) if need_lse else o


def parallel_moda_chunk_visible(q, k, v, g=None, cached_k=None, cached_v=None, scale=None,
                                cu_seqlens=None, moda_group_num=1, head_first=False, need_lse=False,
                                return_depth_grads=True, warn_shape=True, customized_BT=None,
                                customized_BS=None, customized_BT_backward=None,
                                customized_BS_backward=None):
    """Causal MoDA whose queries also see the depth KV of earlier positions of their
    64-query-row chunk (reference: moda_v16.py:3614-3651; oracle chunk_size = 64 // G)."""
    assert CHUNK_VISIBLE_QUERY_ROWS % moda_group_num == 0, "moda_group_num must divide 64"
    q, k, v, cached_k, cached_v, scale = _prepare(
        "parallel_moda_chunk_visible", q, k, v, g, cached_k, cached_v, scale, moda_group_num,
        head_first, return_depth_grads, warn_shape, cu_seqlens)
    o, lse = _ModaFunction.apply(q, k, v, cached_k, cached_v, scale, moda_group_num, MODE_CHUNK_VISIBLE)
    return (o, lse) if need_lse else o


def parallel_fda(q, k=None, v=None, g=None, cached_k=None, cached_v=None, scale=None,
                 cu_seqlens=None, moda_group_num=1, head_first=False, need_lse=False,
                 return_depth_grads=True, warn_shape=True, customized_BT=None, customized_BS=None,
                 customized_BT_backward=None, customized_BS_backward=None, group_bs=None,
                 group_warps=None, depth_bs=None, depth_warps=None):
    """Flash depth attention: each query attends only to the L depth KV of its own
    position (reference: fda_v12.py:1346-1449)."""
    assert k is None and v is None, "Flash Depth Attention does not accept legacy k/v; pass None"
    q, _, _, cached_k, cached_v, scale = _prepare(
        "parallel_fda", q, None, None, g, cached_k, cached_v, scale, moda_group_num, head_first,
        return_depth_grads, warn_shape, cu_seqlens, need_kv=False)
    assert cached_k is not None, "Flash Depth Attention requires L >= 1"                # fda_v12.py:301
    o, lse = _ModaFunction.apply(q, None, None, cached_k, cached_v, scale, moda_group_num, MODE_DEPTH_ONLY)
    return (o, lse) if need_lse else o


# ---- low-level forms (no autograd), same returns as the reference ------------------
def parallel_moda_fwd(q, k, v, g_cumsum=None, scale=None, cu_seqlens=None, cached_k=None,
                      cached_v=None, moda_group_num=1, is_causal=True, customized_BT=None,
                      customized_BS=None, customized_BK=None, customized_BV=None,
                      customized_num_warps=None):
    """(o, lse) — reference: moda_v14.py:381-522."""
    assert g_cumsum is None and cu_seqlens is None
    scale = q.shape[-1] ** -0.5 if scale is None else scale
    return _forward(q, k, v, cached_k, cached_v, scale, moda_group_num,
                    MODE_CAUSAL if is_causal else MODE_NONCAUSAL)


def parallel_moda_bwd(q, k, v, o, g_cumsum, lse, do, scale=None, chunk_size=128, cu_seqlens=None,
                      cached_k=None, cached_v=None, moda_group_num=1, is_causal=True,
                      customized_BT=None, customized_BS=None, customized_BK=None, customized_BV=None,
                      customized_num_warps=None, group_bs=None, group_warps=None, depth_bs=None,
                      depth_warps=None):
    """(dq, dk, dv, dg_cumsum=None, d_cached_k, d_cached_v) — reference: moda_v14.py:1470-1842.
    ``chunk_size`` is unused, as in the reference."""
    assert g_cumsum is None and cu_seqlens is None
    scale = q.shape[-1] ** -0.5 if scale is None else scale
    dq, dk, dv, dkd, dvd = _backward(q, k, v, cached_k, cached_v, o, lse, do, scale, moda_group_num,
                                     MODE_CAUSAL if is_causal else MODE_NONCAUSAL)
    return dq, dk, dv, None, dkd, dvd


def parallel_moda_chunk_visible_fwd(q, k, v, g_cumsum=None, scale=None, cu_seqlens=None,
                                    cached_k=None, cached_v=None, moda_group_num=1,
                                    customized_BT=None, customized_BS=None, customized_BK=None,
                                    customized_BV=None, customized_num_warps=None):
    """(o, lse) — reference: moda_v16.py:498-633."""
    assert g_cumsum is None and cu_seqlens is None
    scale = q.shape[-1] ** -0.5 if scale is None else scale
    return _forward(q, k, v, cached_k, cached_v, scale, moda_group_num, MODE_CHUNK_VISIBLE)


def parallel_moda_chunk_visible_bwd(q, k, v, o, g_cumsum, lse, do, scale=None, chunk_size=128,
                                    cu_seqlens=None, cached_k=None, cached_v=None,
                                    moda_group_num=1, customized_BT=None, customized_BS=None,
                                    customized_BK=None, customized_BV=None, customized_num_warps=None):
    """(dq, dk, dv, None, d_cached_k, d_cached_v) — reference: moda_v16.py:2099-2343."""
    assert g_cumsum is None and cu_seqlens is None
    scale = q.shape[-1] ** -0.5 if scale is None else scale
    dq, dk, dv, dkd, dvd = _backward(q, k, v, cached_k, cached_v, o, lse, do, scale, moda_group_num,
                                     MODE_CHUNK_VISIBLE)
    return dq, dk, dv, None, dkd, dvd


def parallel_fda_fwd(q, g_cumsum=None, scale=None, cu_seqlens=None, cached_k=None, cached_v=None,
                     moda_group_num=1, customized_BT=None, customized_BS=None, customized_BK=None,
                     customized_BV=None, customized_num_warps=None):
    """(o, lse) — reference: fda_v12.py:261-400."""
    assert g_cumsum is None and cu_seqlens is None
    scale = q.shape[-1] ** -0.5 if scale is None else scale
    return _forward(q, None, None, cached_k, cached_v, scale, moda_group_num, MODE_DEPTH_ONLY)


def parallel_fda_bwd(q, o, g_cumsum, lse, do, scale=None, chunk_size=128, cu_seqlens=None,
                     cached_k=None, cached_v=None, moda_group_num=1, customized_BT=None,
                     customized_BS=None, customized_BK=None, customized_BV=None,
                     customized_num_warps=None, group_bs=None, group_warps=None, depth_bs=None,
                     depth_warps=None):
    """(dq, dg_cumsum=None, d_cached_k, d_cached_v) — reference: fda_v12.py:881-1135.
    ``chunk_size`` is unused, as in the reference."""
    assert g_cumsum is None and cu_seqlens is None
    scale = q.shape[-1] ** -0.5 if scale is None else scale
    dq, _, _, dkd, dvd = _backward(q, None, None, cached_k, cached_v, o, lse, do, scale,
                                   moda_group_num, MODE_DEPTH_ONLY)
    return dq, None, dkd, dvd


# ---- projection outputs -> operator inputs, without copies --------------------------
def fold_qkv(q_proj, kv_proj, num_kv_heads: int, groups: int):
    """Views of a block's projection outputs in the operator's layouts — no copy, no kernel.

    ``q_proj [B, N, groups*num_kv_heads*D]`` (output of the query ``Linear``) and
    ``kv_proj [B, N, 2*num_kv_heads*D]`` (output of the fused key/value ``Linear``) become
    ``q [B, N*groups, num_kv_heads, D]`` (GQA folded into time, query head ``g*Hkv + h`` on KV
    head ``h``), ``k`` and ``v [B, N, num_kv_heads, D]``, exactly as the reference's caller forms
    them (vision_tasks/deit/models.py:244-253).  There ``k = kv[:, :, 0]`` and ``v = kv[:, :, 1]``
    are strided views that the reference operator then copies (``@contiguous``,
    fla/utils.py:139-140); this library reads them through their strides, so the projection's
    epilogue already writes the layout the kernels consume and nothing is left to fuse.
    """
    B, N, C = q_proj.shape
    D = C // (groups * num_kv_heads)
    assert C == groups * num_kv_heads * D and kv_proj.shape == (B, N, 2 * num_kv_heads * D)
    q = q_proj.reshape(B, N, groups, num_kv_heads, D).reshape(B, N * groups, num_kv_heads, D)
    kv = kv_proj.reshape(B, N, 2, num_kv_heads, D)
    return q, kv[:, :, 0], kv[:, :, 1]


# ---- unfolded convenience form -----------------------------------------------------
def moda_attention(q, k, v, depth_k=None, depth_v=None, is_causal=True, chunk_size=None,
                   groups=None, scale=None) -> Tuple[torch.Tensor, torch.Tensor]:
    """``q [B,T,Hq,D]``, ``k, v [B,T,Hkv,D]``, ``depth_k, depth_v [B,T,L,Hkv,D]`` ->
    ``(o [B,T,Hq,D], lse [B,T,Hq])``.

    A view of the folded operators: query head ``hq = g*Hkv + h`` attends with KV head
    ``h`` (the DeiT fold, vision_tasks/deit/models.py:248-250).  ``chunk_size`` (query
    rows; only 64 is defined by the reference) selects the chunk-visible operator;
    ``k is None`` selects depth-only attention.  Differentiable.
    """
    B, T, Hq, D = q.shape
    Hkv = (k if k is not None else depth_k).shape[-2]
    G = groups if groups is not None else Hq // Hkv
    assert Hq == G * Hkv, "Hq must equal groups * Hkv"
    qf = q.reshape(B, T, G, Hkv, D).reshape(B, T * G, Hkv, D)
    ck = depth_k.reshape(B, -1, Hkv, D) if depth_k is not None else None
    cv = depth_v.reshape(B, -1, Hkv, D) if depth_v is not None else None
    if k is None:
        o, lse = parallel_fda(qf, cached_k=ck, cached_v=cv, scale=scale, moda_group_num=G,
                              need_lse=True, warn_shape=False)
    elif chunk_size is not None:
        assert is_causal and chunk_size == CHUNK_VISIBLE_QUERY_ROWS, \
            "chunk-visible MoDA is causal with 64 query rows per chunk"
        o, lse = parallel_moda_chunk_visible(qf, k, v, cached_k=ck, cached_v=cv, scale=scale,
                                             moda_group_num=G, need_lse=True, warn_shape=False)
    else:
        o, lse = parallel_moda(qf, k, v, cached_k=ck, cached_v=cv, scale=scale, moda_group_num=G,
                               is_causal=is_causal, need_lse=True, warn_shape=False)
    return o.reshape(B, T, G * Hkv, D), lse.reshape(B, T, G * Hkv)


# ---- backward for callers that may not allocate -----------------------------------
def backward_into_static_scratch(q, k, v, cached_k, cached_v, o, lse, do, dq, dk, dv, d_cached_k,
                                 d_cached_v, scale, moda_group_num, mode,
                                 chunk_rows=CHUNK_VISIBLE_QUERY_ROWS) -> None:
    """Backward into gradient tensors the caller already owns, with the kernels' scratch
    taken from the fixed device array inside the library (``moda_b200_bwd_static_scratch``).

    Nothing is allocated here, neither by torch nor by CUDA: this is the form for callers
    that run where allocation is off limits (inside a region that must not call
    ``cudaMalloc``, or a callback that only receives its buffers).  All tensors must
    already be in a layout the library consumes in place (innermost stride 1, other
    strides multiples of 8 elements, 16-byte aligned) — they are not copied.  Raises
    ``ModaLibraryError`` (status ``MODA_ERR_TOO_LARGE``) when the problem needs more than
    ``_cabi.STATIC_SCRATCH_BYTES`` of scratch.  The array is shared by all calls on a
    device: do not let two such calls overlap on the GPU, and make the first call on a
    device outside stream capture (it resolves the array's address).
    """
    B, T_q, H, D = q.shape
    T_kv = T_q // moda_group_num
    use_depth = cached_k is not None and cached_v is not None
    L = cached_k.shape[1] // T_kv if use_depth else 0
    for x in (q, k, v, cached_k, cached_v, o, do, dq, dk, dv, d_cached_k, d_cached_v):
        if x is not None and _usable(x) is not x:
            raise ValueError("backward_into_static_scratch does not copy: pass tensors with innermost "
                             "stride 1, other strides multiples of 8, 16-byte aligned")
    assert lse.dtype == torch.float32 and lse.is_contiguous()
    prob = _problem(q, T_kv, L, moda_group_num, mode, scale, chunk_rows)
    lib = _cabi.load()
    ts = list(map(_t4, (q, k, v, cached_k, cached_v, o)))
    gs = list(map(_t4, (do, dq, dk, dv, d_cached_k, d_cached_v)))
    with torch.cuda.device(q.device):
        stream = torch.cuda.current_stream().cuda_stream
        rc = lib.moda_b200_bwd_static_scratch(ctypes.byref(prob), *[_ref(t) for t in ts], lse.data_ptr(),
                                              *[_ref(t) for t in gs], stream)
    _cabi.check(rc, "moda_b200_bwd_static_scratch")
