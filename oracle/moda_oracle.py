"""CPU oracle for the MoDA attention hot path (TEST INFRASTRUCTURE, not product code).

This file restates, in vectorised fp32 torch, the algorithm of the reference's own
loop oracles:

* ``naive_mixture_of_depth_causal_ref``   libs/moda_triton/fla/ops/moda/moda_v14.py:1900-1991
  (causal and, through ``_ref_seq_kv_limit`` moda_v14.py:1845-1846, non-causal)
* ``naive_mixture_of_depth_causal_chunk_visible_ref``  moda_v16.py:2487-2582
* ``naive_depth_causal_ref``              fda_v12.py:1143-1196

Gradients are obtained by torch autograd through the restatement, the same way the
reference's tests obtain theirs (tests/ops/test_moda.py:262-276).

Parity pin: the restatement is checked against outputs of those reference functions,
run in the build container and committed as fixtures under ``tests/golden/`` by
``tests/golden/make_golden.py``.

Only ``tests/``, ``__graft_entry__.smoke()`` and ``bench.py``'s CPU-baseline /
``--impl reference`` legs may import this module.  The product package never does: it
fails loudly when its CUDA library is missing.

Tensor convention (identical to the reference, moda_v14.py:2792-2862):
  q                  [B, T_kv*G, H, D]   query row r -> base position t = r // G
  k, v               [B, T_kv,   H, D]
  depth_k, depth_v   [B, T_kv*L, H, D]   row t*L + l = layer l's K/V at position t
  o                  [B, T_kv*G, H, D]   fp32
  lse                [B, T_kv*G, H]      fp32, base-2 units (logsumexp / ln 2)
"""
from __future__ import annotations

import math
from typing import Optional, Tuple

import torch

MODE_CAUSAL = 0
MODE_NONCAUSAL = 1
MODE_CHUNK_VISIBLE = 2
MODE_DEPTH_ONLY = 3

_LN2 = math.log(2.0)


def _visibility(
    mode: int, T_kv: int, G: int, L: int, chunk_positions: int, rows: torch.Tensor
) -> Tuple[Optional[torch.Tensor], Optional[torch.Tensor]]:
    """Boolean masks [rows, T_kv] (sequence keys) and [rows, T_kv*L] (depth rows).

    Sequence: key j visible iff j <= t (causal, chunk-visible: moda_v14.py:1966-1968,
    moda_v16.py:2553) or always (non-causal).  Depth: row t'*L+l visible iff t' == t
    (own position: moda_v14.py:1972) or chunk_start(t) <= t' <= t (moda_v16.py:2557-2561).
    """
    t = rows // G
    seq = None
    if mode != MODE_DEPTH_ONLY:
        j = torch.arange(T_kv)
        if mode == MODE_NONCAUSAL:
            seq = torch.ones(rows.numel(), T_kv, dtype=torch.bool)
        else:
            seq = j[None, :] <= t[:, None]
    dep = None
    if L > 0:
        tp = torch.arange(T_kv * L) // L
        if mode == MODE_CHUNK_VISIBLE:
            start = (t // chunk_positions) * chunk_positions
            dep = (tp[None, :] >= start[:, None]) & (tp[None, :] <= t[:, None])
        else:
            dep = tp[None, :] == t[:, None]
    return seq, dep


def moda_attention_ref(
    q: torch.Tensor,
    k: Optional[torch.Tensor],
    v: Optional[torch.Tensor],
    depth_k: Optional[torch.Tensor] = None,
    depth_v: Optional[torch.Tensor] = None,
    scale: Optional[float] = None,
    moda_group_num: int = 1,
    mode: int = MODE_CAUSAL,
    chunk_positions: int = 64,
    row_block: int = 1024,
) -> Tuple[torch.Tensor, torch.Tensor]:
    """fp32 MoDA attention; returns (o [B,T_q,H,D] fp32, lse [B,T_q,H] fp32 base-2).

    One softmax over the visible sequence keys and the visible depth rows of each
    query (moda_v14.py:1970-1989).  Differentiable by autograd.  Memory is bounded by
    processing ``row_block`` query rows at a time; inside a block only the columns
    any of its rows can see are touched, so cost is O(T^2) for the sequence part and
    O(T*span) for the depth part, like the reference kernels.
    """
    B, T_q, H, D = q.shape
    G = moda_group_num
    assert T_q % G == 0
    T_kv = T_q // G
    use_depth = depth_k is not None and depth_v is not None
    L = depth_k.shape[1] // T_kv if use_depth else 0
    if mode == MODE_DEPTH_ONLY:
        assert use_depth and L > 0
    else:
        assert k is not None and v is not None and k.shape[1] == T_kv
    if scale is None:
        scale = 1.0 / math.sqrt(D)

    qf = q.float().permute(0, 2, 1, 3)  # [B,H,T_q,D]
    kf = k.float().permute(0, 2, 1, 3) if k is not None else None
    vf = v.float().permute(0, 2, 1, 3) if v is not None else None
    kdf = depth_k.float().permute(0, 2, 1, 3) if use_depth else None
    vdf = depth_v.float().permute(0, 2, 1, 3) if use_depth else None

    outs, lses = [], []
    for r0 in range(0, T_q, row_block):
        r1 = min(T_q, r0 + row_block)
        rows = torch.arange(r0, r1)
        t_lo, t_hi = r0 // G, (r1 - 1) // G
        # column windows any row of this block can see
        if mode == MODE_DEPTH_ONLY:
            s_hi = 0
        elif mode == MODE_NONCAUSAL:
            s_hi = T_kv
        else:
            s_hi = t_hi + 1
        if L > 0:
            p_lo = (t_lo // chunk_positions) * chunk_positions if mode == MODE_CHUNK_VISIBLE else t_lo
            d_lo, d_hi = p_lo * L, (t_hi + 1) * L
        else:
            d_lo = d_hi = 0
        seq_mask, dep_mask = _visibility(mode, T_kv, G, L, chunk_positions, rows)
        qb = qf[:, :, r0:r1]
        parts, vals = [], []
        if s_hi > 0:
            s = torch.matmul(qb, kf[:, :, :s_hi].transpose(-1, -2)) * scale
            s = s.masked_fill(~seq_mask[:, :s_hi], float("-inf"))
            parts.append(s)
            vals.append(vf[:, :, :s_hi])
        if d_hi > d_lo:
            s = torch.matmul(qb, kdf[:, :, d_lo:d_hi].transpose(-1, -2)) * scale
            s = s.masked_fill(~dep_mask[:, d_lo:d_hi], float("-inf"))
            parts.append(s)
            vals.append(vdf[:, :, d_lo:d_hi])
        logits = torch.cat(parts, dim=-1)
        w = torch.softmax(logits, dim=-1)
        outs.append(torch.matmul(w, torch.cat(vals, dim=2)))
        lses.append(torch.logsumexp(logits, dim=-1) / _LN2)
    o = torch.cat(outs, dim=2).permute(0, 2, 1, 3).contiguous()
    lse = torch.cat(lses, dim=2).permute(0, 2, 1).contiguous()
    return o, lse


def moda_attention_ref_loop(
    q, k, v, depth_k=None, depth_v=None, scale=None, moda_group_num=1,
    mode=MODE_CAUSAL, chunk_positions=64,
):
    """Per-row Python loop with the reference's exact control flow; small cases only.

    Follows moda_v14.py:1958-1989 / moda_v16.py:2545-2580 / fda_v12.py:1181-1194 line
    by line (per (b,h) upcast, slice visible keys, concatenate logits, one softmax).
    Used to cross-check the vectorised restatement on the CPU.
    """
    B, T_q, H, D = q.shape
    G = moda_group_num
    T_kv = T_q // G
    use_depth = depth_k is not None and depth_v is not None
    L = depth_k.shape[1] // T_kv if use_depth else 0
    if scale is None:
        scale = 1.0 / math.sqrt(D)
    out = torch.empty(B, T_q, H, D, dtype=torch.float32)
    lse = torch.empty(B, T_q, H, dtype=torch.float32)
    for b in range(B):
        for h in range(H):
            q_bh = q[b, :, h].float()
            if mode != MODE_DEPTH_ONLY:
                k_bh, v_bh = k[b, :, h].float(), v[b, :, h].float()
            if use_depth:
                kd_bh = depth_k[b, :, h].float().view(T_kv, L, D)
                vd_bh = depth_v[b, :, h].float().view(T_kv, L, D)
            for r in range(T_q):
                t = r // G
                logit_parts, value_parts = [], []
                if mode != MODE_DEPTH_ONLY:
                    end = T_kv if mode == MODE_NONCAUSAL else t + 1
                    logit_parts.append((q_bh[r] @ k_bh[:end].T) * scale)
                    value_parts.append(v_bh[:end])
                if use_depth:
                    start = (t // chunk_positions) * chunk_positions if mode == MODE_CHUNK_VISIBLE else t
                    kd_sel = kd_bh[start : t + 1].reshape(-1, D)
                    logit_parts.append((kd_sel @ q_bh[r]) * scale)
                    value_parts.append(vd_bh[start : t + 1].reshape(-1, D))
                logits = torch.cat(logit_parts)
                w = torch.softmax(logits, dim=0)
                out[b, r, h] = (w.unsqueeze(1) * torch.cat(value_parts)).sum(0)
                lse[b, r, h] = torch.logsumexp(logits, dim=0) / _LN2
    return out, lse


def moda_attention_ref_grads(
    q, k, v, depth_k, depth_v, dout, scale=None, moda_group_num=1,
    mode=MODE_CAUSAL, chunk_positions=64,
):
    """(o, lse, dq, dk, dv, d_depth_k, d_depth_v) in fp32 via autograd on the oracle.

    Loss = sum(o * dout), as in tests/ops/test_moda.py:262-263; ``dlse`` is not
    propagated (the reference ignores it: moda_v14.py:2727).
    Absent inputs give ``None`` gradients.
    """
    leaves = []
    for x in (q, k, v, depth_k, depth_v):
        leaves.append(None if x is None else x.detach().float().clone().requires_grad_(True))
    o, lse = moda_attention_ref(
        leaves[0], leaves[1], leaves[2], leaves[3], leaves[4], scale,
        moda_group_num, mode, chunk_positions,
    )
    (o * dout.float()).sum().backward()
    grads = [None if x is None else x.grad for x in leaves]
    return (o.detach(), lse.detach(), *grads)


def make_inputs(seed, B, T_kv, H, D, L, G, dtype=torch.float32, with_seq=True, with_dout=True):
    """Seeded i.i.d. N(0,1) inputs on the CPU, drawn in the order q, k, v, depth_k,
    depth_v, dout (each as fp32, then cast), matching the reference test's draw
    order (tests/ops/test_moda.py:233-252)."""
    gen = torch.Generator().manual_seed(seed)
    def draw(*shape):
        return torch.randn(*shape, generator=gen, dtype=torch.float32).to(dtype)
    q = draw(B, T_kv * G, H, D)
    k = draw(B, T_kv, H, D) if with_seq else None
    v = draw(B, T_kv, H, D) if with_seq else None
    kd = draw(B, T_kv * L, H, D) if L > 0 else None
    vd = draw(B, T_kv * L, H, D) if L > 0 else None
    dout = draw(B, T_kv * G, H, D) if with_dout else None
    return q, k, v, kd, vd, dout


# ---------------------------------------------------------------------------------------
# Single-row forms, for sampling rows of problems too large for the full restatement.
# The same rule as moda_attention_ref (one softmax over the visible sequence keys and the
# visible depth rows of the query: moda_v14.py:1966-1989, moda_v16.py:2553-2580), written
# for one (b, h, r) at a time so that cost is O(T) per sampled row.
# ---------------------------------------------------------------------------------------
def row_terms(q, k, v, depth_k, depth_v, dout, b, h, r, scale, G, mode, chunk_positions):
    """fp32 terms of query row r of head (b, h): dict with o, lse (base 2), the softmax
    weights over the visible sequence keys [0, s_end) and depth rows [d_lo, d_hi), and - when
    ``dout`` is given - dS over the same two ranges and dq."""
    D = q.shape[-1]
    T_kv = q.shape[1] // G
    L = depth_k.shape[1] // T_kv if depth_k is not None else 0
    t = r // G
    s_end = 0 if mode == MODE_DEPTH_ONLY else (T_kv if mode == MODE_NONCAUSAL else t + 1)
    t0 = (t // chunk_positions) * chunk_positions if mode == MODE_CHUNK_VISIBLE else t
    d_lo, d_hi = t0 * L, (t + 1) * L
    qr = q[b, r, h].float()
    keys, vals = [], []
    if s_end > 0:
        keys.append(k[b, :s_end, h].float()); vals.append(v[b, :s_end, h].float())
    if d_hi > d_lo:
        keys.append(depth_k[b, d_lo:d_hi, h].float()); vals.append(depth_v[b, d_lo:d_hi, h].float())
    K, V = torch.cat(keys), torch.cat(vals)
    logits = (K @ qr) * scale
    w = torch.softmax(logits, dim=0)
    o = w @ V
    out = {"o": o, "lse": torch.logsumexp(logits, 0) / _LN2, "s_end": s_end, "d_lo": d_lo, "d_hi": d_hi,
           "w_seq": w[:s_end], "w_dep": w[s_end:]}
    if dout is not None:
        dor = dout[b, r, h].float()
        dS = w * (V @ dor - (o * dor).sum())
        out["dS_seq"], out["dS_dep"] = dS[:s_end], dS[s_end:]
        out["dq"] = scale * (dS @ K)
    return out


def depth_row_grads(q, k, v, depth_k, depth_v, dout, b, h, c, scale, G, mode, chunk_positions):
    """(d_depth_k[c], d_depth_v[c]) of depth row c of head (b, h): sums over the (at most one
    chunk of) query rows that can see it."""
    T_kv = q.shape[1] // G
    L = depth_k.shape[1] // T_kv
    tp = c // L
    t_end = min((tp // chunk_positions + 1) * chunk_positions, T_kv) if mode == MODE_CHUNK_VISIBLE else tp + 1
    dk = torch.zeros(q.shape[-1]); dv = torch.zeros(q.shape[-1])
    for r in range(tp * G, t_end * G):
        tm = row_terms(q, k, v, depth_k, depth_v, dout, b, h, r, scale, G, mode, chunk_positions)
        j = c - tm["d_lo"]
        dk += scale * tm["dS_dep"][j] * q[b, r, h].float()
        dv += tm["w_dep"][j] * dout[b, r, h].float()
    return dk, dv


def seq_key_grads(q, k, v, depth_k, depth_v, dout, b, h, j, scale, G, mode, chunk_positions):
    """(dk[j], dv[j]) of sequence key j of head (b, h); cost O(rows that see j) x O(T), so meant
    for keys near the end of a causal sequence."""
    T_q = q.shape[1]
    r_lo = 0 if mode == MODE_NONCAUSAL else j * G
    dk = torch.zeros(q.shape[-1]); dv = torch.zeros(q.shape[-1])
    for r in range(r_lo, T_q):
        tm = row_terms(q, k, v, depth_k, depth_v, dout, b, h, r, scale, G, mode, chunk_positions)
        dk += scale * tm["dS_seq"][j] * q[b, r, h].float()
        dv += tm["w_seq"][j] * dout[b, r, h].float()
    return dk, dv
