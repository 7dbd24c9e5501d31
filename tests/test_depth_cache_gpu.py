"""GPU: the in-place depth-KV cache (``DepthKVCache``, ``moda_b200_depth_append``, the strided
depth layout ``depth_rows_per_pos`` and gradient accumulation) against the scheme it replaces -
rebuilding a packed cache with ``torch.stack`` before every layer, as the reference's caller does
(vision_tasks/deit/models.py:361-390) - and against the CPU oracle differentiated through the
whole stack of layers."""
import pytest
import torch

from oracle import moda_oracle as mo
from tests.helpers import TOL_LSE_MAX_ABS, TOL_O_MAX_ABS, check_grad, max_abs

pytestmark = pytest.mark.gpu


def _layers(seed, n_layers, B, T, H, D, G, dtype=torch.bfloat16):
    gen = torch.Generator().manual_seed(seed)
    mk = lambda rows: torch.randn(B, rows, H, D, generator=gen).to(dtype)  # noqa: E731
    return [(mk(T * G), mk(T), mk(T), mk(T * G)) for _ in range(n_layers)]     # q, k, v, weight of the loss


def _packed(kv_list):
    """The reference caller's cache: [B, T*L, H, D] from the list of earlier layers' (k, v)."""
    if not kv_list:
        return None, None
    ks = torch.stack([kv[0] for kv in kv_list], dim=2)
    vs = torch.stack([kv[1] for kv in kv_list], dim=2)
    B, T, L, H, D = ks.shape
    return ks.reshape(B, T * L, H, D).contiguous(), vs.reshape(B, T * L, H, D).contiguous()


def _call(M, mode, q, k, v, ck, cv, G):
    if mode == mo.MODE_CHUNK_VISIBLE:
        return M.parallel_moda_chunk_visible(q, k, v, cached_k=ck, cached_v=cv, moda_group_num=G, need_lse=True, warn_shape=False)
    return M.parallel_moda(q, k, v, cached_k=ck, cached_v=cv, moda_group_num=G, is_causal=(mode == mo.MODE_CAUSAL),
                           need_lse=True, warn_shape=False)


@pytest.mark.parametrize("mode,B,T,H,D,G,n_layers", [
    (mo.MODE_NONCAUSAL, 2, 197, 3, 64, 1, 4),       # DeiT-like: own-position depth through the bandwidth kernels
    (mo.MODE_CAUSAL, 1, 300, 2, 128, 4, 5),         # tcgen05 kernels, 5-D depth maps (L = 1, 2, 4) and mma.sync (L = 3)
    (mo.MODE_CHUNK_VISIBLE, 2, 160, 2, 64, 2, 3),
    (mo.MODE_CAUSAL, 1, 100, 2, 128, 1, 3),
])
def test_layer_stack_matches_rebuilt_cache_and_oracle(built_library, mode, B, T, H, D, G, n_layers):
    import moda_b200 as M
    from moda_b200 import _cabi
    dev = torch.device("cuda", 0)
    data = _layers(17 + T, n_layers, B, T, H, D, G)

    # (a) in-place cache
    leaves_a = [[x.to(dev).requires_grad_(True) for x in lay[:3]] for lay in data]
    cache = M.DepthKVCache(B, T, n_layers - 1, H, D, torch.bfloat16, dev)
    outs_a, loss = [], 0.
    for i, (q, k, v) in enumerate(leaves_a):
        o, lse = cache.attend(q, k, v, moda_group_num=G, is_causal=(mode != mo.MODE_NONCAUSAL),
                              chunk_visible=(mode == mo.MODE_CHUNK_VISIBLE), need_lse=True)
        outs_a.append((o, lse))
        loss = loss + (o.float() * data[i][3].to(dev).float()).sum()
        if i + 1 < n_layers:
            cache.append(k, v)
    loss.backward()
    assert _cabi.device_status() == 0
    # the cache holds exactly what stacking would have produced
    want_k, _ = _packed([(k.detach(), v.detach()) for _, k, v in leaves_a[:-1]])
    got_k = cache.k.view(B, T, n_layers - 1, H, D).reshape(B, T * (n_layers - 1), H, D)
    assert torch.equal(got_k, want_k)

    # (b) packed cache rebuilt before every layer, through the ordinary operators
    leaves_b = [[x.to(dev).requires_grad_(True) for x in lay[:3]] for lay in data]
    outs_b, loss_b, kv = [], 0., []
    for i, (q, k, v) in enumerate(leaves_b):
        ck, cv = _packed(kv)
        o, lse = _call(M, mode, q, k, v, ck, cv, G)
        outs_b.append((o, lse))
        loss_b = loss_b + (o.float() * data[i][3].to(dev).float()).sum()
        kv.append((k, v))
    loss_b.backward()
    for i, ((oa, la), (ob, lb)) in enumerate(zip(outs_a, outs_b)):
        # Layer i reads i cached layers.  Where both flows run the same kernels (the tcgen05 kernels
        # read an in-place cache only when the layer count divides their 32-row boxes; the other
        # counts fall to the mma.sync kernels) the arithmetic is the same and so are the bits.
        same_kernels = D == 64 and G == 1 or i == 0 or 32 % i == 0 or i == n_layers - 1
        if same_kernels:
            assert torch.equal(oa, ob) and torch.equal(la, lb), f"layer {i}"
            assert torch.equal(leaves_a[i][0].grad, leaves_b[i][0].grad), f"dq of layer {i}"
        else:
            assert max_abs(oa.float(), ob.float()) <= 1e-2 and max_abs(la, lb) <= 1e-4, f"layer {i}"
    for la_, lb_ in zip(leaves_a, leaves_b):
        for xa, xb in zip(la_[1:], lb_[1:]):              # dk, dv: sums of 16-bit terms in a different order
            check_grad("k/v grad vs rebuilt cache", xa.grad.float().cpu(), xb.grad.float().cpu())

    # (c) the CPU oracle differentiated through the whole stack (fp32)
    leaves_c = [[x.float().clone().requires_grad_(True) for x in lay[:3]] for lay in data]
    loss_c, kv = 0., []
    for i, (q, k, v) in enumerate(leaves_c):
        ck, cv = _packed(kv)
        o, lse = mo.moda_attention_ref(q, k, v, ck, cv, None, G, mode, max(64 // G, 1))
        assert max_abs(outs_a[i][0].float().cpu(), o.detach()) <= TOL_O_MAX_ABS
        assert max_abs(outs_a[i][1].cpu(), lse.detach()) <= TOL_LSE_MAX_ABS
        loss_c = loss_c + (o * data[i][3].float()).sum()
        kv.append((k, v))
    loss_c.backward()
    for i, (la_, lc_) in enumerate(zip(leaves_a, leaves_c)):
        for name, xa, xc in zip(("dq", "dk", "dv"), la_, lc_):
            check_grad(f"layer {i} {name}", xa.grad.float().cpu(), xc.grad)


def test_strided_cache_with_forced_tcgen05_path(built_library):
    """Forced tcgen05: a layer count that divides 32 runs on 5-D tensor maps; one that does not is
    refused (the default path serves it with the mma.sync kernels)."""
    import moda_b200 as M
    dev = torch.device("cuda", 0)
    B, T, H, D, G = 1, 200, 2, 128, 2
    data = _layers(5, 4, B, T, H, D, G)
    cache = M.DepthKVCache(B, T, 5, H, D, torch.bfloat16, dev)
    old = M.set_kernel_path(M.PATH_TCGEN05)
    try:
        for i, lay in enumerate(data):
            q, k, v = [x.to(dev).requires_grad_(True) for x in lay[:3]]
            if cache.L == 3:
                with pytest.raises(M.ModaLibraryError, match="does not support"):
                    cache.attend(q, k, v, moda_group_num=G)
                break
            o, lse = cache.attend(q, k, v, moda_group_num=G, need_lse=True)
            ck, cv = _packed([(cache._slot(cache.k, j), cache._slot(cache.v, j)) for j in range(cache.L)])
            o2, lse2 = M.parallel_moda_fwd(q, k, v, cached_k=ck, cached_v=cv, moda_group_num=G)
            assert torch.equal(o, o2) and torch.equal(lse, lse2)
            o.sum().backward()
            cache.append(k.detach(), v.detach())
    finally:
        M.set_kernel_path(old)
