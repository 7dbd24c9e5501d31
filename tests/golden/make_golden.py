"""Generate the golden fixtures in this folder from the REFERENCE's own torch oracles.

Run once in a container that has the reference checkout (it cannot travel to the GPU
box, the fixtures can):

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py /path/to/reference

It imports ``naive_mixture_of_depth_causal_ref`` (moda_v14.py:1900),
``naive_mixture_of_depth_causal_chunk_visible_ref`` (moda_v16.py:2487) and
``naive_depth_causal_ref`` (fda_v12.py:1143) from ``<reference>/libs/moda_triton``, runs
them in fp32 on seeded CPU inputs, differentiates ``sum(o * dout)`` by autograd, and
writes one ``.npz`` per case holding inputs, outputs and gradients.  The inputs come
from ``oracle.moda_oracle.make_inputs`` so tests can also regenerate them by seed.
"""
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle.moda_oracle import (  # noqa: E402
    MODE_CAUSAL, MODE_CHUNK_VISIBLE, MODE_DEPTH_ONLY, MODE_NONCAUSAL, make_inputs,
)

# name, seed, mode, B, T_kv, H, D, L, G, chunk_positions, scale, store_grads, store_inputs
CASES = [
    ("causal_g2_l3", 11, MODE_CAUSAL, 1, 48, 2, 64, 3, 2, 0, None, True, True),
    ("causal_l0", 12, MODE_CAUSAL, 2, 31, 1, 64, 0, 1, 0, 0.5, True, True),
    ("causal_d128_g4", 13, MODE_CAUSAL, 1, 24, 1, 128, 2, 4, 0, None, True, True),
    ("noncausal_l2", 14, MODE_NONCAUSAL, 2, 37, 1, 64, 2, 1, 0, None, True, True),
    ("chunk_g4_l2", 15, MODE_CHUNK_VISIBLE, 1, 40, 2, 64, 2, 4, 16, None, True, True),
    ("chunk_g1_l1", 16, MODE_CHUNK_VISIBLE, 1, 150, 1, 64, 1, 1, 64, 0.2, True, True),
    ("fda_g2_l5", 17, MODE_DEPTH_ONLY, 1, 33, 2, 64, 5, 2, 0, None, True, True),
    # benchmark config 1: B=1,T=256,H=4,D=64,L=4,G=1, seed 0 (outputs only; inputs by seed)
    ("config1", 0, MODE_CAUSAL, 1, 256, 4, 64, 4, 1, 0, None, False, False),
]


def main(ref_root: str) -> None:
    sys.path.insert(0, os.path.join(ref_root, "libs", "moda_triton"))
    from fla.ops.moda import (
        naive_mixture_of_depth_causal_chunk_visible_ref,
        naive_mixture_of_depth_causal_ref,
    )
    from fla.ops.moda.fda_v12 import naive_depth_causal_ref

    for (name, seed, mode, B, T, H, D, L, G, cp, scale, store_grads, store_inputs) in CASES:
        q, k, v, kd, vd, dout = make_inputs(
            seed, B, T, H, D, L, G, with_seq=(mode != MODE_DEPTH_ONLY))
        leaves = {n: (None if x is None else x.clone().requires_grad_(True))
                  for n, x in (("q", q), ("k", k), ("v", v), ("kd", kd), ("vd", vd))}
        if mode == MODE_DEPTH_ONLY:
            o, lse = naive_depth_causal_ref(leaves["q"], leaves["kd"], leaves["vd"],
                                            scale=scale, moda_group_num=G)
        elif mode == MODE_CHUNK_VISIBLE:
            o, lse = naive_mixture_of_depth_causal_chunk_visible_ref(
                leaves["q"], leaves["k"], leaves["v"], kd=leaves["kd"], vd=leaves["vd"],
                scale=scale, moda_group_num=G, chunk_size=cp)
        else:
            o, lse = naive_mixture_of_depth_causal_ref(
                leaves["q"], leaves["k"], leaves["v"], kd=leaves["kd"], vd=leaves["vd"],
                scale=scale, moda_group_num=G, is_causal=(mode == MODE_CAUSAL))
        rec = {
            "meta": np.array([seed, mode, B, T, H, D, L, G, cp], dtype=np.int64),
            "scale": np.array([-1.0 if scale is None else scale], dtype=np.float64),
            "o": o.detach().numpy(), "lse": lse.detach().numpy(),
            "input_checksum": np.array(
                [float(x.double().sum()) for x in (q, k, v, kd, vd, dout) if x is not None]),
        }
        if store_grads:
            (o * dout).sum().backward()
            for n, x in leaves.items():
                if x is not None:
                    rec["d" + n] = x.grad.numpy()
        if store_inputs:
            for n, x in (("q", q), ("k", k), ("v", v), ("kd", kd), ("vd", vd), ("dout", dout)):
                if x is not None:
                    rec["in_" + n] = x.numpy()
        path = os.path.join(HERE, name + ".npz")
        np.savez_compressed(path, **rec)
        print(name, "mean|o|=%.8f mean(lse)=%.8f" % (o.abs().mean().item(), lse.mean().item()),
              os.path.getsize(path), "bytes")


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: make_golden.py <path of a checkout of hustvl/MoDA>")
    main(sys.argv[1])
