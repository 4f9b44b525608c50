"""Writes tests/golden/oracle_tiny.npz: the CPU oracle's lists, images and raw gradient sums on a tiny seeded scene.

The reference has no golden vectors for the rasterizer and cannot be executed (its CUDA sources need the absent saiga
library), so this fixture freezes the oracle's own output; what pins the oracle to the reference is listed in
tests/test_oracle.py and tests/test_oracle_ref_blend.py.   Run:  python tests/golden/make_golden.py
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
from oracle import oracle as O  # noqa: E402
from vet_b200 import scenes  # noqa: E402

out = {}
for mode in (1, 3):
    sc = scenes.tiny_scene(n=400, w=24, h=16, n_views=2, seed=77, crop=True)
    o = O.Oracle()
    r = o.forward(sc, O.default_params(render_mode=mode, num_layers=3))
    counts, keys = o.lists()
    out[f"counts_m{mode}"], out[f"keys_m{mode}"] = counts, keys
    rng = np.random.default_rng(123 + mode)
    grads = [rng.standard_normal(c.shape).astype(np.float32) for c in r["color"]]
    for l in range(3):
        out[f"color_m{mode}_l{l}"] = r["color"][l]
        out[f"grad_m{mode}_l{l}"] = grads[l]
    b = o.backward(grads)
    for k in ("texture", "confidence", "background", "points", "pose", "intrinsics"):
        out[f"bwd_m{mode}_{k}"] = b[k]
np.savez_compressed(os.path.join(os.path.dirname(os.path.abspath(__file__)), "oracle_tiny.npz"), **out)
print("written", {k: v.shape for k, v in out.items() if k.startswith("keys")})
