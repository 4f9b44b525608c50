"""Writes tests/golden/oracle_tiny.npz: the CPU oracle's lists, images, raw gradient sums (all four render modes) and
error-grid sums on tiny seeded scenes.

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
for mode in (0, 1, 2, 3):
    sc = scenes.tiny_scene(n=400, w=24, h=16, n_views=2, seed=77, crop=True)
    o = O.Oracle()
    r = o.forward(sc, O.default_params(render_mode=mode, num_layers=3))
    if mode != 0:  # mode 0 keeps no lists
        counts, keys = o.lists()
        out[f"counts_m{mode}"], out[f"keys_m{mode}"] = counts, keys
    rng = np.random.default_rng(123 + mode)
    grads = [rng.standard_normal(c.shape).astype(np.float32) for c in r["color"]]
    for l in range(3):
        out[f"color_m{mode}_l{l}"] = r["color"][l]
        out[f"weight_m{mode}_l{l}"] = r["weight"][l]
        out[f"depth_m{mode}_l{l}"] = r["depth"][l]
        out[f"grad_m{mode}_l{l}"] = grads[l]
    b = o.backward(grads)
    for k in ("texture", "confidence", "background", "points", "pose", "intrinsics"):
        out[f"bwd_m{mode}_{k}"] = b[k]
    m = o.backward(grads, magnitudes=True)  # the same sums over |addends|: the scale the GPU test's tolerance refers to
    for k in ("texture", "confidence", "background", "points", "pose", "intrinsics"):
        out[f"mag_m{mode}_{k}"] = m[k]

# error-grid rasterisation over the same cameras
sc = scenes.tiny_scene(n=4, w=160, h=128, n_views=2, seed=78, crop=True)
rng = np.random.default_rng(5)
bb_min = rng.uniform(-1.5, 1.5, size=(200, 3)).astype(np.float32)
bb_len = rng.uniform(0.05, 0.6, size=(200, 3)).astype(np.float32)
loss = rng.standard_normal((3, 128, 160)).astype(np.float32)
value, count = np.zeros(200, np.float64), np.zeros(200, np.int64)
for v in sc.views:
    gv, gc = O.grid_loss(sc, v, bb_min, bb_len, loss)
    value += gv
    count += gc
out["grid_bb_min"], out["grid_bb_len"], out["grid_loss_img"] = bb_min, bb_len, loss
out["grid_value"], out["grid_count"] = value, count
np.savez_compressed(os.path.join(os.path.dirname(os.path.abspath(__file__)), "oracle_tiny.npz"), **out)
print("written", {k: v.shape for k, v in out.items() if k.startswith("keys")}, "grid hits", int(count.sum()))
