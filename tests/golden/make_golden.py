"""Writes tests/golden/oracle_tiny.npz: the CPU oracle's lists, images, raw gradient sums (all four render modes),
error-grid sums and environment-map samples on tiny seeded scenes; for the environment map also the result of
libtorch's own operators (grid_sample, sigmoid, autograd) on the same inputs.

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
# texture environment map: the restatement's output, and forward_mps5 evaluated with libtorch's operators
import torch  # noqa: E402
import torch.nn.functional as F  # noqa: E402

sc = scenes.tiny_scene(n=4, w=40, h=28, n_views=2, seed=79, crop=True)
rng = np.random.default_rng(6)
S, R, C, L = 3, 16, 4, 2
env = O.EnvMap(rng.normal(0, 2, size=(S, R, R)).astype(np.float32), rng.normal(0.3, 1, size=(C, S, R, R)).astype(np.float32),
               inner_radius=20.0, radius_factor=5.0, up_axis=1)
weight = [rng.uniform(0, 1, size=(2, 1, 28 >> l, 40 >> l)).astype(np.float32) for l in range(L)]
res = O.envmap_forward(sc, sc.views, L, env, weight)
gout = [rng.standard_normal(r.shape).astype(np.float32) for r in res]
gd, gc, md, mc = O.envmap_backward(sc, sc.views, L, env, weight, gout)
dens_t = torch.from_numpy(env.density)[None, None].clone().requires_grad_(True)
col_t = torch.from_numpy(env.color)[None].clone().requires_grad_(True)
loss = 0
for l in range(L):
    per_view = []
    for b, v in enumerate(sc.views):
        uvz, hit = O.envmap_uvz(sc, v, l, env)
        grid = torch.from_numpy(uvz).reshape(1, -1, 1, 1, 3)
        kw = dict(mode="bilinear", padding_mode="zeros", align_corners=True)
        alpha_all = torch.sigmoid(F.grid_sample(dens_t, grid, **kw).reshape(S, -1))
        col_all = F.grid_sample(col_t, grid, **kw).reshape(C, S, -1).permute(1, 0, 2)
        T = torch.from_numpy(weight[l][b].reshape(-1))
        final = torch.zeros(C, T.numel())
        for s_ in range(S):
            alpha = (torch.ones_like(alpha_all[s_]) if s_ == S - 1 else alpha_all[s_]) * torch.from_numpy(hit[s_])
            final = T.unsqueeze(0) * alpha.unsqueeze(0) * col_all[s_] + final
            T = (1 - alpha) * T
        img = final.reshape(C, v.h >> l, v.w >> l)
        loss = loss + (img * torch.from_numpy(gout[l][b])).sum()
        per_view.append(img.detach().numpy())
    out[f"env_torch_l{l}"] = np.stack(per_view)
loss.backward()
out["env_density"], out["env_color"], out["env_radii"] = env.density, env.color, env.radii
for l in range(L):
    out[f"env_weight_l{l}"], out[f"env_out_l{l}"], out[f"env_gout_l{l}"] = weight[l], res[l], gout[l]
out["env_g_density"], out["env_g_color"], out["env_mag_density"], out["env_mag_color"] = gd, gc, md, mc
out["env_torch_g_density"], out["env_torch_g_color"] = dens_t.grad[0, 0].numpy(), col_t.grad[0].numpy()
np.savez_compressed(os.path.join(os.path.dirname(os.path.abspath(__file__)), "oracle_tiny.npz"), **out)
print("written", {k: v.shape for k, v in out.items() if k.startswith("keys")}, "grid hits", int(count.sum()))
