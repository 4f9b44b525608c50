"""Shared helpers of the parity tests: run the CPU oracle and the CUDA library on the same scene and compare."""
from __future__ import annotations

import numpy as np

from oracle import oracle as O


def oracle_params(params: dict) -> dict:
    p = O.default_params()
    for k in p:
        if k in params:
            p[k] = params[k]
    p["output_background_mask"] = 1
    return p


def run_oracle(scene, params: dict, grads=None, dropout=None, quadratic=False):
    o = O.Oracle()
    p = oracle_params(params)
    p["conf_grad_quadratic"] = int(quadratic)
    fwd = o.forward(scene, p, dropout=dropout)
    counts, keys = o.lists()
    out = dict(fwd=fwd, counts=counts, keys=keys, F=fwd["F"])
    if grads is not None:
        out["bwd"] = o.backward(grads)
        out["bwd_mag"] = o.backward(grads, magnitudes=True)
    return out


def row_major_order(w: int, h: int, levels: int, n_views: int) -> np.ndarray:
    """Pixel-space index of every (view, level, y, x) in row-major order: level l starts after the padded levels before
    it, and inside a level offset(x, y) = (y // B) * B w + B x + y % B with B = VETR_PIXEL_BAND (include/vetr.h)."""
    from vet_b200._lib import PIXEL_BAND as B

    per_view, base = [], 0
    for _ in range(levels):
        y, x = np.meshgrid(np.arange(h), np.arange(w), indexing="ij")
        per_view.append((base + (y // B) * (B * w) + B * x + y % B).ravel())
        base += w * ((h + B - 1) // B * B)
        w //= 2
        h //= 2
    one = np.concatenate(per_view)
    return np.concatenate([one + v * base for v in range(n_views)])


def run_gpu(rast, scene, params: dict, grads=None, dropout=None, capacity=None):
    import torch
    from vet_b200.render import scene_to_device

    dev = rast.device
    tensors = scene_to_device(scene, dev)
    dro = None if dropout is None else torch.from_numpy(np.ascontiguousarray(dropout, np.float32)).to(dev)
    fwd = rast.forward(*tensors, scene.views, params, dropout=dro, capacity=capacity, want_weight=True, want_mask=True,
                       want_depth=True)
    F, longest = rast.fragment_count()
    groups = rast._saved["groups"]
    # the library keeps its pixel space in bands of a few rows (column by column inside a band, last band padded); the
    # oracle's arrays are row-major: bring counts and the concatenated lists into row-major pixel order
    w0, h0 = scene.views[0].w, scene.views[0].h
    Ln = params.get("num_layers", 4)
    counts_parts, keys_parts = [], []
    for (b0, b1, lists, _) in groups:
        c = lists.counts.cpu().numpy()
        e = lists.ends.cpu().numpy().astype(np.int64)
        n = int(e[-1]) if e.size and params.get("render_mode", 1) != 0 else 0
        k = lists.frags[:n, 0].cpu().numpy().view(np.uint64)  # first 8 bytes of a record = key
        order = row_major_order(w0, h0, Ln, b1 - b0)
        c_rm = c[order]
        counts_parts.append(c_rm)
        if params.get("render_mode", 1) != 0:
            starts = (e - c)[order]
            total = int(c_rm.sum())
            seg_first = np.cumsum(c_rm) - c_rm
            idx = np.repeat(starts - seg_first, c_rm) + np.arange(total)
            keys_parts.append(k[idx])
    counts = np.concatenate(counts_parts)
    keys = np.concatenate(keys_parts) if keys_parts else np.zeros(0, np.uint64)
    out = dict(fwd={k: (None if v is None else [t.cpu().numpy() for t in v]) for k, v in fwd.items()}, counts=counts,
               keys=keys, F=F, longest=longest)
    if grads is not None:
        g = rast.backward_raw([torch.from_numpy(x).to(dev) for x in grads])
        torch.cuda.synchronize()
        out["bwd_raw"] = {k: v.cpu().numpy() for k, v in g.items()}
    return out


def l1_grads(color, seed=0):
    """d(L1 loss vs a seeded U(0,1) target)/d(image) for every level: sign(out - target) / numel."""
    rng = np.random.default_rng(seed)
    out = []
    for c in color:
        target = rng.uniform(0.0, 1.0, size=c.shape).astype(np.float32)
        out.append((np.sign(c - target) / c.size).astype(np.float32))
    return out


def random_grads(color, seed=0):
    rng = np.random.default_rng(seed)
    return [rng.standard_normal(c.shape).astype(np.float32) for c in color]


def assert_close(name, got, want, rtol=1e-5, floor_rel=1e-6):
    """|got - want| <= rtol * max(|got|, |want|, floor) with floor = floor_rel * max|want| (summation-order noise
    of fp32 atomics has no meaning relative to an element that cancels to ~0)."""
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    assert got.shape == want.shape, (name, got.shape, want.shape)
    scale = np.maximum(np.abs(got), np.abs(want))
    floor = floor_rel * (np.abs(want).max() if want.size else 0.0)
    bound = rtol * np.maximum(scale, floor) if floor_rel < 1 else rtol * floor
    err = np.abs(got - want)
    bad = err > bound
    if bad.any():
        i = np.unravel_index(np.argmax(err - bound), err.shape)
        raise AssertionError(f"{name}: {bad.sum()} of {bad.size} elements differ; worst at {i}: got {got[i]!r} "
                             f"want {want[i]!r} (err {err[i]:.3e}, bound {bound[i] if np.ndim(bound) else bound:.3e})")


def compare_forward(gpu, ora, exact_images=True):
    assert gpu["F"] == ora["F"], (gpu["F"], ora["F"])
    np.testing.assert_array_equal(gpu["counts"], ora["counts"])
    np.testing.assert_array_equal(gpu["keys"], ora["keys"])
    for name in ("color", "weight", "mask", "depth"):
        for l, (a, b) in enumerate(zip(gpu["fwd"][name], ora["fwd"][name])):
            if exact_images:
                np.testing.assert_array_equal(a, b, err_msg=f"{name}[{l}]")
            else:
                assert_close(f"{name}[{l}]", a, b, rtol=1e-5, floor_rel=1e-6)


def assert_sum_close(name, got, want, magnitude, rtol=1e-5, floor_rel=0.0):
    """For sums of many fp32 addends: |got - want| <= rtol * sum|addends| (+ one ulp-scale term of the value).
    `magnitude` is the oracle's sum of |addend| for the same element."""
    got = np.asarray(got, np.float64)
    want = np.asarray(want, np.float64)
    magnitude = np.asarray(magnitude, np.float64)
    assert got.shape == want.shape == magnitude.shape, (name, got.shape, want.shape, magnitude.shape)
    bound = rtol * np.maximum(magnitude, np.abs(want)) + 1e-30
    if floor_rel:
        bound = bound + floor_rel * (np.abs(want).max() if want.size else 0.0)
    err = np.abs(got - want)
    bad = ~(err <= bound)
    if bad.any():
        i = np.unravel_index(np.argmax(np.where(bad, err / bound, 0)), err.shape)
        raise AssertionError(f"{name}: {bad.sum()} of {bad.size} elements differ; worst at {i}: got {got[i]!r} "
                             f"want {want[i]!r} (err {err[i]:.3e}, bound {bound[i]:.3e}, sum|addends| {magnitude[i]:.3e})")


def compare_backward(gpu_raw, ora, channels, rtol=1e-5, floor_rel=0.0):
    """Raw gradient sums.  The oracle sums in fp64; the GPU adds the same fp32 addends with atomics in an undefined
    order, so each element is held to rtol x (sum of |addends| of that element)."""
    b, m = ora["bwd"], ora["bwd_mag"]
    import functools
    assert_sum_close = functools.partial(globals()["assert_sum_close"], floor_rel=floor_rel)
    assert_sum_close("g_texture", gpu_raw["desc"][:, :channels].T, b["texture"], m["texture"], rtol)
    assert_sum_close("g_confidence", gpu_raw["conf"], b["confidence"], m["confidence"], rtol)
    assert_sum_close("g_background", gpu_raw["background"], b["background"], m["background"], rtol)
    if "points" in gpu_raw and "points" in b:
        np.testing.assert_array_equal(gpu_raw["points"][:, 3], b["points_count"])
        assert_sum_close("g_points", gpu_raw["points"][:, :3], b["points"], m["points"], rtol)
    if "pose" in gpu_raw and "pose" in b:
        assert_sum_close("g_pose", gpu_raw["pose"], b["pose"], m["pose"], rtol)
        assert_sum_close("g_pose_count", gpu_raw["pose_count"], b["pose_count"], m["pose_count"], rtol)
    if "intrinsics" in gpu_raw and "intrinsics" in b:
        assert_sum_close("g_intrinsics", gpu_raw["intrinsics"], b["intrinsics"], m["intrinsics"], rtol)
        assert_sum_close("g_intrinsics_count", gpu_raw["intrinsics_count"], b["intrinsics_count"], m["intrinsics_count"], rtol)


def parity_report(gpu, ora, channels, rtol=1e-5) -> dict:
    """The comparisons of compare_forward / compare_backward as numbers instead of assertions (for bench.py, which
    reports parity at sizes the tests do not run)."""
    rep = dict(F=int(gpu["F"]), F_equal=bool(gpu["F"] == ora["F"]),
               counts_equal=bool(np.array_equal(gpu["counts"], ora["counts"])),
               keys_equal=bool(np.array_equal(gpu["keys"], ora["keys"])))
    rep["image_max_abs"] = max(float(np.abs(a.astype(np.float64) - b).max()) for name in ("color", "weight", "depth")
                               for a, b in zip(gpu["fwd"][name], ora["fwd"][name]))
    rep["images_bit_equal"] = all(np.array_equal(a, b) for name in ("color", "weight", "mask", "depth")
                                  for a, b in zip(gpu["fwd"][name], ora["fwd"][name]))
    if "bwd_raw" in gpu and "bwd" in ora:
        g, b, m = gpu["bwd_raw"], ora["bwd"], ora["bwd_mag"]
        pairs = [(g["desc"][:, :channels].T, "texture"), (g["conf"], "confidence"), (g["background"], "background")]
        if "points" in g and "points" in b:
            pairs.append((g["points"][:, :3], "points"))
            rep["hit_counts_equal"] = bool(np.array_equal(g["points"][:, 3], b["points_count"]))
        for key in ("pose", "intrinsics"):
            if key in g and key in b:
                pairs.append((g[key], key))
        worst = {}
        for got, key in pairs:
            want, mag = np.asarray(b[key], np.float64), np.asarray(m[key], np.float64)
            bound = rtol * np.maximum(mag, np.abs(want)) + 1e-30
            worst[key] = float((np.abs(np.asarray(got, np.float64) - want) / bound).max()) if want.size else 0.0
        rep["grad_worst_over_bound"] = max(worst.values())
        rep["grad_worst_over_bound_by_tensor"] = {k: round(v, 4) for k, v in worst.items()}
    return rep


# ---- environment map cases (shared by tests/test_envmap.py and the smoke check)

def env_scene(n_views=2, w=80, h=56, f=60.0, seed=3):
    from vet_b200 import scenes

    sc = scenes.tiny_scene(n=16, w=w, h=h, n_views=n_views, seed=seed)
    intr = scenes.pinhole_intrinsics(f, f * 1.1, w / 2 - 0.5, h / 2 + 0.25)
    sc.intrinsics = np.repeat(intr[None].astype(np.float32), sc.intrinsics.shape[0], 0)
    return sc


def env_map(rng, S=4, R=48, C=4, up_axis=0, non_subzero=False, inner_radius=20.0):
    density = rng.normal(0.0, 2.0, size=(S, R, R)).astype(np.float32)
    color = rng.normal(0.3, 1.0, size=(C, S, R, R)).astype(np.float32)
    return O.EnvMap(density, color, inner_radius=inner_radius, up_axis=up_axis, non_subzero=non_subzero)


def env_weights(rng, sc, L):
    out = []
    for l in range(L):
        w = rng.uniform(0.0, 1.0, size=(len(sc.views), 1, sc.views[0].h >> l, sc.views[0].w >> l)).astype(np.float32)
        thin = (w >= 0.1) & (w < 0.2)
        w[thin] = (w[thin] - 0.1) * 0.009  # nearly covered pixels: below the 0.001 threshold of no_envmap_at_points
        w[(w < 0.1) & ~thin] = 0.0         # fully covered pixels
        out.append(w)
    return out


def env_gpu_run(sc, env, L, weight, flags, grad_out=None, start=None):
    import torch
    from vet_b200.render import Rasterizer

    dev = torch.device("cuda:0")
    rast = Rasterizer(0)
    poses, intr = torch.from_numpy(sc.poses).to(dev), torch.from_numpy(sc.intrinsics).to(dev)
    density, color = torch.from_numpy(env.density).to(dev), torch.from_numpy(env.color).to(dev)
    kw = dict(up_axis=env.up_axis, non_subzero=env.non_subzero, flags=flags)
    w_t = [torch.from_numpy(w).to(dev) for w in weight]
    out_t = [torch.from_numpy(s).to(dev) for s in start] if start is not None else None
    out_t = rast.envmap_forward(poses, intr, sc.views, L, density, color, env.radii, w_t, out=out_t, **kw)
    res = [o.cpu().numpy() for o in out_t]
    if grad_out is None:
        return res
    g_t = [torch.from_numpy(g).to(dev) for g in grad_out]
    gd, gc = rast.envmap_backward(poses, intr, sc.views, L, density, color, env.radii, w_t, g_t, **kw)
    return res, gd.cpu().numpy(), gc.cpu().numpy()


def env_sample_tolerance(env):
    """A coordinate that differs by e texels changes a bilinear sample by at most e x the largest texel difference; the
    device's asinf / atan2f / expf differ from the host's by a few ulp of a coordinate of size resolution."""
    e = 8 * np.finfo(np.float32).eps * env.resolution
    step = max(np.abs(np.diff(env.color, axis=-1)).max(), np.abs(np.diff(env.color, axis=-2)).max())
    return float(e * step * 2 + 1e-5)


def env_grad_tolerance(mag, env):
    """Bound of |device sum - host sum| per texel.  mag: the summed magnitudes of a texel's addends.  1e-5 of them for the
    order of the fp32 sums; and a sample coordinate that differs by e texels (asinf / atan2f differ by a few ulp between
    device and host) moves the fraction e of an addend between neighbouring texels, so a texel can gain or lose e times
    what its 3 x 3 neighbourhood receives."""
    import torch
    import torch.nn.functional as F

    e = 8 * np.finfo(np.float32).eps * env.resolution
    m = torch.from_numpy(mag).reshape(-1, 1, env.resolution, env.resolution)
    near = (F.avg_pool2d(m, 3, stride=1, padding=1, count_include_pad=True) * 9).reshape(mag.shape).numpy()
    return 1e-5 * mag + 4 * e * near + 1e-6
