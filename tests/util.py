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
