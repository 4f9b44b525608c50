"""The CPU oracle against hand-computed cases, an independent fp64 autograd restatement, invariants and fixtures.

The reference ships no test, golden vector or fixture for this path, so these are what pins the oracle:
  * micro cases whose answer is computed by hand in the test;
  * the descriptor / confidence / background gradients are exact derivatives of the blend: they are compared with
    torch autograd over an fp64 re-implementation of the blend written independently in this file;
  * the literal O(n^2) confidence-gradient loop of the reference against the O(n) suffix-sum form;
  * structural invariants of the lists;
  * committed fixtures (tests/golden) that freeze the oracle's own results.
"""
import os

import numpy as np
import pytest
import torch

from oracle import oracle as O
from tests import util
from vet_b200 import scenes

GOLDEN = os.path.join(os.path.dirname(__file__), "golden", "oracle_tiny.npz")


def one_view_scene(points, radius=1.0, conf=0.5, w=8, h=8, f=8.0, channels=4):
    """Camera at the origin looking down +z with identity pose; pixel = f * x/z + w/2."""
    n = len(points)
    position = np.zeros((n, 4), np.float32)
    position[:, :3] = np.asarray(points, np.float32)
    position[:, 3] = radius
    texture = np.arange(1, channels * n + 1, dtype=np.float32).reshape(channels, n) / 10.0
    confidence = np.full(n, conf, np.float32) if np.isscalar(conf) else np.asarray(conf, np.float32)
    poses = np.array([[0, 0, 0, 1, 0, 0, 0, 0]], np.float64)
    intr = scenes.pinhole_intrinsics(f, f, w / 2, h / 2)[None]
    return scenes.Scene(position, np.arange(n, dtype=np.int32), texture, confidence, np.full(channels, -1.0, np.float32),
                        poses, intr, [scenes.View(w, h)])


def test_single_point_blend_by_hand():
    sc = one_view_scene([(0.0, 0.0, 2.0)], conf=0.25)
    o = O.Oracle()
    r = o.forward(sc, O.default_params(num_layers=1, drop_out_points_by_radius=0, output_background_mask=1))
    assert r["F"] == 1
    c = r["color"][0][0, :, 4, 4]
    want = np.float32(0.25) * sc.texture[:, 0] + np.float32(0.75) * np.float32(-1.0)
    np.testing.assert_allclose(c, want, rtol=1e-6)
    assert r["weight"][0][0, 0, 4, 4] == np.float32(0.75)
    assert r["depth"][0][0, 0, 4, 4] == np.float32(2.0)
    assert r["depth"][0][0, 0, 0, 0] == np.float32(100000.0)
    np.testing.assert_array_equal(r["color"][0][0, :, 0, 0], np.full(4, -1.0, np.float32))  # empty pixel = background
    assert (r["mask"][0] == 1).all()  # mask is 1 unless the transmittance is exactly 0


def test_depth_order_and_tie_break_by_index():
    # three points on the optical axis: index 0 far, 1 and 2 at the same depth (tie -> lower index first)
    sc = one_view_scene([(0, 0, 3.0), (0, 0, 2.0), (0, 0, 2.0)], conf=[0.5, 0.25, 0.75])
    o = O.Oracle()
    r = o.forward(sc, O.default_params(num_layers=1, drop_out_points_by_radius=0))
    counts, keys = o.lists()
    assert counts.sum() == 3 and counts[4 * 8 + 4] == 3
    ids = (keys & np.uint64(0xFFFFFFFF)).astype(int).tolist()
    assert ids == [1, 2, 0]
    depths = (keys >> np.uint64(32)).astype(np.uint32).view(np.float32)
    assert depths.tolist() == [2.0, 2.0, 3.0]
    # front to back by hand
    T, c = 1.0, np.zeros(4)
    for i in ids:
        a = float(sc.confidence[i])
        c = c + T * a * sc.texture[:, i].astype(np.float64)
        T *= 1 - a
    c = c + T * -1.0
    np.testing.assert_allclose(r["color"][0][0, :, 4, 4], c, rtol=1e-6)


def test_rounding_levels_and_radius_dropout():
    # x/z*f + w/2 = 4.5 -> half to even = 4 ; 5.5 -> 6   (RenderForward.cu:888 uses __float2int_rn)
    sc = one_view_scene([(0.125, 0.0, 2.0), (0.375, 0.0, 2.0)], w=16, h=16, f=8.0)
    # pixel x = 8*x/z + 8 = 8.5 and 9.5
    o = O.Oracle()
    o.forward(sc, O.default_params(num_layers=2, drop_out_points_by_radius=0))
    counts, _ = o.lists()
    lvl0 = counts[:256].reshape(16, 16)
    assert lvl0[8, 8] == 1 and lvl0[8, 10] == 1 and lvl0.sum() == 2
    lvl1 = counts[256:256 + 64].reshape(8, 8)  # ip * 0.5 = (4.25, 4) and (4.75, 4) -> 4 and 5
    assert lvl1[4, 4] == 1 and lvl1[4, 5] == 1
    # radius in pixels = fx * r / z = 8 * r / 2; threshold 0.6 -> r = 0.2 gives 0.8 at level 0, 0.4 at level 1
    sc.position[:, 3] = 0.2
    o.forward(sc, O.default_params(num_layers=2, drop_out_points_by_radius=1))
    counts, _ = o.lists()
    assert counts[:256].sum() == 2 and counts[256:].sum() == 0
    # behind the camera and z == 0 are skipped
    sc2 = one_view_scene([(0, 0, -1.0), (0, 0, 0.0), (0, 0, 1.0)])
    o.forward(sc2, O.default_params(num_layers=1, drop_out_points_by_radius=0))
    assert o.lists()[0].sum() == 1


def test_bilinear_corners_by_hand():
    # ip = (4.25, 4.5): corners (4,4) (5,4) (4,5) (5,5) with weights (.75*.5, .25*.5, .75*.5, .25*.5)
    sc = one_view_scene([(0.0625 * 0.5, 0.125 * 0.5, 1.0)], conf=0.8, w=8, h=8, f=8.0)
    o = O.Oracle()
    r = o.forward(sc, O.default_params(render_mode=3, num_layers=1, drop_out_points_by_radius=0))
    assert r["F"] == 4
    T = r["weight"][0][0, 0]
    np.testing.assert_allclose([T[4, 4], T[4, 5], T[5, 4], T[5, 5]],
                               [1 - 0.8 * 0.375, 1 - 0.8 * 0.125, 1 - 0.8 * 0.375, 1 - 0.8 * 0.125], rtol=1e-6)


def _torch_blend_from_lists(scene, params, counts, keys, grads, views):
    """Independent fp64 restatement of the blend (mode 1) on the oracle's lists; returns autograd gradients."""
    tex = torch.tensor(scene.texture, dtype=torch.float64, requires_grad=True)
    conf = torch.tensor(scene.confidence, dtype=torch.float64, requires_grad=True)
    bg = torch.tensor(scene.background, dtype=torch.float64, requires_grad=True)
    starts = np.concatenate([[0], np.cumsum(counts)])
    L = params["num_layers"]
    sizes = O.level_sizes(views[0].w, views[0].h, L)
    P = sum(w * h for w, h in sizes)
    loss = torch.zeros((), dtype=torch.float64)
    ids_all = (keys & np.uint64(0xFFFFFFFF)).astype(np.int64)
    for b in range(len(views)):
        base = 0
        for l, (w, h) in enumerate(sizes):
            G = torch.tensor(grads[l][b], dtype=torch.float64)
            for y in range(h):
                for x in range(w):
                    g = b * P + base + y * w + x
                    ids = ids_all[starts[g]:starts[g + 1]]
                    T = torch.ones((), dtype=torch.float64)
                    c = torch.zeros(tex.shape[0], dtype=torch.float64)
                    for i in ids:
                        k = int(scene.index[i])
                        c = c + T * conf[k] * tex[:, k]
                        T = T * (1 - conf[k])
                    if not params["use_environment_map"]:
                        c = c + T * bg
                    loss = loss + (c * G[:, y, x]).sum()
            base += w * h
    loss.backward()
    zero = lambda t: np.zeros(tuple(t.shape)) if t.grad is None else t.grad.numpy()
    return zero(tex), zero(conf), zero(bg)


@pytest.mark.parametrize("env", [0, 1])
def test_exact_gradients_match_autograd(env):
    sc = scenes.tiny_scene(n=300, w=12, h=10, n_views=2, seed=3)
    params = O.default_params(num_layers=2, use_environment_map=env, background_alpha_to_point0=0,
                              drop_out_points_by_radius=0)
    o = O.Oracle()
    fwd = o.forward(sc, params)
    grads = util.random_grads(fwd["color"], seed=2)
    counts, keys = o.lists()
    b = o.backward(grads)
    mag = o.backward(grads, magnitudes=True)
    gt, gc, gb = _torch_blend_from_lists(sc, params, counts, keys, grads, sc.views)
    # the oracle evaluates each addend in fp32: allow 1e-5 of the element's sum of |addends|
    util.assert_sum_close("texture", b["texture"], gt, mag["texture"])
    util.assert_sum_close("confidence", b["confidence"], gc, mag["confidence"])
    util.assert_sum_close("background", b["background"], gb, mag["background"])


@pytest.mark.parametrize("mode", [1, 3])
def test_quadratic_reference_loop_equals_suffix_form(mode):
    sc = scenes.tiny_scene(n=3000, seed=5)
    outs = []
    for quad in (0, 1):
        o = O.Oracle()
        fwd = o.forward(sc, O.default_params(render_mode=mode, conf_grad_quadratic=quad))
        grads = util.random_grads(fwd["color"], seed=4)
        outs.append((o.backward(grads), o.backward(grads, magnitudes=True)))
    (a, mag), (b, _) = outs
    for k in a:
        util.assert_sum_close(k, a[k], b[k], mag[k])


def test_background_alpha_quirk_goes_to_descriptor_zero():
    """RenderBackward.cu:1130,1157: the background entry's alpha gradient lands on descriptor 0's confidence."""
    sc = scenes.tiny_scene(n=500, seed=6)
    res = {}
    for flag in (0, 1):
        o = O.Oracle()
        fwd = o.forward(sc, O.default_params(background_alpha_to_point0=flag))
        res[flag] = o.backward(util.random_grads(fwd["color"], seed=1))
    d = res[1]["confidence"] - res[0]["confidence"]
    assert d[0] != 0 and np.abs(d[1:]).max() == 0
    for k in ("texture", "background", "points", "pose"):
        np.testing.assert_array_equal(res[0][k], res[1][k])


@pytest.mark.parametrize("mode", [1, 3])
def test_list_invariants(mode):
    sc = scenes.tiny_scene(n=5000, w=48, h=32, n_views=3, seed=9)
    o = O.Oracle()
    r = o.forward(sc, O.default_params(render_mode=mode))
    counts, keys = o.lists()
    assert counts.sum() == r["F"] == keys.size
    starts = np.concatenate([[0], np.cumsum(counts)])
    for g in np.nonzero(counts > 1)[0][:2000]:
        seg = keys[starts[g]:starts[g + 1]]
        assert (seg[1:] > seg[:-1]).all()  # strictly ascending (depth bits, point index)
    for wgt in r["weight"]:
        assert (wgt >= 0).all() and (wgt <= 1).all()
    ids = (keys & np.uint64(0xFFFFFFFF)).astype(np.int64)
    assert ids.min() >= 0 and ids.max() < sc.n


def test_apply_tangent_is_the_se3_exponential():
    rng = np.random.default_rng(0)
    poses = scenes.orbit_poses(rng, 5, 3.0)
    tangent = rng.normal(scale=0.1, size=(5, 6))
    p, t = poses.copy(), tangent.copy()
    O.apply_tangent(t, p)
    assert np.abs(t).max() == 0
    np.testing.assert_allclose(np.linalg.norm(p[:, :4], axis=1), 1.0, atol=1e-12)

    def mat(q, tr):
        x, y, z, w = q
        R = np.array([[1 - 2 * (y * y + z * z), 2 * (x * y - z * w), 2 * (x * z + y * w)],
                      [2 * (x * y + z * w), 1 - 2 * (x * x + z * z), 2 * (y * z - x * w)],
                      [2 * (x * z - y * w), 2 * (y * z + x * w), 1 - 2 * (x * x + y * y)]])
        M = np.eye(4)
        M[:3, :3], M[:3, 3] = R, tr
        return M

    from scipy.linalg import expm
    for i in range(5):
        u, w = tangent[i, :3], tangent[i, 3:]
        xi = np.zeros((4, 4))
        xi[:3, :3] = np.array([[0, -w[2], w[1]], [w[2], 0, -w[0]], [-w[1], w[0], 0]])
        xi[:3, 3] = u
        want = expm(xi) @ mat(poses[i, :4], poses[i, 4:7])
        np.testing.assert_allclose(mat(p[i, :4], p[i, 4:7]), want, atol=1e-10)


def test_golden_fixture():
    """Freezes the oracle: counts, keys, images and gradient sums of a tiny scene in all four modes, and the error-grid
    sums (tests/golden/make_golden.py)."""
    data = np.load(GOLDEN)
    for mode in (0, 1, 2, 3):
        sc = scenes.tiny_scene(n=400, w=24, h=16, n_views=2, seed=77, crop=True)
        o = O.Oracle()
        r = o.forward(sc, O.default_params(render_mode=mode, num_layers=3))
        if mode != 0:
            counts, keys = o.lists()
            np.testing.assert_array_equal(counts, data[f"counts_m{mode}"])
            np.testing.assert_array_equal(keys, data[f"keys_m{mode}"])
        for l in range(3):
            np.testing.assert_array_equal(r["color"][l], data[f"color_m{mode}_l{l}"])
            np.testing.assert_array_equal(r["weight"][l], data[f"weight_m{mode}_l{l}"])
            np.testing.assert_array_equal(r["depth"][l], data[f"depth_m{mode}_l{l}"])
        g = [data[f"grad_m{mode}_l{l}"] for l in range(3)]
        b = o.backward(g)
        for k in ("texture", "confidence", "background", "points", "pose", "intrinsics"):
            np.testing.assert_allclose(b[k], data[f"bwd_m{mode}_{k}"], rtol=1e-12, atol=1e-14)
    sc = scenes.tiny_scene(n=4, w=160, h=128, n_views=2, seed=78, crop=True)
    value, count = np.zeros(200, np.float64), np.zeros(200, np.int64)
    for v in sc.views:
        gv, gc = O.grid_loss(sc, v, data["grid_bb_min"], data["grid_bb_len"], data["grid_loss_img"])
        value += gv
        count += gc
    np.testing.assert_array_equal(count, data["grid_count"])
    np.testing.assert_allclose(value, data["grid_value"], rtol=1e-12)


def _projection_f64(p, xi, q, t, K, dist, crop, rot, centre, scale):
    """The projection (PointRendererHelper.h:184-218 + crop transform, crop rotation and level scale) in float64 torch, as
    a function of the point, a left pose perturbation xi = (translation, rotation) at zero, K and the distortion."""
    x, y, z, w = q
    R = torch.stack([torch.stack([1 - 2 * (y * y + z * z), 2 * (x * y - z * w), 2 * (x * z + y * w)]),
                     torch.stack([2 * (x * y + z * w), 1 - 2 * (x * x + z * z), 2 * (y * z - x * w)]),
                     torch.stack([2 * (x * z - y * w), 2 * (y * z + x * w), 1 - 2 * (x * x + y * y)])])
    v = R @ p + t
    v = v + xi[:3] + torch.linalg.cross(xi[3:], v)       # exp(xi) V p to first order: d/dxi = [I | -skew(v)]
    n = v[:2] / v[2]
    r2 = (n * n).sum()
    k1, k2, k3, k4, k5, k6, p1, p2 = dist
    radial = (1 + k1 * r2 + k2 * r2 ** 2 + k3 * r2 ** 3) / (1 + k4 * r2 + k5 * r2 ** 2 + k6 * r2 ** 3)
    dx = n[0] * radial + 2 * p1 * n[0] * n[1] + p2 * (r2 + 2 * n[0] ** 2)
    dy = n[1] * radial + 2 * p2 * n[0] * n[1] + p1 * (r2 + 2 * n[1] ** 2)
    ix = K[0] * dx + K[4] * dy + K[2]
    iy = K[1] * dy + K[3]
    cx = crop[0] * ix + crop[4] * iy + crop[2]
    cy = crop[1] * iy + crop[3]
    d = torch.stack([cx, cy]) - centre
    return (rot @ d + centre) * scale


def test_projection_backward_is_the_transposed_jacobian():
    """ProjectPointPinholeBackward (PointRendererHelper.h:317-372) chains the transposed Jacobians of TransformPoint,
    DivideByZ, distortNormalizedPoint and normalizedToImage.  The restatement's chain against automatic differentiation
    of the restated projection in float64: point, pose tangent, intrinsics and all eight distortion coefficients, with
    crop transform, crop rotation and a level scale."""
    rng = np.random.default_rng(12)
    sc = scenes.tiny_scene(n=40, w=64, h=48, n_views=3, seed=5, crop=True)
    sc.intrinsics[:, 4] = 0.7                                          # shear
    sc.intrinsics[:, 5:] = rng.uniform(-0.05, 0.05, size=(sc.intrinsics.shape[0], 8)).astype(np.float32)
    checked = 0
    for view in sc.views:
        for level, scale in ((0, 1.0), (2, 0.25)):
            for i in range(sc.n):
                grad = rng.standard_normal(2).astype(np.float32)
                out, g = O.project_with_backward(sc.position[i], sc.poses[view.image_index], sc.intrinsics[view.camera_index],
                                                 view, scale, grad)
                if g is None:
                    continue
                t64 = lambda a: torch.tensor(np.asarray(a, np.float64))
                p = t64(sc.position[i, :3]).requires_grad_(True)
                xi = torch.zeros(6, dtype=torch.float64, requires_grad=True)
                K = t64(sc.intrinsics[view.camera_index, :5]).requires_grad_(True)
                dist = t64(sc.intrinsics[view.camera_index, 5:]).requires_grad_(True)
                pose = sc.poses[view.image_index]
                ip = _projection_f64(p, xi, t64(np.float32(pose[:4])), t64(np.float32(pose[4:7])), K, dist, t64(view.crop),
                                     t64(view.rot).reshape(2, 2), t64([view.w // 2, view.h // 2]), scale)
                np.testing.assert_allclose(out[:2], ip.detach().numpy(), rtol=2e-5, atol=2e-4)
                (ip * t64(grad)).sum().backward()
                ref = np.concatenate([p.grad.numpy(), xi.grad.numpy(), K.grad.numpy(), dist.grad.numpy()])
                scale_of = np.abs(ref).max()
                np.testing.assert_allclose(g, ref, rtol=2e-4, atol=2e-5 * scale_of)
                checked += 1
    assert checked > 100
