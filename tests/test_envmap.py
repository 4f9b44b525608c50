"""Texture environment map (EnvironmentMapImpl::Sample2 / forward_mps5, rendering/EnvironmentMap.cu:378-485, 692-758).

CPU part: the restatement in oracle/ against (1) rays and sphere hits computed independently in float64 and (2) the
libtorch operators the reference itself calls on the sample coordinates: grid_sample on the 5-D parameters, sigmoid,
the per-sphere multiply-add chain, and autograd for the parameter gradients.
GPU part: the CUDA kernels, through the C ABI, against the restatement.
"""
import numpy as np
import pytest
import torch
import torch.nn.functional as F

from oracle import oracle as O
from tests import util
from vet_b200 import scenes


def _rays_f64(sc, view, level):
    """World-space ray of every pixel of a level: origin = the pixel's point on the z = 1 plane, direction from the eye."""
    w, h = view.w >> level, view.h >> level
    q = sc.poses[view.image_index, :4]
    t = sc.poses[view.image_index, 4:7]
    x, y, z, s = q
    Rm = np.array([[1 - 2 * (y * y + z * z), 2 * (x * y - z * s), 2 * (x * z + y * s)],
                   [2 * (x * y + z * s), 1 - 2 * (x * x + z * z), 2 * (y * z - x * s)],
                   [2 * (x * z - y * s), 2 * (y * z + x * s), 1 - 2 * (x * x + y * y)]])
    K = sc.intrinsics[view.camera_index].astype(np.float64)
    crop = np.array(view.crop, np.float64) * 0.5 ** level
    rot = np.array(view.rot, np.float64).reshape(2, 2)
    gy, gx = np.mgrid[0:h, 0:w].astype(np.float64)
    c = np.array([w // 2, h // 2], np.float64)
    ip = np.stack([gx, gy], -1) - c
    ip = ip @ np.linalg.inv(rot).T + c
    py = (ip[..., 1] - crop[3]) / crop[1]
    px = (ip[..., 0] - crop[2] - crop[4] * py) / crop[0]
    ny = (py - K[3]) / K[1]
    nx = (px - K[2] - K[4] * ny) / K[0]
    cam = np.stack([nx, ny, np.ones_like(nx)], -1)
    eye = -Rm.T @ t
    wp = cam @ Rm + eye  # R^T cam + eye
    d = wp - eye
    d /= np.linalg.norm(d, axis=-1, keepdims=True)
    return wp.reshape(-1, 3), d.reshape(-1, 3)


def test_sample_coordinates_against_float64():
    sc = util.env_scene()
    rng = np.random.default_rng(0)
    for up_axis in (0, 1, 2):
        env = util.env_map(rng, S=4, up_axis=up_axis, inner_radius=3.0)  # the orbit cameras sit outside the first sphere
        for level in (0, 1):
            uvz, hit = O.envmap_uvz(sc, sc.views[1], level, env)
            o, d = _rays_f64(sc, sc.views[1], level)
            for s in range(env.n_spheres):
                if s == env.n_spheres - 1:
                    p, ok = d, np.ones(len(d), bool)
                else:
                    # |o + k d| = r, the far root
                    b = (o * d).sum(-1)
                    disc = b * b - ((o * o).sum(-1) - float(env.radii[s]) ** 2)
                    ok = disc >= 0
                    k = -b + np.sqrt(np.where(ok, disc, 0))
                    p = o + k[:, None] * d
                    p /= np.linalg.norm(p, axis=-1, keepdims=True)
                a = [(0, 1, 2), (1, 0, 2), (2, 0, 1)][up_axis]
                lat, lon = np.arcsin(p[:, a[0]]), np.arctan2(p[:, a[1]], p[:, a[2]])
                sure = np.abs(disc) > 1e-4 if s != env.n_spheres - 1 else ok
                assert np.array_equal(hit[s][sure] > 0, ok[sure])
                m = ok & sure
                assert m.sum() > 0
                du = np.abs(uvz[s, m, 0] - lon[m] / np.pi)
                du = np.minimum(du, 2 - du)  # the seam
                assert du.max() < 5e-6
                assert np.abs(uvz[s, m, 1] - 2 * lat[m] / np.pi).max() < 5e-6
                assert np.allclose(uvz[s, :, 2][m], 2 * s / (env.n_spheres - 1) - 1, atol=1e-6)


def test_rays_invert_the_rasterizer_projection():
    """The two halves of a VET image must register: a point placed on the environment-map ray of pixel (x, y) of level l
    is drawn by the rasterizer into exactly that pixel of that level.  Ties the restated unproject2 / SE3 inverse / inverse
    crop rotation to the restated projection, with crop transform, crop rotation and skew-free intrinsics."""
    sc = scenes.tiny_scene(n=4, w=64, h=48, n_views=2, seed=31, crop=True)
    rng = np.random.default_rng(4)
    L = 3
    for b, view in enumerate(sc.views):
        for level in range(L):
            w, h = view.w >> level, view.h >> level
            o, d = O.envmap_rays(sc, view, level)
            pick = rng.choice(w * h, size=25, replace=False)
            t = rng.uniform(2.0, 6.0, size=(25, 1)).astype(np.float32)
            pts = o[pick] + t * d[pick]
            cloud = scenes.Scene(position=np.concatenate([pts, np.full((25, 1), 10.0, np.float32)], 1).astype(np.float32),
                                 index=np.arange(25, dtype=np.int32), texture=np.ones((4, 25), np.float32),
                                 confidence=np.full(25, 0.5, np.float32), background=np.zeros(4, np.float32),
                                 poses=sc.poses, intrinsics=sc.intrinsics, views=sc.views)
            res = O.Oracle().forward(cloud, O.default_params(num_layers=L), views=[view])
            drawn = res["depth"][level][0, 0] < 1000.0  # 100000 where nothing was drawn
            ys, xs = pick // w, pick % w
            assert drawn[ys, xs].all(), (b, level, int((~drawn[ys, xs]).sum()))
            assert drawn.sum() == 25  # and nowhere else on that level


def _torch_forward_mps5(env, uvz, hit, T0, density_t, color_t):
    """forward_mps5 (EnvironmentMap.cu:692-758) with libtorch's operators on given sample coordinates."""
    S, n = uvz.shape[0], uvz.shape[1]
    grid = torch.from_numpy(uvz).reshape(1, S * n, 1, 1, 3)
    dens = F.grid_sample(density_t, grid, mode="bilinear", padding_mode="zeros", align_corners=True).reshape(1, S, n)
    alpha_all = torch.sigmoid(dens.permute(1, 0, 2))
    col = F.grid_sample(color_t, grid, mode="bilinear", padding_mode="zeros", align_corners=True)
    col = col.reshape(env.channels, S, n).permute(1, 0, 2)
    if env.non_subzero:
        col = torch.abs(col)
    final = torch.zeros(env.channels, n)
    T = torch.from_numpy(T0).reshape(n, 1)
    for s in range(S):
        alpha = alpha_all[s]
        if s == S - 1:
            alpha = torch.ones_like(alpha)
        alpha = alpha * torch.from_numpy(hit[s]).unsqueeze(0)
        final = T.squeeze().unsqueeze(0) * alpha * col[s] + final
        T = ((1 - alpha.squeeze()) * T.squeeze()).unsqueeze(1)
    return final


@pytest.mark.parametrize("non_subzero,S", [(False, 4), (True, 3), (False, 1)])
def test_forward_and_backward_against_libtorch_operators(non_subzero, S):
    sc = util.env_scene()
    rng = np.random.default_rng(5)
    env = util.env_map(rng, S=S, non_subzero=non_subzero)
    L = 2
    weight = util.env_weights(rng, sc, L)
    out = O.envmap_forward(sc, sc.views, L, env, weight)
    grad_out = [rng.standard_normal(o.shape).astype(np.float32) for o in out]
    gd, gc, md, mc = O.envmap_backward(sc, sc.views, L, env, weight, grad_out)

    density_t = torch.from_numpy(env.density)[None, None].clone().requires_grad_(True)
    color_t = torch.from_numpy(env.color)[None].clone().requires_grad_(True)
    loss = 0
    for l in range(L):
        for b, view in enumerate(sc.views):
            uvz, hit = O.envmap_uvz(sc, view, l, env)
            assert hit.min() == 1.0  # cameras inside the first sphere: every ray hits every sphere
            ref = _torch_forward_mps5(env, uvz, hit, weight[l][b].reshape(-1), density_t, color_t)
            ref = ref.reshape(env.channels, view.h >> l, view.w >> l)
            # same operators, same order: only the rounding of exp() and of fused multiply-adds can differ
            np.testing.assert_allclose(out[l][b], ref.detach().numpy(), rtol=2e-6, atol=2e-6)
            loss = loss + (ref * torch.from_numpy(grad_out[l][b])).sum()
    loss.backward()
    tgc = color_t.grad[0].numpy()
    tgd = density_t.grad[0, 0].numpy() if S > 1 else np.zeros_like(env.density)  # one sphere: its alpha is the constant 1
    assert np.abs(tgd).max() > 0 or S == 1
    assert np.all(np.abs(gd - tgd) <= 1e-5 * md + 1e-7)
    assert np.all(np.abs(gc - tgc) <= 1e-5 * mc + 1e-7)


def test_flags():
    sc = util.env_scene()
    rng = np.random.default_rng(9)
    env = util.env_map(rng)
    L = 2
    weight = util.env_weights(rng, sc, L)
    plain = O.envmap_forward(sc, sc.views, L, env, weight)
    start = [rng.standard_normal(o.shape).astype(np.float32) for o in plain]
    added = O.envmap_forward(sc, sc.views, L, env, weight, flags=O.ENV_ADD, out=[s.copy() for s in start])
    for a, s, p in zip(added, start, plain):
        assert np.array_equal(a, s + p)
    masked = O.envmap_forward(sc, sc.views, L, env, weight, flags=O.ENV_NOT_AT_POINTS)
    for m, p, w in zip(masked, plain, weight):
        keep = np.broadcast_to(w <= 0.001, p.shape)
        assert np.array_equal(m[keep], p[keep]) and np.all(m[~keep] == 0)
    # mode 0: the weight is a hit count
    counts = [np.floor(w * 3) for w in weight]
    dt = O.envmap_forward(sc, sc.views, L, env, counts, flags=O.ENV_DEPTH_TEST_WEIGHT | O.ENV_ADD, out=[s.copy() for s in start])
    full = O.envmap_forward(sc, sc.views, L, env, [np.ones_like(w) for w in weight])
    for d, s, fl, c in zip(dt, start, full, counts):
        hitp = np.broadcast_to(c > 0.5, s.shape)
        assert np.array_equal(d[hitp], s[hitp]) and np.array_equal(d[~hitp], fl[~hitp])
    # masked pixels send no gradient
    g = [np.ones_like(p) for p in plain]
    gd0, gc0, _, _ = O.envmap_backward(sc, sc.views, L, env, [np.ones_like(w) for w in weight], g, flags=O.ENV_NOT_AT_POINTS)
    assert not gd0.any() and not gc0.any()


def _fixture():
    import os

    g = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "oracle_tiny.npz"))
    sc = scenes.tiny_scene(n=4, w=40, h=28, n_views=2, seed=79, crop=True)  # the scene tests/golden/make_golden.py used
    env = O.EnvMap(g["env_density"], g["env_color"], up_axis=1)
    assert np.array_equal(env.radii, g["env_radii"])
    return g, sc, env, 2


def test_fixture_restatement_and_libtorch_values():
    """The committed fixture holds the restatement's output and, beside it, forward_mps5 evaluated with libtorch's own
    grid_sample / sigmoid / autograd when the fixture was made: the restatement reproduces the first bit for bit and
    agrees with the second."""
    g, sc, env, L = _fixture()
    weight = [g[f"env_weight_l{l}"] for l in range(L)]
    out = O.envmap_forward(sc, sc.views, L, env, weight)
    gd, gc, md, mc = O.envmap_backward(sc, sc.views, L, env, weight, [g[f"env_gout_l{l}"] for l in range(L)])
    for l in range(L):
        assert np.array_equal(out[l], g[f"env_out_l{l}"])
        np.testing.assert_allclose(out[l], g[f"env_torch_l{l}"], rtol=2e-6, atol=2e-6)
    assert np.array_equal(gd, g["env_g_density"]) and np.array_equal(gc, g["env_g_color"])
    assert np.all(np.abs(gd - g["env_torch_g_density"]) <= 1e-5 * md + 1e-7)
    assert np.all(np.abs(gc - g["env_torch_g_color"]) <= 1e-5 * mc + 1e-7)


# ---------------------------------------------------------------------------------------------------------
# CUDA kernels against the restatement


@pytest.mark.gpu
@pytest.mark.parametrize("up_axis,non_subzero,S,flags", [(0, False, 4, 0), (1, True, 3, O.ENV_NOT_AT_POINTS), (2, False, 1, 0),
                                                         (0, False, 8, 0)])
def test_gpu_envmap_matches_oracle(up_axis, non_subzero, S, flags):
    sc = util.env_scene(n_views=3, w=200, h=120, f=150.0)
    rng = np.random.default_rng(11)
    env = util.env_map(rng, S=S, R=64, up_axis=up_axis, non_subzero=non_subzero)
    # smooth textures: the comparison is of the arithmetic, not of how a 1e-6 texel shift samples noise
    k = torch.ones(1, 1, 5, 5) / 25
    env.color = F.conv2d(torch.from_numpy(env.color).reshape(-1, 1, 64, 64), k, padding=2).reshape(env.color.shape).numpy()
    env.density = F.conv2d(torch.from_numpy(env.density).reshape(-1, 1, 64, 64), k, padding=2).reshape(env.density.shape).numpy()
    if non_subzero:  # |.| has no gradient at 0: keep the samples away from it, with both signs present
        sign = np.where(np.arange(env.channels) % 2 == 0, -1.0, 1.0).astype(np.float32)[:, None, None, None]
        env.color = sign * (np.abs(env.color) + 0.1)
    L = 3
    weight = util.env_weights(rng, sc, L)
    ref = O.envmap_forward(sc, sc.views, L, env, weight, flags=flags)
    grad_out = [rng.standard_normal(o.shape).astype(np.float32) for o in ref]
    rgd, rgc, md, mc = O.envmap_backward(sc, sc.views, L, env, weight, grad_out, flags=flags)
    out, gd, gc = util.env_gpu_run(sc, env, L, weight, flags, grad_out)
    tol = util.env_sample_tolerance(env)
    for o, r in zip(out, ref):
        assert np.abs(o - r).max() <= tol
    assert np.abs(rgc).max() > 0
    assert np.all(np.abs(gd - rgd) <= util.env_grad_tolerance(md, env))
    assert np.all(np.abs(gc - rgc) <= util.env_grad_tolerance(mc, env))


@pytest.mark.gpu
def test_gpu_envmap_add_and_depth_test_flags():
    sc = util.env_scene(n_views=2, w=96, h=64, f=80.0)
    rng = np.random.default_rng(13)
    env = util.env_map(rng, S=4, R=32)
    L = 2
    weight = [np.floor(w * 3) for w in util.env_weights(rng, sc, L)]
    flags = O.ENV_ADD | O.ENV_DEPTH_TEST_WEIGHT
    start = [rng.standard_normal((2, 4, 64 >> l, 96 >> l)).astype(np.float32) for l in range(L)]
    ref = O.envmap_forward(sc, sc.views, L, env, weight, flags=flags, out=[s.copy() for s in start])
    out = util.env_gpu_run(sc, env, L, weight, flags, start=start)
    tol = util.env_sample_tolerance(env)
    for o, r in zip(out, ref):
        assert np.abs(o - r).max() <= tol


@pytest.mark.gpu
def test_gpu_envmap_rejects_distortion_and_bad_arguments():
    from vet_b200 import _lib
    from vet_b200.render import Rasterizer

    sc = util.env_scene()
    rng = np.random.default_rng(1)
    env = util.env_map(rng, R=16)
    dev = torch.device("cuda:0")
    rast = Rasterizer(0)
    poses = torch.from_numpy(sc.poses).to(dev)
    density, color = torch.from_numpy(env.density).to(dev), torch.from_numpy(env.color).to(dev)
    w_t = [torch.ones(2, 1, 56, 80, device=dev)]
    distorted = sc.intrinsics.copy()
    distorted[:, 5] = 0.1
    with pytest.raises(_lib.VetrError) as ei:
        rast.envmap_forward(poses, torch.from_numpy(distorted).to(dev), sc.views, 1, density, color, env.radii, w_t)
    assert ei.value.status == _lib.E_UNSUPPORTED
    intr = torch.from_numpy(sc.intrinsics).to(dev)
    with pytest.raises(_lib.VetrError) as ei:
        rast.envmap_forward(poses, intr, sc.views, 1, density, color, env.radii, w_t, up_axis=3)
    assert ei.value.status == _lib.E_INVALID_ARG
    with pytest.raises(_lib.VetrError) as ei:
        rast.envmap_forward(poses, intr, sc.views, 1, density, color, env.radii, w_t, flags=64)
    assert ei.value.status == _lib.E_INVALID_ARG


@pytest.mark.gpu
def test_gpu_envmap_against_fixture():
    """The kernels against the committed fixture: the restatement's values and those of libtorch's operators."""
    g, sc, env, L = _fixture()
    weight = [g[f"env_weight_l{l}"] for l in range(L)]
    gout = [g[f"env_gout_l{l}"] for l in range(L)]
    out, gd, gc = util.env_gpu_run(sc, env, L, weight, 0, gout)
    tol = util.env_sample_tolerance(env)
    for l in range(L):
        assert np.abs(out[l] - g[f"env_out_l{l}"]).max() <= tol
        assert np.abs(out[l] - g[f"env_torch_l{l}"]).max() <= tol
    for mine, ref, mag in ((gd, g["env_torch_g_density"], g["env_mag_density"]), (gc, g["env_torch_g_color"], g["env_mag_color"]),
                           (gd, g["env_g_density"], g["env_mag_density"]), (gc, g["env_g_color"], g["env_mag_color"])):
        assert np.all(np.abs(mine - ref) <= util.env_grad_tolerance(mag, env))
