"""The C++/libtorch operator surface (vet_b200/torch_shim: BlendPointCloud / PointRender autograd function) against the
oracle, through torch autograd: what the reference's pipeline would see."""
import os

import numpy as np
import pytest

from tests import util
from vet_b200 import scenes
from vet_b200.render import default_params

pytestmark = pytest.mark.gpu
SHIM = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "vet_b200", "libvetr_torch.so")


@pytest.fixture(scope="module")
def ops():
    import torch

    assert os.path.exists(SHIM), "build it with: python -m vet_b200.build --shim"
    torch.ops.load_library(SHIM)
    return torch.ops.vetr


def _views(sc, dev):
    import torch

    vi = torch.tensor([[v.w, v.h, v.image_index, v.camera_index, v.camera_model] for v in sc.views], dtype=torch.int32)
    vf = torch.tensor([list(v.crop) + list(v.rot) for v in sc.views], dtype=torch.float32)
    return vi, vf


@pytest.mark.parametrize("mode", [1, 3])
def test_blend_point_cloud_forward_backward(ops, mode):
    import torch

    dev = torch.device("cuda", 0)
    sc = scenes.tiny_scene(n=3000, n_views=3, seed=17, crop=True)
    params = default_params(render_mode=mode)
    ora = util.run_oracle(sc, params)
    grads = util.random_grads(ora["fwd"]["color"], seed=8)
    ora = util.run_oracle(sc, params, grads=grads)

    t = lambda a, rg=False: torch.from_numpy(a).to(dev).requires_grad_(rg)
    texture, background = t(sc.texture, True), t(sc.background, True)
    position, confidence = t(sc.position, True), t(sc.confidence[None], True)
    tangent = torch.zeros(sc.poses.shape[0], 6, dtype=torch.float64, device=dev, requires_grad=True)
    intr = t(sc.intrinsics, True)
    vi, vf = _views(sc, dev)
    out = ops.blend_point_cloud(texture, background, position, t(sc.index[:, None]), t(sc.poses), tangent, intr, confidence,
                                vi, vf, 4, mode, True, True, True, False, True)
    assert len(out) == 12  # colour, depth, mask per level (RenderInfo.cpp:40-42 order)
    for l in range(4):
        np.testing.assert_array_equal(out[l].detach().cpu().numpy(), ora["fwd"]["color"][l])
        np.testing.assert_array_equal(out[4 + l].detach().cpu().numpy(), ora["fwd"]["depth"][l])
        np.testing.assert_array_equal(out[8 + l].detach().cpu().numpy(), ora["fwd"]["mask"][l])
    loss = sum((o * torch.from_numpy(g).to(dev)).sum() for o, g in zip(out[:4], grads))
    loss.backward()
    b, m = ora["bwd"], ora["bwd_mag"]
    util.assert_sum_close("texture.grad", texture.grad.cpu().numpy(), b["texture"], m["texture"])
    util.assert_sum_close("confidence.grad", confidence.grad.cpu().numpy()[0], b["confidence"], m["confidence"])
    util.assert_sum_close("background.grad", background.grad.cpu().numpy(), b["background"], m["background"])
    cnt = np.maximum(b["points_count"], 1)[:, None]
    util.assert_sum_close("points.grad", position.grad.cpu().numpy()[:, :3], b["points"] / cnt, m["points"] / cnt)
    assert float(position.grad[:, 3].abs().max()) == 0.0
    pc = np.where(b["pose_count"] > 0, b["pose_count"], 1)[:, None]
    util.assert_sum_close("tangent.grad", tangent.grad.cpu().numpy(), b["pose"] / pc, m["pose"] / pc)
    ic = np.where(b["intrinsics_count"] > 0, b["intrinsics_count"], 1)[:, None]
    util.assert_sum_close("intrinsics.grad", intr.grad.cpu().numpy(), b["intrinsics"] / ic, m["intrinsics"] / ic)


def test_undefined_gradients_for_inputs_without_grad(ops):
    """PointRenderer.cu:272-300: no gradient tensors for inputs that do not require one."""
    import torch

    dev = torch.device("cuda", 0)
    sc = scenes.tiny_scene(n=1000, n_views=1, seed=19)
    t = lambda a, rg=False: torch.from_numpy(a).to(dev).requires_grad_(rg)
    texture = t(sc.texture, True)
    position, tangent, intr = t(sc.position), torch.zeros(1, 6, dtype=torch.float64, device=dev), t(sc.intrinsics)
    vi, vf = _views(sc, dev)
    out = ops.blend_point_cloud(texture, t(sc.background), position, t(sc.index[:, None]), t(sc.poses), tangent, intr,
                                t(sc.confidence[None]), vi, vf, 4, 1, False, False, True, False, True)
    assert len(out) == 4
    sum(o.sum() for o in out).backward()
    assert texture.grad is not None and position.grad is None and tangent.grad is None and intr.grad is None


def _render(ops, sc, mode=1, layers=4, drop_by_radius=True, backward=True):
    import torch

    dev = torch.device("cuda", 0)
    t = lambda a, rg=False: torch.from_numpy(a).to(dev).requires_grad_(rg)
    texture = t(sc.texture, True)
    tangent = torch.zeros(sc.poses.shape[0], 6, dtype=torch.float64, device=dev)
    vi, vf = _views(sc, dev)
    out = ops.blend_point_cloud(texture, t(sc.background), t(sc.position), t(sc.index[:, None]), t(sc.poses), tangent,
                                t(sc.intrinsics), t(sc.confidence[None]), vi, vf, layers, mode, False, False, drop_by_radius, False, False)
    if backward:
        sum(o.sum() for o in out).backward()
    torch.cuda.synchronize()
    return out, texture


def test_fragment_buffer_follows_what_was_seen(ops):
    """The shim sizes the fragment buffer from the totals of earlier calls (1.5 x the largest seen per view of the same cloud
    and pyramid) instead of the worst case; a view that needs more than that is reported at the next entry into the
    operator, and the call after that is sized safely again."""
    import copy

    sc = scenes.tiny_scene(n=20010, w=96, h=64, n_views=1, seed=33)
    far = copy.deepcopy(sc)
    far.position[500:, 0] += 1000.0  # all but 500 points leave the frustum: a handful of fragments, same tensor shapes
    params = default_params(drop_out_points_by_radius=0)
    ora, ora_far = util.run_oracle(sc, params), util.run_oracle(far, params)
    assert ora_far["F"] * 1.5 + 4096 < ora["F"]
    out, _ = _render(ops, far, drop_by_radius=False)      # first call of this shape: the bound that cannot overflow
    np.testing.assert_array_equal(out[0].detach().cpu().numpy(), ora_far["fwd"]["color"][0])
    out, _ = _render(ops, far, drop_by_radius=False)      # sized from the first call's total
    np.testing.assert_array_equal(out[0].detach().cpu().numpy(), ora_far["fwd"]["color"][0])
    with pytest.raises(RuntimeError, match="overflowed"):
        _render(ops, sc, drop_by_radius=False)            # the dense view exceeds it: reported before its gradients form
    for _ in range(3):                                    # the call after that is safe again, and so are the following ones
        out, _ = _render(ops, sc, drop_by_radius=False)
        np.testing.assert_array_equal(out[0].detach().cpu().numpy(), ora["fwd"]["color"][0])


def test_mode2_skipped_list_is_reported(ops):
    """Mode 2's backward pass skips lists of more than 4096 fragments; through the shim that surfaces as an error at the
    next call instead of silently missing gradients."""
    sc = scenes.tiny_scene(n=45000, w=16, h=12, n_views=1, seed=5)
    _render(ops, sc, mode=2, layers=3, drop_by_radius=False)
    with pytest.raises(RuntimeError, match="4096"):
        _render(ops, sc, mode=2, layers=3, drop_by_radius=False, backward=False)
    _render(ops, sc, mode=2, layers=3, drop_by_radius=False, backward=False)  # a forward-only call has nothing to report


def test_apply_tangent_to_pose(ops):
    import torch
    from oracle import oracle as O

    rng = np.random.default_rng(2)
    poses = scenes.orbit_poses(rng, 4, 3.0)
    tangent = rng.normal(scale=0.05, size=(4, 6))
    p_ref, t_ref = poses.copy(), tangent.copy()
    O.apply_tangent(t_ref, p_ref)
    p, tg = torch.from_numpy(poses).cuda(), torch.from_numpy(tangent).cuda()
    ops.apply_tangent_to_pose(tg, p)
    np.testing.assert_allclose(p.cpu().numpy(), p_ref, atol=1e-12)


def test_fill_scene_grid_with_loss(ops):
    """PointRendererCache::FillSceneGridWithLoss through the libtorch surface, against the CPU restatement."""
    import torch

    from oracle import oracle as O

    dev = torch.device("cuda", 0)
    w, h = 320, 240
    sc = scenes.config_planar(100, w, h, 230.0, n_views=2, seed=4)
    rng = np.random.default_rng(9)
    bb_min = rng.uniform(-8, 8, size=(1500, 3)).astype(np.float32)
    bb_len = rng.uniform(0.3, 2.0, size=(1500, 3)).astype(np.float32)
    loss = rng.standard_normal((3, h, w)).astype(np.float32)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    value = torch.zeros(1500, 1, device=dev)
    count = torch.zeros(1500, 1, dtype=torch.int32, device=dev)
    ref_v, ref_c = np.zeros(1500), np.zeros(1500, np.int64)
    for k, v in enumerate(sc.views):
        vi = torch.tensor([v.w, v.h, v.image_index, v.camera_index, v.camera_model], dtype=torch.int32)
        vf = torch.tensor(list(v.crop) + list(v.rot), dtype=torch.float32)
        ops.fill_scene_grid_with_loss(t(sc.poses), t(sc.intrinsics), vi, vf, t(bb_min), t(bb_len), value, count, t(loss))
        rv, rc = O.grid_loss(sc, v, bb_min, bb_len, loss)
        ref_v += rv
        ref_c += rc
    assert ref_c.sum() > 1000
    np.testing.assert_array_equal(count.cpu().numpy()[:, 0].astype(np.int64), ref_c)
    np.testing.assert_allclose(value.cpu().numpy()[:, 0], ref_v, rtol=1e-5)


def test_environment_map_sample2(ops):
    """EnvironmentMap::Sample2 through the libtorch surface and autograd, against the CPU restatement."""
    import torch

    from oracle import oracle as O

    dev = torch.device("cuda", 0)
    sc = util.env_scene(n_views=2, w=128, h=96, f=100.0)
    rng = np.random.default_rng(21)
    env = util.env_map(rng, S=4, R=32)
    L = 3
    weight = util.env_weights(rng, sc, L)
    ref = O.envmap_forward(sc, sc.views, L, env, weight)
    grads = [rng.standard_normal(r.shape).astype(np.float32) for r in ref]
    rgd, rgc, md, mc = O.envmap_backward(sc, sc.views, L, env, weight, grads)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    density = t(env.density[None, None]).requires_grad_(True)
    color = t(env.color[None]).requires_grad_(True)
    vi, vf = _views(sc, dev)
    out = ops.environment_map_sample2(density, color, 20.0, 5.0, env.up_axis, env.non_subzero, t(sc.poses), t(sc.intrinsics),
                                      vi, vf, L, [t(w) for w in weight])
    assert len(out) == L
    tol = util.env_sample_tolerance(env)
    for o, r in zip(out, ref):
        assert tuple(o.shape) == r.shape
        assert np.abs(o.detach().cpu().numpy() - r).max() <= tol
    sum((o * t(g)).sum() for o, g in zip(out, grads)).backward()
    assert np.all(np.abs(density.grad.cpu().numpy()[0, 0] - rgd) <= util.env_grad_tolerance(md, env))
    assert np.all(np.abs(color.grad.cpu().numpy()[0] - rgc) <= util.env_grad_tolerance(mc, env))


def test_compute_radius(ops):
    """SceneData::ComputeRadius through the libtorch surface, against the all-pairs restatement."""
    import torch

    from oracle import oracle as O

    sc = scenes.config_planar(6000, 64, 64, 50.0, seed=12)
    r = ops.compute_radius(torch.from_numpy(sc.position).cuda(), 4)
    np.testing.assert_array_equal(r.cpu().numpy(), O.knn_radius(sc.position[:, :3], 4))


def test_remove_points_in_place(ops):
    """NeuralScene::RemovePoints through the libtorch surface: the scene's tensors and the optimizer moments shrink in place."""
    import torch

    from oracle import oracle as O
    from tests.test_remove_points import _case

    n = 3000
    remove, (texture, conf, moments), (position, index) = _case(np.random.default_rng(5), n, 400)
    _, ref_last, ref_first = O.remove_points(n, remove, [texture, conf, moments], [position])
    t = lambda a: torch.from_numpy(a).cuda()
    g_tex, g_conf, g_pos, g_idx, g_mom = t(texture), t(conf), t(position), t(index), t(moments)
    kept = ops.remove_points(g_tex, g_conf, g_pos, g_idx, torch.from_numpy(remove), [g_mom])
    assert kept == ref_first[0].shape[0] and tuple(g_tex.shape) == (4, kept) and tuple(g_mom.shape) == (2, 4, kept)
    for g, r in zip((g_tex, g_conf, g_mom, g_pos), ref_last + ref_first):
        np.testing.assert_array_equal(g.cpu().numpy(), r)
    np.testing.assert_array_equal(g_idx.cpu().numpy()[:, 0], np.arange(kept))
