"""CUDA library vs CPU oracle on identical seeded inputs, through the C ABI (vet_b200.render -> libvetr.so).

Bar: per-pixel counts, fragment keys and their order bit-exact; images within 1e-5 relative (they are in fact
bit-equal, the blend is evaluated in the same order with the same fused multiply-add); raw gradient sums within
1e-5 relative to each element's sum of |addends| (fp32 atomic summation order is not defined; the oracle sums the
same fp32 addends in fp64 and also reports that magnitude).
"""
import numpy as np
import pytest

from tests import util
from vet_b200 import scenes
from vet_b200.render import default_params

pytestmark = pytest.mark.gpu


def _roundtrip(rast, scene, params, dropout=None, exact_images=True, grads="random"):
    ora = util.run_oracle(scene, params, dropout=dropout)
    g = util.random_grads(ora["fwd"]["color"], seed=3) if grads == "random" else util.l1_grads(ora["fwd"]["color"], seed=3)
    ora = util.run_oracle(scene, params, grads=g, dropout=dropout)
    gpu = util.run_gpu(rast, scene, params, grads=g, dropout=dropout)
    util.compare_forward(gpu, ora, exact_images=exact_images)
    util.compare_backward(gpu["bwd_raw"], ora, scene.channels)
    return gpu, ora


@pytest.mark.parametrize("mode", [1, 3])
@pytest.mark.parametrize("crop", [False, True])
def test_tiny_scene(rasterizer, mode, crop):
    sc = scenes.tiny_scene(n=3000, crop=crop)
    _roundtrip(rasterizer, sc, default_params(render_mode=mode))


@pytest.mark.parametrize("mode", [1, 3])
def test_dense_lists_no_radius_dropout(rasterizer, mode):
    """Every visible point reaches all levels: lists of hundreds of fragments at the coarse levels."""
    sc = scenes.tiny_scene(n=40000, w=96, h=64, n_views=2, seed=11)
    gpu, _ = _roundtrip(rasterizer, sc, default_params(render_mode=mode, drop_out_points_by_radius=0))
    assert gpu["longest"] > 200


@pytest.mark.parametrize("mode", [1, 3])
def test_long_list_slow_path(rasterizer, mode):
    """Lists beyond the shared-memory fast path (> 1024 fragments in one pixel)."""
    sc = scenes.tiny_scene(n=30000, w=16, h=12, n_views=1, seed=5)
    gpu, _ = _roundtrip(rasterizer, sc, default_params(render_mode=mode, drop_out_points_by_radius=0, num_layers=3))
    assert gpu["longest"] > 2048 + 100


@pytest.mark.parametrize("accept", [0.01, 0.2])
def test_mode2_fuzzy_blend(rasterizer, accept):
    """FUZZY_BLEND: depth-window groups; the reference groups differently in forward and backward, both reproduced."""
    sc = scenes.tiny_scene(n=6000, n_views=2, seed=23, crop=True)
    _roundtrip(rasterizer, sc, default_params(render_mode=2, depth_accept_blend=accept))
    _roundtrip(rasterizer, sc, default_params(render_mode=2, depth_accept_blend=accept, use_environment_map=1))
    _roundtrip(rasterizer, sc, default_params(render_mode=2, depth_accept_blend=accept, debug_max_list_length=3))


def test_mode2_dense_and_long_lists(rasterizer):
    from vet_b200 import _lib as L

    sc = scenes.tiny_scene(n=40000, w=96, h=64, n_views=2, seed=11)
    gpu, _ = _roundtrip(rasterizer, sc, default_params(render_mode=2, drop_out_points_by_radius=0, depth_accept_blend=0.02))
    assert gpu["longest"] > 200
    sc = scenes.tiny_scene(n=12000, w=16, h=12, n_views=1, seed=5)  # lists of 300 .. 1600: whole-list kernel
    gpu, _ = _roundtrip(rasterizer, sc, default_params(render_mode=2, drop_out_points_by_radius=0, num_layers=3))
    assert 256 < gpu["longest"] <= 3072
    # up to 4096 fragments in one list (what the reference sorts of a list) the backward pass handles the list
    sc = scenes.tiny_scene(n=30000, w=16, h=12, n_views=1, seed=5)
    params = default_params(render_mode=2, drop_out_points_by_radius=0, num_layers=3)
    gpu, _ = _roundtrip(rasterizer, sc, params)
    assert 3072 < gpu["longest"] <= 4096
    # beyond that it skips the pixel and says so
    sc = scenes.tiny_scene(n=45000, w=16, h=12, n_views=1, seed=5)
    ora = util.run_oracle(sc, params)
    gpu = util.run_gpu(rasterizer, sc, params, grads=util.random_grads(ora["fwd"]["color"]))
    util.compare_forward(gpu, ora)  # the forward pass has no such limit
    assert gpu["longest"] > 4096
    with pytest.raises(L.VetrError) as e:
        rasterizer.fragment_count()
    assert e.value.status == L.E_TOO_LARGE


def _mode0_roundtrip(rast, scene, params, dropout=None):
    """Mode 0 sums descriptors with float atomics in an undefined order (as the reference does): images are compared
    within 1e-5 of the largest descriptor magnitude instead of bit for bit; weights, depths and masks are exact."""
    ora = util.run_oracle(scene, params, dropout=dropout)
    g = util.random_grads(ora["fwd"]["color"], seed=3)
    ora = util.run_oracle(scene, params, grads=g, dropout=dropout)
    gpu = util.run_gpu(rast, scene, params, grads=g, dropout=dropout)
    assert gpu["F"] == ora["F"]
    np.testing.assert_array_equal(gpu["counts"], ora["counts"])
    tol = 1e-5 * float(np.abs(scene.texture).max())
    for l in range(len(ora["fwd"]["color"])):
        np.testing.assert_allclose(gpu["fwd"]["color"][l], ora["fwd"]["color"][l], rtol=1e-5, atol=tol)
        for name in ("weight", "mask", "depth"):
            np.testing.assert_array_equal(gpu["fwd"][name][l], ora["fwd"][name][l], err_msg=name)
    # the backward pass reads the forward image, which here differs from the oracle's in the last bits: an addend
    # (T - I) * G inherits that difference relative to |I * G|, not to its own size, hence the floor per tensor
    util.compare_backward(gpu["bwd_raw"], ora, scene.channels, rtol=2e-5, floor_rel=1e-6)
    return gpu, ora


def test_mode0_fuzzy_depth_test(rasterizer):
    """FUZZY_DT: nearest-depth pre-pass, depth-tested splat, combine; per-point backward."""
    sc = scenes.tiny_scene(n=6000, n_views=2, seed=29)
    _mode0_roundtrip(rasterizer, sc, default_params(render_mode=0))
    _mode0_roundtrip(rasterizer, sc, default_params(render_mode=0, depth_accept=0.2, drop_out_points_by_radius=0))
    sc3 = scenes.tiny_scene(n=4000, n_views=1, seed=30, channels=3, crop=True)  # crop rotation: the backward pass ignores it
    _mode0_roundtrip(rasterizer, sc3, default_params(render_mode=0))
    rng = np.random.default_rng(0)
    dropout = (rng.uniform(size=(len(sc.views), sc.n)) < 0.3).astype(np.float32)
    _mode0_roundtrip(rasterizer, sc, default_params(render_mode=0), dropout=dropout)
    _mode0_roundtrip(rasterizer, sc, default_params(render_mode=0, ghost_gradients=1), dropout=dropout)
    _mode0_roundtrip(rasterizer, sc, default_params(render_mode=0, viewer_only=1, stability_cutoff_value=0.4))


def test_three_channels_env_map_and_truncation(rasterizer):
    sc = scenes.tiny_scene(n=4000, channels=3, seed=21)
    _roundtrip(rasterizer, sc, default_params(use_environment_map=1))
    _roundtrip(rasterizer, sc, default_params(debug_max_list_length=3))
    _roundtrip(rasterizer, sc, default_params(render_mode=3, debug_max_list_length=2, num_layers=2))


def test_dropout_mask_and_viewer_discard(rasterizer):
    sc = scenes.tiny_scene(n=3000, seed=31)
    rng = np.random.default_rng(0)
    dropout = (rng.uniform(size=(len(sc.views), sc.n)) < 0.25).astype(np.float32)
    _roundtrip(rasterizer, sc, default_params(), dropout=dropout)
    _roundtrip(rasterizer, sc, default_params(viewer_only=1, stability_cutoff_value=0.4))


def test_flags_off(rasterizer):
    sc = scenes.tiny_scene(n=3000, seed=41)
    _roundtrip(rasterizer, sc, default_params(need_point_gradient=0))
    _roundtrip(rasterizer, sc, default_params(background_alpha_to_point0=0))
    _roundtrip(rasterizer, sc, default_params(render_mode=3, need_point_gradient=0))


def test_distortion(rasterizer):
    sc = scenes.tiny_scene(n=3000, seed=51, crop=True)
    sc.intrinsics[0, 5:] = np.array([0.05, -0.02, 0.003, 0.01, 0.002, -0.001, 0.004, -0.003], np.float32)
    sc.intrinsics[0, 4] = 0.01
    _roundtrip(rasterizer, sc, default_params())
    _roundtrip(rasterizer, sc, default_params(render_mode=3, dist_cutoff=0.5))


def test_empty_and_degenerate(rasterizer):
    sc = scenes.tiny_scene(n=64, w=8, h=8, n_views=1, seed=61)
    sc.position[:, :3] += 100.0  # everything outside the frustum: all lists empty
    gpu, ora = _roundtrip(rasterizer, sc, default_params())
    assert gpu["F"] == 0
    sc2 = scenes.tiny_scene(n=1, w=5, h=3, n_views=1, seed=62)
    _roundtrip(rasterizer, sc2, default_params(num_layers=1))
    sc3 = scenes.tiny_scene(n=500, w=40, h=24, n_views=1, seed=63)
    _roundtrip(rasterizer, sc3, default_params(num_layers=5))  # coarsest level is 2x1


def test_invalid_arguments_are_refused(rasterizer):
    """Error behaviour: the reference asserts (aborts); the C ABI returns a status instead."""
    from vet_b200 import _lib as L

    sc = scenes.tiny_scene(n=10, w=5, h=3, n_views=1, seed=62)
    for bad in (dict(num_layers=5), dict(num_layers=0), dict(render_mode=4), dict(render_mode=-1)):
        with pytest.raises(L.VetrError) as e:
            util.run_gpu(rasterizer, sc, default_params(**bad))
        assert e.value.status in (L.E_INVALID_ARG, L.E_UNSUPPORTED)
    sc.views[0].camera_model = 1  # OCam is not built
    with pytest.raises(L.VetrError) as e:
        util.run_gpu(rasterizer, sc, default_params(num_layers=1))
    assert e.value.status == L.E_UNSUPPORTED


def test_many_views_grouped(rasterizer):
    """More views than one launch takes: the host mirror splits the batch."""
    sc = scenes.tiny_scene(n=2000, w=40, h=30, n_views=11, seed=71)
    ora = util.run_oracle(sc, default_params())
    gpu = util.run_gpu(rasterizer, sc, default_params())
    assert gpu["F"] == ora["F"]
    for a, b in zip(gpu["fwd"]["color"], ora["fwd"]["color"]):
        np.testing.assert_array_equal(a, b)


def test_plumbing_config_l1(rasterizer):
    """Configuration 1 of the benchmark set: 100k points, one 512x512 view, L1 loss against a seeded target."""
    sc = scenes.config_plumbing()
    _roundtrip(rasterizer, sc, default_params(), grads="l1")
    _roundtrip(rasterizer, sc, default_params(render_mode=3), grads="l1")


@pytest.mark.parametrize("mode", [1, 3])
def test_benchmark_configs_2_3_4(rasterizer, mode):
    """The generators of benchmark configurations 2, 3 and 4 at a size the oracle finishes in seconds (the full sizes are
    compared inside bench.py): the viewer frame (forward only, 1920x1080), the training step (four 1024x768 views, gradients
    to descriptors, confidences, positions, pose and intrinsics) and the scene inside four concentric point shells."""
    params = default_params(render_mode=mode)
    sc = scenes.config_planar(300_000, 1920, 1080, 1200.0, n_views=1, seed=2002)
    ora = util.run_oracle(sc, params)
    gpu = util.run_gpu(rasterizer, sc, params)
    util.compare_forward(gpu, ora, exact_images=True)
    sc = scenes.config_planar(300_000, 1024, 768, 900.0, n_views=4, seed=3003)
    gpu, _ = _roundtrip(rasterizer, sc, params, grads="l1")
    assert np.abs(gpu["bwd_raw"]["pose"]).sum() > 0 and np.abs(gpu["bwd_raw"]["intrinsics"]).sum() > 0
    sc = scenes.config_shells(n_scene=180_000, n_shell=40_000)
    gpu, _ = _roundtrip(rasterizer, sc, params, grads="l1")
    assert gpu["F"] > 100_000


def test_mode0_sparse_cloud_on_a_large_image(rasterizer):
    """Mode 0 keeps one accumulator record per pixel: with fewer points than pixels the buffer is sized by the pixel space
    (vetr_list_capacity), not by the fragment bound."""
    sc = scenes.tiny_scene(n=500, w=256, h=256, n_views=2, seed=91)
    _mode0_roundtrip(rasterizer, sc, default_params(render_mode=0))


def test_key_buffer_overflow_is_reported(rasterizer):
    from vet_b200 import _lib as L

    sc = scenes.tiny_scene(n=3000, seed=81)
    with pytest.raises(L.VetrError) as e:
        util.run_gpu(rasterizer, sc, default_params(), capacity=100)
    assert e.value.status == L.E_LIST_OVERFLOW


def test_reference_layout_of_lists(rasterizer):
    """vetr_get_lists: collections [2,F_l] (depth bits, point index) and scanned_counting per (view, layer)."""
    import torch

    sc = scenes.tiny_scene(n=3000, seed=91)
    params = default_params()
    ora = util.run_oracle(sc, params)
    util.run_gpu(rasterizer, sc, params)
    P = ora["counts"].size // len(sc.views)
    starts = np.concatenate([[0], np.cumsum(ora["counts"])])
    sizes = [(sc.views[0].w >> l, sc.views[0].h >> l) for l in range(4)]
    base = 0
    for layer, (w, h) in enumerate(sizes):
        for view in range(len(sc.views)):
            g0 = view * P + base
            coll, scanned = rasterizer.lists_of(view, layer)
            coll, scanned = coll.cpu().numpy(), scanned.cpu().numpy()
            keys = ora["keys"][starts[g0]:starts[g0 + w * h]]
            np.testing.assert_array_equal(coll[0].view(np.uint32), (keys >> np.uint64(32)).astype(np.uint32))
            np.testing.assert_array_equal(coll[1].view(np.uint32), (keys & np.uint64(0xffffffff)).astype(np.uint32))
            np.testing.assert_array_equal(scanned, starts[g0:g0 + w * h] - starts[g0])
        base += w * h


def test_apply_tangent(rasterizer):
    import torch
    from oracle import oracle as O

    rng = np.random.default_rng(5)
    n = 37
    poses = scenes.orbit_poses(rng, n, 4.0)
    tangent = rng.normal(scale=0.05, size=(n, 6))
    tangent[0] = 0.0
    tangent[1, 3:] = 1e-13
    p_ref, t_ref = poses.copy(), tangent.copy()
    O.apply_tangent(t_ref, p_ref)
    p = torch.from_numpy(poses).cuda()
    t = torch.from_numpy(tangent).cuda()
    rasterizer.apply_tangent(t, p)
    np.testing.assert_allclose(p.cpu().numpy(), p_ref, rtol=0, atol=1e-12)
    assert float(t.abs().max()) == 0.0


def test_finalize_matches_reference_normalisation(rasterizer):
    import torch

    sc = scenes.tiny_scene(n=3000, seed=101)
    params = default_params()
    ora = util.run_oracle(sc, params)
    g = util.random_grads(ora["fwd"]["color"], seed=1)
    ora = util.run_oracle(sc, params, grads=g)
    util.run_gpu(rasterizer, sc, params)
    raw = rasterizer.backward_raw([torch.from_numpy(x).cuda() for x in g])
    fin = rasterizer.finalize({k: v.clone() for k, v in raw.items()})
    torch.cuda.synchronize()
    b, m = ora["bwd"], ora["bwd_mag"]
    util.assert_sum_close("texture", fin["texture"].cpu().numpy(), b["texture"], m["texture"])
    cnt = np.maximum(b["points_count"], 1)[:, None]
    util.assert_sum_close("points", fin["points"].cpu().numpy()[:, :3], b["points"] / cnt, m["points"] / cnt)
    assert float(fin["points"][:, 3].abs().max()) == 0.0
    pc = np.where(b["pose_count"] > 0, b["pose_count"], 1)[:, None]
    util.assert_sum_close("pose", fin["pose"].cpu().numpy(), b["pose"] / pc, m["pose"] / pc)
    ic = np.where(b["intrinsics_count"] > 0, b["intrinsics_count"], 1)[:, None]
    util.assert_sum_close("intrinsics", fin["intrinsics"].cpu().numpy(), b["intrinsics"] / ic, m["intrinsics"] / ic)


@pytest.mark.parametrize("mode", [0, 1, 2, 3])
def test_committed_fixture(rasterizer, mode):
    """The CUDA path against tests/golden/oracle_tiny.npz alone (no oracle run): lists, images, raw gradient sums."""
    import os

    data = np.load(os.path.join(os.path.dirname(__file__), "golden", "oracle_tiny.npz"))
    sc = scenes.tiny_scene(n=400, w=24, h=16, n_views=2, seed=77, crop=True)
    params = default_params(render_mode=mode, num_layers=3)
    grads = [data[f"grad_m{mode}_l{l}"] for l in range(3)]
    gpu = util.run_gpu(rasterizer, sc, params, grads=grads)
    if mode != 0:
        np.testing.assert_array_equal(gpu["counts"], data[f"counts_m{mode}"])
        np.testing.assert_array_equal(gpu["keys"], data[f"keys_m{mode}"])
    for l in range(3):
        if mode == 0:  # float atomics in no fixed order, in the reference too
            util.assert_close(f"color[{l}]", gpu["fwd"]["color"][l], data[f"color_m{mode}_l{l}"], rtol=1e-5, floor_rel=1e-6)
        else:
            np.testing.assert_array_equal(gpu["fwd"]["color"][l], data[f"color_m{mode}_l{l}"])
        np.testing.assert_array_equal(gpu["fwd"]["weight"][l], data[f"weight_m{mode}_l{l}"])
        np.testing.assert_array_equal(gpu["fwd"]["depth"][l], data[f"depth_m{mode}_l{l}"])
    raw = gpu["bwd_raw"]
    rtol = 2e-5 if mode == 0 else 1e-5
    floor = 1e-6 if mode == 0 else 0.0
    chk = lambda name, got, key: util.assert_sum_close(name, got, data[f"bwd_m{mode}_{key}"], data[f"mag_m{mode}_{key}"], rtol,
                                                       floor_rel=floor)
    chk("g_texture", raw["desc"][:, :4].T, "texture")
    chk("g_confidence", raw["conf"], "confidence")
    chk("g_background", raw["background"], "background")
    chk("g_points", raw["points"][:, :3], "points")
    chk("g_pose", raw["pose"], "pose")
    chk("g_intrinsics", raw["intrinsics"], "intrinsics")


def test_committed_fixture_grid_loss(rasterizer):
    import os

    import torch

    data = np.load(os.path.join(os.path.dirname(__file__), "golden", "oracle_tiny.npz"))
    sc = scenes.tiny_scene(n=4, w=160, h=128, n_views=2, seed=78, crop=True)
    dev = rasterizer.device
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    value = torch.zeros(200, device=dev)
    count = torch.zeros(200, dtype=torch.int32, device=dev)
    for v in sc.views:
        rasterizer.grid_loss(t(sc.poses), t(sc.intrinsics), v, t(data["grid_bb_min"]), t(data["grid_bb_len"]),
                             t(data["grid_loss_img"]), value, count)
    np.testing.assert_array_equal(count.cpu().numpy().astype(np.int64), data["grid_count"])
    np.testing.assert_allclose(value.cpu().numpy(), data["grid_value"], rtol=1e-5)


def test_l1_loss_grad(rasterizer):
    """The one-launch L1 loss + gradient against torch's element-wise operators (odd sizes: unaligned level tails)."""
    import torch

    dev = rasterizer.device
    gen = torch.Generator(device="cpu").manual_seed(2)
    shapes = [(2, 3, 7, 9), (2, 3, 3, 4), (1, 1, 1, 1), (2, 4, 16, 16)]
    images = [torch.rand(s, generator=gen).to(dev) for s in shapes]
    targets = [torch.rand(s, generator=gen).to(dev) for s in shapes]
    targets[0][0, 0, 0, :3] = images[0][0, 0, 0, :3]  # exact zeros: sign(0) = 0
    grads = [torch.full_like(t, float("nan")) for t in images]
    loss = torch.full((), float("nan"), device=dev)
    rasterizer.l1_loss_grad(images, targets, grads, loss)
    want = sum((i - t).abs().mean() for i, t in zip(images, targets))
    assert abs(loss.item() - want.item()) <= 1e-5 * want.item()
    for i, t, g in zip(images, targets, grads):
        assert torch.equal(g, torch.sign(i - t) * (1.0 / i.numel()))


@pytest.mark.parametrize("mode", [1, 3])
def test_backward_in_two_phases(rasterizer, mode):
    """vetr_backward_phase: the per-fragment kernels and the per-point pass as two calls give what one call gives."""
    import torch

    sc = scenes.tiny_scene(n=3000, n_views=2, seed=31, crop=True)
    params = default_params(render_mode=mode)
    dev = rasterizer.device
    from vet_b200.render import scene_to_device

    tensors = scene_to_device(sc, dev)
    out = rasterizer.forward(*tensors, sc.views, params)
    gen = torch.Generator(device="cpu").manual_seed(4)
    grads = [torch.randn(c.shape, generator=gen).to(dev) for c in out["color"]]
    whole = rasterizer.backward_raw(grads)
    first = rasterizer.backward_raw(grads, phases=1)
    if mode == 1:  # nothing of the position / camera gradients exists after the first phase
        assert float(first["points"].abs().sum()) == 0.0 and float(first["pose"].abs().sum()) == 0.0
        assert torch.equal(first["desc"], whole["desc"]) or torch.allclose(first["desc"], whole["desc"], rtol=1e-4, atol=1e-6)
    both = rasterizer.backward_raw(grads, accum=first, phases=2)
    torch.cuda.synchronize()
    assert torch.equal(both["points"], whole["points"])  # one owner per point, fixed summation order
    assert torch.equal(both["pose_count"], whole["pose_count"])
    assert torch.allclose(both["pose"], whole["pose"], rtol=1e-9, atol=1e-12)  # f64 atomics over thread blocks
    for k in ("desc", "conf", "background", "intrinsics"):
        assert torch.allclose(both[k], whole[k], rtol=1e-4, atol=1e-6), k  # float atomics in no fixed order
