"""Error-grid rasterisation (FillSceneGridWithLossRasterize, RenderForward.cu:639-791): the CPU restatement against hand
computed cases, and the CUDA kernel (through the C ABI) against the restatement."""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from vet_b200 import scenes


def _camera_scene(w=256, h=256, f=200.0):
    """Camera at the origin looking down +z (identity world -> camera pose), principal point at the image centre."""
    pose = np.array([[0, 0, 0, 1, 0, 0, 0, 0]], np.float64)
    intr = scenes.pinhole_intrinsics(f, f, w / 2, h / 2)[None].astype(np.float32)
    z = np.zeros((1, 4), np.float32)
    return scenes.Scene(position=z, index=np.zeros(1, np.int32), texture=np.zeros((4, 1), np.float32),
                        confidence=np.zeros(1, np.float32), background=np.zeros(4, np.float32), poses=pose,
                        intrinsics=intr, views=[scenes.View(w, h)])


def test_axis_aligned_cell_by_hand():
    sc = _camera_scene()
    # unit cube in front of the camera: the front face (z = 2) projects to the square [78, 178]^2, the back face lies inside
    bb_min = np.array([[-0.5, -0.5, 2.0]], np.float32)
    bb_len = np.array([[1.0, 1.0, 1.0]], np.float32)
    loss = np.ones((3, 256, 256), np.float32) * np.array([1.0, -2.0, 0.5], np.float32)[:, None, None]
    value, count = O.grid_loss(sc, sc.views[0], bb_min, bb_len, loss)
    assert count[0] == 100 * 100  # x_size = int(178 - 78): pixels 78..177 in both directions
    assert value[0] == pytest.approx(3.5 * 100 * 100, rel=1e-6)


def test_border_clamp_behind_camera_and_offscreen():
    sc = _camera_scene()
    bb_min = np.array([[-4.0, -0.5, 2.0],    # wide box: its rectangle is clamped to the 32-pixel border
                       [-0.5, -0.5, -0.5],   # straddles the camera plane: ignored as a whole
                       [10.0, 10.0, 2.0],    # projects outside the image
                       [-1.2, -1.2, 2.0]],   # entirely inside the left/top border strip
                      np.float32)
    bb_len = np.array([[8.0, 1.0, 1.0], [1.0, 1.0, 1.0], [1.0, 1.0, 1.0], [0.1, 0.1, 0.1]], np.float32)
    loss = np.ones((1, 256, 256), np.float32)
    value, count = O.grid_loss(sc, sc.views[0], bb_min, bb_len, loss)
    assert count[0] == (224 - 32) * 100  # x clamped to [32, 224), y = 78..177
    assert count[1] == 0 and count[2] == 0 and count[3] == 0
    assert value[0] == count[0]


def _random_grid(rng, n_cells, box=10.0):
    bb_min = rng.uniform(-box, box, size=(n_cells, 3)).astype(np.float32)
    bb_len = rng.uniform(0.2, 2.5, size=(n_cells, 3)).astype(np.float32)
    return bb_min, bb_len


def test_accumulates_over_calls():
    sc = scenes.config_planar(100, 320, 240, 220.0, n_views=2, seed=5)
    rng = np.random.default_rng(0)
    bb_min, bb_len = _random_grid(rng, 300)
    loss = rng.standard_normal((3, 240, 320)).astype(np.float32)
    v0, c0 = O.grid_loss(sc, sc.views[0], bb_min, bb_len, loss)
    v1, c1 = O.grid_loss(sc, sc.views[1], bb_min, bb_len, loss)
    assert c0.sum() > 0 and c1.sum() > 0 and not np.array_equal(c0, c1)
    assert (v0[c0 == 0] == 0).all()


@pytest.mark.gpu
@pytest.mark.parametrize("crop", [False, True])
def test_gpu_matches_oracle(crop):
    from vet_b200.render import Rasterizer

    w, h = 640, 480
    sc = scenes.config_planar(100, w, h, 450.0, n_views=3, seed=11)
    if crop:
        # crop transform + crop rotation as the training crops use them
        import math
        ang = 0.3
        for v in sc.views:
            v.crop = (0.9, 1.1, 12.0, -7.0, 0.0)
            v.rot = (math.cos(ang), -math.sin(ang), math.sin(ang), math.cos(ang))
    rng = np.random.default_rng(3)
    bb_min, bb_len = _random_grid(rng, 4000)
    loss = rng.standard_normal((3, h, w)).astype(np.float32)
    dev = torch.device("cuda", 0)
    rast = Rasterizer(0)
    value = torch.zeros(4000, dtype=torch.float32, device=dev)
    count = torch.zeros(4000, dtype=torch.int32, device=dev)
    ref_v = np.zeros(4000, np.float64)
    ref_c = np.zeros(4000, np.int64)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
    for view in sc.views:  # three images accumulate into the same grid
        rast.grid_loss(t(sc.poses), t(sc.intrinsics), view, t(bb_min), t(bb_len), t(loss), value, count)
        v, c = O.grid_loss(sc, view, bb_min, bb_len, loss)
        ref_v += v
        ref_c += c
    torch.cuda.synchronize()
    assert ref_c.sum() > 10000
    np.testing.assert_array_equal(count.cpu().numpy().astype(np.int64), ref_c)  # bit-exact coverage
    np.testing.assert_allclose(value.cpu().numpy(), ref_v, rtol=1e-5, atol=0)   # float sums of non-negative terms


@pytest.mark.gpu
def test_gpu_invalid_arguments():
    import ctypes as C
    from vet_b200 import _lib as L
    from vet_b200.render import Rasterizer

    rast = Rasterizer(0)
    dev = torch.device("cuda", 0)
    poses = torch.zeros(1, 8, dtype=torch.float64, device=dev)
    intr = torch.zeros(1, 13, device=dev)
    cams = L.Cameras(poses.data_ptr(), intr.data_ptr(), 1, 1)
    buf = torch.zeros(64, device=dev)
    cnt = torch.zeros(4, dtype=torch.int32, device=dev)
    view = L.View(64, 64, 0, 0, 0, (C.c_float * 5)(1, 1, 0, 0, 0), (C.c_float * 4)(1, 0, 0, 1))
    p = lambda t: C.c_void_p(t.data_ptr())
    lib = L.lib()
    assert lib.vetr_grid_loss(rast._ctx, C.byref(cams), C.byref(view), 20.0, 0, None, None, None, 3, None, None) == L.OK
    assert lib.vetr_grid_loss(rast._ctx, C.byref(cams), C.byref(view), 20.0, 4, None, p(buf), p(buf), 3, p(buf), p(cnt)) == L.E_INVALID_ARG
    view.image_index = 5
    assert lib.vetr_grid_loss(rast._ctx, C.byref(cams), C.byref(view), 20.0, 4, p(buf), p(buf), p(buf), 3, p(buf), p(cnt)) == L.E_INVALID_ARG
    view.image_index, view.camera_model = 0, 1
    assert lib.vetr_grid_loss(rast._ctx, C.byref(cams), C.byref(view), 20.0, 4, p(buf), p(buf), p(buf), 3, p(buf), p(cnt)) == L.E_UNSUPPORTED
