"""Drop-out radius (SceneData::ComputeRadius, data/SceneData.cpp:554-597): the all-pairs restatement against hand-computed
cases on the CPU, and the grid search on the GPU (through the C ABI) against the restatement, bit for bit."""
import numpy as np
import pytest
import torch

from oracle import oracle as O
from vet_b200 import scenes


def _lattice(m, spacing=1.0):
    ax = np.arange(m, dtype=np.float32) * np.float32(spacing)
    return np.stack(np.meshgrid(ax, ax, ax, indexing="ij"), -1).reshape(-1, 3)


def test_lattice_by_hand():
    g = _lattice(5)
    r4, r7 = O.knn_radius(g, 4).reshape(5, 5, 5), O.knn_radius(g, 7).reshape(5, 5, 5)
    assert r4[2, 2, 2] == 1.0          # six neighbours at distance 1
    assert r4[0, 0, 0] == np.float32(np.sqrt(np.float32(2)))  # a corner: three at 1, then sqrt 2
    assert r4[0, 2, 2] == 1.0          # a face centre: five at 1
    assert r7[2, 2, 2] == np.float32(np.sqrt(np.float32(2)))  # the seventh is a face diagonal


def test_small_clouds_and_duplicates():
    p = np.array([[0, 0, 0], [3, 0, 0], [0, 4, 0]], np.float32)
    assert np.array_equal(O.knn_radius(p, 4), np.array([4, 5, 5], np.float32))  # fewer than k + 1 points: the farthest
    assert np.array_equal(O.knn_radius(p, 1), np.array([3, 3, 4], np.float32))
    assert np.array_equal(O.knn_radius(p[:1], 4), np.zeros(1, np.float32))
    q = np.repeat(np.array([[1, 2, 3]], np.float32), 7, 0)
    assert np.array_equal(O.knn_radius(q, 4), np.zeros(7, np.float32))  # coincident points
    q = np.concatenate([q[:3], [[1, 2, 5]]]).astype(np.float32)
    assert np.array_equal(O.knn_radius(q, 2), np.array([0, 0, 0, 2], np.float32))
    assert np.array_equal(O.knn_radius(q, 3), np.array([2, 2, 2, 2], np.float32))


def test_stride_and_fourth_column_ignored():
    rng = np.random.default_rng(0)
    p4 = rng.standard_normal((300, 4)).astype(np.float32)
    assert np.array_equal(O.knn_radius(p4, 4), O.knn_radius(np.ascontiguousarray(p4[:, :3]), 4))


# ---------------------------------------------------------------------------------------------------------
# CUDA


def _gpu(xyz, k=4, **kw):
    from vet_b200.render import Rasterizer

    rast = Rasterizer(0)
    out = rast.knn_radius(torch.from_numpy(np.ascontiguousarray(xyz)).cuda(), k, **kw)
    res = out.cpu().numpy()
    rast.close()
    return res


def _clouds():
    rng = np.random.default_rng(3)
    sc = scenes.config_planar(12000, 64, 64, 50.0, seed=9)  # planes + 5 % isolated points in a large box
    yield "planes and outliers", sc.position[:, :3]
    yield "cube surface", scenes.config_plumbing(8000, 64).position[:, :3]
    u = rng.uniform(-1, 1, size=(6000, 3)).astype(np.float32)
    u[:500] = np.round(u[:500] * 8) / 8          # lattice points: many equal distances
    u[500:700] = u[:200]                          # exact duplicates
    yield "uniform with ties and duplicates", u
    far = np.concatenate([rng.normal(0, 0.01, size=(3000, 3)), rng.normal(0, 0.01, size=(3000, 3)) + 500.0,
                          [[250.0, 250.0, -900.0]]]).astype(np.float32)
    yield "two far clusters and a lone point", far
    yield "a line", np.stack([np.linspace(-5, 5, 4000), np.zeros(4000), np.full(4000, 2.0)], -1).astype(np.float32)
    yield "offset far from the origin", (rng.uniform(0, 1, size=(5000, 3)) + 4096.0).astype(np.float32)


def test_grid_search_equals_all_pairs():
    """The restatement's uniform-grid search (the timed CPU baseline of this row) against all pairs, bit for bit."""
    for name, xyz in _clouds():
        for k in (1, 4, 16):
            assert np.array_equal(O.knn_radius(xyz, k, grid=True), O.knn_radius(xyz, k)), (name, k)
    p = np.array([[0, 0, 0], [3, 0, 0], [0, 4, 0]], np.float32)
    assert np.array_equal(O.knn_radius(p, 4, grid=True), np.array([4, 5, 5], np.float32))
    assert np.array_equal(O.knn_radius(np.repeat(p[1:2], 9, 0), 4, grid=True), np.zeros(9, np.float32))
    assert O.knn_radius(np.zeros((0, 3), np.float32), 4, grid=True).shape == (0,)


@pytest.mark.gpu
def test_gpu_matches_all_pairs_bit_for_bit():
    for name, xyz in _clouds():
        for k in (1, 4, 8, 16):
            ref = O.knn_radius(xyz, k)
            got = _gpu(xyz, k)
            assert np.array_equal(got, ref), (name, k, int((got != ref).sum()))


@pytest.mark.gpu
def test_gpu_small_and_degenerate_clouds():
    p = np.array([[0, 0, 0], [3, 0, 0], [0, 4, 0]], np.float32)
    assert np.array_equal(_gpu(p, 4), np.array([4, 5, 5], np.float32))
    assert np.array_equal(_gpu(p[:1], 4), np.zeros(1, np.float32))
    assert np.array_equal(_gpu(np.repeat(p[1:2], 50, 0), 4), np.zeros(50, np.float32))
    assert _gpu(np.zeros((0, 3), np.float32), 4).shape == (0,)
    q = np.concatenate([np.repeat(p[1:2], 3, 0), [[3, 0, 2]]]).astype(np.float32)
    assert np.array_equal(_gpu(q, 3), np.array([2, 2, 2, 2], np.float32))


@pytest.mark.gpu
def test_gpu_in_place_radius_column_and_errors():
    from vet_b200 import _lib
    from vet_b200.render import Rasterizer

    sc = scenes.config_planar(5000, 64, 64, 50.0, seed=2)
    ref = O.knn_radius(sc.position[:, :3], 4)
    pos = torch.from_numpy(sc.position.copy()).cuda()
    rast = Rasterizer(0)
    rast.knn_radius(pos, 4, out="w")
    got = pos.cpu().numpy()
    assert np.array_equal(got[:, 3], ref) and np.array_equal(got[:, :3], sc.position[:, :3])
    with pytest.raises(_lib.VetrError) as ei:
        rast.knn_radius(pos, 17)
    assert ei.value.status == _lib.E_INVALID_ARG
    bad = pos.clone()
    bad[7, 1] = float("nan")
    with pytest.raises(_lib.VetrError) as ei:
        rast.knn_radius(bad, 4)
    assert ei.value.status == _lib.E_INVALID_ARG
    rast.close()


@pytest.mark.gpu
def test_gpu_full_size_properties():
    """At sizes the all-pairs restatement cannot reach: a lattice's radius is known in closed form, and the result must
    not depend on the order of the points."""
    g = _lattice(120, 0.25)                       # 1.73 M points
    r = _gpu(g, 4).reshape(120, 120, 120)
    assert np.all(r[1:-1, 1:-1, 1:-1] == 0.25)    # interior: six neighbours at the spacing
    assert r[0, 0, 0] == np.float32(np.sqrt(np.float32(0.125)))
    sc = scenes.config_planar(1_000_000, 64, 64, 50.0, seed=4)
    xyz = sc.position[:, :3]
    perm = np.random.default_rng(1).permutation(len(xyz))
    a, b = _gpu(xyz, 4), _gpu(xyz[perm], 4)
    assert np.array_equal(a[perm], b)
    sub = np.random.default_rng(2).choice(len(xyz), 200, replace=False)   # spot check against all pairs of those points
    d2 = ((xyz[sub, None, :] - xyz[None, :, :]) ** 2)
    d2 = (d2[..., 0] + d2[..., 1]) + d2[..., 2]
    assert np.array_equal(a[sub], np.sqrt(np.partition(d2, 4, axis=1)[:, 4]))
