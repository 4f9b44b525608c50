"""The libtorch operator's point-cloud surgery that is built from libtorch operators, on CPU tensors (the same code runs on
CUDA tensors, where torch's own kernels do the sorting and copying): adding points (NeuralScene::AddNewPoints,
data/NeuralScene.cpp:1013-1074 with NeuralTexture.cpp:118-158, my_adam.cpp:137-170, SceneData.cpp:554-597, 669-691) and the
order a cloud is given when a scene is prepared (SceneData.cpp:105-108, 1005-1018), each against a numpy restatement of
the reference's sequence."""
import os

import numpy as np
import pytest
import torch

from vet_b200 import scenes

SHIM = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "vet_b200", "libvetr_torch.so")


@pytest.fixture(scope="module")
def ops():
    if not os.path.exists(SHIM):
        pytest.skip("libvetr_torch.so is not built (python -m vet_b200.build --shim)")
    torch.ops.load_library(SHIM)
    return torch.ops.vetr


def test_add_new_points_matches_the_reference_sequence(ops):
    rng = np.random.default_rng(3)
    n, m, C = 1000, 37, 4
    position = rng.normal(size=(n, 4)).astype(np.float32)
    texture = rng.normal(size=(C, n)).astype(np.float32)
    confidence = rng.uniform(size=(1, n)).astype(np.float32)
    exp_avg, exp_avg_sq = rng.normal(size=(C, n)).astype(np.float32), rng.uniform(size=(C, n)).astype(np.float32)
    new_xyz = rng.normal(size=(m, 3)).astype(np.float32)
    u = rng.uniform(1e-3, 1.0, size=n + m)
    distance = rng.uniform(0.01, 0.1, size=n + m).astype(np.float32)

    t_tex, t_conf, t_pos = torch.from_numpy(texture.copy()), torch.from_numpy(confidence.copy()), torch.from_numpy(position.copy())
    t_tex.requires_grad_(True)  # a parameter keeps its identity: it is resized in place
    t_idx = torch.arange(n, dtype=torch.int32).reshape(n, 1)
    state = [torch.from_numpy(exp_avg.copy()), torch.from_numpy(exp_avg_sq.copy())]
    total = ops.add_new_points(t_tex, t_conf, t_pos, t_idx, torch.from_numpy(new_xyz), state, False, torch.from_numpy(u),
                               torch.from_numpy(distance))
    assert total == n + m
    # texture: new columns 0.5; confidence and optimizer moments: new columns 0 (ResizeAndFill, appendToInternalState)
    np.testing.assert_array_equal(t_tex.detach().numpy(), np.concatenate([texture, np.full((C, m), 0.5, np.float32)], 1))
    np.testing.assert_array_equal(t_conf.numpy(), np.concatenate([confidence, np.zeros((1, m), np.float32)], 1))
    np.testing.assert_array_equal(state[0].numpy(), np.concatenate([exp_avg, np.zeros((C, m), np.float32)], 1))
    np.testing.assert_array_equal(state[1].numpy(), np.concatenate([exp_avg_sq, np.zeros((C, m), np.float32)], 1))
    assert t_tex.requires_grad and t_tex.shape == (C, n + m)
    # positions appended; radius column of the WHOLE cloud = neighbour distance x sqrt(1 / u) (ComputeRadius); index = iota
    want_xyz = np.concatenate([position[:, :3], new_xyz], 0)
    want_r = distance * np.sqrt(1.0 / u).astype(np.float32)
    np.testing.assert_array_equal(t_pos.numpy()[:, :3], want_xyz)
    np.testing.assert_array_equal(t_pos.numpy()[:, 3], want_r)
    np.testing.assert_array_equal(t_idx.numpy()[:, 0], np.arange(n + m, dtype=np.int32))


def test_add_new_points_random_init_and_empty(ops):
    n, C = 50, 3
    t_tex, t_conf = torch.zeros(C, n), torch.zeros(1, n)
    t_pos, t_idx = torch.zeros(n, 4), torch.arange(n, dtype=torch.int32).reshape(n, 1)
    torch.manual_seed(0)
    ops.add_new_points(t_tex, t_conf, t_pos, t_idx, torch.ones(200, 3), [], True, None, torch.ones(n + 200))
    new = t_tex[:, n:]
    assert new.shape == (C, 200) and float(new.min()) >= -1.0 and float(new.max()) < 1.0 and float(new.std()) > 0.3  # U(-1, 1)
    assert float(t_pos[:, 3].min()) >= 1.0  # distance 1 x sqrt(1 / u), u in (0, 1]
    before = t_pos.clone()
    assert ops.add_new_points(t_tex, t_conf, t_pos, t_idx, torch.zeros(0, 3), [], False, torch.ones(n + 200), before[:, 3].clone()) == n + 200
    np.testing.assert_array_equal(t_pos.numpy(), before.numpy())


def test_scene_preparation_order(ops):
    rng = np.random.default_rng(11)
    n = 5000  # not a multiple of 256: a shorter last block
    xyz = rng.normal(size=(n, 3)).astype(np.float32)
    xyz[100:200] = xyz[0:100]  # equal positions: equal codes, kept in their original order (stable)
    # Morton order + block shuffle against the generator of the synthetic scenes (the same block permutation)
    want = scenes.morton_block_order(xyz.astype(np.float64), np.random.default_rng(5))
    block_perm = np.random.default_rng(5).permutation((n + 255) // 256)
    morton = ops.morton_order(torch.from_numpy(xyz))
    shuffle = ops.random_block_shuffle(n, 256, torch.from_numpy(block_perm))
    np.testing.assert_array_equal(morton[shuffle].numpy(), want)
    assert sorted(shuffle.tolist()) == list(range(n))
    # SortBlocksByRadius: ascending inside every full block of 256, the tail untouched
    radius = rng.uniform(size=n).astype(np.float32)
    order = ops.sort_blocks_by_radius(torch.from_numpy(radius), 256).numpy()
    nb = n // 256
    for b in range(nb):
        blk = order[b * 256:(b + 1) * 256]
        assert sorted(blk.tolist()) == list(range(b * 256, (b + 1) * 256)) and np.all(np.diff(radius[blk]) >= 0)
    np.testing.assert_array_equal(order[nb * 256:], np.arange(nb * 256, n))
    # applying an order moves every per-point tensor together and rebuilds the index
    C = 4
    tex, conf = rng.normal(size=(C, n)).astype(np.float32), rng.uniform(size=(1, n)).astype(np.float32)
    pos = np.concatenate([xyz, radius[:, None]], 1)
    mom = rng.normal(size=(C, n)).astype(np.float32)
    t = [torch.from_numpy(a.copy()) for a in (tex, conf, pos, mom)]
    idx = torch.arange(n, dtype=torch.int32).reshape(n, 1)
    ops.apply_point_order(t[0], t[1], t[2], idx, torch.from_numpy(want.copy()), [t[3]])
    np.testing.assert_array_equal(t[0].numpy(), tex[:, want])
    np.testing.assert_array_equal(t[1].numpy(), conf[:, want])
    np.testing.assert_array_equal(t[2].numpy(), pos[want])
    np.testing.assert_array_equal(t[3].numpy(), mom[:, want])
    np.testing.assert_array_equal(idx.numpy()[:, 0], np.arange(n))
