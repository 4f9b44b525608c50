"""View-sharded data parallelism on CPU ranks (gloo, world size 2): the sharding rule, the fused gradient buffer and
its all-reduce give the same sums as one process rendering the whole batch.  The per-rank renderer here is the CPU
oracle (no GPU in this test); the tested code is vet_b200.dist."""
import os
import socket

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import oracle as O
from tests import util
from vet_b200 import scenes
from vet_b200.dist import GradientBuffer, allreduce_gradients, shard_views


def _free_port():
    s = socket.socket()
    s.bind(("127.0.0.1", 0))
    port = s.getsockname()[1]
    s.close()
    return port


def _oracle_raw(scene, views, grads_of_view):
    """Raw gradient sums of a set of views, packed like the GPU path packs them."""
    o = O.Oracle()
    fwd = o.forward(scene, O.default_params(), views=views)
    grads = [np.stack([grads_of_view[v.image_index][l] for v in views]) for l in range(4)]
    return o.backward(grads), fwd


def _worker(rank, world, port, out_dir):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    scene = scenes.tiny_scene(n=1500, w=32, h=24, n_views=5, seed=13)
    rng = np.random.default_rng(99)
    sizes = O.level_sizes(32, 24, 4)
    grads_of_view = [[rng.standard_normal((scene.channels, h, w)).astype(np.float32) for (w, h) in sizes] for _ in range(5)]
    mine = shard_views(5, rank, world)
    b, _ = _oracle_raw(scene, [scene.views[i] for i in mine], grads_of_view)
    buf = GradientBuffer(scene.n, scene.texture.shape[1], "cpu")
    g = buf.as_accum(scene.channels, scene.poses.shape[0])
    g["desc"][:, :scene.channels] += torch.from_numpy(b["texture"].T.astype(np.float32))
    g["conf"] += torch.from_numpy(b["confidence"].astype(np.float32))
    g["points"][:, :3] += torch.from_numpy(b["points"].astype(np.float32))
    g["points"][:, 3] += torch.from_numpy(b["points_count"].astype(np.float32))
    g["background"] += torch.from_numpy(b["background"].astype(np.float32))
    g["pose"] += torch.from_numpy(b["pose"])
    g["pose_count"] += torch.from_numpy(b["pose_count"].astype(np.float32))
    allreduce_gradients(buf, g)
    if rank == 0:
        np.savez(os.path.join(out_dir, "reduced.npz"), flat=buf.flat.numpy(), background=g["background"].numpy(),
                 pose=g["pose"].numpy(), pose_count=g["pose_count"].numpy())
    dist.destroy_process_group()


def test_shard_views_partition():
    for world in (1, 2, 3, 8):
        seen = sorted(v for r in range(world) for v in shard_views(32, r, world))
        assert seen == list(range(32))
    assert shard_views(5, 1, 2) == [1, 3]


def test_two_ranks_equal_one_process(tmp_path):
    world = 2
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    got = np.load(tmp_path / "reduced.npz")
    scene = scenes.tiny_scene(n=1500, w=32, h=24, n_views=5, seed=13)
    rng = np.random.default_rng(99)
    sizes = O.level_sizes(32, 24, 4)
    grads_of_view = [[rng.standard_normal((scene.channels, h, w)).astype(np.float32) for (w, h) in sizes] for _ in range(5)]
    b, _ = _oracle_raw(scene, scene.views, grads_of_view)
    n, nt = scene.n, scene.texture.shape[1]
    flat = got["flat"]
    desc, points, conf = flat[:4 * nt].reshape(nt, 4), flat[4 * nt:4 * nt + 4 * n].reshape(n, 4), flat[4 * nt + 4 * n:]
    scale = lambda a: 1e-5 * max(1.0, float(np.abs(a).max()))
    np.testing.assert_allclose(desc[:, :scene.channels].T, b["texture"], atol=scale(b["texture"]))
    np.testing.assert_allclose(conf, b["confidence"], atol=scale(b["confidence"]))
    np.testing.assert_allclose(points[:, :3], b["points"], atol=scale(b["points"]))
    np.testing.assert_array_equal(points[:, 3], b["points_count"])
    np.testing.assert_allclose(got["background"], b["background"], atol=scale(b["background"]))
    np.testing.assert_allclose(got["pose"], b["pose"], rtol=1e-9, atol=1e-9)
    np.testing.assert_allclose(got["pose_count"], b["pose_count"], rtol=1e-6)


def test_views_to_ranks_by_cost():
    """bench.py's assignment of a batch's views to ranks for benchmark configuration 5: longest view first to the least
    loaded rank.  Every view is assigned once, the loads add up, and no rank exceeds the greedy bound (mean + largest)."""
    import bench

    rng = np.random.default_rng(4)
    for world in (1, 2, 4, 8):
        costs = rng.uniform(1.8, 4.6, size=32).tolist()
        mine, load = bench.balanced_assignment(costs, world)
        assert sorted(v for m in mine for v in m) == list(range(32))
        assert abs(sum(load) - sum(costs)) < 1e-9
        for m, l in zip(mine, load):
            assert abs(sum(costs[v] for v in m) - l) < 1e-9
        assert max(load) <= sum(costs) / world + max(costs) + 1e-9
    # equal costs: equal shares
    mine, load = bench.balanced_assignment([1.0] * 32, 8)
    assert [len(m) for m in mine] == [4] * 8


def test_algorithmic_bytes_of_a_launch():
    """The per-launch byte count bench.py divides by the measured time: forward 20 N per view + 36 F + 28 P, backward
    32 P + 44 F + 40 N + 80 N_t."""
    import bench

    N, F, P, Nt = 1000, 5000, 300, 700
    assert bench.algorithmic_bytes_per_launch(N, F, P, Nt, 1, False) == 20 * N + 36 * F + 28 * P
    assert bench.algorithmic_bytes_per_launch(N, F, 4 * P, Nt, 4, True) == 20 * N * 4 + 36 * F + 28 * 4 * P + 32 * 4 * P + 44 * F + 40 * N + 80 * Nt
