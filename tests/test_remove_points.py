"""Point removal (NeuralScene::RemovePoints, data/NeuralScene.cpp:1156-1239): the host restatement by hand, and the device
plan + gather (through the C ABI) against it, bit for bit."""
import numpy as np
import pytest
import torch

from oracle import oracle as O


def test_restatement_by_hand():
    tex = np.arange(12, dtype=np.float32).reshape(2, 6)        # [C, N]
    pos = np.arange(24, dtype=np.float32).reshape(6, 4)        # [N, 4]
    new_index, (t,), (p,) = O.remove_points(6, [4, 1, 4], [tex], [pos])
    assert new_index.tolist() == [0, -1, 1, 2, -1, 3]
    assert np.array_equal(t, tex[:, [0, 2, 3, 5]]) and np.array_equal(p, pos[[0, 2, 3, 5]])
    new_index, (t,), _ = O.remove_points(6, [], [tex])
    assert new_index.tolist() == list(range(6)) and np.array_equal(t, tex)
    new_index, (t,), _ = O.remove_points(6, range(6), [tex])
    assert (new_index == -1).all() and t.shape == (2, 0)


def _case(rng, n, m, channels=4):
    remove = rng.integers(0, n, size=m).astype(np.int64)       # with duplicates
    texture = rng.standard_normal((channels, n)).astype(np.float32)
    conf = rng.uniform(size=(1, n)).astype(np.float32)
    moments = rng.standard_normal((2, channels, n)).astype(np.float32)
    position = rng.standard_normal((n, 4)).astype(np.float32)
    index = np.arange(n, dtype=np.int32)[:, None]
    return remove, [texture, conf, moments], [position, index]


@pytest.mark.gpu
@pytest.mark.parametrize("n,m", [(1, 0), (1, 1), (5000, 0), (5000, 700), (4097, 4097 * 3), (1_000_003, 250_000)])
def test_gpu_matches_restatement(n, m):
    from vet_b200.render import Rasterizer

    rng = np.random.default_rng(n + m)
    remove, last, first = _case(rng, n, m)
    if n <= 5000:
        ref_index, ref_last, ref_first = O.remove_points(n, remove, last, first)
    else:  # the host loop of the restatement is slow in Python at this size: the same keep list with numpy
        keep = np.setdiff1d(np.arange(n), remove)
        ref_index = np.full(n, -1, np.int32)
        ref_index[keep] = np.arange(len(keep), dtype=np.int32)
        ref_last, ref_first = [a[..., keep] for a in last], [a[keep] for a in first]
    rast = Rasterizer(0)
    t = lambda a: torch.from_numpy(a).cuda()
    new_index, got_last, got_first = rast.remove_points(n, t(remove), [t(a) for a in last], [t(a) for a in first])
    assert np.array_equal(new_index.cpu().numpy(), ref_index)
    for g, r in zip(got_last + got_first, ref_last + ref_first):
        assert tuple(g.shape) == r.shape and np.array_equal(g.cpu().numpy(), r)
    rast.close()


@pytest.mark.gpu
def test_gpu_rejects_indices_outside_the_cloud():
    from vet_b200 import _lib
    from vet_b200.render import Rasterizer

    rast = Rasterizer(0)
    for bad in ([5, 100], [-1]):
        with pytest.raises(_lib.VetrError) as ei:
            rast.remove_points(100, torch.tensor(bad, dtype=torch.int64, device="cuda"))
        assert ei.value.status == _lib.E_INVALID_ARG
    rast.close()
