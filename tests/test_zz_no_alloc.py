"""vetr_scan_counts_static: the forward pass's scan as a stand-alone call that allocates no device memory (for hosts that
must not allocate while rendering: its scratch is a fixed array inside the library).  Checked against a numpy prefix sum
of the same counts and against what the regular entry point, vetr_forward, leaves in its list buffers, on two calls in a
row with different inputs (the second call reuses the shared scratch array and must not see the first call's contents)."""
import ctypes as C

import numpy as np
import pytest

from vet_b200 import _lib as L
from vet_b200 import scenes
from vet_b200.render import default_params, scene_to_device

pytestmark = pytest.mark.gpu

ITEM_UNITS, ITEM_PIXELS = 512, 128  # work units of one item (1 per fragment, 4 per pixel) and the pixels that allows


def _forward_lists(rast, scene, params):
    import torch

    tensors = scene_to_device(scene, rast.device)
    rast.forward(*tensors, scene.views, params)
    torch.cuda.synchronize()
    lists = rast._saved["groups"][0][2]
    return lists


def _check(rast, scene, params):
    import torch

    lists = _forward_lists(rast, scene, params)
    counts = lists.counts.clone()
    n = counts.numel()
    ends = torch.full((n,), -7, dtype=torch.int32, device=rast.device)
    status = torch.full((4,), -7, dtype=torch.int32, device=rast.device)
    items = torch.full_like(lists.items, -7)
    rc = L.lib().vetr_scan_counts_static(0, None, C.c_void_p(counts.data_ptr()), n, lists.capacity, C.c_void_p(ends.data_ptr()),
                                         C.c_void_p(status.data_ptr()), C.c_void_p(items.data_ptr()), items.numel())
    assert rc == L.OK
    torch.cuda.synchronize()
    # independent of the library: the offsets are the exclusive prefix sum of the counts, the status words hold the total
    # and the longest list, and the work-item table is ascending, starts at pixel 0 and ends at the pixel count
    c = counts.cpu().numpy().astype(np.int64)
    np.testing.assert_array_equal(ends.cpu().numpy(), np.cumsum(c) - c)
    st = status.cpu().numpy()
    assert st[0] == c.sum() and st[1] == 0 and st[2] == c.max()
    table = items[:int(st[3]) + 1].cpu().numpy()
    assert table[0] == 0 and table[-1] == n and np.all(np.diff(table) >= 0)
    # every item holds at most ITEM_PIXELS pixels, and fewer than ITEM_UNITS fragments beyond its first pixel's list
    first = np.minimum(table[:-1], n - 1)
    frag_end = np.concatenate([np.cumsum(c), [c.sum()]])
    beyond_first = frag_end[np.maximum(table[1:], 1) - 1] - frag_end[first]
    assert np.all(np.diff(table) <= ITEM_PIXELS) and np.all(beyond_first < ITEM_UNITS)
    # vetr_forward's collection pass has advanced its offsets from list starts to list ends: ends = starts + counts
    np.testing.assert_array_equal((ends + counts).cpu().numpy(), lists.ends.cpu().numpy())
    st, st_ref = status.cpu().numpy(), lists.status.cpu().numpy()
    np.testing.assert_array_equal(st, st_ref)
    k = int(st[3])
    np.testing.assert_array_equal(items[:k + 1].cpu().numpy(), lists.items[:k + 1].cpu().numpy())
    return int(st[0])


def test_static_scan_matches_forward_twice(rasterizer):
    f1 = _check(rasterizer, scenes.tiny_scene(n=40000, w=96, h=64, n_views=2, seed=11),
                default_params(drop_out_points_by_radius=0))
    f2 = _check(rasterizer, scenes.tiny_scene(n=3000, w=64, h=48, n_views=3, seed=12), default_params(render_mode=3))
    assert f1 > 0 and f2 > 0 and f1 != f2


def test_static_scan_rejects_sizes_beyond_its_scratch(rasterizer):
    import torch

    t = torch.zeros(16, dtype=torch.int32, device=rasterizer.device)
    p = C.c_void_p(t.data_ptr())
    too_many = 16384 * 4096 + 1
    assert L.lib().vetr_scan_counts_static(0, None, p, too_many, 0, p, p, p, 1 << 40) == L.E_TOO_LARGE
    assert L.lib().vetr_scan_counts_static(0, None, p, 16, 0, p, p, p, 0) == L.E_INVALID_ARG  # item table too small
    assert L.lib().vetr_scan_counts_static(0, None, None, 16, 0, p, p, p, 64) == L.E_INVALID_ARG
