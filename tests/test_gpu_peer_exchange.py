"""vetr_exchange_finalize: the sum over ranks + epilogue in one kernel over peer memory.

On one GPU the ranks are emulated: every "rank" has its own raw and output buffer on the same device and the kernel runs
once per rank, one after the other (it waits on nothing, so this is exact).  With two or more GPUs a second test runs real
ranks as child processes over torch symmetric memory and compares with the all-reduce + epilogue path.
"""
import ctypes as C
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _reference(raws, channels, n_tex, n):
    """float32 sums in rank order, then the epilogue of vetr_finalize_gradients."""
    tot = raws[0].copy()
    for r in raws[1:]:
        tot = tot + r
    desc = tot[: 4 * n_tex].reshape(n_tex, 4)
    pts = tot[4 * n_tex: 4 * n_tex + 4 * n].reshape(n, 4).copy()
    conf = tot[4 * n_tex + 4 * n:]
    cnt = pts[:, 3].copy()
    hit = cnt > 0
    pts[hit, :3] = pts[hit, :3] / cnt[hit, None]
    pts[:, 3] = 0
    return desc[:, :channels].T.copy(), pts, conf


@pytest.mark.parametrize("world,channels,n_tex,n", [(2, 4, 1000, 1000), (3, 3, 1237, 911), (8, 4, 5, 3), (1, 4, 64, 64)])
def test_emulated_ranks(world, channels, n_tex, n):
    from vet_b200 import _lib as L
    from vet_b200.render import Rasterizer

    lib = L.lib()
    rast = Rasterizer(0)
    dev = torch.device("cuda", 0)
    raw_floats = int(lib.vetr_exchange_raw_floats(n_tex, n))
    out_floats = int(lib.vetr_exchange_out_floats(channels, n_tex, n))
    assert raw_floats == 5 * n_tex + 4 * n
    rng = np.random.default_rng(world * 1000 + n)
    raws = []
    for k in range(world):
        r = rng.standard_normal(raw_floats).astype(np.float32)
        counts = rng.integers(0, 3, n).astype(np.float32)
        r[4 * n_tex: 4 * n_tex + 4 * n].reshape(n, 4)[:, 3] = counts
        raws.append(r)
    d_raw = [torch.from_numpy(r).to(dev) for r in raws]
    d_out = [torch.full((out_floats,), float("nan"), device=dev) for _ in range(world)]
    for rank in range(world):
        ex = L.Exchange()
        ex.rank, ex.world = rank, world
        for k in range(world):
            ex.raw[k] = d_raw[k].data_ptr()
            ex.out[k] = d_out[k].data_ptr()
        rc = lib.vetr_exchange_finalize(rast._ctx, C.byref(ex), channels, n_tex, n)
        assert rc == L.OK
    torch.cuda.synchronize()
    tex, pts, conf = _reference(raws, channels, n_tex, n)
    p0 = (channels * n_tex + 3) // 4 * 4
    for k in range(world):
        o = d_out[k].cpu().numpy()
        np.testing.assert_array_equal(o[: channels * n_tex].reshape(channels, n_tex), tex)
        np.testing.assert_array_equal(o[p0: p0 + 4 * n].reshape(n, 4), pts)
        np.testing.assert_array_equal(o[p0 + 4 * n:], conf)


def test_invalid_arguments():
    from vet_b200 import _lib as L
    from vet_b200.render import Rasterizer

    lib = L.lib()
    rast = Rasterizer(0)
    buf = torch.zeros(1024, device="cuda")
    ex = L.Exchange()
    ex.rank, ex.world = 0, 1
    ex.raw[0], ex.out[0] = buf.data_ptr(), buf.data_ptr()
    assert lib.vetr_exchange_finalize(rast._ctx, C.byref(ex), 5, 10, 10) == L.E_INVALID_ARG
    ex.rank = 1
    assert lib.vetr_exchange_finalize(rast._ctx, C.byref(ex), 4, 10, 10) == L.E_INVALID_ARG
    ex.rank, ex.world = 0, 17
    assert lib.vetr_exchange_finalize(rast._ctx, C.byref(ex), 4, 10, 10) == L.E_INVALID_ARG
    ex.world = 1
    ex.raw[0] = buf.data_ptr() + 4
    assert lib.vetr_exchange_finalize(rast._ctx, C.byref(ex), 4, 10, 10) == L.E_INVALID_ARG
    ex.raw[0] = 0
    assert lib.vetr_exchange_finalize(rast._ctx, C.byref(ex), 4, 10, 10) == L.E_INVALID_ARG


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_real_ranks():
    env = dict(os.environ, MASTER_ADDR="127.0.0.1", NCCL_NVLS_ENABLE="0")
    cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", "--nproc-per-node", "2", "--master-addr", "127.0.0.1",
           "--master-port", "29533", os.path.join(ROOT, "tests", "peer_exchange_worker.py")]
    res = subprocess.run(cmd, env=env, cwd=ROOT, capture_output=True, text=True, timeout=600)
    assert res.returncode == 0, res.stdout[-3000:] + res.stderr[-3000:]
    assert "PEER_EXCHANGE_OK" in res.stdout
