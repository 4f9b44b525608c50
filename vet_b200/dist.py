"""View-sharded data parallelism for the rasterizer (one process per GPU).

The reference has no multi-GPU code.  A training batch shards by view: the cloud, descriptors and cameras are
replicated, rank r renders the views {v : v mod world == r}, and the only exchange per step is the sum of the
point-parameter gradients.  They live in ONE fused fp32 buffer, so that one exchange moves them - PeerExchange: the sum
over the ranks and the epilogue as one kernel over NVLink peer memory; allreduce_gradients: one NCCL all-reduce:

    [ descriptor gradient  n_tex x 4 | position gradient + hit count  n x 4 | confidence gradient  n_tex ]

Hit counts travel with the sums because the reference averages position gradients by the number of hits
(rendering/PointRenderer.cu:1273-1280): the division has to come after the sum over ranks.  Pose-tangent gradients
and their counts (double / float, a few hundred bytes) are reduced separately.
"""
from __future__ import annotations

import ctypes as C
from typing import List, Optional

import torch
import torch.distributed as dist


def shard_views(n_views_total: int, rank: int, world: int) -> List[int]:
    """Indices of the batch's views that `rank` renders."""
    if not (0 <= rank < world):
        raise ValueError("rank out of range")
    return [v for v in range(n_views_total) if v % world == rank]


class GradientBuffer:
    """Fused accumulation buffer for the point-parameter gradients of one step."""

    def __init__(self, n: int, n_tex: int, device, flat: Optional[torch.Tensor] = None):
        self.n, self.n_tex = n, n_tex
        if flat is None:
            flat = torch.zeros(4 * n_tex + 4 * n + n_tex, dtype=torch.float32, device=device)
        assert flat.numel() == 4 * n_tex + 4 * n + n_tex and flat.dtype == torch.float32 and flat.is_contiguous()
        self.flat = flat
        self.desc = self.flat[: 4 * n_tex].view(n_tex, 4)
        self.points = self.flat[4 * n_tex: 4 * n_tex + 4 * n].view(n, 4)
        self.conf = self.flat[4 * n_tex + 4 * n:]
        assert self.points.data_ptr() % 16 == 0 and self.desc.data_ptr() % 16 == 0

    def zero_(self):
        self.flat.zero_()

    def as_accum(self, channels: int, n_img: int, want_pose: bool = True) -> dict:
        """The dict Rasterizer.backward_raw(accum=...) accumulates into; small per-step tensors are fresh."""
        dev = self.flat.device
        g = dict(desc=self.desc, points=self.points, conf=self.conf,
                 background=torch.zeros(channels, dtype=torch.float32, device=dev))
        if want_pose:
            g["pose"] = torch.zeros(n_img, 6, dtype=torch.float64, device=dev)
            g["pose_count"] = torch.zeros(n_img, dtype=torch.float32, device=dev)
        return g


def allreduce_gradients(buf: GradientBuffer, g: dict, group: Optional[dist.ProcessGroup] = None, async_op: bool = False):
    """Sums the fused point-parameter buffer and the small camera / background gradients over the ranks."""
    if not (dist.is_available() and dist.is_initialized()) or dist.get_world_size(group) == 1:
        return []
    works = [dist.all_reduce(buf.flat, group=group, async_op=async_op)]
    for key in ("background", "pose", "pose_count", "intrinsics", "intrinsics_count"):
        if g.get(key) is not None:
            works.append(dist.all_reduce(g[key], group=group, async_op=async_op))
    return works if async_op else []


class PeerExchange:
    """Sum over the ranks + epilogue of the point-parameter gradients in ONE kernel over NVLink peer memory
    (vetr_exchange_finalize) instead of an NCCL all-reduce followed by the epilogue kernels.

    The raw buffer (what backward accumulates into) and the result buffer of every rank are allocated as torch
    symmetric memory, so that every rank holds a pointer to every other rank's copy.  `run` enqueues, on the current
    stream: all-reduce(pose gradient) -> the exchange kernel -> all-reduce(pose count, background).  The two small
    NCCL collectives are needed anyway and are what orders the kernel after all ranks' backward kernels and its
    consumers after all ranks' exchange kernels; the kernel itself waits on nothing.
    """

    def __init__(self, rast, n: int, n_tex: int, channels: int, device, group=None, multicast: Optional[bool] = None):
        import torch.distributed._symmetric_memory as symm
        from . import _lib as L

        self.rast, self.n, self.n_tex, self.channels = rast, n, n_tex, channels
        self.group = group if group is not None else dist.group.WORLD
        lib = L.lib()
        raw_floats = int(lib.vetr_exchange_raw_floats(n_tex, n))
        out_floats = int(lib.vetr_exchange_out_floats(channels, n_tex, n))
        self.raw = symm.empty(raw_floats, dtype=torch.float32, device=device)
        self.out = symm.empty(out_floats, dtype=torch.float32, device=device)
        self.raw.zero_()
        h_raw = symm.rendezvous(self.raw, self.group)
        h_out = symm.rendezvous(self.out, self.group)
        self.rank, self.world = h_raw.rank, h_raw.world_size
        self.c = L.Exchange()
        self.c.rank, self.c.world = self.rank, self.world
        for k in range(self.world):
            self.c.raw[k] = int(h_raw.buffer_ptrs[k])
            self.c.out[k] = int(h_out.buffer_ptrs[k])
        # NVSwitch multicast objects over both buffers (0 where the platform has none): the sum then happens in the switch
        mc_raw, mc_out = int(getattr(h_raw, "multicast_ptr", 0) or 0), int(getattr(h_out, "multicast_ptr", 0) or 0)
        if multicast is None:
            # measured on 8 x B200: with 2 ranks plain peer loads / stores are faster (0.44 vs 0.76 ms for 8 M points), with
            # 8 ranks the switch-side sum is (0.64 vs 0.85 ms)
            multicast = self.world > 2
        self.multicast = bool(multicast and self.world > 1 and mc_raw and mc_out)
        if self.multicast:
            self.c.raw_multicast, self.c.out_multicast = mc_raw, mc_out
        self._handles = (h_raw, h_out)
        self.buffer = GradientBuffer(n, n_tex, device, flat=self.raw)
        self._token = torch.zeros(1, dtype=torch.float32, device=device)
        self._side = None
        self.ctas_per_sm = 4  # thread blocks per SM of the exchange kernel (1..8)
        p0 = (channels * n_tex + 3) // 4 * 4
        self.texture = self.out[: channels * n_tex].view(channels, n_tex)
        self.points = self.out[p0: p0 + 4 * n].view(n, 4)
        self.confidence = self.out[p0 + 4 * n:].view(1, n_tex)

    def _launch(self, segments: int, ctas_per_sm: int):
        from . import _lib as L

        self.rast._sync_stream()
        rc = L.lib().vetr_exchange_finalize_part(self.rast._ctx, self.c, self.channels, self.n_tex, self.n, segments, ctas_per_sm)
        self.rast._check(rc, "vetr_exchange_finalize_part")

    def _finish(self, g: dict) -> dict:
        """The collective that orders the consumers after all ranks' exchange kernels (and reduces the hit counts of the
        pose gradients), the small remaining reductions and the count normalisation of the camera gradients."""
        from . import _lib as L

        second = g.get("pose_count") if g.get("pose_count") is not None else self._token
        dist.all_reduce(second, group=self.group)
        for key in ("background", "intrinsics", "intrinsics_count"):
            if g.get(key) is not None:
                dist.all_reduce(g[key], group=self.group)
        pose, intr = g.get("pose"), g.get("intrinsics")
        if pose is not None or intr is not None:
            ptr = lambda t: None if t is None else C.c_void_p(t.data_ptr())
            self.rast._sync_stream()
            rc = L.lib().vetr_finalize_gradients(
                self.rast._ctx, self.channels, 0, None, None, 0, None, None,
                0 if pose is None else pose.shape[0], ptr(pose), ptr(g.get("pose_count")),
                0 if intr is None else intr.shape[0], ptr(intr), ptr(g.get("intrinsics_count")))
            self.rast._check(rc, "vetr_finalize_gradients")
        return dict(texture=self.texture, points=self.points, confidence=self.confidence, background=g.get("background"),
                    pose=pose, intrinsics=intr)

    def run(self, g: dict) -> dict:
        """g: the dict backward accumulated into (its desc / points / conf are views of self.buffer).  Returns the
        finished gradients (views of the result buffer, the same on every rank) plus the reduced small tensors."""
        first = g.get("pose") if g.get("pose") is not None else self._token
        dist.all_reduce(first, group=self.group)
        self._launch(7, self.ctas_per_sm)
        return self._finish(g)

    def run_overlapped(self, grad_color, g: dict, bilinear: bool = False) -> dict:
        """Second half of a backward step whose per-fragment kernels (Rasterizer.backward_raw(..., phases=1)) are already
        enqueued: the exchange of the segments those kernels finished (descriptor gradient, and the confidence gradient
        except in mode 3) runs on a side stream with one thread block per SM BESIDE the per-point pass, the rest after it.

            main stream:  all-reduce(token) -> per-point pass -> all-reduce(pose) -> exchange(rest) -> join -> all-reduce(count)
            side stream:        wait        -> exchange(descriptor [, confidence])
        """
        from . import _lib as L

        if self._side is None:
            self._side = torch.cuda.Stream(self.raw.device)
            self._fork, self._join = torch.cuda.Event(), torch.cuda.Event()
        main = torch.cuda.current_stream(self.raw.device)
        early = L.SEG_DESC | (0 if bilinear else L.SEG_CONF)
        dist.all_reduce(self._token, group=self.group)  # every rank's per-fragment kernels have finished
        self._fork.record(main)
        with torch.cuda.stream(self._side):
            self._side.wait_event(self._fork)
            self._launch(early, 1)
            self._join.record(self._side)
        self.rast.backward_raw(grad_color, want_intrinsics=g.get("intrinsics") is not None, accum=g, phases=2)
        first = g.get("pose") if g.get("pose") is not None else self._token
        dist.all_reduce(first, group=self.group)        # every rank's per-point pass has finished
        self._launch(7 & ~early, 4)
        main.wait_event(self._join)
        return self._finish(g)
