"""View-sharded data parallelism for the rasterizer (one process per GPU).

The reference has no multi-GPU code.  A training batch shards by view: the cloud, descriptors and cameras are
replicated, rank r renders the views {v : v mod world == r}, and the only exchange per step is the sum of the
point-parameter gradients.  They live in ONE fused fp32 buffer so that one all-reduce moves them:

    [ descriptor gradient  n_tex x 4 | position gradient + hit count  n x 4 | confidence gradient  n_tex ]

Hit counts travel with the sums because the reference averages position gradients by the number of hits
(rendering/PointRenderer.cu:1273-1280): the division has to come after the sum over ranks.  Pose-tangent gradients
and their counts (double / float, a few hundred bytes) are reduced separately.
"""
from __future__ import annotations

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

    def __init__(self, n: int, n_tex: int, device):
        self.n, self.n_tex = n, n_tex
        self.flat = torch.zeros(4 * n_tex + 4 * n + n_tex, dtype=torch.float32, device=device)
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
