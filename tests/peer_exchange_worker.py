"""Child process of test_gpu_peer_exchange.py::test_two_real_ranks (one rank per GPU, launched with torch.distributed.run).

Renders a small scene view-sharded over the ranks, then obtains the finished gradients twice: PeerExchange (one kernel over
symmetric memory) and NCCL all-reduce + vetr_finalize_gradients.  Both must agree on every rank and between the ranks."""
import datetime
import os
import sys

import numpy as np
import torch
import torch.distributed as dist

sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
from vet_b200 import scenes  # noqa: E402
from vet_b200.dist import GradientBuffer, PeerExchange, allreduce_gradients  # noqa: E402
from vet_b200.render import Rasterizer, default_params, scene_to_device  # noqa: E402


def main():
    rank, world, local = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"]), int(os.environ["LOCAL_RANK"])
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=120))
    scene = scenes.config_planar(20000, 256, 192, 200.0, n_views=2 * world, seed=3)
    views = scene.views[rank::world]
    tensors = scene_to_device(scene, dev)
    position, index, texture, confidence, background, poses, intrinsics = tensors
    n, n_tex, ch = position.shape[0], texture.shape[1], texture.shape[0]
    params = default_params(render_mode=1, num_layers=4, num_channels=ch)
    rast = Rasterizer(local)
    out = rast.forward(*tensors, views, params)
    gen = torch.Generator(device="cpu").manual_seed(100 + rank)
    grads = [torch.randn(c.shape, generator=gen).to(dev) for c in out["color"]]

    # path 1: one kernel over peer memory; first with plain peer loads / stores, then through the NVSwitch multicast
    # object where the platform has one
    results = []
    for multicast in (False, True):
        peer = PeerExchange(rast, n, n_tex, ch, dev, multicast=multicast)
        if multicast and not peer.multicast:
            if rank == 0:
                print("no multicast object on this platform: multimem path not run", flush=True)
            break
        for it in range(2):  # twice: the buffers are reused step after step
            peer.buffer.zero_()
            g1 = rast.backward_raw(grads, want_intrinsics=False, accum=peer.buffer.as_accum(ch, poses.shape[0]))
            r1 = peer.run(g1)
        results.append(tuple(r1[k].clone() for k in ("texture", "points", "confidence", "pose")))
        # the same with the per-point pass beside the exchange of the descriptor / confidence segments
        peer.buffer.zero_()
        g1 = rast.backward_raw(grads, want_intrinsics=False, accum=peer.buffer.as_accum(ch, poses.shape[0]), phases=1)
        r1 = peer.run_overlapped(grads, g1)
        results.append(tuple(r1[k].clone() for k in ("texture", "points", "confidence", "pose")))
        if rank == 0:
            print("exchange ran with multicast =", peer.multicast, flush=True)

    # path 2: NCCL all-reduce of the fused buffer + the epilogue kernels
    buf = GradientBuffer(n, n_tex, dev)
    g2 = rast.backward_raw(grads, want_intrinsics=False, accum=buf.as_accum(ch, poses.shape[0]))
    allreduce_gradients(buf, g2)
    r2 = rast.finalize(g2)
    torch.cuda.synchronize()

    def close(a, b, what):
        a, b = a.double().cpu().numpy().ravel(), b.double().cpu().numpy().ravel()
        scale = max(np.abs(b).max(), 1e-30)
        err = np.abs(a - b).max() / scale
        assert err < 1e-5, (what, err)  # the two paths add the ranks' float sums in different orders

    for tex1, pts1, conf1, pose1 in results:
        close(tex1, r2["texture"], "texture")
        close(pts1, r2["points"], "points")
        close(conf1, r2["confidence"], "confidence")
        close(pose1, r2["pose"], "pose")
        assert int(torch.count_nonzero(pts1).item()) > 0 and int(torch.count_nonzero(tex1).item()) > 0
        # every rank holds the same bits
        for t in (tex1, pts1, conf1):
            ref = t.clone()
            dist.broadcast(ref, src=0)
            assert torch.equal(ref, t)
    dist.barrier()
    if rank == 0:
        print("PEER_EXCHANGE_OK", flush=True)
    dist.destroy_process_group()


if __name__ == "__main__":
    main()
