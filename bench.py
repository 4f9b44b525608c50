#!/usr/bin/env python
"""Benchmark of the blending point rasterizer: forward + backward frames/s at 1920x1080 with an 8M-point cloud.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--points M] [--views V]

One step = one training batch of V views per GPU: forward (count, scan, collect, sort+blend), L1 gradient against
a seeded target, backward (per-fragment kernel + per-point pass), gradient epilogue; with N > 1 the point-parameter
gradients (descriptor, confidence, position + hit count: 9 floats per point) are summed over the ranks and finished by
one kernel over NVLink peer memory (--exchange nccl: NCCL all-reduce + epilogue kernels).  Views are sharded over the
GPUs (weak scaling: V views per GPU and step; by default every rank renders the same V poses so that the per-GPU work is
identical), the cloud is replicated.  The compute part of the step is replayed as a CUDA graph.

The script prints ONE JSON line (rank 0).  `value` times the steps with inputs resident in HBM; `e2e` times the same
steps with the per-step inputs (an 8-bit target image per view) arriving from pinned host memory, the target pyramid
built on the device and the loss read back; `roofline` is the dominant kernel against the measured HBM copy bandwidth; `cpu_baseline` is the CPU
oracle on the host cores on a bounded sample (one view of the same cloud).  `--impl reference` times that CPU
oracle alone (the reference ships no CPU rasterizer and its CUDA sources need a library that is not available, so
the oracle port is the reference arm).
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

METRIC = "rasterizer fwd+bwd frames/s @1920x1080, 8M pts"
UNIT = "frames/s"
W, H, FOCAL, LAYERS, CHANNELS = 1920, 1080, 1200.0, 4, 4
HBM_FALLBACK_GBS = 6650.0


def parse_args():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=100)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--points", type=int, default=8_000_000)
    ap.add_argument("--views", type=int, default=4, help="views per GPU and step")
    ap.add_argument("--mode", type=int, default=1, choices=[1, 3])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-next-rows", action="store_true", help="skip the measurements reported beside the headline (grid loss, mode 3)")
    ap.add_argument("--no-configs", action="store_true",
                    help="skip the blocks for the other benchmark configurations (viewer frame, training step, scene in shells; "
                         "N = 1 only) and the 20 M-point batch of 32 distinct views sharded over the GPUs (every N)")
    ap.add_argument("--min-seconds", type=float, default=1.0,
                    help="the timed region repeats the K steps until it has run at least this long (K steps at a time)")
    ap.add_argument("--prewarm", type=float, default=1.0, help="seconds of untimed load before the warm-up steps")
    ap.add_argument("--views-mode", choices=["same", "distinct"], default="same",
                    help="N > 1: every rank renders the same V camera poses (identical per-GPU work), or V poses of its own")
    ap.add_argument("--exchange", choices=["auto", "multicast", "peer", "nccl"], default="auto",
                    help="N > 1: how the ranks' gradient buffers are summed: one kernel over peer memory, either through the "
                         "NVSwitch multicast object (the switch adds; falls back to peer where there is none) or with plain "
                         "peer loads / stores; auto = peer for 2 ranks, multicast for more; nccl = NCCL all-reduce + "
                         "epilogue kernels")
    ap.add_argument("--exchange-ctas", type=int, default=4, help="N > 1: thread blocks per SM of the exchange kernel (1..8)")
    ap.add_argument("--overlap", action="store_true",
                    help="N > 1: run the per-point pass of the backward step beside the exchange of the descriptor / confidence "
                         "segments (measured no faster at N = 2: the extra collective and launches cost what the overlap saves)")
    ap.add_argument("--torch-loss", action="store_true", help="form the L1 loss and its gradient with torch element-wise kernels")
    ap.add_argument("--no-graph", action="store_true", help="launch every kernel from Python instead of replaying a CUDA graph")
    ap.add_argument("--graph-step", action="store_true",
                    help="N > 1: capture the whole step - NCCL calls, exchange kernel(s) and the side stream of --overlap "
                         "included - as one CUDA graph when every rank can (measured at N = 8: no gain without --overlap, "
                         "2 % with it); by default the collectives and the exchange stay outside the graphs")
    return ap.parse_args()


def measured_peak():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured (MEASURED_PEAKS.json hbm_gbs)"
    except Exception:
        return HBM_FALLBACK_GBS, "fallback (6.65 TB/s: MEASURED_PEAKS.json is absent)"


def make_scene(n_points: int, n_views_total: int):
    from vet_b200 import scenes

    return scenes.config_planar(n_points, W, H, FOCAL, n_views=n_views_total, seed=2002, channels=CHANNELS)


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    QUERY = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,clocks_event_reasons.hw_slowdown,"
             "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
             "clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.proc = None
        self.gpu_index = gpu_index
        self.lines = []  # (arrival time, csv line)
        self.thread = None

    def start(self):
        """Starts sampling (every 200 ms) and waits for the first sample."""
        import threading

        try:
            self.proc = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits",
                                          "-lms", "200", "-i", str(self.gpu_index)], stdout=subprocess.PIPE,
                                         stderr=subprocess.DEVNULL, text=True)
        except Exception:
            self.proc = None
            return

        def reader():
            for line in self.proc.stdout:
                self.lines.append((time.perf_counter(), line))

        self.thread = threading.Thread(target=reader, daemon=True)
        self.thread.start()
        t0 = time.perf_counter()
        while not self.lines and time.perf_counter() - t0 < 5.0:
            time.sleep(0.01)

    def stop(self, t_begin: float, t_end: float) -> dict:
        """Summary of the samples that arrived while the timed region [t_begin, t_end] ran (all samples if none did)."""
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"], "samples": 0}
        time.sleep(0.25)
        self.proc.terminate()
        if self.thread is not None:
            self.thread.join(timeout=5)
        inside = [l for (t, l) in self.lines if t_begin <= t <= t_end + 0.25]
        lines = inside if inside else [l for (_, l) in self.lines]
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in lines:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
            except ValueError:
                continue
            for name, val in zip(names, parts[5:9]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm), "samples_in_timed_region": len(inside)}


# -------------------------------------------------------------------------------------------------------------
# reference arm / CPU baseline: the oracle on the host cores


def cpu_oracle_run(scene, params, steps: int, warmup: int, backward: bool = True):
    """Times forward (+ backward) of ONE view per step with the CPU oracle on all host threads.  Returns (seconds per
    step, threads)."""
    from oracle import oracle as O

    threads = O.use_all_host_threads()  # a process launcher may have pinned OMP_NUM_THREADS to 1
    o = O.Oracle()
    p = O.default_params(**{k: v for k, v in params.items() if k in O.default_params()})
    times = []
    for it in range(warmup + steps):
        view = [scene.views[it % len(scene.views)]]
        t0 = time.perf_counter()
        fwd = o.forward(scene, p, views=view)
        t1 = time.perf_counter()
        t2 = t3 = 0.0
        if backward:
            rng = np.random.default_rng(it)  # seeded L1 target: input preparation, not timed
            grads = [(np.sign(c - rng.uniform(0.0, 1.0, size=c.shape).astype(np.float32)) / c.size).astype(np.float32)
                     for c in fwd["color"]]
            t2 = time.perf_counter()
            o.backward(grads)
            t3 = time.perf_counter()
        if it >= warmup:
            times.append((t1 - t0) + (t3 - t2))
    return float(np.mean(times)), threads


def parity_against_oracle(rast, scene, params, view_index: int = 0, backward: bool = True) -> dict:
    """One view of `scene` through the CUDA library and through the CPU oracle on the same inputs, compared: fragment
    total, per-pixel counts and sorted keys (exact), images (largest absolute difference), raw gradient sums (largest
    error in units of the bound 1e-5 x sum|addends| of the element).  The oracle is the checker here, never the thing
    measured; a difference is reported, not raised."""
    import copy

    from tests import util

    one = copy.copy(scene)
    one.views = [scene.views[view_index]]
    ora = util.run_oracle(one, params)
    grads = util.l1_grads(ora["fwd"]["color"], seed=5) if backward else None
    if backward:
        ora = util.run_oracle(one, params, grads=grads)
    gpu = util.run_gpu(rast, one, params, grads=grads)
    return util.parity_report(gpu, ora, scene.channels)


def envmap_libtorch(torch, density, color, radii, poses, intrinsics, views, layers, weight, grad_out, reps=2):
    """The reference's own formulation of the environment-map row, timed on the GPU beside the fused kernels: forward_mps5
    (rendering/EnvironmentMap.cu:692-758) is two 5-D grid_sample calls, a sigmoid and a multiply-add chain of libtorch
    operators per sphere, and autograd is its backward pass.  The sample coordinates (the reference's two small CUDA kernels
    before it) are formed here with torch operators outside the timed region.  Returns (forward ms, backward ms, result)."""
    import torch.nn.functional as F

    dev = density.device
    S, C = density.shape[0], color.shape[0]
    uvz, T0 = [], []
    for l in range(layers):
        for b, v in enumerate(views):
            w, h = v.w >> l, v.h >> l
            q = poses[v.image_index].to(torch.float32)
            K = intrinsics[v.camera_index]
            crop = torch.tensor(v.crop, device=dev) * 0.5 ** l
            rot = torch.tensor(v.rot, device=dev).reshape(2, 2)
            gy, gx = torch.meshgrid(torch.arange(h, device=dev, dtype=torch.float32),
                                    torch.arange(w, device=dev, dtype=torch.float32), indexing="ij")
            c = torch.tensor([w // 2, h // 2], device=dev, dtype=torch.float32)
            ip = (torch.stack([gx, gy], -1) - c) @ torch.linalg.inv(rot).T + c
            py = (ip[..., 1] - crop[3]) / crop[1]
            px = (ip[..., 0] - crop[2] - crop[4] * py) / crop[0]
            ny = (py - K[3]) / K[1]
            nx = (px - K[2] - K[4] * ny) / K[0]
            x, y, z, s_ = q[0], q[1], q[2], q[3]
            Rm = torch.stack([torch.stack([1 - 2 * (y * y + z * z), 2 * (x * y - z * s_), 2 * (x * z + y * s_)]),
                              torch.stack([2 * (x * y + z * s_), 1 - 2 * (x * x + z * z), 2 * (y * z - x * s_)]),
                              torch.stack([2 * (x * z - y * s_), 2 * (y * z + x * s_), 1 - 2 * (x * x + y * y)])])
            eye = -(Rm.T @ q[4:7])
            o = torch.stack([nx, ny, torch.ones_like(nx)], -1).reshape(-1, 3) @ Rm + eye
            d = torch.nn.functional.normalize(o - eye, dim=-1)
            per_sphere = []
            for s in range(S):
                if s == S - 1:
                    p = d
                else:
                    bq = (o * d).sum(-1)
                    k = -bq + torch.sqrt(torch.clamp(bq * bq - ((o * o).sum(-1) - radii[s] ** 2), min=0))
                    p = torch.nn.functional.normalize(o + k[:, None] * d, dim=-1)
                lat, lon = torch.asin(p[:, 0].clamp(-1, 1)), torch.atan2(p[:, 1], p[:, 2])  # up axis 0
                zc = torch.full_like(lat, 0.0 if S == 1 else 2.0 * s / (S - 1) - 1.0)
                per_sphere.append(torch.stack([lon / np.pi, 2 * lat / np.pi, zc], -1))
            uvz.append(torch.stack(per_sphere))
            T0.append(weight[l][b].reshape(-1))
    uvz = torch.cat(uvz, 1).contiguous()  # [S, rays, 3]
    T0 = torch.cat(T0)
    G = torch.cat([grad_out[l][b].reshape(C, -1) for l in range(layers) for b in range(len(views))], 1)
    n = uvz.shape[1]
    dens_p = density[None, None].clone().requires_grad_(True)
    col_p = color[None].clone().requires_grad_(True)
    opt = dict(mode="bilinear", padding_mode="zeros", align_corners=True)
    ev = [torch.cuda.Event(enable_timing=True) for _ in range(3)]
    fwd_ms = bwd_ms = 0.0
    for it in range(reps + 1):
        dens_p.grad = col_p.grad = None
        ev[0].record()
        grid = uvz.reshape(1, S * n, 1, 1, 3)
        alpha_all = torch.sigmoid(F.grid_sample(dens_p, grid, **opt).reshape(1, S, n).permute(1, 0, 2))
        color_all = F.grid_sample(col_p, grid, **opt).reshape(C, S, n).permute(1, 0, 2)
        final, T = torch.zeros(C, n, device=dev), T0.unsqueeze(1)
        for s in range(S):
            alpha = alpha_all[s]
            if s == S - 1:
                alpha = torch.ones_like(alpha)
            final = T.squeeze().unsqueeze(0) * alpha * color_all[s] + final
            T = ((1 - alpha.squeeze()) * T.squeeze()).unsqueeze(1)
        ev[1].record()
        final.backward(G)
        ev[2].record()
        torch.cuda.synchronize(dev)
        if it > 0:
            fwd_ms += ev[0].elapsed_time(ev[1]) / reps
            bwd_ms += ev[1].elapsed_time(ev[2]) / reps
    return fwd_ms, bwd_ms, final.detach(), dens_p.grad[0, 0], col_p.grad[0]


def run_reference(args):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    # bounded: one step is one 1920x1080 view of the full cloud (about 3 s on 16 host threads); at most 16 of the asked
    # steps are run so that the arm ends within a few minutes whatever K is, and `steps` reports what was timed
    steps, warmup = min(max(1, args.steps), 16), min(args.warmup, 1)
    scene = make_scene(args.points, steps)
    from vet_b200.render import default_params

    sec, threads = cpu_oracle_run(scene, default_params(render_mode=args.mode), steps, warmup)
    value = 1.0 / sec
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": args.gpus, "steps": steps,
        "warmup": warmup, "ms_per_step": sec * 1e3, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f32", "data": "synthetic",
        "config": {"workload": f"headline: {args.points} planar-scene points, 1 view {W}x{H} f={FOCAL:g}, {LAYERS} levels, "
                               f"mode {args.mode}, fwd+bwd, L1 vs seeded target", "l2": "inputs larger than L2"},
        "cpu_baseline": {"value": value, "unit": UNIT, "cores": threads, "kind": "port",
                         "sample": "each step = forward+backward of ONE 1920x1080 view of the full cloud with the CPU "
                                   "oracle (OpenMP, all host threads)"},
        "e2e": {"value": value, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


# -------------------------------------------------------------------------------------------------------------
# our arm


def run_ours(args):
    import torch
    import torch.distributed as dist

    from vet_b200.render import Rasterizer, default_params, level_sizes, scene_to_device

    world = int(os.environ.get("WORLD_SIZE", "1"))
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    torch.cuda.set_device(local_rank)
    dev = torch.device("cuda", local_rank)
    if world > 1:
        import datetime

        dist.init_process_group("nccl", device_id=dev, timeout=datetime.timedelta(seconds=180))
    V = args.views
    params = default_params(render_mode=args.mode, num_layers=LAYERS, num_channels=CHANNELS)

    # the cloud is replicated; every rank renders its own V views per step (view-sharded batch of world * V views)
    if args.views_mode == "same":
        # weak scaling with identical per-GPU work: every rank renders the same V camera poses (against its own seeded
        # targets), so the step time at N GPUs differs from N = 1 by the exchange alone, not by which views a rank drew
        scene = make_scene(args.points, V)
        my_views = scene.views
    else:
        scene = make_scene(args.points, world * V)
        my_views = scene.views[rank * V:(rank + 1) * V]
    tensors = scene_to_device(scene, dev)
    position, index, texture, confidence, background, poses, intrinsics = tensors
    n, n_tex = position.shape[0], texture.shape[1]
    sizes = level_sizes(W, H, LAYERS)
    P = sum(w * h for w, h in sizes)

    stream = torch.cuda.current_stream(dev)
    rast = Rasterizer(local_rank)  # follows torch's current stream, so a step can be captured into a CUDA graph

    # seeded targets of the L1 loss: one 8-bit image per view, as a training loop holds its photographs; the target of a
    # coarser pyramid level is the 2x2 average of the finer one, built on the device.  `value` uses a resident pyramid,
    # `e2e` receives the 8-bit images from pinned host memory every step and builds the pyramid inside the timed region.
    gen = torch.Generator(device="cpu").manual_seed(1234 + rank)
    targets_host = (torch.rand(V, CHANNELS, H, W, generator=gen) * 255.0).to(torch.uint8).pin_memory()

    def build_targets(u8, out):
        torch.mul(u8, 1.0 / 255.0, out=out[0])  # one kernel: 8-bit in, fp32 out
        for l in range(1, len(out)):
            torch.ops.aten.avg_pool2d.out(out[l - 1], [2, 2], [2, 2], [0, 0], False, True, None, out=out[l])

    targets_dev = [torch.empty(V, CHANNELS, h, w, device=dev) for (w, h) in sizes]
    build_targets(targets_host.to(dev), targets_dev)
    numel = [float(t.numel()) for t in targets_dev]
    h2d_bytes = targets_host.numel()

    # fused gradient buffer: [desc 4n_tex | points 4n | conf n_tex] floats.  N > 1: it lives in symmetric memory and the
    # sum over the ranks + the epilogue is one kernel over NVLink peer memory (vet_b200.dist.PeerExchange);
    # --exchange nccl selects an NCCL all-reduce of the buffer followed by the epilogue kernels instead.
    peer = None
    exchange_kind = "none" if world == 1 else args.exchange
    if world > 1 and args.exchange != "nccl":
        from vet_b200.dist import PeerExchange
        why = None
        try:
            peer = PeerExchange(rast, n, n_tex, CHANNELS, dev,
                                multicast=None if args.exchange == "auto" else args.exchange == "multicast")
        except Exception as e:  # noqa: BLE001  (no symmetric memory on this platform)
            why = repr(e)[:160]
        ok = torch.tensor([0.0 if peer is None else 1.0], device=dev)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)  # all ranks take the same path
        if ok.item() < 1.0:
            peer = None
            exchange_kind = "nccl (peer memory unavailable" + (": " + why if why else " on another rank") + ")"
    if peer is not None:
        peer.ctas_per_sm = args.exchange_ctas
        exchange_kind = "multicast" if peer.multicast else "peer"
        flat = peer.raw
    else:
        flat = torch.zeros(4 * n_tex + 4 * n + n_tex, dtype=torch.float32, device=dev)

    overlap = peer is not None and args.overlap

    def grad_views():
        g = dict(desc=flat[:4 * n_tex].view(n_tex, 4), points=flat[4 * n_tex:4 * n_tex + 4 * n].view(n, 4),
                 conf=flat[4 * n_tex + 4 * n:], background=torch.zeros(CHANNELS, device=dev),
                 pose=torch.zeros(poses.shape[0], 6, dtype=torch.float64, device=dev),
                 pose_count=torch.zeros(poses.shape[0], device=dev))
        return g

    grad_bufs = [torch.empty(V, CHANNELS, h, w, device=dev) for (w, h) in sizes]
    diff_bufs = [torch.empty(V, CHANNELS, h, w, device=dev) for (w, h) in sizes]
    loss_buf = torch.zeros((), device=dev)

    def compute(targets):
        """Everything of a step up to the gradient sums of this rank."""
        flat.zero_()
        out = rast.forward(position, index, texture, confidence, background, poses, intrinsics, my_views, params,
                           want_weight=True)
        # L1 loss against the target pyramid and its gradient sign(out - target) / numel: one launch for all levels
        # (plumbing around the path, not part of it; --torch-loss forms it with torch's element-wise kernels instead)
        if args.torch_loss:
            grads, loss = [], None
            for l, (c, t) in enumerate(zip(out["color"], targets)):
                d = torch.sub(c, t, out=diff_bufs[l])
                g = torch.sign(d, out=grad_bufs[l])
                g.mul_(1.0 / numel[l])
                grads.append(g)
                term = d.abs_().sum() / numel[l]
                loss = term if loss is None else loss + term
        else:
            grads, loss = grad_bufs, loss_buf
            rast.l1_loss_grad(out["color"], targets, grad_bufs, loss_buf)
        # N > 1 with the peer-memory exchange: only the per-fragment kernels here; the per-point pass runs in exchange(),
        # beside the exchange of the segments that are already final
        g = rast.backward_raw(grads, want_intrinsics=False, accum=grad_views(), phases=1 if overlap else 3)
        return loss, g

    def exchange(g):
        """The one exchange step of view-sharded data parallelism: sum the gradient buffers over the ranks."""
        if peer is not None:  # sum + epilogue in one kernel over peer memory; returns the finished gradients
            return peer.run_overlapped(grad_bufs, g, bilinear=args.mode == 3) if overlap else peer.run(g)
        if world > 1:
            dist.all_reduce(flat)
            dist.all_reduce(g["pose"])
            dist.all_reduce(g["pose_count"])
        return None

    def step(targets):
        loss, g = compute(targets)
        fin = exchange(g)
        return loss, (fin if fin is not None else rast.finalize(g))

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)

    # ---- the step as CUDA graphs: ~60 kernel launches (library + loss + epilogue) replayed with two calls, so that the
    # host's launch cost is off the critical path.  The all-reduce stays an ordinary NCCL call between the two graphs.
    # Falls back to plain launches if capture fails.
    eager_step = step
    static_targets = [t.clone() for t in targets_dev]
    graph_info = {"used": False}
    if not args.no_graph:
        try:
            for _ in range(2):  # sizes every scratch buffer (nothing may be allocated by the library during capture)
                eager_step(static_targets)
            torch.cuda.synchronize(dev)
            graph_a, graph_b = torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph_a):
                loss_static, g_static = compute(static_targets)
            if peer is None:
                with torch.cuda.graph(graph_b, pool=graph_a.pool()):
                    fin_static = rast.finalize(g_static)
            torch.cuda.synchronize(dev)

            def step(targets):
                if targets is not static_targets:
                    for dst, src in zip(static_targets, targets):
                        if dst.data_ptr() != src.data_ptr():
                            dst.copy_(src, non_blocking=True)
                graph_a.replay()
                fin = exchange(g_static)
                if fin is not None:
                    return loss_static, fin
                graph_b.replay()
                return loss_static, fin_static

            graph_info["used"] = True
        except Exception as e:  # noqa: BLE001
            graph_info["error"] = repr(e)[:200]
            step = eager_step
            torch.cuda.synchronize(dev)
        # N > 1: the whole step as ONE graph - compute, the ordering collectives, the exchange kernel(s) and the side
        # stream of --overlap - so that no host launch sits between the compute part and the exchange.  Used only if every
        # rank captured it (agreed with a collective outside the capture); otherwise the two-graph form above stays.
        if graph_info["used"] and peer is not None and args.graph_step:
            captured = 1.0
            try:
                graph_step = torch.cuda.CUDAGraph()
                with torch.cuda.graph(graph_step, capture_error_mode="thread_local"):
                    loss_whole, fin_whole = eager_step(static_targets)
            except Exception as e:  # noqa: BLE001
                captured = 0.0
                graph_info["whole_step_error"] = repr(e)[:200]
            torch.cuda.synchronize(dev)
            agreed = torch.tensor([captured], device=dev)
            dist.all_reduce(agreed, op=dist.ReduceOp.MIN)
            if agreed.item() >= 1.0:
                def step(targets):  # noqa: F811
                    if targets is not static_targets:
                        for dst, src in zip(static_targets, targets):
                            if dst.data_ptr() != src.data_ptr():
                                dst.copy_(src, non_blocking=True)
                    graph_step.replay()
                    return loss_whole, fin_whole

            graph_info["whole_step"] = bool(agreed.item() >= 1.0)

    # ---- value: inputs resident in HBM
    sampler = ClockSampler(local_rank)
    if rank == 0:
        sampler.start()
    # bring the clocks up before the counted warm-up steps (a cold GPU needs a few hundred ms of load to boost).  The
    # number of these steps is agreed between the ranks: every step holds collectives, so all ranks must run the same count.
    n_pre = 0
    if args.prewarm > 0:
        step(static_targets)
        torch.cuda.synchronize(dev)
        t_pre = time.perf_counter()
        step(static_targets)
        torch.cuda.synchronize(dev)
        one = torch.tensor([time.perf_counter() - t_pre], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(one, op=dist.ReduceOp.MAX)
        n_pre = int(min(500, max(1, args.prewarm / max(float(one.item()), 1e-4))))
    for _ in range(n_pre):
        step(static_targets)
    for _ in range(args.warmup):
        step(static_targets)
    F_total, longest = rast.fragment_count()
    barrier()
    launches0 = rast.launch_count()
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    barrier()
    # the timed region: K steps, repeated (K at a time) until it has run for --min-seconds, so that a small K still gives
    # the clock sampler and the end-to-end leg a region of about a second.  The repeat count is agreed between the ranks
    # from the prewarm step time, before the region starts.
    repeats = 1
    if args.min_seconds > 0 and args.prewarm > 0:
        repeats = int(min(1000, max(1, np.ceil(args.min_seconds / max(float(one.item()) * args.steps, 1e-6)))))
    timed_steps = repeats * args.steps
    t_begin = time.perf_counter()
    step_events = [torch.cuda.Event(enable_timing=True) for _ in range(args.steps + 1)]
    e0.record(stream)
    step_events[0].record(stream)
    for i in range(timed_steps):
        loss, fin = step(static_targets)
        if i < args.steps:
            step_events[i + 1].record(stream)
    e1.record(stream)
    barrier()
    t_end = time.perf_counter()
    ms = e0.elapsed_time(e1)
    step_ms = [step_events[i].elapsed_time(step_events[i + 1]) for i in range(args.steps)]
    launches = rast.launch_count() - launches0
    if graph_info["used"]:
        l0 = rast.launch_count()
        eager_step(static_targets)
        launches = (rast.launch_count() - l0) * timed_steps  # the graph replays exactly the launches of one eager step
    clocks = sampler.stop(t_begin, t_end) if rank == 0 else None
    t = torch.tensor([ms], dtype=torch.float64, device=dev)
    if world > 1:
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
    ms_total = float(t.item())
    frames = world * V * timed_steps
    value = frames / (ms_total * 1e-3)
    # per-rank load (the step time is the max over the ranks): fragments of the rank's views, ms of its compute graph
    per_rank = None
    if world > 1:
        c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        c0.record(stream)
        for _ in range(3):
            if graph_info["used"]:
                graph_a.replay()
            else:
                compute(static_targets)
        c1.record(stream)
        torch.cuda.synchronize(dev)
        mine = torch.tensor([float(F_total), c0.elapsed_time(c1) / 3], dtype=torch.float64, device=dev)
        allr = [torch.zeros_like(mine) for _ in range(world)]
        dist.all_gather(allr, mine)
        per_rank = [{"fragments": int(t[0].item()), "compute_ms": round(float(t[1].item()), 3)} for t in allr]

    # ---- N > 1: one untimed step whose exchanged result (the kernel over peer memory, plain or through the NVSwitch
    # multicast object) is compared with an NCCL all-reduce of the same raw buffers followed by the epilogue kernels, and
    # whose bits are compared between the ranks
    exchange_check = None
    if world > 1 and peer is not None:
        try:
            _, g_c = compute(static_targets)
            if overlap:  # compute() then stops after the per-fragment kernels: add the per-point pass
                rast.backward_raw(grad_bufs, want_intrinsics=False, accum=g_c, phases=2)
            torch.cuda.synchronize(dev)
            raw_copy = flat.clone()
            pose_copy, pose_count_copy = g_c["pose"].clone(), g_c["pose_count"].clone()
            fin_x = peer.run(g_c)
            torch.cuda.synchronize(dev)
            got = {k: fin_x[k].clone() for k in ("texture", "points", "confidence")}
            dist.all_reduce(raw_copy)
            dist.all_reduce(pose_copy)
            dist.all_reduce(pose_count_copy)
            ref = rast.finalize(dict(desc=raw_copy[:4 * n_tex].view(n_tex, 4), points=raw_copy[4 * n_tex:4 * n_tex + 4 * n].view(n, 4),
                                     conf=raw_copy[4 * n_tex + 4 * n:], background=torch.zeros(CHANNELS, device=dev),
                                     pose=pose_copy, pose_count=pose_count_copy))
            diffs, scale = {}, {}
            for k in got:
                a, b = got[k].reshape(-1), ref[k].reshape(-1)
                diffs[k] = float((a - b).abs().max().item())
                scale[k] = float(b.abs().max().item())
            diffs["pose"] = float((fin_x["pose"] - ref["pose"]).abs().max().item())
            # the same bits on every rank: a 64-bit sum of the results' bit patterns, gathered and compared
            word = torch.stack([got[k].reshape(-1).view(torch.int32).to(torch.int64).sum() for k in ("texture", "points", "confidence")])
            words = [torch.zeros_like(word) for _ in range(world)]
            dist.all_gather(words, word)
            worst = torch.tensor([max(diffs[k] / max(scale.get(k, 1.0), 1e-30) for k in got)], dtype=torch.float64, device=dev)
            dist.all_reduce(worst, op=dist.ReduceOp.MAX)
            exchange_check = {"kind": exchange_kind, "max_abs_diff": diffs, "max_abs_value": scale,
                              "max_diff_relative_to_largest_value_over_ranks": float(worst.item()),
                              "identical_on_all_ranks": bool(all(torch.equal(w, words[0]) for w in words)),
                              "compared_with": "NCCL all-reduce of the same raw buffers + vetr_finalize_gradients"}
            del raw_copy, got, ref
        except Exception as e:  # noqa: BLE001
            exchange_check = {"error": repr(e)[:300]}

    # ---- e2e: per-step targets arrive from pinned host memory (prefetched on a copy stream), loss read back
    e2e = None
    if not args.no_e2e:
        copy_stream = torch.cuda.Stream(dev)
        bufs = [torch.empty_like(targets_host, device=dev) for _ in range(2)]
        ready = [torch.cuda.Event() for _ in range(2)]
        consumed = [torch.cuda.Event() for _ in range(2)]
        loss_host = torch.zeros(2).pin_memory()
        loss_read = [torch.cuda.Event() for _ in range(2)]

        def prefetch(i):
            with torch.cuda.stream(copy_stream):
                copy_stream.wait_event(consumed[i % 2])
                bufs[i % 2].copy_(targets_host, non_blocking=True)
                ready[i % 2].record(copy_stream)

        def e2e_run(k):
            for ev in consumed:
                ev.record(stream)
            prefetch(0)
            for i in range(k):
                if i + 1 < k:
                    prefetch(i + 1)
                stream.wait_event(ready[i % 2])
                build_targets(bufs[i % 2], static_targets)
                consumed[i % 2].record(stream)
                loss, _ = step(static_targets)
                # device -> host read of the step's result: asynchronous, and the host waits for the PREVIOUS step's value
                # before it goes on, so it never runs more than one step ahead and every loss has arrived at the end
                loss_host[i % 2:i % 2 + 1].copy_(loss.reshape(1), non_blocking=True)
                loss_read[i % 2].record(stream)
                if i > 0:
                    loss_read[(i - 1) % 2].synchronize()
            loss_read[(k - 1) % 2].synchronize()

        e2e_run(min(2, args.warmup))
        barrier()
        t0 = time.perf_counter()
        e0.record(stream)
        e2e_run(timed_steps)
        e1.record(stream)
        barrier()
        wall = (time.perf_counter() - t0) * 1e3
        t = torch.tensor([max(e0.elapsed_time(e1), 0.0), wall], dtype=torch.float64, device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        e2e = {"value": frames / (float(t[0].item()) * 1e-3), "unit": UNIT, "h2d_bytes_per_step": h2d_bytes,
               "d2h_bytes_per_step": 4, "wall_ms_per_step": float(t[1].item()) / timed_steps,
               "note": "the views' 8-bit target images copied from pinned host memory every step (double-buffered on a copy "
                       "stream), target pyramid built on the device, loss scalar read back every step"}

    # ---- the same step through the C++/libtorch operator surface (torch.ops.vetr.blend_point_cloud: the PointRender
    # autograd node of vet_b200/torch_shim, what the reference's pipeline calls) with torch's own L1 loss and
    # loss.backward(), inputs and loss crossing the host boundary as in the e2e leg.  Rank 0 at N = 1.
    e2e_shim = None
    if not args.no_e2e and world == 1 and args.mode == 1:
        try:
            shim = os.path.join(ROOT, "vet_b200", "libvetr_torch.so")
            torch.ops.load_library(shim)
            leaf = lambda t: t.detach().clone().requires_grad_(True)
            sh_tex, sh_bg, sh_pos, sh_conf = leaf(texture), leaf(background), leaf(position), leaf(confidence[None])
            sh_tan = torch.zeros(poses.shape[0], 6, dtype=torch.float64, device=dev, requires_grad=True)
            vi = torch.tensor([[v.w, v.h, v.image_index, v.camera_index, v.camera_model] for v in my_views], dtype=torch.int32)
            vf = torch.tensor([list(v.crop) + list(v.rot) for v in my_views], dtype=torch.float32)
            leaves = (sh_tex, sh_bg, sh_pos, sh_conf, sh_tan)
            cs2 = torch.cuda.Stream(dev)
            bufs2 = [torch.empty_like(targets_host, device=dev) for _ in range(2)]
            ready2, used2 = [torch.cuda.Event() for _ in range(2)], [torch.cuda.Event() for _ in range(2)]
            loss_host2 = torch.zeros(1).pin_memory()

            def shim_steps(k):
                for ev in used2:
                    ev.record(stream)
                for i in range(k):
                    with torch.cuda.stream(cs2):
                        cs2.wait_event(used2[i % 2])
                        bufs2[i % 2].copy_(targets_host, non_blocking=True)
                        ready2[i % 2].record(cs2)
                    stream.wait_event(ready2[i % 2])
                    build_targets(bufs2[i % 2], static_targets)
                    used2[i % 2].record(stream)
                    for t in leaves:
                        t.grad = None
                    outs = torch.ops.vetr.blend_point_cloud(sh_tex, sh_bg, sh_pos, index[:, None], poses, sh_tan, intrinsics, sh_conf,
                                                            vi, vf, LAYERS, 1, False, False, True, False, True)
                    l1 = sum((o - t).abs().mean() for o, t in zip(outs[:LAYERS], static_targets))
                    l1.backward()
                    loss_host2.copy_(l1.detach().reshape(1), non_blocking=True)
                torch.cuda.synchronize(dev)

            shim_steps(3)
            base_alloc = torch.cuda.memory_allocated(dev)
            torch.cuda.reset_peak_memory_stats(dev)
            k_shim = max(5, min(timed_steps, 50))
            s0, s1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            t0 = time.perf_counter()
            s0.record(stream)
            shim_steps(k_shim)
            s1.record(stream)
            torch.cuda.synchronize(dev)
            wall = (time.perf_counter() - t0) * 1e3
            peak_extra = torch.cuda.max_memory_allocated(dev) - base_alloc
            e2e_shim = {"value": V * k_shim / (s0.elapsed_time(s1) * 1e-3), "unit": UNIT, "steps": k_shim,
                        "wall_ms_per_step": wall / k_shim, "h2d_bytes_per_step": h2d_bytes, "d2h_bytes_per_step": 4,
                        "peak_extra_device_bytes": int(peak_extra), "fragment_records_bytes": int(F_total) * 32,
                        "loss": float(loss_host2.item()),
                        "note": "torch.ops.vetr.blend_point_cloud + torch L1 loss + loss.backward(); the fragment buffer is sized "
                                "from the totals of earlier calls; peak_extra = device memory above the resident tensors while a "
                                "step runs (lists, scratch, images, gradients, autograd's saved tensors)"}
            del leaves, sh_tex, sh_bg, sh_pos, sh_conf, sh_tan, bufs2
            torch.cuda.empty_cache()
        except Exception as e:  # noqa: BLE001
            e2e_shim = {"error": repr(e)[:300]}

    # ---- per-kernel timing (CUDA events on the launching stream, outside the timed region) and roofline
    rast.set_timing(True)
    acc = {}
    reps = 5
    for _ in range(reps):
        loss_e, fin = eager_step(targets_dev)
        for k, v in rast.timings().items():
            acc[k] = acc.get(k, 0.0) + v / reps
    rast.set_timing(False)
    touched = int(torch.count_nonzero(fin["points"][:, :3].abs().sum(dim=1)).item()) if fin.get("points") is not None else 0
    F, N, PT = F_total, n, P * V
    # algorithmic bytes per launch (one launch = V views); N_t = points with a position gradient
    kernel_bytes = {
        "count": 16 * N * V + 4 * PT,                       # positions streamed once per view; counts written
        "scan": 12 * PT,                                    # counts read twice, offsets written
        "collect": 16 * N * V + 8 * F,                      # positions again; one 8-byte key per fragment
        "sort_blend": 16 * F + 20 * F + 4 * PT + (4 * CHANNELS + 4) * PT,   # keys read + written back, descriptor and
                                                                            # confidence gather, offsets, colour + weight
        # the backward step's bytes (keys, descriptor / confidence / position of every fragment, offsets, gradient +
        # forward image, one read + one write of each touched gradient element) split over its two kernels: the position
        # part belongs to the per-point pass.  The image-space gradients the first kernel parks for the second one are
        # not algorithmic bytes.
        "backward": 8 * F + 20 * F + 4 * PT + 8 * CHANNELS * PT + 2 * 20 * touched,
        "point_backward": 16 * F + 2 * 16 * touched,
        "finalize": 32 * n_tex + 32 * N,                    # transpose descriptor gradient, normalise point gradient
    }
    if peer is not None:
        # the rank reads its 1/world slice of every rank's 36-byte-per-point raw sums and writes the finished slice to
        # every rank: 2 x 36 bytes per point cross this GPU's links or HBM either way
        kernel_bytes["exchange"] = 2 * 36 * N
        kernel_bytes.pop("finalize")
    peak, peak_src = measured_peak()
    kernels = {k: {"ms": acc.get(k, 0.0), "bytes": kernel_bytes[k],
                   "gbs": (kernel_bytes[k] / (acc[k] * 1e-3) / 1e9) if acc.get(k, 0.0) > 0 else None} for k in kernel_bytes}
    dominant = max(kernels, key=lambda k: kernels[k]["ms"])
    whole_bytes = sum(kernel_bytes.values()) + 4 * flat.numel()  # + zero fill of the gradient buffer
    roofline = {"bound": "hbm", "kernel": dominant, "achieved": kernels[dominant]["gbs"], "peak": peak, "unit": "GB/s",
                "frac": (kernels[dominant]["gbs"] or 0.0) / peak,
                "traffic": (TRAFFIC_OVER_ALGORITHMIC[dominant] * kernel_bytes[dominant]
                            if dominant in TRAFFIC_OVER_ALGORITHMIC else None),
                "peak_source": peak_src, "kernels": kernels,
                "whole_step": {"algorithmic_bytes": whole_bytes,
                               "achieved_gbs": whole_bytes * timed_steps / (ms_total * 1e-3) / 1e9,
                               "frac": whole_bytes * timed_steps / (ms_total * 1e-3) / 1e9 / peak},
                "counts": {"N": N, "N_touched": touched, "F": F, "pixels": PT, "views_per_launch": V,
                           "longest_list": longest}}

    # ---- the path's next row, measured beside the headline: error-grid rasterisation of one view's loss image over a
    # 128^3 grid around the scene (FillSceneGridWithLoss; one launch per training image at the end of an epoch)
    next_rows = None
    if rank == 0 and world == 1 and not args.no_next_rows:
        # informative rows: a failure here is reported in the line and never costs the headline measurement
        next_rows = {}
        try:
            cells = 128
            ax = torch.linspace(-10.0, 10.0, cells + 1, device=dev)[:-1]
            gx, gy, gz = torch.meshgrid(ax, ax, ax, indexing="ij")
            bb_min = torch.stack([gx, gy, gz], dim=-1).reshape(-1, 3).contiguous()
            bb_len = torch.full_like(bb_min, 20.0 / cells)
            loss_img = torch.rand(3, H, W, device=dev)
            cell_value = torch.zeros(bb_min.shape[0], device=dev)
            cell_count = torch.zeros(bb_min.shape[0], dtype=torch.int32, device=dev)
            g0, g1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            for it in range(4):
                if it == 1:
                    g0.record(stream)
                rast.grid_loss(poses, intrinsics, my_views[0], bb_min, bb_len, loss_img, cell_value, cell_count)
            g1.record(stream)
            torch.cuda.synchronize(dev)
            next_rows.update({"grid_loss": {"ms": g0.elapsed_time(g1) / 3, "cells": int(bb_min.shape[0]),
                                       "covered_pixels_per_launch": int(cell_count.sum().item()) // 4,
                                       "workload": f"{cells}^3 cells over a 20-unit box, one {W}x{H} view, 3-channel loss image"}})
            del bb_min, bb_len, loss_img, cell_value, cell_count

            # texture environment map (EnvironmentMapImpl::Sample2 and its gradient): four spheres of 1024 x 1024 texels, four
            # colour channels, sampled for every pixel of the step's views and levels from a random transmittance
            S_env, R_env = 4, 1024
            density = torch.randn(S_env, R_env, R_env, device=dev)
            color = torch.rand(CHANNELS, S_env, R_env, R_env, device=dev)
            radii = [20.0 * 5.0 ** i for i in range(S_env)]
            weight_env = [torch.rand(V, 1, H >> l, W >> l, device=dev) for l in range(LAYERS)]
            grad_env = [torch.randn(V, CHANNELS, H >> l, W >> l, device=dev) for l in range(LAYERS)]
            g_density, g_color = torch.zeros_like(density), torch.zeros_like(color)
            e0, e1, e2 = (torch.cuda.Event(enable_timing=True) for _ in range(3))
            env_flags = 8  # zero distortion vouched for: no read-back inside the timed loop
            for it in range(4):
                if it == 1:
                    e0.record(stream)
                env_out = rast.envmap_forward(poses, intrinsics, my_views, LAYERS, density, color, radii, weight_env, flags=env_flags)
            e1.record(stream)
            for it in range(3):
                rast.envmap_backward(poses, intrinsics, my_views, LAYERS, density, color, radii, weight_env, grad_env, flags=env_flags,
                                     g_density=g_density, g_color=g_color)
            e2.record(stream)
            torch.cuda.synchronize(dev)
            env_px = sum(V * (H >> l) * (W >> l) for l in range(LAYERS))
            fwd_ms, bwd_ms = e0.elapsed_time(e1) / 3, e1.elapsed_time(e2) / 3
            next_rows["envmap"] = {"forward_ms": fwd_ms, "backward_ms": bwd_ms, "pixels": env_px,
                                   "forward_GBps": env_px * 4 * (1 + CHANNELS) / (fwd_ms * 1e-3) / 1e9,
                                   "workload": f"{S_env} spheres of {R_env}^2 texels, {CHANNELS} channels, {V} views x {LAYERS} levels"}
            # the reference's formulation of the same work (libtorch operators + autograd), timed beside it; also a check of the
            # fused kernels against it on the full-size workload
            try:
                g_density.zero_(), g_color.zero_()
                rast.envmap_backward(poses, intrinsics, my_views, LAYERS, density, color, radii, weight_env, grad_env, flags=env_flags,
                                     g_density=g_density, g_color=g_color)
                lt_f, lt_b, lt_out, lt_gd, lt_gc = envmap_libtorch(torch, density, color, radii, poses, intrinsics, my_views, LAYERS,
                                                                   weight_env, grad_env)
                mine = torch.cat([env_out[l][b].reshape(CHANNELS, -1) for l in range(LAYERS) for b in range(V)], 1)
                next_rows["envmap"]["libtorch_operators"] = {
                    "forward_ms": lt_f, "backward_ms": lt_b,
                    "max_abs_difference_forward": float((mine - lt_out).abs().max().item()),
                    "relative_difference_g_color": float(((g_color - lt_gc).norm() / lt_gc.norm()).item()),
                    "relative_difference_g_density": float(((g_density - lt_gd).norm() / lt_gd.norm()).item()),
                    "note": "forward_mps5 as the reference writes it (grid_sample x2, sigmoid, per-sphere chain; autograd backward) on "
                            "precomputed sample coordinates, same GPU; coordinates from torch operators, so samples differ by the "
                            "rounding of the coordinates"}
                del lt_out, lt_gd, lt_gc, mine
            except Exception as e:  # the comparison is informative; the row's own numbers stand without it
                next_rows["envmap"]["libtorch_operators"] = {"error": repr(e)[:200]}
            if not args.no_cpu_baseline:
                # CPU baseline of this row (part of the cpu_baseline leg): the oracle's forward pass of ONE view on the host
                # cores, same textures and transmittance, and its largest difference from the kernel's result for that view
                try:
                    from oracle import oracle as O

                    env_cpu = O.EnvMap(density.cpu().numpy(), color.cpu().numpy(), inner_radius=20.0, radius_factor=5.0)
                    w_cpu = [w[:1].cpu().numpy() for w in weight_env]
                    c0 = time.perf_counter()
                    ref_env = O.envmap_forward(scene, my_views[:1], LAYERS, env_cpu, w_cpu)
                    cpu_s = time.perf_counter() - c0
                    next_rows["envmap"]["cpu_baseline"] = {
                        "forward_seconds_per_view": cpu_s, "cores": O.threads(), "kind": "port",
                        "max_abs_difference": max(float(np.abs(env_out[l][:1].cpu().numpy() - ref_env[l]).max()) for l in range(LAYERS)),
                        "sample": "forward pass of one view (4 levels) with the oracle (OpenMP)"}
                    del env_cpu, w_cpu, ref_env
                except Exception as e:
                    next_rows["envmap"]["cpu_baseline"] = {"error": repr(e)[:200]}
            del density, color, weight_env, grad_env, g_density, g_color, env_out
            torch.cuda.empty_cache()

            # drop-out radius of the benchmark cloud (SceneData::ComputeRadius: distance to the 4th nearest other point), one call
            # including its host round trips, after one warm-up call that allocates the grid scratch
            rad = rast.knn_radius(position, 4)
            torch.cuda.synchronize(dev)
            k0 = time.perf_counter()
            rad = rast.knn_radius(position, 4, out=rad)
            torch.cuda.synchronize(dev)
            next_rows["knn_radius"] = {"ms": (time.perf_counter() - k0) * 1e3, "points": int(position.shape[0]), "k": 4,
                                       "mean_radius": float(rad.mean().item()),
                                       "workload": "the benchmark cloud; wall time of one call (binning, cell-size search, both passes)"}
            if not args.no_cpu_baseline:
                # CPU baseline of this row (part of the cpu_baseline leg): the oracle's grid search on the host cores, same
                # cloud, and a comparison of all values (the kernel's are bit-equal to it by construction)
                try:
                    from oracle import oracle as O

                    xyz_host = np.ascontiguousarray(scene.position[:, :3])
                    c0 = time.perf_counter()
                    rad_cpu = O.knn_radius(xyz_host, 4, grid=True)
                    cpu_s = time.perf_counter() - c0
                    next_rows["knn_radius"]["cpu_baseline"] = {
                        "seconds": cpu_s, "cores": O.threads(), "kind": "port",
                        "values_that_differ": int((rad.cpu().numpy() != rad_cpu).sum()),
                        "sample": "the whole cloud, one call of the oracle's uniform-grid search (OpenMP)"}
                except Exception as e:
                    next_rows["knn_radius"]["cpu_baseline"] = {"error": repr(e)[:200]}
            del rad

            # the same step in mode 3 (bilinear splats: four fragments per point and level; the mode the reference's shipped
            # configuration trains with), a few launches without graph replay, reported beside the headline
            if args.mode == 1:
                p3 = default_params(render_mode=3, num_layers=LAYERS, num_channels=CHANNELS)
                rast._lists_cache.clear()
                torch.cuda.empty_cache()
                m0, m1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                reps3 = 3
                for it in range(reps3 + 1):
                    if it == 1:
                        m0.record(stream)
                    out3 = rast.forward(position, index, texture, confidence, background, poses, intrinsics, my_views, p3,
                                        want_weight=True)
                    rast.l1_loss_grad(out3["color"], targets_dev, grad_bufs, loss_buf)
                    flat.zero_()
                    g3 = rast.backward_raw(grad_bufs, want_intrinsics=False, accum=grad_views())
                    rast.finalize(g3)
                m1.record(stream)
                torch.cuda.synchronize(dev)
                F3, longest3 = rast.fragment_count()
                ms3 = m0.elapsed_time(m1) / reps3
                next_rows["mode3"] = {"ms_per_step": ms3, "frames_per_s": V / (ms3 * 1e-3), "fragments": F3,
                                      "longest_list": longest3, "workload": "the headline step in render mode 3"}
                # per-kernel table and roofline of the mode-3 step (one more step with the passes bracketed by events): the
                # algorithmic bytes are those of mode 1 with mode 3's own F, plus 16 F for the (u, v, corner) side data the
                # reference writes once and reads once per fragment
                try:
                    rast.set_timing(True)
                    out3 = rast.forward(position, index, texture, confidence, background, poses, intrinsics, my_views, p3,
                                        want_weight=True)
                    rast.l1_loss_grad(out3["color"], targets_dev, grad_bufs, loss_buf)
                    flat.zero_()
                    g3 = rast.backward_raw(grad_bufs, want_intrinsics=False, accum=grad_views())
                    touched3 = int(torch.count_nonzero(g3["points"][:, 3]).item())
                    rast.finalize(g3)
                    t3 = rast.timings()
                    rast.set_timing(False)
                    bytes3 = {"count": 16 * N * V + 4 * PT, "scan": 12 * PT, "collect": 16 * N * V + 8 * F3,
                              "sort_blend": 36 * F3 + 4 * PT + (4 * CHANNELS + 4) * PT,
                              "backward": 28 * F3 + 4 * PT + 8 * CHANNELS * PT + 2 * 20 * touched3,
                              "point_backward": 16 * F3 + 2 * 16 * touched3, "finalize": 32 * n_tex + 32 * N}
                    k3 = {k: {"ms": t3.get(k, 0.0), "bytes": b, "gbs": (b / (t3[k] * 1e-3) / 1e9) if t3.get(k, 0.0) > 0 else None}
                          for k, b in bytes3.items()}
                    whole3 = sum(bytes3.values()) + 16 * F3 + 4 * flat.numel()
                    dom3 = max(k3, key=lambda k: k3[k]["ms"])
                    next_rows["mode3"]["roofline"] = {
                        "bound": "hbm", "kernel": dom3, "achieved": k3[dom3]["gbs"], "peak": peak, "unit": "GB/s",
                        "frac": (k3[dom3]["gbs"] or 0.0) / peak, "traffic": None, "kernels": k3,
                        "whole_step": {"algorithmic_bytes": whole3, "achieved_gbs": whole3 / (ms3 * 1e-3) / 1e9,
                                       "frac": whole3 / (ms3 * 1e-3) / 1e9 / peak},
                        "counts": {"N": N, "N_touched": touched3, "F": F3, "pixels": PT, "longest_list": longest3}}
                except Exception as e:  # noqa: BLE001
                    rast.set_timing(False)
                    next_rows["mode3"]["roofline"] = {"error": repr(e)[:200]}
                del out3, g3
                rast._lists_cache.clear()
                rast._saved = None
                torch.cuda.empty_cache()
        except Exception as e:
            next_rows["error"] = repr(e)[:300]

    # ---- CPU baseline on the host cores (rank 0, N = 1 only)
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        sec, threads = cpu_oracle_run(scene, params, steps=2, warmup=1)
        cpu = {"value": 1.0 / sec, "unit": UNIT, "cores": threads, "kind": "port",
               "sample": "2 timed steps after 1 warm-up; each step = forward+backward of ONE 1920x1080 view of the same "
                         f"{N}-point cloud with the CPU oracle (OpenMP, all host threads)"}

    # ---- parity at the benchmark's own size: view 0 of the cloud that was timed, CUDA library against the CPU oracle
    parity_headline = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        try:
            parity_headline = parity_against_oracle(rast, scene, params)
        except Exception as e:  # noqa: BLE001
            parity_headline = {"error": repr(e)[:300]}

    # ---- the other benchmark configurations
    configs = None
    if not args.no_configs:
        rast._lists_cache.clear()
        rast._saved = None
        torch.cuda.empty_cache()
        try:
            configs = run_configs(args, torch, dist, rast, dev, rank, world, peak)
        except Exception as e:  # noqa: BLE001
            configs = {"error": repr(e)[:300]}

    if rank == 0:
        line = {
            "metric": METRIC, "value": value, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": ms_total / timed_steps, "timed_steps": timed_steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
            "dtype": "f32", "data": "synthetic",
            "config": {"workload": f"headline: {N} planar-scene points replicated, {V} views {W}x{H} f={FOCAL:g} per GPU and "
                                   f"step, {LAYERS} levels, mode {args.mode}, fwd+bwd, L1 vs seeded target"
                                   + (f", gradients of 9 floats per point summed over the ranks ({exchange_kind})" if world > 1 else ""),
                       "views_per_gpu": V, "views_mode": args.views_mode if world > 1 else None, "points": N, "l2": "inputs larger than L2 (cloud 128 MB + descriptors 160 MB + "
                                                              "pyramids; gradient buffer 288 MB rewritten every step)"},
            "clocks": clocks, "e2e": e2e, "e2e_shim": e2e_shim, "gpu_launches": launches, "roofline": roofline, "cpu_baseline": cpu,
            "loss": float(loss.item()), "step_ms": [round(x, 3) for x in step_ms], "cuda_graph": graph_info, "exchange": exchange_kind + ("+overlap" if overlap else ""), "per_rank": per_rank, "next_rows": next_rows,
            "parity_headline": parity_headline, "exchange_check": exchange_check, "configs": configs,
        }
        print(json.dumps(line), flush=True)
    if world > 1:
        # Every rank is idle here (all work synchronised, the line printed).  Releasing graphs that hold NCCL kernels and
        # tearing the process group down has been seen not to return; the result must not depend on that, so a watchdog
        # ends the process if the teardown has not finished after a while.
        import threading

        torch.cuda.synchronize(dev)
        dist.barrier()
        torch.cuda.synchronize(dev)
        sys.stdout.flush()
        watchdog = threading.Timer(20.0, lambda: os._exit(0))
        watchdog.daemon = True
        watchdog.start()
        try:
            dist.destroy_process_group()
        finally:
            # the interpreter's own teardown (graphs, symmetric memory, the libraries' static objects) is skipped as well:
            # everything this process had to report is out
            sys.stdout.flush()
            sys.stderr.flush()
            os._exit(0)


# -------------------------------------------------------------------------------------------------------------
# the other benchmark configurations, reported as blocks beside the headline


def algorithmic_bytes_per_launch(N, F, P_total, touched, n_views, backward):
    """Per launch of n_views views: forward 20 N per view + 36 F + 28 P; backward 32 P + 44 F + 40 N (the zero fill, once)
    + 80 N_t (one read + one write per touched gradient element)."""
    b = 20 * N * n_views + 36 * F + 28 * P_total
    if backward:
        b += 32 * P_total + 44 * F + 40 * N + 80 * touched
    return b


class ConfigRun:
    """One configuration: the scene on the device, seeded random L1 targets, and a step = forward (+ L1 gradient +
    backward into one gradient buffer + epilogue) over `views` in launches of at most `chunk` views."""

    def __init__(self, torch, rast, dev, scene, params, backward=True, want_intrinsics=True, chunk=4, flat=None):
        from vet_b200.render import level_sizes, scene_to_device

        self.torch, self.rast, self.dev, self.scene, self.params = torch, rast, dev, scene, params
        self.backward, self.want_intrinsics, self.chunk = backward, want_intrinsics, chunk
        self.tensors = scene_to_device(scene, dev)
        self.n, self.n_tex = scene.n, scene.texture.shape[1]
        w, h = scene.views[0].w, scene.views[0].h
        self.sizes = level_sizes(w, h, LAYERS)
        self.P = sum(a * b for a, b in self.sizes)
        gen = torch.Generator(device=dev).manual_seed(99)
        self.targets = [torch.rand(chunk, CHANNELS, hh, ww, device=dev, generator=gen) for (ww, hh) in self.sizes]
        self.grads = [torch.empty(chunk, CHANNELS, hh, ww, device=dev) for (ww, hh) in self.sizes]
        self.loss = torch.zeros((), device=dev)
        n, n_tex = self.n, self.n_tex
        self.flat = flat if flat is not None else torch.zeros(4 * n_tex + 4 * n + n_tex, dtype=torch.float32, device=dev)
        self.fragments = {}  # view index -> fragments of the launch it was part of / views in that launch

    def accum(self):
        torch, n, n_tex, flat = self.torch, self.n, self.n_tex, self.flat
        g = dict(desc=flat[:4 * n_tex].view(n_tex, 4), points=flat[4 * n_tex:4 * n_tex + 4 * n].view(n, 4),
                 conf=flat[4 * n_tex + 4 * n:4 * n_tex + 4 * n + n_tex], background=torch.zeros(CHANNELS, device=self.dev),
                 pose=torch.zeros(self.scene.poses.shape[0], 6, dtype=torch.float64, device=self.dev),
                 pose_count=torch.zeros(self.scene.poses.shape[0], device=self.dev))
        if self.want_intrinsics:
            g["intrinsics"] = torch.zeros(self.scene.intrinsics.shape[0], 13, device=self.dev)
            g["intrinsics_count"] = torch.zeros(self.scene.intrinsics.shape[0], device=self.dev)
        return g

    def local_step(self, view_ids, read_counts=False):
        """Forward (+ backward) of the given views; returns the raw gradient dict (or None)."""
        rast = self.rast
        g = None
        if self.backward:
            self.flat.zero_()
            g = self.accum()
        for c0 in range(0, len(view_ids), self.chunk):
            ids = view_ids[c0:c0 + self.chunk]
            views = [self.scene.views[i] for i in ids]
            out = rast.forward(*self.tensors, views, self.params, want_weight=True)
            if read_counts:
                F, longest = rast.fragment_count()
                for i in ids:
                    self.fragments[i] = (F / len(ids), longest)
            if self.backward:
                k = len(ids)
                rast.l1_loss_grad(out["color"], [t[:k] for t in self.targets], [t[:k] for t in self.grads], self.loss)
                rast.backward_raw([t[:k] for t in self.grads], want_intrinsics=self.want_intrinsics, accum=g)
        return g

    def time_local(self, view_ids, reps=5, warmup=2, finalize=True):
        torch = self.torch
        st = torch.cuda.current_stream(self.dev)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for it in range(warmup + reps):
            if it == warmup:
                e0.record(st)
            g = self.local_step(view_ids)
            if g is not None and finalize:
                fin = self.rast.finalize(g)
        e1.record(st)
        torch.cuda.synchronize(self.dev)
        return e0.elapsed_time(e1) / reps


def config_block(torch, rast, dev, scene, params, peak, workload, backward=True, want_intrinsics=True, cpu=True, parity=True):
    """frames/s, fraction of the HBM roofline, CPU frames/s and parity (view 0) of one single-GPU configuration."""
    run = ConfigRun(torch, rast, dev, scene, params, backward=backward, want_intrinsics=want_intrinsics)
    ids = list(range(len(scene.views)))
    g = run.local_step(ids, read_counts=True)
    F = sum(run.fragments[i][0] for i in ids)
    longest = max(run.fragments[i][1] for i in ids)
    touched = int(torch.count_nonzero(g["points"][:, 3]).item()) if g is not None else 0
    ms = run.time_local(ids)
    V = len(ids)
    launches = [ids[c0:c0 + run.chunk] for c0 in range(0, V, run.chunk)]
    bytes_step = sum(algorithmic_bytes_per_launch(scene.n, F * len(l) / V, run.P * len(l), touched if k == 0 else 0, len(l), backward)
                     for k, l in enumerate(launches))
    gbs = bytes_step / (ms * 1e-3) / 1e9
    block = {"workload": workload, "ms_per_step": ms, "frames_per_s": V / (ms * 1e-3), "views_per_step": V,
             "counts": {"N": scene.n, "F": int(F), "pixels": run.P * V, "N_touched": touched, "longest_list": int(longest)},
             "roofline": {"bound": "hbm", "algorithmic_bytes": int(bytes_step), "achieved": gbs, "peak": peak, "unit": "GB/s",
                          "frac": gbs / peak}}
    del run
    rast._lists_cache.clear()
    rast._saved = None
    torch.cuda.empty_cache()
    if cpu:
        sec, threads = cpu_oracle_run(scene, params, steps=1, warmup=0, backward=backward)
        block["cpu_baseline"] = {"value": 1.0 / sec, "unit": UNIT, "cores": threads, "kind": "port",
                                 "sample": "one view of this configuration, forward" + (" + backward" if backward else "")}
    if parity:
        try:
            # (the sorted lists are compared too: keep them even where the timed configuration does not)
            block["parity"] = parity_against_oracle(rast, scene, dict(params, keep_sorted_lists=1), backward=backward)
        except Exception as e:  # noqa: BLE001
            block["parity"] = {"error": repr(e)[:300]}
        rast._lists_cache.clear()
        rast._saved = None
        torch.cuda.empty_cache()
    return block


def balanced_assignment(costs, world):
    """Views -> ranks, longest processing time first: the next most expensive view goes to the least loaded rank."""
    load, mine = [0.0] * world, [[] for _ in range(world)]
    for v in sorted(range(len(costs)), key=lambda i: -costs[i]):
        r = min(range(world), key=lambda k: (load[k], k))
        load[r] += costs[v]
        mine[r].append(v)
    return [sorted(m) for m in mine], load


def run_configs(args, torch, dist, rast, dev, rank, world, peak):
    from vet_b200 import scenes
    from vet_b200.render import default_params

    out = {}
    p1 = default_params(render_mode=1, num_layers=LAYERS, num_channels=CHANNELS)
    if world == 1 and rank == 0:
        sc = scenes.config_planar(3_000_000, W, H, FOCAL, n_views=1, seed=2002, channels=CHANNELS)
        out["config2_viewer_frame"] = config_block(
            torch, rast, dev, sc, dict(p1, keep_sorted_lists=0), peak,
            "3 M planar-scene points, one 1920x1080 view (f = 1200), 4 levels, forward only", backward=False)
        sc = scenes.config_planar(8_000_000, 1024, 768, 900.0, n_views=4, seed=2002, channels=CHANNELS)
        out["config3_training_step"] = config_block(
            torch, rast, dev, sc, p1, peak,
            "8 M planar-scene points, 4 views 1024x768 (f = 900), forward + backward with gradients to descriptors, "
            "confidences, positions, pose and intrinsics")
        sc = scenes.config_shells()
        out["config4_scene_in_shells"] = config_block(
            torch, rast, dev, sc, p1, peak,
            "5 M planar-scene points + 4 shells of 1 M points (radii 10/20/40/80), one 1920x1080 view from the scene "
            "centre, forward + backward")
        del sc

    # configuration 5: ONE fixed batch of 32 distinct 1920x1080 views of a 20 M-point cloud, sharded over the ranks
    # (strong scaling of the batch: N = 1 renders all 32), gradients of 9 floats per point summed over the ranks.
    n5, views5 = 20_000_000, 32
    sc = scenes.config_planar(n5, W, H, FOCAL, n_views=views5, seed=5005, channels=CHANNELS)
    peer = None
    if world > 1 and args.exchange != "nccl":
        try:
            from vet_b200.dist import PeerExchange

            peer = PeerExchange(rast, sc.n, sc.texture.shape[1], CHANNELS, dev,
                                multicast=None if args.exchange == "auto" else args.exchange == "multicast")
            peer.ctas_per_sm = args.exchange_ctas
        except Exception:  # noqa: BLE001
            peer = None
        ok = torch.tensor([0.0 if peer is None else 1.0], device=dev)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if ok.item() < 1.0:
            peer = None
    run = ConfigRun(torch, rast, dev, sc, p1, want_intrinsics=False, flat=None if peer is None else peer.raw)
    st = torch.cuda.current_stream(dev)

    def sharded_step(mine):
        g = run.local_step(mine)
        if peer is not None:
            return peer.run(g)
        if world > 1:
            dist.all_reduce(run.flat)
            dist.all_reduce(g["pose"])
            dist.all_reduce(g["pose_count"])
        return rast.finalize(g)

    def time_sharded(assignment, reps=3, warmup=1):
        mine = assignment[rank]
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        for _ in range(warmup):
            sharded_step(mine)
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize(dev)
        e0.record(st)
        for _ in range(reps):
            sharded_step(mine)
        e1.record(st)
        torch.cuda.synchronize(dev)
        c0.record(st)  # this rank's own work without the exchange: how unequal the shards are
        run.local_step(mine)
        c1.record(st)
        torch.cuda.synchronize(dev)
        t = torch.tensor([e0.elapsed_time(e1) / reps, c0.elapsed_time(c1)], dtype=torch.float64, device=dev)
        per = [torch.zeros_like(t) for _ in range(world)]
        if world > 1:
            dist.all_gather(per, t)
        else:
            per = [t]
        step_ms = max(float(x[0].item()) for x in per)
        local = [float(x[1].item()) for x in per]
        return step_ms, local

    # per-view cost (what a training loop knows from the previous epoch): every rank renders its round-robin share one
    # view per launch, forward + backward, and times each view on the device; fragments are counted on the way
    round_robin = [[v for v in range(views5) if v % world == r] for r in range(world)]
    run.chunk = 1
    cost = torch.zeros(views5, dtype=torch.float64, device=dev)
    frag = torch.zeros(views5, dtype=torch.float64, device=dev)
    v0, v1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    for v in round_robin[rank]:
        run.local_step([v], read_counts=True)  # untimed: sizes the scratch of a one-view launch, reads the fragment count
        v0.record(st)
        run.local_step([v])
        v1.record(st)
        torch.cuda.synchronize(dev)
        cost[v] = v0.elapsed_time(v1)
        frag[v] = run.fragments[v][0]
    run.chunk = 4
    if world > 1:
        dist.all_reduce(cost)
        dist.all_reduce(frag)
    frag = [float(x) for x in frag.tolist()]
    costs = [float(x) for x in cost.tolist()]
    balanced, load = balanced_assignment(costs, world)
    rr_ms, rr_local = time_sharded(round_robin)
    bal_ms, bal_local = (rr_ms, rr_local) if world == 1 else time_sharded(balanced)
    F5 = sum(frag)
    touched = 0
    block = {"workload": f"{n5} planar-scene points replicated, one batch of {views5} distinct 1920x1080 views sharded over "
                         f"{world} GPU(s), forward + backward, 9 gradient floats per point summed over the ranks"
                         + (f" ({'multicast' if peer is not None and peer.multicast else 'peer' if peer is not None else 'nccl'})" if world > 1 else ""),
             "scaling": "strong", "n_gpus": world, "views_per_step": views5,
             "round_robin": {"ms_per_step": rr_ms, "frames_per_s": views5 / (rr_ms * 1e-3), "local_ms_per_rank": [round(x, 3) for x in rr_local],
                             "slowest_over_fastest_rank": max(rr_local) / max(min(rr_local), 1e-9)},
             "balanced_by_view_cost": {"ms_per_step": bal_ms, "frames_per_s": views5 / (bal_ms * 1e-3),
                                       "local_ms_per_rank": [round(x, 3) for x in bal_local],
                                       "slowest_over_fastest_rank": max(bal_local) / max(min(bal_local), 1e-9),
                                       "views_per_rank": [len(m) for m in balanced]},
             "fragments_per_view": {"min": min(frag), "max": max(frag), "total": F5},
             "ms_per_view_alone": {"min": min(costs), "max": max(costs)},
             "exchange_bytes_per_rank": 36 * n5}
    best = min(rr_ms, bal_ms)
    bytes_step = sum(algorithmic_bytes_per_launch(n5, F5 * 4 / views5, run.P * 4, 0, 4, True) for _ in range(views5 // 4)) + 80 * n5
    block["roofline"] = {"bound": "hbm", "algorithmic_bytes": int(bytes_step), "achieved": bytes_step / world / (best * 1e-3) / 1e9,
                         "peak": peak, "unit": "GB/s per GPU", "frac": bytes_step / world / (best * 1e-3) / 1e9 / peak}
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        sec, threads = cpu_oracle_run(sc, p1, steps=1, warmup=0)
        block["cpu_baseline"] = {"value": 1.0 / sec, "unit": UNIT, "cores": threads, "kind": "port",
                                 "sample": "one view of this configuration, forward + backward"}
    out["config5_sharded_batch"] = block
    return out


# DRAM traffic of each kernel relative to its algorithmic bytes, from the ncu captures summarised under profiles/
# (dram__bytes_read.sum + dram__bytes_write.sum of one launch of a small case: 2 M points, 1 view, 3.32 M fragments,
# divided by the algorithmic bytes of that launch).  The full-size workload is too large to capture with --set full;
# traffic is taken to grow in proportion to the algorithmic bytes.
TRAFFIC_OVER_ALGORITHMIC = {
    # pack_images_kernel + backward_kernel (the "backward" pass that is timed as one)
    "backward": (88.13e6 + 37.15e6 + 237.17e6 + 34.80e6) / 228.388e6,
    "point_backward": (79.19e6 + 3.93e6) / 82.153e6,
    "sort_blend": (117.44e6 + 104.31e6) / 185.585e6,
    "count": 42.51e6 / 43.016e6,
    # the collection pass writes the whole 32-byte record (key + what the blend gathers), not only the 8-byte key
    "collect": (67.49e6 + 85.40e6) / 58.553e6,
}


def main():
    args = parse_args()
    if args.impl == "reference":
        run_reference(args)
    else:
        run_ours(args)


if __name__ == "__main__":
    main()
