"""Host-side mirror of the reference's render operator on top of the C ABI.

`Rasterizer` plays the role of PointRendererCache + BlendPointCloudForward / BlendPointCloudBackward
(rendering/PointRenderer.h:112-248, PointRenderer.cu:657-1069, 1111-1323): it owns the per-call scratch
(the reference caches it between calls and re-allocates when (C, N, L, B, h, w) changes, PointRenderer.cu:313-336),
sequences forward and backward, and returns the tensors in the reference's layouts.  torch is used for device
memory and streams only; all arithmetic happens in libvetr.so.  Batches larger than the library's per-launch view
limit are processed in groups.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional, Sequence

import torch

from . import _lib as L


def default_params(**kw) -> dict:
    """RenderParams defaults the kernels read (data/Settings.h:27-73)."""
    p = dict(render_mode=L.MODE_FULL_BLEND, num_layers=4, num_channels=4, drop_out_points_by_radius=1,
             drop_out_radius_threshold=0.6, dist_cutoff=20.0, use_environment_map=0, viewer_only=0,
             stability_cutoff_value=10000.0, debug_max_list_length=-1, need_point_gradient=1,
             K_gradient_factor=0.5, distortion_gradient_factor=0.005, output_background_mask_value=0.0,
             background_alpha_to_point0=1, keep_sorted_lists=1, depth_accept_blend=0.01,
             depth_accept=0.01, ghost_gradients=0)
    p.update(kw)
    return p


def level_sizes(w: int, h: int, num_layers: int):
    out = []
    for _ in range(num_layers):
        out.append((w, h))
        w //= 2
        h //= 2
    return out


def _ptr(t: Optional[torch.Tensor]):
    return None if t is None else C.c_void_p(t.data_ptr())


def _ptr_array(ts: Optional[Sequence[torch.Tensor]]):
    if ts is None:
        return None
    return (C.c_void_p * len(ts))(*[t.data_ptr() for t in ts])


class FragmentLists:
    """Device buffers of vetr_lists for one group of views."""

    def __init__(self, device, n_pixels_total: int, capacity: int):
        i32 = dict(dtype=torch.int32, device=device)
        self.capacity = int(capacity)
        self.counts = torch.empty(n_pixels_total, **i32)
        self.ends = torch.empty(n_pixels_total, **i32)
        self.frags = torch.empty(max(self.capacity, 1), 4, dtype=torch.int64, device=device)  # 32-byte records
        self.status = torch.zeros(4, **i32)
        n_items = int(L.lib().vetr_item_table_entries(self.capacity, n_pixels_total))
        self.items = torch.empty(n_items, **i32)
        self.c = L.Lists(self.counts.data_ptr(), self.ends.data_ptr(), self.frags.data_ptr(), self.capacity,
                         self.status.data_ptr(), self.items.data_ptr(), n_items, None, None, None)
        self.level_mask = None
        self.point_grad = None
        self.pixel_scratch = None
        self.n_pixels_total = n_pixels_total

    def ensure_pixel_scratch(self):
        """[n_pixels*8] floats of backward scratch (channel-interleaved forward image and its gradient)."""
        if self.pixel_scratch is None:
            self.pixel_scratch = torch.empty(max(self.n_pixels_total, 1) * 8, dtype=torch.float32, device=self.counts.device)
            self.c.pixel_scratch = self.pixel_scratch.data_ptr()

    def ensure_level_mask(self, n_entries: int):
        """[n_views*n] bytes written by the forward pass (which levels of a view hold a fragment of a point)."""
        if self.level_mask is None or self.level_mask.numel() < n_entries:
            self.level_mask = torch.empty(max(n_entries, 1), dtype=torch.uint8, device=self.counts.device)
            self.c.level_mask = self.level_mask.data_ptr()

    def ensure_point_grad(self, n_floats: int):
        """[n_views*num_layers*n*2] floats of backward scratch (image-space gradient per fragment)."""
        if self.point_grad is None or self.point_grad.numel() < n_floats:
            self.point_grad = torch.empty(max(n_floats, 1), dtype=torch.float32, device=self.counts.device)
            self.c.point_grad = self.point_grad.data_ptr()


class Rasterizer:
    """One context (device + stream).  Inputs are CUDA tensors in the reference's layouts."""

    def __init__(self, device: int = 0, stream: Optional[torch.cuda.Stream] = None):
        if not torch.cuda.is_available():
            raise RuntimeError("vet_b200.Rasterizer needs a CUDA device; there is no CPU path")
        self.device = torch.device("cuda", device)
        self._ctx = C.c_void_p()
        st = C.c_void_p(stream.cuda_stream) if stream is not None else None
        self._stream = stream
        rc = L.lib().vetr_create(C.byref(self._ctx), device, st)
        if rc != L.OK:
            raise L.VetrError(rc, "vetr_create")
        self._lists_cache = {}
        self._saved = None
        self._cur_stream = 0 if stream is None else stream.cuda_stream
        self._sync_stream()

    def close(self):
        if self._ctx:
            L.lib().vetr_destroy(self._ctx)
            self._ctx = C.c_void_p()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def _sync_stream(self):
        """Without an explicit stream the context follows torch's current stream (also the capture stream of
        torch.cuda.graph, so a whole step of forward + backward can be recorded into a CUDA graph and replayed)."""
        if self._stream is None:
            cur = torch.cuda.current_stream(self.device).cuda_stream
            if cur != self._cur_stream:
                self._check(L.lib().vetr_set_stream(self._ctx, C.c_void_p(cur)), "vetr_set_stream")
                self._cur_stream = cur

    def _check(self, rc: int, where: str):
        if rc != L.OK:
            raise L.VetrError(rc, where, L.lib().vetr_last_cuda_error(self._ctx))

    # ---- helpers -----------------------------------------------------------------------------------------
    def _views(self, views):
        arr = (L.View * len(views))()
        for i, v in enumerate(views):
            arr[i] = L.View(v.w, v.h, v.image_index, v.camera_index, v.camera_model, (C.c_float * 5)(*v.crop),
                            (C.c_float * 4)(*v.rot))
        return arr

    def _lists(self, slot: int, n_pixels_total: int, capacity: int, exact: bool = False) -> FragmentLists:
        key = (slot, n_pixels_total)
        cur = self._lists_cache.get(key)
        if cur is None or cur.capacity < capacity or (exact and cur.capacity != capacity):
            cur = FragmentLists(self.device, n_pixels_total, capacity)
            self._lists_cache[key] = cur
        return cur

    # ---- forward -----------------------------------------------------------------------------------------
    def forward(self, position, index, texture, confidence, background, poses, intrinsics, views, params: dict,
                dropout=None, capacity: Optional[int] = None, want_weight=True, want_mask=False, want_depth=False):
        """Returns dict(color=[L x [B,C,h,w]], weight=..., mask=..., depth=...).  Keeps what backward() needs."""
        lib = L.lib()
        self._sync_stream()
        prm = L.Params(**{k: params[k] for k, _ in L.Params._fields_})
        B, Cn, Ln = len(views), texture.shape[0], prm.num_layers
        prm.num_channels = Cn
        w, h = views[0].w, views[0].h
        sizes = level_sizes(w, h, Ln)
        P = int(lib.vetr_pyramid_pixels(w, h, Ln))
        if P <= 0:
            raise L.VetrError(L.E_INVALID_ARG, "vetr_pyramid_pixels")
        f32 = dict(dtype=torch.float32, device=self.device)
        color = [torch.empty(B, Cn, hh, ww, **f32) for (ww, hh) in sizes]
        weight = [torch.empty(B, 1, hh, ww, **f32) for (ww, hh) in sizes] if want_weight else None
        mask = [torch.empty(B, 1, hh, ww, **f32) for (ww, hh) in sizes] if want_mask else None
        depth = [torch.empty(B, 1, hh, ww, **f32) for (ww, hh) in sizes] if want_depth else None
        cloud = L.Cloud(position.data_ptr(), index.data_ptr(), position.shape[0])
        tex = L.Texture(texture.data_ptr(), confidence.data_ptr(), background.data_ptr(), texture.shape[1])
        cams = L.Cameras(poses.data_ptr(), intrinsics.data_ptr(), poses.shape[0], intrinsics.shape[0])
        groups = []
        for gi, b0 in enumerate(range(0, B, L.MAX_VIEWS)):
            b1 = min(B, b0 + L.MAX_VIEWS)
            nb = b1 - b0
            cap = capacity if capacity is not None else int(lib.vetr_list_capacity(position.shape[0], nb, w, h, C.byref(prm)))
            lists = self._lists(gi, P * nb, cap, exact=capacity is not None)
            if prm.render_mode == 3 or (prm.render_mode in (1, 2) and prm.need_point_gradient):
                lists.ensure_level_mask(nb * position.shape[0])
            varr = self._views(views[b0:b1])
            sl = lambda ts: None if ts is None else [t[b0:b1] for t in ts]
            dro = None if dropout is None else dropout[b0:b1]
            rc = lib.vetr_forward(self._ctx, C.byref(prm), C.byref(cloud), C.byref(tex), C.byref(cams), varr, nb,
                                  _ptr(dro), C.byref(lists.c), _ptr_array(sl(color)), _ptr_array(sl(weight)),
                                  _ptr_array(sl(mask)), _ptr_array(sl(depth)))
            self._check(rc, "vetr_forward")
            groups.append((b0, b1, lists, varr))
        self._saved = dict(prm=prm, cloud=cloud, tex=tex, cams=cams, groups=groups, color=color, P=P, sizes=sizes,
                           tensors=(position, index, texture, confidence, background, poses, intrinsics, dropout))
        return dict(color=color, weight=weight, mask=mask, depth=depth)

    def fragment_count(self):
        """(total fragments, longest list) of the last forward; synchronises. Raises on key-buffer overflow."""
        self._sync_stream()
        total, longest = 0, 0
        for (_, _, lists, _) in self._saved["groups"]:
            t, m = C.c_int64(), C.c_int32()
            self._check(L.lib().vetr_read_status(self._ctx, C.byref(lists.c), C.byref(t), C.byref(m)), "vetr_read_status")
            total += t.value
            longest = max(longest, m.value)
        return total, longest

    def lists_of(self, view: int, layer: int):
        """Reference layout of one (view, layer): collections [2,F_l] int32 and scanned_counting [h_l*w_l] int32."""
        s = self._saved
        self._sync_stream()
        for (b0, b1, lists, varr) in s["groups"]:
            if b0 <= view < b1:
                w, h = s["sizes"][0]
                n = C.c_int64()
                args = (self._ctx, C.byref(lists.c), w, h, s["prm"].num_layers, b1 - b0, view - b0, layer)
                self._check(L.lib().vetr_get_lists(*args, None, None, C.byref(n)), "vetr_get_lists")
                lw, lh = s["sizes"][layer]
                coll = torch.empty(2, max(n.value, 0), dtype=torch.int32, device=self.device)
                scanned = torch.empty(lw * lh, dtype=torch.int32, device=self.device)
                self._check(L.lib().vetr_get_lists(*args, _ptr(coll), _ptr(scanned), C.byref(n)), "vetr_get_lists")
                return coll, scanned
        raise IndexError(view)

    # ---- backward ----------------------------------------------------------------------------------------
    def backward_raw(self, grad_color, want_points=True, want_pose=True, want_intrinsics=True, accum=None, phases=3):
        """Raw gradient sums of the last forward: dict(desc [n_tex,4], conf [n_tex], points [n,4] (xyz sum, hit count),
        background [C], pose [n_img,6] f64, pose_count, intrinsics [n_cam,13], intrinsics_count).
        `accum` (a dict from an earlier call) accumulates further views into the same buffers.
        `phases`: 1 = the per-fragment kernels only, 2 = the per-point pass only (with the `accum` of the first call and the
        same `grad_color`), 3 = both (vetr_backward_phase)."""
        s = self._saved
        lib = L.lib()
        self._sync_stream()
        position, index, texture = s["tensors"][0], s["tensors"][1], s["tensors"][2]
        poses, intrinsics = s["tensors"][5], s["tensors"][6]
        n, n_tex, Cn = position.shape[0], texture.shape[1], texture.shape[0]
        f32 = dict(dtype=torch.float32, device=self.device)
        g = accum
        if g is None:
            g = dict(desc=torch.zeros(n_tex, 4, **f32), conf=torch.zeros(n_tex, **f32),
                     background=torch.zeros(Cn, **f32))
            if want_points:
                g["points"] = torch.zeros(n, 4, **f32)
            if want_pose:
                g["pose"] = torch.zeros(poses.shape[0], 6, dtype=torch.float64, device=self.device)
                g["pose_count"] = torch.zeros(poses.shape[0], **f32)
            if want_intrinsics:
                g["intrinsics"] = torch.zeros(intrinsics.shape[0], 13, **f32)
                g["intrinsics_count"] = torch.zeros(intrinsics.shape[0], **f32)
        grad_color = [x.contiguous() for x in grad_color]
        for (b0, b1, lists, varr) in s["groups"]:
            oc = [t[b0:b1] for t in s["color"]]
            gc = [t[b0:b1] for t in grad_color]
            dro = s["tensors"][7]
            lists.ensure_pixel_scratch()
            if lists.level_mask is not None:  # 2 floats per (view, level, point), 4 (one per bilinear corner) in mode 3
                per = 4 if s["prm"].render_mode == 3 else 2
                lists.ensure_point_grad((b1 - b0) * s["prm"].num_layers * n * per)
            rc = lib.vetr_backward_phase(self._ctx, C.byref(s["prm"]), C.byref(s["cloud"]), C.byref(s["tex"]),
                                         C.byref(s["cams"]), varr, b1 - b0, _ptr(None if dro is None else dro[b0:b1]),
                                         C.byref(lists.c), _ptr_array(oc), _ptr_array(gc),
                                         _ptr(g["desc"]), _ptr(g["conf"]), _ptr(g.get("points")), _ptr(g["background"]),
                                         _ptr(g.get("pose")), _ptr(g.get("pose_count")), _ptr(g.get("intrinsics")),
                                         _ptr(g.get("intrinsics_count")), phases)
            self._check(rc, "vetr_backward_phase")
        return g

    def finalize(self, g: dict):
        """Raw sums -> the reference's return tensors (PointRenderer.cu:1251-1322): texture [C,n_tex], confidence
        [1,n_tex], background [C], points [n,4] averaged by hit count, pose tangent and intrinsics averaged."""
        self._sync_stream()
        n_tex = g["desc"].shape[0]
        Cn = g["background"].shape[0]
        g_texture = torch.empty(Cn, n_tex, dtype=torch.float32, device=self.device)
        pts, pose, intr = g.get("points"), g.get("pose"), g.get("intrinsics")
        rc = L.lib().vetr_finalize_gradients(
            self._ctx, Cn, n_tex, _ptr(g["desc"]), _ptr(g_texture), 0 if pts is None else pts.shape[0], _ptr(pts), None,
            0 if pose is None else pose.shape[0], _ptr(pose), _ptr(g.get("pose_count")),
            0 if intr is None else intr.shape[0], _ptr(intr), _ptr(g.get("intrinsics_count")))
        self._check(rc, "vetr_finalize_gradients")
        return dict(texture=g_texture, confidence=g["conf"].view(1, -1), background=g["background"], points=pts,
                    pose=pose, intrinsics=intr)

    def grid_loss(self, poses, intrinsics, view, cell_bb_min, cell_bb_len, loss_img, cell_value, cell_access_count,
                  dist_cutoff: float = 20.0):
        """FillSceneGridWithLoss (RenderForward.cu:761-791): adds the L1 loss under every grid cell's projected box to
        cell_value [n_cells] f32 and the number of covered pixels to cell_access_count [n_cells] i32 (both CUDA, in place)."""
        assert cell_bb_min.dtype == torch.float32 and cell_bb_len.dtype == torch.float32 and loss_img.dtype == torch.float32
        assert cell_value.dtype == torch.float32 and cell_access_count.dtype == torch.int32
        assert all(t.is_contiguous() for t in (cell_bb_min, cell_bb_len, loss_img, cell_value, cell_access_count))
        assert loss_img.shape[1] == view.h and loss_img.shape[2] == view.w
        self._sync_stream()
        cams = L.Cameras(poses.data_ptr(), intrinsics.data_ptr(), poses.shape[0], intrinsics.shape[0])
        v = self._views([view])
        rc = L.lib().vetr_grid_loss(self._ctx, C.byref(cams), v, dist_cutoff, cell_bb_min.shape[0], _ptr(cell_bb_min),
                                    _ptr(cell_bb_len), _ptr(loss_img), loss_img.shape[0], _ptr(cell_value),
                                    _ptr(cell_access_count))
        self._check(rc, "vetr_grid_loss")

    def _envmap(self, density, color, radii, up_axis, non_subzero):
        assert density.dtype == torch.float32 and color.dtype == torch.float32 and density.is_contiguous() and color.is_contiguous()
        n_spheres, res = density.shape[-3], density.shape[-1]
        channels = color.shape[-4]
        assert density.shape[-2] == res and tuple(color.shape[-3:]) == (n_spheres, res, res) and len(radii) == n_spheres
        r = (C.c_float * 8)(*([float(x) for x in radii] + [0.0] * (8 - n_spheres)))
        return L.EnvMap(density.data_ptr(), color.data_ptr(), r, n_spheres, res, channels, int(up_axis), int(bool(non_subzero)))

    def envmap_forward(self, poses, intrinsics, views, num_layers, density, color, radii, weight, up_axis=0, non_subzero=False,
                       flags=0, out=None):
        """EnvironmentMapImpl::Sample2 (EnvironmentMap.cu:378-485): samples the sphere textures density [S,R,R] (or
        [1,1,S,R,R]) and color [C,S,R,R] along every pixel's ray, front to back, starting from the transmittance planes
        `weight` (per level [n_views,1,h_l,w_l]).  Returns per level [n_views,C,h_l,w_l]; with ENV_ADD in `flags` the result
        is added to the images given as `out`."""
        self._sync_stream()
        env = self._envmap(density, color, radii, up_axis, non_subzero)
        h, w = views[0].h, views[0].w
        if out is None:
            out = [torch.empty((len(views), env.channels, h >> l, w >> l), dtype=torch.float32, device=density.device)
                   for l in range(num_layers)]
        assert all(t.is_contiguous() and t.dtype == torch.float32 for t in list(weight) + list(out))
        cams = L.Cameras(poses.data_ptr(), intrinsics.data_ptr(), poses.shape[0], intrinsics.shape[0])
        rc = L.lib().vetr_envmap_forward(self._ctx, C.byref(cams), self._views(views), len(views), num_layers, C.byref(env),
                                         _ptr_array(weight), _ptr_array(out), flags)
        self._check(rc, "vetr_envmap_forward")
        return out

    def envmap_backward(self, poses, intrinsics, views, num_layers, density, color, radii, weight, grad_out, up_axis=0,
                        non_subzero=False, flags=0, g_density=None, g_color=None):
        """Adds the gradients of the map's parameters to g_density / g_color (zero-filled when not given) and returns them."""
        self._sync_stream()
        env = self._envmap(density, color, radii, up_axis, non_subzero)
        if g_density is None:
            g_density = torch.zeros_like(density)
        if g_color is None:
            g_color = torch.zeros_like(color)
        assert all(t.is_contiguous() and t.dtype == torch.float32 for t in list(weight) + list(grad_out) + [g_density, g_color])
        cams = L.Cameras(poses.data_ptr(), intrinsics.data_ptr(), poses.shape[0], intrinsics.shape[0])
        rc = L.lib().vetr_envmap_backward(self._ctx, C.byref(cams), self._views(views), len(views), num_layers, C.byref(env),
                                          _ptr_array(weight), _ptr_array(grad_out), flags, _ptr(g_density), _ptr(g_color))
        self._check(rc, "vetr_envmap_backward")
        return g_density, g_color

    def knn_radius(self, position, k: int = 4, out=None):
        """SceneData::ComputeRadius (data/SceneData.cpp:554-597): distance of every point to its k-th nearest other point.
        position: CUDA float32 [n,3] or [n,4].  out: None (a new [n] tensor is returned), or the string "w" to write the
        radius column of a [n,4] position tensor in place (t_position's layout).  Synchronises the stream."""
        assert position.dtype == torch.float32 and position.is_contiguous() and position.dim() == 2 and position.shape[1] in (3, 4)
        self._sync_stream()
        n, stride = position.shape
        if isinstance(out, str):
            assert out == "w" and stride == 4
            rc = L.lib().vetr_knn_radius(self._ctx, position.data_ptr(), 4, n, k, position.data_ptr() + 12, 4)
            self._check(rc, "vetr_knn_radius")
            return position
        if out is None:
            out = torch.empty(n, dtype=torch.float32, device=position.device)
        rc = L.lib().vetr_knn_radius(self._ctx, position.data_ptr(), stride, n, k, out.data_ptr(), 1)
        self._check(rc, "vetr_knn_radius")
        return out

    def remove_points(self, n: int, remove, point_last=(), point_first=()):
        """NeuralScene::RemovePoints (data/NeuralScene.cpp:1156-1239) on the device.  remove: CUDA int64 indices.
        point_last: tensors [..., n] (texture [C,N], confidence [1,N], optimizer moments); point_first: tensors [n, w]
        (t_position [N,4], t_index [N,1]).  Returns (new_index [n] int32: position after the removal or -1,
        the shrunken point_last tensors, the shrunken point_first tensors).  Synchronises the stream once."""
        assert remove.dtype == torch.int64 and remove.is_contiguous() and remove.is_cuda
        self._sync_stream()
        new_index = torch.empty(max(n, 1), dtype=torch.int32, device=self.device)
        kept = C.c_int(0)
        rc = L.lib().vetr_remove_points_plan(self._ctx, n, _ptr(remove) if remove.numel() else None, remove.numel(),
                                             _ptr(new_index), C.byref(kept))
        self._check(rc, "vetr_remove_points_plan")
        k = kept.value
        arrays, outs_last, outs_first = [], [], []
        for t in point_last:
            assert t.is_contiguous() and t.element_size() == 4 and t.shape[-1] == n
            o = torch.empty(tuple(t.shape[:-1]) + (k,), dtype=t.dtype, device=t.device)
            rows = t.numel() // n if n else 1
            arrays.append(L.PointArray(t.data_ptr(), o.data_ptr(), max(rows, 1), 1))
            outs_last.append(o)
        for t in point_first:
            assert t.is_contiguous() and t.element_size() == 4 and t.shape[0] == n and t.dim() == 2
            o = torch.empty((k, t.shape[1]), dtype=t.dtype, device=t.device)
            arrays.append(L.PointArray(t.data_ptr(), o.data_ptr(), 1, t.shape[1]))
            outs_first.append(o)
        if arrays:
            arr = (L.PointArray * len(arrays))(*arrays)
            self._check(L.lib().vetr_gather_points(self._ctx, n, k, _ptr(new_index), arr, len(arrays)), "vetr_gather_points")
        return new_index[:n], outs_last, outs_first

    def l1_loss_grad(self, images, targets, grads, loss):
        """loss (device scalar) = sum over levels of mean |image - target|; grads[l] = sign(image - target) / numel, one launch."""
        self._sync_stream()
        n = len(images)
        numel = (C.c_int64 * n)(*[t.numel() for t in images])
        rc = L.lib().vetr_l1_loss_grad(self._ctx, n, _ptr_array(images), _ptr_array(targets), _ptr_array(grads), numel, _ptr(loss))
        self._check(rc, "vetr_l1_loss_grad")

    def set_timing(self, enable: bool):
        self._sync_stream()
        self._check(L.lib().vetr_set_timing(self._ctx, int(enable)), "vetr_set_timing")

    def timings(self) -> dict:
        """Milliseconds of the most recent launch of every pass (timing must be enabled); synchronises."""
        ms = (C.c_float * len(L.TIMING_NAMES))()
        self._sync_stream()
        self._check(L.lib().vetr_get_timings(self._ctx, ms), "vetr_get_timings")
        return {k: float(ms[i]) for i, k in enumerate(L.TIMING_NAMES)}

    def launch_count(self) -> int:
        return int(L.lib().vetr_launch_count(self._ctx))

    def apply_tangent(self, tangent: torch.Tensor, poses: torch.Tensor):
        """ApplyTangentToPose (PointRenderer.cu:1343-1349), in place."""
        assert tangent.dtype == torch.float64 and poses.dtype == torch.float64
        assert tangent.is_contiguous() and poses.is_contiguous()
        self._sync_stream()
        self._check(L.lib().vetr_apply_tangent(self._ctx, _ptr(tangent), _ptr(poses), poses.shape[0]), "vetr_apply_tangent")


def scene_to_device(scene, device):
    """numpy Scene (vet_b200.scenes) -> CUDA tensors in the order Rasterizer.forward takes them."""
    t = lambda a: torch.from_numpy(a).to(device)
    return (t(scene.position), t(scene.index), t(scene.texture), t(scene.confidence), t(scene.background),
            t(scene.poses), t(scene.intrinsics))
