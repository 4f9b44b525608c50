"""ctypes front end of the CPU oracle (oracle/vet_oracle.cpp).

TEST INFRASTRUCTURE ONLY: imported by tests/, by the smoke check and by the CPU-baseline leg of the
benchmark.  The product package never imports this module.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB = None


class OParams(C.Structure):
    _fields_ = [
        ("render_mode", C.c_int), ("num_layers", C.c_int), ("num_channels", C.c_int),
        ("drop_out_points_by_radius", C.c_int), ("drop_out_radius_threshold", C.c_float),
        ("dist_cutoff", C.c_float), ("use_environment_map", C.c_int), ("viewer_only", C.c_int),
        ("stability_cutoff_value", C.c_float), ("debug_max_list_length", C.c_int),
        ("need_point_gradient", C.c_int), ("K_gradient_factor", C.c_float),
        ("distortion_gradient_factor", C.c_float), ("output_background_mask", C.c_int),
        ("output_background_mask_value", C.c_float), ("conf_grad_quadratic", C.c_int),
        ("background_alpha_to_point0", C.c_int), ("depth_accept_blend", C.c_float), ("depth_accept", C.c_float),
        ("ghost_gradients", C.c_int),
    ]


class OView(C.Structure):
    _fields_ = [("w", C.c_int), ("h", C.c_int), ("image_index", C.c_int), ("camera_index", C.c_int),
                ("camera_model", C.c_int), ("crop", C.c_float * 5), ("rot", C.c_float * 4)]


def build(force: bool = False) -> str:
    path = os.path.join(_HERE, "libvet_oracle.so")
    src = os.path.join(_HERE, "vet_oracle.cpp")
    if force or not os.path.exists(path) or os.path.getmtime(path) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "libvet_oracle.so"], stdout=subprocess.DEVNULL)
    return path


def lib():
    global _LIB
    if _LIB is None:
        _LIB = C.CDLL(build())
        _LIB.vo_create.restype = C.c_void_p
        _LIB.vo_destroy.argtypes = [C.c_void_p]
        _LIB.vo_forward.restype = C.c_int64
        _LIB.vo_pixels_per_view.restype = C.c_int64
        _LIB.vo_pixels_per_view.argtypes = [C.c_void_p]
        _LIB.vo_set_abs_mode.argtypes = [C.c_void_p, C.c_int]
        _LIB.vo_blend.restype = C.c_float
        _LIB.vo_blend.argtypes = [C.c_float] * 4 + [C.c_int]
        _LIB.vo_new_T.restype = C.c_float
        _LIB.vo_new_T.argtypes = [C.c_float] * 2
        _LIB.vo_blending_fac.argtypes = [C.c_float, C.c_float, C.c_void_p, C.c_void_p]
    return _LIB


def default_params(**kw) -> dict:
    p = dict(render_mode=1, num_layers=4, num_channels=4, drop_out_points_by_radius=1,
             drop_out_radius_threshold=0.6, dist_cutoff=20.0, use_environment_map=0, viewer_only=0,
             stability_cutoff_value=10000.0, debug_max_list_length=-1, need_point_gradient=1,
             K_gradient_factor=0.5, distortion_gradient_factor=0.005, output_background_mask=0,
             output_background_mask_value=0.0, conf_grad_quadratic=0, background_alpha_to_point0=1,
             depth_accept_blend=0.01, depth_accept=0.01, ghost_gradients=0)
    p.update(kw)
    return p


def level_sizes(w: int, h: int, L: int):
    out = []
    for _ in range(L):
        out.append((w, h))
        w //= 2
        h //= 2
    return out


def _ptr(a):
    return a.ctypes.data_as(C.c_void_p) if a is not None else None


def _ptr_array(arrs):
    if arrs is None:
        return None
    return (C.c_void_p * len(arrs))(*[a.ctypes.data for a in arrs])


class Oracle:
    """One forward (+ optional backward) of the rasterizer on the CPU."""

    def __init__(self):
        self._h = C.c_void_p(lib().vo_create())
        self._keep = None

    def __del__(self):
        try:
            lib().vo_destroy(self._h)
        except Exception:
            pass

    def forward(self, scene, params: dict, dropout=None, views=None):
        views = scene.views if views is None else views
        B = len(views)
        prm = OParams(**{k: v for k, v in params.items() if k in dict(OParams._fields_)})
        L, Cn = prm.num_layers, scene.channels
        prm.num_channels = Cn
        ov = (OView * B)()
        for i, v in enumerate(views):
            ov[i] = OView(v.w, v.h, v.image_index, v.camera_index, v.camera_model, (C.c_float * 5)(*v.crop),
                          (C.c_float * 4)(*v.rot))
        sizes = level_sizes(views[0].w, views[0].h, L)
        color = [np.zeros((B, Cn, h, w), np.float32) for (w, h) in sizes]
        weight = [np.zeros((B, 1, h, w), np.float32) for (w, h) in sizes]
        mask = [np.zeros((B, 1, h, w), np.float32) for (w, h) in sizes]
        depth = [np.zeros((B, 1, h, w), np.float32) for (w, h) in sizes]
        dro = None if dropout is None else np.ascontiguousarray(dropout, np.float32)
        self._keep = (scene, prm, ov, dro, sizes, B)
        F = lib().vo_forward(self._h, C.byref(prm), C.c_int(scene.n), _ptr(scene.position), _ptr(scene.index),
                             C.c_int(scene.texture.shape[1]), _ptr(scene.texture), _ptr(scene.confidence),
                             _ptr(scene.background), C.c_int(scene.poses.shape[0]), _ptr(scene.poses),
                             C.c_int(scene.intrinsics.shape[0]), _ptr(scene.intrinsics), ov, C.c_int(B), _ptr(dro),
                             _ptr_array(color), _ptr_array(weight), _ptr_array(mask), _ptr_array(depth))
        if F < 0:
            raise ValueError("oracle: invalid arguments")
        self.F = int(F)
        self.P = int(lib().vo_pixels_per_view(self._h))
        return dict(color=color, weight=weight, mask=mask, depth=depth, F=self.F)

    def lists(self):
        """(counts [B*P] int32, keys [F] uint64) of the last forward; keys = depth bits << 32 | point id."""
        B = self._keep[5]
        counts = np.zeros(B * self.P, np.int32)
        keys = np.zeros(self.F, np.uint64)
        lib().vo_get_lists(self._h, _ptr(counts), _ptr(keys))
        return counts, keys

    def backward(self, grad_color, want_points=True, want_pose=True, want_intrinsics=True, magnitudes=False):
        """Raw gradient sums (fp64).  With `magnitudes`, the sums of |addend| instead: the scale against which the
        rounding noise of an fp32 accumulation of the same addends has to be judged."""
        lib().vo_set_abs_mode(self._h, C.c_int(1 if magnitudes else 0))
        scene = self._keep[0]
        Cn, nt, n = scene.channels, scene.texture.shape[1], scene.n
        n_img, n_cam = scene.poses.shape[0], scene.intrinsics.shape[0]
        g = [np.ascontiguousarray(x, np.float32) for x in grad_color]
        out = dict(texture=np.zeros((Cn, nt)), confidence=np.zeros(nt), background=np.zeros(Cn))
        if want_points:
            out.update(points=np.zeros((n, 3)), points_count=np.zeros(n))
        if want_pose:
            out.update(pose=np.zeros((n_img, 6)), pose_count=np.zeros(n_img))
        if want_intrinsics:
            out.update(intrinsics=np.zeros((n_cam, 13)), intrinsics_count=np.zeros(n_cam))
        lib().vo_backward(self._h, _ptr_array(g), _ptr(out["texture"]), _ptr(out["confidence"]),
                          _ptr(out["background"]), _ptr(out.get("points")), _ptr(out.get("points_count")),
                          _ptr(out.get("pose")), _ptr(out.get("pose_count")), _ptr(out.get("intrinsics")),
                          _ptr(out.get("intrinsics_count")))
        lib().vo_set_abs_mode(self._h, C.c_int(0))
        return out


def apply_tangent(tangent: np.ndarray, poses: np.ndarray):
    """In place: poses <- exp(tangent) * poses, tangent <- 0 (both float64)."""
    assert tangent.dtype == np.float64 and poses.dtype == np.float64
    lib().vo_apply_tangent(_ptr(tangent), _ptr(poses), C.c_int(poses.shape[0]))


def threads() -> int:
    return int(lib().vo_threads())


def use_all_host_threads() -> int:
    """Lets the oracle use every core this process may run on, whatever OMP_NUM_THREADS says (process launchers such as
    torchrun set it to 1 for their workers).  Returns the thread count now in use."""
    import os

    try:
        n = len(os.sched_getaffinity(0))
    except AttributeError:
        n = os.cpu_count() or 1
    lib().vo_set_threads(C.c_int(max(1, n)))
    return threads()


def grid_loss(scene, view, bb_min, bb_len, loss_img, dist_cutoff: float = 20.0):
    """FillSceneGridWithLossRasterize on the CPU: returns (value [n_cells] f32, access count [n_cells] i32)."""
    bb_min = np.ascontiguousarray(bb_min, np.float32)
    bb_len = np.ascontiguousarray(bb_len, np.float32)
    loss_img = np.ascontiguousarray(loss_img, np.float32)
    n = bb_min.shape[0]
    ch, h, w = loss_img.shape
    value = np.zeros(n, np.float32)
    count = np.zeros(n, np.int32)
    ov = OView(view.w, view.h, view.image_index, view.camera_index, view.camera_model, (C.c_float * 5)(*view.crop),
               (C.c_float * 4)(*view.rot))
    f = lib().vo_grid_loss
    f.restype = C.c_int
    rc = f(_ptr(scene.poses), _ptr(scene.intrinsics), C.byref(ov), C.c_float(dist_cutoff), C.c_int(n), _ptr(bb_min),
           _ptr(bb_len), _ptr(loss_img), C.c_int(ch), C.c_int(h), C.c_int(w), _ptr(value), _ptr(count))
    if rc != 0:
        raise ValueError("oracle: invalid arguments")
    return value, count


ENV_ADD, ENV_NOT_AT_POINTS, ENV_DEPTH_TEST_WEIGHT = 1, 2, 4


class EnvMap:
    """EnvironmentMapImpl's parameters (rendering/EnvironmentMap.h:286-301) as numpy arrays."""

    def __init__(self, density, color, inner_radius=20.0, radius_factor=5.0, up_axis=0, non_subzero=False):
        self.density = np.ascontiguousarray(density, np.float32)   # [S,R,R]
        self.color = np.ascontiguousarray(color, np.float32)       # [C,S,R,R]
        self.n_spheres, self.resolution = self.density.shape[0], self.density.shape[1]
        self.channels = self.color.shape[0]
        # radii.push_back(inner_radius * pow(radius_factor, i)) into a std::vector<float>, EnvironmentMap.cu:109-113
        self.radii = np.array([np.float32(inner_radius * radius_factor ** i) for i in range(self.n_spheres)], np.float32)
        self.up_axis, self.non_subzero = int(up_axis), bool(non_subzero)


def _oviews(views):
    return (OView * len(views))(*[OView(v.w, v.h, v.image_index, v.camera_index, v.camera_model,
                                        (C.c_float * 5)(*v.crop), (C.c_float * 4)(*v.rot)) for v in views])


def _env_args(env):
    return (_ptr(env.density), _ptr(env.color), _ptr(env.radii), C.c_int(env.n_spheres), C.c_int(env.resolution),
            C.c_int(env.channels), C.c_int(env.up_axis), C.c_int(int(env.non_subzero)))


def envmap_forward(scene, views, num_layers, env, weight, flags=0, out=None):
    """EnvironmentMapImpl::Sample2 on the CPU.  weight: per level [n_views,1,h_l,w_l]; returns per level [n_views,C,h_l,w_l]
    (`out`, when given, is updated in place: the starting images of ENV_ADD)."""
    weight = [np.ascontiguousarray(w, np.float32) for w in weight]
    if out is None:
        out = [np.zeros((len(views), env.channels) + w.shape[-2:], np.float32) for w in weight]
    f = lib().vo_envmap_forward
    f.restype = C.c_int
    rc = f(_ptr(scene.poses), _ptr(scene.intrinsics), _oviews(views), C.c_int(len(views)), C.c_int(num_layers),
           *_env_args(env), _ptr_array(weight), _ptr_array(out), C.c_int(flags))
    if rc != 0:
        raise ValueError("oracle: invalid arguments")
    return out


def envmap_uvz(scene, view, level, env):
    """Sample coordinates [S, h_l*w_l, 3] and hit mask [S, h_l*w_l] of one view and level."""
    w, h = view.w >> level, view.h >> level
    uvz = np.zeros((env.n_spheres, h * w, 3), np.float32)
    hit = np.zeros((env.n_spheres, h * w), np.float32)
    f = lib().vo_envmap_uvz
    f.restype = C.c_int
    f(_ptr(scene.poses), _ptr(scene.intrinsics), C.byref(_oviews([view])[0]), C.c_int(level), _ptr(env.radii),
      C.c_int(env.n_spheres), C.c_int(env.resolution), C.c_int(env.up_axis), _ptr(uvz), _ptr(hit))
    return uvz, hit


def envmap_rays(scene, view, level):
    """World-space ray origin and direction [h_l*w_l, 3] of every pixel of one view and level."""
    w, h = view.w >> level, view.h >> level
    o = np.zeros((h * w, 3), np.float32)
    d = np.zeros((h * w, 3), np.float32)
    f = lib().vo_envmap_rays
    f.restype = C.c_int
    f(_ptr(scene.poses), _ptr(scene.intrinsics), C.byref(_oviews([view])[0]), C.c_int(level), _ptr(o), _ptr(d))
    return o, d


def envmap_backward(scene, views, num_layers, env, weight, grad_out, flags=0):
    """Returns (g_density [S,R,R], g_color [C,S,R,R], mag_density, mag_color); the mag arrays are the sums of the
    absolute addends of every element."""
    weight = [np.ascontiguousarray(w, np.float32) for w in weight]
    grad_out = [np.ascontiguousarray(g, np.float32) for g in grad_out]
    gd, gc = np.zeros_like(env.density), np.zeros_like(env.color)
    md, mc = np.zeros_like(env.density), np.zeros_like(env.color)
    f = lib().vo_envmap_backward
    f.restype = C.c_int
    rc = f(_ptr(scene.poses), _ptr(scene.intrinsics), _oviews(views), C.c_int(len(views)), C.c_int(num_layers),
           *_env_args(env), _ptr_array(weight), _ptr_array(grad_out), C.c_int(flags), _ptr(gd), _ptr(gc), _ptr(md), _ptr(mc))
    if rc != 0:
        raise ValueError("oracle: invalid arguments")
    return gd, gc, md, mc


def knn_radius(xyz, k: int = 4, grid: bool = False):
    """SceneData::ComputeRadius on the CPU: distance of every point to its k-th nearest other point.  All pairs by default;
    grid=True uses a uniform grid (same values, usable on millions of points: the timed CPU baseline of this row)."""
    xyz = np.ascontiguousarray(xyz, np.float32)
    n, stride = xyz.shape
    out = np.zeros(n, np.float32)
    f = lib().vo_knn_radius_grid if grid else lib().vo_knn_radius
    f.restype = C.c_int
    if f(_ptr(xyz), C.c_int(stride), C.c_int(n), C.c_int(k), _ptr(out)) != 0:
        raise ValueError("oracle: invalid arguments")
    return out


def remove_points(n: int, remove, point_last=(), point_first=()):
    """NeuralScene::RemovePoints (data/NeuralScene.cpp:1156-1239) as the reference does it on the host: sort the indices,
    walk the points once to list the ones to keep (:1169-1181), index_select every per-point tensor with that list
    (NeuralTexture.cpp:160-173, my_adam.cpp:107-135).  Returns (new_index [n] int32, shrunken point_last, point_first)."""
    indices = sorted(int(i) for i in remove)
    keep, it = [], 0
    for i in range(n):
        while it < len(indices) and indices[it] < i:   # duplicates and indices already passed
            it += 1
        if it < len(indices) and indices[it] == i:
            it += 1
        else:
            keep.append(i)
    keep = np.asarray(keep, np.int64)
    new_index = np.full(n, -1, np.int32)
    new_index[keep] = np.arange(len(keep), dtype=np.int32)
    return (new_index, [np.ascontiguousarray(np.take(a, keep, axis=-1)) for a in point_last],
            [np.ascontiguousarray(np.take(a, keep, axis=0)) for a in point_first])


def project_with_backward(pos4, pose8, intr13, view, level_scale, grad2, dist_cutoff=20.0):
    """(image position at the level + z [3], gradients [22] = point 3, pose tangent 6, K 5, distortion 8) of one point, or
    None for the gradients when the point is behind the camera."""
    pos4, intr13 = np.ascontiguousarray(pos4, np.float32), np.ascontiguousarray(intr13, np.float32)
    pose8, grad2 = np.ascontiguousarray(pose8, np.float64), np.ascontiguousarray(grad2, np.float32)
    out, g = np.zeros(3, np.float32), np.zeros(22, np.float32)
    f = lib().vo_project_with_backward
    f.restype = C.c_int
    rc = f(_ptr(pos4), _ptr(pose8), _ptr(intr13), C.byref(_oviews([view])[0]), C.c_float(level_scale), _ptr(grad2),
           C.c_float(dist_cutoff), _ptr(out), _ptr(g))
    return out, (g if rc == 0 else None)
