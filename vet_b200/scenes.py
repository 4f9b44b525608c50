"""Seeded synthetic scenes for the rasterizer: the five benchmark configurations and small test scenes.

The reference measures on captured scenes that are not redistributable; these generators stand in for
them with the same tensor layouts the rasterizer consumes:

    position   [N,4] f32   xyz + drop-out radius        (rendering/NeuralPointCloudCuda.cpp:38-44)
    index      [N]   i32   point -> descriptor column   (rendering/NeuralPointCloudCuda.cpp:62-67)
    texture    [C,N] f32   channel-major descriptors    (models/NeuralTexture.h:114-116)
    confidence [N]   f32   in (0,1)                     (models/NeuralTexture.h:120-122)
    background [C]   f32                                (models/NeuralTexture.h:125)
    poses      [n,8] f64   world->camera, quaternion xyzw + translation + pad (data/NeuralStructure.h:30-34)
    intrinsics [n,13] f32  fx fy cx cy s + 8 distortion coefficients          (data/NeuralStructure.h:56-59)

Points are ordered as the reference's preprocessing orders them (data/SceneData.cpp:105-108): by Morton code
of the position, then whole blocks of 256 points shuffled.  The drop-out radius follows the reference's rule
(data/SceneData.cpp:566-596): a neighbour distance scaled by sqrt(1/u), u uniform; the neighbour distance is
taken from the generator's known surface density instead of a k-nearest-neighbour search.
"""
from __future__ import annotations

import dataclasses
import math

import numpy as np


@dataclasses.dataclass
class View:
    """ReducedImageInfo (data/SceneData.h:39-50)."""

    w: int
    h: int
    image_index: int = 0
    camera_index: int = 0
    camera_model: int = 0  # 0 = pinhole + distortion
    crop: tuple = (1.0, 1.0, 0.0, 0.0, 0.0)  # fx fy cx cy s
    rot: tuple = (1.0, 0.0, 0.0, 1.0)  # row-major 2x2


@dataclasses.dataclass
class Scene:
    position: np.ndarray
    index: np.ndarray
    texture: np.ndarray
    confidence: np.ndarray
    background: np.ndarray
    poses: np.ndarray
    intrinsics: np.ndarray
    views: list

    @property
    def n(self) -> int:
        return self.position.shape[0]

    @property
    def channels(self) -> int:
        return self.texture.shape[0]


# ---------------------------------------------------------------------------------------------------------
# ordering


def _part1by2(v: np.ndarray) -> np.ndarray:
    v = v.astype(np.uint64) & np.uint64(0x1FFFFF)
    v = (v | (v << np.uint64(32))) & np.uint64(0x1F00000000FFFF)
    v = (v | (v << np.uint64(16))) & np.uint64(0x1F0000FF0000FF)
    v = (v | (v << np.uint64(8))) & np.uint64(0x100F00F00F00F00F)
    v = (v | (v << np.uint64(4))) & np.uint64(0x10C30C30C30C30C3)
    v = (v | (v << np.uint64(2))) & np.uint64(0x1249249249249249)
    return v


def morton_block_order(xyz: np.ndarray, rng: np.random.Generator, block: int = 256) -> np.ndarray:
    """Permutation: Morton order of the normalised positions, then blocks of `block` points shuffled."""
    lo = xyz.min(axis=0)
    span = np.maximum(xyz.max(axis=0) - lo, 1e-12)
    q = np.clip(((xyz - lo) / span * (2**21 - 1)).astype(np.int64), 0, 2**21 - 1)
    code = _part1by2(q[:, 0]) | (_part1by2(q[:, 1]) << np.uint64(1)) | (_part1by2(q[:, 2]) << np.uint64(2))
    order = np.argsort(code, kind="stable")
    n = order.shape[0]
    nb = (n + block - 1) // block
    perm_blocks = rng.permutation(nb)
    idx = (perm_blocks[:, None] * block + np.arange(block)[None, :]).reshape(-1)
    idx = idx[idx < n]
    return order[idx]


# ---------------------------------------------------------------------------------------------------------
# cameras


def _quat_from_matrix(R: np.ndarray) -> np.ndarray:
    """Rotation matrix -> quaternion (x, y, z, w)."""
    t = np.trace(R)
    if t > 0:
        s = math.sqrt(t + 1.0) * 2
        w = 0.25 * s
        x = (R[2, 1] - R[1, 2]) / s
        y = (R[0, 2] - R[2, 0]) / s
        z = (R[1, 0] - R[0, 1]) / s
    elif R[0, 0] > R[1, 1] and R[0, 0] > R[2, 2]:
        s = math.sqrt(1.0 + R[0, 0] - R[1, 1] - R[2, 2]) * 2
        w = (R[2, 1] - R[1, 2]) / s
        x = 0.25 * s
        y = (R[0, 1] + R[1, 0]) / s
        z = (R[0, 2] + R[2, 0]) / s
    elif R[1, 1] > R[2, 2]:
        s = math.sqrt(1.0 + R[1, 1] - R[0, 0] - R[2, 2]) * 2
        w = (R[0, 2] - R[2, 0]) / s
        x = (R[0, 1] + R[1, 0]) / s
        y = 0.25 * s
        z = (R[1, 2] + R[2, 1]) / s
    else:
        s = math.sqrt(1.0 + R[2, 2] - R[0, 0] - R[1, 1]) * 2
        w = (R[1, 0] - R[0, 1]) / s
        x = (R[0, 2] + R[2, 0]) / s
        y = (R[1, 2] + R[2, 1]) / s
        z = 0.25 * s
    q = np.array([x, y, z, w], dtype=np.float64)
    return q / np.linalg.norm(q)


def look_at_pose(eye, target, up=(0.0, -1.0, 0.0)) -> np.ndarray:
    """World->camera pose row [qx qy qz qw tx ty tz 0] for a camera at `eye` looking at `target`
    (+z forward, +y down in the image)."""
    eye = np.asarray(eye, dtype=np.float64)
    fwd = np.asarray(target, dtype=np.float64) - eye
    fwd /= np.linalg.norm(fwd)
    down = -np.asarray(up, dtype=np.float64)
    right = np.cross(down, fwd)
    if np.linalg.norm(right) < 1e-8:
        right = np.cross(np.array([1.0, 0.0, 0.0]), fwd)
    right /= np.linalg.norm(right)
    down = np.cross(fwd, right)
    R_cw = np.stack([right, down, fwd], axis=1)  # camera -> world
    R_wc = R_cw.T
    t = -R_wc @ eye
    return np.concatenate([_quat_from_matrix(R_wc), t, [0.0]])


def pinhole_intrinsics(fx, fy, cx, cy) -> np.ndarray:
    k = np.zeros(13, dtype=np.float32)
    k[:4] = (fx, fy, cx, cy)
    return k


def orbit_poses(rng: np.random.Generator, n: int, radius: float, target=(0, 0, 0)) -> np.ndarray:
    poses = []
    for _ in range(n):
        az = rng.uniform(0, 2 * math.pi)
        el = rng.uniform(math.radians(-20), math.radians(30))
        r = radius * rng.uniform(0.85, 1.15)
        eye = np.array([r * math.cos(el) * math.cos(az), -r * math.sin(el), r * math.cos(el) * math.sin(az)])
        poses.append(look_at_pose(eye + np.asarray(target, dtype=np.float64), target))
    return np.stack(poses)


# ---------------------------------------------------------------------------------------------------------
# clouds


def _radius_from_density(rho: np.ndarray, rng: np.random.Generator) -> np.ndarray:
    u = rng.uniform(1e-3, 1.0, size=rho.shape[0])
    return (np.sqrt(4.0 / (math.pi * rho)) * np.sqrt(1.0 / u)).astype(np.float32)


def cube_surface_points(n: int, rng: np.random.Generator, jitter: float = 0.005):
    """n points on the surface of the unit cube centred at the origin, Gaussian jitter; returns xyz, radius."""
    face = rng.integers(0, 6, size=n)
    uv = rng.uniform(-0.5, 0.5, size=(n, 2))
    xyz = np.empty((n, 3))
    axis = face // 2
    sign = np.where(face % 2 == 0, -0.5, 0.5)
    for a in range(3):
        m = axis == a
        others = [k for k in range(3) if k != a]
        xyz[m, a] = sign[m]
        xyz[m, others[0]] = uv[m, 0]
        xyz[m, others[1]] = uv[m, 1]
    xyz += rng.normal(0.0, jitter, size=xyz.shape)
    rho = np.full(n, n / 6.0)
    return xyz, _radius_from_density(rho, rng)


def planar_scene_points(n: int, rng: np.random.Generator, n_planes: int = 40, box: float = 20.0,
                        outlier_frac: float = 0.05, jitter: float = 0.01):
    """Union of random rectangles (sides 2-10 units, random orientation, centres inside the box) plus
    uniform outliers; returns xyz, radius."""
    n_out = int(round(n * outlier_frac))
    n_pl = n - n_out
    ext = rng.uniform(2.0, 10.0, size=(n_planes, 2))
    area = ext[:, 0] * ext[:, 1]
    centers = rng.uniform(-box / 2 + 3.0, box / 2 - 3.0, size=(n_planes, 3))
    bases = []
    for _ in range(n_planes):
        q, _ = np.linalg.qr(rng.normal(size=(3, 3)))
        bases.append(q)
    counts = np.floor(area / area.sum() * n_pl).astype(np.int64)
    counts[0] += n_pl - counts.sum()
    xyz_parts, rho_parts = [], []
    for k in range(n_planes):
        c = int(counts[k])
        uv = rng.uniform(-0.5, 0.5, size=(c, 2)) * ext[k]
        p = centers[k] + uv[:, :1] * bases[k][:, 0] + uv[:, 1:] * bases[k][:, 1]
        xyz_parts.append(p + rng.normal(0.0, jitter, size=p.shape))
        rho_parts.append(np.full(c, c / area[k]))
    xyz = np.concatenate(xyz_parts)
    radius = _radius_from_density(np.concatenate(rho_parts), rng)
    if n_out:
        out = rng.uniform(-box / 2, box / 2, size=(n_out, 3))
        rho_vol = n_out / box**3
        u = rng.uniform(1e-3, 1.0, size=n_out)
        r_out = ((3.0 * 4.0 / (4.0 * math.pi * rho_vol)) ** (1.0 / 3.0) * np.sqrt(1.0 / u)).astype(np.float32)
        xyz = np.concatenate([xyz, out])
        radius = np.concatenate([radius, r_out])
    return xyz, radius


def fibonacci_shell_points(n: int, radius: float, rng: np.random.Generator):
    """Fibonacci-sphere placement on a shell (data/NeuralScene.cpp:582-646) with a seeded random rotation."""
    i = np.arange(n) + 0.5
    phi = np.arccos(1 - 2 * i / n)
    theta = math.pi * (1 + 5**0.5) * i
    xyz = radius * np.stack([np.cos(theta) * np.sin(phi), np.sin(theta) * np.sin(phi), np.cos(phi)], axis=1)
    q, _ = np.linalg.qr(rng.normal(size=(3, 3)))
    xyz = xyz @ q.T
    rho = np.full(n, n / (4 * math.pi * radius**2))
    return xyz, _radius_from_density(rho, rng)


def _assemble(xyz, radius, rng, channels, confidence_kind, poses, intrinsics, views, reorder=True) -> Scene:
    n = xyz.shape[0]
    if reorder:
        perm = morton_block_order(xyz, rng)
        xyz, radius = xyz[perm], radius[perm]
    position = np.concatenate([xyz.astype(np.float32), radius.astype(np.float32)[:, None]], axis=1)
    texture = rng.standard_normal(size=(channels, n)).astype(np.float32)
    if confidence_kind == "logit":  # sigmoid(10 * U(-2,2)), models/NeuralTexture.h:38-41
        raw = rng.uniform(-2.0, 2.0, size=n)
        confidence = (1.0 / (1.0 + np.exp(-10.0 * raw))).astype(np.float32)
    else:
        confidence = rng.uniform(0.0, 1.0, size=n).astype(np.float32)
    background = np.full(channels, -1.0, dtype=np.float32)  # models/NeuralTexture.cpp:31
    return Scene(np.ascontiguousarray(position), np.arange(n, dtype=np.int32), texture, confidence, background,
                 np.ascontiguousarray(poses, dtype=np.float64), np.ascontiguousarray(intrinsics, dtype=np.float32),
                 views)


def config_plumbing(n: int = 100_000, size: int = 512, seed: int = 1001, channels: int = 4) -> Scene:
    """Config 1: points on the unit-cube surface, one 512x512 view (f=450) at distance 3 looking at the origin."""
    rng = np.random.default_rng(seed)
    xyz, radius = cube_surface_points(n, rng)
    az, el = rng.uniform(0, 2 * math.pi), rng.uniform(0.2, 0.6)
    eye = 3.0 * np.array([math.cos(el) * math.cos(az), -math.sin(el), math.cos(el) * math.sin(az)])
    poses = look_at_pose(eye, (0, 0, 0))[None]
    f = 450.0 * size / 512.0
    intr = pinhole_intrinsics(f, f, size / 2, size / 2)[None]
    return _assemble(xyz, radius, rng, channels, "logit", poses, intr, [View(size, size)])


def config_planar(n: int, w: int, h: int, f: float, n_views: int = 1, seed: int = 2002, channels: int = 4,
                  confidence_kind: str = "uniform", orbit_radius: float = 9.0) -> Scene:
    """Configs 2, 3, 5 and the headline: planar scene, `n_views` pinhole views on a seeded random orbit."""
    rng = np.random.default_rng(seed)
    xyz, radius = planar_scene_points(n, rng)
    poses = orbit_poses(rng, n_views, orbit_radius)
    intr = pinhole_intrinsics(f, f, w / 2, h / 2)[None]
    views = [View(w, h, image_index=i) for i in range(n_views)]
    return _assemble(xyz, radius, rng, channels, confidence_kind, poses, intr, views)


def config_shells(n_scene: int = 5_000_000, n_shell: int = 1_000_000, w: int = 1920, h: int = 1080, f: float = 1200.0,
                  seed: int = 4004, channels: int = 4) -> Scene:
    """Config 4: planar scene plus four concentric Fibonacci shells (radii 10/20/40/80), one view from the centre."""
    rng = np.random.default_rng(seed)
    xyz, radius = planar_scene_points(n_scene, rng)
    parts_x, parts_r = [xyz], [radius]
    for r in (10.0, 20.0, 40.0, 80.0):
        sx, sr = fibonacci_shell_points(n_shell, r, rng)
        parts_x.append(sx)
        parts_r.append(sr)
    xyz, radius = np.concatenate(parts_x), np.concatenate(parts_r)
    target = rng.normal(size=3)
    poses = look_at_pose(np.zeros(3), target / np.linalg.norm(target))[None]
    intr = pinhole_intrinsics(f, f, w / 2, h / 2)[None]
    return _assemble(xyz, radius, rng, channels, "uniform", poses, intr, [View(w, h)])


def tiny_scene(n: int = 2000, w: int = 64, h: int = 48, n_views: int = 2, seed: int = 7, channels: int = 4,
               crop: bool = False) -> Scene:
    """Small dense scene for exhaustive parity checks: long lists at coarse levels, ties in depth, points behind
    the camera and outside the frustum, optional crop transform and crop rotation."""
    rng = np.random.default_rng(seed)
    xyz = rng.uniform(-1.0, 1.0, size=(n, 3))
    xyz[: n // 8] = np.round(xyz[: n // 8] * 4) / 4  # lattice points: exact depth ties between points
    radius = rng.uniform(0.002, 0.2, size=n).astype(np.float32)
    poses = orbit_poses(rng, n_views, 2.5)
    f = 0.9 * w
    intr = pinhole_intrinsics(f, f * 1.03, w / 2 + 0.3, h / 2 - 0.2)[None]
    views = []
    for i in range(n_views):
        if crop:
            a = rng.uniform(-0.3, 0.3)
            views.append(View(w, h, image_index=i, crop=(1.1, 0.95, -2.0, 1.5, 0.0),
                              rot=(math.cos(a), -math.sin(a), math.sin(a), math.cos(a))))
        else:
            views.append(View(w, h, image_index=i))
    return _assemble(xyz, radius, rng, channels, "uniform", poses, intr, views, reorder=False)
