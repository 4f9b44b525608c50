"""ctypes binding of libvetr.so (include/vetr.h).  There is no fallback: a missing library is an error."""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.environ.get("VETR_LIB", os.path.join(_HERE, "libvetr.so"))  # VETR_LIB: a tuning variant of the library

MAX_LAYERS = 5
MAX_VIEWS = 8
MODE_FUZZY_DT = 0
MODE_FULL_BLEND = 1
MODE_FUZZY_BLEND = 2
MODE_BILINEAR_BLEND = 3

OK, E_INVALID_ARG, E_CUDA, E_UNSUPPORTED, E_LIST_OVERFLOW, E_TOO_LARGE = 0, -1, -2, -3, -4, -5


class Params(C.Structure):
    _fields_ = [
        ("render_mode", C.c_int32), ("num_layers", C.c_int32), ("num_channels", C.c_int32),
        ("drop_out_points_by_radius", C.c_int32), ("drop_out_radius_threshold", C.c_float),
        ("dist_cutoff", C.c_float), ("use_environment_map", C.c_int32), ("viewer_only", C.c_int32),
        ("stability_cutoff_value", C.c_float), ("debug_max_list_length", C.c_int32),
        ("need_point_gradient", C.c_int32), ("K_gradient_factor", C.c_float),
        ("distortion_gradient_factor", C.c_float), ("output_background_mask_value", C.c_float),
        ("background_alpha_to_point0", C.c_int32), ("keep_sorted_lists", C.c_int32),
        ("depth_accept_blend", C.c_float), ("depth_accept", C.c_float), ("ghost_gradients", C.c_int32),
    ]


class View(C.Structure):
    _fields_ = [("w", C.c_int32), ("h", C.c_int32), ("image_index", C.c_int32), ("camera_index", C.c_int32),
                ("camera_model", C.c_int32), ("crop", C.c_float * 5), ("rot", C.c_float * 4)]


class Cloud(C.Structure):
    _fields_ = [("position", C.c_void_p), ("index", C.c_void_p), ("n", C.c_int32)]


class Texture(C.Structure):
    _fields_ = [("texture", C.c_void_p), ("confidence", C.c_void_p), ("background", C.c_void_p), ("n_tex", C.c_int32)]


class Cameras(C.Structure):
    _fields_ = [("poses_se3", C.c_void_p), ("intrinsics", C.c_void_p), ("n_img", C.c_int32), ("n_cam", C.c_int32)]


class Lists(C.Structure):
    _fields_ = [("counts", C.c_void_p), ("ends", C.c_void_p), ("frags", C.c_void_p), ("capacity", C.c_int64),
                ("status", C.c_void_p), ("items", C.c_void_p), ("items_capacity", C.c_int64),
                ("level_mask", C.c_void_p), ("point_grad", C.c_void_p),
                ("pixel_scratch", C.c_void_p)]


MAX_RANKS = 16
PIXEL_BAND = 4  # VETR_PIXEL_BAND: rows per band of the pixel space


class PointArray(C.Structure):
    _fields_ = [("src", C.c_void_p), ("dst", C.c_void_p), ("rows", C.c_int32), ("width", C.c_int32)]


class EnvMap(C.Structure):
    _fields_ = [("density", C.c_void_p), ("color", C.c_void_p), ("radii", C.c_float * 8), ("n_spheres", C.c_int32),
                ("resolution", C.c_int32), ("channels", C.c_int32), ("up_axis", C.c_int32), ("non_subzero_texture", C.c_int32)]


class Exchange(C.Structure):
    _fields_ = [("rank", C.c_int32), ("world", C.c_int32), ("raw", C.c_void_p * MAX_RANKS), ("out", C.c_void_p * MAX_RANKS),
                ("raw_multicast", C.c_void_p), ("out_multicast", C.c_void_p)]


EXPORTS = [
    "vetr_create", "vetr_destroy", "vetr_set_stream", "vetr_strerror", "vetr_last_cuda_error", "vetr_pyramid_pixels",
    "vetr_item_table_entries", "vetr_max_fragments", "vetr_list_capacity", "vetr_forward", "vetr_backward", "vetr_finalize_gradients",
    "vetr_apply_tangent", "vetr_read_status", "vetr_get_lists", "vetr_set_timing", "vetr_get_timings",
    "vetr_launch_count", "vetr_scan_counts_static", "vetr_exchange_raw_floats", "vetr_exchange_out_floats",
    "vetr_exchange_finalize", "vetr_grid_loss", "vetr_l1_loss_grad", "vetr_backward_phase", "vetr_exchange_finalize_part",
    "vetr_envmap_forward", "vetr_envmap_backward", "vetr_knn_radius", "vetr_remove_points_plan", "vetr_gather_points",
]
ENV_ADD, ENV_NOT_AT_POINTS, ENV_DEPTH_TEST_WEIGHT, ENV_NO_DISTORTION_CHECK = 1, 2, 4, 8
BACKWARD_FRAGMENTS, BACKWARD_POINTS = 1, 2
SEG_DESC, SEG_POINTS, SEG_CONF = 1, 2, 4
TIMING_NAMES = ["count", "scan", "collect", "sort_blend", "backward", "finalize", "point_backward", "exchange", "envmap", "knn"]

_lib = None


class VetrError(RuntimeError):
    def __init__(self, status: int, where: str, cuda: int = 0):
        self.status = status
        msg = lib().vetr_strerror(status).decode()
        super().__init__(f"{where}: {msg} (status {status}" + (f", cudaError {cuda})" if cuda else ")"))


def lib():
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(f"{LIB_PATH} is missing: build it with `python -m vet_b200.build` "
                               "(nvcc, sm_100a). There is no CPU or PyTorch fallback.")
        L = C.CDLL(LIB_PATH)
        L.vetr_create.argtypes = [C.POINTER(C.c_void_p), C.c_int, C.c_void_p]
        L.vetr_destroy.argtypes = [C.c_void_p]
        L.vetr_destroy.restype = None
        L.vetr_set_stream.argtypes = [C.c_void_p, C.c_void_p]
        L.vetr_strerror.argtypes = [C.c_int]
        L.vetr_strerror.restype = C.c_char_p
        L.vetr_last_cuda_error.argtypes = [C.c_void_p]
        L.vetr_pyramid_pixels.argtypes = [C.c_int, C.c_int, C.c_int]
        L.vetr_pyramid_pixels.restype = C.c_int64
        L.vetr_item_table_entries.argtypes = [C.c_int64, C.c_int64]
        L.vetr_item_table_entries.restype = C.c_int64
        L.vetr_max_fragments.argtypes = [C.c_int, C.c_int, C.POINTER(Params)]
        L.vetr_max_fragments.restype = C.c_int64
        L.vetr_list_capacity.argtypes = [C.c_int, C.c_int, C.c_int, C.c_int, C.POINTER(Params)]
        L.vetr_list_capacity.restype = C.c_int64
        vp = C.c_void_p
        L.vetr_forward.argtypes = [vp, C.POINTER(Params), C.POINTER(Cloud), C.POINTER(Texture), C.POINTER(Cameras),
                                   C.POINTER(View), C.c_int, vp, C.POINTER(Lists), vp, vp, vp, vp]
        L.vetr_backward.argtypes = [vp, C.POINTER(Params), C.POINTER(Cloud), C.POINTER(Texture), C.POINTER(Cameras),
                                    C.POINTER(View), C.c_int, vp, C.POINTER(Lists), vp, vp, vp, vp, vp, vp, vp, vp, vp, vp]
        L.vetr_backward_phase.argtypes = L.vetr_backward.argtypes + [C.c_int]
        L.vetr_finalize_gradients.argtypes = [vp, C.c_int, C.c_int, vp, vp, C.c_int, vp, vp, C.c_int, vp, vp, C.c_int,
                                              vp, vp]
        L.vetr_apply_tangent.argtypes = [vp, vp, vp, C.c_int]
        L.vetr_read_status.argtypes = [vp, C.POINTER(Lists), C.POINTER(C.c_int64), C.POINTER(C.c_int32)]
        L.vetr_get_lists.argtypes = [vp, C.POINTER(Lists), C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int, vp, vp,
                                     C.POINTER(C.c_int64)]
        L.vetr_set_timing.argtypes = [vp, C.c_int]
        L.vetr_get_timings.argtypes = [vp, C.POINTER(C.c_float)]
        L.vetr_launch_count.argtypes = [vp]
        L.vetr_launch_count.restype = C.c_int64
        L.vetr_scan_counts_static.argtypes = [C.c_int, vp, vp, C.c_int64, C.c_int64, vp, vp, vp, C.c_int64]
        L.vetr_exchange_raw_floats.argtypes = [C.c_int, C.c_int]
        L.vetr_exchange_raw_floats.restype = C.c_int64
        L.vetr_exchange_out_floats.argtypes = [C.c_int, C.c_int, C.c_int]
        L.vetr_exchange_out_floats.restype = C.c_int64
        L.vetr_exchange_finalize.argtypes = [vp, C.POINTER(Exchange), C.c_int, C.c_int, C.c_int]
        L.vetr_exchange_finalize_part.argtypes = [vp, C.POINTER(Exchange), C.c_int, C.c_int, C.c_int, C.c_int, C.c_int]
        L.vetr_l1_loss_grad.argtypes = [vp, C.c_int, vp, vp, vp, C.POINTER(C.c_int64), vp]
        L.vetr_grid_loss.argtypes = [vp, C.POINTER(Cameras), C.POINTER(View), C.c_float, C.c_int, vp, vp, vp, C.c_int, vp, vp]
        L.vetr_envmap_forward.argtypes = [vp, C.POINTER(Cameras), C.POINTER(View), C.c_int, C.c_int, C.POINTER(EnvMap), vp, vp, C.c_int]
        L.vetr_envmap_backward.argtypes = [vp, C.POINTER(Cameras), C.POINTER(View), C.c_int, C.c_int, C.POINTER(EnvMap), vp, vp,
                                           C.c_int, vp, vp]
        L.vetr_knn_radius.argtypes = [vp, vp, C.c_int, C.c_int, C.c_int, vp, C.c_int]
        L.vetr_remove_points_plan.argtypes = [vp, C.c_int, vp, C.c_int, vp, C.POINTER(C.c_int)]
        L.vetr_gather_points.argtypes = [vp, C.c_int, C.c_int, vp, C.POINTER(PointArray), C.c_int]
        _lib = L
    return _lib
