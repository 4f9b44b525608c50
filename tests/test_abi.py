"""The C ABI without a GPU: the library loads, exports every function include/vetr.h declares, and its host-only entry
points behave.  No kernel is launched here."""
import ctypes as C
import os
import re

import pytest

from vet_b200 import _lib as L

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_functions():
    text = open(os.path.join(ROOT, "include", "vetr.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(vetr_[a-z_0-9]+)\s*\(", text)))


def test_every_declared_symbol_is_exported():
    names = declared_functions()
    assert len(names) >= 15
    lib = L.lib()
    missing = [n for n in names if not hasattr(lib, n)]
    assert not missing, missing
    assert sorted(L.EXPORTS) == [n for n in names], "vet_b200._lib.EXPORTS is out of step with include/vetr.h"


def test_host_only_entry_points():
    lib = L.lib()
    # every level's height is padded to a multiple of VETR_PIXEL_BAND (4) rows in the pixel space
    assert L.PIXEL_BAND == 4
    assert lib.vetr_pyramid_pixels(1920, 1080, 4) == 1920 * 1080 + 960 * 540 + 480 * 272 + 240 * 136
    assert lib.vetr_pyramid_pixels(5, 3, 2) == 5 * 4 + 2 * 4
    assert lib.vetr_pyramid_pixels(0, 3, 2) == -1 and lib.vetr_pyramid_pixels(4, 4, 6) == -1
    p = L.Params(render_mode=1, num_layers=4)
    assert lib.vetr_max_fragments(1000, 3, C.byref(p)) == 12000
    p.render_mode = 3
    assert lib.vetr_max_fragments(1000, 3, C.byref(p)) == 48000
    # the buffer bound: fragments in modes 1-3, one accumulator record per pixel of the pixel space in mode 0
    assert lib.vetr_list_capacity(1000, 3, 64, 48, C.byref(p)) == 48000
    p.render_mode = 0
    assert lib.vetr_list_capacity(500, 2, 256, 256, C.byref(p)) == 2 * lib.vetr_pyramid_pixels(256, 256, 4)
    assert lib.vetr_item_table_entries(0, 0) >= 2
    assert lib.vetr_item_table_entries(10**6, 10**6) > (10**6 + 4 * 10**6) // 1024
    assert lib.vetr_strerror(0) == b"ok"
    assert b"buffer" in lib.vetr_strerror(L.E_LIST_OVERFLOW)
    assert lib.vetr_launch_count(None) == 0


def test_struct_sizes_match_the_header():
    # include/vetr.h: 19 four-byte fields; 5 ints + 9 floats; pointers + ints
    assert C.sizeof(L.Params) == 76
    assert C.sizeof(L.View) == 56
    assert C.sizeof(L.Cloud) == 24 and C.sizeof(L.Texture) == 32 and C.sizeof(L.Cameras) == 24
    assert C.sizeof(L.Lists) == 80
    assert C.sizeof(L.EnvMap) == 72  # two pointers, eight radii, five ints, padded to the pointer size
    assert C.sizeof(L.Exchange) == 8 + 2 * 8 * L.MAX_RANKS + 16


def test_create_without_gpu_reports_cuda_error():
    import torch

    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    ctx = C.c_void_p()
    assert L.lib().vetr_create(C.byref(ctx), 0, None) == L.E_CUDA
    assert not ctx.value


def test_host_mirror_refuses_to_run_without_cuda():
    import torch
    from vet_b200.render import Rasterizer

    if torch.cuda.is_available():
        pytest.skip("a GPU is present")
    with pytest.raises(RuntimeError, match="no CPU path"):
        Rasterizer(0)
