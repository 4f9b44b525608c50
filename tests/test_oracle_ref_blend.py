"""Pins the oracle's blend algebra to the REFERENCE's own code.

oracle/_ref/libref_blend.so is rendering/PointBlending.h of the reference, compiled unmodified from the reference
tree (oracle/Makefile target `_ref`) against a stand-in for the one saiga header it includes.  It is the only piece
of the rasterizer path the reference can be made to execute here; its CUDA sources need the whole saiga library.
Compared: compute_blend (+ its four Jacobians), compute_new_alphadest (+ two), compute_blending_fac (+ J_uv).
"""
import ctypes as C
import os

import numpy as np
import pytest

from oracle import oracle as O

REF = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref", "libref_blend.so")
pytestmark = pytest.mark.skipif(not os.path.exists(REF), reason="oracle/_ref/libref_blend.so not built (needs the reference tree)")


@pytest.fixture(scope="module")
def ref():
    lib = C.CDLL(REF)
    lib.ref_compute_blend.restype = C.c_float
    lib.ref_compute_blend.argtypes = [C.c_float] * 4 + [C.c_void_p]
    lib.ref_compute_new_alphadest.restype = C.c_float
    lib.ref_compute_new_alphadest.argtypes = [C.c_float] * 2 + [C.c_void_p]
    lib.ref_compute_blending_fac.argtypes = [C.c_float, C.c_float, C.c_void_p, C.c_void_p]
    return lib


def test_compute_blend_and_alphadest(ref):
    rng = np.random.default_rng(0)
    vo = O.lib()
    J4 = (C.c_float * 4)()
    J2 = (C.c_float * 2)()
    for _ in range(2000):
        T, a = np.float32(rng.uniform()), np.float32(rng.uniform())
        c, dst = np.float32(rng.normal()), np.float32(rng.normal())
        r = ref.ref_compute_blend(T, a, c, dst, J4)
        # the reference header compiled for the CPU evaluates T*a*c + dst without a fused multiply-add
        assert r == vo.vo_blend(T, a, c, dst, 0)
        # the fused form (what nvcc makes of the same expression, and what the oracle and the kernels use) differs by
        # at most one rounding of the product
        fused = vo.vo_blend(T, a, c, dst, 1)
        assert abs(fused - r) <= 1.2e-7 * max(abs(np.float32(T * a * c)), abs(r), 1e-30)
        # Jacobians: d/d alpha_s, d/d color, d/d alpha_dest, d/d color_dest  (PointBlending.h:95-111)
        np.testing.assert_array_equal(np.array(J4[:], np.float32), np.array([T * c, T * a, a * c, 1], np.float32))
        t2 = ref.ref_compute_new_alphadest(T, a, J2)
        assert t2 == vo.vo_new_T(T, a)
        np.testing.assert_array_equal(np.array(J2[:], np.float32), np.array([-T, np.float32(1) - a], np.float32))


def test_compute_blending_fac(ref):
    rng = np.random.default_rng(1)
    vo = O.lib()
    w_ref, J_ref = np.zeros(4, np.float32), np.zeros(8, np.float32)
    w_o, J_o = np.zeros(4, np.float32), np.zeros(8, np.float32)
    pts = np.concatenate([rng.uniform(-50, 2000, size=(2000, 2)), [[3.0, 7.0], [0.5, 0.5], [-0.25, 1e-3], [1919.999, 0.0]]])
    for u, v in pts.astype(np.float32):
        ref.ref_compute_blending_fac(u, v, w_ref.ctypes.data, J_ref.ctypes.data)
        vo.vo_blending_fac(u, v, w_o.ctypes.data, J_o.ctypes.data)
        np.testing.assert_array_equal(w_ref, w_o)
        np.testing.assert_array_equal(J_ref, J_o)
        assert abs(float(w_ref.sum()) - 1.0) < 1e-6
