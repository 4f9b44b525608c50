// C exports around the REFERENCE's own blend algebra: this file includes rendering/PointBlending.h from the reference
// tree where it lies (see oracle/Makefile, target _ref) and forwards to it unchanged.  The result,
// oracle/_ref/libref_blend.so, pins the oracle's restatement of the same functions (tests/test_oracle_ref_blend.py).
// TEST INFRASTRUCTURE ONLY.
#include "PointBlending.h"

extern "C"
{
// compute_blend with all four Jacobians (PointBlending.h:90-114)
float ref_compute_blend(float alpha_dest, float alpha_s, float color, float color_dest, float* J4)
{
    return compute_blend(alpha_dest, alpha_s, color, color_dest, J4 ? &J4[0] : nullptr, J4 ? &J4[1] : nullptr,
                         J4 ? &J4[2] : nullptr, J4 ? &J4[3] : nullptr);
}
// compute_new_alphadest (PointBlending.h:116-129)
float ref_compute_new_alphadest(float alphadest_old, float alpha_s, float* J2)
{
    return compute_new_alphadest(alphadest_old, alpha_s, J2 ? &J2[0] : nullptr, J2 ? &J2[1] : nullptr);
}
// compute_blending_fac (PointBlending.h:12-44): weights[4], J[4][2]
void ref_compute_blending_fac(float u, float v, float* weights, float* J)
{
    vec2 uv;
    uv(0) = u;
    uv(1) = v;
    Matrix<float, 4, 2> Juv;
    vec4 w = compute_blending_fac(uv, J ? &Juv : nullptr);
    for (int i = 0; i < 4; ++i) weights[i] = w(i);
    if (J)
        for (int i = 0; i < 4; ++i)
            for (int k = 0; k < 2; ++k) J[2 * i + k] = Juv(i, k);
}
}
