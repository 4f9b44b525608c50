// Camera arithmetic and blend algebra of the rasterizer kernels (device side).
//
// Everything that decides a fragment's pixel, depth bits or forward alpha (the functions marked STRICT) is written
// with the __f*_rn intrinsics, which the compiler never fuses into multiply-adds: every product and sum is rounded
// separately, in the order written, so that those values are a pure function of the inputs and are reproduced bit
// for bit by a CPU build made without floating-point contraction.  The one deliberate fused multiply-add of the
// forward pass is the blend step (vetr_blend), where the reference's expression
// `alpha_dest * alpha_s * color + color_dest` (PointBlending.h:90-114) is contracted by its own compiler.
// The gradient arithmetic (Jacobians, sweeps) is ordinary fp32 and may be contracted.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace vetr
{
struct Pose  // world -> camera; Sophus::SE3d memory (quaternion xyzw, translation) cast to float per use (RenderConstants.h:78)
{
    float qx, qy, qz, qw, tx, ty, tz;
};

struct Camera  // everything a kernel needs to project into one view
{
    Pose V;
    float K[5];     // fx fy cx cy s
    float dist[8];  // k1 k2 k3 k4 k5 k6 p1 p2
    float crop[5];  // crop_transform fx fy cx cy s
    float rot[4];   // crop_rotation row-major
    float cx, cy;   // rotation centre (w/2, h/2) with integer division (RenderForward.cu:156)
    float R[9];     // rotation matrix of V (backward only)
    bool has_dist;
};

#define VM(a, b) __fmul_rn((a), (b))
#define VA(a, b) __fadd_rn((a), (b))
#define VS(a, b) __fsub_rn((a), (b))

__device__ __forceinline__ float3 cross3(float3 a, float3 b)  // STRICT
{
    return make_float3(VS(VM(a.y, b.z), VM(a.z, b.y)), VS(VM(a.z, b.x), VM(a.x, b.z)), VS(VM(a.x, b.y), VM(a.y, b.x)));
}

// STRICT.  Eigen quaternion transform: v + w * uv + qv x uv with uv = 2 (qv x v); then the translation.
__device__ __forceinline__ float3 transform_point(const Pose& P, float3 v)
{
    float3 qv = make_float3(P.qx, P.qy, P.qz);
    float3 uv = cross3(qv, v);
    uv        = make_float3(VA(uv.x, uv.x), VA(uv.y, uv.y), VA(uv.z, uv.z));
    float3 c  = cross3(qv, uv);
    float3 r  = make_float3(VA(VA(v.x, VM(P.qw, uv.x)), c.x), VA(VA(v.y, VM(P.qw, uv.y)), c.y),
                            VA(VA(v.z, VM(P.qw, uv.z)), c.z));
    return make_float3(VA(r.x, P.tx), VA(r.y, P.ty), VA(r.z, P.tz));
}

__device__ __forceinline__ void rotation_matrix(const Pose& P, float R[9])
{
    float x = P.qx, y = P.qy, z = P.qz, w = P.qw;
    float tx = 2 * x, ty = 2 * y, tz = 2 * z;
    float twx = tx * w, twy = ty * w, twz = tz * w;
    float txx = tx * x, txy = ty * x, txz = tz * x;
    float tyy = ty * y, tyz = tz * y, tzz = tz * z;
    R[0] = 1 - (tyy + tzz);
    R[1] = txy - twz;
    R[2] = txz + twy;
    R[3] = txy + twz;
    R[4] = 1 - (txx + tzz);
    R[5] = tyz - twx;
    R[6] = txz - twy;
    R[7] = tyz + twx;
    R[8] = 1 - (txx + tyy);
}

// OpenCV rational distortion; returns the sentinel (100000, 100000) beyond the cutoff radius, which the caller
// turns into z = 0 (PointRendererHelper.h:207-212).
template <bool kJacobians>
__device__ __forceinline__ float2 distort(float2 p, const float* d, float cutoff, float* J_p, float* J_d)
{
    // the value path is STRICT (it decides pixels); the Jacobians are not
    float x = p.x, y = p.y;
    float x2 = VM(x, x), y2 = VM(y, y), xy = VM(x, y);
    float r2 = VA(x2, y2);
    if (r2 > VM(cutoff, cutoff))
    {
        if (kJacobians)
        {
            for (int i = 0; i < 4; ++i) J_p[i] = 0.f;
            for (int i = 0; i < 16; ++i) J_d[i] = 0.f;
        }
        return make_float2(100000.f, 100000.f);
    }
    float r4 = VM(r2, r2), r6 = VM(r4, r2);
    float k1 = d[0], k2 = d[1], k3 = d[2], k4 = d[3], k5 = d[4], k6 = d[5], p1 = d[6], p2 = d[7];
    float num    = VA(VA(VA(1.f, VM(k1, r2)), VM(k2, r4)), VM(k3, r6));
    float den    = VA(VA(VA(1.f, VM(k4, r2)), VM(k5, r4)), VM(k6, r6));
    float radial = num / den;
    float tx     = VA(VM(VM(2.f, p1), xy), VM(p2, VA(r2, VM(2.f, x2))));
    float ty     = VA(VM(VM(2.f, p2), xy), VM(p1, VA(r2, VM(2.f, y2))));
    float2 out   = make_float2(VA(VM(x, radial), tx), VA(VM(y, radial), ty));
    if (kJacobians)
    {
        float dnum_dr2 = k1 + 2.f * k2 * r2 + 3.f * k3 * r4;
        float dden_dr2 = k4 + 2.f * k5 * r2 + 3.f * k6 * r4;
        float drad_dr2 = (dnum_dr2 * den - num * dden_dr2) / (den * den);
        float drad_dx = drad_dr2 * 2.f * x, drad_dy = drad_dr2 * 2.f * y;
        J_p[0] = radial + x * drad_dx + 2.f * p1 * y + p2 * (2.f * x + 4.f * x);
        J_p[1] = x * drad_dy + 2.f * p1 * x + p2 * (2.f * y);
        J_p[2] = y * drad_dx + 2.f * p2 * y + p1 * (2.f * x);
        J_p[3] = radial + y * drad_dy + 2.f * p2 * x + p1 * (2.f * y + 4.f * y);
        float inv_den = 1.f / den;
        float a       = -num / (den * den);
        J_d[0] = x * r2 * inv_den, J_d[1] = x * r4 * inv_den, J_d[2] = x * r6 * inv_den;
        J_d[3] = x * a * r2, J_d[4] = x * a * r4, J_d[5] = x * a * r6;
        J_d[6] = 2.f * xy, J_d[7] = r2 + 2.f * x2;
        J_d[8] = y * r2 * inv_den, J_d[9] = y * r4 * inv_den, J_d[10] = y * r6 * inv_den;
        J_d[11] = y * a * r2, J_d[12] = y * a * r4, J_d[13] = y * a * r6;
        J_d[14] = r2 + 2.f * y2, J_d[15] = 2.f * xy;
    }
    return out;
}

// STRICT.  IntrinsicsPinhole::normalizedToImage, coefficient order fx fy cx cy s.
__device__ __forceinline__ float2 k_apply(const float* K, float2 p)
{
    return make_float2(VA(VA(VM(K[0], p.x), VM(K[4], p.y)), K[2]), VA(VM(K[1], p.y), K[3]));
}

struct Projected
{
    float2 ip;        // level-0 image position after crop transform and crop rotation
    float z;          // max(view z, 0); 0 = not rendered
    float radius_px;  // drop-out radius in level-0 pixels
};

// STRICT.  ProjPoint (RenderForward.cu:117-158, pinhole branch) over ProjectPointPinhole (PointRendererHelper.h:184-218).
__device__ __forceinline__ Projected project_point(const float4 pos, const Camera& cam, float dist_cutoff,
                                                   bool apply_crop_rotation = true)
{
    float3 vp = transform_point(cam.V, make_float3(pos.x, pos.y, pos.z));
    float z   = fmaxf(vp.z, 0.f);
    float2 np = make_float2(vp.x / vp.z, vp.y / vp.z);
    float2 dp = np;
    if (cam.has_dist)
    {
        dp = distort<false>(np, cam.dist, dist_cutoff, nullptr, nullptr);
        if (dp.x == 100000.f) z = 0.f;
    }
    else
    {
        // all coefficients zero: the model returns its input bit for bit (radial = 1, tangential = 0); only the
        // cutoff test remains
        if (VA(VM(np.x, np.x), VM(np.y, np.y)) > VM(dist_cutoff, dist_cutoff)) z = 0.f;
    }
    float2 ip       = k_apply(cam.K, dp);
    float radius_px = VM(VM(cam.K[0], cam.crop[0]), pos.w) / z;
    ip              = k_apply(cam.crop, ip);
    if (apply_crop_rotation)  // mode 0's backward pass projects without it (RenderBackward.cu:78-116)
    {
        float dx = VS(ip.x, cam.cx), dy = VS(ip.y, cam.cy);
        ip = make_float2(VA(VM(cam.rot[0], dx), VM(cam.rot[1], dy)), VA(VM(cam.rot[2], dx), VM(cam.rot[3], dy)));
        ip = make_float2(VA(ip.x, cam.cx), VA(ip.y, cam.cy));
    }
    Projected r;
    r.ip        = ip;
    r.z         = z;
    r.radius_px = radius_px;
    return r;
}

__device__ __forceinline__ int round_half_even(float v)  // __float2int_rn with everything unrepresentable sent outside
{
    if (!(v > -1.0e9f && v < 1.0e9f)) return INT32_MIN;
    return __float2int_rn(v);
}
__device__ __forceinline__ int round_down(float v)  // __float2int_rd
{
    if (!(v > -1.0e9f && v < 1.0e9f)) return INT32_MIN;
    return __float2int_rd(v);
}

// STRICT.  compute_blending_fac, PointBlending.h:12-44: weight of corner `bi` (= 2*y_j + x_i) and its row of J_uv.
__device__ __forceinline__ float blending_fac(float2 uv, int bi, float* Jx, float* Jy)
{
    float sx = VS(uv.x, floorf(uv.x)), sy = VS(uv.y, floorf(uv.y));
    float w, jx, jy;
    if (bi == 0)
        w = VM(VS(1.f, sx), VS(1.f, sy)), jx = sy - 1, jy = sx - 1;
    else if (bi == 1)
        w = VM(sx, VS(1.f, sy)), jx = 1 - sy, jy = -sx;
    else if (bi == 2)
        w = VM(VS(1.f, sx), sy), jx = -sy, jy = 1 - sx;
    else
        w = VM(sx, sy), jx = sy, jy = sx;
    if (Jx) *Jx = jx;
    if (Jy) *Jy = jy;
    return w;
}

// compute_blend / compute_new_alphadest, PointBlending.h:90-129.
__device__ __forceinline__ float vetr_blend(float T, float a, float c, float dst) { return __fmaf_rn(VM(T, a), c, dst); }
__device__ __forceinline__ float vetr_new_T(float T, float a) { return VM(VS(1.f, a), T); }

struct BackOut
{
    float g_point[3], g_pose[6], g_k[5], g_dis[8];
};

// ProjectPointPinholeBackward, PointRendererHelper.h:317-372, in two steps: what depends on the point and the camera
// only (computed once per point and view), and the chain of transposed Jacobians applied to one image-space gradient.
// `cropK` is crop_transform.scale(0.5^level).
struct PointJac
{
    float3 vp;
    float iz, gzx, gzy;  // 1/z and the z column of the division's Jacobian
    float2 dp;
    float Jpd[4], Jdd[16];
};

__device__ __forceinline__ bool project_backward_prepare(const float4 pos, const Camera& cam, float dist_cutoff,
                                                         bool want_intrinsics, PointJac& j)
{
    j.vp = transform_point(cam.V, make_float3(pos.x, pos.y, pos.z));
    if (!(j.vp.z > 0)) return false;
    j.iz = 1.f / j.vp.z;
    float2 np = make_float2(j.vp.x / j.vp.z, j.vp.y / j.vp.z);
    j.Jpd[0] = 1.f, j.Jpd[1] = 0.f, j.Jpd[2] = 0.f, j.Jpd[3] = 1.f;
    j.dp = np;
    if (cam.has_dist || want_intrinsics) j.dp = distort<true>(np, cam.dist, dist_cutoff, j.Jpd, j.Jdd);
    j.gzx = -j.vp.x * j.iz * j.iz;
    j.gzy = -j.vp.y * j.iz * j.iz;
    return true;
}

__device__ __forceinline__ void project_backward_apply(const PointJac& j, float2 grad, const Camera& cam, const float cropK[5],
                                                       bool want_intrinsics, BackOut& o)
{
    const float* R = cam.R;
    const float3 vp = j.vp;
    // grad_p_rot = rot^T grad ; grad_p_k2 = J_p_K2^T grad_p_rot ; then J_p_K1^T, J_p_dis^T, J_div^T
    float2 g_rot = make_float2(cam.rot[0] * grad.x + cam.rot[2] * grad.y, cam.rot[1] * grad.x + cam.rot[3] * grad.y);
    float2 g_k2  = make_float2(cropK[0] * g_rot.x + 0.f * g_rot.y, cropK[4] * g_rot.x + cropK[1] * g_rot.y);
    float2 g_k1  = make_float2(cam.K[0] * g_k2.x + 0.f * g_k2.y, cam.K[4] * g_k2.x + cam.K[1] * g_k2.y);
    float2 g_dis = make_float2(j.Jpd[0] * g_k1.x + j.Jpd[2] * g_k1.y, j.Jpd[1] * g_k1.x + j.Jpd[3] * g_k1.y);
    float gv0 = j.iz * g_dis.x + 0.f * g_dis.y;
    float gv1 = 0.f * g_dis.x + j.iz * g_dis.y;
    float gv2 = j.gzx * g_dis.x + j.gzy * g_dis.y;
    for (int k = 0; k < 3; ++k) o.g_point[k] = R[0 + k] * gv0 + R[3 + k] * gv1 + R[6 + k] * gv2;
    // J_pose = [ I | -skew(vp) ]
    o.g_pose[0] = gv0;
    o.g_pose[1] = gv1;
    o.g_pose[2] = gv2;
    o.g_pose[3] = 0.f * gv0 + (-vp.z) * gv1 + vp.y * gv2;
    o.g_pose[4] = vp.z * gv0 + 0.f * gv1 + (-vp.x) * gv2;
    o.g_pose[5] = (-vp.y) * gv0 + vp.x * gv1 + 0.f * gv2;
    if (want_intrinsics)
    {
        o.g_k[0] = j.dp.x * g_k2.x;
        o.g_k[1] = j.dp.y * g_k2.y;
        o.g_k[2] = g_k2.x;
        o.g_k[3] = g_k2.y;
        o.g_k[4] = j.dp.y * g_k2.x;
        for (int k = 0; k < 8; ++k) o.g_dis[k] = j.Jdd[k] * g_k1.x + j.Jdd[8 + k] * g_k1.y;
    }
}

__device__ __forceinline__ bool project_backward(const float4 pos, float2 grad, const Camera& cam, const float cropK[5],
                                                 float dist_cutoff, bool want_intrinsics, BackOut& o)
{
    PointJac j;
    if (!project_backward_prepare(pos, cam, dist_cutoff, want_intrinsics, j)) return false;
    project_backward_apply(j, grad, cam, cropK, want_intrinsics, o);
    return true;
}

}  // namespace vetr
