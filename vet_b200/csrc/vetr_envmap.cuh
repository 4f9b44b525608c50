// Texture environment map kernels: EnvironmentMapImpl::Sample2 / forward_mps5 (rendering/EnvironmentMap.cu:378-485,
// 692-758) as one forward and one backward kernel over all views, levels and pixels.
//
// The reference builds a ray list (BuildSphericalRayList, :201-287), writes sample coordinates for every sphere
// (CreateSampleUVMapAllSpheres, :587-684), calls grid_sample twice on [S * rays] coordinates, and then runs about ten
// element-wise libtorch operators per sphere; autograd replays all of it backwards.  Here a thread owns a pixel: ray,
// sphere hits, the trilinear fetches of grid_sample (bilinear, zero padding, align_corners) and the front-to-back
// chain stay in registers; per pixel the forward kernel reads 4 bytes (the transmittance) and writes 4 C bytes, and the
// textures (S R^2 (C + 1) floats) are shared by all pixels through L2.
//
// The arithmetic is written operation for operation like the CPU restatement the tests compare with (the build uses
// -fmad=false, so nothing is contracted); asinf, atan2f and expf are the device's own.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

#include "vetr_math.cuh"

namespace vetr
{
constexpr int kEnvMaxSpheres = 8;  // MAX_NUM_SPHERES, EnvironmentMap.cu:91
constexpr int kEnvThreads    = 256;

struct EnvView
{
    int image_index, camera_index;
    float crop[5];
    float rot[4];
};

struct EnvArgs  // kernel parameter block
{
    int n_views, L, S, R, C, up_axis, non_subzero, flags;
    int lw[VETR_MAX_LAYERS], lh[VETR_MAX_LAYERS];
    long long lend[VETR_MAX_LAYERS];  // pixels of levels 0..l over all views (running total)
    float scale[VETR_MAX_LAYERS];     // 0.5^l
    float radii[kEnvMaxSpheres];
    EnvView views[VETR_MAX_VIEWS];
    const double* poses;
    const float* intr;
    const float* density;  // [S,R,R]
    const float* color;    // [C,S,R,R]
    const float* weight[VETR_MAX_LAYERS];  // [n_views,1,h_l,w_l]
    float* out[VETR_MAX_LAYERS];           // [n_views,C,h_l,w_l]
    const float* grad[VETR_MAX_LAYERS];    // incoming gradient of out (backward)
    float* g_density;
    float* g_color;
};

struct EnvCam  // what a pixel needs of its view: camera -> world, intrinsics, inverse crop rotation
{
    Pose Vi;  // Sophus SE3::inverse: (q^-1, q^-1 * (-t))
    float K[5], crop[5], rinv[4];
};

__device__ __forceinline__ float3 rotate_vector(const Pose& P, float3 v)  // Eigen quaternion * vector
{
    float3 qv = make_float3(P.qx, P.qy, P.qz);
    float3 uv = cross3(qv, v);
    uv        = make_float3(uv.x + uv.x, uv.y + uv.y, uv.z + uv.z);
    float3 c  = cross3(qv, uv);
    return make_float3(v.x + P.qw * uv.x + c.x, v.y + P.qw * uv.y + c.y, v.z + P.qw * uv.z + c.z);
}

__device__ __forceinline__ EnvCam load_env_cam(const EnvArgs& a, int b)
{
    EnvCam c;
    const EnvView& v = a.views[b];
    const double* p  = a.poses + 8 * (long long)v.image_index;
    Pose V;
    V.qx = (float)p[0], V.qy = (float)p[1], V.qz = (float)p[2], V.qw = (float)p[3];
    V.tx = (float)p[4], V.ty = (float)p[5], V.tz = (float)p[6];
    c.Vi.qx = -V.qx, c.Vi.qy = -V.qy, c.Vi.qz = -V.qz, c.Vi.qw = V.qw;
    c.Vi.tx = c.Vi.ty = c.Vi.tz = 0.f;
    float3 ti = rotate_vector(c.Vi, make_float3(-V.tx, -V.ty, -V.tz));
    c.Vi.tx = ti.x, c.Vi.ty = ti.y, c.Vi.tz = ti.z;
    const float* k = a.intr + 13 * (long long)v.camera_index;
    for (int i = 0; i < 5; ++i) c.K[i] = k[i], c.crop[i] = v.crop[i];
    // Eigen's 2x2 inverse of crop_rotation
    const float det = v.rot[0] * v.rot[3] - v.rot[2] * v.rot[1];
    const float inv = 1.f / det;
    c.rinv[0] = v.rot[3] * inv, c.rinv[1] = -v.rot[1] * inv, c.rinv[2] = -v.rot[2] * inv, c.rinv[3] = v.rot[0] * inv;
    return c;
}

__device__ __forceinline__ float2 env_unproject2(const float* K, float2 ip)  // IntrinsicsPinhole::unproject2
{
    float y = (ip.y - K[3]) / K[1];
    float x = (ip.x - K[2] - K[4] * y) / K[0];
    return make_float2(x, y);
}

struct EnvRay
{
    float3 o, d;
    float q2a, qb, f;  // coefficients of the sphere intersection, EnvironmentMap.cu:616-618
};

// BuildSphericalRayList, pinhole branch (EnvironmentMap.cu:201-241): the origin is the pixel's point on the camera's
// z = 1 plane in world space, the direction points away from the eye.
__device__ __forceinline__ EnvRay env_ray(const EnvCam& c, int lw, int lh, float scale, int gx, int gy)
{
    const float cx = (float)(lw / 2), cy = (float)(lh / 2);
    const float dx = (float)gx - cx, dy = (float)gy - cy;
    float2 ip = make_float2(c.rinv[0] * dx + c.rinv[1] * dy, c.rinv[2] * dx + c.rinv[3] * dy);
    ip        = make_float2(ip.x + cx, ip.y + cy);
    float crop[5];
#pragma unroll
    for (int k = 0; k < 5; ++k) crop[k] = c.crop[k] * scale;
    const float2 np = env_unproject2(c.K, env_unproject2(crop, ip));
    const float3 r  = rotate_vector(c.Vi, make_float3(np.x, np.y, 1.f));
    EnvRay ray;
    ray.o = make_float3(r.x + c.Vi.tx, r.y + c.Vi.ty, r.z + c.Vi.tz);
    float3 d = make_float3(ray.o.x - c.Vi.tx, ray.o.y - c.Vi.ty, ray.o.z - c.Vi.tz);
    const float n2 = d.x * d.x + d.y * d.y + d.z * d.z;
    if (n2 > 0.f)
    {
        const float n = sqrtf(n2);
        d = make_float3(d.x / n, d.y / n, d.z / n);
    }
    ray.d   = d;
    ray.q2a = 2.f * (d.x * d.x) + 2.f * (d.y * d.y) + 2.f * (d.z * d.z);
    ray.qb  = 2.f * (ray.o.x * d.x) + 2.f * (ray.o.y * d.y) + 2.f * (ray.o.z * d.z);
    ray.f   = ray.qb * ray.qb - 2.f * ray.q2a * (ray.o.x * ray.o.x + ray.o.y * ray.o.y + ray.o.z * ray.o.z);
    return ray;
}

struct EnvTap  // one sphere's sample: base texel and trilinear weights
{
    bool hit;
    int x0, y0, z0;
    float wx[2], wy[2], wz[2];
};

__device__ __forceinline__ float env_unnormalize(float c, int size) { return ((c + 1.f) / 2.f) * (float)(size - 1); }

// CreateSampleUVMapAllSpheres for one sphere (EnvironmentMap.cu:620-682) + grid_sample's coordinate arithmetic.
__device__ __forceinline__ EnvTap env_tap(const EnvArgs& a, const EnvRay& ray, int s)
{
    EnvTap t;
    t.hit = true;
    t.x0 = t.y0 = t.z0 = 0;
    t.wx[0] = t.wx[1] = t.wy[0] = t.wy[1] = t.wz[0] = t.wz[1] = 0.f;
    float3 sv = ray.d;
    if (s != a.S - 1)
    {
        const float r   = a.radii[s];
        const float det = ray.f + 2.f * ray.q2a * (r * r);
        t.hit           = det >= 0.f;
        if (!t.hit) return t;
        const float res = (-ray.qb + sqrtf(det)) / ray.q2a;
        const float3 p  = make_float3(ray.o.x + res * ray.d.x, ray.o.y + res * ray.d.y, ray.o.z + res * ray.d.z);
        const float len = sqrtf(p.x * p.x + p.y * p.y + p.z * p.z);
        sv = make_float3(p.x / len, p.y / len, p.z / len);
    }
    const float pi = 3.14159265358979323846f;
    float la, lb, lc;  // lat = asin(la), lon = atan2(lb, lc)
    if (a.up_axis == 0) la = sv.x, lb = sv.y, lc = sv.z;
    else if (a.up_axis == 1) la = sv.y, lb = sv.x, lc = sv.z;
    else la = sv.z, lb = sv.x, lc = sv.y;
    la = fminf(fmaxf(la, -1.f), 1.f);
    const float lat = asinf(la), lon = atan2f(lb, lc);
    const float u = 2.f * (lon / 2.f / pi);
    const float v = 2.f * (lat / pi);
    const float z = a.S == 1 ? 0.f : (float)s / (float)(a.S - 1) * 2.f - 1.f;
    const float ix = env_unnormalize(u, a.R), iy = env_unnormalize(v, a.R), iz = env_unnormalize(z, a.S);
    const float fx = floorf(ix), fy = floorf(iy), fz = floorf(iz);
    // the base texel, kept inside [-2, size] so that the int conversion and the + 1 of the far corners are defined for
    // every float (anything out there is outside the texture and reads zero either way)
    t.x0 = (int)fminf(fmaxf(fx, -2.f), (float)a.R), t.y0 = (int)fminf(fmaxf(fy, -2.f), (float)a.R);
    t.z0 = (int)fminf(fmaxf(fz, -2.f), (float)a.S);
    t.wx[1] = ix - fx, t.wx[0] = (fx + 1.f) - ix;
    t.wy[1] = iy - fy, t.wy[0] = (fy + 1.f) - iy;
    t.wz[1] = iz - fz, t.wz[0] = (fz + 1.f) - iz;
    return t;
}

// The eight corners of a tap: texel offset inside one [S,R,R] plane (-1 = outside, reads zero) and weight.
struct EnvCorners
{
    int off[8];
    float w[8];
};

__device__ __forceinline__ void env_corners(const EnvArgs& a, const EnvTap& t, EnvCorners& c)
{
#pragma unroll
    for (int k = 0; k < 2; ++k)
#pragma unroll
        for (int j = 0; j < 2; ++j)
#pragma unroll
            for (int i = 0; i < 2; ++i)
            {
                const int x = t.x0 + i, y = t.y0 + j, z = t.z0 + k;
                const bool in = x >= 0 && x < a.R && y >= 0 && y < a.R && z >= 0 && z < a.S;
                const float w = t.wx[i] * t.wy[j] * t.wz[k];
                c.off[4 * k + 2 * j + i] = in ? (z * a.R + y) * a.R + x : -1;
                c.w[4 * k + 2 * j + i]   = w;
            }
}

__device__ __forceinline__ float env_fetch(const float* plane, const EnvCorners& c)
{
    float acc = 0.f;
#pragma unroll
    for (int q = 0; q < 8; ++q)
        if (c.off[q] >= 0 && c.w[q] != 0.f) acc += __ldg(plane + c.off[q]) * c.w[q];  // weight 0 adds nothing to a finite texture
    return acc;
}

// Decodes a thread's pixel: level, view, x, y.  Pixels are numbered level by level, and inside a level view by view in
// row-major order, so that a warp covers 32 consecutive pixels of a row.
struct EnvPixelId
{
    int l, b, x, y;
    long long pix;  // index inside the level's [n_views, h, w] plane
};

__device__ __forceinline__ bool env_locate(const EnvArgs& a, long long idx, EnvPixelId& p)
{
    if (idx >= a.lend[a.L - 1]) return false;
    int l = 0;
    while (idx >= a.lend[l]) ++l;
    const long long base = l == 0 ? 0 : a.lend[l - 1];
    p.l   = l;
    p.pix = idx - base;
    const int per_view = a.lw[l] * a.lh[l];
    p.b   = (int)(p.pix / per_view);
    const int r = (int)(p.pix - (long long)p.b * per_view);
    p.y   = r / a.lw[l];
    p.x   = r - p.y * a.lw[l];
    return true;
}

__device__ __forceinline__ float env_start_T(float weight, int flags)
{
    return (flags & VETR_ENV_DEPTH_TEST_WEIGHT) ? (weight > 0.5f ? 0.f : 1.f) : weight;
}

#ifndef VETR_ENV_FWD_CTAS
#    define VETR_ENV_FWD_CTAS 0  // resident thread blocks per SM the forward kernel is compiled for (0: the compiler's choice, 64 registers)
#endif
#if VETR_ENV_FWD_CTAS > 0
__global__ void __launch_bounds__(kEnvThreads, VETR_ENV_FWD_CTAS) envmap_forward_kernel(const __grid_constant__ EnvArgs a)
#else
__global__ void __launch_bounds__(kEnvThreads) envmap_forward_kernel(const __grid_constant__ EnvArgs a)
#endif
{
    __shared__ EnvCam s_cam[VETR_MAX_VIEWS];
    if (threadIdx.x < a.n_views) s_cam[threadIdx.x] = load_env_cam(a, threadIdx.x);
    __syncthreads();
    const long long plane = (long long)a.S * a.R * a.R;
    for (long long idx = (long long)blockIdx.x * kEnvThreads + threadIdx.x; idx < a.lend[a.L - 1];
         idx += (long long)gridDim.x * kEnvThreads)
    {
        EnvPixelId p;
        env_locate(a, idx, p);
        const int lw = a.lw[p.l], lh = a.lh[p.l];
        const float wgt   = a.weight[p.l][p.pix];
        const bool masked = (a.flags & VETR_ENV_NOT_AT_POINTS) && wgt > 0.001f;
        float acc[4] = {0.f, 0.f, 0.f, 0.f};
        float T      = env_start_T(wgt, a.flags);
        if (!masked)
        {
            const EnvRay ray = env_ray(s_cam[p.b], lw, lh, a.scale[p.l], p.x, p.y);
            for (int s = 0; s < a.S; ++s)
            {
                const EnvTap t = env_tap(a, ray, s);
                if (!t.hit) continue;  // alpha = 0: nothing added, T unchanged
                EnvCorners c;
                env_corners(a, t, c);
                float alpha = 1.f;
                if (s != a.S - 1) alpha = 1.f / (1.f + expf(-env_fetch(a.density, c)));
#pragma unroll
                for (int ch = 0; ch < 4; ++ch)
                    if (ch < a.C)
                    {
                        float col = env_fetch(a.color + ch * plane, c);
                        if (a.non_subzero) col = fabsf(col);
                        acc[ch] = T * alpha * col + acc[ch];
                    }
                T = (1.f - alpha) * T;
            }
        }
        const long long per_view = (long long)lw * lh;
        float* o = a.out[p.l] + ((long long)p.b * a.C) * per_view + (p.pix - (long long)p.b * per_view);
#pragma unroll
        for (int ch = 0; ch < 4; ++ch)
            if (ch < a.C)
            {
                float v = acc[ch];
                if (a.flags & VETR_ENV_ADD)
                {
                    float base = o[ch * per_view];
                    if ((a.flags & VETR_ENV_DEPTH_TEST_WEIGHT) && !(wgt > 0.5f)) base = 0.f;
                    v = base + acc[ch];
                }
                o[ch * per_view] = v;
            }
    }
}

// Backward.  Per pixel, with D_s = colour_s . G and the transmittance T_s in front of sphere s:
//   d env / d colour_s = T_s alpha_s G,    d env / d alpha_s = T_s (D_s - rest_s),
//   rest_s = sum over the spheres behind s of their contribution per unit of transmittance behind s
//          = alpha_{s+1} D_{s+1} + (1 - alpha_{s+1}) rest_{s+1}
// (no division by 1 - alpha, which a saturated sigmoid makes zero).  First sweep, front to back: sample, keep alpha,
// sigmoid, D, T and the colours' signs.  Second sweep, back to front: the gradients of the sphere's samples, scattered
// to the eight corners of its tap.  Neighbouring pixels of a row fall into the same texel (a level-0 row of 1920 pixels
// crosses a few hundred texels), so before the atomics the lanes of a warp that share a base texel, in runs of
// consecutive lanes, are summed with a segmented shuffle reduction and the run's first lane issues one atomic per
// corner and value.
#ifndef VETR_ENV_BACK_CTAS
#    define VETR_ENV_BACK_CTAS 3  // 80 registers with a few spills: 5.3 -> 4.1 ms on the benchmark row (2: 118 registers, 4: 64 registers, 4.5 ms)
#endif
__global__ void __launch_bounds__(kEnvThreads, VETR_ENV_BACK_CTAS) envmap_backward_kernel(const __grid_constant__ EnvArgs a)
{
    __shared__ EnvCam s_cam[VETR_MAX_VIEWS];
    if (threadIdx.x < a.n_views) s_cam[threadIdx.x] = load_env_cam(a, threadIdx.x);
    __syncthreads();
    const long long plane = (long long)a.S * a.R * a.R;
    const int lane        = threadIdx.x & 31;
    const long long total = a.lend[a.L - 1];
    const long long span  = (total + 31) / 32 * 32;  // whole warps stay in the loop together
    for (long long idx = (long long)blockIdx.x * kEnvThreads + threadIdx.x; idx < span; idx += (long long)gridDim.x * kEnvThreads)
    {
        EnvPixelId p;
        bool active = env_locate(a, idx, p);
        float G[4]  = {0.f, 0.f, 0.f, 0.f};
        float wgt   = 0.f;
        EnvRay ray;
        if (active)
        {
            wgt = a.weight[p.l][p.pix];
            if ((a.flags & VETR_ENV_NOT_AT_POINTS) && wgt > 0.001f) active = false;
        }
        if (active)
        {
            const long long per_view = (long long)a.lw[p.l] * a.lh[p.l];
            const float* g = a.grad[p.l] + ((long long)p.b * a.C) * per_view + (p.pix - (long long)p.b * per_view);
#pragma unroll
            for (int ch = 0; ch < 4; ++ch)
                if (ch < a.C) G[ch] = g[ch * per_view];
            ray = env_ray(s_cam[p.b], a.lw[p.l], a.lh[p.l], a.scale[p.l], p.x, p.y);
        }
        float alpha[kEnvMaxSpheres], sig[kEnvMaxSpheres], dot[kEnvMaxSpheres], Tin[kEnvMaxSpheres];
        unsigned negative = 0;  // bit 4 s + ch: the raw colour sample is negative; bit 32.. not needed (S <= 8, C <= 4)
        unsigned zero     = 0;  // the raw colour sample is exactly zero (abs has no gradient there)
        float T = env_start_T(wgt, a.flags);
#pragma unroll
        for (int s = 0; s < kEnvMaxSpheres; ++s)
        {
            alpha[s] = 0.f, sig[s] = 0.f, dot[s] = 0.f, Tin[s] = T;
            if (s < a.S && active)
            {
                const EnvTap t = env_tap(a, ray, s);
                if (t.hit)
                {
                    EnvCorners c;
                    env_corners(a, t, c);
                    alpha[s] = 1.f;
                    if (s != a.S - 1)
                    {
                        sig[s]   = 1.f / (1.f + expf(-env_fetch(a.density, c)));
                        alpha[s] = sig[s];
                    }
                    float d = 0.f;
#pragma unroll
                    for (int ch = 0; ch < 4; ++ch)
                        if (ch < a.C)
                        {
                            float col = env_fetch(a.color + ch * plane, c);
                            if (a.non_subzero)
                            {
                                if (col < 0.f) negative |= 1u << (4 * s + ch);
                                if (col == 0.f) zero |= 1u << (4 * s + ch);
                                col = fabsf(col);
                            }
                            d += col * G[ch];
                        }
                    dot[s] = d;
                }
                T = (1.f - alpha[s]) * T;
            }
        }
        float rest = 0.f;
#pragma unroll
        for (int s = kEnvMaxSpheres - 1; s >= 0; --s)
        {
            if (s >= a.S) continue;  // uniform over the grid
            const float g_alpha = Tin[s] * (dot[s] - rest);
            rest                = alpha[s] * dot[s] + (1.f - alpha[s]) * rest;
            EnvTap t;
            t.hit = false;
            if (active) t = env_tap(a, ray, s);
            const bool live = active && t.hit;
            EnvCorners c;
            float gv[5] = {0.f, 0.f, 0.f, 0.f, 0.f};  // gradient of the density sample, then of the colour samples
            int key = -1 - lane;                      // never equal between lanes
            if (live)
            {
                env_corners(a, t, c);
                key   = (t.z0 * a.R + t.y0) * a.R + t.x0;
                gv[0] = s == a.S - 1 ? 0.f : g_alpha * (sig[s] * (1.f - sig[s]));
#pragma unroll
                for (int ch = 0; ch < 4; ++ch)
                    if (ch < a.C)
                    {
                        float v = Tin[s] * alpha[s] * G[ch];
                        if (negative >> (4 * s + ch) & 1) v = -v;
                        if (zero >> (4 * s + ch) & 1) v = 0.f;
                        gv[1 + ch] = v;
                    }
            }
            else
            {
#pragma unroll
                for (int q = 0; q < 8; ++q) c.off[q] = -1, c.w[q] = 0.f;
            }
            // runs of consecutive lanes with the same base texel (the corner offsets of such lanes are the same)
            const int prev       = __shfl_up_sync(0xffffffffu, key, 1);
            const bool head      = lane == 0 || key != prev;
            const unsigned heads = __ballot_sync(0xffffffffu, head);
            const int seg        = __popc(heads & (0xffffffffu >> (31 - lane)));
            unsigned same = 0;  // bit k: lane + 2^k belongs to this lane's run
#pragma unroll
            for (int k = 0; k < 5; ++k)
            {
                const int other = __shfl_down_sync(0xffffffffu, seg, 1 << k);
                if (lane + (1 << k) < 32 && other == seg) same |= 1u << k;
            }
#pragma unroll
            for (int q = 0; q < 8; ++q)
            {
                // a corner no lane of the warp uses (outside the texture, or the empty z slice of a tap that sits on a slice)
                if (!__any_sync(0xffffffffu, c.off[q] >= 0 && c.w[q] != 0.f)) continue;
#pragma unroll
                for (int v = 0; v < 5; ++v)
                {
                    if (v > a.C) continue;
                    if (v == 0 && s == a.S - 1) continue;  // the last sphere's alpha is the constant 1
                    float x = c.off[q] >= 0 ? c.w[q] * gv[v] : 0.f;
                    // (one atomic per lane without this pre-sum was measured 3 % slower)
#pragma unroll
                    for (int k = 0; k < 5; ++k)
                    {
                        const float y = __shfl_down_sync(0xffffffffu, x, 1 << k);
                        if (same >> k & 1) x += y;
                    }
                    if (head && c.off[q] >= 0 && x != 0.f)
                        atomicAdd((v == 0 ? a.g_density : a.g_color + (v - 1) * plane) + c.off[q], x);
                }
            }
        }
    }
}

}  // namespace vetr
