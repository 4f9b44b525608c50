// CPU oracle of VET's differentiable blending point rasterizer.
//
// TEST INFRASTRUCTURE ONLY.  This file is the checker for the CUDA library: it is linked by nothing
// that ships.  It restates, on the CPU and in the same order of fp32 operations as the CUDA kernels
// use for everything that decides a fragment's pixel and depth bits, the algorithm of the reference's
// rasterizer:
//
//   projection            src/lib/rendering/PointRendererHelper.h:184-218, RenderForward.cu:117-158
//   level loop / counting src/lib/rendering/RenderForward.cu:806-905
//   scan + list sizes     src/lib/rendering/PointRenderer.cu:788-824
//   collection            src/lib/rendering/RenderForward.cu:1011-1137
//   per-pixel sort        src/lib/rendering/AlphaListSort.cu:601-703   (ascending depth)
//   blend (mode 1)        src/lib/rendering/RenderForward.cu:1303-1357, PointBlending.h:90-129
//   mode 0 (FUZZY_DT)     src/lib/rendering/RenderForward.cu:180-406, PointRenderer.cu:24-52,
//                         RenderBackward.cu:27-128, 131-474
//   blend (mode 2)        src/lib/rendering/RenderForward.cu:1393-1503
//   blend (mode 3)        src/lib/rendering/RenderForward.cu:1539-1644, PointBlending.h:12-44
//   mask                  src/lib/rendering/PointRenderer.cu:216-235
//   backward (mode 1)     src/lib/rendering/RenderBackward.cu:1083-1513
//   backward (mode 2)     src/lib/rendering/RenderBackward.cu:570-1080
//   backward (mode 3)     src/lib/rendering/RenderBackward.cu:2893-3232
//   projection backward   src/lib/rendering/PointRendererHelper.h:317-372
//   normalisation         src/lib/rendering/PointRenderer.cu:1072-1109,1251-1308
//   tangent application   src/lib/rendering/PointRenderer.cu:1325-1349
//   error grid            src/lib/rendering/RenderForward.cu:639-791
//   environment map       src/lib/rendering/EnvironmentMap.cu:201-287, 378-485, 587-758
//   drop-out radius       src/lib/data/SceneData.cpp:554-597 (ComputeRadius)
//
// PARITY UNPINNED for the camera arithmetic: the reference takes TransformPoint, DivideByZ,
// distortNormalizedPoint, IntrinsicsPinhole::normalizedToImage/scale, ImageView::distanceFromEdge and
// Sophus::se3_expd from the saiga / Sophus libraries (git submodule External/saiga, no pinned commit,
// directory empty in the reference snapshot), and ships no test or golden vector for this path.  Those
// functions are restated here from their published definitions.  The blend algebra IS pinned: the
// reference's own PointBlending.h is compiled (oracle/Makefile, target _ref) and compared with the
// functions below by tests/test_oracle_ref_blend.py.
//
// Canonical list order: ascending (depth bits, point index).  The reference orders by depth only and
// leaves equal depths in atomic arrival order; every order it can produce equals the canonical one up
// to permutations inside runs of equal depth.
//
// Build: see oracle/Makefile (-O3 -fopenmp -ffp-contract=off: no fused multiply-add may be formed by
// the compiler, so that the fp32 results of the projection match the CUDA build made with -fmad=false).

#include <algorithm>
#include <cmath>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#ifdef _OPENMP
#    include <omp.h>
#endif

namespace
{
constexpr int kMaxLayers = 5;  // RenderConstants.h:33

struct OParams  // mirrors the fields of RenderParams the kernels read (Settings.h:19-73)
{
    int render_mode;                  // 0 FUZZY_DT, 1 FULL_BLEND, 2 FUZZY_BLEND, 3 BILINEAR_BLEND (PointRenderer.h: RenderMode)
    int num_layers;                   // 1..5
    int num_channels;                 // 3 or 4
    int drop_out_points_by_radius;    // bool
    float drop_out_radius_threshold;  // 0.6
    float dist_cutoff;                // 20
    int use_environment_map;          // bool: skip the background term
    int viewer_only;                  // bool: low-confidence discard (RenderForward.cu:168-176)
    float stability_cutoff_value;     // 10000
    int debug_max_list_length;        // -1
    int need_point_gradient;          // bool
    float K_gradient_factor;          // 0.5
    float distortion_gradient_factor; // 0.005
    int output_background_mask;       // bool
    float output_background_mask_value;
    int conf_grad_quadratic;          // oracle only: 1 = literal O(n^2) loop of RenderBackward.cu:1160-1178
    int background_alpha_to_point0;   // quirk: RenderBackward.cu:1130,1157 (mode 1)
    float depth_accept_blend;         // 0.01, mode 2 (Settings.h:29)
    float depth_accept;               // 0.01, mode 0 (Settings.h:28)
    int ghost_gradients;              // mode 0: position gradients from dropped-out points instead (Settings.h:31)
};

struct OView  // ReducedImageInfo, data/SceneData.h:39-50
{
    int w, h, image_index, camera_index, camera_model;
    float crop[5];  // fx fy cx cy s
    float rot[4];   // row-major 2x2
};

struct V2
{
    float x, y;
};
struct V3
{
    float x, y, z;
};

// ---------------------------------------------------------------------------------------------
// Camera arithmetic (restated from saiga / Sophus; op order is the contract shared with the kernels)

struct Pose
{
    float q[4];  // x y z w
    float t[3];
};

inline Pose load_pose(const double* p)  // Sophus::SE3d memory: quaternion xyzw, translation, pad; cast per use
{
    Pose r;
    for (int i = 0; i < 4; ++i) r.q[i] = (float)p[i];
    for (int i = 0; i < 3; ++i) r.t[i] = (float)p[4 + i];
    return r;
}

inline V3 cross(V3 a, V3 b) { return {a.y * b.z - a.z * b.y, a.z * b.x - a.x * b.z, a.x * b.y - a.y * b.x}; }

inline V3 rotate(const Pose& P, V3 v)  // Eigen quaternion _transformVector: v + w*uv + qv x uv, uv = 2 qv x v
{
    V3 qv{P.q[0], P.q[1], P.q[2]};
    V3 uv = cross(qv, v);
    uv    = {uv.x + uv.x, uv.y + uv.y, uv.z + uv.z};
    V3 c  = cross(qv, uv);
    float w = P.q[3];
    return {v.x + w * uv.x + c.x, v.y + w * uv.y + c.y, v.z + w * uv.z + c.z};
}

inline V3 transform_point(const Pose& P, V3 p)
{
    V3 r = rotate(P, p);
    return {r.x + P.t[0], r.y + P.t[1], r.z + P.t[2]};
}

inline void rotation_matrix(const Pose& P, float R[9])  // so3().matrix(), Eigen toRotationMatrix order
{
    float x = P.q[0], y = P.q[1], z = P.q[2], w = P.q[3];
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

// OpenCV rational model, coefficients k1 k2 k3 k4 k5 k6 p1 p2; sentinel 100000 beyond the cutoff radius.
inline V2 distort(V2 p, const float* d, float cutoff, float* J_p /*2x2*/, float* J_d /*2x8*/)
{
    float x = p.x, y = p.y;
    float x2 = x * x, y2 = y * y, xy = x * y;
    float r2 = x2 + y2;
    if (r2 > cutoff * cutoff)
    {
        if (J_p) std::fill(J_p, J_p + 4, 0.f);
        if (J_d) std::fill(J_d, J_d + 16, 0.f);
        return {100000.f, 100000.f};
    }
    float r4 = r2 * r2, r6 = r4 * r2;
    float k1 = d[0], k2 = d[1], k3 = d[2], k4 = d[3], k5 = d[4], k6 = d[5], p1 = d[6], p2 = d[7];
    float num    = 1.f + k1 * r2 + k2 * r4 + k3 * r6;
    float den    = 1.f + k4 * r2 + k5 * r4 + k6 * r6;
    float radial = num / den;
    float tx     = 2.f * p1 * xy + p2 * (r2 + 2.f * x2);
    float ty     = 2.f * p2 * xy + p1 * (r2 + 2.f * y2);
    V2 out{x * radial + tx, y * radial + ty};
    if (J_p)
    {
        float dnum_dr2 = k1 + 2.f * k2 * r2 + 3.f * k3 * r4;
        float dden_dr2 = k4 + 2.f * k5 * r2 + 3.f * k6 * r4;
        float drad_dr2 = (dnum_dr2 * den - num * dden_dr2) / (den * den);
        float drad_dx = drad_dr2 * 2.f * x, drad_dy = drad_dr2 * 2.f * y;
        J_p[0] = radial + x * drad_dx + 2.f * p1 * y + p2 * (2.f * x + 4.f * x);
        J_p[1] = x * drad_dy + 2.f * p1 * x + p2 * (2.f * y);
        J_p[2] = y * drad_dx + 2.f * p2 * y + p1 * (2.f * x);
        J_p[3] = radial + y * drad_dy + 2.f * p2 * x + p1 * (2.f * y + 4.f * y);
    }
    if (J_d)
    {
        float inv_den = 1.f / den;
        float a       = -num / (den * den);
        float jx[8]   = {x * r2 * inv_den, x * r4 * inv_den, x * r6 * inv_den, x * a * r2,
                         x * a * r4,       x * a * r6,       2.f * xy,         r2 + 2.f * x2};
        float jy[8]   = {y * r2 * inv_den, y * r4 * inv_den, y * r6 * inv_den, y * a * r2,
                         y * a * r4,       y * a * r6,       r2 + 2.f * y2,    2.f * xy};
        for (int i = 0; i < 8; ++i)
        {
            J_d[i]     = jx[i];
            J_d[8 + i] = jy[i];
        }
    }
    return out;
}

// IntrinsicsPinhole::normalizedToImage with coefficients fx fy cx cy s (data/SceneData.h:198-199)
inline V2 k_apply(const float* K, V2 p) { return {K[0] * p.x + K[4] * p.y + K[2], K[1] * p.y + K[3]}; }

struct Projected
{
    V2 ip;
    float z;
    float radius_px;
};

// ProjPoint, RenderForward.cu:117-158 (pinhole branch) on top of ProjectPointPinhole
inline Projected project(const float* pos4, const Pose& V, const float* intr /*13*/, const OView& cam,
                         float dist_cutoff, bool apply_crop_rotation = true)
{
    V3 vp   = transform_point(V, {pos4[0], pos4[1], pos4[2]});
    float z = std::fmax(vp.z, 0.f);
    V2 np{vp.x / vp.z, vp.y / vp.z};
    V2 dp = distort(np, intr + 5, dist_cutoff, nullptr, nullptr);
    if (dp.x == 100000.f) z = 0;
    V2 ip = k_apply(intr, dp);
    float radius_px = intr[0] * cam.crop[0] * pos4[3] / z;
    ip = k_apply(cam.crop, ip);
    if (!apply_crop_rotation) return {ip, z, radius_px};  // mode 0's backward copy of ProjPoint, RenderBackward.cu:78-116
    float cx = (float)(cam.w / 2), cy = (float)(cam.h / 2);  // integer division, RenderForward.cu:156
    float dx = ip.x - cx, dy = ip.y - cy;
    ip = {cam.rot[0] * dx + cam.rot[1] * dy, cam.rot[2] * dx + cam.rot[3] * dy};
    ip = {ip.x + cx, ip.y + cy};
    return {ip, z, radius_px};
}

inline int round_half_even(float v)  // __float2int_rn; out-of-range and NaN go outside every image
{
    if (!(v > -1.0e9f && v < 1.0e9f)) return INT32_MIN;
    return (int)std::nearbyintf(v);
}
inline int round_down(float v)  // __float2int_rd
{
    if (!(v > -1.0e9f && v < 1.0e9f)) return INT32_MIN;
    return (int)std::floor(v);
}

// compute_blending_fac, PointBlending.h:12-44
inline void blending_fac(V2 uv, float w[4], float J[8] /*4x2 or null*/)
{
    float sx = uv.x - std::floor(uv.x), sy = uv.y - std::floor(uv.y);
    w[0] = (1 - sx) * (1 - sy);
    w[1] = sx * (1 - sy);
    w[2] = (1 - sx) * sy;
    w[3] = sx * sy;
    if (J)
    {
        J[0] = sy - 1;
        J[1] = sx - 1;
        J[2] = 1 - sy;
        J[3] = -sx;
        J[4] = -sy;
        J[5] = 1 - sx;
        J[6] = sy;
        J[7] = sx;
    }
}

// compute_blend / compute_new_alphadest, PointBlending.h:90-129.  nvcc contracts the reference's
// `alpha_dest * alpha_s * color + color_dest` into one fused multiply-add; so do we, explicitly.
inline float blend(float T, float a, float c, float dst) { return std::fmaf(T * a, c, dst); }
inline float new_T(float T, float a) { return (1 - a) * T; }

struct BackOut
{
    float g_point[3], g_pose[6], g_k[5], g_dis[8];
};

// ProjectPointPinholeBackward, PointRendererHelper.h:317-372
inline bool project_backward(const float* pos4, V2 grad, const Pose& V, const float* intr, const float cropK[5],
                             const float rot[4], float dist_cutoff, BackOut& o)
{
    std::memset(&o, 0, sizeof(o));
    V3 vp = transform_point(V, {pos4[0], pos4[1], pos4[2]});
    if (vp.z <= 0) return false;
    float R[9];
    rotation_matrix(V, R);  // J_point
    // J_pose = [ I | -skew(vp) ]
    float Jpose[18] = {1, 0, 0, 0,     vp.z,  -vp.y,   //
                       0, 1, 0, -vp.z, 0,     vp.x,    //
                       0, 0, 1, vp.y,  -vp.x, 0};
    float iz = 1.f / vp.z;
    float Jdiv[6] = {iz, 0, -vp.x * iz * iz, 0, iz, -vp.y * iz * iz};
    V2 np{vp.x / vp.z, vp.y / vp.z};
    float Jpd[4], Jdd[16];
    V2 dp = distort(np, intr + 5, dist_cutoff, Jpd, Jdd);
    float JpK1[4] = {intr[0], intr[4], 0, intr[1]};
    float JkK1[10] = {dp.x, 0, 1, 0, dp.y,  //
                      0, dp.y, 0, 1, 0};
    float JpK2[4] = {cropK[0], cropK[4], 0, cropK[1]};

    // grad_p_rot = rot^T grad
    V2 g_rot{rot[0] * grad.x + rot[2] * grad.y, rot[1] * grad.x + rot[3] * grad.y};
    V2 g_k2{JpK2[0] * g_rot.x + JpK2[2] * g_rot.y, JpK2[1] * g_rot.x + JpK2[3] * g_rot.y};
    V2 g_k1{JpK1[0] * g_k2.x + JpK1[2] * g_k2.y, JpK1[1] * g_k2.x + JpK1[3] * g_k2.y};
    V2 g_dis{Jpd[0] * g_k1.x + Jpd[2] * g_k1.y, Jpd[1] * g_k1.x + Jpd[3] * g_k1.y};
    float g_view[3] = {Jdiv[0] * g_dis.x + Jdiv[3] * g_dis.y, Jdiv[1] * g_dis.x + Jdiv[4] * g_dis.y,
                       Jdiv[2] * g_dis.x + Jdiv[5] * g_dis.y};
    for (int k = 0; k < 3; ++k) o.g_point[k] = R[0 + k] * g_view[0] + R[3 + k] * g_view[1] + R[6 + k] * g_view[2];
    for (int k = 0; k < 6; ++k)
        o.g_pose[k] = Jpose[0 + k] * g_view[0] + Jpose[6 + k] * g_view[1] + Jpose[12 + k] * g_view[2];
    for (int k = 0; k < 5; ++k) o.g_k[k] = JkK1[k] * g_k2.x + JkK1[5 + k] * g_k2.y;
    for (int k = 0; k < 8; ++k) o.g_dis[k] = Jdd[k] * g_k1.x + Jdd[8 + k] * g_k1.y;
    return true;
}

struct Level
{
    int w, h;
    int64_t base;  // offset of this level inside one view's pyramid
};

struct Oracle
{
    OParams prm{};
    int B = 0, L = 0, C = 0;
    int64_t P = 0;  // pyramid pixels per view
    Level lv[kMaxLayers]{};
    std::vector<OView> views;
    std::vector<int32_t> count;    // [B*P]
    std::vector<int64_t> start;    // [B*P + 1] exclusive scan
    std::vector<uint64_t> keys;    // [F] sorted per pixel: depth bits << 32 | point id
    std::vector<float> uv;         // mode 3: [F,2] level-space ip of the fragment (per_point_data cols 1,2)
    std::vector<uint8_t> corner;   // mode 3: [F] blend index (per_point_data col 3)
    std::vector<std::vector<float>> out_color;  // per level [B,C,h,w]
    // inputs kept for backward
    int n = 0, n_tex = 0, n_img = 0, n_cam = 0;
    const float* position = nullptr;
    const int* index      = nullptr;
    const float* texture  = nullptr;
    const float* conf     = nullptr;
    const float* bg       = nullptr;
    const double* poses   = nullptr;
    const float* intr     = nullptr;
    bool abs_mode         = false;
    // mode 0
    std::vector<float> depth0;     // [B*P] nearest depth (100000 where empty)
    std::vector<float> weight0;    // [B*P] number of accepted points
    std::vector<float> dropout;    // copy of the drop-out mask (the backward pass reads it)
};

void setup_levels(Oracle& o, int w, int h)
{
    int64_t base = 0;
    for (int l = 0; l < o.L; ++l)
    {
        o.lv[l] = {w, h, base};
        base += (int64_t)w * h;
        w /= 2;  // PointRenderer.cu:378-380
        h /= 2;
    }
    o.P = base;
}

// Visits every fragment of one point in one view in the order of the level loop.
template <class F>
inline void for_fragments(const Oracle& o, int b, int pid, const float* dropout, F&& f)
{
    const OParams& prm = o.prm;
    if (dropout && dropout[(int64_t)b * o.n + pid] == 1.f) return;
    int tex = o.index[pid];
    if (prm.viewer_only && o.conf[tex] < prm.stability_cutoff_value) return;  // RenderForward.cu:168-176
    const OView& cam = o.views[b];
    Pose V           = load_pose(o.poses + 8 * cam.image_index);
    Projected pr     = project(o.position + 4 * pid, V, o.intr + 13 * cam.camera_index, cam, prm.dist_cutoff);
    if (pr.z == 0) return;
    V2 ip        = pr.ip;
    float radius = pr.radius_px;
    uint32_t zb;
    std::memcpy(&zb, &pr.z, 4);
    for (int l = 0; l < o.L; ++l, radius *= 0.5f, ip = {ip.x * 0.5f, ip.y * 0.5f})
    {
        if (prm.drop_out_points_by_radius && radius < prm.drop_out_radius_threshold) break;
        const Level& lv = o.lv[l];
        if (prm.render_mode == 3)
        {
            int bx = round_down(ip.x), by = round_down(ip.y);
            for (int yj = 0; yj <= 1; ++yj)
                for (int xi = 0; xi <= 1; ++xi)
                {
                    int64_t x = (int64_t)bx + xi, y = (int64_t)by + yj;
                    if (x < 0 || y < 0 || x >= lv.w || y >= lv.h) continue;
                    f(l, (int)x, (int)y, zb, ip, yj * 2 + xi);
                }
        }
        else
        {
            int x = round_half_even(ip.x), y = round_half_even(ip.y);
            if (x < 0 || y < 0 || x >= lv.w || y >= lv.h) continue;
            f(l, x, y, zb, ip, 0);
        }
    }
}

}  // namespace

extern "C"
{
void* vo_create() { return new Oracle(); }
void vo_destroy(void* h) { delete (Oracle*)h; }
int vo_threads()
{
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
// Number of OpenMP threads of the following calls (a launcher may have set OMP_NUM_THREADS=1 for the process).
void vo_set_threads(int n)
{
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#endif
}

// Forward.  out_color[l] is [B,C,h_l,w_l]; out_weight[l], out_mask[l] (nullable), out_depth[l] (nullable) are
// [B,1,h_l,w_l].  Returns the number of fragments F, or a negative value on invalid arguments.
int64_t vo_forward(void* h, const OParams* prm, int n, const float* position, const int* index, int n_tex,
                   const float* texture, const float* confidence, const float* background, int n_img,
                   const double* poses, int n_cam, const float* intrinsics, const OView* views, int B,
                   const float* dropout, float* const* out_color, float* const* out_weight, float* const* out_mask,
                   float* const* out_depth)
{
    Oracle& o = *(Oracle*)h;
    if (prm->num_layers < 1 || prm->num_layers > kMaxLayers || B < 1) return -1;
    if (prm->render_mode < 0 || prm->render_mode > 3) return -1;
    for (int b = 0; b < B; ++b)
        if (views[b].camera_model != 0 || views[b].w != views[0].w || views[b].h != views[0].h) return -1;
    o.prm = *prm;
    o.B = B, o.L = prm->num_layers, o.C = prm->num_channels;
    o.views.assign(views, views + B);
    o.n = n, o.n_tex = n_tex, o.n_img = n_img, o.n_cam = n_cam;
    o.position = position, o.index = index, o.texture = texture, o.conf = confidence, o.bg = background;
    o.poses = poses, o.intr = intrinsics;
    setup_levels(o, views[0].w, views[0].h);
    const bool bilinear = prm->render_mode == 3;
    const int64_t PT    = o.P * B;
    o.dropout.clear();
    if (dropout) o.dropout.assign(dropout, dropout + (int64_t)B * n);

    if (prm->render_mode == 0)
    {
        // FUZZY_DT: DepthPrepassMulti (no drop-out test), RenderForwardMulti (drop-out test, depth test against the
        // nearest depth), CombineAndFill.
        const int C = prm->num_channels;
        o.count.assign(PT, 0);
        o.keys.clear();
        o.depth0.assign(PT, 100000.f);
        o.weight0.assign(PT, 0.f);
        std::vector<double> accum((size_t)PT * C, 0.0);
        for (int b = 0; b < B; ++b)
            for (int pid = 0; pid < n; ++pid)
                for_fragments(o, b, pid, nullptr, [&](int l, int x, int y, uint32_t zb, V2, int) {
                    float z;
                    std::memcpy(&z, &zb, 4);
                    float& d = o.depth0[b * o.P + o.lv[l].base + (int64_t)y * o.lv[l].w + x];
                    d = std::min(d, z);
                });
        int64_t F0 = 0;
        for (int b = 0; b < B; ++b)
            for (int pid = 0; pid < n; ++pid)
                for_fragments(o, b, pid, dropout, [&](int l, int x, int y, uint32_t zb, V2, int) {
                    float z;
                    std::memcpy(&z, &zb, 4);
                    int64_t g = b * o.P + o.lv[l].base + (int64_t)y * o.lv[l].w + x;
                    if (z > o.depth0[g] * (prm->depth_accept + 1)) return;
                    int tex = index[pid];
                    for (int ci = 0; ci < C; ++ci) accum[(size_t)g * C + ci] += (double)texture[(int64_t)ci * n_tex + tex];
                    o.weight0[g] += 1.f;
                    o.count[g] += 1;
                    ++F0;
                });
        o.out_color.resize(o.L);
        for (int l = 0; l < o.L; ++l)
        {
            const Level& lv  = o.lv[l];
            const int64_t hw = (int64_t)lv.w * lv.h;
            o.out_color[l].assign((size_t)B * C * hw, 0.f);
            for (int b = 0; b < B; ++b)
                for (int64_t q = 0; q < hw; ++q)
                {
                    int64_t g = b * o.P + lv.base + q;
                    float w   = o.weight0[g];
                    for (int ci = 0; ci < C; ++ci)
                    {
                        float v = w == 0 ? background[ci] : (float)accum[(size_t)g * C + ci] / w;
                        o.out_color[l][((int64_t)b * C + ci) * hw + q] = v;
                        if (out_color) out_color[l][((int64_t)b * C + ci) * hw + q] = v;
                    }
                    if (out_weight) out_weight[l][b * hw + q] = w;
                    if (out_mask) out_mask[l][b * hw + q] = (w == 0.f) ? prm->output_background_mask_value : 1.f;
                    if (out_depth) out_depth[l][b * hw + q] = o.depth0[g];
                }
        }
        o.start.assign(PT + 1, 0);
        return F0;
    }

    // counting pass
    o.count.assign(PT, 0);
    for (int b = 0; b < B; ++b)
    {
        int32_t* cnt = o.count.data() + b * o.P;
#pragma omp parallel for schedule(static)
        for (int pid = 0; pid < n; ++pid)
            for_fragments(o, b, pid, dropout, [&](int l, int x, int y, uint32_t, V2, int) {
#pragma omp atomic
                cnt[o.lv[l].base + (int64_t)y * o.lv[l].w + x] += 1;
            });
    }
    // scan
    o.start.resize(PT + 1);
    int64_t acc = 0;
    for (int64_t i = 0; i < PT; ++i)
    {
        o.start[i] = acc;
        acc += o.count[i];
    }
    o.start[PT]     = acc;
    const int64_t F = acc;
    o.keys.resize(F);
    if (bilinear)
    {
        o.uv.resize(2 * F);
        o.corner.resize(F);
    }
    // collection pass (serial over points per view so that the cursor needs no atomics across the big arrays)
    std::vector<int32_t> cursor(PT, 0);
    std::vector<uint32_t> aux;  // mode 3: arrival slot -> (uv, corner) before sorting
    std::vector<float> uv_unsorted;
    std::vector<uint8_t> corner_unsorted;
    if (bilinear)
    {
        uv_unsorted.resize(2 * F);
        corner_unsorted.resize(F);
    }
    for (int b = 0; b < B; ++b)
    {
        const int64_t vb = b * o.P;
#pragma omp parallel for schedule(static)
        for (int pid = 0; pid < n; ++pid)
            for_fragments(o, b, pid, dropout, [&](int l, int x, int y, uint32_t zb, V2 ip, int corner) {
                int64_t g = vb + o.lv[l].base + (int64_t)y * o.lv[l].w + x;
                int32_t pos;
#pragma omp atomic capture
                pos = cursor[g]++;
                int64_t slot  = o.start[g] + pos;
                o.keys[slot]  = ((uint64_t)zb << 32) | (uint32_t)pid;
                if (bilinear)
                {
                    uv_unsorted[2 * slot]     = ip.x;
                    uv_unsorted[2 * slot + 1] = ip.y;
                    corner_unsorted[slot]     = (uint8_t)corner;
                }
            });
    }
    // sort every list by (depth bits, point id); mode 3 carries uv and corner along
#pragma omp parallel
    {
        std::vector<std::pair<uint64_t, int64_t>> tmp;
#pragma omp for schedule(dynamic, 4096)
        for (int64_t g = 0; g < PT; ++g)
        {
            int64_t s = o.start[g], e = o.start[g + 1];
            if (e - s == 0) continue;
            if (!bilinear)
            {
                if (e - s > 1) std::sort(o.keys.begin() + s, o.keys.begin() + e);
                continue;
            }
            tmp.clear();
            for (int64_t i = s; i < e; ++i) tmp.push_back({o.keys[i], i});
            std::sort(tmp.begin(), tmp.end());
            for (int64_t i = s; i < e; ++i)
            {
                int64_t src       = tmp[i - s].second;
                o.keys[i]         = tmp[i - s].first;
                o.uv[2 * i]       = uv_unsorted[2 * src];
                o.uv[2 * i + 1]   = uv_unsorted[2 * src + 1];
                o.corner[i]       = corner_unsorted[src];
            }
        }
    }
    // blend
    const int C = o.C;
    o.out_color.resize(o.L);
    for (int l = 0; l < o.L; ++l)
    {
        const Level& lv = o.lv[l];
        const int64_t hw = (int64_t)lv.w * lv.h;
        o.out_color[l].assign((size_t)B * C * hw, 0.f);
#pragma omp parallel for schedule(dynamic, 64) collapse(2)
        for (int b = 0; b < B; ++b)
            for (int y = 0; y < lv.h; ++y)
                for (int x = 0; x < lv.w; ++x)
                {
                    int64_t g  = b * o.P + lv.base + (int64_t)y * lv.w + x;
                    int64_t s  = o.start[g];
                    int cnt    = o.count[g];
                    if (prm->debug_max_list_length > 0) cnt = std::min(prm->debug_max_list_length, cnt);
                    float T    = 1.f;
                    float c[4] = {0, 0, 0, 0};
                    if (prm->render_mode == 2)
                    {
                        // BlendMultiFuzzy, RenderForward.cu:1412-1492, transcribed literally: fragments within
                        // depth_accept_blend of the FIRST depth are averaged; after that group the reference resets its
                        // reference depth to -100000, so every later fragment is a group of its own.
                        float last_min_d = 0.f, acc_conf = 0.f, acc_desc[4] = {0, 0, 0, 0};
                        int n_acc = 0;
                        auto accumulate = [&]() {
                            float conf = acc_conf / float(n_acc);
                            for (int ci = 0; ci < C; ++ci) c[ci] = blend(T, conf, acc_desc[ci] / float(n_acc), c[ci]);
                            T = new_T(T, conf);
                        };
                        for (int i = 0; i < cnt; ++i)
                        {
                            uint32_t zb = (uint32_t)(o.keys[s + i] >> 32);
                            float d;
                            std::memcpy(&d, &zb, 4);
                            int tex = index[(int)(uint32_t)o.keys[s + i]];
                            if (last_min_d == 0.f) last_min_d = d;
                            if (!(d - last_min_d < prm->depth_accept_blend))
                            {
                                accumulate();
                                last_min_d = -100000.f;
                                acc_conf   = 0.f;
                                n_acc      = 0;
                                for (int ci = 0; ci < C; ++ci) acc_desc[ci] = 0.f;
                            }
                            acc_conf += confidence[tex];
                            for (int ci = 0; ci < C; ++ci) acc_desc[ci] += texture[(int64_t)ci * n_tex + tex];
                            ++n_acc;
                        }
                        if (n_acc > 0) accumulate();
                        cnt = 0;  // the plain loop below has nothing left to do
                    }
                    for (int i = 0; i < cnt; ++i)
                    {
                        int pid   = (int)(uint32_t)o.keys[s + i];
                        int tex   = index[pid];
                        float a   = confidence[tex];
                        if (bilinear)
                        {
                            float w4[4];
                            blending_fac({o.uv[2 * (s + i)], o.uv[2 * (s + i) + 1]}, w4, nullptr);
                            a = w4[o.corner[s + i]] * a;
                        }
                        for (int ci = 0; ci < C; ++ci) c[ci] = blend(T, a, texture[(int64_t)ci * n_tex + tex], c[ci]);
                        T = new_T(T, a);
                        if (bilinear && T < 0.001f) break;
                    }
                    for (int ci = 0; ci < C; ++ci)
                    {
                        bool add_bg = !prm->use_environment_map && !(bilinear && !(T >= 0.001f));
                        if (add_bg) c[ci] = blend(T, 1.f, background[ci], c[ci]);
                        float v = c[ci];
                        o.out_color[l][((int64_t)b * C + ci) * hw + (int64_t)y * lv.w + x] = v;
                        if (out_color) out_color[l][((int64_t)b * C + ci) * hw + (int64_t)y * lv.w + x] = v;
                    }
                    int64_t pi = (int64_t)b * hw + (int64_t)y * lv.w + x;
                    if (out_weight) out_weight[l][pi] = T;
                    if (out_mask) out_mask[l][pi] = (T == 0.f) ? prm->output_background_mask_value : 1.f;
                    if (out_depth)
                    {
                        float d = 100000.f;  // MAX_DEPTH_CONST; atomicMin of depth bits == first list entry
                        if (o.count[g] > 0)
                        {
                            uint32_t zb = (uint32_t)(o.keys[s] >> 32);
                            std::memcpy(&d, &zb, 4);
                        }
                        out_depth[l][pi] = d;
                    }
                }
    }
    return F;
}

int64_t vo_pixels_per_view(void* h) { return ((Oracle*)h)->P; }

// Copies the per-pixel counts [B*P] and the sorted keys [F] of the last forward.
void vo_get_lists(void* h, int32_t* counts, uint64_t* keys)
{
    Oracle& o = *(Oracle*)h;
    if (counts) std::memcpy(counts, o.count.data(), o.count.size() * sizeof(int32_t));
    if (keys) std::memcpy(keys, o.keys.data(), o.keys.size() * sizeof(uint64_t));
}

// Backward of the last forward.  grad_color[l] is [B,C,h_l,w_l].  All outputs are RAW SUMS in double
// (each addend computed in fp32 exactly as the reference computes it, then accumulated in fp64 so that
// the oracle carries no summation-order noise of its own):
//   g_texture [C,n_tex], g_confidence [n_tex], g_background [C], g_points [n,3], g_points_count [n],
//   g_pose [n_img,6], g_pose_count [n_img], g_intr [n_cam,13], g_intr_count [n_cam].  Nullable from g_points on.
int vo_backward(void* h, const float* const* grad_color, double* g_texture, double* g_confidence,
                double* g_background, double* g_points, double* g_points_count, double* g_pose, double* g_pose_count,
                double* g_intr, double* g_intr_count)
{
    Oracle& o          = *(Oracle*)h;
    const OParams& prm = o.prm;
#define ACC(dst, v)                                                              \
    do                                                                           \
    {                                                                            \
        double v_ = o.abs_mode ? std::fabs((double)(v)) : (double)(v);           \
        _Pragma("omp atomic") (dst) += v_;                                       \
    } while (0)
#define ACCL(dst, v) (dst) += (o.abs_mode ? std::fabs((double)(v)) : (double)(v))  /* a thread's own accumulator */
    const int C = o.C, B = o.B;
    const bool bilinear = prm.render_mode == 3;
    const int n_tex     = o.n_tex;
    std::fill(g_texture, g_texture + (int64_t)C * n_tex, 0.0);
    std::fill(g_confidence, g_confidence + n_tex, 0.0);
    std::fill(g_background, g_background + C, 0.0);
    if (g_points) std::fill(g_points, g_points + 3 * (int64_t)o.n, 0.0);
    if (g_points_count) std::fill(g_points_count, g_points_count + o.n, 0.0);
    if (g_pose) std::fill(g_pose, g_pose + 6 * o.n_img, 0.0);
    if (g_pose_count) std::fill(g_pose_count, g_pose_count + o.n_img, 0.0);
    if (g_intr) std::fill(g_intr, g_intr + 13 * o.n_cam, 0.0);
    if (g_intr_count) std::fill(g_intr_count, g_intr_count + o.n_cam, 0.0);

    if (prm.render_mode == 0)
    {
        // CombineAndFillBackward: the background receives the gradient of every empty pixel
        for (int l = 0; l < o.L; ++l)
        {
            const Level& lv  = o.lv[l];
            const int64_t hw = (int64_t)lv.w * lv.h;
            for (int b = 0; b < B; ++b)
                for (int64_t q = 0; q < hw; ++q)
                    if (o.weight0[b * o.P + lv.base + q] == 0)
                        for (int ci = 0; ci < C; ++ci) ACC(g_background[ci], grad_color[l][((int64_t)b * C + ci) * hw + q]);
        }
        // RenderBackward: one pass over the points per view; pixel positions come from the backward's own copy of the
        // projection, which leaves out the crop rotation
        for (int b = 0; b < B; ++b)
        {
            const OView& cam = o.views[b];
            Pose V           = load_pose(o.poses + 8 * cam.image_index);
            const float* K   = o.intr + 13 * cam.camera_index;
            for (int pid = 0; pid < o.n; ++pid)
            {
                const bool drop_out = !o.dropout.empty() && o.dropout[(int64_t)b * o.n + pid] == 1.f;
                Projected pr = project(o.position + 4 * pid, V, K, cam, prm.dist_cutoff, false);
                if (pr.z == 0) continue;
                const int tex = o.index[pid];
                V2 ip = pr.ip;
                float radius = pr.radius_px, scale = 1.f;
                for (int l = 0; l < o.L; ++l, scale *= 0.5f, radius *= 0.5f, ip = {ip.x * 0.5f, ip.y * 0.5f})
                {
                    if (prm.drop_out_points_by_radius && radius < prm.drop_out_radius_threshold) continue;
                    const Level& lv = o.lv[l];
                    const int64_t hw = (int64_t)lv.w * lv.h;
                    int x = round_half_even(ip.x), y = round_half_even(ip.y);
                    if (x < 0 || y < 0 || x >= lv.w || y >= lv.h) continue;
                    int64_t g = b * o.P + lv.base + (int64_t)y * lv.w + x;
                    float w   = o.weight0[g];
                    if (w == 0) continue;
                    if (pr.z > o.depth0[g] * (prm.depth_accept + 1)) continue;
                    const float* G = grad_color[l] + (int64_t)b * C * hw;
                    const float* I = o.out_color[l].data() + (int64_t)b * C * hw;
                    if (!drop_out)
                    {
                        float iw = 1.f / w;
                        for (int ci = 0; ci < C; ++ci) ACC(g_texture[(int64_t)ci * n_tex + tex], iw * G[ci * hw + (int64_t)y * lv.w + x]);
                    }
                    bool point_grad = (prm.ghost_gradients && drop_out) | (!prm.ghost_gradients && !drop_out);
                    int dist_edge   = std::min(std::min(x, lv.w - 1 - x), std::min(y, lv.h - 1 - y));
                    if (!(point_grad && dist_edge > 2)) continue;
                    float dx = 0, dy = 0;
                    for (int ci = 0; ci < C; ++ci)
                    {
                        float Tp = o.texture[(int64_t)ci * n_tex + tex];
                        auto at  = [&](const float* img, int xx, int yy) { return img[ci * hw + (int64_t)yy * lv.w + xx]; };
                        float a0 = -((Tp - at(I, x - 1, y)) * at(G, x - 1, y));
                        float a1 = (Tp - at(I, x + 1, y)) * at(G, x + 1, y);
                        float b0 = -((Tp - at(I, x, y - 1)) * at(G, x, y - 1));
                        float b1 = (Tp - at(I, x, y + 1)) * at(G, x, y + 1);
                        dx += 0.5f * (a0 + a1);
                        dy += 0.5f * (b0 + b1);
                    }
                    V2 dR{dx / (float)C, dy / (float)C};
                    float crop2[5];
                    for (int k = 0; k < 5; ++k) crop2[k] = cam.crop[k] * scale;
                    BackOut bo;
                    if (!project_backward(o.position + 4 * pid, dR, V, K, crop2, cam.rot, prm.dist_cutoff, bo)) continue;
                    if (g_points)
                    {
                        for (int k = 0; k < 3; ++k) ACC(g_points[3 * (int64_t)pid + k], bo.g_point[k]);
                        g_points_count[pid] += 1.0;
                    }
                    if (g_pose)
                    {
                        for (int k = 0; k < 6; ++k) ACC(g_pose[6 * cam.image_index + k], bo.g_pose[k]);
                        g_pose_count[cam.image_index] += 1.0;  // RenderBackward.cu:379
                    }
                    if (g_intr)
                    {
                        bo.g_k[4] *= 0;
                        for (int k = 0; k < 5; ++k) ACC(g_intr[13 * cam.camera_index + k], prm.K_gradient_factor * bo.g_k[k]);
                        bo.g_dis[2] *= 0.25f;
                        for (int k = 3; k < 8; ++k) bo.g_dis[k] *= 0.1f;
                        for (int k = 0; k < 8; ++k)
                            ACC(g_intr[13 * cam.camera_index + 5 + k], prm.distortion_gradient_factor * bo.g_dis[k]);
                        g_intr_count[cam.camera_index] += (double)(1.f / 1024.f);
                    }
                }
            }
        }
        return 0;
    }

    std::vector<float> galpha;  // mode 3: gradient_sum_backwards row 0
    if (bilinear) galpha.assign(o.keys.size(), 0.f);

    for (int l = 0; l < o.L; ++l)
    {
        const Level& lv  = o.lv[l];
        const int64_t hw = (int64_t)lv.w * lv.h;
        float level_scale = 1.f;
        for (int i = 0; i < l; ++i) level_scale *= 0.5f;  // powf(0.5f, layer) is exact
        for (int b = 0; b < B; ++b)
        {
            const OView& cam = o.views[b];
            const float* G   = grad_color[l] + (int64_t)b * C * hw;
            const float* I   = o.out_color[l].data() + (int64_t)b * C * hw;
            Pose V           = load_pose(o.poses + 8 * cam.image_index);
            const float* K   = o.intr + 13 * cam.camera_index;
            float crop2[5];
            for (int k = 0; k < 5; ++k) crop2[k] = cam.crop[k] * level_scale;  // IntrinsicsPinhole::scale
            // Rows in parallel; the per-point fp64 accumulators are updated atomically (their summation order then
            // varies from run to run at the 1e-16 level, far below what is compared).  The sums that every pixel of a
            // view adds to (camera, background, descriptor 0's confidence term of the background entry) are kept per
            // thread and added once per thread: atomics on those few addresses would serialise the threads.
#pragma omp parallel
            {
            double t_bg[4] = {0, 0, 0, 0}, t_conf0 = 0, t_pose[6] = {0, 0, 0, 0, 0, 0}, t_pose_count = 0, t_intr[13], t_intr_count = 0;
            for (int k = 0; k < 13; ++k) t_intr[k] = 0;
#pragma omp for schedule(dynamic, 4) nowait
            for (int y = 0; y < lv.h; ++y)
                for (int x = 0; x < lv.w; ++x)
                {
                    int64_t g = b * o.P + lv.base + (int64_t)y * lv.w + x;
                    int64_t s = o.start[g];
                    int cnt   = o.count[g];
                    if (prm.debug_max_list_length > 0) cnt = std::min(prm.debug_max_list_length, cnt);
                    float gin[4];
                    for (int ci = 0; ci < C; ++ci) gin[ci] = G[ci * hw + (int64_t)y * lv.w + x];

                    auto alpha_of = [&](int j) {
                        int tex = o.index[(int)(uint32_t)o.keys[s + j]];
                        float a = o.conf[tex];
                        if (bilinear)
                        {
                            float w4[4];
                            blending_fac({o.uv[2 * (s + j)], o.uv[2 * (s + j) + 1]}, w4, nullptr);
                            a = w4[o.corner[s + j]] * a;
                        }
                        return a;
                    };

                    // (i) mode 2: BlendBackwardsFuzzy, RenderBackward.cu:603-749, transcribed literally.  Groups here are formed
                    // against the first depth of EVERY group (unlike the forward pass) and the background is an entry of
                    // depth 100000; the alpha gradient passed to earlier entries is not divided by their group size.
                    if (prm.render_mode == 2)
                    {
                        const int list_size = prm.use_environment_map ? cnt : cnt + 1;
                        float last_min_d = 0.f, acc_conf = 0.f, acc_desc[4] = {0, 0, 0, 0}, T = 1.f;
                        int n_acc = 0, start = 0;
                        static thread_local std::vector<float> group_conf;  // gradient_sum_backwards row C
                        group_conf.assign(list_size, 0.f);
                        auto tex_of = [&](int t) { return o.index[(int)(uint32_t)o.keys[s + t]]; };
                        auto accumulate = [&]() {
                            float inv_w = 1.f / float(n_acc);
                            float conf  = acc_conf * inv_w;
                            float colors[4], g_colors[4], g_alpha = 0;
                            for (int ci = 0; ci < C; ++ci) colors[ci] = acc_desc[ci] * inv_w;
                            for (int ci = 0; ci < C; ++ci)
                            {
                                g_colors[ci] = T * conf * gin[ci];
                                g_alpha += colors[ci] * gin[ci];
                            }
                            g_alpha *= T;
                            for (int t = start; t < start + n_acc; ++t)
                            {
                                bool fg = t != cnt;
                                for (int ci = 0; ci < C; ++ci)
                                {
                                    if (fg)
                                        ACC(g_texture[(int64_t)ci * n_tex + tex_of(t)], g_colors[ci] * inv_w);
                                    else
                                        ACCL(t_bg[ci], g_colors[ci] * inv_w);
                                }
                                if (fg)
                                {
                                    ACC(g_confidence[tex_of(t)], g_alpha * inv_w);
                                    group_conf[t] = conf;
                                }
                            }
                            for (int j = 0; j < start; ++j)
                            {
                                float g_iter = 0;
                                for (int ci = 0; ci < C; ++ci) g_iter -= (gin[ci] * colors[ci] * T * conf / (1 - group_conf[j] + 1e-9f));
                                ACC(g_confidence[tex_of(j)], g_iter);
                            }
                            T = new_T(T, conf);
                        };
                        for (int i = 0; i < list_size; ++i)
                        {
                            bool fg = i != cnt;
                            float d = 100000.f;
                            if (fg)
                            {
                                uint32_t zb = (uint32_t)(o.keys[s + i] >> 32);
                                std::memcpy(&d, &zb, 4);
                            }
                            if (!(d - last_min_d < prm.depth_accept_blend))
                            {
                                if (i != 0) accumulate();
                                acc_conf = 0.f, n_acc = 0;
                                for (int ci = 0; ci < C; ++ci) acc_desc[ci] = 0.f;
                                last_min_d = d;
                                start      = i;
                            }
                            acc_conf += fg ? o.conf[tex_of(i)] : 1.f;
                            for (int ci = 0; ci < C; ++ci) acc_desc[ci] += fg ? o.texture[(int64_t)ci * n_tex + tex_of(i)] : o.bg[ci];
                            ++n_acc;
                        }
                        if (n_acc > 0) accumulate();
                    }
                    // (i) colour / alpha gradients: RenderBackward.cu:1118-1181 and :2936-3019
                    else
                    {
                        float T       = 1.f;
                        const int cnt0 = cnt;
                        int list_size = prm.use_environment_map ? cnt : cnt + 1;
                        // O(n) form needs the per-entry weights first
                        static thread_local std::vector<float> Ti, ai, doti;
                        Ti.clear(), ai.clear(), doti.clear();
                        int processed = 0;
                        for (int i = 0; i < list_size; ++i)
                        {
                            bool fg  = i != cnt;
                            int tex  = fg ? o.index[(int)(uint32_t)o.keys[s + i]] : 0;
                            float a  = fg ? alpha_of(i) : 1.f;
                            float col[4];
                            for (int ci = 0; ci < C; ++ci) col[ci] = fg ? o.texture[(int64_t)ci * n_tex + tex] : o.bg[ci];
                            float g_alpha = 0;
                            for (int ci = 0; ci < C; ++ci)
                            {
                                float g_col = T * a * gin[ci];
                                if (fg)
                                    ACC(g_texture[(int64_t)ci * n_tex + tex], g_col);
                                else
                                    ACCL(t_bg[ci], g_col);
                                g_alpha += col[ci] * gin[ci];
                            }
                            g_alpha *= T;
                            if (!bilinear)
                            {
                                if (fg)
                                    ACC(g_confidence[tex], g_alpha);
                                else if (prm.background_alpha_to_point0)
                                    ACCL(t_conf0, g_alpha);  // the background entry's texture index stays 0
                            }
                            else if (fg)
                                galpha[s + i] += o.abs_mode ? std::fabs(g_alpha) : g_alpha;

                            if (prm.conf_grad_quadratic)
                            {
                                for (int j = 0; j < i; ++j)
                                {
                                    float aj     = alpha_of(j);
                                    float g_iter = 0;
                                    for (int ci = 0; ci < C; ++ci)
                                        g_iter -= (gin[ci] * col[ci] * T * a / (1 - aj + 1e-9f));
                                    if (!bilinear)
                                        ACC(g_confidence[o.index[(int)(uint32_t)o.keys[s + j]]], g_iter);
                                    else
                                        galpha[s + j] += o.abs_mode ? std::fabs(g_iter) : g_iter;
                                }
                            }
                            else
                            {
                                float dot = 0;
                                for (int ci = 0; ci < C; ++ci) dot += gin[ci] * col[ci];
                                Ti.push_back(T), ai.push_back(a), doti.push_back(dot);
                            }
                            processed = i + 1;
                            T         = new_T(T, a);
                            if (bilinear && T < 0.001f)
                            {
                                if (fg) cnt = i + 1;
                                break;
                            }
                        }
                        if (!prm.conf_grad_quadratic)
                        {
                            // d alpha_j -= S_j / (1 - alpha_j + eps),  S_j = sum_{i>j} T_i alpha_i (d_i . G)
                            double S = 0;
                            for (int j = processed - 1; j >= 0; --j)
                            {
                                if (j < cnt0)
                                {
                                    double sub = -S / (double)(1 - ai[j] + 1e-9f);
                                    if (!bilinear)
                                        ACC(g_confidence[o.index[(int)(uint32_t)o.keys[s + j]]], sub);
                                    else
                                        galpha[s + j] += (float)(o.abs_mode ? std::fabs(sub) : sub);
                                }
                                S += o.abs_mode ? std::fabs((double)(Ti[j] * ai[j] * doti[j])) : (double)(Ti[j] * ai[j] * doti[j]);
                            }
                        }
                    }

                    // (ii) spatial gradients
                    int dist_edge = std::min(std::min(x, lv.w - 1 - x), std::min(y, lv.h - 1 - y));
                    if (!(dist_edge > 2)) continue;
                    if (!bilinear && !prm.need_point_gradient) continue;
                    for (int i = 0; i < cnt; ++i)
                    {
                        int pid = (int)(uint32_t)o.keys[s + i];
                        int tex = o.index[pid];
                        V2 dR;
                        if (!bilinear)
                        {
                            float dx = 0, dy = 0;
                            for (int ci = 0; ci < C; ++ci)
                            {
                                float Tp = o.texture[(int64_t)ci * n_tex + tex];
                                auto at  = [&](const float* img, int xx, int yy) { return img[ci * hw + (int64_t)yy * lv.w + xx]; };
                                float a0 = -(Tp - at(I, x - 1, y)) * at(G, x - 1, y);
                                float a1 = (Tp - at(I, x + 1, y)) * at(G, x + 1, y);
                                float b0 = -(Tp - at(I, x, y - 1)) * at(G, x, y - 1);
                                float b1 = (Tp - at(I, x, y + 1)) * at(G, x, y + 1);
                                dx += 0.5f * (a0 + a1);
                                dy += 0.5f * (b0 + b1);
                            }
                            dR = {dx / (float)C, dy / (float)C};
                        }
                        else
                        {
                            float w4[4], J[8];
                            blending_fac({o.uv[2 * (s + i)], o.uv[2 * (s + i) + 1]}, w4, J);
                            int bi        = o.corner[s + i];
                            float ga      = galpha[s + i];
                            ACC(g_confidence[tex], w4[bi] * ga);  // RenderBackward.cu:3076-3079
                            if (!prm.need_point_gradient) continue;
                            float single = o.conf[tex] * ga;
                            dR = {J[2 * bi] * single, J[2 * bi + 1] * single};
                        }
                        BackOut bo;
                        if (!project_backward(o.position + 4 * pid, dR, V, K, crop2, cam.rot, prm.dist_cutoff, bo)) continue;
                        if (g_points)
                        {
                            for (int k = 0; k < 3; ++k) ACC(g_points[3 * (int64_t)pid + k], bo.g_point[k]);
                            _Pragma("omp atomic") g_points_count[pid] += 1.0;
                        }
                        if (g_pose)
                        {
                            for (int k = 0; k < 6; ++k) ACCL(t_pose[k], bo.g_pose[k]);
                            t_pose_count += bilinear ? 1.0 : (double)(1.f / 1024.f);
                        }
                        if (g_intr)
                        {
                            bo.g_k[4] *= 0;
                            for (int k = 0; k < 5; ++k) ACCL(t_intr[k], prm.K_gradient_factor * bo.g_k[k]);
                            bo.g_dis[2] *= 0.25f;
                            for (int k = 3; k < 8; ++k) bo.g_dis[k] *= 0.1f;
                            for (int k = 0; k < 8; ++k) ACCL(t_intr[5 + k], prm.distortion_gradient_factor * bo.g_dis[k]);
                            t_intr_count += (double)(1.f / 1024.f);
                        }
                    }
                }
            // (atomic: other threads may still be adding to descriptor 0's confidence gradient from their pixels)
            {
                for (int ci = 0; ci < C; ++ci) _Pragma("omp atomic") g_background[ci] += t_bg[ci];
                _Pragma("omp atomic") g_confidence[0] += t_conf0;
                if (g_pose)
                {
                    for (int k = 0; k < 6; ++k) _Pragma("omp atomic") g_pose[6 * cam.image_index + k] += t_pose[k];
                    _Pragma("omp atomic") g_pose_count[cam.image_index] += t_pose_count;
                }
                if (g_intr)
                {
                    for (int k = 0; k < 13; ++k) _Pragma("omp atomic") g_intr[13 * cam.camera_index + k] += t_intr[k];
                    _Pragma("omp atomic") g_intr_count[cam.camera_index] += t_intr_count;
                }
            }
            }
        }
    }
#undef ACC
#undef ACCL
    return 0;
}

// The blend algebra on its own, for the comparison with the reference's PointBlending.h (compiled separately).
// vo_blend evaluates the colour step without the fused multiply-add (as a CPU build of the reference does) when
// `fused` is 0, and with it (as the CUDA build of the reference and this library do) when `fused` is 1.
float vo_blend(float T, float a, float c, float dst, int fused) { return fused ? blend(T, a, c, dst) : T * a * c + dst; }
float vo_new_T(float T, float a) { return new_T(T, a); }
void vo_blending_fac(float u, float v, float* w4, float* J8) { blending_fac({u, v}, w4, J8); }

// One point through the restated projection and its backward function, for the test that compares the chain of
// transposed Jacobians with automatic differentiation of the same projection in float64.
//   out[0..1] image position at the level, out[2] z; g[0..2] point, g[3..8] pose tangent, g[9..13] K, g[14..21] distortion
int vo_project_with_backward(const float* pos4, const double* pose8, const float* intr13, const OView* view, float level_scale,
                             const float* grad2, float dist_cutoff, float* out, float* g)
{
    const Pose V = load_pose(pose8);
    const Projected pr = project(pos4, V, intr13, *view, dist_cutoff);
    out[0] = pr.ip.x * level_scale, out[1] = pr.ip.y * level_scale, out[2] = pr.z;
    float crop2[5];
    for (int k = 0; k < 5; ++k) crop2[k] = view->crop[k] * level_scale;  // IntrinsicsPinhole::scale
    BackOut bo;
    if (!project_backward(pos4, {grad2[0], grad2[1]}, V, intr13, crop2, view->rot, dist_cutoff, bo)) return 1;
    for (int k = 0; k < 3; ++k) g[k] = bo.g_point[k];
    for (int k = 0; k < 6; ++k) g[3 + k] = bo.g_pose[k];
    for (int k = 0; k < 5; ++k) g[9 + k] = bo.g_k[k];
    for (int k = 0; k < 8; ++k) g[14 + k] = bo.g_dis[k];
    return 0;
}

// Magnitude shadow: with `on`, vo_backward accumulates |addend| instead of addend into every gradient sum (counts
// are unchanged).  The result bounds the rounding noise an fp32 sum of the same addends can carry in any order.
void vo_set_abs_mode(void* h, int on) { ((Oracle*)h)->abs_mode = on != 0; }


// ApplyTangent, PointRenderer.cu:1325-1341: pose <- exp_se3(tangent) * pose, tangent <- 0, in double.
// Tangent = (translation part, rotation part) as Sophus::SE3d::exp consumes it.
void vo_apply_tangent(double* tangent, double* poses, int n)
{
    for (int i = 0; i < n; ++i)
    {
        double* t = tangent + 6 * i;
        double* p = poses + 8 * i;
        double ux = t[0], uy = t[1], uz = t[2], wx = t[3], wy = t[4], wz = t[5];
        double th2 = wx * wx + wy * wy + wz * wz, th = std::sqrt(th2);
        // SO3 exp -> quaternion
        double imag, real;
        if (th < 1e-10)
        {
            double th4 = th2 * th2;
            imag = 0.5 - th2 / 48.0 + th4 / 3840.0;
            real = 1.0 - th2 / 8.0 + th4 / 384.0;
        }
        else
        {
            imag = std::sin(0.5 * th) / th;
            real = std::cos(0.5 * th);
        }
        double qe[4] = {imag * wx, imag * wy, imag * wz, real};
        // V = I + a*Omega + b*Omega^2
        double a, bb;
        if (th < 1e-10)
        {
            a  = 0.5;
            bb = 1.0 / 6.0;
        }
        else
        {
            a  = (1 - std::cos(th)) / th2;
            bb = (th - std::sin(th)) / (th2 * th);
        }
        double O[9]  = {0, -wz, wy, wz, 0, -wx, -wy, wx, 0};
        double O2[9];
        for (int r = 0; r < 3; ++r)
            for (int c = 0; c < 3; ++c) O2[3 * r + c] = O[3 * r] * O[c] + O[3 * r + 1] * O[3 + c] + O[3 * r + 2] * O[6 + c];
        double u[3] = {ux, uy, uz}, te[3];
        for (int r = 0; r < 3; ++r)
        {
            te[r] = u[r];
            for (int c = 0; c < 3; ++c) te[r] += (a * O[3 * r + c] + bb * O2[3 * r + c]) * u[c];
        }
        // compose: q = qe * qp ; t = Re * tp + te
        double x1 = qe[0], y1 = qe[1], z1 = qe[2], w1 = qe[3];
        double x2 = p[0], y2 = p[1], z2 = p[2], w2 = p[3];
        double q[4] = {w1 * x2 + x1 * w2 + y1 * z2 - z1 * y2, w1 * y2 - x1 * z2 + y1 * w2 + z1 * x2,
                       w1 * z2 + x1 * y2 - y1 * x2 + z1 * w2, w1 * w2 - x1 * x2 - y1 * y2 - z1 * z2};
        double nrm = std::sqrt(q[0] * q[0] + q[1] * q[1] + q[2] * q[2] + q[3] * q[3]);
        for (double& v : q) v /= nrm;
        // rotate tp by qe
        double tp[3] = {p[4], p[5], p[6]};
        double cx = y1 * tp[2] - z1 * tp[1], cy = z1 * tp[0] - x1 * tp[2], cz = x1 * tp[1] - y1 * tp[0];
        cx *= 2, cy *= 2, cz *= 2;
        double rx = tp[0] + w1 * cx + (y1 * cz - z1 * cy);
        double ry = tp[1] + w1 * cy + (z1 * cx - x1 * cz);
        double rz = tp[2] + w1 * cz + (x1 * cy - y1 * cx);
        p[0] = q[0], p[1] = q[1], p[2] = q[2], p[3] = q[3];
        p[4] = rx + te[0], p[5] = ry + te[1], p[6] = rz + te[2];
        for (int k = 0; k < 6; ++k) t[k] = 0;
    }
}
// Error-grid rasterisation, FillSceneGridWithLossRasterize (RenderForward.cu:639-791): every cell of the scene grid
// whose eight corners are in front of the camera collects the L1 loss of the pixels its projected box covers (32-pixel
// border excluded): value += sum over channels of |loss|, access count += 1 per pixel.  The reference adds with float
// atomics in no fixed order; here the value of a cell is summed in double (compare with a relative tolerance), the
// count is exact.
static inline float tri_sign(V2 p1, V2 p2, V2 p3) { return (p1.x - p3.x) * (p2.y - p3.y) - (p2.x - p3.x) * (p1.y - p3.y); }
static inline bool point_in_triangle(V2 pt, V2 v1, V2 v2, V2 v3)
{
    float d1 = tri_sign(pt, v1, v2), d2 = tri_sign(pt, v2, v3), d3 = tri_sign(pt, v3, v1);
    bool has_neg = (d1 < 0) || (d2 < 0) || (d3 < 0);
    bool has_pos = (d1 > 0) || (d2 > 0) || (d3 > 0);
    return !(has_neg && has_pos);
}

int vo_grid_loss(const double* poses, const float* intrinsics, const OView* view, float dist_cutoff, int n_cells,
                 const float* bb_min, const float* bb_len, const float* loss_img, int channels, int h, int w,
                 float* cell_value, int* cell_count)
{
    if (!poses || !intrinsics || !view || n_cells < 0 || channels < 1) return -1;
    const Pose V      = load_pose(poses + 8 * (int64_t)view->image_index);
    const float* intr = intrinsics + 13 * (int64_t)view->camera_index;
    static const float fac[8][3]  = {{0, 0, 0}, {1, 0, 0}, {0, 1, 0}, {0, 0, 1}, {1, 1, 0}, {1, 0, 1}, {0, 1, 1}, {1, 1, 1}};
    static const int tris[12][3]  = {{0, 1, 4}, {0, 4, 2}, {1, 5, 7}, {1, 7, 4}, {5, 3, 6}, {5, 6, 7},
                                     {3, 0, 6}, {0, 6, 2}, {3, 0, 5}, {0, 5, 1}, {2, 4, 6}, {4, 6, 7}};
    const float border = 32.f;
#pragma omp parallel for schedule(dynamic, 16)
    for (int c = 0; c < n_cells; ++c)
    {
        V2 pp[8];
        bool behind = false;
        for (int i = 0; i < 8; ++i)
        {
            float pos4[4] = {bb_min[3 * c] + bb_len[3 * c] * fac[i][0], bb_min[3 * c + 1] + bb_len[3 * c + 1] * fac[i][1],
                             bb_min[3 * c + 2] + bb_len[3 * c + 2] * fac[i][2], 0.f};
            Projected pr = project(pos4, V, intr, *view, dist_cutoff);
            if (pr.z <= 0) behind = true;
            pp[i] = pr.ip;
        }
        if (behind) continue;
        V2 mx{-10000000.f, -10000000.f}, mn{10000000.f, 10000000.f};
        for (int i = 0; i < 8; ++i)
        {
            mx.x = std::fmax(pp[i].x, mx.x), mx.y = std::fmax(pp[i].y, mx.y);
            mn.x = std::fmin(pp[i].x, mn.x), mn.y = std::fmin(pp[i].y, mn.y);
        }
        if (mx.x < border || mn.x >= (float)w - border || mx.y < border || mn.y >= (float)h - border) continue;
        mn.x = std::fmax(mn.x, border), mn.y = std::fmax(mn.y, border);
        mx.x = std::fmin(mx.x, (float)w - border), mx.y = std::fmin(mx.y, (float)h - border);
        const int y_size = (int)(mx.y - mn.y), x_size = (int)(mx.x - mn.x);
        double sum = 0.0;
        int hits   = 0;
        for (int64_t xy = 0; xy < (int64_t)y_size * x_size; ++xy)
        {
            const int x_c = (int)((float)(int)(xy % x_size) + mn.x);
            const int y_c = (int)((float)(int)(xy / x_size) + mn.y);
            bool in = false;
            for (int t = 0; t < 12 && !in; ++t)
                in = point_in_triangle({(float)x_c, (float)y_c}, pp[tris[t][0]], pp[tris[t][1]], pp[tris[t][2]]);
            if (!in) continue;
            float g = 0.f;
            for (int i = 0; i < channels; ++i) g += std::fabs(loss_img[((int64_t)i * h + y_c) * w + x_c]);
            sum += (double)g;
            ++hits;
        }
        cell_value[c] += (float)sum;
        cell_count[c] += hits;
    }
    return 0;
}
}  // extern "C"

// ---------------------------------------------------------------------------------------------
// Texture environment map: EnvironmentMapImpl::Sample2 / forward_mps5 (EnvironmentMap.cu:378-485, 692-758).
// The ray of a pixel (BuildSphericalRayList, :201-287, pinhole branch), the sample coordinates on every sphere
// (CreateSampleUVMapAllSpheres, :587-684) and the trilinear fetch of libtorch's grid_sample (bilinear, zero padding,
// align_corners) are restated; tests compare the fetch and the composition with torch's own operators on the CPU.
// saiga's IntrinsicsPinhole::unproject2 and Sophus' SE3::inverse are restated from their published definitions
// (parity unpinned, as for the projection above).

namespace
{
struct EnvRay
{
    V3 o, d;
};

inline V2 k_unproject2(const float* K, V2 ip)  // IntrinsicsPinhole::unproject2: the inverse of normalizedToImage
{
    float y = (ip.y - K[3]) / K[1];
    float x = (ip.x - K[2] - K[4] * y) / K[0];
    return {x, y};
}

inline EnvRay env_ray(const Pose& V, const float* intr, const OView& cam, int lw, int lh, float scale, int gx, int gy)
{
    // inverse crop rotation about the level's centre (integer division), Eigen's 2x2 inverse
    const float det = cam.rot[0] * cam.rot[3] - cam.rot[2] * cam.rot[1];
    const float inv = 1.f / det;
    const float r00 = cam.rot[3] * inv, r01 = -cam.rot[1] * inv, r10 = -cam.rot[2] * inv, r11 = cam.rot[0] * inv;
    const float cx = (float)(lw / 2), cy = (float)(lh / 2);
    float dx = (float)gx - cx, dy = (float)gy - cy;
    V2 ip{r00 * dx + r01 * dy, r10 * dx + r11 * dy};
    ip = {ip.x + cx, ip.y + cy};
    float crop[5];
    for (int k = 0; k < 5; ++k) crop[k] = cam.crop[k] * scale;  // IntrinsicsPinhole::scale
    V2 np = k_unproject2(intr, k_unproject2(crop, ip));          // zero distortion: the undistortion is the identity
    // Sophus SE3::inverse: (q^-1, q^-1 * (-t))
    Pose Vi;
    Vi.q[0] = -V.q[0], Vi.q[1] = -V.q[1], Vi.q[2] = -V.q[2], Vi.q[3] = V.q[3];
    V3 ti = rotate(Vi, {-V.t[0], -V.t[1], -V.t[2]});
    V3 r  = rotate(Vi, {np.x, np.y, 1.f});
    V3 wp{r.x + ti.x, r.y + ti.y, r.z + ti.z};
    V3 d{wp.x - ti.x, wp.y - ti.y, wp.z - ti.z};
    float n2 = d.x * d.x + d.y * d.y + d.z * d.z;
    if (n2 > 0.f)
    {
        float n = std::sqrt(n2);
        d = {d.x / n, d.y / n, d.z / n};
    }
    return {wp, d};
}

struct EnvTap  // one sphere's sample: trilinear base texel and weights, or a miss
{
    bool hit;
    float u, v, z;
    int x0, y0, z0;
    float wx[2], wy[2], wz[2];
};

inline float env_unnormalize(float c, int size) { return ((c + 1.f) / 2.f) * (float)(size - 1); }

inline EnvTap env_tap(const EnvRay& ray, float q2a, float qb, float f, int s, int S, int R, const float* radii, int up_axis)
{
    EnvTap t;
    std::memset(&t, 0, sizeof(t));
    V3 sv = ray.d;
    t.hit = true;
    if (s != S - 1)
    {
        const float r   = radii[s];
        const float det = f + 2.f * q2a * (r * r);
        t.hit           = det >= 0.f;
        if (!t.hit) return t;
        const float res = (-qb + std::sqrt(det)) / q2a;
        V3 p{ray.o.x + res * ray.d.x, ray.o.y + res * ray.d.y, ray.o.z + res * ray.d.z};
        const float len = std::sqrt(p.x * p.x + p.y * p.y + p.z * p.z);
        sv = {p.x / len, p.y / len, p.z / len};
    }
    const float pi = 3.14159265358979323846f;
    float a, b, c;  // lat = asin(a), lon = atan2(b, c)
    if (up_axis == 0) a = sv.x, b = sv.y, c = sv.z;
    else if (up_axis == 1) a = sv.y, b = sv.x, c = sv.z;
    else a = sv.z, b = sv.x, c = sv.y;
    a = std::fmin(std::fmax(a, -1.f), 1.f);  // a unit vector's component may round to 1 + 1 ulp
    const float lat = std::asin(a), lon = std::atan2(b, c);
    t.u = 2.f * (lon / 2.f / pi);
    t.v = 2.f * (lat / pi);
    t.z = S == 1 ? 0.f : (float)s / (float)(S - 1) * 2.f - 1.f;
    const float ix = env_unnormalize(t.u, R), iy = env_unnormalize(t.v, R), iz = env_unnormalize(t.z, S);
    const float fx = std::floor(ix), fy = std::floor(iy), fz = std::floor(iz);
    // kept inside [-2, size]: defined int conversion for every float; out there everything reads zero either way
    t.x0 = (int)std::fmin(std::fmax(fx, -2.f), (float)R), t.y0 = (int)std::fmin(std::fmax(fy, -2.f), (float)R);
    t.z0 = (int)std::fmin(std::fmax(fz, -2.f), (float)S);
    t.wx[1] = ix - fx, t.wx[0] = (fx + 1.f) - ix;
    t.wy[1] = iy - fy, t.wy[0] = (fy + 1.f) - iy;
    t.wz[1] = iz - fz, t.wz[0] = (fz + 1.f) - iz;
    return t;
}

// grid_sample's trilinear fetch of one plane: corners in the order z, y, x; out-of-range corners read zero
inline float env_fetch(const float* plane /*[S,R,R]*/, const EnvTap& t, int S, int R)
{
    float acc = 0.f;
    for (int k = 0; k < 2; ++k)
        for (int j = 0; j < 2; ++j)
            for (int i = 0; i < 2; ++i)
            {
                const int x = t.x0 + i, y = t.y0 + j, z = t.z0 + k;
                if (x < 0 || x >= R || y < 0 || y >= R || z < 0 || z >= S) continue;
                const float w = t.wx[i] * t.wy[j] * t.wz[k];
                acc += plane[((int64_t)z * R + y) * R + x] * w;
            }
    return acc;
}

struct EnvPixel
{
    EnvTap tap[8];
    float alpha[8];    // hit * sigmoid(density), 1 on the last sphere
    float sig[8];      // sigmoid(density)
    float col[8][4];   // sampled colour (|.| when non_subzero)
    float raw[8][4];   // before the abs
    float T[9];        // transmittance in front of sphere s
};

constexpr int kEnvAdd = 1, kEnvNotAtPoints = 2, kEnvDepthTestWeight = 4;

inline void env_pixel(const Pose& V, const float* intr, const OView& cam, int lw, int lh, float scale, int gx, int gy,
                      const float* density, const float* color, const float* radii, int S, int R, int C, int up_axis,
                      int non_subzero, float T0, EnvPixel& px)
{
    const EnvRay ray = env_ray(V, intr, cam, lw, lh, scale, gx, gy);
    const float q2a = 2.f * (ray.d.x * ray.d.x) + 2.f * (ray.d.y * ray.d.y) + 2.f * (ray.d.z * ray.d.z);
    const float qb  = 2.f * (ray.o.x * ray.d.x) + 2.f * (ray.o.y * ray.d.y) + 2.f * (ray.o.z * ray.d.z);
    const float f   = qb * qb - 2.f * q2a * (ray.o.x * ray.o.x + ray.o.y * ray.o.y + ray.o.z * ray.o.z);
    px.T[0] = T0;
    for (int s = 0; s < S; ++s)
    {
        px.tap[s] = env_tap(ray, q2a, qb, f, s, S, R, radii, up_axis);
        const EnvTap& t = px.tap[s];
        px.sig[s] = 0.f, px.alpha[s] = 0.f;
        for (int c = 0; c < 4; ++c) px.col[s][c] = px.raw[s][c] = 0.f;
        if (t.hit)
        {
            if (s == S - 1)
                px.alpha[s] = 1.f;
            else
            {
                const float dv = env_fetch(density, t, S, R);
                px.sig[s]      = 1.f / (1.f + std::exp(-dv));
                px.alpha[s]    = px.sig[s];
            }
            for (int c = 0; c < C; ++c)
            {
                px.raw[s][c] = env_fetch(color + (int64_t)c * S * R * R, t, S, R);
                px.col[s][c] = non_subzero ? std::fabs(px.raw[s][c]) : px.raw[s][c];
            }
        }
        px.T[s + 1] = (1.f - px.alpha[s]) * px.T[s];
    }
}

inline float env_start_T(float weight, int flags) { return (flags & kEnvDepthTestWeight) ? (weight > 0.5f ? 0.f : 1.f) : weight; }
}  // namespace

extern "C" {
int vo_envmap_forward(const double* poses, const float* intrinsics, const OView* views, int n_views, int L,
                      const float* density, const float* color, const float* radii, int S, int R, int C, int up_axis,
                      int non_subzero, const float* const* weight, float* const* out, int flags)
{
    if (!poses || !intrinsics || !views || n_views < 1 || L < 1 || L > kMaxLayers || S < 1 || S > 8 || C < 1 || C > 4 || R < 1)
        return -1;
    int lw = views[0].w, lh = views[0].h;
    float scale = 1.f;
    for (int l = 0; l < L; ++l, lw /= 2, lh /= 2, scale *= 0.5f)
        for (int b = 0; b < n_views; ++b)
        {
            const Pose V      = load_pose(poses + 8 * (int64_t)views[b].image_index);
            const float* intr = intrinsics + 13 * (int64_t)views[b].camera_index;
#pragma omp parallel for schedule(static)
            for (int y = 0; y < lh; ++y)
                for (int x = 0; x < lw; ++x)
                {
                    const int64_t pix = ((int64_t)b * lh + y) * lw + x;
                    const float wgt   = weight[l][pix];
                    EnvPixel px;
                    env_pixel(V, intr, views[b], lw, lh, scale, x, y, density, color, radii, S, R, C, up_axis, non_subzero,
                              env_start_T(wgt, flags), px);
                    const bool masked = (flags & kEnvNotAtPoints) && wgt > 0.001f;
                    for (int c = 0; c < C; ++c)
                    {
                        float acc = 0.f;
                        for (int s = 0; s < S; ++s) acc = px.T[s] * px.alpha[s] * px.col[s][c] + acc;
                        if (masked) acc = 0.f;
                        float& o = out[l][(((int64_t)b * C + c) * lh + y) * lw + x];
                        if (flags & kEnvAdd)
                        {
                            float base = o;
                            if ((flags & kEnvDepthTestWeight) && !(wgt > 0.5f)) base = 0.f;
                            o = base + acc;
                        }
                        else
                            o = acc;
                    }
                }
        }
    return 0;
}

// Sample coordinates of one view and level, for the tests that run libtorch's own grid_sample on them:
// uvz [S, h_l*w_l, 3], hit [S, h_l*w_l].
int vo_envmap_uvz(const double* poses, const float* intrinsics, const OView* view, int level, const float* radii, int S,
                  int R, int up_axis, float* uvz, float* hit)
{
    int lw = view->w, lh = view->h;
    float scale = 1.f;
    for (int l = 0; l < level; ++l) lw /= 2, lh /= 2, scale *= 0.5f;
    const Pose V      = load_pose(poses + 8 * (int64_t)view->image_index);
    const float* intr = intrinsics + 13 * (int64_t)view->camera_index;
    for (int y = 0; y < lh; ++y)
        for (int x = 0; x < lw; ++x)
        {
            const EnvRay ray = env_ray(V, intr, *view, lw, lh, scale, x, y);
            const float q2a = 2.f * (ray.d.x * ray.d.x) + 2.f * (ray.d.y * ray.d.y) + 2.f * (ray.d.z * ray.d.z);
            const float qb  = 2.f * (ray.o.x * ray.d.x) + 2.f * (ray.o.y * ray.d.y) + 2.f * (ray.o.z * ray.d.z);
            const float f   = qb * qb - 2.f * q2a * (ray.o.x * ray.o.x + ray.o.y * ray.o.y + ray.o.z * ray.o.z);
            for (int s = 0; s < S; ++s)
            {
                const EnvTap t  = env_tap(ray, q2a, qb, f, s, S, R, radii, up_axis);
                const int64_t i = (int64_t)s * lw * lh + (int64_t)y * lw + x;
                uvz[3 * i] = t.u, uvz[3 * i + 1] = t.v, uvz[3 * i + 2] = t.z;
                hit[i] = t.hit ? 1.f : 0.f;
            }
        }
    return 0;
}

// World-space rays of one view and level (BuildSphericalRayList): origin, direction [h_l*w_l, 3].  For the test that
// ties the ray construction to the rasterizer's projection: a point on the ray of a pixel must be drawn into that pixel.
int vo_envmap_rays(const double* poses, const float* intrinsics, const OView* view, int level, float* origin, float* direction)
{
    int lw = view->w, lh = view->h;
    float scale = 1.f;
    for (int l = 0; l < level; ++l) lw /= 2, lh /= 2, scale *= 0.5f;
    const Pose V      = load_pose(poses + 8 * (int64_t)view->image_index);
    const float* intr = intrinsics + 13 * (int64_t)view->camera_index;
    for (int y = 0; y < lh; ++y)
        for (int x = 0; x < lw; ++x)
        {
            const EnvRay ray = env_ray(V, intr, *view, lw, lh, scale, x, y);
            const int64_t i  = (int64_t)y * lw + x;
            origin[3 * i] = ray.o.x, origin[3 * i + 1] = ray.o.y, origin[3 * i + 2] = ray.o.z;
            direction[3 * i] = ray.d.x, direction[3 * i + 1] = ray.d.y, direction[3 * i + 2] = ray.d.z;
        }
    return 0;
}

// Gradients of density [S,R,R] and color [C,S,R,R], added to g_density / g_color; sums are formed in double.
// mag_density / mag_color (optional): the sums of the absolute addends, for the tests' tolerance.
int vo_envmap_backward(const double* poses, const float* intrinsics, const OView* views, int n_views, int L,
                       const float* density, const float* color, const float* radii, int S, int R, int C, int up_axis,
                       int non_subzero, const float* const* weight, const float* const* grad_out, int flags,
                       float* g_density, float* g_color, float* mag_density, float* mag_color)
{
    if (!poses || !intrinsics || !views || n_views < 1 || L < 1 || L > kMaxLayers || S < 1 || S > 8 || C < 1 || C > 4 || R < 1)
        return -1;
    const int64_t plane = (int64_t)S * R * R;
    std::vector<double> gd(plane, 0.0), gc(plane * C, 0.0), md(plane, 0.0), mc(plane * C, 0.0);
    int lw = views[0].w, lh = views[0].h;
    float scale = 1.f;
    for (int l = 0; l < L; ++l, lw /= 2, lh /= 2, scale *= 0.5f)
        for (int b = 0; b < n_views; ++b)
        {
            const Pose V      = load_pose(poses + 8 * (int64_t)views[b].image_index);
            const float* intr = intrinsics + 13 * (int64_t)views[b].camera_index;
            for (int y = 0; y < lh; ++y)
                for (int x = 0; x < lw; ++x)
                {
                    const int64_t pix = ((int64_t)b * lh + y) * lw + x;
                    const float wgt   = weight[l][pix];
                    if ((flags & kEnvNotAtPoints) && wgt > 0.001f) continue;
                    EnvPixel px;
                    env_pixel(V, intr, views[b], lw, lh, scale, x, y, density, color, radii, S, R, C, up_axis, non_subzero,
                              env_start_T(wgt, flags), px);
                    float G[4] = {0, 0, 0, 0};
                    for (int c = 0; c < C; ++c) G[c] = grad_out[l][(((int64_t)b * C + c) * lh + y) * lw + x];
                    // rest[s] = d(sum of the spheres behind s, per unit of transmittance behind s) . G
                    float rest = 0.f;
                    for (int s = S - 1; s >= 0; --s)
                    {
                        float dot = 0.f;
                        for (int c = 0; c < C; ++c) dot += px.col[s][c] * G[c];
                        const float g_alpha = px.T[s] * (dot - rest);
                        rest                = px.alpha[s] * dot + (1.f - px.alpha[s]) * rest;
                        const EnvTap& t     = px.tap[s];
                        if (!t.hit) continue;
                        const float g_dens = s == S - 1 ? 0.f : g_alpha * (px.sig[s] * (1.f - px.sig[s]));
                        float g_col[4];
                        for (int c = 0; c < C; ++c)
                        {
                            g_col[c] = px.T[s] * px.alpha[s] * G[c];
                            if (non_subzero) g_col[c] = px.raw[s][c] > 0.f ? g_col[c] : (px.raw[s][c] < 0.f ? -g_col[c] : 0.f);
                        }
                        for (int k = 0; k < 2; ++k)
                            for (int j = 0; j < 2; ++j)
                                for (int i = 0; i < 2; ++i)
                                {
                                    const int tx = t.x0 + i, ty = t.y0 + j, tz = t.z0 + k;
                                    if (tx < 0 || tx >= R || ty < 0 || ty >= R || tz < 0 || tz >= S) continue;
                                    const float w   = t.wx[i] * t.wy[j] * t.wz[k];
                                    const int64_t a = ((int64_t)tz * R + ty) * R + tx;
                                    gd[a] += (double)(w * g_dens);
                                    md[a] += std::fabs((double)(w * g_dens));
                                    for (int c = 0; c < C; ++c)
                                    {
                                        gc[c * plane + a] += (double)(w * g_col[c]);
                                        mc[c * plane + a] += std::fabs((double)(w * g_col[c]));
                                    }
                                }
                    }
                }
        }
    for (int64_t i = 0; i < plane; ++i) g_density[i] += (float)gd[i];
    for (int64_t i = 0; i < plane * C; ++i) g_color[i] += (float)gc[i];
    if (mag_density)
        for (int64_t i = 0; i < plane; ++i) mag_density[i] = (float)md[i];
    if (mag_color)
        for (int64_t i = 0; i < plane * C; ++i) mag_color[i] = (float)mc[i];
    return 0;
}
}  // extern "C"

// ---------------------------------------------------------------------------------------------
// SceneData::ComputeRadius (data/SceneData.cpp:554-597): data[i](0) = the distance from point i to the last of its
// n + 1 nearest points, itself included (a KD-tree query in the reference; here every pair is visited).  The value
// is the (n + 1)-th smallest of the distances |p_i - p_j| over all j, which does not depend on how ties are
// ordered.  With fewer than n + 1 points it is the distance to the farthest one.
extern "C" int vo_knn_radius(const float* position, int stride, int n_points, int k, float* radius)
{
    if (!position || !radius || n_points < 0 || k < 1 || stride < 3) return -1;
#pragma omp parallel
    {
        std::vector<float> d2((size_t)n_points);
#pragma omp for schedule(static)
        for (int i = 0; i < n_points; ++i)
        {
            const float* a = position + (int64_t)i * stride;
            for (int j = 0; j < n_points; ++j)
            {
                const float* b = position + (int64_t)j * stride;
                const float dx = a[0] - b[0], dy = a[1] - b[1], dz = a[2] - b[2];
                d2[j] = dx * dx + dy * dy + dz * dz;
            }
            const int kth = std::min(k, n_points - 1);
            std::nth_element(d2.begin(), d2.begin() + kth, d2.end());
            radius[i] = std::sqrt(d2[kth]);
        }
    }
    return 0;
}

// The same query with a uniform grid instead of all pairs (what a host implementation would do, as the reference's
// KD-tree does, in O(n) cells): bit-equal to vo_knn_radius, and fast enough to be timed on the benchmark cloud as
// the CPU baseline of this row.  Cell size: halved from 1/32 of the longest extent until an occupied cell holds at
// most 8 points on average; rings of cells around the point's cell until the k-th nearest distance found is smaller
// than the distance to the faces of the visited cube.
extern "C" int vo_knn_radius_grid(const float* position, int stride, int n_points, int k, float* radius)
{
    if (!position || !radius || n_points < 0 || k < 1 || stride < 3) return -1;
    const int n = n_points;
    if (n == 0) return 0;
    float lo[3] = {INFINITY, INFINITY, INFINITY}, hi[3] = {-INFINITY, -INFINITY, -INFINITY};
    for (int i = 0; i < n; ++i)
        for (int a = 0; a < 3; ++a)
        {
            const float v = position[(int64_t)i * stride + a];
            if (!std::isfinite(v)) return -1;
            lo[a] = std::min(lo[a], v), hi[a] = std::max(hi[a], v);
        }
    float ext = 0.f, maxabs = 0.f;
    for (int a = 0; a < 3; ++a)
    {
        ext    = std::max(ext, hi[a] - lo[a]);
        maxabs = std::max(maxabs, std::max(std::fabs(lo[a]), std::fabs(hi[a])));
    }
    float cell = ext > 0.f ? ext / 32.f : 1.f;
    int d[3];
    std::vector<int> cell_of((size_t)n), start;
    auto dims_for = [&](float c, int* dd)
    {
        int64_t cells = 1;
        for (int a = 0; a < 3; ++a)
        {
            dd[a] = (int)std::min(std::floor((double)(hi[a] - lo[a]) / c) + 1.0, 1.0e9);
            cells = cells > ((int64_t)1 << 40) ? cells : cells * dd[a];
        }
        return cells;
    };
    auto coord = [&](float p, int a, float inv) { return (int)std::fmin(std::fmax(std::floor((p - lo[a]) * inv), 0.f), (float)(d[a] - 1)); };
    int64_t cells = dims_for(cell, d);
    for (int iter = 0; iter < 24; ++iter)
    {
        const float inv = 1.f / cell;
        start.assign((size_t)cells + 1, 0);
        for (int i = 0; i < n; ++i)
        {
            const float* p = position + (int64_t)i * stride;
            cell_of[i]     = (coord(p[2], 2, inv) * d[1] + coord(p[1], 1, inv)) * d[0] + coord(p[0], 0, inv);
            ++start[(size_t)cell_of[i] + 1];
        }
        int64_t occupied = 0;
        for (int64_t c = 0; c < cells; ++c) occupied += start[(size_t)c + 1] > 0;
        int d2[3];
        if (ext <= 0.f || (double)n / (double)occupied <= 8.0 || dims_for(cell * 0.5f, d2) > ((int64_t)1 << 26)) break;
        cell *= 0.5f;
        cells = dims_for(cell, d);
    }
    for (int64_t c = 0; c < cells; ++c) start[(size_t)c + 1] += start[(size_t)c];
    std::vector<int> cursor(start.begin(), start.end() - 1), order((size_t)n);
    for (int i = 0; i < n; ++i) order[(size_t)cursor[(size_t)cell_of[i]]++] = i;
    const float inv = 1.f / cell, slack = 1e-3f * cell + 4e-6f * (maxabs + ext);
    const int k1 = std::min(k, n - 1) + 1;
#pragma omp parallel for schedule(dynamic, 1024)
    for (int s = 0; s < n; ++s)
    {
        const int i    = order[(size_t)s];
        const float* p = position + (int64_t)i * stride;
        const int c[3] = {coord(p[0], 0, inv), coord(p[1], 1, inv), coord(p[2], 2, inv)};
        std::vector<float> best((size_t)k1, INFINITY);  // ascending
        const int r_max = std::max(std::max(std::max(c[0], d[0] - 1 - c[0]), std::max(c[1], d[1] - 1 - c[1])), std::max(c[2], d[2] - 1 - c[2]));
        for (int r = 0;; ++r)
        {
            for (int z = std::max(c[2] - r, 0); z <= std::min(c[2] + r, d[2] - 1); ++z)
                for (int y = std::max(c[1] - r, 0); y <= std::min(c[1] + r, d[1] - 1); ++y)
                {
                    const bool face = std::abs(z - c[2]) == r || std::abs(y - c[1]) == r;
                    auto visit = [&](int x)
                    {
                        const int64_t ci = ((int64_t)z * d[1] + y) * d[0] + x;
                        for (int j = start[(size_t)ci]; j < start[(size_t)ci + 1]; ++j)
                        {
                            const float* q = position + (int64_t)order[(size_t)j] * stride;
                            const float dx = p[0] - q[0], dy = p[1] - q[1], dz = p[2] - q[2];
                            const float dd = dx * dx + dy * dy + dz * dz;
                            if (dd < best[(size_t)k1 - 1])
                            {
                                int at = k1 - 1;
                                while (at > 0 && best[(size_t)at - 1] > dd) best[(size_t)at] = best[(size_t)at - 1], --at;
                                best[(size_t)at] = dd;
                            }
                        }
                    };
                    if (face)  // a row on the shell's y or z face: all its cells
                        for (int x = std::max(c[0] - r, 0); x <= std::min(c[0] + r, d[0] - 1); ++x) visit(x);
                    else  // an inner row: its two end cells
                    {
                        if (c[0] - r >= 0) visit(c[0] - r);
                        if (c[0] + r < d[0]) visit(c[0] + r);
                    }
                }
            float m = INFINITY;
            for (int a = 0; a < 3; ++a)
            {
                if (c[a] - r > 0) m = std::min(m, p[a] - (lo[a] + (float)(c[a] - r) * cell));
                if (c[a] + r < d[a] - 1) m = std::min(m, (lo[a] + (float)(c[a] + r + 1) * cell) - p[a]);
            }
            m -= slack;
            if (r >= r_max || (m > 0.f && best[(size_t)k1 - 1] <= m * m)) break;
        }
        radius[i] = std::sqrt(best[(size_t)k1 - 1]);
    }
    return 0;
}

