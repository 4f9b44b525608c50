// B200 (sm_100a) kernels and C ABI of the blending point rasterizer.  See include/vetr.h for the interface and the
// reference functions each entry point replaces.
//
// Data layout in HBM
//   pixel space : all views and all pyramid levels of a call form ONE array of PT = n_views * P pixels
//                 (view-major, then level, then bands of VETR_PIXEL_BAND rows, column by column inside a band; see
//                 pixel_offset).  counts[PT], ends[PT] (int32).
//   records     : one 32-byte record per fragment = one DRAM sector: 64-bit key (depth bits << 32 | point index),
//                 alpha, descriptor index, descriptor.  The list of pixel g is recs[ends[g] - counts[g] .. ends[g]).
//                 Lists of consecutive pixels are contiguous, so a CTA that owns a run of pixels streams its fragments
//                 with coalesced loads.
//   work items  : the pixel space is cut into runs of ~kQuantum units of work (1 per fragment, kPixelWork per pixel)
//                 by the scan itself (item_start[]), so the persistent item kernels are balanced by fragments, not
//                 by pixels, and no host round trip is needed to size anything.
//   backward    : level_mask[n_views * n] (which levels hold a fragment of a point), point_grad[(view, level, point)]
//                 (image-space gradient parked per fragment), img4 / grad4[PT] (channel-interleaved image copies).
//
// Kernels (nothing here is a contraction, so no tensor cores)
//   project_kernel<count>    stream positions, strict-fp32 projection, per-level pixel, one reduction per fragment
//   scan_*                   three-phase exclusive scan of counts -> ends, total F, longest list, work-item table
//   project_kernel<collect>  re-project, reserve all slots of a thread's points, then store the 32-byte records
//   sort_blend_kernel        per work item: stage records in shared memory, rank-sort each list by (depth, index),
//                            write the sorted records back, blend front to back, write all outputs (+ _long variant)
//   pack_images_kernel       channel-interleaved copies of the forward image and its gradient
//   backward_kernel          per work item: stream sorted records, image-space gradient of each fragment (parked for
//                            the per-point pass), O(n) transmittance / suffix sweeps per pixel, vector reductions of
//                            descriptor / confidence gradients (+ _long variants; mode 3 forms its spatial gradient here)
//   point_backward_kernel    modes 1, 2: one thread per point over all views: projection Jacobians per fragment,
//                            position gradient written once, camera gradients reduced per CTA and view
//   fuzzy_dt_*               mode 0 (no lists): depth pre-pass, splat, combine, per-point backward
//   exchange_finalize_kernel multi-GPU: sum over ranks + epilogue over NVLink peer memory (plain or multicast)
//   grid_loss_kernel         error-grid rasterisation (one warp per grid cell)
//   transpose / normalize / apply_tangent   small epilogues
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <new>
#include <vector>

#include "../../include/vetr.h"
#include "vetr_math.cuh"

namespace vetr
{
#ifndef VETR_ITEM_THREADS
#    define VETR_ITEM_THREADS 128
#endif
#ifndef VETR_QUANTUM
#    define VETR_QUANTUM 512
#endif
#ifndef VETR_LONG_LIST
#    define VETR_LONG_LIST 256
#endif
#ifndef VETR_MIN_CTAS
#    define VETR_MIN_CTAS 10
#endif
constexpr int kThreads    = VETR_ITEM_THREADS;  // CTA size of the item kernels
constexpr int kQuantum    = VETR_QUANTUM;       // units of work per item
#ifndef VETR_PIXEL_WORK
#    define VETR_PIXEL_WORK 4
#endif
constexpr int kPixelWork  = VETR_PIXEL_WORK;     // work units charged per pixel -> at most kQuantum / kPixelWork pixels per item
constexpr int kMaxPixels  = kQuantum / kPixelWork;
constexpr int kLongList   = VETR_LONG_LIST;         // lists longer than this take the slow path
constexpr int kCap        = kQuantum + kLongList;   // fragments staged per item (an item holds < kQuantum + its first list)
constexpr int kMinCtas    = VETR_MIN_CTAS;          // resident CTAs per SM the item kernels are compiled for
constexpr int kProjThreads     = 256;
#ifndef VETR_COLLECT_POINTS
#    define VETR_COLLECT_POINTS 2
#endif
constexpr int kPointsPerThread = 4;                      // count pass
constexpr int kCollectPoints   = VETR_COLLECT_POINTS;    // collection pass (its slots and payload live in registers)
static_assert(kQuantum % kPixelWork == 0, "an item of kQuantum work units holds at most kQuantum / kPixelWork pixels");
static_assert(kMaxPixels <= kThreads, "one thread per pixel of an item");
static_assert(kMaxPixels <= 256, "seg_of is a byte");
constexpr int kScanTile   = 4096;  // elements per CTA in the scan (256 threads x 16)
constexpr float kMaxDepth = 100000.f;  // MAX_DEPTH_CONST, RenderConstants.h:30

struct ViewDev
{
    int image_index, camera_index;
    float crop[5];
    float rot[4];
};

struct Frame  // kernel parameter block (travels by value; no global or __constant__ state)
{
    int n_views, L, C, n, n_tex, w, h;
    int mode, drop_by_radius, use_env, viewer_only, dbg_max_len, need_point_grad, bg_alpha_to_point0, keep_sorted;
    float radius_threshold, dist_cutoff, stability_cutoff, k_grad_factor, dist_grad_factor, mask_value, accept_blend;
    float depth_accept;
    int ghost;
    int lw[VETR_MAX_LAYERS], lh[VETR_MAX_LAYERS];
    float inv_lw[VETR_MAX_LAYERS], inv_band[VETR_MAX_LAYERS];  // 1 / w and 1 / (kBand w) of a level
    long long lbase[VETR_MAX_LAYERS];  // first pixel of a level in the pixel space of one view (banded order, see pixel_offset)
    long long rbase[VETR_MAX_LAYERS];  // the same in plain row-major order (the interleaved image copies)
    long long P, PT;                   // pixels of one view / of all views in the pixel space (levels padded to whole bands)
    long long Prm;                     // row-major pixels of one view (sum of w * h)
    ViewDev views[VETR_MAX_VIEWS];
    const float4* position;
    const int* index;
    const float* texture;
    const float* confidence;
    const float* background;
    const double* poses;
    const float* intr;
    const float* dropout;
    int* counts;
    int* ends;
    uint4* recs;  // 32-byte fragment records: [2i] = {point index, depth bits, alpha bits, descriptor index}, [2i+1] = descriptor
    long long capacity;
    int* status;      // {F, overflow, longest, number of work items}
    int* item_start;  // [n_items + 1]
    unsigned char* level_mask;  // [n_views * n]: levels of the view on which the point has a fragment (written by collect)
    float2* point_grad;         // [(view * L + level) * n + point]: image-space gradient of that fragment (backward scratch)
    float4* img4;               // [PT] forward image, channels interleaved, indexed like counts[] (backward scratch)
    float4* grad4;              // [PT] its incoming gradient
};

// Order of the pixels of a level in the pixel space: bands of kBand = 4 rows, column by column inside a band,
//     offset(x, y) = (y / 4) * 4 w + 4 x + y % 4,
// so that 4-row x k-column patches of the image are contiguous.  Points arrive in Morton order: the
// fragments of neighbouring points then land in a few nearby runs of the fragment buffer instead of one run per image
// row, and a work item (a run of consecutive pixels) covers a compact patch.  The last band of a level is padded to
// full height; padded pixels have no fragments and are skipped wherever pixels are visited.
constexpr int kBand = VETR_PIXEL_BAND;  // rows per band (a power of two); 4 measured best among 1, 2, 4, 8, 16
constexpr int kBandShift = kBand == 1 ? 0 : kBand == 2 ? 1 : kBand == 4 ? 2 : kBand == 8 ? 3 : 4;
static_assert((1 << kBandShift) == kBand, "VETR_PIXEL_BAND must be 1, 2, 4, 8 or 16");
__device__ __forceinline__ int pixel_offset(int w, int x, int y) { return (y >> kBandShift) * (w << kBandShift) + (x << kBandShift) + (y & (kBand - 1)); }

// Mode 3 keeps the bilinear corner of a fragment in the two top bits of the record's descriptor index.
constexpr int kCornerShift = 30;
constexpr int kTexMask     = (1 << kCornerShift) - 1;

// One fragment record = one 32-byte sector.
__device__ __forceinline__ void store_record(const Frame& f, int slot, unsigned long long key, float alpha, int tex, float4 d)
{
    f.recs[2 * (size_t)slot]     = make_uint4((unsigned)key, (unsigned)(key >> 32), __float_as_uint(alpha), (unsigned)tex);
    f.recs[2 * (size_t)slot + 1] = make_uint4(__float_as_uint(d.x), __float_as_uint(d.y), __float_as_uint(d.z), __float_as_uint(d.w));
}
__device__ __forceinline__ unsigned long long record_key(uint4 h) { return ((unsigned long long)h.y << 32) | h.x; }
__device__ __forceinline__ float4 as_float4(uint4 v)
{
    return make_float4(__uint_as_float(v.x), __uint_as_float(v.y), __uint_as_float(v.z), __uint_as_float(v.w));
}

__device__ __forceinline__ Camera load_camera(const Frame& f, int b)
{
    Camera c;
    const ViewDev& v = f.views[b];
    const double* p  = f.poses + 8 * (long long)v.image_index;
    c.V.qx = (float)p[0], c.V.qy = (float)p[1], c.V.qz = (float)p[2], c.V.qw = (float)p[3];
    c.V.tx = (float)p[4], c.V.ty = (float)p[5], c.V.tz = (float)p[6];
    const float* k = f.intr + 13 * (long long)v.camera_index;
#pragma unroll
    for (int i = 0; i < 5; ++i) c.K[i] = k[i];
    bool hd = false;
#pragma unroll
    for (int i = 0; i < 8; ++i)
    {
        c.dist[i] = k[5 + i];
        hd |= c.dist[i] != 0.f;
    }
    c.has_dist = hd;
#pragma unroll
    for (int i = 0; i < 5; ++i) c.crop[i] = v.crop[i];
#pragma unroll
    for (int i = 0; i < 4; ++i) c.rot[i] = v.rot[i];
    c.cx = (float)(f.w / 2);
    c.cy = (float)(f.h / 2);
    rotation_matrix(c.V, c.R);
    return c;
}

// ---------------------------------------------------------------------------------------------------------
// Pass 1 and 3: projection + counting / collection.  kPts points per thread.  Modes 1 and 2 run in three sweeps over
// the thread's points so that independent memory operations are in flight together: (1) project and find the pixel of
// every (point, level), (2) issue ALL count reductions / slot reservations, (3) load the payload and store the records.
// (The slot reservation is an atomic with a return value: with one in flight per thread the kernel waits on it.)

__device__ __forceinline__ bool point_is_live(const Frame& f, int b, int pid)
{
    if (f.dropout && f.dropout[(size_t)b * f.n + pid] == 1.f) return false;
    if (f.viewer_only && f.confidence[f.index[pid]] < f.stability_cutoff) return false;
    return true;
}

template <bool kCollect, int kPts>
__global__ void __launch_bounds__(kProjThreads) project_kernel(const __grid_constant__ Frame f)
{
    __shared__ Camera s_cam;
    const int b = blockIdx.y;
    if (threadIdx.x == 0) s_cam = load_camera(f, b);
    __syncthreads();
    const Camera& cam   = s_cam;
    const int vbase     = b * (int)f.P;
    const bool bilinear = f.mode == VETR_MODE_BILINEAR_BLEND;
    const int first     = blockIdx.x * (kProjThreads * kPts) + threadIdx.x;

    float4 pos[kPts];
#pragma unroll
    for (int it = 0; it < kPts; ++it)
    {
        const int pid = first + it * kProjThreads;
        pos[it]       = pid < f.n ? __ldg(f.position + pid) : make_float4(0.f, 0.f, 0.f, 0.f);
    }

    if (!bilinear)
    {
        int g[kPts][VETR_MAX_LAYERS];  // pixel of (point, level) in the global pixel space, then its record slot; -1 = none
        unsigned zbits[kPts];
#pragma unroll
        for (int it = 0; it < kPts; ++it)
        {
            const int pid = first + it * kProjThreads;
#pragma unroll
            for (int l = 0; l < VETR_MAX_LAYERS; ++l) g[it][l] = -1;
            zbits[it] = 0;
            if (pid >= f.n || !point_is_live(f, b, pid)) continue;
            const Projected pr = project_point(pos[it], cam, f.dist_cutoff);
            if (pr.z == 0.f) continue;
            zbits[it]    = __float_as_uint(pr.z);
            float2 ip    = pr.ip;
            float radius = pr.radius_px;
            bool alive   = true;
#pragma unroll
            for (int l = 0; l < VETR_MAX_LAYERS; ++l)
            {
                if (l >= f.L || (f.drop_by_radius && radius < f.radius_threshold)) alive = false;
                if (alive)
                {
                    const int lw = f.lw[l], lh = f.lh[l];
                    const int x = round_half_even(ip.x), y = round_half_even(ip.y);
                    if ((unsigned)x < (unsigned)lw && (unsigned)y < (unsigned)lh) g[it][l] = vbase + (int)f.lbase[l] + pixel_offset(lw, x, y);
                }
                radius *= 0.5f, ip.x *= 0.5f, ip.y *= 0.5f;
            }
        }
        if constexpr (!kCollect)
        {
#pragma unroll
            for (int it = 0; it < kPts; ++it)
#pragma unroll
                for (int l = 0; l < VETR_MAX_LAYERS; ++l)
                    if (g[it][l] >= 0) atomicAdd(f.counts + g[it][l], 1);
            return;
        }
        else
        {
#pragma unroll
            for (int it = 0; it < kPts; ++it)
#pragma unroll
                for (int l = 0; l < VETR_MAX_LAYERS; ++l)
                    if (g[it][l] >= 0) g[it][l] = atomicAdd(f.ends + g[it][l], 1);
        // what the blend needs of the point travels next to every key (coalesced loads here, one per point, instead of
        // a dependent gather per fragment later)
#pragma unroll
        for (int it = 0; it < kPts; ++it)
        {
            const int pid = first + it * kProjThreads;
            if (pid >= f.n) break;
            unsigned bits = 0;
#pragma unroll
            for (int l = 0; l < VETR_MAX_LAYERS; ++l) bits |= g[it][l] >= 0 ? 1u << l : 0u;
            if (f.level_mask) f.level_mask[(size_t)b * f.n + pid] = (unsigned char)bits;
            if (!bits) continue;
            const int tex   = __ldg(f.index + pid);
            const float conf = __ldg(f.confidence + tex);
            float4 desc;
            desc.x = __ldg(f.texture + tex);
            desc.y = __ldg(f.texture + (size_t)f.n_tex + tex);
            desc.z = __ldg(f.texture + 2 * (size_t)f.n_tex + tex);
            desc.w = f.C > 3 ? __ldg(f.texture + 3 * (size_t)f.n_tex + tex) : 0.f;
            const unsigned long long key = ((unsigned long long)zbits[it] << 32) | (unsigned)pid;
#pragma unroll
            for (int l = 0; l < VETR_MAX_LAYERS; ++l)
                if (g[it][l] >= 0 && (long long)g[it][l] < f.capacity) store_record(f, g[it][l], key, conf, tex, desc);
        }
        }
        return;
    }

    // mode 3: every (point, level) touches the four pixels around its position.  The record's descriptor index carries
    // the corner (0..3) in its two top bits: the backward pass files a fragment's result under (point, level, corner).
#pragma unroll
    for (int it = 0; it < kPts; ++it)
    {
        const int pid = first + it * kProjThreads;
        if (pid >= f.n) break;
        unsigned level_bits = 0;
        Projected pr;
        pr.z = 0.f;
        if (point_is_live(f, b, pid)) pr = project_point(pos[it], cam, f.dist_cutoff);
        if (pr.z == 0.f)
        {
            if (kCollect && f.level_mask) f.level_mask[(size_t)b * f.n + pid] = 0;
            continue;
        }
        float2 ip     = pr.ip;
        float radius  = pr.radius_px;
        const unsigned long long key = ((unsigned long long)__float_as_uint(pr.z) << 32) | (unsigned)pid;
        int tex      = 0;
        float conf   = 0.f;
        float4 desc  = make_float4(0.f, 0.f, 0.f, 0.f);
        if (kCollect && !(f.drop_by_radius && radius < f.radius_threshold))
        {
            tex    = __ldg(f.index + pid);
            conf   = __ldg(f.confidence + tex);
            desc.x = __ldg(f.texture + tex);
            desc.y = __ldg(f.texture + (size_t)f.n_tex + tex);
            desc.z = __ldg(f.texture + 2 * (size_t)f.n_tex + tex);
            desc.w = f.C > 3 ? __ldg(f.texture + 3 * (size_t)f.n_tex + tex) : 0.f;
        }
#pragma unroll 1
        for (int l = 0; l < f.L; ++l, radius *= 0.5f, ip.x *= 0.5f, ip.y *= 0.5f)
        {
            if (f.drop_by_radius && radius < f.radius_threshold) break;
            const int lw = f.lw[l], lh = f.lh[l];
            const int gbase = vbase + (int)f.lbase[l];
            const int bx = round_down(ip.x), by = round_down(ip.y);
            if (bx == INT32_MIN || by == INT32_MIN) continue;  // unrepresentable position
            int slot[4];
#pragma unroll
            for (int cidx = 0; cidx < 4; ++cidx)
            {
                const int x = bx + (cidx & 1), y = by + (cidx >> 1);
                slot[cidx]  = -1;
                if ((unsigned)x >= (unsigned)lw || (unsigned)y >= (unsigned)lh) continue;
                const int g = gbase + pixel_offset(lw, x, y);
                if (!kCollect)
                    atomicAdd(f.counts + g, 1);
                else
                    slot[cidx] = atomicAdd(f.ends + g, 1);
            }
            if (kCollect)
            {
#pragma unroll
                for (int cidx = 0; cidx < 4; ++cidx)
                {
                    if (slot[cidx] < 0) continue;
                    level_bits |= 1u << l;
                    if ((long long)slot[cidx] < f.capacity)
                        store_record(f, slot[cidx], key, blending_fac(ip, cidx, nullptr, nullptr) * conf,  // RenderForward.cu:1619
                                     tex | (cidx << kCornerShift), desc);
                }
            }
        }
        if (kCollect && f.level_mask) f.level_mask[(size_t)b * f.n + pid] = (unsigned char)level_bits;
    }
}

// ---------------------------------------------------------------------------------------------------------
// Pass 2: exclusive scan of counts -> ends (start offsets until the collection pass has advanced them to the
// list ends), total fragment count, longest list, and the work-item table.

__global__ void __launch_bounds__(256) scan_tile_sums_kernel(const int* __restrict__ counts, long long n,
                                                             long long* __restrict__ tile_sums, int* status)
{
    __shared__ long long s_sum[8];
    __shared__ int s_max[8];
    const long long base = (long long)blockIdx.x * kScanTile;
    long long sum = 0;
    int mx        = 0;
    for (int i = threadIdx.x; i < kScanTile; i += 256)
    {
        long long g = base + i;
        int c       = g < n ? counts[g] : 0;
        sum += c;
        mx = max(mx, c);
    }
    for (int o = 16; o > 0; o >>= 1)
    {
        sum += __shfl_down_sync(0xffffffffu, sum, o);
        mx = max(mx, __shfl_down_sync(0xffffffffu, mx, o));
    }
    if ((threadIdx.x & 31) == 0) s_sum[threadIdx.x >> 5] = sum, s_max[threadIdx.x >> 5] = mx;
    __syncthreads();
    if (threadIdx.x == 0)
    {
        for (int i = 1; i < 8; ++i) sum += s_sum[i], mx = max(mx, s_max[i]);
        tile_sums[blockIdx.x] = sum;
        if (mx > 0) atomicMax(status + 2, mx);
    }
}

// One CTA: exclusive scan of the tile sums in place; writes F, the overflow flag and the number of work items.
__global__ void __launch_bounds__(1024) scan_spine_kernel(long long* tile_sums, int n_tiles, long long n_pixels,
                                                          long long capacity, int* status, int* item_start)
{
    __shared__ long long s_warp[32];
    __shared__ long long s_carry;
    if (threadIdx.x == 0) s_carry = 0;
    __syncthreads();
    for (int base = 0; base < n_tiles; base += 1024)
    {
        int i         = base + threadIdx.x;
        long long v   = i < n_tiles ? tile_sums[i] : 0;
        long long inc = v;
        for (int o = 1; o < 32; o <<= 1)
        {
            long long t = __shfl_up_sync(0xffffffffu, inc, o);
            if ((threadIdx.x & 31) >= o) inc += t;
        }
        if ((threadIdx.x & 31) == 31) s_warp[threadIdx.x >> 5] = inc;
        __syncthreads();
        if (threadIdx.x < 32)
        {
            long long w = s_warp[threadIdx.x];
            for (int o = 1; o < 32; o <<= 1)
            {
                long long t = __shfl_up_sync(0xffffffffu, w, o);
                if (threadIdx.x >= o) w += t;
            }
            s_warp[threadIdx.x] = w;
        }
        __syncthreads();
        long long carry  = s_carry;
        long long before = carry + (threadIdx.x >= 32 ? s_warp[(threadIdx.x >> 5) - 1] : 0) + inc - v;
        if (i < n_tiles) tile_sums[i] = before;
        __syncthreads();
        if (threadIdx.x == 1023) s_carry = carry + s_warp[31];
        __syncthreads();
    }
    if (threadIdx.x == 0)
    {
        long long F   = s_carry;
        bool overflow = F > capacity || F > 0x7fffffffLL;
        status[0]     = (int)(F > 0x7fffffffLL ? 0x7fffffffLL : F);
        status[1]     = overflow ? 1 : 0;
        long long work = F + (long long)kPixelWork * n_pixels;
        int items      = overflow ? 0 : (int)((work + kQuantum - 1) / kQuantum);
        status[3]      = items;
        item_start[items] = (int)n_pixels;  // sentinel
    }
}

// Writes the exclusive offsets and cuts the pixel space into work items: with work(p) = end(p) + kPixelWork*(p+1)
// (strictly increasing), item k owns the pixels with k*Q < work(p) <= (k+1)*Q; pixel p opens every item k with
// work(p-1) <= k*Q < work(p).
__global__ void __launch_bounds__(256) scan_apply_kernel(const int* __restrict__ counts, long long n,
                                                         const long long* __restrict__ tile_offsets,
                                                         int* __restrict__ ends, const int* __restrict__ status,
                                                         int* __restrict__ item_start)
{
    __shared__ int s_warp[8];
    const long long base = (long long)blockIdx.x * kScanTile + threadIdx.x * 16;
    int c[16];
    int local = 0;
#pragma unroll
    for (int i = 0; i < 16; ++i)
    {
        long long g = base + i;
        c[i]        = g < n ? counts[g] : 0;
        local += c[i];
    }
    int inc = local;
    for (int o = 1; o < 32; o <<= 1)
    {
        int t = __shfl_up_sync(0xffffffffu, inc, o);
        if ((threadIdx.x & 31) >= o) inc += t;
    }
    if ((threadIdx.x & 31) == 31) s_warp[threadIdx.x >> 5] = inc;
    __syncthreads();
    int warp_before = 0;
    for (int i = 0; i < (int)(threadIdx.x >> 5); ++i) warp_before += s_warp[i];
    long long run       = tile_offsets[blockIdx.x] + warp_before + inc - local;
    const bool overflow = status[1] != 0;
#pragma unroll
    for (int i = 0; i < 16; ++i)
    {
        long long g = base + i;
        if (g < n)
        {
            ends[g] = (int)run;
            if (!overflow)
            {
                long long w_prev = run + (long long)kPixelWork * g;                // work(g-1)
                long long w_here = run + c[i] + (long long)kPixelWork * (g + 1);   // work(g)
                for (long long k = (w_prev + kQuantum - 1) / kQuantum; k * kQuantum < w_here; ++k)
                    item_start[k] = (int)g;
            }
        }
        run += c[i];
    }
}

// ---------------------------------------------------------------------------------------------------------
// Shared pieces of the item kernels.

struct PixInfo  // decoded pixel of the global pixel space, 8 bytes
{
    short x, y;
    unsigned char level, view;
    unsigned char interior;  // ImageView::distanceFromEdge > 2: the pixel takes part in the position gradient
    unsigned char valid;     // 0: padding row of the level's last band
};

// View, level and offset inside the level of pixel g, without divisions (a run of comparisons each).
__device__ __forceinline__ void locate_pixel(const Frame& f, unsigned g, int& view, int& level, unsigned& offset)
{
    const unsigned P = (unsigned)f.P;
    int v = 0;
#pragma unroll
    for (int i = 1; i < VETR_MAX_VIEWS; ++i)
        if (i < f.n_views && g >= i * P) v = i;
    unsigned q = g - v * P;
    int l      = 0;
#pragma unroll
    for (int i = 1; i < VETR_MAX_LAYERS; ++i)
        if (i < f.L && q >= (unsigned)f.lbase[i]) l = i;
    view = v, level = l, offset = q - (unsigned)f.lbase[l];
}

__device__ __forceinline__ PixInfo decode_pixel(const Frame& f, unsigned g)
{
    PixInfo r;
    int view, l;
    unsigned q;
    locate_pixel(f, g, view, l, q);
    const int w = f.lw[l], h = f.lh[l], bw = w << kBandShift;
    // band = q / (kBand w): float estimate, then one correction step either way (exact: the estimate is off by at most one)
    int band = __float2int_rz(__fmul_rn((float)q, f.inv_band[l]));
    int rem  = (int)q - band * bw;
    if (rem < 0) rem += bw, --band;
    if (rem >= bw) rem -= bw, ++band;
    const int x = rem >> kBandShift, y = (band << kBandShift) + (rem & (kBand - 1));
    r.x = (short)x, r.y = (short)y, r.level = (unsigned char)l, r.view = (unsigned char)view;
    r.valid    = y < h;
    r.interior = min(min(x, w - 1 - x), min(y, h - 1 - y)) > 2;
    return r;
}

// Index of a pixel in the row-major image copies (img4 / grad4).
__device__ __forceinline__ int row_major_index(const Frame& f, const PixInfo& px)
{
    return px.view * (int)f.Prm + (int)f.rbase[px.level] + px.y * f.lw[px.level] + px.x;
}

__device__ __forceinline__ int list_end(const Frame& f, int g) { return g < 0 ? 0 : f.ends[g]; }

// In-place ascending sort of a list (keys with their payload) in global memory by the whole CTA, for lists longer
// than kLongList.  Sorting network with all comparators pointing the same way, so that positions >= n behave as
// +infinity without padding.
__device__ void sort_long_list(const Frame& f, int first, int n)
{
    uint4* recs = f.recs + 2 * (size_t)first;
    int n2 = 1;
    while (n2 < n) n2 <<= 1;
    for (int k = 2; k <= n2; k <<= 1)
    {
        for (int j = k >> 1; j > 0; j >>= 1)
        {
            for (int i = threadIdx.x; i < n2; i += blockDim.x)
            {
                int partner = (j == (k >> 1)) ? (i ^ (k - 1)) : (i ^ j);
                if (partner > i && partner < n)
                {
                    uint4 a = recs[2 * i], b = recs[2 * partner];
                    if (record_key(a) > record_key(b))
                    {
                        recs[2 * i] = b, recs[2 * partner] = a;
                        uint4 da = recs[2 * i + 1], db = recs[2 * partner + 1];
                        recs[2 * i + 1] = db, recs[2 * partner + 1] = da;
                    }
                }
            }
            __syncthreads();
        }
    }
}

// Which list a staged fragment belongs to.  The thread that owns a pixel writes its index over the pixel's slots when
// the list is short; the few long lists of an item are recorded separately and matched by range.  (A binary search
// per fragment costs more instructions than everything else the sort does for it.)
constexpr int kFillMax  = 128;
constexpr int kMaxLong  = kCap / kFillMax + 1;
struct SegTable
{
    unsigned char seg_of[kCap];
    unsigned char long_pix[kMaxLong];
    int n_long[2];  // alternating between consecutive items, so that the reset never races with a fill
};
__device__ __forceinline__ void seg_fill(SegTable& t, int parity, int pixel, int ss, int se)
{
    if (se - ss <= kFillMax)
        for (int k = ss; k < se; ++k) t.seg_of[k] = (unsigned char)pixel;
    else
        t.long_pix[atomicAdd(&t.n_long[parity], 1)] = (unsigned char)pixel;
}
__device__ __forceinline__ int seg_lookup(const SegTable& t, int parity, const int* seg_end, int i)
{
    int a = t.seg_of[i];
    const int nl = t.n_long[parity];
    for (int k = 0; k < nl; ++k)
    {
        const int p = t.long_pix[k];
        if (i >= seg_end[p] && i < seg_end[p + 1]) a = p;
    }
    return a;
}

__device__ __forceinline__ float4 load_descriptor(const Frame& f, int tex)
{
    float4 d;
    d.x = __ldg(f.texture + tex);
    d.y = __ldg(f.texture + (size_t)f.n_tex + tex);
    d.z = __ldg(f.texture + 2 * (size_t)f.n_tex + tex);
    d.w = f.C > 3 ? __ldg(f.texture + 3 * (size_t)f.n_tex + tex) : 0.f;
    return d;
}

// First pixel of an item that the item kernels leave to the long-list kernels (0 or 1 pixels).
__device__ __forceinline__ int long_prefix(const Frame& f, int lo)
{
    return (f.ends[lo] - list_end(f, lo - 1)) > kLongList ? 1 : 0;
}

// Work items whose first pixel holds a long list, for the kernels that take one such list per CTA.  Testing an item costs
// four dependent loads (two table entries, two list ends), and only a few items in a thousand qualify, so the threads of
// a CTA test one item each and the CTA then works through the hits: next() is called by all threads and returns the same
// pixel to all of them.  CTA b owns the items b, b + gridDim.x, ... (long lists cluster at the coarse levels, i.e. in
// consecutive items: the stride spreads them over the CTAs).
struct LongItemScan
{
    int base, k, n;  // base: index of the next batch among the CTA's own items
    __device__ __forceinline__ LongItemScan() : base(0), k(0), n(0) {}
    __device__ bool next(const Frame& f, int n_items, int* s_hits, int* s_count, int& lo)
    {
        for (;;)
        {
            if (k < n)
            {
                lo = s_hits[k++];
                return true;
            }
            __syncthreads();  // every thread has taken the last hit of the previous batch
            if ((long long)blockIdx.x + (long long)base * gridDim.x >= n_items) return false;
            if (threadIdx.x == 0) *s_count = 0;
            __syncthreads();
            const long long item = (long long)blockIdx.x + (long long)(base + threadIdx.x) * gridDim.x;
            if (item < n_items)
            {
                const int first = f.item_start[item], last = f.item_start[item + 1];
                if (first < last && long_prefix(f, first)) s_hits[atomicAdd(s_count, 1)] = first;
            }
            __syncthreads();
            n = *s_count, k = 0;
            base += blockDim.x;
        }
    }
};

struct OutPtrs
{
    float* color[VETR_MAX_LAYERS];
    float* weight[VETR_MAX_LAYERS];
    float* mask[VETR_MAX_LAYERS];
    float* depth[VETR_MAX_LAYERS];
};

// Outputs of pixel g of the global pixel space (planar [view, channel, y, x] tensors per level).
__device__ __forceinline__ void write_pixel(const Frame& f, const OutPtrs& out, unsigned g, const float c[4], float T, float depth)
{
    const PixInfo px = decode_pixel(f, g);
    if (!px.valid) return;
    const int level = px.level, view = px.view;
    const int w = f.lw[level], hw = w * f.lh[level], o = px.y * w + px.x;
    float* col = out.color[level] + (size_t)(view * f.C) * hw + o;
    col[0] = c[0], col[hw] = c[1], col[2 * hw] = c[2];
    if (f.C > 3) col[3 * hw] = c[3];
    const size_t po = (size_t)view * hw + o;
    if (out.weight[0]) out.weight[level][po] = T;
    if (out.mask[0]) out.mask[level][po] = (T == 0.f) ? f.mask_value : 1.f;
    if (out.depth[0]) out.depth[level][po] = depth;
}

// Front-to-back fold of one list (BlendMulti / BlendMultiBilinear, RenderForward.cu:1320-1356, 1597-1639).
struct Fold
{
    float T;
    float c[4];
    __device__ __forceinline__ void init()
    {
        T    = 1.f;
        c[0] = c[1] = c[2] = c[3] = 0.f;
    }
    __device__ __forceinline__ void add(float a, float4 d)
    {
        c[0] = vetr_blend(T, a, d.x, c[0]);
        c[1] = vetr_blend(T, a, d.y, c[1]);
        c[2] = vetr_blend(T, a, d.z, c[2]);
        c[3] = vetr_blend(T, a, d.w, c[3]);
        T    = vetr_new_T(T, a);
    }
    __device__ __forceinline__ void background(const Frame& f, const float bg[4])
    {
        const bool bilinear = f.mode == VETR_MODE_BILINEAR_BLEND;
        if (!f.use_env && !(bilinear && !(T >= 0.001f)))
        {
            c[0] = vetr_blend(T, 1.f, bg[0], c[0]), c[1] = vetr_blend(T, 1.f, bg[1], c[1]), c[2] = vetr_blend(T, 1.f, bg[2], c[2]);
            if (f.C > 3) c[3] = vetr_blend(T, 1.f, bg[3], c[3]);
        }
    }
};

// Mode 2 (BlendMultiFuzzy, RenderForward.cu:1412-1492): fragments within depth_accept_blend of the list's FIRST depth
// are averaged and blended as one; the reference then resets its reference depth to -100000, so every later fragment
// is a group of its own.  Transcribed literally.
struct FuzzyFold
{
    Fold fold;
    float last_min_d, acc_conf, acc_desc[4];
    int n_acc;
    __device__ __forceinline__ void init()
    {
        fold.init();
        last_min_d = acc_conf = 0.f;
        acc_desc[0] = acc_desc[1] = acc_desc[2] = acc_desc[3] = 0.f;
        n_acc       = 0;
    }
    __device__ __forceinline__ void flush()
    {
        const float n    = (float)n_acc;
        const float conf = acc_conf / n;
        fold.add(conf, make_float4(acc_desc[0] / n, acc_desc[1] / n, acc_desc[2] / n, acc_desc[3] / n));
    }
    __device__ __forceinline__ void add(float depth, float conf, float4 d, float accept)
    {
        if (last_min_d == 0.f) last_min_d = depth;
        if (!(depth - last_min_d < accept))
        {
            flush();
            last_min_d = -100000.f;
            acc_conf   = 0.f;
            n_acc      = 0;
            acc_desc[0] = acc_desc[1] = acc_desc[2] = acc_desc[3] = 0.f;
        }
        acc_conf += conf;
        acc_desc[0] += d.x, acc_desc[1] += d.y, acc_desc[2] += d.z, acc_desc[3] += d.w;
        ++n_acc;
    }
    __device__ __forceinline__ void finish()
    {
        if (n_acc > 0) flush();
    }
};

// ---------------------------------------------------------------------------------------------------------
// Pass 4: sort + blend.

struct BlendSmem
{
    unsigned long long key[kCap];  // arrival order
    float4 desc[kCap];
    float alpha[kCap];
    int tex[kCap];
    unsigned short perm[kCap];     // sorted position -> arrival slot
    int seg_end[kMaxPixels + 1];
    SegTable seg;
};

__global__ void __launch_bounds__(kThreads, kMinCtas) sort_blend_kernel(const __grid_constant__ Frame f,
                                                                        const __grid_constant__ OutPtrs out)
{
    extern __shared__ __align__(16) unsigned char smem_raw[];
    BlendSmem& s = *reinterpret_cast<BlendSmem*>(smem_raw);
    const int tid     = threadIdx.x;
    const int n_items = f.status[3];
    const bool bilinear = f.mode == VETR_MODE_BILINEAR_BLEND;
    const float bg[4]   = {f.background[0], f.background[1], f.background[2], f.C > 3 ? f.background[3] : 0.f};
    if (tid == 0) s.seg.n_long[0] = s.seg.n_long[1] = 0;
    int parity = 0;

    for (int item = blockIdx.x; item < n_items; item += gridDim.x)
    {
        int lo = f.item_start[item];
        const int hi = f.item_start[item + 1];
        if (lo >= hi) continue;
        lo += long_prefix(f, lo);
        if (lo >= hi) continue;
        __syncthreads();  // every warp has left the previous item
        parity ^= 1;
        if (tid == 0) s.seg.n_long[parity ^ 1] = 0;
        const int f0 = list_end(f, lo - 1);
        const int np = hi - lo;
        const int nf = f.ends[hi - 1] - f0;
        // the thread's first record is requested before the per-pixel set-up, each further one before the previous is stored
        uint4 h_next = make_uint4(0, 0, 0, 0), d_next = h_next;
        if (tid < nf) h_next = f.recs[2 * (size_t)(f0 + tid)], d_next = f.recs[2 * (size_t)(f0 + tid) + 1];
        if (tid < np)
        {
            const int ss = list_end(f, lo + tid - 1) - f0, se = f.ends[lo + tid] - f0;
            s.seg_end[tid + 1] = se;
            seg_fill(s.seg, parity, tid, ss, se);
        }
        if (tid == 0) s.seg_end[0] = 0;
        // stream keys and payload of the item (contiguous, coalesced)
        for (int i = tid; i < nf; i += kThreads)
        {
            const uint4 h = h_next, d = d_next;
            if (i + kThreads < nf)
                h_next = f.recs[2 * (size_t)(f0 + i + kThreads)], d_next = f.recs[2 * (size_t)(f0 + i + kThreads) + 1];
            s.desc[i]     = as_float4(d);
            s.key[i]      = record_key(h);
            s.alpha[i]    = __uint_as_float(h.z);
            s.tex[i]      = (int)h.w;
        }
        __syncthreads();
        // rank sort inside each list; keys are unique (distinct point indices), so ranks are a permutation
        for (int i = tid; i < nf; i += kThreads)
        {
            const int a  = seg_lookup(s.seg, parity, s.seg_end, i);
            const int ss = s.seg_end[a], se = s.seg_end[a + 1];
            const unsigned long long key = s.key[i];
            int rank = 0;
            for (int k = ss; k < se; ++k) rank += s.key[k] < key;
            s.perm[ss + rank] = (unsigned short)i;
        }
        __syncthreads();
        // write the sorted lists back for the backward pass
        if (f.keep_sorted)
            for (int r = tid; r < nf; r += kThreads)
            {
                const int u = s.perm[r];
                store_record(f, f0 + r, s.key[u], s.alpha[u], s.tex[u], s.desc[u]);
            }
        // fold: one thread per pixel
        if (tid < np)
        {
            const int ss = s.seg_end[tid], se = s.seg_end[tid + 1];
            int cnt = se - ss;
            if (f.dbg_max_len > 0) cnt = min(cnt, f.dbg_max_len);
            Fold fold;
            if (f.mode == VETR_MODE_FUZZY_BLEND)
            {
                FuzzyFold ff;
                ff.init();
                for (int r = ss; r < ss + cnt; ++r)
                {
                    const int u = s.perm[r];
                    ff.add(__uint_as_float((unsigned)(s.key[u] >> 32)), s.alpha[u], s.desc[u], f.accept_blend);
                }
                ff.finish();
                fold = ff.fold;
            }
            else
            {
                fold.init();
                for (int r = ss; r < ss + cnt; ++r)
                {
                    const int u = s.perm[r];
                    fold.add(s.alpha[u], s.desc[u]);
                    if (bilinear && fold.T < 0.001f) break;
                }
            }
            fold.background(f, bg);
            float depth = se > ss ? __uint_as_float((unsigned)(s.key[s.perm[ss]] >> 32)) : kMaxDepth;
            write_pixel(f, out, (unsigned)(lo + tid), fold.c, fold.T, depth);
        }
    }
}

// Lists longer than kLongList: one CTA per list.  Up to kLongSortMax fragments the whole list is staged in shared memory,
// rank-sorted there and written back in order (the reference's <= 4096 bucket is a CTA-wide shared-memory sort as well,
// AlphaListSort.cu:601-703); longer lists are sorted in global memory.  The fold runs in blocks of kCap fragments.
constexpr int kLongSortMax = 2048;
struct LongSortSmem
{
    uint4 rec[2 * kLongSortMax];
    unsigned long long key[kLongSortMax];
    unsigned short perm[kLongSortMax];
};
constexpr size_t kLongBlendSmem = sizeof(LongSortSmem) > sizeof(BlendSmem) ? sizeof(LongSortSmem) : sizeof(BlendSmem);

__device__ void sort_long_list_shared(const Frame& f, LongSortSmem& ls, int first, int n)
{
    uint4* recs = f.recs + 2 * (size_t)first;
    for (int i = threadIdx.x; i < n; i += blockDim.x)
    {
        const uint4 h = recs[2 * i];
        ls.rec[2 * i] = h, ls.rec[2 * i + 1] = recs[2 * i + 1];
        ls.key[i]     = record_key(h);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += blockDim.x)
    {
        const unsigned long long key = ls.key[i];
        int rank = 0;
        for (int k = 0; k < n; ++k) rank += ls.key[k] < key;
        ls.perm[rank] = (unsigned short)i;
    }
    __syncthreads();
    for (int r = threadIdx.x; r < n; r += blockDim.x)
    {
        const int u = ls.perm[r];
        recs[2 * r] = ls.rec[2 * u], recs[2 * r + 1] = ls.rec[2 * u + 1];
    }
    __syncthreads();  // the fold below reads the sorted records back and reuses this shared memory
}

__global__ void __launch_bounds__(kThreads) sort_blend_long_kernel(const __grid_constant__ Frame f,
                                                                   const __grid_constant__ OutPtrs out)
{
    if (f.status[2] <= kLongList) return;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    BlendSmem& s = *reinterpret_cast<BlendSmem*>(smem_raw);
    __shared__ float s_fold[16];  // carried between blocks: T, colour, stop flag; mode 2: reference depth, sums, count
    const int tid       = threadIdx.x;
    const int n_items   = f.status[3];
    const bool bilinear = f.mode == VETR_MODE_BILINEAR_BLEND;
    __shared__ int s_long_hits[kThreads], s_long_count;
    LongItemScan scan;
    int lo;
    while (scan.next(f, n_items, s_long_hits, &s_long_count, lo))
    {
        const int e0 = list_end(f, lo - 1);
        const int n  = f.ends[lo] - e0;
        __syncthreads();
        if (n <= kLongSortMax)
            sort_long_list_shared(f, *reinterpret_cast<LongSortSmem*>(smem_raw), e0, n);
        else
            sort_long_list(f, e0, n);
        int cnt = n;
        if (f.dbg_max_len > 0) cnt = min(cnt, f.dbg_max_len);
        if (tid == 0)
        {
            s_fold[0] = 1.f;
            for (int k = 1; k < 16; ++k) s_fold[k] = 0.f;
        }
        __syncthreads();
        for (int blk = 0; blk < cnt; blk += kCap)
        {
            const int m = min(kCap, cnt - blk);
            for (int i = tid; i < m; i += kThreads)
            {
                const uint4 h = f.recs[2 * (size_t)(e0 + blk + i)];
                s.key[i]      = record_key(h);
                s.alpha[i]    = __uint_as_float(h.z);
                s.desc[i]     = as_float4(f.recs[2 * (size_t)(e0 + blk + i) + 1]);
            }
            __syncthreads();
            if (tid == 0 && s_fold[5] == 0.f)
            {
                FuzzyFold ff;
                ff.fold.T = s_fold[0];
                for (int k = 0; k < 4; ++k) ff.fold.c[k] = s_fold[1 + k];
                ff.last_min_d = s_fold[6], ff.acc_conf = s_fold[7], ff.n_acc = (int)s_fold[12];
                for (int k = 0; k < 4; ++k) ff.acc_desc[k] = s_fold[8 + k];
                for (int i = 0; i < m; ++i)
                {
                    if (f.mode == VETR_MODE_FUZZY_BLEND)
                        ff.add(__uint_as_float((unsigned)(s.key[i] >> 32)), s.alpha[i], s.desc[i], f.accept_blend);
                    else
                    {
                        ff.fold.add(s.alpha[i], s.desc[i]);
                        if (bilinear && ff.fold.T < 0.001f)
                        {
                            s_fold[5] = 1.f;
                            break;
                        }
                    }
                }
                s_fold[0] = ff.fold.T;
                for (int k = 0; k < 4; ++k) s_fold[1 + k] = ff.fold.c[k];
                s_fold[6] = ff.last_min_d, s_fold[7] = ff.acc_conf, s_fold[12] = (float)ff.n_acc;
                for (int k = 0; k < 4; ++k) s_fold[8 + k] = ff.acc_desc[k];
            }
            __syncthreads();
        }
        if (tid == 0)
        {
            FuzzyFold ff;
            ff.fold.T = s_fold[0];
            for (int k = 0; k < 4; ++k) ff.fold.c[k] = s_fold[1 + k];
            ff.last_min_d = s_fold[6], ff.acc_conf = s_fold[7], ff.n_acc = (int)s_fold[12];
            for (int k = 0; k < 4; ++k) ff.acc_desc[k] = s_fold[8 + k];
            if (f.mode == VETR_MODE_FUZZY_BLEND) ff.finish();
            Fold fold = ff.fold;
            const float bg[4] = {f.background[0], f.background[1], f.background[2], f.C > 3 ? f.background[3] : 0.f};
            fold.background(f, bg);
            write_pixel(f, out, (unsigned)lo, fold.c, fold.T, __uint_as_float(f.recs[2 * (size_t)e0].y));
        }
    }
}

// ---------------------------------------------------------------------------------------------------------
// Backward.

struct BackPtrs
{
    const float* out_color[VETR_MAX_LAYERS];
    const float* grad_color[VETR_MAX_LAYERS];
    float4* g_desc;
    float* g_conf;
    float4* g_points;
    float* g_background;
    double* g_pose;
    float* g_pose_count;
    float* g_intr;
    float* g_intr_count;
};

struct BackSmem
{
    int pid[kCap];
    int tex[kCap];
    float alpha[kCap];
    float dot[kCap];     // d_i . G  ->  replaced by the alpha gradient of the fragment
    float trans[kCap];   // T_i ; NaN = fragment not blended (early termination / list truncation)
    float4 grad[kMaxPixels];  // incoming gradient of the pixel
    int seg_end[kMaxPixels + 1];
    PixInfo pix[kMaxPixels];
    SegTable seg;
    double red[kThreads / 32][8];  // cross-warp reduction scratch
};

// Mode 2 additionally needs every fragment's descriptor and depth (groups average them) and two group markers.
struct BackSmemFuzzy : BackSmem
{
    float4 desc[kCap];
    float depth[kCap];
    float gv[kCap];               // at the first fragment of a group: sum_c G_c * colour_c * T * conf of that group
    unsigned char gfirst[kCap];   // 1 = first fragment of its group
};

// Gradient accumulation with fire-and-forget reductions.  The gradient buffers are never read by these kernels, so
// the compiler may move other memory operations across them (no memory clobber).
__device__ __forceinline__ void red_add_v4(float4* addr, float4 v)
{
    asm volatile("red.global.add.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(addr), "f"(v.x), "f"(v.y), "f"(v.z), "f"(v.w));
}
__device__ __forceinline__ void red_add(float* addr, float v)
{
    asm volatile("red.global.add.f32 [%0], %1;" ::"l"(addr), "f"(v));
}

// Camera-gradient accumulators of one thread for the pixels of a single view: pose in double like the reference's
// atomics (RenderBackward.cu:1423), the rest in float.
template <bool kIntr>
struct CamAcc
{
    double pose[6];
    float pose_count;
    float intr[kIntr ? 14 : 1];  // 13 gradients + count
    __device__ __forceinline__ void clear()
    {
#pragma unroll
        for (int k = 0; k < 6; ++k) pose[k] = 0.0;
        pose_count = 0.f;
#pragma unroll
        for (int k = 0; k < (kIntr ? 14 : 1); ++k) intr[k] = 0.f;
    }
};

// Sums the accumulators over the CTA and adds the totals to the outputs of `view`: one atomic per value and
// (CTA, view) instead of one per fragment.
template <bool kIntr>
__device__ void reduce_cam(const Frame& f, const BackPtrs& bp, CamAcc<kIntr>& acc, int view, double (*red)[8])
{
    constexpr int kN = kIntr ? 21 : 7;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const ViewDev& vw = f.views[view];
    for (int base = 0; base < kN; base += 8)
    {
        __syncthreads();
        for (int k = base; k < min(base + 8, kN); ++k)
        {
            double x = k < 6 ? acc.pose[k] : (k == 6 ? (double)acc.pose_count : (double)acc.intr[kIntr ? k - 7 : 0]);
            for (int o = 16; o > 0; o >>= 1) x += __shfl_down_sync(0xffffffffu, x, o);
            if (lane == 0) red[warp][k - base] = x;
        }
        __syncthreads();
        const int k = base + threadIdx.x;
        if (threadIdx.x < 8 && k < kN)
        {
            double x = 0.0;
            for (int w = 0; w < (int)blockDim.x / 32; ++w) x += red[w][threadIdx.x];
            if (x != 0.0)
            {
                if (k < 6)
                    atomicAdd(bp.g_pose + 6 * vw.image_index + k, x);
                else if (k == 6)
                    atomicAdd(bp.g_pose_count + vw.image_index, (float)x);
                else if (k < 20)
                    atomicAdd(bp.g_intr + 13 * vw.camera_index + (k - 7), (float)x);
                else
                    atomicAdd(bp.g_intr_count + vw.camera_index, (float)x);
            }
        }
    }
    acc.clear();
}

// Spatial gradient of one fragment: image-space gradient dR -> point, pose and intrinsics gradients
// (RenderBackward.cu:1380-1460 and :3097-3180).
template <bool kIntr>
__device__ __forceinline__ void spatial_terms(const Frame& f, const BackPtrs& bp, const Camera& cam, int level,
                                              const PointJac& jac, float2 dR, CamAcc<kIntr>& acc, BackOut& bo)
{
    float scale = 1.f;
    for (int l = 0; l < level; ++l) scale *= 0.5f;
    float crop2[5];
#pragma unroll
    for (int k = 0; k < 5; ++k) crop2[k] = cam.crop[k] * scale;  // IntrinsicsPinhole::scale
    project_backward_apply(jac, dR, cam, crop2, kIntr, bo);
    if (bp.g_pose)
    {
#pragma unroll
        for (int k = 0; k < 6; ++k) acc.pose[k] += (double)bo.g_pose[k];
        // RenderBackward.cu:379 (mode 0) and :3144 (mode 3) count 1 per hit, :993 and :1425 (modes 2, 1) count 1/1024
        acc.pose_count += (f.mode == VETR_MODE_BILINEAR_BLEND || f.mode == VETR_MODE_FUZZY_DT) ? 1.f : (1.f / 1024.f);
    }
    if (kIntr)
    {
        bo.g_k[4] *= 0.f;
#pragma unroll
        for (int k = 0; k < 5; ++k) acc.intr[k] += f.k_grad_factor * bo.g_k[k];
        bo.g_dis[2] *= 0.25f;
#pragma unroll
        for (int k = 3; k < 8; ++k) bo.g_dis[k] *= 0.1f;
#pragma unroll
        for (int k = 0; k < 8; ++k) acc.intr[5 + k] += f.dist_grad_factor * bo.g_dis[k];
        acc.intr[kIntr ? 13 : 0] += 1.f / 1024.f;
    }
}

template <bool kIntr>
__device__ __forceinline__ void spatial_backward(const Frame& f, const BackPtrs& bp, const Camera& cam, const PixInfo& px,
                                                 int pid, float4 pos, float2 dR, CamAcc<kIntr>& acc)
{
    PointJac jac;
    if (!project_backward_prepare(pos, cam, f.dist_cutoff, kIntr, jac)) return;
    BackOut bo;
    spatial_terms<kIntr>(f, bp, cam, px.level, jac, dR, acc, bo);
    if (bp.g_points) red_add_v4(bp.g_points + pid, make_float4(bo.g_point[0], bo.g_point[1], bo.g_point[2], 1.f));
}

// Modes 1 and 2: approximate image-space gradient of a fragment from the neighbouring pixels
// (RenderBackward.cu:1347-1374).  `g` is the pixel in the global pixel space; the images are the channel-interleaved
// copies pack_images_kernel makes, so the eight neighbour values of all channels are eight 16-byte loads.
struct Neighbours
{
    float4 il, ir, iu, id, gl, gr, gu, gd;  // forward image and its gradient left / right / above / below the pixel
    __device__ __forceinline__ void load(const Frame& f, int g, int w)
    {
        const float4* I  = f.img4 + g;
        const float4* Gp = f.grad4 + g;
        il = __ldg(I - 1), ir = __ldg(I + 1), iu = __ldg(I - w), id = __ldg(I + w);
        gl = __ldg(Gp - 1), gr = __ldg(Gp + 1), gu = __ldg(Gp - w), gd = __ldg(Gp + w);
    }
    __device__ __forceinline__ float2 gradient(const Frame& f, float4 d) const
    {
        const float dv[4] = {d.x, d.y, d.z, d.w};
        const float Il[4] = {il.x, il.y, il.z, il.w}, Ir[4] = {ir.x, ir.y, ir.z, ir.w};
        const float Iu[4] = {iu.x, iu.y, iu.z, iu.w}, Id[4] = {id.x, id.y, id.z, id.w};
        const float Gl[4] = {gl.x, gl.y, gl.z, gl.w}, Gr[4] = {gr.x, gr.y, gr.z, gr.w};
        const float Gu[4] = {gu.x, gu.y, gu.z, gu.w}, Gd[4] = {gd.x, gd.y, gd.z, gd.w};
        float dx = 0.f, dy = 0.f;
#pragma unroll
        for (int ci = 0; ci < 4; ++ci)
        {
            if (ci < f.C)
            {
                float Tp = dv[ci];
                float a0 = -(Tp - Il[ci]) * Gl[ci];
                float a1 = (Tp - Ir[ci]) * Gr[ci];
                float b0 = -(Tp - Iu[ci]) * Gu[ci];
                float b1 = (Tp - Id[ci]) * Gd[ci];
                dx += 0.5f * (a0 + a1);
                dy += 0.5f * (b0 + b1);
            }
        }
        // x / 4 and x * 0.25 round alike
        return f.C == 4 ? make_float2(dx * 0.25f, dy * 0.25f) : make_float2(dx / (float)f.C, dy / (float)f.C);
    }
};

__device__ __forceinline__ float2 neighbour_gradient(const Frame& f, int g, int w, float4 d)
{
    Neighbours nb;
    nb.load(f, g, w);
    return nb.gradient(f, d);
}

__device__ __forceinline__ float4 load_grad(const Frame& f, int g) { return __ldg(f.grad4 + g); }

// Channel-interleaved copies of the forward image and of its gradient over the global pixel space (the caller's
// tensors are planar [view, channel, y, x] per level).
__global__ void __launch_bounds__(256) pack_images_kernel(const __grid_constant__ Frame f, const __grid_constant__ BackPtrs bp)
{
    // one thread per pixel in plain row-major order (view, level, y, x): coalesced reads of the planar tensors
    const long long r = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (r >= f.Prm * f.n_views) return;
    const int Prm  = (int)f.Prm;
    int view = 0;
#pragma unroll
    for (int i = 1; i < VETR_MAX_VIEWS; ++i)
        if (i < f.n_views && r >= (long long)i * Prm) view = i;
    const int q = (int)(r - (long long)view * Prm);
    int l = 0;
#pragma unroll
    for (int i = 1; i < VETR_MAX_LAYERS; ++i)
        if (i < f.L && q >= (int)f.rbase[i]) l = i;
    const int o  = q - (int)f.rbase[l];  // y * w + x
    const int hw = f.lw[l] * f.lh[l];
    const float* I = bp.out_color[l] + (size_t)(view * f.C) * hw + o;
    const float* G = bp.grad_color[l] + (size_t)(view * f.C) * hw + o;
    f.img4[r]  = make_float4(__ldg(I), __ldg(I + hw), __ldg(I + 2 * hw), f.C > 3 ? __ldg(I + 3 * hw) : 0.f);
    f.grad4[r] = make_float4(__ldg(G), __ldg(G + hw), __ldg(G + 2 * hw), f.C > 3 ? __ldg(G + 3 * hw) : 0.f);
}

__device__ __forceinline__ float dot4(float4 a, float4 b, int C)
{
    // same order as the reference's loop over channels (RenderBackward.cu:1146-1155)
    float r = 0.f;
    r += a.x * b.x;
    r += a.y * b.y;
    r += a.z * b.z;
    if (C > 3) r += a.w * b.w;
    return r;
}

// Image-space gradient of a fragment that takes no part in the position gradient (border pixel, cut-off list).
constexpr int kNoGradientBits = 0x7fffffff;

// Stage A of a fragment (needs nothing from the sweeps): streams the fragment's key and payload, computes d.G, and
// in modes 1 and 2 its image-space gradient (which depends on the descriptor and the neighbouring pixels only).  That
// gradient is parked under (view, level, point); point_backward_kernel turns it into position / camera gradients with
// coalesced position loads and without atomics, instead of a position gather per fragment here.
template <bool kBilinear>
__device__ __forceinline__ void fragment_stage_a(const Frame& f, BackSmem& s, int g, const PixInfo& px, float4 G, int slot,
                                                 uint4 h, uint4 payload, bool blended, float4* desc_out = nullptr,
                                                 float* depth_out = nullptr)
{
    const float4 d = as_float4(payload);
    const int pid  = (int)h.x;
    if (desc_out) desc_out[slot] = d, depth_out[slot] = __uint_as_float(h.y);
    s.pid[slot]    = pid;
    s.tex[slot]    = (int)h.w;
    s.alpha[slot]  = __uint_as_float(h.z);
    s.dot[slot]    = dot4(d, G, f.C);
    if (!kBilinear && f.need_point_grad)
    {
        float2 dR = make_float2(__int_as_float(kNoGradientBits), 0.f);
        if (blended && px.interior) dR = neighbour_gradient(f, row_major_index(f, px), f.lw[px.level], d);
        f.point_grad[((size_t)px.view * f.L + px.level) * f.n + pid] = dR;
    }
}

// Stage B of a fragment (after the sweeps): the descriptor gradient, and the confidence gradient - directly in modes 1
// and 2; in mode 3 it is weighted by the bilinear weight of the fragment's corner, which needs the point's projection, so
// the fragment's alpha gradient is parked under (view, level, point, corner) for point_backward_kernel (the reference
// writes it for interior pixels only, RenderBackward.cu:3053).  `blended` = false: the list ended before this fragment.
template <bool kBilinear>
__device__ __forceinline__ void fragment_stage_b(const Frame& f, const BackPtrs& bp, const PixInfo& px, float4 G, int pid,
                                                 int tex_word, float Ta, float galpha, bool blended)
{
    if (kBilinear)
    {
        const int corner  = (unsigned)tex_word >> kCornerShift;
        float* parked     = reinterpret_cast<float*>(f.point_grad);
        const size_t slot = ((((size_t)px.view * f.L + px.level) * f.n + pid) << 2) + corner;
        parked[slot]      = blended && px.interior ? galpha : __int_as_float(kNoGradientBits);
        if (!blended) return;
    }
    const int tex = kBilinear ? tex_word & kTexMask : tex_word;
    // descriptor gradient: T * alpha * G  (RenderBackward.cu:1149-1152)
    red_add_v4(bp.g_desc + tex, make_float4(Ta * G.x, Ta * G.y, Ta * G.z, f.C > 3 ? Ta * G.w : 0.f));
    if (!kBilinear) red_add(bp.g_conf + tex, galpha);
}

// Transmittance forward and suffix sum backward over one list held in shared memory: the O(n) form of the
// reference's double loop (RenderBackward.cu:1118-1181).  Leaves T_i in trans[] and d(loss)/d(alpha_i) in dot[].
__device__ __forceinline__ void sweep_list(const Frame& f, BackSmem& s, int ss, int se, float4 G, float4 bgc,
                                           float bg_acc[4], float& p0_acc)
{
    const bool bilinear = f.mode == VETR_MODE_BILINEAR_BLEND;
    int cnt = se - ss;
    if (f.dbg_max_len > 0) cnt = min(cnt, f.dbg_max_len);
    float T = 1.f;
    int eff = cnt;
    for (int i = 0; i < cnt; ++i)
    {
        s.trans[ss + i] = T;
        T               = vetr_new_T(T, s.alpha[ss + i]);
        if (bilinear && T < 0.001f)
        {
            eff = i + 1;
            break;
        }
    }
    for (int i = ss + eff; i < se; ++i) s.trans[i] = __int_as_float(0x7fffffff);  // NaN: not blended, no gradient
    const bool bg_term = !f.use_env && !(bilinear && !(T >= 0.001f));
    float S = 0.f;
    if (bg_term)
    {
        float dotb = dot4(bgc, G, f.C);
        bg_acc[0] += T * 1.f * G.x, bg_acc[1] += T * 1.f * G.y, bg_acc[2] += T * 1.f * G.z;
        if (f.C > 3) bg_acc[3] += T * 1.f * G.w;
        if (!bilinear && f.bg_alpha_to_point0) p0_acc += dotb * T;
        S = T * 1.f * dotb;
    }
    for (int i = ss + eff - 1; i >= ss; --i)
    {
        float a = s.alpha[i], Ti = s.trans[i], dt = s.dot[i];
        s.dot[i]   = Ti * dt - S / (1 - a + 1e-9f);
        s.trans[i] = Ti * a;  // from here on: the factor of G in the fragment's descriptor gradient
        S += Ti * a * dt;
    }
}

// Mode 2 sweeps over one list (BlendBackwardsFuzzy, RenderBackward.cu:603-749) in O(n): groups are formed against the
// first depth of every group, the background is an entry of depth 100000 (confidence 1, colour = background), a
// group's descriptor / confidence gradients are shared equally by its fragments, and the term a later group passes to
// the confidence of an earlier fragment uses that fragment's GROUP confidence and is not divided by the group size.
// Leaves the factor of G of the descriptor gradient in trans[] (NaN = not blended) and the confidence gradient in dot[].
__device__ __forceinline__ void sweep_list_fuzzy(const Frame& f, float* alpha, float* dot, float* trans, const float4* desc,
                                                 const float* depth, float* gv, unsigned char* gfirst, int ss, int se,
                                                 float4 G, float4 bgc, float bg_acc[4])
{
    int cnt = se - ss;
    if (f.dbg_max_len > 0) cnt = min(cnt, f.dbg_max_len);
    for (int i = ss + cnt; i < se; ++i) trans[i] = __int_as_float(0x7fffffff);
    const int list_size = f.use_env ? cnt : cnt + 1;
    float last_min_d = 0.f, acc_conf = 0.f, T = 1.f, S_tail = 0.f;
    float4 acc_desc = make_float4(0.f, 0.f, 0.f, 0.f);
    int n_acc = 0, start = 0;
    auto close_group = [&]()
    {
        const float inv_w = 1.f / (float)n_acc;
        const float conf  = acc_conf * inv_w;
        const float4 col  = make_float4(acc_desc.x * inv_w, acc_desc.y * inv_w, acc_desc.z * inv_w, acc_desc.w * inv_w);
        const float g_alpha = dot4(col, G, f.C) * T;
        float v = 0.f;
        v += G.x * col.x * T * conf;
        v += G.y * col.y * T * conf;
        v += G.z * col.z * T * conf;
        if (f.C > 3) v += G.w * col.w * T * conf;
        for (int t = start; t < start + n_acc; ++t)
        {
            if (t < cnt)
            {
                trans[ss + t]  = T * conf * inv_w;
                dot[ss + t]    = g_alpha * inv_w;
                alpha[ss + t]  = conf;  // the group's confidence, used below for earlier fragments
                gfirst[ss + t] = t == start;
                gv[ss + t]     = v;
            }
            else
            {
                bg_acc[0] += T * conf * G.x * inv_w, bg_acc[1] += T * conf * G.y * inv_w, bg_acc[2] += T * conf * G.z * inv_w;
                if (f.C > 3) bg_acc[3] += T * conf * G.w * inv_w;
            }
        }
        if (start >= cnt) S_tail = v;  // the group consists of the background entry alone
        T = vetr_new_T(T, conf);
    };
    for (int i = 0; i < list_size; ++i)
    {
        const bool fg = i != cnt;
        const float d = fg ? depth[ss + i] : kMaxDepth;
        if (!(d - last_min_d < f.accept_blend))
        {
            if (i != 0) close_group();
            acc_conf = 0.f, n_acc = 0, acc_desc = make_float4(0.f, 0.f, 0.f, 0.f);
            last_min_d = d;
            start      = i;
        }
        const float4 c = fg ? desc[ss + i] : bgc;
        acc_conf += fg ? alpha[ss + i] : 1.f;
        acc_desc.x += c.x, acc_desc.y += c.y, acc_desc.z += c.z, acc_desc.w += c.w;
        ++n_acc;
    }
    if (n_acc > 0) close_group();
    float S = S_tail;  // sum of v over the groups after the current one
    for (int t = cnt - 1; t >= 0; --t)
    {
        dot[ss + t] -= S / (1 - alpha[ss + t] + 1e-9f);
        if (gfirst[ss + t]) S += gv[ss + t];
    }
}

// Background gradient and the confidence term the reference routes to descriptor 0: CTA reduction, one atomic each.
__device__ __forceinline__ void reduce_background(const Frame& f, const BackPtrs& bp, BackSmem& s, const float bg_acc[4],
                                                  float p0_acc)
{
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float v[5] = {bg_acc[0], bg_acc[1], bg_acc[2], bg_acc[3], p0_acc};
    for (int k = 0; k < 5; ++k)
    {
        float x = v[k];
        for (int o = 16; o > 0; o >>= 1) x += __shfl_down_sync(0xffffffffu, x, o);
        if (lane == 0) s.red[warp][k] = (double)x;
    }
    __syncthreads();
    if (threadIdx.x < 5)
    {
        float x = 0.f;
        for (int w = 0; w < kThreads / 32; ++w) x += (float)s.red[w][threadIdx.x];
        if (x != 0.f)
        {
            if (threadIdx.x < 4)
            {
                if ((int)threadIdx.x < f.C) atomicAdd(bp.g_background + threadIdx.x, x);
            }
            else
                atomicAdd(bp.g_conf + 0, x);
        }
    }
}


template <bool kFuzzy>
struct BackSmemOf
{
    using type = BackSmem;
};
template <>
struct BackSmemOf<true>
{
    using type = BackSmemFuzzy;
};

// Position / camera gradients are left to point_backward_kernel in every mode.
template <bool kFuzzy, bool kBilinear>
__global__ void __launch_bounds__(kThreads, kFuzzy ? 1 : kMinCtas) backward_kernel(const __grid_constant__ Frame f,
                                                                                   const __grid_constant__ BackPtrs bp)
{
    static_assert(!(kFuzzy && kBilinear), "mode 2 and mode 3 exclude each other");
    using Smem = typename BackSmemOf<kFuzzy>::type;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    Smem& s = *reinterpret_cast<Smem*>(smem_raw);
    const int tid     = threadIdx.x;
    const int n_items = f.status[3];
    const float4 bgc  = make_float4(f.background[0], f.background[1], f.background[2], f.C > 3 ? f.background[3] : 0.f);
    float bg_acc[4] = {0.f, 0.f, 0.f, 0.f};
    float p0_acc    = 0.f;
    if (tid == 0) s.seg.n_long[0] = s.seg.n_long[1] = 0;
    int parity = 0;

    for (int item = blockIdx.x; item < n_items; item += gridDim.x)
    {
        int lo = f.item_start[item];
        const int hi = f.item_start[item + 1];
        if (lo >= hi) continue;
        lo += long_prefix(f, lo);
        if (lo >= hi) continue;
        {
            __syncthreads();  // every warp has left the previous item
            parity ^= 1;
            if (tid == 0) s.seg.n_long[parity ^ 1] = 0;
            const int f0 = list_end(f, lo - 1);
            const int np = hi - lo;
            if (tid < np)
            {
                const int ss = list_end(f, lo + tid - 1) - f0, se = f.ends[lo + tid] - f0;
                s.seg_end[tid + 1] = se;
                const PixInfo px   = decode_pixel(f, (unsigned)(lo + tid));
                s.pix[tid]         = px;
                s.grad[tid]        = px.valid ? load_grad(f, row_major_index(f, px)) : make_float4(0.f, 0.f, 0.f, 0.f);
                seg_fill(s.seg, parity, tid, ss, se);
            }
            if (tid == 0) s.seg_end[0] = 0;
            __syncthreads();
            const int nf = s.seg_end[np];
            for (int i = tid; i < nf; i += kThreads)
            {
                // Measured slower, both times through registers (spills, or one resident CTA less): requesting the next
                // record before working on this one; requesting the eight neighbour values together with the record.
                const uint4 h = f.recs[2 * (size_t)(f0 + i)], d = f.recs[2 * (size_t)(f0 + i) + 1];
                const int a = seg_lookup(s.seg, parity, s.seg_end, i);
                const bool blended = f.dbg_max_len <= 0 || i - s.seg_end[a] < f.dbg_max_len;  // list truncation
                if constexpr (kFuzzy)
                    fragment_stage_a<false>(f, s, lo + a, s.pix[a], s.grad[a], i, h, d, blended, s.desc, s.depth);
                else
                    fragment_stage_a<kBilinear>(f, s, lo + a, s.pix[a], s.grad[a], i, h, d, blended);
            }
            __syncthreads();
            if (tid < np && s.pix[tid].valid)
            {
                if constexpr (kFuzzy)
                    sweep_list_fuzzy(f, s.alpha, s.dot, s.trans, s.desc, s.depth, s.gv, s.gfirst, s.seg_end[tid], s.seg_end[tid + 1],
                                     s.grad[tid], bgc, bg_acc);
                else
                    sweep_list(f, s, s.seg_end[tid], s.seg_end[tid + 1], s.grad[tid], bgc, bg_acc, p0_acc);
            }
            __syncthreads();
            for (int i = tid; i < nf; i += kThreads)
            {
                const float Ti     = s.trans[i];
                const bool blended = Ti == Ti;  // NaN: the list ended before this fragment
                if (!kBilinear && !blended) continue;
                const int a = seg_lookup(s.seg, parity, s.seg_end, i);
                fragment_stage_b<kBilinear>(f, bp, s.pix[a], s.grad[a], s.pid[i], s.tex[i], Ti, s.dot[i], blended);
            }
        }
    }
    reduce_background(f, bp, s, bg_acc, p0_acc);
}

// Lists longer than kLongList: one CTA per list, blocks of kCap fragments, a forward sweep that records the
// transmittance at every block start and a backward sweep over the blocks that carries the suffix sum.
template <bool kBilinear>
__global__ void __launch_bounds__(kThreads) backward_long_kernel(const __grid_constant__ Frame f,
                                                                 const __grid_constant__ BackPtrs bp)
{
    if (f.status[2] <= kLongList) return;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    BackSmem& s = *reinterpret_cast<BackSmem*>(smem_raw);
    __shared__ float s_carry[4];      // {T, S, stop position}
    __shared__ float s_block_T[256];  // transmittance at block starts; lists beyond 256 * kCap fragments are cut there
    const int tid       = threadIdx.x;
    const int n_items   = f.status[3];
    constexpr bool bilinear = kBilinear;
    const float4 bgc    = make_float4(f.background[0], f.background[1], f.background[2], f.C > 3 ? f.background[3] : 0.f);
    float bg_acc[4] = {0.f, 0.f, 0.f, 0.f};
    float p0_acc    = 0.f;

    __shared__ int s_long_hits[kThreads], s_long_count;
    LongItemScan scan;
    int lo;
    while (scan.next(f, n_items, s_long_hits, &s_long_count, lo))
    {
        const int e0 = list_end(f, lo - 1);
        const int n  = f.ends[lo] - e0;
        const PixInfo px = decode_pixel(f, (unsigned)lo);
        __syncthreads();
        const float4 G = load_grad(f, row_major_index(f, px));
        int cnt = n;
        if (f.dbg_max_len > 0) cnt = min(cnt, f.dbg_max_len);
        cnt = min(cnt, 256 * kCap);
        const int n_blocks = (cnt + kCap - 1) / kCap;
        if (tid == 0) s_carry[0] = 1.f, s_carry[2] = (float)cnt;
        __syncthreads();
        // sweep 1: transmittance at block starts and the position where a mode-3 list stops
        for (int blk = 0; blk < n_blocks; ++blk)
        {
            const int m = min(kCap, cnt - blk * kCap);
            for (int i = tid; i < m; i += kThreads) s.alpha[i] = __uint_as_float(f.recs[2 * (size_t)(e0 + blk * kCap + i)].z);
            __syncthreads();
            if (tid == 0)
            {
                float T        = s_carry[0];
                s_block_T[blk] = T;
                int stop       = (int)s_carry[2];
                for (int i = 0; i < m && blk * kCap + i < stop; ++i)
                {
                    T = vetr_new_T(T, s.alpha[i]);
                    if (bilinear && T < 0.001f) stop = blk * kCap + i + 1;
                }
                s_carry[0] = T;
                s_carry[2] = (float)stop;
            }
            __syncthreads();
        }
        const int eff_cnt = (int)s_carry[2];
        const float T_end = s_carry[0];
        if (tid == 0)
        {
            const bool bg_term = !f.use_env && !(bilinear && !(T_end >= 0.001f));
            float S = 0.f;
            if (bg_term)
            {
                float dotb = dot4(bgc, G, f.C);
                bg_acc[0] += T_end * 1.f * G.x, bg_acc[1] += T_end * 1.f * G.y, bg_acc[2] += T_end * 1.f * G.z;
                if (f.C > 3) bg_acc[3] += T_end * 1.f * G.w;
                if (!bilinear && f.bg_alpha_to_point0) p0_acc += dotb * T_end;
                S = T_end * 1.f * dotb;
            }
            s_carry[1] = S;
        }
        __syncthreads();
        // sweep 2: blocks back to front
        for (int blk = (eff_cnt + kCap - 1) / kCap - 1; blk >= 0; --blk)
        {
            const int m = min(kCap, eff_cnt - blk * kCap);
            for (int i = tid; i < m; i += kThreads)
                fragment_stage_a<kBilinear>(f, s, lo, px, G, i, f.recs[2 * (size_t)(e0 + blk * kCap + i)],
                                            f.recs[2 * (size_t)(e0 + blk * kCap + i) + 1], true);
            __syncthreads();
            if (tid == 0)
            {
                float T = s_block_T[blk];
                for (int i = 0; i < m; ++i)
                {
                    s.trans[i] = T;
                    T          = vetr_new_T(T, s.alpha[i]);
                }
                float S = s_carry[1];
                for (int i = m - 1; i >= 0; --i)
                {
                    float a = s.alpha[i], Ti = s.trans[i], dt = s.dot[i];
                    s.dot[i]   = Ti * dt - S / (1 - a + 1e-9f);
                    s.trans[i] = Ti * a;
                    S += Ti * a * dt;
                }
                s_carry[1] = S;
            }
            __syncthreads();
            for (int i = tid; i < m; i += kThreads)
                fragment_stage_b<kBilinear>(f, bp, px, G, s.pid[i], s.tex[i], s.trans[i], s.dot[i], true);
            __syncthreads();
        }
        // fragments behind the cut take no part in the position gradient (mode 3: nor in the confidence gradient)
        if (kBilinear || f.need_point_grad)
            for (int i = eff_cnt + tid; i < n; i += kThreads)
            {
                const uint4 h = f.recs[2 * (size_t)(e0 + i)];
                if (kBilinear)
                    fragment_stage_b<kBilinear>(f, bp, px, G, (int)h.x, (int)h.w, 0.f, 0.f, false);
                else
                    f.point_grad[((size_t)px.view * f.L + px.level) * f.n + (int)h.x] = make_float2(__int_as_float(kNoGradientBits), 0.f);
            }
    }
    reduce_background(f, bp, s, bg_acc, p0_acc);
}

// Mode 2, lists longer than kLongList: one CTA per list with the whole list staged (the group structure does not split
// into blocks).  Lists beyond kFuzzyLongMax are skipped and flagged in the status word (the reference itself sorts only
// the first 4096 fragments of a list, AlphaListSort.cu:289-290, so its result for longer lists is not defined either).
constexpr int kFuzzyLongMax = 4096;  // what the reference sorts of a list (AlphaListSort.cu:289-290)
struct FuzzyLongSmem
{
    float4 desc[kFuzzyLongMax];
    int pid[kFuzzyLongMax];
    int tex[kFuzzyLongMax];
    float alpha[kFuzzyLongMax];
    float dot[kFuzzyLongMax];
    float trans[kFuzzyLongMax];
    float depth[kFuzzyLongMax];
    float gv[kFuzzyLongMax];
    unsigned char gfirst[kFuzzyLongMax];
};

__global__ void __launch_bounds__(kThreads) backward_fuzzy_long_kernel(const __grid_constant__ Frame f,
                                                                       const __grid_constant__ BackPtrs bp)
{
    if (f.status[2] <= kLongList) return;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    FuzzyLongSmem& s = *reinterpret_cast<FuzzyLongSmem*>(smem_raw);
    const int tid     = threadIdx.x;
    const int n_items = f.status[3];
    const float4 bgc  = make_float4(f.background[0], f.background[1], f.background[2], f.C > 3 ? f.background[3] : 0.f);
    float bg_acc[4] = {0.f, 0.f, 0.f, 0.f};
    __shared__ int s_long_hits[kThreads], s_long_count;
    LongItemScan scan;
    int lo;
    while (scan.next(f, n_items, s_long_hits, &s_long_count, lo))
    {
        const int e0 = list_end(f, lo - 1);
        const int n  = f.ends[lo] - e0;
        if (n > kFuzzyLongMax)
        {
            if (tid == 0) atomicOr(f.status + 1, 2);
            continue;
        }
        const PixInfo px = decode_pixel(f, (unsigned)lo);
        const float4 G = load_grad(f, row_major_index(f, px));
        __syncthreads();  // every warp has left the previous list
        const bool spatial = px.interior;
        for (int i = tid; i < n; i += kThreads)
        {
            const uint4 h  = f.recs[2 * (size_t)(e0 + i)];
            const float4 d = as_float4(f.recs[2 * (size_t)(e0 + i) + 1]);
            s.pid[i] = (int)h.x, s.tex[i] = (int)h.w, s.alpha[i] = __uint_as_float(h.z), s.depth[i] = __uint_as_float(h.y);
            s.desc[i] = d;
            const bool blended = f.dbg_max_len <= 0 || i < f.dbg_max_len;
            if (f.need_point_grad)
                f.point_grad[((size_t)px.view * f.L + px.level) * f.n + (int)h.x] =
                    spatial && blended ? neighbour_gradient(f, row_major_index(f, px), f.lw[px.level], d)
                                       : make_float2(__int_as_float(kNoGradientBits), 0.f);
        }
        __syncthreads();
        if (tid == 0) sweep_list_fuzzy(f, s.alpha, s.dot, s.trans, s.desc, s.depth, s.gv, s.gfirst, 0, n, G, bgc, bg_acc);
        __syncthreads();
        for (int i = tid; i < n; i += kThreads)
        {
            const float coef = s.trans[i];
            if (coef != coef) continue;
            red_add_v4(bp.g_desc + s.tex[i], make_float4(coef * G.x, coef * G.y, coef * G.z, f.C > 3 ? coef * G.w : 0.f));
            red_add(bp.g_conf + s.tex[i], s.dot[i]);
        }
    }
    if (tid == 0)
        for (int ci = 0; ci < f.C; ++ci)
            if (bg_acc[ci] != 0.f) atomicAdd(bp.g_background + ci, bg_acc[ci]);
}

// ---------------------------------------------------------------------------------------------------------
// Position, pose and intrinsics gradients (and the confidence gradient of mode 3), one pass over the points.
//
// Modes 1 and 2: every fragment's term is ProjectPointPinholeBackward of the image-space gradient that stage A parked
// for it.  Mode 3: the fragment's alpha gradient was parked under (view, level, point, corner); here the point is
// projected once per view exactly as the forward pass did (same bits), which gives the corner weights and their
// Jacobians (compute_blending_fac) of all its fragments: confidence gradient += w * g_alpha, image-space gradient =
// J_uv * confidence * g_alpha (RenderBackward.cu:3076-3180).  In every mode a fragment's term is evaluated with the
// arithmetic of the per-fragment form (each addend has the reference's bits); a point's terms are summed in registers
// in a fixed order and added to g_points by the one thread that owns the point.  Positions, masks and parked values are
// read coalesced; camera gradients are summed per thread block and view.

#ifndef VETR_POINT_BACK_POINTS
#    define VETR_POINT_BACK_POINTS 2
#endif
constexpr int kPointBackPoints = VETR_POINT_BACK_POINTS;

#ifndef VETR_POINT_BACK_CTAS
#    define VETR_POINT_BACK_CTAS 4
#endif
template <bool kIntr, bool kBilinear>
__global__ void __launch_bounds__(kProjThreads, VETR_POINT_BACK_CTAS) point_backward_kernel(const __grid_constant__ Frame f,
                                                                      const __grid_constant__ BackPtrs bp)
{
    __shared__ Camera s_cam[VETR_MAX_VIEWS];
    __shared__ double s_red[kProjThreads / 32][8];
    if (f.status[1] != 0) return;  // overflow / skipped list: some fragments never parked a value
    if (threadIdx.x < f.n_views) s_cam[threadIdx.x] = load_camera(f, threadIdx.x);
    __syncthreads();
    const int first     = blockIdx.x * (kProjThreads * kPointBackPoints) + threadIdx.x;
    const bool want_cam = bp.g_pose != nullptr || kIntr;
    const bool spatial  = f.need_point_grad != 0;
    float4 pos[kPointBackPoints], gp[kPointBackPoints];
#pragma unroll
    for (int it = 0; it < kPointBackPoints; ++it)
    {
        const int pid = first + it * kProjThreads;
        pos[it]       = pid < f.n ? __ldg(f.position + pid) : make_float4(0.f, 0.f, 0.f, 0.f);
        gp[it]        = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    for (int b = 0; b < f.n_views; ++b)
    {
        CamAcc<kIntr> acc;
        acc.clear();
        unsigned mask[kPointBackPoints];
#pragma unroll
        for (int it = 0; it < kPointBackPoints; ++it)
        {
            const int pid = first + it * kProjThreads;
            mask[it]      = pid < f.n ? f.level_mask[(size_t)b * f.n + pid] : 0u;
        }
        bool any = false;
#pragma unroll
        for (int it = 0; it < kPointBackPoints; ++it)
        {
            const int pid = first + it * kProjThreads;
            if (!mask[it]) continue;
            if constexpr (!kBilinear)
            {
                float2 dR[VETR_MAX_LAYERS];
#pragma unroll
                for (int l = 0; l < VETR_MAX_LAYERS; ++l)
                    if (mask[it] >> l & 1u) dR[l] = f.point_grad[((size_t)b * f.L + l) * f.n + pid];
                PointJac jac;
                if (!project_backward_prepare(pos[it], s_cam[b], f.dist_cutoff, kIntr, jac)) continue;
#pragma unroll
                for (int l = 0; l < VETR_MAX_LAYERS; ++l)
                {
                    if (!(mask[it] >> l & 1u) || __float_as_int(dR[l].x) == kNoGradientBits) continue;
                    BackOut bo;
                    spatial_terms<kIntr>(f, bp, s_cam[b], l, jac, dR[l], acc, bo);
                    gp[it].x += bo.g_point[0], gp[it].y += bo.g_point[1], gp[it].z += bo.g_point[2], gp[it].w += 1.f;
                    any = true;
                }
            }
            else
            {
                const float* parked = reinterpret_cast<const float*>(f.point_grad);
                float4 ga[VETR_MAX_LAYERS];  // the four corners' alpha gradients of every level
#pragma unroll
                for (int l = 0; l < VETR_MAX_LAYERS; ++l)
                    if (mask[it] >> l & 1u) ga[l] = *reinterpret_cast<const float4*>(parked + ((((size_t)b * f.L + l) * f.n + pid) << 2));
                const int tex    = __ldg(f.index + pid);
                const float conf = __ldg(f.confidence + tex);
                const Projected pr = project_point(pos[it], s_cam[b], f.dist_cutoff);
                PointJac jac;
                const bool jac_ok = spatial && project_backward_prepare(pos[it], s_cam[b], f.dist_cutoff, kIntr, jac);
                float2 ip   = pr.ip;
                float gconf = 0.f;
#pragma unroll
                for (int l = 0; l < VETR_MAX_LAYERS; ++l, ip.x *= 0.5f, ip.y *= 0.5f)
                {
                    if (!(mask[it] >> l & 1u)) continue;
                    const int bx = round_down(ip.x), by = round_down(ip.y);
                    const float gl[4] = {ga[l].x, ga[l].y, ga[l].z, ga[l].w};
#pragma unroll
                    for (int c = 0; c < 4; ++c)
                    {
                        // the same in-image test as the collection pass: corners outside never became fragments
                        const int x = bx + (c & 1), y = by + (c >> 1);
                        if ((unsigned)x >= (unsigned)f.lw[l] || (unsigned)y >= (unsigned)f.lh[l]) continue;
                        if (__float_as_int(gl[c]) == kNoGradientBits) continue;
                        float jx, jy;
                        const float w = blending_fac(ip, c, &jx, &jy);
                        gconf += w * gl[c];  // RenderBackward.cu:3076-3079
                        if (!jac_ok) continue;
                        const float single = conf * gl[c];
                        BackOut bo;
                        spatial_terms<kIntr>(f, bp, s_cam[b], l, jac, make_float2(jx * single, jy * single), acc, bo);
                        gp[it].x += bo.g_point[0], gp[it].y += bo.g_point[1], gp[it].z += bo.g_point[2], gp[it].w += 1.f;
                        any = true;
                    }
                }
                if (gconf != 0.f) red_add(bp.g_conf + tex, gconf);
            }
        }
        if (want_cam && __syncthreads_or(any)) reduce_cam<kIntr>(f, bp, acc, b, s_red);
    }
    if (bp.g_points)
    {
#pragma unroll
        for (int it = 0; it < kPointBackPoints; ++it)
        {
            const int pid = first + it * kProjThreads;
            if (pid < f.n && gp[it].w != 0.f)
            {
                float4 cur = bp.g_points[pid];
                cur.x += gp[it].x, cur.y += gp[it].y, cur.z += gp[it].z, cur.w += gp[it].w;
                bp.g_points[pid] = cur;
            }
        }
    }
}

// ---------------------------------------------------------------------------------------------------------
// Mode 0 (FUZZY_DT): no lists.  Per pixel: nearest depth (int bits, in `ends`), accumulators in the fragment buffer
// (record g: float4 descriptor sum, then the number of accepted points as a float), count of accepted points (`counts`).

// Mode 0 reads the caller's planar images directly (its backward pass is point-parallel: one fragment per point).
__device__ __forceinline__ float2 neighbour_gradient_planar(const Frame& f, const BackPtrs& bp, const PixInfo& px, float4 d)
{
    const int w = f.lw[px.level], h = f.lh[px.level];
    const int hw = w * h;
    const int o  = (px.view * f.C) * hw + px.y * w + px.x;
    const float* I  = bp.out_color[px.level] + o;
    const float* Gp = bp.grad_color[px.level] + o;
    float dx = 0.f, dy = 0.f;
    const float dv[4] = {d.x, d.y, d.z, d.w};
#pragma unroll
    for (int ci = 0; ci < 4; ++ci)
    {
        if (ci < f.C)
        {
            const float* Ic = I + ci * hw;
            const float* Gc = Gp + ci * hw;
            float Tp = dv[ci];
            float a0 = -(Tp - __ldg(Ic - 1)) * __ldg(Gc - 1);
            float a1 = (Tp - __ldg(Ic + 1)) * __ldg(Gc + 1);
            float b0 = -(Tp - __ldg(Ic - w)) * __ldg(Gc - w);
            float b1 = (Tp - __ldg(Ic + w)) * __ldg(Gc + w);
            dx += 0.5f * (a0 + a1);
            dy += 0.5f * (b0 + b1);
        }
    }
    return make_float2(dx / (float)f.C, dy / (float)f.C);
}

__device__ __forceinline__ float4 load_grad_planar(const Frame& f, const BackPtrs& bp, const PixInfo& px)
{
    const int w = f.lw[px.level], h = f.lh[px.level];
    const int hw = w * h;
    const float* G = bp.grad_color[px.level] + (px.view * f.C) * hw + px.y * w + px.x;
    float4 g;
    g.x = __ldg(G);
    g.y = __ldg(G + hw);
    g.z = __ldg(G + 2 * hw);
    g.w = f.C > 3 ? __ldg(G + 3 * hw) : 0.f;
    return g;
}

__global__ void fill_int_kernel(int* p, int v, long long n)
{
    long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) p[i] = v;
}

// kPass 0: DepthPrepassMulti (RenderForward.cu:180-308; no drop-out test).  kPass 1: RenderForwardMulti (:312-406).
template <int kPass>
__global__ void __launch_bounds__(kProjThreads) fuzzy_dt_point_kernel(const __grid_constant__ Frame f)
{
    __shared__ Camera s_cam;
    const int b = blockIdx.y;
    if (threadIdx.x == 0) s_cam = load_camera(f, b);
    __syncthreads();
    const Camera& cam = s_cam;
    const int vbase   = b * (int)f.P;
    const int pid     = blockIdx.x * kProjThreads + threadIdx.x;
    if (pid >= f.n) return;
    const int tex = __ldg(f.index + pid);
    if (f.viewer_only && f.confidence[tex] < f.stability_cutoff) return;
    if (kPass == 1 && f.dropout && f.dropout[(size_t)b * f.n + pid] == 1.f) return;
    const Projected pr = project_point(__ldg(f.position + pid), cam, f.dist_cutoff);
    if (pr.z == 0.f) return;
    float2 ip    = pr.ip;
    float radius = pr.radius_px;
    float4 desc  = make_float4(0.f, 0.f, 0.f, 0.f);
    if (kPass == 1)
    {
        desc.x = __ldg(f.texture + tex);
        desc.y = __ldg(f.texture + (size_t)f.n_tex + tex);
        desc.z = __ldg(f.texture + 2 * (size_t)f.n_tex + tex);
        desc.w = f.C > 3 ? __ldg(f.texture + 3 * (size_t)f.n_tex + tex) : 0.f;
    }
    for (int l = 0; l < f.L; ++l, radius *= 0.5f, ip.x *= 0.5f, ip.y *= 0.5f)
    {
        if (f.drop_by_radius && radius < f.radius_threshold) break;
        const int lw = f.lw[l], lh = f.lh[l];
        const int x = round_half_even(ip.x), y = round_half_even(ip.y);
        if ((unsigned)x >= (unsigned)lw || (unsigned)y >= (unsigned)lh) continue;
        const int g = vbase + (int)f.lbase[l] + pixel_offset(lw, x, y);
        if (kPass == 0)
            atomicMin(f.ends + g, __float_as_int(pr.z));  // z > 0: integer order = float order
        else
        {
            const float image_depth = __int_as_float(f.ends[g]);
            if (pr.z > image_depth * (f.depth_accept + 1)) continue;
            red_add_v4(reinterpret_cast<float4*>(f.recs + 2 * (size_t)g), desc);
            red_add(reinterpret_cast<float*>(f.recs + 2 * (size_t)g + 1), 1.f);
        }
    }
}

// CombineAndFill (PointRenderer.cu:24-52) + CreateMask + depth output, one thread per pixel of the pixel space.
__global__ void __launch_bounds__(256) fuzzy_dt_combine_kernel(const __grid_constant__ Frame f, const __grid_constant__ OutPtrs out)
{
    __shared__ int s_sum[8], s_max[8];
    const long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    int n_acc = 0;
    if (g < f.PT)
    {
        const float4 acc = as_float4(f.recs[2 * (size_t)g]);
        const float w    = __uint_as_float(f.recs[2 * (size_t)g + 1].x);
        n_acc            = (int)w;
        f.counts[g]      = n_acc;
        float c[4];
        if (w == 0.f)
            c[0] = f.background[0], c[1] = f.background[1], c[2] = f.background[2], c[3] = f.C > 3 ? f.background[3] : 0.f;
        else
            c[0] = acc.x / w, c[1] = acc.y / w, c[2] = acc.z / w, c[3] = acc.w / w;
        write_pixel(f, out, (unsigned)g, c, w, __int_as_float(f.ends[g]));
    }
    int sum = n_acc, mx = n_acc;
    for (int o = 16; o > 0; o >>= 1)
    {
        sum += __shfl_down_sync(0xffffffffu, sum, o);
        mx = max(mx, __shfl_down_sync(0xffffffffu, mx, o));
    }
    if ((threadIdx.x & 31) == 0) s_sum[threadIdx.x >> 5] = sum, s_max[threadIdx.x >> 5] = mx;
    __syncthreads();
    if (threadIdx.x == 0)
    {
        for (int i = 1; i < 8; ++i) sum += s_sum[i], mx = max(mx, s_max[i]);
        if (sum) atomicAdd(f.status + 0, sum);
        if (mx) atomicMax(f.status + 2, mx);
    }
}

// CombineAndFillBackward (RenderBackward.cu:27-76): the background colour receives the gradient of every empty pixel.
__global__ void __launch_bounds__(256) fuzzy_dt_background_kernel(const __grid_constant__ Frame f,
                                                                   const __grid_constant__ BackPtrs bp)
{
    __shared__ float s_red[8][4];
    float v[4] = {0.f, 0.f, 0.f, 0.f};
    for (long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x; g < f.PT; g += (long long)gridDim.x * blockDim.x)
        if (f.counts[g] == 0)
        {
            const PixInfo px = decode_pixel(f, (unsigned)g);
            if (!px.valid) continue;
            const float4 G = load_grad_planar(f, bp, px);
            v[0] += G.x, v[1] += G.y, v[2] += G.z, v[3] += G.w;
        }
    for (int k = 0; k < 4; ++k)
    {
        float x = v[k];
        for (int o = 16; o > 0; o >>= 1) x += __shfl_down_sync(0xffffffffu, x, o);
        if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5][k] = x;
    }
    __syncthreads();
    if ((int)threadIdx.x < f.C)
    {
        float x = 0.f;
        for (int w = 0; w < 8; ++w) x += s_red[w][threadIdx.x];
        if (x != 0.f) atomicAdd(bp.g_background + threadIdx.x, x);
    }
}

// RenderBackward (RenderBackward.cu:131-474): one thread per point and view.  Pixel positions come from the backward's own
// copy of the projection, which leaves out the crop rotation (RenderBackward.cu:78-116).
template <bool kIntr>
__global__ void __launch_bounds__(kProjThreads) fuzzy_dt_backward_kernel(const __grid_constant__ Frame f,
                                                                         const __grid_constant__ BackPtrs bp)
{
    __shared__ Camera s_cam;
    __shared__ double s_red[kProjThreads / 32][8];
    const int b = blockIdx.y;
    if (threadIdx.x == 0) s_cam = load_camera(f, b);
    __syncthreads();
    const Camera& cam = s_cam;
    const int vbase   = b * (int)f.P;
    const int pid     = blockIdx.x * kProjThreads + threadIdx.x;
    CamAcc<kIntr> acc;
    acc.clear();
    if (pid < f.n)
    {
        const bool drop_out = f.dropout && f.dropout[(size_t)b * f.n + pid] == 1.f;
        const float4 pos    = __ldg(f.position + pid);
        const Projected pr  = project_point(pos, cam, f.dist_cutoff, false);
        if (pr.z != 0.f)
        {
            const int tex = __ldg(f.index + pid);
            float2 ip     = pr.ip;
            float radius  = pr.radius_px;
            for (int l = 0; l < f.L; ++l, radius *= 0.5f, ip.x *= 0.5f, ip.y *= 0.5f)
            {
                if (f.drop_by_radius && radius < f.radius_threshold) continue;
                const int lw = f.lw[l], lh = f.lh[l];
                const int x = round_half_even(ip.x), y = round_half_even(ip.y);
                if ((unsigned)x >= (unsigned)lw || (unsigned)y >= (unsigned)lh) continue;
                const int g   = vbase + (int)f.lbase[l] + pixel_offset(lw, x, y);
                const float w = (float)f.counts[g];
                if (w == 0.f) continue;
                if (pr.z > __int_as_float(f.ends[g]) * (f.depth_accept + 1)) continue;
                PixInfo px;
                px.x = (short)x, px.y = (short)y, px.level = (unsigned char)l, px.view = (unsigned char)b, px.valid = 1;
                px.interior = min(min(x, f.lw[l] - 1 - x), min(y, f.lh[l] - 1 - y)) > 2;
                if (!drop_out)
                {
                    const float iw = 1.f / w;
                    const float4 G = load_grad_planar(f, bp, px);
                    red_add_v4(bp.g_desc + tex, make_float4(iw * G.x, iw * G.y, iw * G.z, f.C > 3 ? iw * G.w : 0.f));
                }
                const bool point_grad = (f.ghost && drop_out) | (!f.ghost && !drop_out);
                if (!(point_grad && px.interior)) continue;
                spatial_backward<kIntr>(f, bp, cam, px, pid, pos, neighbour_gradient_planar(f, bp, px, load_descriptor(f, tex)), acc);
            }
        }
    }
    if (bp.g_pose != nullptr || kIntr) reduce_cam<kIntr>(f, bp, acc, b, s_red);
}

// ---------------------------------------------------------------------------------------------------------
// Epilogues.

__global__ void transpose_desc_kernel(const float4* __restrict__ g_desc, float* __restrict__ g_texture, int n_tex, int C)
{
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n_tex) return;
    float4 v = g_desc[i];
    g_texture[i] = v.x;
    g_texture[(long long)n_tex + i] = v.y;
    g_texture[2LL * n_tex + i] = v.z;
    if (C > 3) g_texture[3LL * n_tex + i] = v.w;
}

// NormalizeGradient for points (PointRenderer.cu:1273-1280): divide by the hit count where it is positive.
__global__ void normalize_points_kernel(float4* g_points, float* g_count, int n)
{
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float4 v = g_points[i];
    float c  = v.w;
    if (g_count) g_count[i] = c;
    if (c > 0) v.x = v.x / c, v.y = v.y / c, v.z = v.z / c;
    v.w         = 0.f;
    g_points[i] = v;
}

template <typename T, int N>
__global__ void normalize_rows_kernel(T* g, const float* count, int n)  // NormalizeGradientDevTensor, :1092-1109
{
    int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    float c = count[i];
    if (c > 0)
        for (int k = 0; k < N; ++k) g[(long long)i * N + k] = g[(long long)i * N + k] / c;
}

// ApplyTangent (PointRenderer.cu:1325-1341): pose <- exp_se3(t) * pose in double; tangent = (translation, rotation).
__global__ void apply_tangent_kernel(double* tangent, double* poses, int n)
{
    int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n) return;
    double* t = tangent + 6 * idx;
    double* p = poses + 8 * idx;
    double ux = t[0], uy = t[1], uz = t[2], wx = t[3], wy = t[4], wz = t[5];
    double th2 = wx * wx + wy * wy + wz * wz, th = sqrt(th2);
    double imag, real, a, bb;
    if (th < 1e-10)
    {
        double th4 = th2 * th2;
        imag = 0.5 - th2 / 48.0 + th4 / 3840.0;
        real = 1.0 - th2 / 8.0 + th4 / 384.0;
        a    = 0.5;
        bb   = 1.0 / 6.0;
    }
    else
    {
        imag = sin(0.5 * th) / th;
        real = cos(0.5 * th);
        a    = (1 - cos(th)) / th2;
        bb   = (th - sin(th)) / (th2 * th);
    }
    double x1 = imag * wx, y1 = imag * wy, z1 = imag * wz, w1 = real;
    double O[9] = {0, -wz, wy, wz, 0, -wx, -wy, wx, 0};
    double u[3] = {ux, uy, uz}, te[3];
    for (int r = 0; r < 3; ++r)
    {
        te[r] = u[r];
        for (int c = 0; c < 3; ++c)
        {
            double o2 = O[3 * r] * O[c] + O[3 * r + 1] * O[3 + c] + O[3 * r + 2] * O[6 + c];
            te[r] += (a * O[3 * r + c] + bb * o2) * u[c];
        }
    }
    double x2 = p[0], y2 = p[1], z2 = p[2], w2 = p[3];
    double q[4] = {w1 * x2 + x1 * w2 + y1 * z2 - z1 * y2, w1 * y2 - x1 * z2 + y1 * w2 + z1 * x2,
                   w1 * z2 + x1 * y2 - y1 * x2 + z1 * w2, w1 * w2 - x1 * x2 - y1 * y2 - z1 * z2};
    double nrm = sqrt(q[0] * q[0] + q[1] * q[1] + q[2] * q[2] + q[3] * q[3]);
    double tp[3] = {p[4], p[5], p[6]};
    double cx = y1 * tp[2] - z1 * tp[1], cy = z1 * tp[0] - x1 * tp[2], cz = x1 * tp[1] - y1 * tp[0];
    cx *= 2, cy *= 2, cz *= 2;
    double rx = tp[0] + w1 * cx + (y1 * cz - z1 * cy);
    double ry = tp[1] + w1 * cy + (z1 * cx - x1 * cz);
    double rz = tp[2] + w1 * cz + (x1 * cy - y1 * cx);
    for (int k = 0; k < 4; ++k) p[k] = q[k] / nrm;
    p[4] = rx + te[0], p[5] = ry + te[1], p[6] = rz + te[2];
    for (int k = 0; k < 6; ++k) t[k] = 0.0;
}

// ---------------------------------------------------------------------------------------------------------
// Multi-GPU epilogue: sum of the raw gradient buffers of all ranks + the count normalisation + the channel-major
// transpose, in one kernel over peer memory.  Every rank owns one contiguous slice of each of the three segments
// (descriptor, position, confidence gradients): it reads that slice from every rank's raw buffer (peer loads over
// NVLink, summed in rank order, so every rank ends up with the same bits), finalises it and stores the result into
// every rank's output buffer (peer stores).  The kernel waits on nothing: the caller orders it after the backward
// kernels of ALL ranks and orders the consumers after the exchange kernels of ALL ranks (a collective on the same
// stream before and after, e.g. the all-reduce of the pose gradients and of their counts).

struct ExchangeArgs
{
    int rank, world, C, n_tex, n;
    long long out_points, out_conf;  // float offsets of the position / confidence segments in the output buffers
    const float* raw[VETR_MAX_RANKS];
    float* out[VETR_MAX_RANKS];
    const float* raw_mc;  // multicast address of the raw buffers (NVLink SHARP), or nullptr
    float* out_mc;        // multicast address of the output buffers
    int segments;         // VETR_SEG_* bits: which of the three segments this launch handles
};

__device__ __forceinline__ void slice_of(long long count, int rank, int world, long long& lo, long long& hi)
{
    lo = count * rank / world;
    hi = count * (rank + 1) / world;
}

// Every access is 16 bytes per lane and contiguous across a warp: few large requests cross a link (and the switch)
// faster than many small ones.  kMulticast: the accesses go through the NVSwitch multicast object that spans all
// ranks' buffers - multimem.ld_reduce returns the sum over the ranks of one address (the switch fetches and adds),
// multimem.st stores to all ranks at once - so the SM issues 1/world of the loads and stores.

__device__ __forceinline__ float4 add4(float4 a, float4 b) { return make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w); }

// sum over the ranks of the float4 at float offset `at` of the raw buffers (rank order 0, 1, ... in the plain form)
template <bool kMulticast>
__device__ __forceinline__ float4 rank_sum4(const ExchangeArgs& a, long long at)
{
    if constexpr (kMulticast)
    {
        float4 v;
        asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                     : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w)
                     : "l"(a.raw_mc + at)
                     : "memory");
        return v;
    }
    else
    {
        float4 v = __ldcg(reinterpret_cast<const float4*>(a.raw[0] + at));
        for (int k = 1; k < a.world; ++k) v = add4(v, __ldcg(reinterpret_cast<const float4*>(a.raw[k] + at)));
        return v;
    }
}

// store one float4 at float offset `at` of every rank's output buffer
template <bool kMulticast>
__device__ __forceinline__ void rank_store4(const ExchangeArgs& a, long long at, float4 v)
{
    if constexpr (kMulticast)
        asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(a.out_mc + at), "f"(v.x), "f"(v.y),
                     "f"(v.z), "f"(v.w)
                     : "memory");
    else
        for (int k = 0; k < a.world; ++k) *reinterpret_cast<float4*>(a.out[k] + at) = v;
}

// scalar forms for the few elements that do not fill a 16-byte group (plain peer accesses in both variants)
__device__ __forceinline__ float rank_sum1(const ExchangeArgs& a, long long at)
{
    float v = __ldcg(a.raw[0] + at);
    for (int k = 1; k < a.world; ++k) v += __ldcg(a.raw[k] + at);
    return v;
}
__device__ __forceinline__ void rank_store1(const ExchangeArgs& a, long long at, float v)
{
    for (int k = 0; k < a.world; ++k) a.out[k][at] = v;
}

constexpr int kExchangeWarps = 8;

template <bool kMulticast>
__global__ void __launch_bounds__(32 * kExchangeWarps) exchange_finalize_kernel(const __grid_constant__ ExchangeArgs a)
{
    __shared__ float4 s_tile[kExchangeWarps][2][32];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const long long gtid    = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long stride  = (long long)gridDim.x * blockDim.x;
    const long long gwarp   = (long long)blockIdx.x * kExchangeWarps + warp;
    const long long n_warps = (long long)gridDim.x * kExchangeWarps;
    const long long n_tex   = a.n_tex;
    const long long raw_points = 4 * n_tex, raw_conf = 4 * n_tex + 4LL * a.n;
    long long lo, hi;

    // descriptor gradient [n_tex] float4 -> texture gradient [C, n_tex].  A warp takes 32 texels (one coalesced float4
    // load per lane), turns them by 90 degrees in shared memory and stores 4 texels x 1 channel per lane, i.e. a
    // 128-byte run in each channel row.  Rows start at c * n_tex floats: 16-byte aligned only if n_tex % 4 == 0.
    const long long tiles = (n_tex & 3) == 0 ? n_tex / 32 : 0;
    slice_of(tiles, a.rank, a.world, lo, hi);
    if (!(a.segments & VETR_SEG_DESC)) hi = lo;
    const int c = lane >> 3, q = lane & 7;
    for (long long tile = lo + gwarp; tile < hi; tile += 2 * n_warps)
    {
        const bool second = tile + n_warps < hi;
        const float4 v0 = rank_sum4<kMulticast>(a, 4 * (tile * 32 + lane));
        float4 v1       = make_float4(0.f, 0.f, 0.f, 0.f);
        if (second) v1 = rank_sum4<kMulticast>(a, 4 * ((tile + n_warps) * 32 + lane));
        s_tile[warp][0][lane] = v0;
        s_tile[warp][1][lane] = v1;
        __syncwarp();
#pragma unroll
        for (int u = 0; u < 2; ++u)
        {
            if (u == 1 && !second) break;
            const float* tf = reinterpret_cast<const float*>(s_tile[warp][u]);
            const float4 o  = make_float4(tf[(4 * q) * 4 + c], tf[(4 * q + 1) * 4 + c], tf[(4 * q + 2) * 4 + c], tf[(4 * q + 3) * 4 + c]);
            if (c < a.C) rank_store4<kMulticast>(a, c * n_tex + (tile + u * n_warps) * 32 + 4 * q, o);
        }
        __syncwarp();
    }
    // texels that do not fill a tile (all of them if the rows are not 16-byte aligned), one by one
    {
        const long long first = tiles * 32;
        slice_of(n_tex - first, a.rank, a.world, lo, hi);
        if (!(a.segments & VETR_SEG_DESC)) hi = lo;
        for (long long t = first + lo + gtid; t < first + hi; t += stride)
        {
            const float4 v = rank_sum4<false>(a, 4 * t);
            rank_store1(a, t, v.x), rank_store1(a, n_tex + t, v.y), rank_store1(a, 2 * n_tex + t, v.z);
            if (a.C > 3) rank_store1(a, 3 * n_tex + t, v.w);
        }
    }

    // position gradient sums with the hit count in .w -> average (NormalizeGradient, PointRenderer.cu:1273-1280)
    slice_of(a.n, a.rank, a.world, lo, hi);
    if (!(a.segments & VETR_SEG_POINTS)) hi = lo;
    for (long long base = lo + gtid; base < hi; base += stride * 4)
    {
        float4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
            if (base + u * stride < hi) v[u] = rank_sum4<kMulticast>(a, raw_points + 4 * (base + u * stride));
#pragma unroll
        for (int u = 0; u < 4; ++u)
        {
            if (base + u * stride >= hi) continue;
            float4 r = v[u];
            if (r.w > 0) r.x = r.x / r.w, r.y = r.y / r.w, r.z = r.z / r.w;
            r.w = 0.f;
            rank_store4<kMulticast>(a, a.out_points + 4 * (base + u * stride), r);
        }
    }

    // confidence gradient, four texels per access (every segment offset is a multiple of 4 floats); the last rank also
    // takes the n_tex % 4 texels that are left over
    const long long groups = n_tex / 4;
    slice_of(groups, a.rank, a.world, lo, hi);
    if (!(a.segments & VETR_SEG_CONF)) hi = lo;
    for (long long base = lo + gtid; base < hi; base += stride * 4)
    {
        float4 v[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
            if (base + u * stride < hi) v[u] = rank_sum4<kMulticast>(a, raw_conf + 4 * (base + u * stride));
#pragma unroll
        for (int u = 0; u < 4; ++u)
            if (base + u * stride < hi) rank_store4<kMulticast>(a, a.out_conf + 4 * (base + u * stride), v[u]);
    }
    if (a.rank == a.world - 1 && (a.segments & VETR_SEG_CONF))
        for (long long t = 4 * groups + gtid; t < n_tex; t += stride) rank_store1(a, a.out_conf + t, rank_sum1(a, raw_conf + t));
    __threadfence_system();  // the peer stores are performed before the kernel counts as finished
}

// ---------------------------------------------------------------------------------------------------------
// Error-grid rasterisation (FillSceneGridWithLossRasterize, RenderForward.cu:639-791): the step between a training
// epoch and the point spawning.  One warp per grid cell: eight lanes project the corners of the cell's box, all lanes
// walk the pixels of its screen rectangle (32-pixel border excluded), test them against the twelve triangles of the
// box and add up the L1 loss.  The reference issues two global atomics per covered pixel; here a lane sums in
// registers and the warp adds once per cell.

struct GridArgs
{
    const float* bb_min;
    const float* bb_len;
    const float* loss;
    float* value;
    int* count;
    int n_cells, channels, h, w, view;
};

__device__ __forceinline__ float tri_sign(float2 p1, float2 p2, float2 p3)
{
    return VS(VM(VS(p1.x, p3.x), VS(p2.y, p3.y)), VM(VS(p2.x, p3.x), VS(p1.y, p3.y)));
}
__device__ __forceinline__ bool point_in_triangle(float2 pt, float2 v1, float2 v2, float2 v3)
{
    const float d1 = tri_sign(pt, v1, v2), d2 = tri_sign(pt, v2, v3), d3 = tri_sign(pt, v3, v1);
    const bool has_neg = (d1 < 0) || (d2 < 0) || (d3 < 0);
    const bool has_pos = (d1 > 0) || (d2 > 0) || (d3 > 0);
    return !(has_neg && has_pos);
}

constexpr int kGridWarps = 4;
constexpr int kGridChunk = 4096;             // pixels of a cell's screen rectangle one warp walks
constexpr int kGridQueueCap = 4 * 1024 * 1024;  // (cell, chunk) pairs handed to the second kernel

// Screen rectangle of a cell: the eight projected corners (left in pp[]) and the clamped bounding rectangle.
// Returns the number of pixels to test (0: cell ignored).  Called by a whole warp; s_pp is the warp's staging row.
__device__ __forceinline__ long long grid_cell_rectangle(const Frame& f, const GridArgs& a, const Camera& cam, int c, int lane,
                                                         float2* s_pp, float2 pp[8], float2& mn, int& x_size)
{
    const float border = 32.f;
    bool behind = false;
    if (lane < 8)
    {
        // corner order of the reference: (0,0,0) (1,0,0) (0,1,0) (0,0,1) (1,1,0) (1,0,1) (0,1,1) (1,1,1)
        const float fx = (lane == 1 || lane == 4 || lane == 5 || lane == 7) ? 1.f : 0.f;
        const float fy = (lane == 2 || lane == 4 || lane == 6 || lane == 7) ? 1.f : 0.f;
        const float fz = (lane == 3 || lane == 5 || lane == 6 || lane == 7) ? 1.f : 0.f;
        const float4 pos = make_float4(VA(a.bb_min[3 * c], VM(a.bb_len[3 * c], fx)), VA(a.bb_min[3 * c + 1], VM(a.bb_len[3 * c + 1], fy)),
                                       VA(a.bb_min[3 * c + 2], VM(a.bb_len[3 * c + 2], fz)), 0.f);
        const Projected pr = project_point(pos, cam, f.dist_cutoff);
        behind      = pr.z <= 0.f;  // one corner behind the camera: the whole cell is ignored
        s_pp[lane]  = pr.ip;
    }
    behind = __any_sync(0xffffffffu, behind);
    __syncwarp();
#pragma unroll
    for (int i = 0; i < 8; ++i) pp[i] = s_pp[i];
    __syncwarp();  // the staging row is free for the warp's next cell
    if (behind) return 0;
    float2 mx = make_float2(-10000000.f, -10000000.f);
    mn        = make_float2(10000000.f, 10000000.f);
#pragma unroll
    for (int i = 0; i < 8; ++i)
    {
        mx.x = fmaxf(pp[i].x, mx.x), mx.y = fmaxf(pp[i].y, mx.y);
        mn.x = fminf(pp[i].x, mn.x), mn.y = fminf(pp[i].y, mn.y);
    }
    const float W = (float)a.w, H = (float)a.h;
    if (mx.x < border || mn.x >= VS(W, border) || mx.y < border || mn.y >= VS(H, border)) return 0;
    mn.x = fmaxf(mn.x, border), mn.y = fmaxf(mn.y, border);
    mx.x = fminf(mx.x, VS(W, border)), mx.y = fminf(mx.y, VS(H, border));
    const int y_size = (int)VS(mx.y, mn.y);
    x_size           = (int)VS(mx.x, mn.x);
    return (long long)y_size * x_size;
}

// Pixels [first, last) of a cell's rectangle, one per lane and step; adds the warp's totals to the cell.
__device__ __forceinline__ void grid_cell_pixels(const GridArgs& a, int c, int lane, const float2 pp[8], float2 mn, int x_size,
                                                 long long first, long long last)
{
    float sum = 0.f;
    int hits  = 0;
    for (long long xy = first + lane; xy < last; xy += 32)
    {
        const int x_c = (int)VA((float)(int)(xy % x_size), mn.x);
        const int y_c = (int)VA((float)(int)(xy / x_size), mn.y);
        const float2 pt = make_float2((float)x_c, (float)y_c);
        bool in = false;
        // faces of the box as pairs of triangles (RenderForward.cu:676-677)
        in |= point_in_triangle(pt, pp[0], pp[1], pp[4]) || point_in_triangle(pt, pp[0], pp[4], pp[2]);
        in |= point_in_triangle(pt, pp[1], pp[5], pp[7]) || point_in_triangle(pt, pp[1], pp[7], pp[4]);
        in |= point_in_triangle(pt, pp[5], pp[3], pp[6]) || point_in_triangle(pt, pp[5], pp[6], pp[7]);
        in |= point_in_triangle(pt, pp[3], pp[0], pp[6]) || point_in_triangle(pt, pp[0], pp[6], pp[2]);
        in |= point_in_triangle(pt, pp[3], pp[0], pp[5]) || point_in_triangle(pt, pp[0], pp[5], pp[1]);
        in |= point_in_triangle(pt, pp[2], pp[4], pp[6]) || point_in_triangle(pt, pp[4], pp[6], pp[7]);
        if (!in) continue;
        float g = 0.f;
        for (int i = 0; i < a.channels; ++i) g += fabsf(__ldg(a.loss + ((long long)i * a.h + y_c) * a.w + x_c));
        sum += g;
        ++hits;
    }
    for (int o = 16; o > 0; o >>= 1)
    {
        sum += __shfl_down_sync(0xffffffffu, sum, o);
        hits += __shfl_down_sync(0xffffffffu, hits, o);
    }
    if (lane == 0 && hits > 0)
    {
        atomicAdd(a.value + c, sum);
        atomicAdd(a.count + c, hits);
    }
}

// First kernel: one warp per cell.  Rectangles of up to kGridChunk pixels are walked right away; larger ones (a cell next
// to the camera covers 10^5 pixels, a distant one 10) are cut into chunks that go to a queue, so that the second kernel
// can spread them over all SMs.  If the queue is full the warp walks the whole rectangle itself.
__global__ void __launch_bounds__(32 * kGridWarps) grid_loss_kernel(const __grid_constant__ Frame f, const __grid_constant__ GridArgs a,
                                                                     int2* queue, int* queue_count)
{
    __shared__ Camera s_cam;
    __shared__ float2 s_pp[kGridWarps][8];
    if (threadIdx.x == 0) s_cam = load_camera(f, a.view);
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int c = blockIdx.x * kGridWarps + warp; c < a.n_cells; c += gridDim.x * kGridWarps)
    {
        float2 pp[8], mn;
        int x_size;
        const long long total = grid_cell_rectangle(f, a, s_cam, c, lane, s_pp[warp], pp, mn, x_size);
        if (total <= 0) continue;
        if (total > kGridChunk)
        {
            const int chunks = (int)((total + kGridChunk - 1) / kGridChunk);
            int base = 0;
            if (lane == 0) base = atomicAdd(queue_count, chunks);
            base = __shfl_sync(0xffffffffu, base, 0);
            if (base + chunks <= kGridQueueCap)
            {
                for (int k = lane; k < chunks; k += 32) queue[base + k] = make_int2(c, k);
                continue;
            }
            // no room for all chunks: whatever part of the reservation lies inside the queue is marked unused, and the warp
            // walks the whole rectangle itself
            for (int k = lane; k < chunks && base + k < kGridQueueCap; k += 32) queue[base + k] = make_int2(-1, 0);
        }
        grid_cell_pixels(a, c, lane, pp, mn, x_size, 0, total);
    }
}

// Second kernel: one warp per queued (cell, chunk).
__global__ void __launch_bounds__(32 * kGridWarps) grid_loss_chunk_kernel(const __grid_constant__ Frame f, const __grid_constant__ GridArgs a,
                                                                           const int2* queue, const int* queue_count)
{
    __shared__ Camera s_cam;
    __shared__ float2 s_pp[kGridWarps][8];
    if (threadIdx.x == 0) s_cam = load_camera(f, a.view);
    __syncthreads();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    // reservations past the capacity were never written: those cells were walked by the first kernel
    const int n = min(*queue_count, kGridQueueCap);
    for (int e = blockIdx.x * kGridWarps + warp; e < n; e += gridDim.x * kGridWarps)
    {
        const int2 q = queue[e];
        if (q.x < 0) continue;
        float2 pp[8], mn;
        int x_size;
        const long long total = grid_cell_rectangle(f, a, s_cam, q.x, lane, s_pp[warp], pp, mn, x_size);
        const long long first = (long long)q.y * kGridChunk;
        grid_cell_pixels(a, q.x, lane, pp, mn, x_size, first, min(first + kGridChunk, total));
    }
}

// ---------------------------------------------------------------------------------------------------------
// L1 loss of the whole output pyramid against a target pyramid and its gradient, in one launch (what a training step
// does between the forward and the backward pass; with library element-wise kernels it is seven launches per level).

struct L1Args
{
    const float* image[VETR_MAX_LAYERS];
    const float* target[VETR_MAX_LAYERS];
    float* grad[VETR_MAX_LAYERS];
    long long end[VETR_MAX_LAYERS];  // running element count: level l covers [end[l-1], end[l])
    float inv_numel[VETR_MAX_LAYERS];
    int levels;
    float* loss;
};

__global__ void __launch_bounds__(256) l1_loss_grad_kernel(const __grid_constant__ L1Args a)
{
    __shared__ float s_part[8];
    const long long total  = a.end[a.levels - 1];
    const long long stride = (long long)gridDim.x * blockDim.x * 4;
    float sum = 0.f;
    // four consecutive elements per thread where they lie in one level and are 16-byte aligned, else one by one
    for (long long i = ((long long)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < total; i += stride)
    {
        int l = 0;
#pragma unroll
        for (int k = 1; k < VETR_MAX_LAYERS; ++k)
            if (k < a.levels && i >= a.end[k - 1]) l = k;
        const long long base = l ? a.end[l - 1] : 0, j = i - base, n = a.end[l] - base;
        const float w = a.inv_numel[l];
        if (j + 4 <= n && ((j & 3) == 0))
        {
            const float4 x = __ldg(reinterpret_cast<const float4*>(a.image[l] + j));
            const float4 t = __ldg(reinterpret_cast<const float4*>(a.target[l] + j));
            const float d[4] = {x.x - t.x, x.y - t.y, x.z - t.z, x.w - t.w};
            float g[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) g[k] = d[k] > 0.f ? w : (d[k] < 0.f ? -w : 0.f), sum += fabsf(d[k]) * w;
            *reinterpret_cast<float4*>(a.grad[l] + j) = make_float4(g[0], g[1], g[2], g[3]);
        }
        else
        {
            for (long long e = i; e < min(i + 4, total); ++e)
            {
                int le = 0;
#pragma unroll
                for (int k = 1; k < VETR_MAX_LAYERS; ++k)
                    if (k < a.levels && e >= a.end[k - 1]) le = k;
                const long long je = e - (le ? a.end[le - 1] : 0);
                const float d = a.image[le][je] - a.target[le][je], we = a.inv_numel[le];
                a.grad[le][je] = d > 0.f ? we : (d < 0.f ? -we : 0.f);
                sum += fabsf(d) * we;
            }
        }
    }
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_down_sync(0xffffffffu, sum, o);
    if ((threadIdx.x & 31) == 0) s_part[threadIdx.x >> 5] = sum;
    __syncthreads();
    if (threadIdx.x == 0)
    {
        float t = 0.f;
        for (int k = 0; k < 8; ++k) t += s_part[k];
        atomicAdd(a.loss, t);
    }
}

}  // namespace vetr

#include "vetr_envmap.cuh"
#include "vetr_knn.cuh"
#include "vetr_points.cuh"

// =========================================================================================================
// C ABI

using namespace vetr;

struct vetr_ctx
{
    int device           = 0;
    cudaStream_t stream  = nullptr;
    int last_cuda        = 0;
    int sm_count         = 148;
    long long* tile_sums = nullptr;  // scan scratch
    long long tile_cap   = 0;
    int2* grid_queue     = nullptr;  // (cell, chunk) queue of vetr_grid_loss, allocated by its first call
    int* grid_queue_count = nullptr;
    // scratch of vetr_knn_radius, grown on demand: per point (sorted copy, cell, queue) and per cell (starts, ends)
    float4* knn_sorted   = nullptr;
    int* knn_point_cell  = nullptr;
    int* knn_queue       = nullptr;
    long long knn_cap_points = 0;
    int* knn_starts      = nullptr;
    int* knn_ends        = nullptr;
    long long knn_cap_cells = 0;
    int* knn_tile_sums   = nullptr;  // 16384 tile sums, then 16 words: bounds[6], occupied (64 bit), queue count, 2 of the point removal
    int* points_flags    = nullptr;  // keep flags of vetr_remove_points_plan
    long long points_cap = 0;
    int blend_ctas_per_sm = 1, back_ctas_per_sm = 1, fuzzy_ctas_per_sm = 1, bilinear_ctas_per_sm = 1;
    long long launches   = 0;
    bool timing          = false;
    cudaEvent_t ev[VETR_T_N][2] = {};
    bool ev_used[VETR_T_N]      = {};
};

// Brackets the launches of one pass with events when timing is on, and counts kernels.
struct PassScope
{
    vetr_ctx* c;
    int id;
    PassScope(vetr_ctx* ctx, int pass, int kernels) : c(ctx), id(pass)
    {
        c->launches += kernels;
        if (c->timing) cudaEventRecord(c->ev[id][0], c->stream);
    }
    ~PassScope()
    {
        if (c->timing)
        {
            cudaEventRecord(c->ev[id][1], c->stream);
            c->ev_used[id] = true;
        }
    }
};

#define VETR_CUDA(ctx, call)                      \
    do                                            \
    {                                             \
        cudaError_t e_ = (call);                  \
        if (e_ != cudaSuccess)                    \
        {                                         \
            (ctx)->last_cuda = (int)e_;           \
            return VETR_E_CUDA;                   \
        }                                         \
    } while (0)

static int __float_as_int_host(float v)
{
    int i;
    memcpy(&i, &v, 4);
    return i;
}

// Pixel space of one view: every level's height is padded to a multiple of kBand rows (the banded order of pixel_offset).
// rbase / *row_major: the same levels in plain row-major order without padding.
static int64_t pyramid(int w, int h, int L, int* lw, int* lh, long long* lbase, long long* rbase = nullptr,
                       long long* row_major = nullptr)
{
    long long base = 0, rm = 0;
    for (int l = 0; l < L; ++l)
    {
        if (lw) lw[l] = w, lh[l] = h, lbase[l] = base;
        if (rbase) rbase[l] = rm;
        base += (long long)w * ((h + kBand - 1) / kBand * kBand);
        rm += (long long)w * h;
        w /= 2;
        h /= 2;
    }
    if (row_major) *row_major = rm;
    return base;
}

extern "C" int64_t vetr_pyramid_pixels(int w, int h, int num_layers)
{
    if (w <= 0 || h <= 0 || num_layers < 1 || num_layers > VETR_MAX_LAYERS) return -1;
    return pyramid(w, h, num_layers, nullptr, nullptr, nullptr);
}

extern "C" int64_t vetr_item_table_entries(int64_t capacity, int64_t n_pixels_total)
{
    if (capacity < 0 || n_pixels_total < 0) return -1;
    int64_t cap = capacity < 0x7fffffffLL ? capacity : 0x7fffffffLL;
    return (cap + (int64_t)kPixelWork * n_pixels_total + kQuantum - 1) / kQuantum + 2;
}

extern "C" int64_t vetr_max_fragments(int n_points, int n_views, const vetr_params* p)
{
    if (!p) return -1;
    int64_t f = (int64_t)n_points * p->num_layers * n_views;
    if (p->render_mode == VETR_MODE_BILINEAR_BLEND) f *= 4;
    return f;
}

extern "C" int64_t vetr_list_capacity(int n_points, int n_views, int w, int h, const vetr_params* p)
{
    if (!p) return -1;
    int64_t f = vetr_max_fragments(n_points, n_views, p);
    if (p->render_mode == VETR_MODE_FUZZY_DT)
    {
        // mode 0 keeps no lists: the buffer holds one accumulator record per pixel of the pixel space instead
        const int64_t px = vetr_pyramid_pixels(w, h, p->num_layers);
        if (px < 0) return -1;
        f = px * n_views;
    }
    return f;
}

extern "C" const char* vetr_strerror(int status)
{
    switch (status)
    {
        case VETR_OK: return "ok";
        case VETR_E_INVALID_ARG: return "invalid argument";
        case VETR_E_CUDA: return "CUDA runtime error";
        case VETR_E_UNSUPPORTED: return "unsupported camera model or option";
        case VETR_E_LIST_OVERFLOW: return "fragment buffer too small";
        case VETR_E_TOO_LARGE: return "size exceeds a fixed limit";
        default: return "unknown status";
    }
}

extern "C" int vetr_last_cuda_error(const vetr_ctx* ctx) { return ctx ? ctx->last_cuda : 0; }

static int ensure_scratch(vetr_ctx* ctx, long long n_tiles)
{
    if (n_tiles > ctx->tile_cap)
    {
        if (ctx->tile_sums) cudaFree(ctx->tile_sums);
        ctx->tile_sums = nullptr;
        long long cap  = n_tiles + n_tiles / 4 + 16;
        VETR_CUDA(ctx, cudaMalloc(&ctx->tile_sums, cap * sizeof(long long)));
        ctx->tile_cap = cap;
    }
    return VETR_OK;
}

extern "C" int vetr_create(vetr_ctx** out, int device, void* cuda_stream)
{
    if (!out) return VETR_E_INVALID_ARG;
    vetr_ctx* ctx = new (std::nothrow) vetr_ctx();
    if (!ctx) return VETR_E_INVALID_ARG;
    ctx->device = device;
    ctx->stream = (cudaStream_t)cuda_stream;
    cudaError_t e = cudaSetDevice(device);
    cudaDeviceProp prop;
    if (e == cudaSuccess) e = cudaGetDeviceProperties(&prop, device);
    if (e == cudaSuccess) ctx->sm_count = prop.multiProcessorCount;
    const int blend_smem = (int)sizeof(BlendSmem), back_smem = (int)sizeof(BackSmem);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(sort_blend_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, blend_smem);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(sort_blend_long_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kLongBlendSmem);
    const int fuzzy_smem = (int)sizeof(BackSmemFuzzy), fuzzy_long_smem = (int)sizeof(FuzzyLongSmem);
    const auto smem_attr = cudaFuncAttributeMaxDynamicSharedMemorySize;
    if (e == cudaSuccess) e = cudaFuncSetAttribute(backward_kernel<false, false>, smem_attr, back_smem);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(backward_kernel<false, true>, smem_attr, back_smem);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(backward_kernel<true, false>, smem_attr, fuzzy_smem);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(backward_fuzzy_long_kernel, smem_attr, fuzzy_long_smem);
    if (e == cudaSuccess)
        e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&ctx->fuzzy_ctas_per_sm, backward_kernel<true, false>, kThreads, fuzzy_smem);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(backward_long_kernel<false>, smem_attr, back_smem);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(backward_long_kernel<true>, smem_attr, back_smem);
    if (e == cudaSuccess)
        e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&ctx->blend_ctas_per_sm, sort_blend_kernel, kThreads, blend_smem);
    if (e == cudaSuccess)
        e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&ctx->back_ctas_per_sm, backward_kernel<false, false>, kThreads, back_smem);
    if (e == cudaSuccess)
        e = cudaOccupancyMaxActiveBlocksPerMultiprocessor(&ctx->bilinear_ctas_per_sm, backward_kernel<false, true>, kThreads, back_smem);
    if (e != cudaSuccess)
    {
        delete ctx;
        *out = nullptr;
        return VETR_E_CUDA;
    }
    if (ctx->blend_ctas_per_sm < 1) ctx->blend_ctas_per_sm = 1;
    if (ctx->back_ctas_per_sm < 1) ctx->back_ctas_per_sm = 1;
    if (ctx->fuzzy_ctas_per_sm < 1) ctx->fuzzy_ctas_per_sm = 1;
    if (ctx->bilinear_ctas_per_sm < 1) ctx->bilinear_ctas_per_sm = 1;
    *out = ctx;
    return VETR_OK;
}

extern "C" void vetr_destroy(vetr_ctx* ctx)
{
    if (!ctx) return;
    cudaSetDevice(ctx->device);
    if (ctx->tile_sums) cudaFree(ctx->tile_sums);
    if (ctx->grid_queue) cudaFree(ctx->grid_queue);
    cudaFree(ctx->knn_sorted), cudaFree(ctx->knn_point_cell), cudaFree(ctx->knn_queue);
    cudaFree(ctx->knn_starts), cudaFree(ctx->knn_ends), cudaFree(ctx->knn_tile_sums), cudaFree(ctx->points_flags);
    for (int i = 0; i < VETR_T_N; ++i)
        for (int k = 0; k < 2; ++k)
            if (ctx->ev[i][k]) cudaEventDestroy(ctx->ev[i][k]);
    delete ctx;
}

extern "C" int vetr_set_timing(vetr_ctx* ctx, int enable)
{
    if (!ctx) return VETR_E_INVALID_ARG;
    VETR_CUDA(ctx, cudaSetDevice(ctx->device));
    if (enable && !ctx->ev[0][0])
        for (int i = 0; i < VETR_T_N; ++i)
            for (int k = 0; k < 2; ++k) VETR_CUDA(ctx, cudaEventCreate(&ctx->ev[i][k]));
    ctx->timing = enable != 0;
    for (int i = 0; i < VETR_T_N; ++i) ctx->ev_used[i] = false;
    return VETR_OK;
}

extern "C" int vetr_get_timings(vetr_ctx* ctx, float* out_ms)
{
    if (!ctx || !out_ms) return VETR_E_INVALID_ARG;
    VETR_CUDA(ctx, cudaSetDevice(ctx->device));
    VETR_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    for (int i = 0; i < VETR_T_N; ++i)
    {
        out_ms[i] = 0.f;
        if (ctx->ev_used[i]) VETR_CUDA(ctx, cudaEventElapsedTime(&out_ms[i], ctx->ev[i][0], ctx->ev[i][1]));
    }
    return VETR_OK;
}

extern "C" int64_t vetr_launch_count(const vetr_ctx* ctx) { return ctx ? ctx->launches : 0; }

extern "C" int vetr_set_stream(vetr_ctx* ctx, void* cuda_stream)
{
    if (!ctx) return VETR_E_INVALID_ARG;
    ctx->stream = (cudaStream_t)cuda_stream;
    return VETR_OK;
}

static int fill_frame(vetr_ctx* ctx, Frame& f, const vetr_params* p, const vetr_cloud* cloud, const vetr_texture* tex,
                      const vetr_cameras* cams, const vetr_view* views, int n_views, const vetr_lists* lists)
{
    if (!ctx || !p || !cloud || !tex || !cams || !views || !lists) return VETR_E_INVALID_ARG;
    if (n_views < 1 || n_views > VETR_MAX_VIEWS) return VETR_E_INVALID_ARG;
    if (p->num_layers < 1 || p->num_layers > VETR_MAX_LAYERS) return VETR_E_INVALID_ARG;
    if (p->num_channels != 3 && p->num_channels != 4) return VETR_E_INVALID_ARG;
    if (p->render_mode < VETR_MODE_FUZZY_DT || p->render_mode > VETR_MODE_BILINEAR_BLEND) return VETR_E_UNSUPPORTED;
    if (cloud->n < 0 || tex->n_tex < 1 || !cloud->position || !cloud->index || !tex->texture || !tex->confidence ||
        !tex->background || !cams->poses_se3 || !cams->intrinsics)
        return VETR_E_INVALID_ARG;
    if (((uintptr_t)cloud->position & 15) != 0) return VETR_E_INVALID_ARG;
    if (!lists->counts || !lists->ends || !lists->frags || !lists->status || lists->capacity < 0 ||
        ((uintptr_t)lists->frags & 31) != 0)
        return VETR_E_INVALID_ARG;
    memset(&f, 0, sizeof(f));
    f.n_views = n_views, f.L = p->num_layers, f.C = p->num_channels, f.n = cloud->n, f.n_tex = tex->n_tex;
    f.w = views[0].w, f.h = views[0].h;
    if (f.w <= 0 || f.h <= 0) return VETR_E_INVALID_ARG;
    for (int b = 0; b < n_views; ++b)
    {
        const vetr_view& v = views[b];
        if (v.w != f.w || v.h != f.h) return VETR_E_INVALID_ARG;
        if (v.camera_model != 0) return VETR_E_UNSUPPORTED;
        if (v.image_index < 0 || v.image_index >= cams->n_img || v.camera_index < 0 || v.camera_index >= cams->n_cam)
            return VETR_E_INVALID_ARG;
        f.views[b].image_index = v.image_index, f.views[b].camera_index = v.camera_index;
        memcpy(f.views[b].crop, v.crop, sizeof(v.crop));
        memcpy(f.views[b].rot, v.rot, sizeof(v.rot));
    }
    f.mode = p->render_mode, f.drop_by_radius = p->drop_out_points_by_radius, f.use_env = p->use_environment_map;
    f.viewer_only = p->viewer_only, f.dbg_max_len = p->debug_max_list_length, f.need_point_grad = p->need_point_gradient;
    f.bg_alpha_to_point0 = p->background_alpha_to_point0, f.keep_sorted = p->keep_sorted_lists;
    f.radius_threshold = p->drop_out_radius_threshold, f.dist_cutoff = p->dist_cutoff;
    f.stability_cutoff = p->stability_cutoff_value, f.k_grad_factor = p->K_gradient_factor;
    f.dist_grad_factor = p->distortion_gradient_factor, f.mask_value = p->output_background_mask_value;
    f.accept_blend = p->depth_accept_blend, f.depth_accept = p->depth_accept, f.ghost = p->ghost_gradients;
    f.P  = pyramid(f.w, f.h, f.L, f.lw, f.lh, f.lbase, f.rbase, &f.Prm);
    f.PT = f.P * n_views;
    if (f.lw[f.L - 1] < 1 || f.lh[f.L - 1] < 1) return VETR_E_INVALID_ARG;  // the reference asserts w > 0 && h > 0 per level
    for (int l = 0; l < f.L; ++l) f.inv_lw[l] = 1.f / (float)f.lw[l], f.inv_band[l] = 1.f / (float)(kBand * f.lw[l]);
    if (f.PT > 0x7fffffffLL || (long long)f.lw[0] * f.lh[0] * f.C * n_views > 0x7fffffffLL) return VETR_E_TOO_LARGE;
    f.position = (const float4*)cloud->position, f.index = cloud->index;
    f.texture = tex->texture, f.confidence = tex->confidence, f.background = tex->background;
    f.poses = cams->poses_se3, f.intr = cams->intrinsics;
    f.counts = lists->counts, f.ends = lists->ends, f.recs = (uint4*)lists->frags;
    f.capacity = lists->capacity, f.status = lists->status;
    long long n_tiles = (f.PT + kScanTile - 1) / kScanTile;
    if (!lists->items || lists->items_capacity < vetr_item_table_entries(lists->capacity, f.PT)) return VETR_E_INVALID_ARG;
    VETR_CUDA(ctx, cudaSetDevice(ctx->device));
    int rc = ensure_scratch(ctx, n_tiles);
    if (rc != VETR_OK) return rc;
    f.item_start = lists->items;
    f.level_mask = lists->level_mask;
    f.point_grad = (float2*)lists->point_grad;
    f.img4       = (float4*)lists->pixel_scratch;
    f.grad4      = f.img4 ? f.img4 + f.PT : nullptr;
    return VETR_OK;
}

extern "C" int vetr_forward(vetr_ctx* ctx, const vetr_params* params, const vetr_cloud* cloud, const vetr_texture* texture,
                            const vetr_cameras* cameras, const vetr_view* views, int n_views, const float* dropout,
                            const vetr_lists* lists, float* const* out_color, float* const* out_weight,
                            float* const* out_mask, float* const* out_depth)
{
    Frame f;
    int rc = fill_frame(ctx, f, params, cloud, texture, cameras, views, n_views, lists);
    if (rc != VETR_OK) return rc;
    if (!out_color) return VETR_E_INVALID_ARG;
    f.dropout = dropout;
    OutPtrs out;
    memset(&out, 0, sizeof(out));
    for (int l = 0; l < f.L; ++l)
    {
        if (!out_color[l]) return VETR_E_INVALID_ARG;
        out.color[l] = out_color[l];
        if ((out_weight && !out_weight[l]) || (out_mask && !out_mask[l]) || (out_depth && !out_depth[l])) return VETR_E_INVALID_ARG;
        if (out_weight) out.weight[l] = out_weight[l];
        if (out_mask) out.mask[l] = out_mask[l];
        if (out_depth) out.depth[l] = out_depth[l];
    }
    cudaStream_t st = ctx->stream;
    if (f.mode == VETR_MODE_FUZZY_DT)
    {
        if (f.capacity < f.PT) return VETR_E_INVALID_ARG;  // the fragment buffer holds one accumulator record per pixel
        VETR_CUDA(ctx, cudaMemsetAsync(f.status, 0, 4 * sizeof(int), st));
        VETR_CUDA(ctx, cudaMemsetAsync(f.recs, 0, (size_t)f.PT * 32, st));
        const int ctas = (f.n + kProjThreads - 1) / kProjThreads;
        {
            PassScope t(ctx, VETR_T_COUNT, 2 + (ctas > 0));
            fill_int_kernel<<<(unsigned)((f.PT + 255) / 256), 256, 0, st>>>(f.ends, __float_as_int_host(kMaxDepth), f.PT);
            if (ctas > 0) fuzzy_dt_point_kernel<0><<<dim3(ctas, n_views), kProjThreads, 0, st>>>(f);
        }
        if (ctas > 0)
        {
            PassScope t(ctx, VETR_T_COLLECT, 1);
            fuzzy_dt_point_kernel<1><<<dim3(ctas, n_views), kProjThreads, 0, st>>>(f);
        }
        {
            PassScope t(ctx, VETR_T_SORT_BLEND, 1);
            fuzzy_dt_combine_kernel<<<(unsigned)((f.PT + 255) / 256), 256, 0, st>>>(f, out);
        }
        VETR_CUDA(ctx, cudaGetLastError());
        return VETR_OK;
    }
    VETR_CUDA(ctx, cudaMemsetAsync(f.counts, 0, f.PT * sizeof(int), st));
    VETR_CUDA(ctx, cudaMemsetAsync(f.status, 0, 4 * sizeof(int), st));
    const int point_ctas = (f.n + kProjThreads * kPointsPerThread - 1) / (kProjThreads * kPointsPerThread);
    if (point_ctas > 0)
    {
        PassScope t(ctx, VETR_T_COUNT, 1);
        project_kernel<false, kPointsPerThread><<<dim3(point_ctas, n_views), kProjThreads, 0, st>>>(f);
    }
    const int n_tiles = (int)((f.PT + kScanTile - 1) / kScanTile);
    {
        PassScope t(ctx, VETR_T_SCAN, 3);
        scan_tile_sums_kernel<<<n_tiles, 256, 0, st>>>(f.counts, f.PT, ctx->tile_sums, f.status);
        scan_spine_kernel<<<1, 1024, 0, st>>>(ctx->tile_sums, n_tiles, f.PT, f.capacity, f.status, f.item_start);
        scan_apply_kernel<<<n_tiles, 256, 0, st>>>(f.counts, f.PT, ctx->tile_sums, f.ends, f.status, f.item_start);
    }
    if (point_ctas > 0)
    {
        PassScope t(ctx, VETR_T_COLLECT, 1);
        const int ctas = (f.n + kProjThreads * kCollectPoints - 1) / (kProjThreads * kCollectPoints);
        project_kernel<true, kCollectPoints><<<dim3(ctas, n_views), kProjThreads, 0, st>>>(f);
    }
    {
        PassScope t(ctx, VETR_T_SORT_BLEND, 2);
        const int grid = ctx->sm_count * ctx->blend_ctas_per_sm;
        sort_blend_kernel<<<grid, kThreads, sizeof(BlendSmem), st>>>(f, out);
        sort_blend_long_kernel<<<ctx->sm_count * 2, kThreads, kLongBlendSmem, st>>>(f, out);
    }
    VETR_CUDA(ctx, cudaGetLastError());
    return VETR_OK;
}

extern "C" int vetr_backward(vetr_ctx* ctx, const vetr_params* params, const vetr_cloud* cloud, const vetr_texture* texture,
                             const vetr_cameras* cameras, const vetr_view* views, int n_views, const float* dropout,
                             const vetr_lists* lists, const float* const* out_color, const float* const* grad_color,
                             float* g_desc, float* g_conf,
                             float* g_points, float* g_background, double* g_pose, float* g_pose_count, float* g_intr,
                             float* g_intr_count)
{
    return vetr_backward_phase(ctx, params, cloud, texture, cameras, views, n_views, dropout, lists, out_color, grad_color,
                               g_desc, g_conf, g_points, g_background, g_pose, g_pose_count, g_intr, g_intr_count,
                               VETR_BACKWARD_FRAGMENTS | VETR_BACKWARD_POINTS);
}

extern "C" int vetr_backward_phase(vetr_ctx* ctx, const vetr_params* params, const vetr_cloud* cloud,
                                   const vetr_texture* texture, const vetr_cameras* cameras, const vetr_view* views,
                                   int n_views, const float* dropout, const vetr_lists* lists,
                                   const float* const* out_color, const float* const* grad_color, float* g_desc,
                                   float* g_conf, float* g_points, float* g_background, double* g_pose,
                                   float* g_pose_count, float* g_intr, float* g_intr_count, int phases)
{
    if ((phases & ~(VETR_BACKWARD_FRAGMENTS | VETR_BACKWARD_POINTS)) != 0 || phases == 0) return VETR_E_INVALID_ARG;
    Frame f;
    int rc = fill_frame(ctx, f, params, cloud, texture, cameras, views, n_views, lists);
    if (rc != VETR_OK) return rc;
    if (!out_color || !grad_color || !g_desc || !g_conf || !g_background) return VETR_E_INVALID_ARG;
    if ((g_pose != nullptr) != (g_pose_count != nullptr) || (g_intr != nullptr) != (g_intr_count != nullptr))
        return VETR_E_INVALID_ARG;
    if (((uintptr_t)g_desc & 15) != 0 || ((uintptr_t)g_points & 15) != 0) return VETR_E_INVALID_ARG;
    BackPtrs bp;
    memset(&bp, 0, sizeof(bp));
    for (int l = 0; l < f.L; ++l)
    {
        if (!out_color[l] || !grad_color[l]) return VETR_E_INVALID_ARG;
        bp.out_color[l] = out_color[l], bp.grad_color[l] = grad_color[l];
    }
    bp.g_desc = (float4*)g_desc, bp.g_conf = g_conf, bp.g_points = (float4*)g_points, bp.g_background = g_background;
    bp.g_pose = g_pose, bp.g_pose_count = g_pose_count, bp.g_intr = g_intr, bp.g_intr_count = g_intr_count;
    if (!f.need_point_grad && f.mode != VETR_MODE_BILINEAR_BLEND && f.mode != VETR_MODE_FUZZY_DT) bp.g_points = nullptr;
    f.dropout = dropout;
    if (f.mode == VETR_MODE_FUZZY_DT)
    {
        if (!(phases & VETR_BACKWARD_FRAGMENTS)) return VETR_OK;  // mode 0 has one phase
        PassScope t(ctx, VETR_T_BACKWARD, 2);
        cudaStream_t st = ctx->stream;
        fuzzy_dt_background_kernel<<<ctx->sm_count * 4, 256, 0, st>>>(f, bp);
        const int ctas = (f.n + kProjThreads - 1) / kProjThreads;
        if (ctas > 0)
        {
            if (g_intr)
                fuzzy_dt_backward_kernel<true><<<dim3(ctas, n_views), kProjThreads, 0, st>>>(f, bp);
            else
                fuzzy_dt_backward_kernel<false><<<dim3(ctas, n_views), kProjThreads, 0, st>>>(f, bp);
        }
        VETR_CUDA(ctx, cudaGetLastError());
        return VETR_OK;
    }
    const bool bilinear = f.mode == VETR_MODE_BILINEAR_BLEND;
    // position / camera gradients (and mode 3's confidence gradient) come from the per-point pass over what the
    // per-fragment kernel parks
    const bool spatial    = f.need_point_grad && (bp.g_points || g_pose || g_intr);
    const bool point_pass = bilinear || spatial;
    if (!spatial) f.need_point_grad = 0;
    if (point_pass && (!f.level_mask || !f.point_grad || ((uintptr_t)f.point_grad & 15) != 0)) return VETR_E_INVALID_ARG;
    if (bilinear && f.n_tex > kTexMask) return VETR_E_TOO_LARGE;
    if (!f.img4 || ((uintptr_t)f.img4 & 15) != 0) return VETR_E_INVALID_ARG;
    if (phases & VETR_BACKWARD_FRAGMENTS)
    {
        PassScope t(ctx, VETR_T_BACKWARD, 3);
        cudaStream_t st = ctx->stream;
        pack_images_kernel<<<(unsigned)((f.Prm * n_views + 255) / 256), 256, 0, st>>>(f, bp);
        if (f.mode == VETR_MODE_FUZZY_BLEND)
        {
            const int grid = ctx->sm_count * ctx->fuzzy_ctas_per_sm;
            backward_kernel<true, false><<<grid, kThreads, sizeof(BackSmemFuzzy), st>>>(f, bp);
            backward_fuzzy_long_kernel<<<ctx->sm_count, kThreads, sizeof(FuzzyLongSmem), st>>>(f, bp);
        }
        else if (bilinear)
        {
            const int grid = ctx->sm_count * ctx->bilinear_ctas_per_sm;
            backward_kernel<false, true><<<grid, kThreads, sizeof(BackSmem), st>>>(f, bp);
            backward_long_kernel<true><<<ctx->sm_count, kThreads, sizeof(BackSmem), st>>>(f, bp);
        }
        else
        {
            const int grid = ctx->sm_count * ctx->back_ctas_per_sm;
            backward_kernel<false, false><<<grid, kThreads, sizeof(BackSmem), st>>>(f, bp);
            backward_long_kernel<false><<<ctx->sm_count, kThreads, sizeof(BackSmem), st>>>(f, bp);
        }
    }
    if ((phases & VETR_BACKWARD_POINTS) && point_pass && f.n > 0)
    {
        PassScope t(ctx, VETR_T_POINT_BACKWARD, 1);
        const int ctas = (f.n + kProjThreads * kPointBackPoints - 1) / (kProjThreads * kPointBackPoints);
        cudaStream_t st = ctx->stream;
        if (bilinear)
        {
            if (g_intr)
                point_backward_kernel<true, true><<<ctas, kProjThreads, 0, st>>>(f, bp);
            else
                point_backward_kernel<false, true><<<ctas, kProjThreads, 0, st>>>(f, bp);
        }
        else
        {
            if (g_intr)
                point_backward_kernel<true, false><<<ctas, kProjThreads, 0, st>>>(f, bp);
            else
                point_backward_kernel<false, false><<<ctas, kProjThreads, 0, st>>>(f, bp);
        }
    }
    VETR_CUDA(ctx, cudaGetLastError());
    return VETR_OK;
}

extern "C" int vetr_finalize_gradients(vetr_ctx* ctx, int channels, int n_tex, const float* g_desc, float* g_texture,
                                       int n, float* g_points, float* g_points_count, int n_img, double* g_pose,
                                       const float* g_pose_count, int n_cam, float* g_intr, const float* g_intr_count)
{
    if (!ctx) return VETR_E_INVALID_ARG;
    VETR_CUDA(ctx, cudaSetDevice(ctx->device));
    cudaStream_t st = ctx->stream;
    const int n_kernels = (g_desc && g_texture && n_tex > 0) + (g_points && n > 0) + (g_pose && g_pose_count && n_img > 0) +
                          (g_intr && g_intr_count && n_cam > 0);
    PassScope t(ctx, VETR_T_FINALIZE, n_kernels);
    if (g_desc && g_texture && n_tex > 0)
    {
        if (channels != 3 && channels != 4) return VETR_E_INVALID_ARG;
        transpose_desc_kernel<<<(n_tex + 255) / 256, 256, 0, st>>>((const float4*)g_desc, g_texture, n_tex, channels);
    }
    if (g_points && n > 0) normalize_points_kernel<<<(n + 255) / 256, 256, 0, st>>>((float4*)g_points, g_points_count, n);
    if (g_pose && g_pose_count && n_img > 0)
        normalize_rows_kernel<double, 6><<<(n_img + 127) / 128, 128, 0, st>>>(g_pose, g_pose_count, n_img);
    if (g_intr && g_intr_count && n_cam > 0)
        normalize_rows_kernel<float, 13><<<(n_cam + 127) / 128, 128, 0, st>>>(g_intr, g_intr_count, n_cam);
    VETR_CUDA(ctx, cudaGetLastError());
    return VETR_OK;
}

extern "C" int64_t vetr_exchange_raw_floats(int n_tex, int n)
{
    if (n_tex < 0 || n < 0) return -1;
    return 5LL * n_tex + 4LL * n;
}

static long long exchange_out_points(int channels, int n_tex) { return ((long long)channels * n_tex + 3) / 4 * 4; }

extern "C" int64_t vetr_exchange_out_floats(int channels, int n_tex, int n)
{
    if ((channels != 3 && channels != 4) || n_tex < 0 || n < 0) return -1;
    return exchange_out_points(channels, n_tex) + 4LL * n + n_tex;
}

extern "C" int vetr_exchange_finalize(vetr_ctx* ctx, const vetr_exchange* ex, int channels, int n_tex, int n)
{
    return vetr_exchange_finalize_part(ctx, ex, channels, n_tex, n, VETR_SEG_DESC | VETR_SEG_POINTS | VETR_SEG_CONF, 4);
}

extern "C" int vetr_exchange_finalize_part(vetr_ctx* ctx, const vetr_exchange* ex, int channels, int n_tex, int n,
                                           int segments, int ctas_per_sm)
{
    if (!ctx || !ex || (channels != 3 && channels != 4) || n_tex < 1 || n < 0) return VETR_E_INVALID_ARG;
    if (segments <= 0 || (segments & ~(VETR_SEG_DESC | VETR_SEG_POINTS | VETR_SEG_CONF)) != 0) return VETR_E_INVALID_ARG;
    if (ctas_per_sm < 1 || ctas_per_sm > 8) return VETR_E_INVALID_ARG;
    if (ex->world < 1 || ex->world > VETR_MAX_RANKS || ex->rank < 0 || ex->rank >= ex->world) return VETR_E_INVALID_ARG;
    ExchangeArgs a;
    memset(&a, 0, sizeof(a));
    a.rank = ex->rank, a.world = ex->world, a.C = channels, a.n_tex = n_tex, a.n = n;
    a.out_points = exchange_out_points(channels, n_tex);
    a.out_conf   = a.out_points + 4LL * n;
    for (int k = 0; k < ex->world; ++k)
    {
        if (!ex->raw[k] || !ex->out[k] || ((uintptr_t)ex->raw[k] & 15) != 0 || ((uintptr_t)ex->out[k] & 15) != 0)
            return VETR_E_INVALID_ARG;
        a.raw[k] = ex->raw[k], a.out[k] = ex->out[k];
    }
    if ((ex->raw_multicast != nullptr) != (ex->out_multicast != nullptr)) return VETR_E_INVALID_ARG;
    if (((uintptr_t)ex->raw_multicast & 15) != 0 || ((uintptr_t)ex->out_multicast & 15) != 0) return VETR_E_INVALID_ARG;
    a.raw_mc = ex->raw_multicast, a.out_mc = ex->out_multicast;
    a.segments = segments;
    VETR_CUDA(ctx, cudaSetDevice(ctx->device));
    PassScope t(ctx, VETR_T_EXCHANGE, 1);
    if (a.raw_mc)
        exchange_finalize_kernel<true><<<ctx->sm_count * ctas_per_sm, 32 * kExchangeWarps, 0, ctx->stream>>>(a);
    else
        exchange_finalize_kernel<false><<<ctx->sm_count * ctas_per_sm, 32 * kExchangeWarps, 0, ctx->stream>>>(a);
    VETR_CUDA(ctx, cudaGetLastError());
    return VETR_OK;
}

extern "C" int vetr_grid_loss(vetr_ctx* ctx, const vetr_cameras* cams, const vetr_view* view, float dist_cutoff, int n_cells,
                              const float* cell_bb_min, const float* cell_bb_len, const float* loss_img, int channels,
                              float* cell_value, int32_t* cell_access_count)
{
    if (!ctx || !cams || !view || !cams->poses_se3 || !cams->intrinsics || n_cells < 0 || channels < 1) return VETR_E_INVALID_ARG;
    if (n_cells > 0 && (!cell_bb_min || !cell_bb_len || !loss_img || !cell_value || !cell_access_count)) return VETR_E_INVALID_ARG;
    if (view->w <= 0 || view->h <= 0) return VETR_E_INVALID_ARG;
    if (view->camera_model != 0) return VETR_E_UNSUPPORTED;
    if (view->image_index < 0 || view->image_index >= cams->n_img || view->camera_index < 0 || view->camera_index >= cams->n_cam)
        return VETR_E_INVALID_ARG;
    if ((long long)channels * view->w * view->h > 0x7fffffffLL) return VETR_E_TOO_LARGE;
    Frame f;
    memset(&f, 0, sizeof(f));
    f.n_views = 1, f.w = view->w, f.h = view->h, f.dist_cutoff = dist_cutoff;
    f.views[0].image_index = view->image_index, f.views[0].camera_index = view->camera_index;
    memcpy(f.views[0].crop, view->crop, sizeof(view->crop));
    memcpy(f.views[0].rot, view->rot, sizeof(view->rot));
    f.poses = cams->poses_se3, f.intr = cams->intrinsics;
    GridArgs a;
    a.bb_min = cell_bb_min, a.bb_len = cell_bb_len, a.loss = loss_img, a.value = cell_value, a.count = cell_access_count;
    a.n_cells = n_cells, a.channels = channels, a.h = view->h, a.w = view->w, a.view = 0;
    VETR_CUDA(ctx, cudaSetDevice(ctx->device));
    if (n_cells > 0)
    {
        if (!ctx->grid_queue)
        {
            VETR_CUDA(ctx, cudaMalloc(&ctx->grid_queue, (size_t)kGridQueueCap * sizeof(int2) + 256));
            ctx->grid_queue_count = reinterpret_cast<int*>(ctx->grid_queue + kGridQueueCap);
        }
        VETR_CUDA(ctx, cudaMemsetAsync(ctx->grid_queue_count, 0, sizeof(int), ctx->stream));
        ctx->launches += 2;
        const int ctas = min((n_cells + kGridWarps - 1) / kGridWarps, ctx->sm_count * 16);
        grid_loss_kernel<<<ctas, 32 * kGridWarps, 0, ctx->stream>>>(f, a, ctx->grid_queue, ctx->grid_queue_count);
        grid_loss_chunk_kernel<<<ctx->sm_count * 16, 32 * kGridWarps, 0, ctx->stream>>>(f, a, ctx->grid_queue, ctx->grid_queue_count);
    }
    VETR_CUDA(ctx, cudaGetLastError());
    return VETR_OK;
}

// Shared argument checks and parameter block of the two environment map calls, for views [v0, v0 + nv).
static int envmap_args(const vetr_cameras* cams, const vetr_view* views, int n_views, int num_layers, const vetr_envmap* env,
                       const float* const* weight, int flags, int v0, int nv, EnvArgs& a)
{
    if (!cams || !views || !env || !weight || !cams->poses_se3 || !cams->intrinsics || !env->density || !env->color)
        return VETR_E_INVALID_ARG;
    if (n_views < 1 || num_layers < 1 || num_layers > VETR_MAX_LAYERS) return VETR_E_INVALID_ARG;
    if (env->n_spheres < 1 || env->n_spheres > kEnvMaxSpheres || env->channels < 1 || env->channels > 4 || env->resolution < 1 ||
        env->up_axis < 0 || env->up_axis > 2 || (flags & ~15) != 0)
        return VETR_E_INVALID_ARG;
    if ((long long)env->n_spheres * env->resolution * env->resolution > 0x7fffffffLL) return VETR_E_TOO_LARGE;
    const int w = views[0].w, h = views[0].h;
    if (w <= 0 || h <= 0 || (w >> (num_layers - 1)) < 1 || (h >> (num_layers - 1)) < 1) return VETR_E_INVALID_ARG;
    memset(&a, 0, sizeof(a));
    a.n_views = nv, a.L = num_layers, a.S = env->n_spheres, a.R = env->resolution, a.C = env->channels;
    a.up_axis = env->up_axis, a.non_subzero = env->non_subzero_texture, a.flags = flags;
    memcpy(a.radii, env->radii, sizeof(a.radii));
    a.poses = cams->poses_se3, a.intr = cams->intrinsics, a.density = env->density, a.color = env->color;
    for (int b = 0; b < nv; ++b)
    {
        const vetr_view& v = views[v0 + b];
        if (v.w != w || v.h != h) return VETR_E_INVALID_ARG;
        if (v.camera_model != 0) return VETR_E_UNSUPPORTED;
        if (v.image_index < 0 || v.image_index >= cams->n_img || v.camera_index < 0 || v.camera_index >= cams->n_cam)
            return VETR_E_INVALID_ARG;
        a.views[b].image_index = v.image_index, a.views[b].camera_index = v.camera_index;
        memcpy(a.views[b].crop, v.crop, sizeof(v.crop));
        memcpy(a.views[b].rot, v.rot, sizeof(v.rot));
    }
    long long run = 0;
    int lw = w, lh = h;
    float scale = 1.f;
    for (int l = 0; l < num_layers; ++l, lw /= 2, lh /= 2, scale *= 0.5f)
    {
        if (!weight[l]) return VETR_E_INVALID_ARG;
        if ((long long)n_views * 4 * lw * lh > 0x7fffffffLL) return VETR_E_TOO_LARGE;
        a.lw[l] = lw, a.lh[l] = lh, a.scale[l] = scale;
        run += (long long)nv * lw * lh;
        a.lend[l]   = run;
        a.weight[l] = weight[l] + (long long)v0 * lw * lh;
    }
    return VETR_OK;
}

// The cameras' distortion coefficients must all be zero: read back once per call (a few hundred bytes; synchronises).
static int envmap_check_distortion(vetr_ctx* ctx, const vetr_cameras* cams, const vetr_view* views, int n_views)
{
    std::vector<float> k((size_t)cams->n_cam * 13);
    VETR_CUDA(ctx, cudaMemcpyAsync(k.data(), cams->intrinsics, k.size() * sizeof(float), cudaMemcpyDeviceToHost, ctx->stream));
    VETR_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    for (int b = 0; b < n_views; ++b)
    {
        if (views[b].camera_index < 0 || views[b].camera_index >= cams->n_cam) return VETR_E_INVALID_ARG;
        for (int i = 5; i < 13; ++i)
            if (k[(size_t)views[b].camera_index * 13 + i] != 0.f) return VETR_E_UNSUPPORTED;
    }
    return VETR_OK;
}

extern "C" int vetr_envmap_forward(vetr_ctx* ctx, const vetr_cameras* cams, const vetr_view* views, int n_views, int num_layers,
                                   const vetr_envmap* env, const float* const* weight, float* const* out, int flags)
{
    if (!ctx || !out) return VETR_E_INVALID_ARG;
    VETR_CUDA(ctx, cudaSetDevice(ctx->device));
    PassScope scope(ctx, VETR_T_ENVMAP, 0);
    for (int v0 = 0; v0 < n_views || v0 == 0; v0 += VETR_MAX_VIEWS)
    {
        const int nv = std::min(VETR_MAX_VIEWS, n_views - v0);
        EnvArgs a;
        int rc = envmap_args(cams, views, n_views, num_layers, env, weight, flags, v0, nv, a);
        if (rc != VETR_OK) return rc;
        if (v0 == 0 && !(flags & VETR_ENV_NO_DISTORTION_CHECK) && (rc = envmap_check_distortion(ctx, cams, views, n_views)) != VETR_OK) return rc;
        for (int l = 0; l < num_layers; ++l)
        {
            if (!out[l]) return VETR_E_INVALID_ARG;
            a.out[l] = out[l] + (long long)v0 * env->channels * a.lw[l] * a.lh[l];
        }
        const long long blocks = (a.lend[num_layers - 1] + kEnvThreads - 1) / kEnvThreads;
        ctx->launches += 1;
        envmap_forward_kernel<<<(int)std::min<long long>(blocks, (long long)ctx->sm_count * 32), kEnvThreads, 0, ctx->stream>>>(a);
    }
    VETR_CUDA(ctx, cudaGetLastError());
    return VETR_OK;
}

extern "C" int vetr_envmap_backward(vetr_ctx* ctx, const vetr_cameras* cams, const vetr_view* views, int n_views, int num_layers,
                                    const vetr_envmap* env, const float* const* weight, const float* const* grad_out, int flags,
                                    float* g_density, float* g_color)
{
    if (!ctx || !grad_out || !g_density || !g_color) return VETR_E_INVALID_ARG;
    VETR_CUDA(ctx, cudaSetDevice(ctx->device));
    PassScope scope(ctx, VETR_T_ENVMAP, 0);
    for (int v0 = 0; v0 < n_views || v0 == 0; v0 += VETR_MAX_VIEWS)
    {
        const int nv = std::min(VETR_MAX_VIEWS, n_views - v0);
        EnvArgs a;
        int rc = envmap_args(cams, views, n_views, num_layers, env, weight, flags, v0, nv, a);
        if (rc != VETR_OK) return rc;
        if (v0 == 0 && !(flags & VETR_ENV_NO_DISTORTION_CHECK) && (rc = envmap_check_distortion(ctx, cams, views, n_views)) != VETR_OK) return rc;
        for (int l = 0; l < num_layers; ++l)
        {
            if (!grad_out[l]) return VETR_E_INVALID_ARG;
            a.grad[l] = grad_out[l] + (long long)v0 * env->channels * a.lw[l] * a.lh[l];
        }
        a.g_density = g_density, a.g_color = g_color;
        const long long blocks = (a.lend[num_layers - 1] + kEnvThreads - 1) / kEnvThreads;
        ctx->launches += 1;
        envmap_backward_kernel<<<(int)std::min<long long>(blocks, (long long)ctx->sm_count * 32), kEnvThreads, 0, ctx->stream>>>(a);
    }
    VETR_CUDA(ctx, cudaGetLastError());
    return VETR_OK;
}

template <int KMAX>
static void knn_launch_search(vetr_ctx* ctx, const KnnSearch& a)
{
    knn_near_kernel<KMAX><<<(a.n + 127) / 128, 128, 0, ctx->stream>>>(a);
    knn_far_kernel<KMAX><<<ctx->sm_count * 8, 128, 0, ctx->stream>>>(a);
}

extern "C" int vetr_knn_radius(vetr_ctx* ctx, const float* position, int position_stride, int n, int k, float* radius, int radius_stride)
{
    if (!ctx || n < 0 || k < 1 || k > kKnnMaxK || position_stride < 3 || radius_stride < 1) return VETR_E_INVALID_ARG;
    if (n == 0) return VETR_OK;
    if (!position || !radius) return VETR_E_INVALID_ARG;
    VETR_CUDA(ctx, cudaSetDevice(ctx->device));
    PassScope scope(ctx, VETR_T_KNN, 0);
    cudaStream_t st = ctx->stream;
    if (n > ctx->knn_cap_points)
    {
        cudaFree(ctx->knn_sorted), cudaFree(ctx->knn_point_cell), cudaFree(ctx->knn_queue);
        ctx->knn_sorted = nullptr, ctx->knn_point_cell = nullptr, ctx->knn_queue = nullptr, ctx->knn_cap_points = 0;
        VETR_CUDA(ctx, cudaMalloc(&ctx->knn_sorted, (size_t)n * sizeof(float4)));
        VETR_CUDA(ctx, cudaMalloc(&ctx->knn_point_cell, (size_t)n * sizeof(int)));
        VETR_CUDA(ctx, cudaMalloc(&ctx->knn_queue, (size_t)n * sizeof(int)));
        ctx->knn_cap_points = n;
    }
    if (!ctx->knn_tile_sums) VETR_CUDA(ctx, cudaMalloc(&ctx->knn_tile_sums, (16384 + 16) * sizeof(int)));
    unsigned* d_bounds          = reinterpret_cast<unsigned*>(ctx->knn_tile_sums + 16384);
    unsigned long long* d_occ   = reinterpret_cast<unsigned long long*>(ctx->knn_tile_sums + 16384 + 8);
    int* d_queue_count          = ctx->knn_tile_sums + 16384 + 10;

    // bounding box
    const unsigned init[6] = {0xffffffffu, 0xffffffffu, 0xffffffffu, 0u, 0u, 0u};
    unsigned keys[6];
    VETR_CUDA(ctx, cudaMemcpyAsync(d_bounds, init, sizeof(init), cudaMemcpyHostToDevice, st));
    const int sweep = std::min((n + 255) / 256, ctx->sm_count * 8);
    knn_bounds_kernel<<<sweep, 256, 0, st>>>(position, position_stride, n, d_bounds);
    VETR_CUDA(ctx, cudaMemcpyAsync(keys, d_bounds, sizeof(keys), cudaMemcpyDeviceToHost, st));
    VETR_CUDA(ctx, cudaStreamSynchronize(st));
    float lo[3], hi[3], ext = 0.f, maxabs = 0.f;
    for (int a = 0; a < 3; ++a)
    {
        lo[a] = knn_unkey(keys[a]), hi[a] = knn_unkey(keys[3 + a]);
        if (!(lo[a] <= hi[a]) || std::isinf(lo[a]) || std::isinf(hi[a])) return VETR_E_INVALID_ARG;  // NaN or infinite coordinates
        ext    = std::max(ext, hi[a] - lo[a]);
        maxabs = std::max(maxabs, std::max(std::fabs(lo[a]), std::fabs(hi[a])));
    }

    // cell size: halve from 1/32 of the longest extent until an occupied cell holds 8 points or fewer on average
    KnnGrid g;
    g.ox = lo[0], g.oy = lo[1], g.oz = lo[2];
    auto dims_for = [&](float cell, int d[3]) -> long long
    {
        long long cells = 1;
        for (int a = 0; a < 3; ++a)
        {
            const double c = std::floor((double)(hi[a] - lo[a]) / cell) + 1.0;
            d[a] = (int)std::min(c, 1.0e9);
            cells = cells > (1ll << 40) ? cells : cells * d[a];
        }
        return cells;
    };
    float cell = ext > 0.f ? ext / 32.f : 1.f;
    int d[3];
    long long cells = dims_for(cell, d);
    for (int iter = 0; iter < 24 && ext > 0.f; ++iter)
    {
        if (cells > ctx->knn_cap_cells)
        {
            cudaFree(ctx->knn_starts), cudaFree(ctx->knn_ends);
            ctx->knn_starts = nullptr, ctx->knn_ends = nullptr, ctx->knn_cap_cells = 0;
            const long long cap = std::min(kKnnMaxCells, std::max(cells * 8, 1ll << 20));
            VETR_CUDA(ctx, cudaMalloc(&ctx->knn_starts, (size_t)cap * sizeof(int)));
            VETR_CUDA(ctx, cudaMalloc(&ctx->knn_ends, (size_t)cap * sizeof(int)));
            ctx->knn_cap_cells = cap;
        }
        g.cell = cell, g.inv_cell = 1.f / cell, g.nx = d[0], g.ny = d[1], g.nz = d[2];
        VETR_CUDA(ctx, cudaMemsetAsync(ctx->knn_starts, 0, (size_t)cells * sizeof(int), st));
        VETR_CUDA(ctx, cudaMemsetAsync(d_occ, 0, sizeof(unsigned long long), st));
        knn_count_kernel<<<sweep, 256, 0, st>>>(position, position_stride, n, g, ctx->knn_starts, nullptr);
        knn_occupied_kernel<<<(int)std::min<long long>((cells + 255) / 256, ctx->sm_count * 16), 256, 0, st>>>(ctx->knn_starts, cells, d_occ);
        unsigned long long occupied = 0;
        VETR_CUDA(ctx, cudaMemcpyAsync(&occupied, d_occ, sizeof(occupied), cudaMemcpyDeviceToHost, st));
        VETR_CUDA(ctx, cudaStreamSynchronize(st));
        ctx->launches += 2;
        if (occupied == 0 || (double)n / (double)occupied <= 8.0) break;
        int d2[3];
        const long long finer = dims_for(cell * 0.5f, d2);
        if (finer > kKnnMaxCells) break;
        cell *= 0.5f, cells = finer;
        d[0] = d2[0], d[1] = d2[1], d[2] = d2[2];
    }
    if (cells > ctx->knn_cap_cells)  // only when all points coincide (no iteration ran)
    {
        cudaFree(ctx->knn_starts), cudaFree(ctx->knn_ends);
        ctx->knn_starts = nullptr, ctx->knn_ends = nullptr, ctx->knn_cap_cells = 0;
        VETR_CUDA(ctx, cudaMalloc(&ctx->knn_starts, (size_t)(1ll << 20) * sizeof(int)));
        VETR_CUDA(ctx, cudaMalloc(&ctx->knn_ends, (size_t)(1ll << 20) * sizeof(int)));
        ctx->knn_cap_cells = 1ll << 20;
    }
    g.cell = cell, g.inv_cell = 1.f / cell, g.nx = d[0], g.ny = d[1], g.nz = d[2];

    // counting sort into the chosen grid
    const int n_tiles = (int)((cells + kKnnScanTile - 1) / kKnnScanTile);
    VETR_CUDA(ctx, cudaMemsetAsync(ctx->knn_starts, 0, (size_t)cells * sizeof(int), st));
    VETR_CUDA(ctx, cudaMemsetAsync(d_queue_count, 0, sizeof(int), st));
    knn_count_kernel<<<sweep, 256, 0, st>>>(position, position_stride, n, g, ctx->knn_starts, ctx->knn_point_cell);
    knn_tile_sums_kernel<<<n_tiles, 256, 0, st>>>(ctx->knn_starts, cells, ctx->knn_tile_sums);
    knn_spine_kernel<<<1, 1024, 0, st>>>(ctx->knn_tile_sums, n_tiles);
    knn_apply_kernel<<<n_tiles, 256, 0, st>>>(ctx->knn_starts, cells, ctx->knn_tile_sums, ctx->knn_starts);
    VETR_CUDA(ctx, cudaMemcpyAsync(ctx->knn_ends, ctx->knn_starts, (size_t)cells * sizeof(int), cudaMemcpyDeviceToDevice, st));
    knn_scatter_kernel<<<sweep, 256, 0, st>>>(position, position_stride, n, ctx->knn_point_cell, ctx->knn_ends, ctx->knn_sorted);

    // search
    KnnSearch a;
    a.g = g, a.sorted = ctx->knn_sorted, a.starts = ctx->knn_starts, a.ends = ctx->knn_ends, a.n = n;
    const int k1 = std::min(k, n - 1) + 1;  // list entries that count: the point itself and its k nearest
    a.slack = 1e-3f * cell + 4e-6f * (maxabs + ext);
    a.radius = radius, a.radius_stride = radius_stride, a.queue = ctx->knn_queue, a.queue_count = d_queue_count;
    if (k1 <= 5)
        a.dummies = 5 - k1, knn_launch_search<5>(ctx, a);
    else if (k1 <= 9)
        a.dummies = 9 - k1, knn_launch_search<9>(ctx, a);
    else
        a.dummies = 17 - k1, knn_launch_search<17>(ctx, a);
    ctx->launches += 8;
    VETR_CUDA(ctx, cudaGetLastError());
    return VETR_OK;
}

extern "C" int vetr_remove_points_plan(vetr_ctx* ctx, int n, const int64_t* remove, int m, int32_t* new_index, int* n_kept)
{
    if (!ctx || n < 0 || m < 0 || !n_kept || (n > 0 && !new_index) || (m > 0 && !remove)) return VETR_E_INVALID_ARG;
    if ((long long)n > kKnnMaxCells) return VETR_E_TOO_LARGE;  // one spine block scans 16384 tiles of 4096 flags
    *n_kept = 0;
    if (n == 0) return m == 0 ? VETR_OK : VETR_E_INVALID_ARG;
    VETR_CUDA(ctx, cudaSetDevice(ctx->device));
    cudaStream_t st = ctx->stream;
    if (n > ctx->points_cap)
    {
        cudaFree(ctx->points_flags);
        ctx->points_flags = nullptr, ctx->points_cap = 0;
        VETR_CUDA(ctx, cudaMalloc(&ctx->points_flags, (size_t)n * sizeof(int) + 16));
        ctx->points_cap = n;
    }
    if (!ctx->knn_tile_sums) VETR_CUDA(ctx, cudaMalloc(&ctx->knn_tile_sums, (16384 + 16) * sizeof(int)));
    int* d_small = ctx->knn_tile_sums + 16384 + 12;  // {bad index flag, survivors}
    VETR_CUDA(ctx, cudaMemsetAsync(d_small, 0, 2 * sizeof(int), st));
    const int sweep = std::min((n + 255) / 256, ctx->sm_count * 8);
    const int n_tiles = (n + kKnnScanTile - 1) / kKnnScanTile;
    points_fill_kernel<<<sweep, 256, 0, st>>>(ctx->points_flags, n, 1);
    if (m > 0) points_mark_removed_kernel<<<std::min((m + 255) / 256, ctx->sm_count * 8), 256, 0, st>>>((const long long*)remove, m, n, ctx->points_flags, d_small);
    knn_tile_sums_kernel<<<n_tiles, 256, 0, st>>>(ctx->points_flags, n, ctx->knn_tile_sums);
    knn_spine_kernel<<<1, 1024, 0, st>>>(ctx->knn_tile_sums, n_tiles);
    knn_apply_kernel<<<n_tiles, 256, 0, st>>>(ctx->points_flags, n, ctx->knn_tile_sums, new_index);
    points_new_index_kernel<<<sweep, 256, 0, st>>>(ctx->points_flags, n, new_index, d_small + 1);
    ctx->launches += 6;
    int host[2] = {0, 0};
    VETR_CUDA(ctx, cudaMemcpyAsync(host, d_small, sizeof(host), cudaMemcpyDeviceToHost, st));
    VETR_CUDA(ctx, cudaStreamSynchronize(st));
    if (host[0]) return VETR_E_INVALID_ARG;
    *n_kept = host[1];
    return VETR_OK;
}

extern "C" int vetr_gather_points(vetr_ctx* ctx, int n, int n_kept, const int32_t* new_index, const vetr_point_array* arrays, int n_arrays)
{
    if (!ctx || n < 0 || n_kept < 0 || n_kept > n || n_arrays < 0 || (n_arrays > 0 && !arrays) || (n > 0 && !new_index))
        return VETR_E_INVALID_ARG;
    for (int k = 0; k < n_arrays; ++k)
    {
        const vetr_point_array& a = arrays[k];
        if (a.rows < 1 || a.width < 1 || (n > 0 && !a.src) || (n_kept > 0 && !a.dst)) return VETR_E_INVALID_ARG;
        if (a.width == 4 && ((((uintptr_t)a.src | (uintptr_t)a.dst) & 15) != 0)) return VETR_E_INVALID_ARG;
    }
    if (n == 0 || n_kept == 0) return VETR_OK;
    VETR_CUDA(ctx, cudaSetDevice(ctx->device));
    for (int k = 0; k < n_arrays; ++k)
    {
        const vetr_point_array& a = arrays[k];
        const long long total = (long long)a.rows * n;
        const int blocks = (int)std::min<long long>((total + 255) / 256, (long long)ctx->sm_count * 16);
        points_gather_kernel<<<blocks, 256, 0, ctx->stream>>>((const uint32_t*)a.src, (uint32_t*)a.dst, new_index, n, n_kept, a.rows, a.width);
        ctx->launches += 1;
    }
    VETR_CUDA(ctx, cudaGetLastError());
    return VETR_OK;
}

extern "C" int vetr_l1_loss_grad(vetr_ctx* ctx, int num_levels, const float* const* image, const float* const* target,
                                 float* const* grad, const int64_t* numel, float* loss)
{
    if (!ctx || num_levels < 1 || num_levels > VETR_MAX_LAYERS || !image || !target || !grad || !numel || !loss)
        return VETR_E_INVALID_ARG;
    L1Args a;
    memset(&a, 0, sizeof(a));
    long long run = 0;
    for (int l = 0; l < num_levels; ++l)
    {
        if (!image[l] || !target[l] || !grad[l] || numel[l] < 1) return VETR_E_INVALID_ARG;
        if ((((uintptr_t)image[l] | (uintptr_t)target[l] | (uintptr_t)grad[l]) & 15) != 0) return VETR_E_INVALID_ARG;
        a.image[l] = image[l], a.target[l] = target[l], a.grad[l] = grad[l];
        run += numel[l];
        a.end[l]       = run;
        a.inv_numel[l] = 1.f / (float)numel[l];
    }
    a.levels = num_levels, a.loss = loss;
    VETR_CUDA(ctx, cudaSetDevice(ctx->device));
    VETR_CUDA(ctx, cudaMemsetAsync(loss, 0, sizeof(float), ctx->stream));
    ctx->launches += 1;
    l1_loss_grad_kernel<<<ctx->sm_count * 8, 256, 0, ctx->stream>>>(a);
    VETR_CUDA(ctx, cudaGetLastError());
    return VETR_OK;
}

extern "C" int vetr_apply_tangent(vetr_ctx* ctx, double* tangent, double* poses_se3, int n)
{
    if (!ctx || !tangent || !poses_se3 || n < 0) return VETR_E_INVALID_ARG;
    VETR_CUDA(ctx, cudaSetDevice(ctx->device));
    if (n > 0)
    {
        ctx->launches += 1;
        apply_tangent_kernel<<<(n + 127) / 128, 128, 0, ctx->stream>>>(tangent, poses_se3, n);
    }
    VETR_CUDA(ctx, cudaGetLastError());
    return VETR_OK;
}

extern "C" int vetr_read_status(vetr_ctx* ctx, const vetr_lists* lists, int64_t* total_fragments, int32_t* longest_list)
{
    if (!ctx || !lists || !lists->status) return VETR_E_INVALID_ARG;
    int h[4];
    VETR_CUDA(ctx, cudaSetDevice(ctx->device));
    VETR_CUDA(ctx, cudaMemcpyAsync(h, lists->status, sizeof(h), cudaMemcpyDeviceToHost, ctx->stream));
    VETR_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    if (total_fragments) *total_fragments = h[0];
    if (longest_list) *longest_list = h[2];
    if (h[1] & 1) return VETR_E_LIST_OVERFLOW;
    return (h[1] & 2) ? VETR_E_TOO_LARGE : VETR_OK;
}

// ---------------------------------------------------------------------------------------------------------
// Scan without any allocation.
//
// Some hosts must not allocate device memory while they render: an interactive viewer whose frame loop cannot afford
// the device-wide stall of cudaMalloc / cudaFree, a process whose device memory is handed out once at start-up by an
// arena it does not own, or code running inside a region where the driver forbids allocation.  For them the scan's
// only scratch (one partial sum per tile of 4096 pixels) lives in a fixed array inside the library image instead of a
// buffer grown on demand.  Every GPU that loads the library carries these 128 KB until the process exits.
namespace vetr
{
constexpr int kStaticScanTiles = 16384;  // 16384 tiles x 4096 pixels = 67 108 864 pixels per call
static __device__ __align__(256) long long g_static_tile_sums[kStaticScanTiles];
}  // namespace vetr
static long long* g_static_tile_ptr[64] = {};  // device address of the array above, per device ordinal

extern "C" int vetr_scan_counts_static(int device, void* cuda_stream, const int32_t* counts, int64_t n_pixels,
                                       int64_t capacity, int32_t* ends, int32_t* status, int32_t* items,
                                       int64_t items_capacity)
{
    if (device < 0 || device >= 64 || !counts || !ends || !status || !items || n_pixels < 1 || capacity < 0)
        return VETR_E_INVALID_ARG;
    if (n_pixels > 0x7fffffffLL) return VETR_E_TOO_LARGE;
    const long long n_tiles = (n_pixels + kScanTile - 1) / kScanTile;
    if (n_tiles > kStaticScanTiles) return VETR_E_TOO_LARGE;  // more pixels than the fixed scratch covers
    if (items_capacity < vetr_item_table_entries(capacity, n_pixels)) return VETR_E_INVALID_ARG;
    // the launches below go to `device`; the caller's current device is put back before returning
    int caller_device = device;
    if (cudaGetDevice(&caller_device) != cudaSuccess) return VETR_E_CUDA;
    struct RestoreDevice
    {
        int to, from;
        ~RestoreDevice()
        {
            if (to != from) cudaSetDevice(to);
        }
    } restore{caller_device, device};
    if (caller_device != device && cudaSetDevice(device) != cudaSuccess) return VETR_E_CUDA;
    if (!g_static_tile_ptr[device])
    {
        // The array's name is only a handle on the host; kernels need its address on THIS device.
        long long* p = nullptr;
        if (cudaGetSymbolAddress((void**)&p, g_static_tile_sums) != cudaSuccess || !p) return VETR_E_CUDA;
        g_static_tile_ptr[device] = p;
    }
    long long* tile_sums = g_static_tile_ptr[device];
    cudaStream_t st      = (cudaStream_t)cuda_stream;
    // the status words are accumulated into (longest list is an atomic maximum): start them at zero
    if (cudaMemsetAsync(status, 0, 4 * sizeof(int), st) != cudaSuccess) return VETR_E_CUDA;
    scan_tile_sums_kernel<<<(int)n_tiles, 256, 0, st>>>(counts, n_pixels, tile_sums, status);
    scan_spine_kernel<<<1, 1024, 0, st>>>(tile_sums, (int)n_tiles, n_pixels, capacity, status, items);
    scan_apply_kernel<<<(int)n_tiles, 256, 0, st>>>(counts, n_pixels, tile_sums, ends, status, items);
    return cudaGetLastError() == cudaSuccess ? VETR_OK : VETR_E_CUDA;
}

// Parity / debugging: the lists of one (view, level) in the reference's layout.  The reference keeps its lists in
// row-major pixel order; here they are stored in the banded order of the pixel space, so the level is brought to the
// host, reordered there and copied back (a debugging call: it synchronises and is not meant for large scenes).
extern "C" int vetr_get_lists(vetr_ctx* ctx, const vetr_lists* lists, int w, int h, int num_layers, int n_views, int view,
                              int layer, int32_t* out_collections, int32_t* out_scanned_counting, int64_t* n_fragments)
{
    if (!ctx || !lists || num_layers < 1 || num_layers > VETR_MAX_LAYERS || view < 0 || view >= n_views || layer < 0 ||
        layer >= num_layers)
        return VETR_E_INVALID_ARG;
    int lw[VETR_MAX_LAYERS], lh[VETR_MAX_LAYERS];
    long long lbase[VETR_MAX_LAYERS];
    const long long P    = pyramid(w, h, num_layers, lw, lh, lbase);
    const long long g0   = (long long)view * P + lbase[layer];
    const int W = lw[layer], H = lh[layer];
    const long long npad = (long long)W * ((H + kBand - 1) / kBand * kBand);  // pixels of the level in the pixel space
    if ((long long)W * H == 0)
    {
        if (n_fragments) *n_fragments = 0;
        return VETR_OK;
    }
    VETR_CUDA(ctx, cudaSetDevice(ctx->device));
    std::vector<int> counts((size_t)npad), ends((size_t)npad);
    VETR_CUDA(ctx, cudaMemcpyAsync(counts.data(), lists->counts + g0, npad * 4, cudaMemcpyDeviceToHost, ctx->stream));
    VETR_CUDA(ctx, cudaMemcpyAsync(ends.data(), lists->ends + g0, npad * 4, cudaMemcpyDeviceToHost, ctx->stream));
    VETR_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    const long long first = (long long)ends[0] - counts[0];
    const long long n     = (long long)ends[(size_t)npad - 1] - first;
    if (n_fragments) *n_fragments = n;
    if (!out_collections && !out_scanned_counting) return VETR_OK;
    std::vector<uint4> recs;
    if (out_collections && n > 0)
    {
        recs.resize((size_t)(2 * n));
        VETR_CUDA(ctx, cudaMemcpyAsync(recs.data(), (const uint4*)lists->frags + 2 * first, (size_t)n * 32, cudaMemcpyDeviceToHost,
                                       ctx->stream));
        VETR_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    }
    std::vector<int> scanned((size_t)W * H), coll(out_collections ? (size_t)(2 * n) : 0);
    long long run = 0;
    for (int y = 0; y < H; ++y)
        for (int x = 0; x < W; ++x)
        {
            const size_t k = (size_t)(y >> kBandShift) * ((size_t)W << kBandShift) + ((size_t)x << kBandShift) + (y & (kBand - 1));  // pixel_offset
            scanned[(size_t)y * W + x] = (int)run;
            if (out_collections)
                for (int j = 0; j < counts[k]; ++j)
                {
                    const uint4 r = recs[(size_t)(2 * ((long long)ends[k] - counts[k] - first + j))];
                    coll[(size_t)(run + j)]     = (int)r.y;  // row 0: depth bits
                    coll[(size_t)(n + run + j)] = (int)r.x;  // row 1: point index
                }
            run += counts[k];
        }
    if (out_collections && n > 0)
        VETR_CUDA(ctx, cudaMemcpyAsync(out_collections, coll.data(), (size_t)(2 * n) * 4, cudaMemcpyHostToDevice, ctx->stream));
    if (out_scanned_counting)
        VETR_CUDA(ctx, cudaMemcpyAsync(out_scanned_counting, scanned.data(), (size_t)W * H * 4, cudaMemcpyHostToDevice, ctx->stream));
    VETR_CUDA(ctx, cudaStreamSynchronize(ctx->stream));
    return VETR_OK;
}
