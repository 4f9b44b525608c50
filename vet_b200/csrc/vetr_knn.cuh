// Drop-out radius of a point cloud: SceneData::ComputeRadius (data/SceneData.cpp:554-597), the distance from every point
// to its k-th nearest other point.  The reference builds a KD-tree on the host and queries it per point; here the points
// are binned into a uniform grid by a counting sort (count per cell, exclusive scan, scatter), and every point searches
// the cells around its own in growing cubes until the k-th nearest distance found so far is smaller than the distance to
// the cube's faces, beyond which nothing has been looked at.  Most points end after the first cube of 3 x 3 x 3 cells,
// with one thread per point; the rest (isolated points, whose cubes grow to tens of cells a side) go to a queue and are
// finished by one warp per point, whose lanes split the rows of a cube that grows by half from stage to stage.
//
// The result is the (k+1)-th smallest of a multiset of fp32 squared distances, each formed as (dx dx + dy dy) + dz dz
// without contraction, so it does not depend on the order in which candidates are met and is bit-equal to an all-pairs
// evaluation on the host.
#pragma once
#include <cuda_runtime.h>
#include <math_constants.h>
#include <stdint.h>

namespace vetr
{
constexpr int kKnnMaxK       = 16;
constexpr int kKnnScanTile   = 4096;       // cells per thread block of the scan (256 threads x 16)
constexpr long long kKnnMaxCells = 1ll << 26;  // 64 Mi cells: 16384 scan tiles, one spine block

struct KnnGrid
{
    float ox, oy, oz;  // origin: the cloud's minimum corner
    float cell, inv_cell;
    int nx, ny, nz;
};

// Order-preserving map between floats and unsigned integers, for atomicMin / atomicMax on coordinates.
__device__ __forceinline__ unsigned knn_key(float f)
{
    const unsigned b = __float_as_uint(f);
    return (b & 0x80000000u) ? ~b : (b | 0x80000000u);
}
__host__ __device__ inline float knn_unkey(unsigned k)
{
    const unsigned b = (k & 0x80000000u) ? (k & 0x7fffffffu) : ~k;
#ifdef __CUDA_ARCH__
    return __uint_as_float(b);
#else
    float f;
    memcpy(&f, &b, 4);
    return f;
#endif
}

// bounds[0..2] = min keys (initialised to 0xffffffff), bounds[3..5] = max keys (initialised to 0)
__global__ void __launch_bounds__(256) knn_bounds_kernel(const float* __restrict__ pos, int stride, int n, unsigned* bounds)
{
    unsigned lo[3] = {0xffffffffu, 0xffffffffu, 0xffffffffu}, hi[3] = {0u, 0u, 0u};
    for (int i = blockIdx.x * 256 + threadIdx.x; i < n; i += gridDim.x * 256)
    {
        const float* p = pos + (size_t)i * stride;
#pragma unroll
        for (int a = 0; a < 3; ++a)
        {
            const unsigned k = knn_key(p[a]);
            lo[a] = min(lo[a], k), hi[a] = max(hi[a], k);
        }
    }
#pragma unroll
    for (int a = 0; a < 3; ++a)
    {
        for (int o = 16; o > 0; o >>= 1)
        {
            lo[a] = min(lo[a], __shfl_xor_sync(0xffffffffu, lo[a], o));
            hi[a] = max(hi[a], __shfl_xor_sync(0xffffffffu, hi[a], o));
        }
        if ((threadIdx.x & 31) == 0)
        {
            atomicMin(bounds + a, lo[a]);
            atomicMax(bounds + 3 + a, hi[a]);
        }
    }
}

__device__ __forceinline__ int knn_cell_coord(float p, float origin, float inv_cell, int n)
{
    const float c = floorf((p - origin) * inv_cell);
    return (int)fminf(fmaxf(c, 0.f), (float)(n - 1));  // also sends NaN to cell 0: every access stays inside the grid
}

__device__ __forceinline__ int knn_cell_of(const KnnGrid& g, float x, float y, float z, int& cx, int& cy, int& cz)
{
    cx = knn_cell_coord(x, g.ox, g.inv_cell, g.nx);
    cy = knn_cell_coord(y, g.oy, g.inv_cell, g.ny);
    cz = knn_cell_coord(z, g.oz, g.inv_cell, g.nz);
    return (cz * g.ny + cy) * g.nx + cx;
}

// counts[cell] += 1 for every point; point_cell[i] = its cell.
__global__ void __launch_bounds__(256) knn_count_kernel(const float* __restrict__ pos, int stride, int n, const __grid_constant__ KnnGrid g,
                                                        int* counts, int* point_cell)
{
    for (int i = blockIdx.x * 256 + threadIdx.x; i < n; i += gridDim.x * 256)
    {
        const float* p = pos + (size_t)i * stride;
        int cx, cy, cz;
        const int c = knn_cell_of(g, p[0], p[1], p[2], cx, cy, cz);
        if (point_cell) point_cell[i] = c;
        atomicAdd(counts + c, 1);
    }
}

// Number of non-empty cells (the cell size is chosen from the points per occupied cell).
__global__ void __launch_bounds__(256) knn_occupied_kernel(const int* __restrict__ counts, long long n_cells, unsigned long long* occupied)
{
    int mine = 0;
    for (long long i = (long long)blockIdx.x * 256 + threadIdx.x; i < n_cells; i += (long long)gridDim.x * 256) mine += counts[i] > 0;
    for (int o = 16; o > 0; o >>= 1) mine += __shfl_xor_sync(0xffffffffu, mine, o);
    if ((threadIdx.x & 31) == 0 && mine) atomicAdd(occupied, (unsigned long long)mine);
}

// Exclusive scan of the cell counts in three kernels: sums of tiles, scan of the tile sums by one block, scan inside the tiles.
__global__ void __launch_bounds__(256) knn_tile_sums_kernel(const int* __restrict__ counts, long long n_cells, int* tile_sums)
{
    const long long base = (long long)blockIdx.x * kKnnScanTile;
    int s = 0;
    for (int k = threadIdx.x; k < kKnnScanTile; k += 256)
        if (base + k < n_cells) s += counts[base + k];
    __shared__ int part[8];
    for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(0xffffffffu, s, o);
    if ((threadIdx.x & 31) == 0) part[threadIdx.x >> 5] = s;
    __syncthreads();
    if (threadIdx.x == 0)
    {
        int t = 0;
        for (int w = 0; w < 8; ++w) t += part[w];
        tile_sums[blockIdx.x] = t;
    }
}

__global__ void __launch_bounds__(1024) knn_spine_kernel(int* tile_sums, int n_tiles)
{
    // 1024 threads x 16 consecutive tiles each = 16384 tiles at most
    __shared__ int warp_tot[32];
    const int first = threadIdx.x * 16;
    int local[16], s = 0;
#pragma unroll
    for (int k = 0; k < 16; ++k)
    {
        local[k] = first + k < n_tiles ? tile_sums[first + k] : 0;
        s += local[k];
    }
    int incl = s;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int o = 1; o < 32; o <<= 1)
    {
        const int v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
    }
    if (lane == 31) warp_tot[warp] = incl;
    __syncthreads();
    if (warp == 0)
    {
        int w = warp_tot[lane], wi = w;
        for (int o = 1; o < 32; o <<= 1)
        {
            const int v = __shfl_up_sync(0xffffffffu, wi, o);
            if (lane >= o) wi += v;
        }
        warp_tot[lane] = wi - w;  // exclusive
    }
    __syncthreads();
    int run = warp_tot[warp] + incl - s;
#pragma unroll
    for (int k = 0; k < 16; ++k)
        if (first + k < n_tiles)
        {
            tile_sums[first + k] = run;
            run += local[k];
        }
}

// starts[cell] = exclusive scan of counts (in place is allowed: starts may alias counts).
__global__ void __launch_bounds__(256) knn_apply_kernel(const int* counts, long long n_cells, const int* __restrict__ tile_sums, int* starts)
{
    __shared__ int warp_tot[8];
    const long long base = (long long)blockIdx.x * kKnnScanTile + threadIdx.x * 16;
    int local[16], s = 0;
#pragma unroll
    for (int k = 0; k < 16; ++k)
    {
        local[k] = base + k < n_cells ? counts[base + k] : 0;
        s += local[k];
    }
    int incl = s;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    for (int o = 1; o < 32; o <<= 1)
    {
        const int v = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += v;
    }
    if (lane == 31) warp_tot[warp] = incl;
    __syncthreads();
    int before = 0;
    for (int w = 0; w < warp; ++w) before += warp_tot[w];
    int run = tile_sums[blockIdx.x] + before + incl - s;
#pragma unroll
    for (int k = 0; k < 16; ++k)
        if (base + k < n_cells)
        {
            starts[base + k] = run;
            run += local[k];
        }
}

// Counting sort, last step: sorted[slot] = (x, y, z, index bits); cursor[cell] starts at the cell's first slot and ends
// at its last + 1.
__global__ void __launch_bounds__(256) knn_scatter_kernel(const float* __restrict__ pos, int stride, int n, const int* __restrict__ point_cell,
                                                          int* cursor, float4* sorted)
{
    for (int i = blockIdx.x * 256 + threadIdx.x; i < n; i += gridDim.x * 256)
    {
        const float* p = pos + (size_t)i * stride;
        const int slot = atomicAdd(cursor + point_cell[i], 1);
        sorted[slot]   = make_float4(p[0], p[1], p[2], __int_as_float(i));
    }
}

struct KnnSearch
{
    KnnGrid g;
    const float4* sorted;
    const int* starts;  // first slot of a cell
    const int* ends;    // last slot + 1
    int n;
    int dummies;   // list entries pre-filled with -inf so that the (k+1)-th smallest distance sits in the last entry
    float slack;   // rounding allowance of the cube-face distances
    float* radius;
    int radius_stride;
    int* queue;        // sorted indices of the points the first pass could not finish
    int* queue_count;
};

// best[] ascending; inserts d and drops the largest.
template <int KMAX>
__device__ __forceinline__ void knn_insert(float (&best)[KMAX], float d)
{
    float v = d;
#pragma unroll
    for (int j = 0; j < KMAX; ++j)
    {
        const float lo = fminf(best[j], v);
        v              = fmaxf(best[j], v);
        best[j]        = lo;
    }
}

template <int KMAX>
__device__ __forceinline__ void knn_scan_slots(const KnnSearch& a, int b, int e, float x, float y, float z, float (&best)[KMAX])
{
    for (int j = b; j < e; ++j)
    {
        const float4 q = __ldg(a.sorted + j);
        const float dx = x - q.x, dy = y - q.y, dz = z - q.z;
        const float d  = dx * dx + dy * dy + dz * dz;
        if (d < best[KMAX - 1]) knn_insert<KMAX>(best, d);
    }
}

// Distance from p to the nearest face of the cube of cells [c - r, c + r]^3 behind which unvisited cells remain
// (+inf if the cube covers the grid), minus the rounding allowance.
__device__ __forceinline__ float knn_margin(const KnnSearch& a, float x, float y, float z, int cx, int cy, int cz, int r)
{
    float m = CUDART_INF_F;
    const KnnGrid& g = a.g;
    if (cx - r > 0) m = fminf(m, x - (g.ox + (float)(cx - r) * g.cell));
    if (cx + r < g.nx - 1) m = fminf(m, (g.ox + (float)(cx + r + 1) * g.cell) - x);
    if (cy - r > 0) m = fminf(m, y - (g.oy + (float)(cy - r) * g.cell));
    if (cy + r < g.ny - 1) m = fminf(m, (g.oy + (float)(cy + r + 1) * g.cell) - y);
    if (cz - r > 0) m = fminf(m, z - (g.oz + (float)(cz - r) * g.cell));
    if (cz + r < g.nz - 1) m = fminf(m, (g.oz + (float)(cz + r + 1) * g.cell) - z);
    return m - a.slack;
}

__device__ __forceinline__ bool knn_done(float kth_d2, float margin) { return margin > 0.f && kth_d2 <= margin * margin; }

// First pass: one thread per point (in cell order, so that a warp's points share their cells), the cube of 3^3 cells.
template <int KMAX>
__global__ void __launch_bounds__(128) knn_near_kernel(const __grid_constant__ KnnSearch a)
{
    const int i = blockIdx.x * 128 + threadIdx.x;
    if (i >= a.n) return;
    const float4 p = a.sorted[i];
    int cx, cy, cz;
    knn_cell_of(a.g, p.x, p.y, p.z, cx, cy, cz);
    float best[KMAX];
#pragma unroll
    for (int j = 0; j < KMAX; ++j) best[j] = j < a.dummies ? -CUDART_INF_F : CUDART_INF_F;
    const int x0 = max(cx - 1, 0), x1 = min(cx + 1, a.g.nx - 1);
    for (int z = max(cz - 1, 0); z <= min(cz + 1, a.g.nz - 1); ++z)
        for (int y = max(cy - 1, 0); y <= min(cy + 1, a.g.ny - 1); ++y)
        {
            const int row = (z * a.g.ny + y) * a.g.nx;
            knn_scan_slots<KMAX>(a, a.starts[row + x0], a.ends[row + x1], p.x, p.y, p.z, best);  // x-neighbours are contiguous
        }
    if (knn_done(best[KMAX - 1], knn_margin(a, p.x, p.y, p.z, cx, cy, cz, 1)))
        a.radius[(size_t)__float_as_int(p.w) * a.radius_stride] = sqrtf(best[KMAX - 1]);
    else
        a.queue[atomicAdd(a.queue_count, 1)] = i;
}

// Second pass: one warp per queued point.  The cube [c - R, c + R]^3 grows its half-width R by half from stage to stage.  The
// rows (y, z) of the cube that lie inside the grid are dealt to the lanes; the cells of a row are consecutive in the sorted
// array, so a row costs one or two range look-ups whatever its length: the whole row if it lies outside the previous
// cube, else the two pieces left and right of it.  After each stage the lanes' lists are merged into the k+1 smallest
// overall and the stopping rule is applied to the cube's faces.
template <int KMAX>
__global__ void __launch_bounds__(128) knn_far_kernel(const __grid_constant__ KnnSearch a)
{
    const int lane = threadIdx.x & 31;
    const int n_q  = *a.queue_count;
    for (int w = blockIdx.x * 4 + (threadIdx.x >> 5); w < n_q; w += gridDim.x * 4)
    {
        const float4 p = a.sorted[a.queue[w]];
        int cx, cy, cz;
        knn_cell_of(a.g, p.x, p.y, p.z, cx, cy, cz);
        float best[KMAX];
#pragma unroll
        for (int j = 0; j < KMAX; ++j) best[j] = (lane == 0 && j < a.dummies) ? -CUDART_INF_F : CUDART_INF_F;
        const int r_max = max(max(max(cx, a.g.nx - 1 - cx), max(cy, a.g.ny - 1 - cy)), max(cz, a.g.nz - 1 - cz));
        int r_prev = -1;  // half-width of the cube already visited (-1: nothing yet)
        for (int r = 1;; r = min(r + max(r / 2, 1), max(r_max, 1)))  // 1, 2, 3, 4, 6, 9, 13, ...
        {
            const int ylo = max(cy - r, 0), yhi = min(cy + r, a.g.ny - 1), zlo = max(cz - r, 0), zhi = min(cz + r, a.g.nz - 1);
            const int wz = zhi - zlo + 1, rows = (yhi - ylo + 1) * wz;  // <= ny nz <= 2^26
            const int x0 = max(cx - r, 0), x1 = min(cx + r, a.g.nx - 1);
            for (int t = lane; t < rows; t += 32)
            {
                const int y = ylo + t / wz, z = zlo + t % wz;
                const int row = (z * a.g.ny + y) * a.g.nx;
                if (abs(y - cy) > r_prev || abs(z - cz) > r_prev)
                    knn_scan_slots<KMAX>(a, a.starts[row + x0], a.ends[row + x1], p.x, p.y, p.z, best);
                else
                {
                    const int left = cx - r_prev - 1, right = cx + r_prev + 1;  // the cells next to the visited piece
                    if (left >= x0) knn_scan_slots<KMAX>(a, a.starts[row + x0], a.ends[row + left], p.x, p.y, p.z, best);
                    if (right <= x1) knn_scan_slots<KMAX>(a, a.starts[row + right], a.ends[row + x1], p.x, p.y, p.z, best);
                }
            }
            // merge: KMAX times, take the smallest head of all lanes
            float merged[KMAX];
#pragma unroll
            for (int j = 0; j < KMAX; ++j)
            {
                float m = best[0];
                for (int o = 16; o > 0; o >>= 1) m = fminf(m, __shfl_xor_sync(0xffffffffu, m, o));
                const unsigned holders = __ballot_sync(0xffffffffu, best[0] == m);
                if (lane == __ffs(holders) - 1)
                {
#pragma unroll
                    for (int q = 0; q + 1 < KMAX; ++q) best[q] = best[q + 1];
                    best[KMAX - 1] = CUDART_INF_F;
                }
                merged[j] = m;
            }
#pragma unroll
            for (int j = 0; j < KMAX; ++j) best[j] = lane == 0 ? merged[j] : CUDART_INF_F;
            const float kth = merged[KMAX - 1];
            if (r >= r_max || knn_done(kth, knn_margin(a, p.x, p.y, p.z, cx, cy, cz, r)))
            {
                if (lane == 0) a.radius[(size_t)__float_as_int(p.w) * a.radius_stride] = sqrtf(kth);
                break;
            }
            r_prev = r;
        }
    }
}

}  // namespace vetr
