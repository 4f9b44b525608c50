// Removing points from a cloud on the device: NeuralScene::RemovePoints (data/NeuralScene.cpp:1156-1239).  The reference
// sorts the indices on the host, builds the list of indices to keep in a host loop (:1169-1181), rebuilds the cloud through
// a CPU mesh (:1191-1193) and index_selects every per-point tensor with the keep list: texture, confidence
// (NeuralTexture.cpp:160-173) and the optimizer's moments (my_adam.cpp:107-135).  Here: flag the removed points, one
// exclusive scan gives every surviving point its new index, and one gather kernel per tensor copies the survivors, in
// their old order, exactly as index_select with the sorted keep list does.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace vetr
{
// flags[i] = 0 for every listed point (duplicates allowed); an index outside [0, n) sets *bad.
__global__ void __launch_bounds__(256) points_mark_removed_kernel(const long long* __restrict__ remove, int m, int n, int* flags, int* bad)
{
    for (int j = blockIdx.x * 256 + threadIdx.x; j < m; j += gridDim.x * 256)
    {
        const long long i = remove[j];
        if (i < 0 || i >= n)
            *bad = 1;
        else
            flags[i] = 0;
    }
}

__global__ void __launch_bounds__(256) points_fill_kernel(int* a, int n, int v)
{
    for (int i = blockIdx.x * 256 + threadIdx.x; i < n; i += gridDim.x * 256) a[i] = v;
}

// new_index[i] (the exclusive scan of the flags on entry) becomes -1 for removed points; *n_kept = survivors.
__global__ void __launch_bounds__(256) points_new_index_kernel(const int* __restrict__ flags, int n, int* new_index, int* n_kept)
{
    for (int i = blockIdx.x * 256 + threadIdx.x; i < n; i += gridDim.x * 256)
    {
        const int f = flags[i], s = new_index[i];
        if (i == n - 1) *n_kept = s + f;
        if (!f) new_index[i] = -1;
    }
}

// dst[r, new_index[i], :] = src[r, i, :] for the survivors; arrays are [rows, points, width] of 4-byte elements.
__global__ void __launch_bounds__(256) points_gather_kernel(const uint32_t* __restrict__ src, uint32_t* __restrict__ dst,
                                                            const int* __restrict__ new_index, int n, int n_kept, int rows, int width)
{
    const long long total = (long long)rows * n;
    for (long long t = (long long)blockIdx.x * 256 + threadIdx.x; t < total; t += (long long)gridDim.x * 256)
    {
        const int r = (int)(t / n), i = (int)(t - (long long)r * n);
        const int j = new_index[i];
        if (j < 0) continue;
        const uint32_t* s = src + ((long long)r * n + i) * width;
        uint32_t* d       = dst + ((long long)r * n_kept + j) * width;
        if (width == 4)
            *reinterpret_cast<uint4*>(d) = *reinterpret_cast<const uint4*>(s);  // [N,4] rows are 16-byte aligned by contract
        else
            for (int e = 0; e < width; ++e) d[e] = s[e];
    }
}
}  // namespace vetr
