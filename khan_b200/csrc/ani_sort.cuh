// AniSort on the device: stable sort of a batch's atoms by element id (a 2-bit key), returned
// as the three index arrays of the reference op (gpu_featurizer/ani_sort.cpp:71-115):
//   scatter[i] = rank of atom i among atoms of its element, gather[i] = element start + rank,
//   counts[4].
//
// The batch is cut into tiles of kSortTile consecutive atoms, one CTA per tile.  Inside a tile
// the rank is a warp-level split: each warp ranks its 32-atom segments with one ballot per
// element and a popc of the lanes below, and segment/warp bases come from a small scan in
// shared memory.  What differs between the two variants is where a tile learns how many atoms
// of each element precede it:
//   * single launch (batches up to kSortSingleLaunchMax atoms): every CTA recounts the atoms
//     in front of its tile straight from the (L2-resident) input, so no scratch memory and
//     no second launch are needed;
//   * three launches (any size): a histogram kernel writes per-tile counts to a scratch
//     array of (tiles + 1) x 4 ints, one CTA scans it in place, and the ranking kernel reads
//     the scanned entry of its tile.
#pragma once

#include "ani_common.cuh"

namespace ani {

constexpr int kSortThreads = 256;
constexpr int kSortItems = 4;                                  // atoms per thread (one int4)
constexpr int kSortTile = kSortThreads * kSortItems;           // 1024 atoms per CTA
constexpr int kSortSingleLaunchMax = 64 * kSortTile;           // 65536 atoms

struct Count4 {
    int c[kTypes];
};

__device__ __forceinline__ int checked_type(int t)
{
    if (t < 0 || t >= kTypes) {
        report(ANI_ERR_BAD_ELEMENT);
        t &= 3;
    }
    return t;
}

__device__ __forceinline__ void tally(Count4& v, int t)
{
    t = checked_type(t);
#pragma unroll
    for (int g = 0; g < kTypes; g++) v.c[g] += (t == g) ? 1 : 0;
}

// Sum of per-thread Count4 over the CTA; result valid in every thread.
__device__ __forceinline__ Count4 block_sum(Count4 v, int (*red)[kTypes])
{
    const int lane = lane_id(), warp = warp_id();
#pragma unroll
    for (int g = 0; g < kTypes; g++) {
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) v.c[g] += __shfl_xor_sync(kFull, v.c[g], o);
        if (lane == 0) red[warp][g] = v.c[g];
    }
    __syncthreads();
    Count4 out;
#pragma unroll
    for (int g = 0; g < kTypes; g++) {
        int s = 0;
#pragma unroll
        for (int w = 0; w < kSortThreads / kWarp; w++) s += red[w][g];
        out.c[g] = s;
    }
    __syncthreads();
    return out;
}

// Count the elements of types[lo, hi) with the whole CTA (vectorised where aligned).
__device__ __forceinline__ Count4 count_range(const int* __restrict__ types, int lo, int hi)
{
    Count4 v = {{0, 0, 0, 0}};
    // lo is a multiple of kSortTile, so the vector path only needs an aligned base pointer.
    const bool aligned = (reinterpret_cast<uintptr_t>(types + lo) & 15u) == 0;
    const int nvec = aligned ? (hi - lo) / 4 : 0;
    const int4* p4 = reinterpret_cast<const int4*>(types + lo);
    for (int k = threadIdx.x; k < nvec; k += kSortThreads) {
        const int4 q = p4[k];
        tally(v, q.x);
        tally(v, q.y);
        tally(v, q.z);
        tally(v, q.w);
    }
    for (int k = lo + nvec * 4 + threadIdx.x; k < hi; k += kSortThreads) tally(v, types[k]);
    return v;
}

// Ranks the atoms of tile `tile` given the per-element counts in front of the tile (`before`)
// and in the whole batch (`total`).
__device__ __forceinline__ void rank_tile(const int* __restrict__ types, int n_atoms, int tile,
                                          const Count4& before, const Count4& total,
                                          int* __restrict__ scatter, int* __restrict__ gather,
                                          int (*warp_counts)[kTypes])
{
    const int lane = lane_id(), warp = warp_id();
    const int tile_base = tile * kSortTile;
    // warp w ranks segments [w*kSortItems, (w+1)*kSortItems) of 32 consecutive atoms
    int t[kSortItems];
    int rank_in_warp[kSortItems];
    int seen[kTypes] = {0, 0, 0, 0};
#pragma unroll
    for (int s = 0; s < kSortItems; s++) {
        const int i = tile_base + (warp * kSortItems + s) * kWarp + lane;
        t[s] = i < n_atoms ? checked_type(types[i]) : -1;
        rank_in_warp[s] = 0;
#pragma unroll
        for (int g = 0; g < kTypes; g++) {
            const unsigned m = __ballot_sync(kFull, t[s] == g);
            if (t[s] == g) rank_in_warp[s] = seen[g] + __popc(m & lanemask_lt());
            seen[g] += __popc(m);
        }
    }
    if (lane == 0) {
#pragma unroll
        for (int g = 0; g < kTypes; g++) warp_counts[warp][g] = seen[g];
    }
    __syncthreads();
    int start[kTypes];
    {
        int acc = 0;
#pragma unroll
        for (int g = 0; g < kTypes; g++) {
            start[g] = acc;
            acc += total.c[g];
        }
    }
#pragma unroll
    for (int s = 0; s < kSortItems; s++) {
        const int i = tile_base + (warp * kSortItems + s) * kWarp + lane;
        if (i < n_atoms) {
            int r = rank_in_warp[s];
#pragma unroll
            for (int g = 0; g < kTypes; g++) {
                if (t[s] == g) {
                    r += before.c[g];
                    for (int w = 0; w < warp; w++) r += warp_counts[w][g];
                    scatter[i] = r;
                    gather[i] = start[g] + r;
                }
            }
        }
    }
}

// Single launch: grid = number of tiles.
__global__ void __launch_bounds__(kSortThreads)
    sort_single_kernel(const int* __restrict__ types, int n_atoms, int* __restrict__ scatter,
                       int* __restrict__ gather, int* __restrict__ counts)
{
    __shared__ int red[kSortThreads / kWarp][kTypes];
    const int tile = blockIdx.x;
    const int tile_base = tile * kSortTile;
    const Count4 before = block_sum(count_range(types, 0, tile_base), red);
    const Count4 rest = block_sum(count_range(types, tile_base, n_atoms), red);
    Count4 total;
#pragma unroll
    for (int g = 0; g < kTypes; g++) total.c[g] = before.c[g] + rest.c[g];
    if (tile == 0 && threadIdx.x < kTypes) counts[threadIdx.x] = total.c[threadIdx.x];
    rank_tile(types, n_atoms, tile, before, total, scatter, gather, red);
}

// Large batches, first: per-tile element counts into scratch[tile][4].
__global__ void __launch_bounds__(kSortThreads)
    sort_histogram_kernel(const int* __restrict__ types, int n_atoms, int* __restrict__ tile_counts)
{
    __shared__ int red[kSortThreads / kWarp][kTypes];
    const int tile = blockIdx.x;
    const int lo = tile * kSortTile;
    const int hi = min(n_atoms, lo + kSortTile);
    const Count4 c = block_sum(count_range(types, lo, hi), red);
    if (threadIdx.x < kTypes) tile_counts[tile * kTypes + threadIdx.x] = c.c[threadIdx.x];
}

// Large batches, second: exclusive scan over tiles, in place, by one CTA.  On return
// tile_counts[tile] holds the counts in front of the tile and tile_counts[n_tiles] the totals.
__global__ void __launch_bounds__(kSortThreads)
    sort_scan_kernel(int* __restrict__ tile_counts, int n_tiles)
{
    __shared__ int warp_tot[kSortThreads / kWarp][kTypes];
    __shared__ int carry[kTypes];
    const int lane = lane_id(), warp = warp_id();
    if (threadIdx.x < kTypes) carry[threadIdx.x] = 0;
    __syncthreads();
    for (int k0 = 0; k0 < n_tiles; k0 += kSortThreads) {
        const int k = k0 + threadIdx.x;
        int v[kTypes], incl[kTypes];
#pragma unroll
        for (int g = 0; g < kTypes; g++) {
            v[g] = k < n_tiles ? tile_counts[k * kTypes + g] : 0;
            int x = v[g];
#pragma unroll
            for (int o = 1; o < kWarp; o <<= 1) {
                const int y = __shfl_up_sync(kFull, x, o);
                if (lane >= o) x += y;
            }
            incl[g] = x;
            if (lane == kWarp - 1) warp_tot[warp][g] = x;
        }
        __syncthreads();
#pragma unroll
        for (int g = 0; g < kTypes; g++) {
            int base = carry[g];
            for (int w = 0; w < warp; w++) base += warp_tot[w][g];
            if (k < n_tiles) tile_counts[k * kTypes + g] = base + incl[g] - v[g];
        }
        __syncthreads();
        if (threadIdx.x < kTypes) {
            int s = carry[threadIdx.x];
            for (int w = 0; w < kSortThreads / kWarp; w++) s += warp_tot[w][threadIdx.x];
            carry[threadIdx.x] = s;
        }
        __syncthreads();
    }
    if (threadIdx.x < kTypes) tile_counts[n_tiles * kTypes + threadIdx.x] = carry[threadIdx.x];
}

// Large batches, third: rank each tile from the scanned counts.
__global__ void __launch_bounds__(kSortThreads)
    sort_rank_kernel(const int* __restrict__ types, int n_atoms,
                     const int* __restrict__ tile_counts, int n_tiles, int* __restrict__ scatter,
                     int* __restrict__ gather, int* __restrict__ counts)
{
    __shared__ int red[kSortThreads / kWarp][kTypes];
    const int tile = blockIdx.x;
    Count4 before, total;
#pragma unroll
    for (int g = 0; g < kTypes; g++) {
        before.c[g] = tile_counts[tile * kTypes + g];
        total.c[g] = tile_counts[n_tiles * kTypes + g];
    }
    if (tile == 0 && threadIdx.x < kTypes) counts[threadIdx.x] = total.c[threadIdx.x];
    rank_tile(types, n_atoms, tile, before, total, scatter, gather, red);
}

// n_atoms == 0: the reference still returns atom_counts = {0, 0, 0, 0}.
__global__ void sort_empty_kernel(int* counts)
{
    if (threadIdx.x < kTypes) counts[threadIdx.x] = 0;
}

}  // namespace ani
