// AniSort on the device: stable sort of a batch's atoms by element id (a 2-bit key), returned
// as the three index arrays of the reference op (gpu_featurizer/ani_sort.cpp:71-115):
//   scatter[i] = rank of atom i among atoms of its element, gather[i] = element start + rank,
//   counts[4].
//
// The batch is cut into tiles of kSortTile consecutive atoms, one CTA per tile, one thread per
// atom.  Inside a tile the rank is a warp-level split: each warp ranks its 32-atom segment
// with one ballot per element and a popc of the lanes below, and the warp bases come from a
// scan of the 32 per-warp counts by the first warp.  What differs between the two variants is
// where a tile learns how many atoms of each element precede it:
//   * single launch (batches up to kSortSingleLaunchMax atoms): every CTA recounts the whole
//     batch straight from the (L2-resident) input with wide, unrolled loads, so no scratch
//     memory and no second launch are needed;
//   * three launches (any size): a histogram kernel writes per-tile counts to a scratch
//     array of (tiles + 1) x 4 ints, one CTA scans it in place, and the ranking kernel reads
//     the scanned entry of its tile.
#pragma once

#include "ani_common.cuh"

namespace ani {

constexpr int kSortThreads = 1024;
constexpr int kSortWarps = kSortThreads / kWarp;
constexpr int kSortTile = kSortThreads;                 // 1024 atoms per CTA
constexpr int kSortSingleLaunchMax = 64 * kSortTile;    // 65536 atoms

struct Count4 {
    int c[kTypes];
};

__device__ __forceinline__ void tally(Count4& v, int t, bool on)
{
    t = checked_type(t);
#pragma unroll
    for (int g = 0; g < kTypes; g++) v.c[g] += (on && t == g) ? 1 : 0;
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
        int s = lane < kSortWarps ? red[lane][g] : 0;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) s += __shfl_xor_sync(kFull, s, o);
        out.c[g] = s;
    }
    __syncthreads();
    return out;
}

// Counts types[0, n) twice in one sweep: everything (`total`) and the part in front of
// `split` (`before`).  `split` is a multiple of 4.  Loads are 16 bytes wide and issued four
// at a time so that their L2 latencies overlap.
__device__ __forceinline__ void count_two_ranges(const int* __restrict__ types, int n, int split,
                                                 Count4* before, Count4* total)
{
    Count4 vb = {{0, 0, 0, 0}}, vt = {{0, 0, 0, 0}};
    const bool aligned = (reinterpret_cast<uintptr_t>(types) & 15u) == 0;
    const int nvec = aligned ? n / 4 : 0;
    const int4* p4 = reinterpret_cast<const int4*>(types);
    constexpr int kUnroll = 4;
    for (int k0 = threadIdx.x; k0 < nvec; k0 += kSortThreads * kUnroll) {
        int4 q[kUnroll];
#pragma unroll
        for (int u = 0; u < kUnroll; u++) {
            const int k = k0 + u * kSortThreads;
            q[u] = k < nvec ? p4[k] : make_int4(0, 0, 0, 0);
        }
#pragma unroll
        for (int u = 0; u < kUnroll; u++) {
            const int k = k0 + u * kSortThreads;
            const bool on = k < nvec, front = on && 4 * k < split;
            tally(vt, q[u].x, on); tally(vt, q[u].y, on); tally(vt, q[u].z, on); tally(vt, q[u].w, on);
            tally(vb, q[u].x, front); tally(vb, q[u].y, front); tally(vb, q[u].z, front);
            tally(vb, q[u].w, front);
        }
    }
    for (int k = nvec * 4 + threadIdx.x; k < n; k += kSortThreads) {
        const int t = types[k];
        tally(vt, t, true);
        tally(vb, t, k < split);
    }
    *before = vb;
    *total = vt;
}

// Ranks the atoms of tile `tile` given the per-element counts in front of the tile (`before`)
// and in the whole batch (`total`).
__device__ __forceinline__ void rank_tile(const int* __restrict__ types, int n_atoms, int tile,
                                          const Count4& before, const Count4& total,
                                          int* __restrict__ scatter, int* __restrict__ gather,
                                          int (*warp_counts)[kTypes])
{
    const int lane = lane_id(), warp = warp_id();
    const int i = tile * kSortTile + threadIdx.x;
    const int t = i < n_atoms ? checked_type(types[i]) : -1;
    int rank = 0;
#pragma unroll
    for (int g = 0; g < kTypes; g++) {
        const unsigned m = __ballot_sync(kFull, t == g);
        if (t == g) rank = __popc(m & lanemask_lt());
        if (lane == 0) warp_counts[warp][g] = __popc(m);
    }
    __syncthreads();
    if (warp == 0) {  // exclusive scan over the warps, one element per step
#pragma unroll
        for (int g = 0; g < kTypes; g++) {
            const int v = warp_counts[lane][g];
            int x = v;
#pragma unroll
            for (int o = 1; o < kWarp; o <<= 1) {
                const int y = __shfl_up_sync(kFull, x, o);
                if (lane >= o) x += y;
            }
            warp_counts[lane][g] = x - v;
        }
    }
    __syncthreads();
    if (i < n_atoms) {
        int start = 0;
#pragma unroll
        for (int g = 0; g < kTypes; g++) {
            if (t == g) {
                const int r = before.c[g] + warp_counts[warp][g] + rank;
                scatter[i] = r;
                gather[i] = start + r;
            }
            start += total.c[g];
        }
    }
}

// Single launch: grid = number of tiles.
__global__ void __launch_bounds__(kSortThreads)
    sort_single_kernel(const int* __restrict__ types, int n_atoms, int* __restrict__ scatter,
                       int* __restrict__ gather, int* __restrict__ counts)
{
    __shared__ int red[kSortWarps][kTypes];
    const int tile = blockIdx.x;
    Count4 vb, vt;
    count_two_ranges(types, n_atoms, tile * kSortTile, &vb, &vt);
    const Count4 before = block_sum(vb, red);
    const Count4 total = block_sum(vt, red);
    if (tile == 0 && threadIdx.x == 0) {
#pragma unroll
        for (int g = 0; g < kTypes; g++) counts[g] = total.c[g];
    }
    rank_tile(types, n_atoms, tile, before, total, scatter, gather, red);
}

// Large batches, first: per-tile element counts into scratch[tile][4].
__global__ void __launch_bounds__(kSortThreads)
    sort_histogram_kernel(const int* __restrict__ types, int n_atoms, int* __restrict__ tile_counts)
{
    __shared__ int red[kSortWarps][kTypes];
    const int tile = blockIdx.x;
    const int i = tile * kSortTile + threadIdx.x;
    Count4 v = {{0, 0, 0, 0}};
    if (i < n_atoms) tally(v, types[i], true);
    const Count4 c = block_sum(v, red);
    if (threadIdx.x == 0) {
#pragma unroll
        for (int g = 0; g < kTypes; g++) tile_counts[tile * kTypes + g] = c.c[g];
    }
}

// Large batches, second: exclusive scan over tiles, in place, by one CTA.  On return
// tile_counts[tile] holds the counts in front of the tile and tile_counts[n_tiles] the totals.
__global__ void __launch_bounds__(kSortThreads)
    sort_scan_kernel(int* __restrict__ tile_counts, int n_tiles)
{
    __shared__ int warp_tot[kSortWarps][kTypes];
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
            for (int w = 0; w < kSortWarps; w++) s += warp_tot[w][threadIdx.x];
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
    __shared__ int red[kSortWarps][kTypes];
    const int tile = blockIdx.x;
    Count4 before, total;
#pragma unroll
    for (int g = 0; g < kTypes; g++) {
        before.c[g] = tile_counts[tile * kTypes + g];
        total.c[g] = tile_counts[n_tiles * kTypes + g];
    }
    if (tile == 0 && threadIdx.x == 0) {
#pragma unroll
        for (int g = 0; g < kTypes; g++) counts[g] = total.c[g];
    }
    rank_tile(types, n_atoms, tile, before, total, scatter, gather, red);
}

// n_atoms == 0: the reference still returns atom_counts = {0, 0, 0, 0}.
__global__ void sort_empty_kernel(int* counts)
{
    if (threadIdx.x < kTypes) counts[threadIdx.x] = 0;
}

}  // namespace ani
