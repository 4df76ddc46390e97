// Device-side building blocks shared by the featurizer kernels: the per-device status word,
// warp helpers, per-central-atom neighbour lists and the enumeration of neighbour pairs.
//
// Work decomposition used by every featurizer kernel: ONE WARP PER CENTRAL ATOM, no cooperation
// between the warps of a CTA beyond a shared work counter (one __syncthreads, at the start).  The work list has S = 2^slot_shift
// items per molecule (S is chosen per launch: the power of two next above the mean molecule
// size, 4 <= S <= 32); item (m, s) covers atoms s, s + S, ... of molecule m and is empty when
// the molecule has fewer atoms.  The grid is persistent (a few CTAs per SM): warp w takes
// items w, w + W, w + 2W, ... (W = warps in the grid, a multiple of 32), so an empty
// item costs one cached load instead of a CTA slot, and consecutive warps -- the warps of one
// CTA -- work on the same molecule, whose coordinates they read straight from global memory
// (L1 hits).  Each warp keeps the neighbourhood of its atom in its own slice of shared memory.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "ani_params.h"
#include "../../include/ani_b200.h"

namespace ani {

constexpr int kWarp = 32;
constexpr unsigned kFull = 0xffffffffu;
constexpr int kSlotsPerMol = 32;  // most work-list slots per molecule; a launch uses 2^slot_shift <= 32 of them

// First device-side problem seen since the last read (0 = none).  One word per device: the
// variable is instantiated once per loaded module and context.  (This header is included by
// exactly one translation unit.)
__device__ int g_status = 0;

__device__ __forceinline__ void report(int code) { atomicCAS(&g_status, 0, code); }

__device__ __forceinline__ int lane_id() { return threadIdx.x & (kWarp - 1); }
__device__ __forceinline__ int warp_id() { return threadIdx.x >> 5; }
__device__ __forceinline__ unsigned lanemask_lt()
{
    unsigned m;
    asm("mov.u32 %0, %%lanemask_lt;" : "=r"(m));
    return m;
}

// Parameter tables in constant memory, for loops whose index is a lane-dependent runtime value.
struct ParamTables {
    float R_Rs[kNumRs];
    float A_Rs[kNumARs];
    double cos_t[kNumThetas];
    double sin_t[kNumThetas];
};
__constant__ ParamTables c_tab = {
    {5.0000000e-01f, 7.5625000e-01f, 1.0125000e+00f, 1.2687500e+00f, 1.5250000e+00f, 1.7812500e+00f,
     2.0375000e+00f, 2.2937500e+00f, 2.5500000e+00f, 2.8062500e+00f, 3.0625000e+00f, 3.3187500e+00f,
     3.5750000e+00f, 3.8312500e+00f, 4.0875000e+00f, 4.3437500e+00f},
    {5.0000000e-01f, 1.1500000e+00f, 1.8000000e+00f, 2.4500000e+00f},
    {1.0, 0.70710676573223721282, 7.5497899548918749969e-8, -0.70710678540262942905,
     -0.99999999999999617863, -0.70710683035554063407, 1.1924880454806034642e-8,
     0.70710667863246853197},
    {0.0, 0.70710679664085749822, 0.99999999999999715003, 0.70710677697046559462,
     -8.7422780003724745258e-8, -0.70710673201755099574, -0.9999999999999999289,
     -0.70710688374061164307}};

// Four consecutive values from 16-byte aligned shared memory (float) / two 16-byte reads (double).
__device__ __forceinline__ void load4(const float* p, float* v)
{
    const float4 q = *reinterpret_cast<const float4*>(p);
    v[0] = q.x; v[1] = q.y; v[2] = q.z; v[3] = q.w;
}
__device__ __forceinline__ void load4(const double* p, double* v)
{
    const double2 a = *reinterpret_cast<const double2*>(p);
    const double2 b = *reinterpret_cast<const double2*>(p + 2);
    v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
}

// Work list.  A molecule has S = 2^slot_shift slots (slot s covers atoms s, s + S, ...), so there
// are n_mols * S items.  Warp w of the grid statically owns items w, w + W, ... (W = warps in the
// grid); inside a CTA those items are handed out from a counter in shared memory instead, so
// that a warp that drew cheap atoms takes more of them (the spread in cost per item is large --
// a hydrogen at the edge of a small molecule against a carbon inside a large one -- and a warp
// only sees a few items).  Two orders of the list:
//   molecule-major  item = m * S + slot (slot rotated per round): the warps of a CTA work on the
//                   same molecule and share its coordinates in L1 -- best for large molecules;
//   slot-major      item = slot * n_mols + m: the warps of a CTA, and the rounds of a warp, see a
//                   mix of molecules, and the first atoms of all molecules (the heavy atoms, in
//                   the usual ordering of data sets) come before the last ones, most of which are
//                   hydrogens or empty slots -- best balance for small molecules.
// Returns false when the CTA's list is exhausted.
template <int NW>
__device__ __forceinline__ bool next_work(int* counter, int n_mols, int slot_shift, bool slot_major, int* m, int* slot)
{
    int t = 0;
    if (lane_id() == 0) t = atomicAdd(counter, 1);
    t = __shfl_sync(kFull, t, 0);
    const int round = t / NW;
    const long long item = (long long)blockIdx.x * NW + (t % NW) + (long long)round * gridDim.x * NW;
    if (item >= ((long long)n_mols << slot_shift)) return false;
    if (slot_major) {
        const int s = (int)(item / n_mols);
        *slot = s;
        *m = (int)(item - (long long)s * n_mols);
    } else {
        const int mask = (1 << slot_shift) - 1;
        *m = (int)(item >> slot_shift);
        *slot = (((int)item & mask) + 11 * round) & mask;   // a permutation of the slots: W is a multiple of 32
    }
    return true;
}

// One molecule as the kernels see it, validated.
struct MolRange {
    int base;  // index of its first atom in the batch
    int n;     // atoms
};

// Reads and checks molecule m.  Returns false (after recording the problem) when the molecule
// must be skipped.
__device__ __forceinline__ bool load_molecule(const int* __restrict__ mol_offsets,
                                              const int* __restrict__ mol_counts, int m,
                                              int n_atoms, MolRange* out)
{
    const int n = mol_counts[m], base = mol_offsets[m];
    out->base = base;
    out->n = n;
    if (n <= 0) return false;
    if (base < 0 || n > n_atoms || base > n_atoms - n) {
        report(ANI_ERR_BAD_INDEX);
        return false;
    }
    return true;
}

__device__ __forceinline__ int checked_type(int t)
{
    if (t < 0 || t >= kTypes) {
        report(ANI_ERR_BAD_ELEMENT);
        t &= 3;
    }
    return t;
}

template <typename T> struct alignas(sizeof(T) * 4) Vec4 {
    T x, y, z, w;
};
template <typename T> struct alignas(sizeof(T) * 2) Vec2 {
    T x, y;
};

// Warp-uniform value picked from four registers by a lane-dependent index 0..3.
template <typename V> __device__ __forceinline__ V pick4(const V* v, int k)
{
    return k == 0 ? v[0] : (k == 1 ? v[1] : (k == 2 ? v[2] : v[3]));
}

// r = |d| and 1/r from the squared length with one SFU op (float) / full precision (double).
// A zero length (two atoms at one point) yields r = 0, inv = 0 instead of Inf/NaN, so that a
// degenerate pair cannot poison the shared-memory lists that later atoms reuse.
__device__ __forceinline__ void length_and_inverse(float d2, float* r, float* inv)
{
    const float rs = d2 > 0.0f ? sfu_rsqrt(d2) : 0.0f;
    *inv = rs;
    *r = d2 * rs;
}
__device__ __forceinline__ void length_and_inverse(double d2, double* r, double* inv)
{
    const double rr = sqrt(d2);
    *r = rr;
    *inv = d2 > 0.0 ? 1.0 / rr : 0.0;
}

// ---------------------------------------------------------------------------------------
// Padded, bucket-major enumeration of the unordered pairs of an angular neighbour list that is
// kept as four per-element sub-lists of capacity CAPT (entry index = type * CAPT + position).
// Bucket bk = pair_bucket(ta, tb), ta <= tb.  The pairs of bucket bk occupy positions
// [off, off + cnt) of a range whose length is rounded up to a multiple of 4, so that the
// contraction pass of the forward kernel always reads four pairs at a time.
// ---------------------------------------------------------------------------------------
struct alignas(16) PairBucketInfo {
    int off;      // padded start position
    int cnt;      // real pairs in the bucket
    int packed;   // base_a | base_b << 8 | nb << 16 | same << 24
    float inv_nb; // 1 / size of group tb
};

constexpr int kQuadTable = 168;  // quads (4 padded positions) in the bucket table: 640 pairs + one chunk

struct PairTables {
    PairBucketInfo tab[kPairBuckets];
    int off[kPairBuckets + 2];            // off[bk], off[10] = padded total
    alignas(8) unsigned char quad_bucket[kQuadTable];   // kPairBuckets = "past the end"
};

constexpr int kMaxPaddedPairs = (kQuadTable - 8) * 4;   // lists with more pairs take the slow path

// ta / tb of bucket k, two bits each.
constexpr unsigned kBucketTa = 0u | (0u << 2) | (0u << 4) | (0u << 6) | (1u << 8) | (1u << 10) |
                               (1u << 12) | (2u << 14) | (2u << 16) | (3u << 18);
constexpr unsigned kBucketTb = 0u | (1u << 2) | (2u << 4) | (3u << 6) | (1u << 8) | (2u << 10) |
                               (3u << 12) | (2u << 14) | (3u << 16) | (3u << 18);

// Lanes 0..9 each build one bucket record; the padded offsets come from a warp scan.  Returns
// the padded total (warp-uniform).  Ends with __syncwarp().
template <int CAPT>
__device__ __forceinline__ int build_pair_tables(PairTables& pt, const int* ang_count)
{
    const int lane = lane_id();
    const int ta = (kBucketTa >> (2 * lane)) & 3, tb = (kBucketTb >> (2 * lane)) & 3;
    const int na = pick4(ang_count, ta), nb = pick4(ang_count, tb);
    const int cnt = lane < kPairBuckets ? (ta == tb ? na * (na - 1) / 2 : na * nb) : 0;
    const int pad = (cnt + 3) & ~3;
    int incl = pad;
#pragma unroll
    for (int o = 1; o < 16; o <<= 1) {
        const int y = __shfl_up_sync(kFull, incl, o);
        if (lane >= o) incl += y;
    }
    const int off = incl - pad;
    if (lane < kPairBuckets) {
        PairBucketInfo e;
        e.off = off;
        e.cnt = cnt;
        e.packed = (ta * CAPT) | ((tb * CAPT) << 8) | (nb << 16) | ((ta == tb ? 1 : 0) << 24);
        e.inv_nb = 1.0f / (float)(nb > 0 ? nb : 1);
        pt.tab[lane] = e;
    }
    if (lane <= kPairBuckets) pt.off[lane] = off;
    if (lane == kPairBuckets + 1) pt.off[lane] = 0x7fffffff;   // sentinel behind the total
    const int total = __shfl_sync(kFull, incl, kPairBuckets - 1);
    __syncwarp();
    // Bucket of every quad of padded positions (all bucket starts are multiples of 4), through
    // one chunk past the end of the list; quads past the end get the id kPairBuckets.  Each of
    // lanes 0..9 fills the quads of its own bucket, lane 10 the tail.
    if (total <= kMaxPaddedPairs) {
        int q_lo = off >> 2, q_hi = (off + pad) >> 2;
        if (lane == kPairBuckets) q_hi = (((total + kWarp - 1) & ~(kWarp - 1)) >> 2) + 8;
        if (lane <= kPairBuckets)
            for (int q = q_lo; q < q_hi; q++) pt.quad_bucket[q] = (unsigned char)lane;
    }
    __syncwarp();
    return total;
}

// Row b of q = b(b-1)/2 + a (a < b), the strictly-lower-triangular enumeration.
__device__ __forceinline__ int tri_row(int q)
{
    const float x = 8.0f * (float)q + 1.0f;
    int b = (int)((1.0f + x * sfu_rsqrt(x)) * 0.5f);
    if (b * (b - 1) / 2 > q) b--;
    if ((b + 1) * b / 2 <= q) b++;
    return b;
}

// Padded position p -> (bucket, list index a, list index b).  Returns false for a padding slot
// (a and b then point at entry 0 of the list).
__device__ __forceinline__ bool decode_pair(const PairTables& pt, int p, int* bucket, int* a, int* b)
{
    // the caller guarantees total <= kMaxPaddedPairs, so p >> 2 is inside the table
    const int bk = min((int)pt.quad_bucket[p >> 2], kPairBuckets - 1);
    const PairBucketInfo e = pt.tab[bk];
    const int q = p - e.off;
    const bool valid = q < e.cnt;
    const int nb = (e.packed >> 16) & 0xff;
    int ia, ib;
    if (e.packed >> 24) {
        ib = tri_row(q);
        ia = q - ib * (ib - 1) / 2;
    } else {
        ia = (int)(((float)q + 0.5f) * e.inv_nb);
        ib = q - ia * nb;
        if (ib < 0) { ia--; ib += nb; }
        if (ib >= nb) { ia++; ib -= nb; }
    }
    *bucket = bk;
    *a = valid ? (e.packed & 0xff) + ia : 0;
    *b = valid ? ((e.packed >> 8) & 0xff) + ib : 0;
    return valid;
}

}  // namespace ani
