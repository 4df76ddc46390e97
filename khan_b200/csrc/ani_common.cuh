// Device-side building blocks shared by the featurizer kernels: the per-device status word,
// warp helpers, per-central-atom neighbour lists and the enumeration of neighbour pairs.
//
// Work decomposition used by every featurizer kernel: ONE WARP PER CENTRAL ATOM, no cooperation
// between the warps of a CTA (no __syncthreads anywhere).  The grid gives every molecule
// kSlotsPerMol warps; warp s of molecule m handles atoms s, s + kSlotsPerMol, ... of that
// molecule and exits at once when the molecule has fewer atoms.  A warp reads its molecule's
// coordinates straight from global memory (the warps of one CTA belong to the same molecule, so
// these loads hit L1) and keeps the neighbourhood of its atom in its own slice of shared memory.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "ani_params.h"
#include "../../include/ani_b200.h"

namespace ani {

constexpr int kWarp = 32;
constexpr unsigned kFull = 0xffffffffu;
constexpr int kSlotsPerMol = 32;  // warps per molecule in the grid

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

// ---------------------------------------------------------------------------------------
// Angular neighbour list of one central atom: every j != i with r_ij < A_Rc, kept as four
// per-element sub-lists of capacity CAPT (entry index = type * CAPT + position), each in
// ascending order of j.
// ---------------------------------------------------------------------------------------
template <typename T, int CAPT, bool GRAD> struct AngularList {
    T ux[kTypes * CAPT], uy[kTypes * CAPT], uz[kTypes * CAPT];  // (x_i - x_j) / r_ij
    T r[kTypes * CAPT];
    T fc[kTypes * CAPT];                        // f_C(r_ij, A_Rc)
    T dfc[GRAD ? kTypes * CAPT : 1];            // its derivative
    int atom[GRAD ? kTypes * CAPT : 1];         // batch index of j
};

// ---------------------------------------------------------------------------------------
// Padded, bucket-major enumeration of the unordered pairs of an angular list.  Bucket
// bk = pair_bucket(ta, tb), ta <= tb.  The pairs of bucket bk occupy positions
// [off[bk], off[bk] + cnt) of a range whose length is rounded up to a multiple of 4
// (off[bk+1] - off[bk]), so that the contraction pass always reads four pairs at a time.
// ---------------------------------------------------------------------------------------
struct PairOffsets {
    int off[kPairBuckets + 1];
};

struct PairBucketInfo {
    int cnt;      // real pairs in the bucket
    int base_a;   // list index of the first entry of group ta
    int base_b;   // list index of the first entry of group tb
    int nb_same;  // size of group tb | (ta == tb) << 16
};

// Every lane computes the offsets (they are warp-uniform); lanes 0..9 also write the per-bucket
// record used by decode_pair, and the offsets are mirrored to `off_smem[0..10]` for code that
// indexes them with a runtime (warp-uniform) bucket number.  Ends with __syncwarp().
template <int CAPT>
__device__ __forceinline__ void build_pair_table(PairBucketInfo* tab, int* off_smem,
                                                 const int* ang_count, PairOffsets* po)
{
    int off = 0;
    const int lane = lane_id();
#pragma unroll
    for (int ta = 0; ta < kTypes; ta++) {
#pragma unroll
        for (int tb = ta; tb < kTypes; tb++) {
            const int bk = kTypes * (kTypes - 1) / 2 - (kTypes - ta) * (kTypes - ta - 1) / 2 + tb;
            const int na = ang_count[ta], nb = ang_count[tb];
            const int cnt = ta == tb ? na * (na - 1) / 2 : na * nb;
            po->off[bk] = off;
            if (lane == bk) {
                PairBucketInfo e;
                e.cnt = cnt;
                e.base_a = ta * CAPT;
                e.base_b = tb * CAPT;
                e.nb_same = nb | ((ta == tb ? 1 : 0) << 16);
                tab[bk] = e;
                off_smem[bk] = off;
            }
            off += (cnt + 3) & ~3;
        }
    }
    po->off[kPairBuckets] = off;
    if (lane == kPairBuckets) off_smem[kPairBuckets] = off;
    __syncwarp();
}

// Row b of q = b(b-1)/2 + a (a < b), the strictly-lower-triangular enumeration.
__device__ __forceinline__ int tri_row(int q)
{
    int b = (int)((1.0f + sqrtf(8.0f * (float)q + 1.0f)) * 0.5f);
    if (b * (b - 1) / 2 > q) b--;
    if ((b + 1) * b / 2 <= q) b++;
    return b;
}

// Padded position p -> (bucket, list index a, list index b).  Returns false for a padding slot
// (a and b then point at entry 0, which is always readable).
__device__ __forceinline__ bool decode_pair(const PairBucketInfo* tab, const PairOffsets& po, int p,
                                            int* bucket, int* a, int* b)
{
    int bk = 0;
#pragma unroll
    for (int k = 1; k < kPairBuckets; k++) bk += (p >= po.off[k]) ? 1 : 0;
    int start = po.off[0];
#pragma unroll
    for (int k = 1; k < kPairBuckets; k++) start = (p >= po.off[k]) ? po.off[k] : start;
    const PairBucketInfo e = tab[bk];
    const int q = p - start;
    const bool valid = q < e.cnt;
    const int nb = e.nb_same & 0xffff;
    int ia, ib;
    if (e.nb_same >> 16) {
        ib = tri_row(q);
        ia = q - ib * (ib - 1) / 2;
    } else {
        // q / nb for q < 2^22 via a float reciprocal, corrected by one step
        ia = (int)(((float)q + 0.5f) * (1.0f / (float)(nb > 0 ? nb : 1)));
        ib = q - ia * nb;
        if (ib < 0) { ia--; ib += nb; }
        if (ib >= nb && nb > 0) { ia++; ib -= nb; }
    }
    *bucket = bk;
    *a = valid ? e.base_a + ia : 0;
    *b = valid ? e.base_b + ib : 0;
    return valid;
}

}  // namespace ani
