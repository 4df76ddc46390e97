// Device-side building blocks shared by the featurizer kernels: the per-device status word,
// warp helpers, staging of one molecule into shared memory in element order, and the
// per-central-atom neighbour lists.
#pragma once

#include <cuda_runtime.h>
#include <stdint.h>

#include "ani_params.h"
#include "../../include/ani_b200.h"

namespace ani {

constexpr int kWarp = 32;
constexpr unsigned kFull = 0xffffffffu;

// Largest molecule staged in shared memory by the featurizer kernels.
constexpr int kMaxAtomsPerMol = 512;
constexpr int kMaxChunks = kMaxAtomsPerMol / kWarp;

// First device-side problem seen since the last read (0 = none).  One word per device: the
// variable is instantiated once per loaded module and context.  (This header is included by
// exactly one translation unit.)
__device__ int g_status = 0;

__device__ __forceinline__ void report(int code) { atomicCAS(&g_status, 0, code); }

__device__ __forceinline__ int lane_id() { return threadIdx.x & (kWarp - 1); }
__device__ __forceinline__ int warp_id() { return threadIdx.x >> 5; }
__device__ __forceinline__ unsigned lanes_below(int k)  // bit l set for l < k, k clamped to 0..32
{
    return k <= 0 ? 0u : (k >= 32 ? kFull : ((1u << k) - 1u));
}
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

// ---------------------------------------------------------------------------------------
// One molecule in shared memory, atoms reordered stably by element so that every neighbour
// list built from it is grouped by element too.
// ---------------------------------------------------------------------------------------
template <typename T> struct MolShared {
    T x[kMaxAtomsPerMol];
    T y[kMaxAtomsPerMol];
    T z[kMaxAtomsPerMol];
    int orig[kMaxAtomsPerMol];          // slot -> index of the atom inside the molecule
    int chunk_count[kMaxChunks][kTypes];
    int group_start[kTypes + 1];        // slot range of each element
};

// Element of a slot, from the group boundaries.
__device__ __forceinline__ int slot_type(const int* gs, int slot)
{
    return (slot >= gs[1]) + (slot >= gs[2]) + (slot >= gs[3]);
}

// Cooperative (whole CTA) load of molecule [base, base + n) into `ms`, sorted by element.
// Every thread of the CTA must call it; it ends with a __syncthreads().
template <typename T, int NW>
__device__ __forceinline__ void stage_molecule(MolShared<T>& ms, const T* __restrict__ xs,
                                               const T* __restrict__ ys, const T* __restrict__ zs,
                                               const int* __restrict__ types, int base, int n)
{
    const int lane = lane_id(), warp = warp_id();
    const int nchunks = (n + kWarp - 1) / kWarp;
    for (int c = warp; c < nchunks; c += NW) {
        const int j = c * kWarp + lane;
        int t = j < n ? types[base + j] : -1;
        if (j < n && (t < 0 || t >= kTypes)) {
            report(ANI_ERR_BAD_ELEMENT);
            t &= 3;
        }
#pragma unroll
        for (int g = 0; g < kTypes; g++) {
            const int cnt = __popc(__ballot_sync(kFull, t == g));
            if (lane == 0) ms.chunk_count[c][g] = cnt;
        }
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int tot[kTypes] = {0, 0, 0, 0};
        for (int c = 0; c < nchunks; c++)
#pragma unroll
            for (int g = 0; g < kTypes; g++) tot[g] += ms.chunk_count[c][g];
        ms.group_start[0] = 0;
#pragma unroll
        for (int g = 0; g < kTypes; g++) ms.group_start[g + 1] = ms.group_start[g] + tot[g];
    }
    __syncthreads();
    for (int c = warp; c < nchunks; c += NW) {
        const int j = c * kWarp + lane;
        int t = j < n ? (types[base + j] & 3) : -1;
        unsigned same = 0;
#pragma unroll
        for (int g = 0; g < kTypes; g++) {
            const unsigned m = __ballot_sync(kFull, t == g);
            if (t == g) same = m;
        }
        if (j < n) {
            int before = 0;
            for (int cc = 0; cc < c; cc++) before += ms.chunk_count[cc][t];
            const int slot = ms.group_start[t] + before + __popc(same & lanemask_lt());
            ms.x[slot] = xs[base + j];
            ms.y[slot] = ys[base + j];
            ms.z[slot] = zs[base + j];
            ms.orig[slot] = j;
        }
    }
    __syncthreads();
}

// ---------------------------------------------------------------------------------------
// Neighbour lists of one central atom, one set per warp.  Both lists are grouped by
// element (they inherit the order of MolShared) and `count[g]` gives the group sizes.
//   radial list : every j != i with r_ij < R_Rc
//   angular list: every j != i with r_ij < A_Rc
// ---------------------------------------------------------------------------------------
template <typename T, int ACAP, int RCAP, bool GRAD> struct NeighborLists {
    T ang_ux[ACAP], ang_uy[ACAP], ang_uz[ACAP];  // unit vector (x_i - x_j) / r_ij
    T ang_r[ACAP];
    T ang_fc[ACAP];                              // f_C(r_ij, A_Rc)
    T ang_dfc[GRAD ? ACAP : 1];
    int ang_slot[GRAD ? ACAP : 1];
    T rad_r[RCAP];
    T rad_fc[RCAP];                              // f_C(r_ij, R_Rc)
    T rad_dfc[GRAD ? RCAP : 1];
    T rad_ux[GRAD ? RCAP : 1], rad_uy[GRAD ? RCAP : 1], rad_uz[GRAD ? RCAP : 1];
    int rad_slot[GRAD ? RCAP : 1];
};

struct NeighborCounts {
    int ang[kTypes];
    int rad[kTypes];
    int n_ang, n_rad;
};

// Warp-cooperative build of both lists for the atom in slot `i`.  Returns false when a list
// would exceed its capacity (the lists are then incomplete and must not be used).
template <typename T, int ACAP, int RCAP, bool GRAD>
__device__ __forceinline__ bool build_neighbors(const MolShared<T>& ms, int n, int i,
                                                NeighborLists<T, ACAP, RCAP, GRAD>& nl,
                                                NeighborCounts& nc)
{
    const int lane = lane_id();
    const T xi = ms.x[i], yi = ms.y[i], zi = ms.z[i];
    const int gs0 = ms.group_start[0], gs1 = ms.group_start[1], gs2 = ms.group_start[2],
              gs3 = ms.group_start[3], gs4 = ms.group_start[4];
    const int gsv[kTypes + 1] = {gs0, gs1, gs2, gs3, gs4};
#pragma unroll
    for (int g = 0; g < kTypes; g++) nc.ang[g] = nc.rad[g] = 0;
    int n_ang = 0, n_rad = 0;
    for (int j0 = 0; j0 < n; j0 += kWarp) {
        const int j = j0 + lane;
        const bool valid = j < n && j != i;
        const int jj = j < n ? j : 0;
        const T dx = xi - ms.x[jj], dy = yi - ms.y[jj], dz = zi - ms.z[jj];
        const T r = Num<T>::sqrt_(dx * dx + dy * dy + dz * dz);
        const bool in_rad = valid && r < (T)kR_Rc;
        const bool in_ang = valid && r < (T)kA_Rc;
        const unsigned m_rad = __ballot_sync(kFull, in_rad);
        const unsigned m_ang = __ballot_sync(kFull, in_ang);
        if (in_rad) {
            const int pos = n_rad + __popc(m_rad & lanemask_lt());
            if (pos < RCAP) {
                T fc, dfc;
                cutoff<T>(r, (T)kR_Rc, &fc, &dfc);
                nl.rad_r[pos] = r;
                nl.rad_fc[pos] = fc;
                if (GRAD) {
                    const T inv = (T)1 / r;
                    nl.rad_dfc[pos] = dfc;
                    nl.rad_ux[pos] = dx * inv;
                    nl.rad_uy[pos] = dy * inv;
                    nl.rad_uz[pos] = dz * inv;
                    nl.rad_slot[pos] = j;
                }
            }
        }
        if (in_ang) {
            const int pos = n_ang + __popc(m_ang & lanemask_lt());
            if (pos < ACAP) {
                T fc, dfc;
                cutoff<T>(r, (T)kA_Rc, &fc, &dfc);
                const T inv = (T)1 / r;
                nl.ang_ux[pos] = dx * inv;
                nl.ang_uy[pos] = dy * inv;
                nl.ang_uz[pos] = dz * inv;
                nl.ang_r[pos] = r;
                nl.ang_fc[pos] = fc;
                if (GRAD) {
                    nl.ang_dfc[pos] = dfc;
                    nl.ang_slot[pos] = j;
                }
            }
        }
        // group sizes: lanes of this chunk whose slot lies in [gs[g], gs[g+1])
#pragma unroll
        for (int g = 0; g < kTypes; g++) {
            const unsigned in_group = lanes_below(gsv[g + 1] - j0) & ~lanes_below(gsv[g] - j0);
            nc.rad[g] += __popc(m_rad & in_group);
            nc.ang[g] += __popc(m_ang & in_group);
        }
        n_rad += __popc(m_rad);
        n_ang += __popc(m_ang);
    }
    nc.n_ang = n_ang;
    nc.n_rad = n_rad;
    __syncwarp();
    return n_ang <= ACAP && n_rad <= RCAP;
}

// Row q = b(b-1)/2 + a (a < b) of a strictly-lower-triangular enumeration -> b.
__device__ __forceinline__ int tri_row(int q)
{
    int b = (int)((1.0f + sqrtf(8.0f * (float)q + 1.0f)) * 0.5f);
    if (b * (b - 1) / 2 > q) b--;
    if ((b + 1) * b / 2 <= q) b++;
    return b;
}

// Bucket table of the padded, bucket-major enumeration of neighbour pairs used by the
// angular passes.  Bucket bk = pair_bucket(ta, tb), ta <= tb.  Pairs of one bucket occupy
// [off, off + cnt) of a range whose length is rounded up to a multiple of 4, so that the
// contraction pass can always read four pairs at a time.
struct PairBucket {
    int off;       // padded start
    int cnt;       // real pairs
    int sa_sb;     // list start of group ta | list start of group tb << 16
    int nb_same;   // size of group tb | (ta == tb) << 16
};

// Lanes 0..9 fill `tab[0..9]`, lane 10 fills tab[10].off = padded total.  Returns the padded total.
__device__ __forceinline__ int build_pair_table(PairBucket* tab, const int* ang_count)
{
    int start[kTypes + 1];
    start[0] = 0;
#pragma unroll
    for (int g = 0; g < kTypes; g++) start[g + 1] = start[g] + ang_count[g];
    int off = 0;
    const int lane = lane_id();
#pragma unroll
    for (int ta = 0; ta < kTypes; ta++) {
#pragma unroll
        for (int tb = ta; tb < kTypes; tb++) {
            const int bk = kTypes * (kTypes - 1) / 2 - (kTypes - ta) * (kTypes - ta - 1) / 2 + tb;
            const int na = ang_count[ta], nb = ang_count[tb];
            const int cnt = ta == tb ? na * (na - 1) / 2 : na * nb;
            if (lane == bk) {
                tab[bk].off = off;
                tab[bk].cnt = cnt;
                tab[bk].sa_sb = start[ta] | (start[tb] << 16);
                tab[bk].nb_same = nb | ((ta == tb ? 1 : 0) << 16);
            }
            off += (cnt + 3) & ~3;
        }
    }
    if (lane == kPairBuckets) {
        tab[kPairBuckets].off = off;
        tab[kPairBuckets].cnt = 0;
        tab[kPairBuckets].sa_sb = 0;
        tab[kPairBuckets].nb_same = 1;
    }
    __syncwarp();
    return off;
}

// Padded position p -> (bucket, list index a, list index b, valid).
__device__ __forceinline__ bool decode_pair(const PairBucket* tab, int p, int* bucket, int* a,
                                            int* b)
{
    int bk = 0;
#pragma unroll
    for (int k = 1; k < kPairBuckets; k++) bk += (p >= tab[k].off) ? 1 : 0;
    const PairBucket e = tab[bk];
    const int q = p - e.off;
    const bool valid = q < e.cnt;
    const int sa = e.sa_sb & 0xffff, sb = e.sa_sb >> 16;
    const int nb = e.nb_same & 0xffff;
    const bool same = (e.nb_same >> 16) != 0;
    int ia, ib;
    if (same) {
        ib = tri_row(q);
        ia = q - ib * (ib - 1) / 2;
    } else {
        ia = q / (nb > 0 ? nb : 1);
        ib = q - ia * nb;
    }
    *bucket = bk;
    *a = valid ? sa + ia : 0;
    *b = valid ? sb + ib : 0;
    return valid;
}

}  // namespace ani
