// Forward kernel: radial + angular atomic environment vectors.
//
// Work decomposition: one CTA stages one molecule (element-sorted) in shared memory; each
// warp then owns one central atom at a time.  For its atom a warp
//   A. builds the two neighbour lists (lane = candidate neighbour),
//   R. accumulates the 64 radial features with lane = (half, radial shift),
//   B. evaluates, 32 neighbour pairs at a time (lane = pair), the 8 theta factors and the
//      4 radial factors of each triplet into shared memory,
//   C. contracts them with lane = (theta, shift): acc += A[theta][pair] * BF[shift][pair],
//      walking the pairs bucket by bucket (unordered element pair), so every 32-wide block
//      of the angular features is finished in registers and written once, coalesced.
// No feature row is touched twice and nothing is accumulated with atomics, so the output
// needs no zero fill and is bit-reproducible from run to run.
//
// Computes what featurize_cpu of the reference computes (gpu_featurizer/kernel_cpu.cpp:406-537)
// and replaces its CUDA kernel (gpu_featurizer/kernel.cu:72-268), which used one thread per
// atom and 32 global atomicAdd per pair and per triplet.
#pragma once

#include "ani_common.cuh"

namespace ani {

constexpr int kPadStride = 36;  // 32 pairs + 4 words: keeps the 16-byte reads of pass C conflict-free

template <typename T> struct FeaturizeWarpShared {
    T A[kNumThetas][kPadStride];
    T BF[kNumARs][kPadStride];
    PairBucket tab[kPairBuckets + 1];
};

template <typename T, int NW, int ACAP, int RCAP> struct FeaturizeShared {
    MolShared<T> mol;
    NeighborLists<T, ACAP, RCAP, false> nl[NW];
    FeaturizeWarpShared<T> ws[NW];
};

template <typename T> __device__ __forceinline__ T* element_buffer(int t, T* h, T* c, T* n, T* o)
{
    return t == 0 ? h : (t == 1 ? c : (t == 2 ? n : o));
}

// Slow path for an atom whose neighbourhood does not fit the lists: lane = (theta, shift)
// for the angular part, lane = (half, radial shift) for the radial part, every pair of
// molecule atoms tested directly.  Same results, O(n^2) distance tests per atom.
template <typename T>
__device__ __noinline__ void featurize_atom_streaming(const MolShared<T>& ms, int n, int i, T* row)
{
    const int lane = lane_id();
    const T xi = ms.x[i], yi = ms.y[i], zi = ms.z[i];
    {
        const int half = lane >> 4;
        const T shift = (T)c_tab.R_Rs[lane & 15];
        T acc[kTypes];
#pragma unroll
        for (int g = 0; g < kTypes; g++) {
            acc[g] = (T)0;
            for (int j = ms.group_start[g] + half; j < ms.group_start[g + 1]; j += 2) {
                if (j == i) continue;
                const T dx = xi - ms.x[j], dy = yi - ms.y[j], dz = zi - ms.z[j];
                const T r = Num<T>::sqrt_(dx * dx + dy * dy + dz * dz);
                if (r < (T)kR_Rc) {
                    const T d = r - shift;
                    acc[g] += Num<T>::exp_neg((T)kR_eta, d * d) * cutoff_value<T>(r, (T)kR_Rc);
                }
            }
            acc[g] += __shfl_xor_sync(kFull, acc[g], 16);
        }
        row[lane] = lane < 16 ? acc[0] : acc[1];
        row[32 + lane] = lane < 16 ? acc[2] : acc[3];
    }
    const T ct = (T)c_tab.cos_t[lane >> 2], st = (T)c_tab.sin_t[lane >> 2];
    const T shift = (T)c_tab.A_Rs[lane & 3];
#pragma unroll 1
    for (int ta = 0; ta < kTypes; ta++) {
#pragma unroll 1
        for (int tb = ta; tb < kTypes; tb++) {
            T acc = (T)0;
            for (int j = ms.group_start[ta]; j < ms.group_start[ta + 1]; j++) {
                if (j == i) continue;
                const T dxj = xi - ms.x[j], dyj = yi - ms.y[j], dzj = zi - ms.z[j];
                const T rj = Num<T>::sqrt_(dxj * dxj + dyj * dyj + dzj * dzj);
                if (!(rj < (T)kA_Rc)) continue;
                const T fj = cutoff_value<T>(rj, (T)kA_Rc);
                const int k0 = ta == tb ? j + 1 : ms.group_start[tb];
                for (int k = k0; k < ms.group_start[tb + 1]; k++) {
                    if (k == i) continue;
                    const T dxk = xi - ms.x[k], dyk = yi - ms.y[k], dzk = zi - ms.z[k];
                    const T rk = Num<T>::sqrt_(dxk * dxk + dyk * dyk + dzk * dzk);
                    if (!(rk < (T)kA_Rc)) continue;
                    const T fk = cutoff_value<T>(rk, (T)kA_Rc);
                    T c = (dxj * dxk + dyj * dyk + dzj * dzk) / (rj * rk);
                    c = Num<T>::max_((T)-1, Num<T>::min_((T)1, c));
                    const T s = Num<T>::sqrt_(Num<T>::max_((T)0, (T)1 - c * c));
                    const T b = (T)1 + (c * ct + s * st);
                    const T b2 = b * b, b4 = b2 * b2;
                    const T d = (T)0.5 * (rj + rk) - shift;
                    acc += b4 * b4 * Num<T>::exp_neg((T)kA_eta, d * d) * ((T)kA_pref * fj * fk);
                }
            }
            row[kRadial + pair_bucket(ta, tb) * kTS + lane] = acc;
        }
    }
}

template <typename T, int NW, int ACAP, int RCAP>
__global__ void __launch_bounds__(NW* kWarp)
    featurize_kernel(const T* __restrict__ xs, const T* __restrict__ ys, const T* __restrict__ zs,
                     const int* __restrict__ types, const int* __restrict__ mol_offsets,
                     const int* __restrict__ mol_counts, int n_mols, int n_atoms,
                     const int* __restrict__ scatter, T* out_h, T* out_c, T* out_n, T* out_o,
                     int acs0, int acs1, int acs2, int acs3, int nsplit)
{
    extern __shared__ __align__(16) unsigned char smem_raw[];
    auto& sh = *reinterpret_cast<FeaturizeShared<T, NW, ACAP, RCAP>*>(smem_raw);
    const int lane = lane_id(), warp = warp_id();
    auto& nl = sh.nl[warp];
    auto& ws = sh.ws[warp];
    const int acs[kTypes] = {acs0, acs1, acs2, acs3};

    for (int item = blockIdx.x; item < n_mols * nsplit; item += gridDim.x) {
        const int m = item / nsplit, split = item - m * nsplit;
        const int n = mol_counts[m], base = mol_offsets[m];
        if (n <= 0) continue;
        if (n > kMaxAtomsPerMol) {
            if (threadIdx.x == 0) report(ANI_ERR_MOL_TOO_LARGE);
            continue;
        }
        if (base < 0 || base + n > n_atoms) {
            if (threadIdx.x == 0) report(ANI_ERR_BAD_INDEX);
            continue;
        }
        __syncthreads();  // previous molecule fully consumed before restaging
        stage_molecule<T, NW>(sh.mol, xs, ys, zs, types, base, n);
        const MolShared<T>& ms = sh.mol;

        // heaviest elements (most neighbours) first
        for (int i = n - 1 - (split * NW + warp); i >= 0; i -= nsplit * NW) {
            const int ti = slot_type(ms.group_start, i);
            const int gi = base + ms.orig[i];
            const int srow = scatter[gi];
            if (srow < 0 || srow >= acs[ti]) {
                if (lane == 0) report(ANI_ERR_BAD_INDEX);
                continue;
            }
            T* row = element_buffer<T>(ti, out_h, out_c, out_n, out_o) + (size_t)srow * kTotal;

            NeighborCounts nc;
            if (!build_neighbors<T, ACAP, RCAP, false>(ms, n, i, nl, nc)) {
                featurize_atom_streaming<T>(ms, n, i, row);
                __syncwarp();
                continue;
            }

            // ---- R: radial features, lane = (half, shift) ----
            {
                const int half = lane >> 4;
                const T shift = (T)c_tab.R_Rs[lane & 15];
                T acc[kTypes];
                int start = 0;
#pragma unroll
                for (int g = 0; g < kTypes; g++) {
                    acc[g] = (T)0;
                    const int end = start + nc.rad[g];
                    for (int p = start + half; p < end; p += 2) {
                        const T d = nl.rad_r[p] - shift;
                        acc[g] += Num<T>::exp_neg((T)kR_eta, d * d) * nl.rad_fc[p];
                    }
                    start = end;
                    acc[g] += __shfl_xor_sync(kFull, acc[g], 16);
                }
                row[lane] = lane < 16 ? acc[0] : acc[1];
                row[32 + lane] = lane < 16 ? acc[2] : acc[3];
            }

            // ---- B + C: angular features ----
            const int total = build_pair_table(ws.tab, nc.ang);
            const int my_t = lane >> 2, my_s = lane & 3;
            int cur = 0;          // bucket being accumulated
            T acc = (T)0;
            for (int c0 = 0; c0 < total; c0 += kWarp) {
                {   // B: lane = pair
                    int bk, a, b;
                    const bool valid = decode_pair(ws.tab, c0 + lane, &bk, &a, &b);
                    const T cosv = nl.ang_ux[a] * nl.ang_ux[b] + nl.ang_uy[a] * nl.ang_uy[b] +
                                   nl.ang_uz[a] * nl.ang_uz[b];
                    const T rbar = (T)0.5 * (nl.ang_r[a] + nl.ang_r[b]);
                    const T fcprod = valid ? nl.ang_fc[a] * nl.ang_fc[b] : (T)0;
                    T A[kNumThetas], BF[kNumARs];
                    angular_factors<T>(valid ? cosv : (T)0, rbar, fcprod, A, BF);
#pragma unroll
                    for (int t = 0; t < kNumThetas; t++) ws.A[t][lane] = A[t];
#pragma unroll
                    for (int q = 0; q < kNumARs; q++) ws.BF[q][lane] = BF[q];
                }
                __syncwarp();
                {   // C: lane = (theta, shift)
                    const int chunk_end = min(c0 + kWarp, total);
                    int pp = c0;
                    while (pp < chunk_end) {
                        while (ws.tab[cur + 1].off <= pp) {
                            row[kRadial + cur * kTS + lane] = acc;
                            acc = (T)0;
                            cur++;
                        }
                        const int seg_end = min(chunk_end, ws.tab[cur + 1].off);
                        for (; pp < seg_end; pp += 4) {
                            const int o = pp - c0;
#pragma unroll
                            for (int u = 0; u < 4; u++) acc += ws.A[my_t][o + u] * ws.BF[my_s][o + u];
                        }
                    }
                }
                __syncwarp();
            }
            for (; cur < kPairBuckets; cur++) {
                row[kRadial + cur * kTS + lane] = acc;
                acc = (T)0;
            }
        }
    }
}

}  // namespace ani
