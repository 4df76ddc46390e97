// Forward kernel: radial + angular atomic environment vectors.
//
// One warp per central atom (see ani_common.cuh).  For its atom a warp
//   A. scans the molecule (lane = candidate neighbour j, coordinates from global memory) and
//      compacts the neighbours into per-element sub-lists in its slice of shared memory:
//      (r, f_C) for r < R_Rc, and (unit vector, r, f_C) for r < A_Rc;
//   R. accumulates the 64 radial features with lane = (element, pair of radial shifts), every
//      lane walking the radial sub-list of its element;
//   B. evaluates, 32 neighbour pairs at a time (lane = pair), the 8 theta factors and the
//      4 radial factors of each triplet into shared memory;
//   C. contracts them with lane = (theta, shift): acc += A[theta][pair] * BF[shift][pair],
//      walking the pairs bucket by bucket (unordered element pair), so every 32-wide block of
//      the angular features is finished in registers and written once, coalesced.
// No feature row is touched twice and nothing is accumulated with atomics, so the output
// needs no zero fill and is bit-reproducible from run to run.
//
// Computes what featurize_cpu of the reference computes (gpu_featurizer/kernel_cpu.cpp:406-537)
// and replaces its CUDA kernel (gpu_featurizer/kernel.cu:72-268), which used one thread per
// atom and 32 global atomicAdd per pair and per triplet.
#pragma once

#include "ani_common.cuh"
#include "ani_device_math.cuh"

namespace ani {

constexpr int kPadStride = 36;  // 32 pairs + 4 words: keeps the 16-byte reads of pass C conflict-free

template <typename T, int CAPT, int CAPR> struct FeaturizeWarpShared {
    Vec4<T> ang_u[kTypes * CAPT];   // (x_i - x_j) / r_ij and r_ij, per-element sub-lists
    T ang_fc[kTypes * CAPT];        // f_C(r_ij, A_Rc)
    Vec2<T> rad[kTypes * CAPR];     // (r_ij, f_C(r_ij, R_Rc)), per-element sub-lists
    alignas(16) T A[kNumThetas][kPadStride];
    alignas(16) T BF[kNumARs][kPadStride];
    PairTables pt;
};

template <typename T> __device__ __forceinline__ T* element_buffer(int t, T* h, T* c, T* n, T* o)
{
    return t == 0 ? h : (t == 1 ? c : (t == 2 ? n : o));
}

// Slow path for an atom whose neighbourhood does not fit the sub-lists: every pair of molecule
// atoms is tested directly, lane = (theta, shift) for the angular part and lane = (half,
// radial shift) for the radial part.  Same results; O(n^2) distance tests per atom.
template <typename T>
__device__ __noinline__ void featurize_atom_streaming(const T* __restrict__ xs,
                                                      const T* __restrict__ ys,
                                                      const T* __restrict__ zs,
                                                      const int* __restrict__ types, int base,
                                                      int n, int i, T* row)
{
    const int lane = lane_id();
    const T xi = xs[base + i], yi = ys[base + i], zi = zs[base + i];
    {
        const int half = lane >> 4;
        const T shift = (T)c_tab.R_Rs[lane & 15];
        T acc[kTypes] = {(T)0, (T)0, (T)0, (T)0};
        for (int j = half; j < n; j += 2) {
            if (j == i) continue;
            const T dx = xi - xs[base + j], dy = yi - ys[base + j], dz = zi - zs[base + j];
            const T r = Num<T>::sqrt_(dx * dx + dy * dy + dz * dz);
            if (r < (T)kR_Rc) {
                const T d = r - shift;
                const T v = Num<T>::exp_neg((T)kR_eta, d * d) * cutoff_value<T>(r, (T)kR_Rc);
                const int tj = types[base + j] & 3;
#pragma unroll
                for (int g = 0; g < kTypes; g++) acc[g] += tj == g ? v : (T)0;
            }
        }
#pragma unroll
        for (int g = 0; g < kTypes; g++) acc[g] += __shfl_xor_sync(kFull, acc[g], 16);
        row[lane] = lane < 16 ? acc[0] : acc[1];
        row[32 + lane] = lane < 16 ? acc[2] : acc[3];
    }
    const T ct = (T)c_tab.cos_t[lane >> 2], st = (T)c_tab.sin_t[lane >> 2];
    const T shift = (T)c_tab.A_Rs[lane & 3];
    T acc[kPairBuckets];
#pragma unroll
    for (int b = 0; b < kPairBuckets; b++) acc[b] = (T)0;
    for (int j = 0; j < n; j++) {
        if (j == i) continue;
        const T dxj = xi - xs[base + j], dyj = yi - ys[base + j], dzj = zi - zs[base + j];
        const T rj = Num<T>::sqrt_(dxj * dxj + dyj * dyj + dzj * dzj);
        if (!(rj < (T)kA_Rc)) continue;
        const T fj = cutoff_value<T>(rj, (T)kA_Rc);
        const int tj = types[base + j] & 3;
        for (int k = j + 1; k < n; k++) {
            if (k == i) continue;
            const T dxk = xi - xs[base + k], dyk = yi - ys[base + k], dzk = zi - zs[base + k];
            const T rk = Num<T>::sqrt_(dxk * dxk + dyk * dyk + dzk * dzk);
            if (!(rk < (T)kA_Rc)) continue;
            const T fk = cutoff_value<T>(rk, (T)kA_Rc);
            T c = (dxj * dxk + dyj * dyk + dzj * dzk) / (rj * rk);
            c = Num<T>::max_((T)-1, Num<T>::min_((T)1, c));
            const T s = Num<T>::sqrt_(Num<T>::max_((T)0, (T)1 - c * c));
            const T b = (T)1 + (c * ct + s * st);
            const T b2 = b * b, b4 = b2 * b2;
            const T d = (T)0.5 * (rj + rk) - shift;
            const T v = b4 * b4 * Num<T>::exp_neg((T)kA_eta, d * d) * ((T)kA_pref * fj * fk);
            const int bk = pair_bucket(tj, types[base + k] & 3);
#pragma unroll
            for (int q = 0; q < kPairBuckets; q++) acc[q] += bk == q ? v : (T)0;
        }
    }
#pragma unroll
    for (int b = 0; b < kPairBuckets; b++) row[kRadial + b * kTS + lane] = acc[b];
}

#ifndef ANI_FWD_MIN_CTAS
#define ANI_FWD_MIN_CTAS 8
#endif

template <typename T, int NW, int CAPT, int CAPR>
__global__ void __launch_bounds__(NW* kWarp, sizeof(T) == 4 ? ANI_FWD_MIN_CTAS * 4 / NW : 1)
    featurize_kernel(const T* __restrict__ xs, const T* __restrict__ ys, const T* __restrict__ zs,
                     const int* __restrict__ types, const int* __restrict__ mol_offsets,
                     const int* __restrict__ mol_counts, int n_mols, int n_atoms, int slot_shift,
                     const int* __restrict__ scatter, T* out_h, T* out_c, T* out_n, T* out_o,
                     int acs0, int acs1, int acs2, int acs3)
{
    extern __shared__ __align__(128) unsigned char smem_raw[];
    using WarpShared = FeaturizeWarpShared<T, CAPT, CAPR>;
    const int lane = lane_id(), warp = warp_id();
    WarpShared& ws = reinterpret_cast<WarpShared*>(smem_raw)[warp];

    // The angular list is read at entry 0 by padding lanes and may be read before this warp
    // ever wrote it: give every entry a finite value once.
    for (int e = lane; e < kTypes * CAPT; e += kWarp) {
        ws.ang_u[e] = Vec4<T>{(T)1, (T)0, (T)0, (T)1};
        ws.ang_fc[e] = (T)0;
    }
    __syncwarp();

    __shared__ int cta_next_item;
    if (threadIdx.x == 0) cta_next_item = 0;
    __syncthreads();
    for (;;) {
        int m, slot;
        if (!next_work<NW>(&cta_next_item, n_mols, slot_shift & 31, (slot_shift & 32) != 0, &m, &slot)) break;
        if (slot >= mol_counts[m]) continue;   // empty item: one cached load
        MolRange mol;
        if (!load_molecule(mol_offsets, mol_counts, m, n_atoms, &mol)) continue;
        const int n = mol.n, base = mol.base;

        for (int i = slot; i < n; i += 1 << (slot_shift & 31)) {
            const int gi = base + i;
            // everything this atom needs from global memory is requested before any of it is used
            const int j_first = lane < n ? lane : 0;
            T px = xs[base + j_first], py = ys[base + j_first], pz = zs[base + j_first];
            int pt = types[base + j_first];
            const T xi = xs[gi], yi = ys[gi], zi = zs[gi];
            const int ti = checked_type(types[gi]);
            const int srow = scatter[gi];
            const int cap = ti == 0 ? acs0 : (ti == 1 ? acs1 : (ti == 2 ? acs2 : acs3));
            if (srow < 0 || srow >= cap) {
                if (lane == 0) report(ANI_ERR_BAD_INDEX);
                continue;
            }
            T* row = element_buffer<T>(ti, out_h, out_c, out_n, out_o) + (size_t)srow * kTotal;

            // ---- A: neighbour scan, lane = j ----
            int cA[kTypes] = {0, 0, 0, 0}, cR[kTypes] = {0, 0, 0, 0};
            for (int j0 = 0; j0 < n; j0 += kWarp) {
                const int j = j0 + lane;
                const bool live = j < n;
                if (j0 > 0) {   // chunk 0 was requested above
                    const int gj = base + (live ? j : 0);
                    px = xs[gj]; py = ys[gj]; pz = zs[gj];
                    pt = types[gj];
                }
                const T dx = xi - px, dy = yi - py, dz = zi - pz;
                const int tj = live ? checked_type(pt) : -1;
                T r, inv;
                length_and_inverse(dx * dx + dy * dy + dz * dz, &r, &inv);
                const bool in_rad = live && j != i && r < (T)kR_Rc;
                const bool in_ang = in_rad && r < (T)kA_Rc;
                unsigned tm[kTypes];
#pragma unroll
                for (int g = 0; g < kTypes; g++) tm[g] = __ballot_sync(kFull, tj == g);
                const unsigned mR = __ballot_sync(kFull, in_rad);
                const unsigned mA = __ballot_sync(kFull, in_ang);
                const unsigned mine = pick4(tm, tj) & lanemask_lt();
                if (in_rad) {
                    const int pos = pick4(cR, tj) + __popc(mR & mine);
                    if (pos < CAPR) ws.rad[tj * CAPR + pos] = Vec2<T>{r, cutoff_value<T>(r, (T)kR_Rc)};
                }
                if (in_ang) {
                    const int pos = pick4(cA, tj) + __popc(mA & mine);
                    if (pos < CAPT) {
                        ws.ang_u[tj * CAPT + pos] = Vec4<T>{dx * inv, dy * inv, dz * inv, r};
                        ws.ang_fc[tj * CAPT + pos] = cutoff_value<T>(r, (T)kA_Rc);
                    }
                }
#pragma unroll
                for (int g = 0; g < kTypes; g++) {
                    cR[g] += __popc(mR & tm[g]);
                    cA[g] += __popc(mA & tm[g]);
                }
            }
            __syncwarp();
            bool fits = true;
#pragma unroll
            for (int g = 0; g < kTypes; g++) fits = fits && cA[g] <= CAPT && cR[g] <= CAPR;
            if (!fits) {
                featurize_atom_streaming<T>(xs, ys, zs, types, base, n, i, row);
                __syncwarp();
                continue;
            }

            // ---- R: radial features, lane = (element of the neighbour, pair of shifts): every lane
            // walks the radial sub-list of its element and finishes two of the 64 features ----
            {
                const int g = lane >> 3, sp = lane & 7;
                const Pair<T> neg_shift{-(T)c_tab.R_Rs[2 * sp], -(T)c_tab.R_Rs[2 * sp + 1]};
                const int n_g = pick4(cR, g);
                const int n_max = max(max(cR[0], cR[1]), max(cR[2], cR[3]));
                Pair<T> acc{(T)0, (T)0};
                for (int p = 0; p < n_max; p++) {
                    if (p < n_g) {
                        const Vec2<T> e = ws.rad[g * CAPR + p];
                        const Pair<T> d = padd(Pair<T>{e.x, e.x}, neg_shift);
                        const Pair<T> d2 = pmul(d, d);
                        const Pair<T> v{Num<T>::exp_neg((T)kR_eta, d2.x), Num<T>::exp_neg((T)kR_eta, d2.y)};
                        acc = pfma(v, Pair<T>{e.y, e.y}, acc);
                    }
                }
                *reinterpret_cast<Vec2<T>*>(row + g * kNumRs + 2 * sp) = Vec2<T>{acc.x, acc.y};
            }

            // ---- B + C: angular features ----
            const int total = build_pair_tables<CAPT>(ws.pt, cA);
            if (total > kMaxPaddedPairs) {   // more pairs than the bucket table covers: slow path
                featurize_atom_streaming<T>(xs, ys, zs, types, base, n, i, row);
                __syncwarp();
                continue;
            }
            const T* a_row = &ws.A[lane >> 2][0];
            const T* b_row = &ws.BF[lane & 3][0];
            // blocks of element pairs that do not occur around this atom are zero
#pragma unroll
            for (int bk = 0; bk < kPairBuckets; bk++)
                if (ws.pt.off[bk + 1] == ws.pt.off[bk]) row[kRadial + bk * kTS + lane] = (T)0;
            Pair<T> acc{(T)0, (T)0};
            for (int c0 = 0; c0 < total; c0 += kWarp) {
                {   // B: lane = pair
                    int bk, a, b;
                    const bool valid = decode_pair(ws.pt, c0 + lane, &bk, &a, &b);
                    const Vec4<T> ua = ws.ang_u[a], ub = ws.ang_u[b];
                    const T cosv = ua.x * ub.x + ua.y * ub.y + ua.z * ub.z;
                    const T rbar = (T)0.5 * (ua.w + ub.w);
                    const T fcprod = valid ? ws.ang_fc[a] * ws.ang_fc[b] : (T)0;
                    T A[kNumThetas], BF[kNumARs];
                    angular_factors_dev<T>(cosv, rbar, fcprod, A, BF);
#pragma unroll
                    for (int t = 0; t < kNumThetas; t++) ws.A[t][lane] = A[t];
#pragma unroll
                    for (int q = 0; q < kNumARs; q++) ws.BF[q][lane] = BF[q];
                }
                __syncwarp();
                {   // C: lane = (theta, shift).  All 8 quads of the chunk, fully unrolled (slots past
                    // the end of the list hold zeros).  A block is written when the next quad belongs
                    // to another element pair; ids[8] is the first quad of the next chunk.
                    const unsigned long long ids = *reinterpret_cast<const unsigned long long*>(&ws.pt.quad_bucket[c0 >> 2]);
                    const unsigned next_id = ws.pt.quad_bucket[(c0 >> 2) + 8];
#pragma unroll
                    for (int q = 0; q < 8; q++) {
                        if (c0 + 4 * q >= total) break;   // the rest of the chunk is past the list
                        T av[4], bv[4];
                        load4(a_row + 4 * q, av);
                        load4(b_row + 4 * q, bv);
                        acc = pfma(Pair<T>{av[0], av[1]}, Pair<T>{bv[0], bv[1]}, acc);
                        acc = pfma(Pair<T>{av[2], av[3]}, Pair<T>{bv[2], bv[3]}, acc);
                        const unsigned id = (unsigned)(ids >> (8 * q)) & 0xffu;
                        const unsigned id_next = q < 7 ? (unsigned)(ids >> (8 * q + 8)) & 0xffu : next_id;
                        if (id != id_next && id < kPairBuckets) {
                            row[kRadial + id * kTS + lane] = acc.x + acc.y;
                            acc = Pair<T>{(T)0, (T)0};
                        }
                    }
                }
                __syncwarp();
            }
        }
    }
}

}  // namespace ani
