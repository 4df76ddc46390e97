// Coordinate-gradient (vector-Jacobian product) kernel: dL/dx, dL/dy, dL/dz from dL/dAEV.
//
// Computes what featurize_grad_cpu of the reference computes
// (gpu_featurizer/kernel_cpu.cpp:217-366); the reference has no GPU kernel for this op.
//
// Same decomposition as the forward kernel: CTA = molecule, warp = central atom i.  The
// warp copies the 384 upstream values of row(i) into shared memory, then
//   R. lane = radial neighbour j: contracts the 16 upstream values of block type(j) with the
//      radial derivatives and pushes +/- D u_ij onto atoms i and j;
//   B. lane = neighbour pair (j, k): contracts the 32 upstream values of block
//      (type j, type k) into three scalars (dL/dcos, dL/dr_ij, dL/dr_ik), turns them into
//      the forces on j and k, and adds those to per-neighbour accumulators of the warp.
// The force on i is minus the sum over its neighbours (every term depends on coordinate
// differences only).  Forces are summed per molecule in shared memory and written once.
#pragma once

#include "ani_common.cuh"

namespace ani {

constexpr int kGradBucketStride = 36;  // upstream values of one type pair, padded against bank conflicts
constexpr int kGradRowWords = kRadial + kPairBuckets * kGradBucketStride;

template <typename T, int ACAP> struct GradWarpShared {
    T g[kGradRowWords];      // upstream row: radial [0,64), then 10 blocks of 32 at stride 36
    T facc[ACAP][3];         // force on each angular neighbour, from this central atom
    PairBucket tab[kPairBuckets + 1];
};

template <typename T, int NW, int ACAP, int RCAP> struct GradShared {
    MolShared<T> mol;
    T fmol[kMaxAtomsPerMol][3];  // per-slot gradient of the molecule
    NeighborLists<T, ACAP, RCAP, true> nl[NW];
    GradWarpShared<T, ACAP> ws[NW];
};

// Slow path for an atom whose neighbourhood does not fit the lists.  lane = k for the
// angular part (j is a warp-uniform loop), lane = j for the radial part.
template <typename T>
__device__ __noinline__ void grad_atom_streaming(const MolShared<T>& ms, int n, int i, const T* g,
                                                 T (*fmol)[3])
{
    const int lane = lane_id();
    const T xi = ms.x[i], yi = ms.y[i], zi = ms.z[i];
    T fix = (T)0, fiy = (T)0, fiz = (T)0;
    for (int j = lane; j < n; j += kWarp) {
        if (j == i) continue;
        const T dx = xi - ms.x[j], dy = yi - ms.y[j], dz = zi - ms.z[j];
        const T r = Num<T>::sqrt_(dx * dx + dy * dy + dz * dz);
        if (!(r < (T)kR_Rc)) continue;
        T fc, dfc;
        cutoff<T>(r, (T)kR_Rc, &fc, &dfc);
        const T d = radial_vjp<T, T>(r, fc, dfc, g + slot_type(ms.group_start, j) * kNumRs) / r;
        fix += d * dx; fiy += d * dy; fiz += d * dz;
        atomicAdd(&fmol[j][0], -d * dx);
        atomicAdd(&fmol[j][1], -d * dy);
        atomicAdd(&fmol[j][2], -d * dz);
    }
    for (int j = 0; j < n; j++) {
        if (j == i) continue;
        const T dxj = xi - ms.x[j], dyj = yi - ms.y[j], dzj = zi - ms.z[j];
        const T rj = Num<T>::sqrt_(dxj * dxj + dyj * dyj + dzj * dzj);
        if (!(rj < (T)kA_Rc)) continue;
        T fj, dfj;
        cutoff<T>(rj, (T)kA_Rc, &fj, &dfj);
        const int tj = slot_type(ms.group_start, j);
        const T ujx = dxj / rj, ujy = dyj / rj, ujz = dzj / rj;
        T fjx = (T)0, fjy = (T)0, fjz = (T)0;
        for (int k0 = j + 1; k0 < n; k0 += kWarp) {
            const int k = k0 + lane;
            if (k < n && k != i) {
                const T dxk = xi - ms.x[k], dyk = yi - ms.y[k], dzk = zi - ms.z[k];
                const T rk = Num<T>::sqrt_(dxk * dxk + dyk * dyk + dzk * dzk);
                if (rk < (T)kA_Rc) {
                    T fk, dfk;
                    cutoff<T>(rk, (T)kA_Rc, &fk, &dfk);
                    const T ukx = dxk / rk, uky = dyk / rk, ukz = dzk / rk;
                    T c = ujx * ukx + ujy * uky + ujz * ukz;
                    c = Num<T>::max_((T)-1, Num<T>::min_((T)1, c));
                    const int bk = pair_bucket(tj, slot_type(ms.group_start, k));
                    T dc, drj, drk;
                    const T s2 = sin2_from_cross<T>(ujx, ujy, ujz, ukx, uky, ukz);
                    angular_vjp<T, T>(c, s2, rj, rk, fj, dfj, fk, dfk,
                                      g + kRadial + bk * kGradBucketStride, &dc, &drj, &drk);
                    const T aj = -dc / rj, bj = c * dc / rj - drj;
                    const T ak = -dc / rk, bkk = c * dc / rk - drk;
                    const T gjx = aj * ukx + bj * ujx, gjy = aj * uky + bj * ujy, gjz = aj * ukz + bj * ujz;
                    const T gkx = ak * ujx + bkk * ukx, gky = ak * ujy + bkk * uky, gkz = ak * ujz + bkk * ukz;
                    fjx += gjx; fjy += gjy; fjz += gjz;
                    fix -= gjx + gkx; fiy -= gjy + gky; fiz -= gjz + gkz;
                    atomicAdd(&fmol[k][0], gkx);
                    atomicAdd(&fmol[k][1], gky);
                    atomicAdd(&fmol[k][2], gkz);
                }
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            fjx += __shfl_xor_sync(kFull, fjx, o);
            fjy += __shfl_xor_sync(kFull, fjy, o);
            fjz += __shfl_xor_sync(kFull, fjz, o);
        }
        if (lane == 0) {
            atomicAdd(&fmol[j][0], fjx);
            atomicAdd(&fmol[j][1], fjy);
            atomicAdd(&fmol[j][2], fjz);
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        fix += __shfl_xor_sync(kFull, fix, o);
        fiy += __shfl_xor_sync(kFull, fiy, o);
        fiz += __shfl_xor_sync(kFull, fiz, o);
    }
    if (lane == 0) {
        atomicAdd(&fmol[i][0], fix);
        atomicAdd(&fmol[i][1], fiy);
        atomicAdd(&fmol[i][2], fiz);
    }
}

template <typename T, int NW, int ACAP, int RCAP>
__global__ void __launch_bounds__(NW* kWarp)
    featurize_grad_kernel(const T* __restrict__ xs, const T* __restrict__ ys,
                          const T* __restrict__ zs, const int* __restrict__ types,
                          const int* __restrict__ mol_offsets, const int* __restrict__ mol_counts,
                          int n_mols, int n_atoms, const int* __restrict__ scatter,
                          const T* __restrict__ gh, const T* __restrict__ gc,
                          const T* __restrict__ gn, const T* __restrict__ go, T* gx, T* gy, T* gz,
                          int acs0, int acs1, int acs2, int acs3, int nsplit)
{
    extern __shared__ __align__(16) unsigned char smem_raw[];
    auto& sh = *reinterpret_cast<GradShared<T, NW, ACAP, RCAP>*>(smem_raw);
    const int lane = lane_id(), warp = warp_id();
    auto& nl = sh.nl[warp];
    auto& ws = sh.ws[warp];

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
        __syncthreads();
        for (int s = threadIdx.x; s < n * 3; s += NW * kWarp) (&sh.fmol[0][0])[s] = (T)0;
        stage_molecule<T, NW>(sh.mol, xs, ys, zs, types, base, n);
        const MolShared<T>& ms = sh.mol;

        for (int i = n - 1 - (split * NW + warp); i >= 0; i -= nsplit * NW) {
            const int ti = slot_type(ms.group_start, i);
            const int gi = base + ms.orig[i];
            const int srow = scatter[gi];
            const int cap = ti == 0 ? acs0 : (ti == 1 ? acs1 : (ti == 2 ? acs2 : acs3));
            if (srow < 0 || srow >= cap) {
                if (lane == 0) report(ANI_ERR_BAD_INDEX);
                continue;
            }
            const T* grow = (ti == 0 ? gh : (ti == 1 ? gc : (ti == 2 ? gn : go))) + (size_t)srow * kTotal;
            // upstream row -> shared memory (12 coalesced loads of 32 values)
            ws.g[lane] = grow[lane];
            ws.g[32 + lane] = grow[32 + lane];
#pragma unroll
            for (int bk = 0; bk < kPairBuckets; bk++)
                ws.g[kRadial + bk * kGradBucketStride + lane] = grow[kRadial + bk * kTS + lane];

            NeighborCounts nc;
            const bool fits = build_neighbors<T, ACAP, RCAP, true>(ms, n, i, nl, nc);  // ends with __syncwarp
            if (!fits) {
                grad_atom_streaming<T>(ms, n, i, ws.g, sh.fmol);
                __syncwarp();
                continue;
            }

            T fix = (T)0, fiy = (T)0, fiz = (T)0;
            // ---- R: radial, lane = neighbour ----
            {
                const int c1 = nc.rad[0], c2 = c1 + nc.rad[1], c3 = c2 + nc.rad[2];
                for (int p = lane; p < nc.n_rad; p += kWarp) {
                    const int tj = (p >= c1) + (p >= c2) + (p >= c3);
                    const T d = radial_vjp<T, T>(nl.rad_r[p], nl.rad_fc[p], nl.rad_dfc[p],
                                                 ws.g + tj * kNumRs);
                    const T fx = d * nl.rad_ux[p], fy = d * nl.rad_uy[p], fz = d * nl.rad_uz[p];
                    fix += fx; fiy += fy; fiz += fz;
                    const int sj = nl.rad_slot[p];
                    atomicAdd(&sh.fmol[sj][0], -fx);
                    atomicAdd(&sh.fmol[sj][1], -fy);
                    atomicAdd(&sh.fmol[sj][2], -fz);
                }
            }
            // ---- B: angular, lane = pair ----
            for (int p = lane; p < nc.n_ang; p += kWarp) {
                ws.facc[p][0] = (T)0;
                ws.facc[p][1] = (T)0;
                ws.facc[p][2] = (T)0;
            }
            const int total = build_pair_table(ws.tab, nc.ang);  // ends with __syncwarp
            for (int c0 = 0; c0 < total; c0 += kWarp) {
                int bk, a, b;
                const bool valid = decode_pair(ws.tab, c0 + lane, &bk, &a, &b);
                if (valid) {
                    const T uax = nl.ang_ux[a], uay = nl.ang_uy[a], uaz = nl.ang_uz[a];
                    const T ubx = nl.ang_ux[b], uby = nl.ang_uy[b], ubz = nl.ang_uz[b];
                    const T ra = nl.ang_r[a], rb = nl.ang_r[b];
                    T c = uax * ubx + uay * uby + uaz * ubz;
                    c = Num<T>::max_((T)-1, Num<T>::min_((T)1, c));
                    T gl[kTS];
                    const T* gsrc = ws.g + kRadial + bk * kGradBucketStride;
#pragma unroll
                    for (int q = 0; q < kTS; q++) gl[q] = gsrc[q];
                    T dc, dra, drb;
                    const T s2 = sin2_from_cross<T>(uax, uay, uaz, ubx, uby, ubz);
                    angular_vjp<T, T>(c, s2, ra, rb, nl.ang_fc[a], nl.ang_dfc[a], nl.ang_fc[b],
                                      nl.ang_dfc[b], gl, &dc, &dra, &drb);
                    const T ira = (T)1 / ra, irb = (T)1 / rb;
                    const T aa = -dc * ira, ba = c * dc * ira - dra;
                    const T ab = -dc * irb, bb = c * dc * irb - drb;
                    atomicAdd(&ws.facc[a][0], aa * ubx + ba * uax);
                    atomicAdd(&ws.facc[a][1], aa * uby + ba * uay);
                    atomicAdd(&ws.facc[a][2], aa * ubz + ba * uaz);
                    atomicAdd(&ws.facc[b][0], ab * uax + bb * ubx);
                    atomicAdd(&ws.facc[b][1], ab * uay + bb * uby);
                    atomicAdd(&ws.facc[b][2], ab * uaz + bb * ubz);
                }
            }
            __syncwarp();
            for (int p = lane; p < nc.n_ang; p += kWarp) {
                const T fx = ws.facc[p][0], fy = ws.facc[p][1], fz = ws.facc[p][2];
                fix -= fx; fiy -= fy; fiz -= fz;
                const int sj = nl.ang_slot[p];
                atomicAdd(&sh.fmol[sj][0], fx);
                atomicAdd(&sh.fmol[sj][1], fy);
                atomicAdd(&sh.fmol[sj][2], fz);
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                fix += __shfl_xor_sync(kFull, fix, o);
                fiy += __shfl_xor_sync(kFull, fiy, o);
                fiz += __shfl_xor_sync(kFull, fiz, o);
            }
            if (lane == 0) {
                atomicAdd(&sh.fmol[i][0], fix);
                atomicAdd(&sh.fmol[i][1], fiy);
                atomicAdd(&sh.fmol[i][2], fiz);
            }
            __syncwarp();
        }
        __syncthreads();
        for (int s = threadIdx.x; s < n; s += NW * kWarp) {
            const int gi = base + ms.orig[s];
            if (nsplit == 1) {
                gx[gi] = sh.fmol[s][0];
                gy[gi] = sh.fmol[s][1];
                gz[gi] = sh.fmol[s][2];
            } else {
                atomicAdd(&gx[gi], sh.fmol[s][0]);
                atomicAdd(&gy[gi], sh.fmol[s][1]);
                atomicAdd(&gz[gi], sh.fmol[s][2]);
            }
        }
    }
}

// Zero fill of the three gradient arrays in one launch (atoms that belong to no molecule, or
// to a skipped one, must read as zero, as they do after the reference's memset,
// gpu_featurizer/functor_op_cpu.cpp:70-72).
template <typename T> __global__ void zero3_kernel(T* a, T* b, T* c, int n)
{
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        a[i] = (T)0;
        b[i] = (T)0;
        c[i] = (T)0;
    }
}

}  // namespace ani
