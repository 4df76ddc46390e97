// Coordinate-gradient (vector-Jacobian product) kernel: dL/dx, dL/dy, dL/dz from dL/dAEV.
//
// Computes what featurize_grad_cpu of the reference computes
// (gpu_featurizer/kernel_cpu.cpp:217-366); the reference has no GPU kernel for this op.
//
// One warp per central atom i (see ani_common.cuh).  The warp copies the 384 upstream values of
// row(i) into shared memory, then
//   A. scans the molecule with lane = candidate neighbour j.  A lane whose j is within R_Rc
//      contracts the 16 upstream values of radial block type(j) with the radial derivatives on
//      the spot and adds -D u_ij to the gradient of atom j; neighbours within A_Rc are also
//      compacted into the per-element angular sub-lists;
//   B. walks the neighbour pairs 32 at a time with lane = pair (j, k): the 32 upstream values of
//      block (type j, type k) are contracted into three scalars (dL/dcos, dL/dr_ij, dL/dr_ik),
//      turned into the forces on j and k and added to per-neighbour accumulators of the warp;
//   C. adds every neighbour's accumulated force to the output and, since all terms depend on
//      coordinate differences only, minus the total to atom i.
// Contributions of different central atoms to the same atom meet in the output arrays through
// floating-point atomic adds, so the outputs must be zero before the kernel starts and the
// summation order (hence the last bits) may differ between runs.
#pragma once

#include "ani_common.cuh"

namespace ani {

constexpr int kGradBucketStride = 36;  // upstream values of one type pair, padded against bank conflicts
constexpr int kGradRowWords = kRadial + kPairBuckets * kGradBucketStride;

template <typename T, int CAPT> struct GradWarpShared {
    AngularList<T, CAPT, true> ang;
    alignas(16) T g[kGradRowWords];  // upstream row: radial [0,64), then 10 blocks of 32 at stride 36
    T facc[kTypes * CAPT][3];        // force on each angular neighbour, from this central atom
    alignas(16) PairBucketInfo tab[kPairBuckets];
    int off[kPairBuckets + 2];
};

// Slow path for an atom whose angular neighbourhood does not fit the sub-lists: angular part
// only (the radial part never needs a list).  lane = k, j is a warp-uniform loop.
template <typename T>
__device__ __noinline__ void grad_atom_streaming(const T* __restrict__ xs, const T* __restrict__ ys,
                                                 const T* __restrict__ zs,
                                                 const int* __restrict__ types, int base, int n,
                                                 int i, const T* g, T* gx, T* gy, T* gz)
{
    const int lane = lane_id();
    const T xi = xs[base + i], yi = ys[base + i], zi = zs[base + i];
    T fix = (T)0, fiy = (T)0, fiz = (T)0;
    for (int j = 0; j < n; j++) {
        if (j == i) continue;
        const T dxj = xi - xs[base + j], dyj = yi - ys[base + j], dzj = zi - zs[base + j];
        const T rj = Num<T>::sqrt_(dxj * dxj + dyj * dyj + dzj * dzj);
        if (!(rj < (T)kA_Rc)) continue;
        T fj, dfj;
        cutoff<T>(rj, (T)kA_Rc, &fj, &dfj);
        const int tj = types[base + j] & 3;
        const T ujx = dxj / rj, ujy = dyj / rj, ujz = dzj / rj;
        T fjx = (T)0, fjy = (T)0, fjz = (T)0;
        for (int k0 = j + 1; k0 < n; k0 += kWarp) {
            const int k = k0 + lane;
            if (k < n && k != i) {
                const T dxk = xi - xs[base + k], dyk = yi - ys[base + k], dzk = zi - zs[base + k];
                const T rk = Num<T>::sqrt_(dxk * dxk + dyk * dyk + dzk * dzk);
                if (rk < (T)kA_Rc) {
                    T fk, dfk;
                    cutoff<T>(rk, (T)kA_Rc, &fk, &dfk);
                    const T ukx = dxk / rk, uky = dyk / rk, ukz = dzk / rk;
                    T c = ujx * ukx + ujy * uky + ujz * ukz;
                    c = Num<T>::max_((T)-1, Num<T>::min_((T)1, c));
                    const int bk = pair_bucket(tj, types[base + k] & 3);
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
                    atomicAdd(&gx[base + k], gkx);
                    atomicAdd(&gy[base + k], gky);
                    atomicAdd(&gz[base + k], gkz);
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
            atomicAdd(&gx[base + j], fjx);
            atomicAdd(&gy[base + j], fjy);
            atomicAdd(&gz[base + j], fjz);
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        fix += __shfl_xor_sync(kFull, fix, o);
        fiy += __shfl_xor_sync(kFull, fiy, o);
        fiz += __shfl_xor_sync(kFull, fiz, o);
    }
    if (lane == 0) {
        atomicAdd(&gx[base + i], fix);
        atomicAdd(&gy[base + i], fiy);
        atomicAdd(&gz[base + i], fiz);
    }
}

template <typename T, int NW, int CAPT>
__global__ void __launch_bounds__(NW* kWarp)
    featurize_grad_kernel(const T* __restrict__ xs, const T* __restrict__ ys,
                          const T* __restrict__ zs, const int* __restrict__ types,
                          const int* __restrict__ mol_offsets, const int* __restrict__ mol_counts,
                          int n_mols, int n_atoms, const int* __restrict__ scatter,
                          const T* __restrict__ gh, const T* __restrict__ gc,
                          const T* __restrict__ gn, const T* __restrict__ go, T* gx, T* gy, T* gz,
                          int acs0, int acs1, int acs2, int acs3)
{
    extern __shared__ __align__(16) unsigned char smem_raw[];
    using WarpShared = GradWarpShared<T, CAPT>;
    const int lane = lane_id(), warp = warp_id();
    WarpShared& ws = reinterpret_cast<WarpShared*>(smem_raw)[warp];

    constexpr int kCtasPerMol = kSlotsPerMol / NW;
    for (long long cta = blockIdx.x; cta < (long long)n_mols * kCtasPerMol; cta += gridDim.x) {
        const int m = (int)(cta / kCtasPerMol);
        const int slot = (int)(cta - (long long)m * kCtasPerMol) * NW + warp;
        MolRange mol;
        if (!load_molecule(mol_offsets, mol_counts, m, n_atoms, &mol)) continue;
        const int n = mol.n, base = mol.base;

        for (int i = slot; i < n; i += kSlotsPerMol) {
            const int gi = base + i;
            const int ti = checked_type(types[gi]);
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
            __syncwarp();
            const T xi = xs[gi], yi = ys[gi], zi = zs[gi];
            T fix = (T)0, fiy = (T)0, fiz = (T)0;  // this lane's share of the force on atom i

            // ---- A: neighbour scan + radial part, lane = j ----
            int cA[kTypes] = {0, 0, 0, 0};
            for (int j0 = 0; j0 < n; j0 += kWarp) {
                const int j = j0 + lane;
                const bool live = j < n;
                const int gj = base + (live ? j : 0);
                const T dx = xi - xs[gj], dy = yi - ys[gj], dz = zi - zs[gj];
                const int tj = live ? checked_type(types[gj]) : -1;
                const T r = Num<T>::sqrt_(dx * dx + dy * dy + dz * dz);
                const bool in_rad = live && j != i && r < (T)kR_Rc;
                const bool in_ang = in_rad && r < (T)kA_Rc;
                T ux = (T)0, uy = (T)0, uz = (T)0;
                if (in_rad) {
                    const T inv = (T)1 / r;
                    ux = dx * inv; uy = dy * inv; uz = dz * inv;
                    T fc, dfc;
                    cutoff<T>(r, (T)kR_Rc, &fc, &dfc);
                    const T d = radial_vjp<T, T>(r, fc, dfc, ws.g + tj * kNumRs);
                    const T fx = d * ux, fy = d * uy, fz = d * uz;
                    fix += fx; fiy += fy; fiz += fz;
                    atomicAdd(&gx[gj], -fx);
                    atomicAdd(&gy[gj], -fy);
                    atomicAdd(&gz[gj], -fz);
                }
                T fcA = (T)0, dfcA = (T)0;
                if (in_ang) cutoff<T>(r, (T)kA_Rc, &fcA, &dfcA);
#pragma unroll
                for (int g = 0; g < kTypes; g++) {
                    const unsigned mA = __ballot_sync(kFull, in_ang && tj == g);
                    if (in_ang && tj == g) {
                        const int pos = cA[g] + __popc(mA & lanemask_lt());
                        if (pos < CAPT) {
                            const int e = g * CAPT + pos;
                            ws.ang.ux[e] = ux;
                            ws.ang.uy[e] = uy;
                            ws.ang.uz[e] = uz;
                            ws.ang.r[e] = r;
                            ws.ang.fc[e] = fcA;
                            ws.ang.dfc[e] = dfcA;
                            ws.ang.atom[e] = gj;
                            ws.facc[e][0] = (T)0;
                            ws.facc[e][1] = (T)0;
                            ws.facc[e][2] = (T)0;
                        }
                    }
                    cA[g] += __popc(mA);
                }
            }
            __syncwarp();
            bool fits = true;
#pragma unroll
            for (int g = 0; g < kTypes; g++) fits = fits && cA[g] <= CAPT;

            if (!fits) {
                grad_atom_streaming<T>(xs, ys, zs, types, base, n, i, ws.g, gx, gy, gz);
            } else {
                // ---- B: angular part, lane = pair ----
                PairOffsets po;
                build_pair_table<CAPT>(ws.tab, ws.off, cA, &po);
                const int total = po.off[kPairBuckets];
                for (int c0 = 0; c0 < total; c0 += kWarp) {
                    int bk, a, b;
                    const bool valid = decode_pair(ws.tab, po, c0 + lane, &bk, &a, &b);
                    if (valid) {
                        const T uax = ws.ang.ux[a], uay = ws.ang.uy[a], uaz = ws.ang.uz[a];
                        const T ubx = ws.ang.ux[b], uby = ws.ang.uy[b], ubz = ws.ang.uz[b];
                        const T ra = ws.ang.r[a], rb = ws.ang.r[b];
                        T c = uax * ubx + uay * uby + uaz * ubz;
                        c = Num<T>::max_((T)-1, Num<T>::min_((T)1, c));
                        const T s2 = sin2_from_cross<T>(uax, uay, uaz, ubx, uby, ubz);
                        T gl[kTS];
                        const T* gsrc = ws.g + kRadial + bk * kGradBucketStride;
#pragma unroll
                        for (int q = 0; q < kTS; q += 4) load4(gsrc + q, gl + q);
                        T dc, dra, drb;
                        angular_vjp<T, T>(c, s2, ra, rb, ws.ang.fc[a], ws.ang.dfc[a], ws.ang.fc[b],
                                          ws.ang.dfc[b], gl, &dc, &dra, &drb);
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
                // ---- C: push the neighbour forces out ----
#pragma unroll
                for (int g = 0; g < kTypes; g++) {
                    for (int p = lane; p < cA[g]; p += kWarp) {
                        const int e = g * CAPT + p;
                        const T fx = ws.facc[e][0], fy = ws.facc[e][1], fz = ws.facc[e][2];
                        fix -= fx; fiy -= fy; fiz -= fz;
                        const int gj = ws.ang.atom[e];
                        atomicAdd(&gx[gj], fx);
                        atomicAdd(&gy[gj], fy);
                        atomicAdd(&gz[gj], fz);
                    }
                }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                fix += __shfl_xor_sync(kFull, fix, o);
                fiy += __shfl_xor_sync(kFull, fiy, o);
                fiz += __shfl_xor_sync(kFull, fiz, o);
            }
            if (lane == 0) {
                atomicAdd(&gx[gi], fix);
                atomicAdd(&gy[gi], fiy);
                atomicAdd(&gz[gi], fiz);
            }
            __syncwarp();
        }
    }
}

// Zero fill of the three gradient arrays in one launch (the gradient kernel accumulates into
// them; the reference zero-fills in its functor, gpu_featurizer/functor_op_cpu.cpp:70-72).
template <typename T> __global__ void zero3_kernel(T* a, T* b, T* c, int n)
{
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n; i += gridDim.x * blockDim.x) {
        a[i] = (T)0;
        b[i] = (T)0;
        c[i] = (T)0;
    }
}

}  // namespace ani
