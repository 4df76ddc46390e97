// Damped Coulomb energy of every molecule and its derivative with respect to the charges.
//
//   E_m = k_e * sum_{i<j} q_i q_j (1 - f_C(r_ij, R_Rc)) / r_ij ,    dL/dq_i = dL/dE_m * dE_m/dq_i .
//
// Both follow from the damped potential at every atom,
//   phi_i = sum_{j != i} q_j (1 - f_C(r_ij)) / r_ij :   E_m = k_e/2 sum_i q_i phi_i,  dE_m/dq_i = k_e phi_i,
// so one routine serves the two kernels.  One warp per molecule: the warp walks the molecule in
// chunks of 32 atoms, lane = atom i; for every chunk of partners it loads 32 atoms (lane = j,
// coalesced) and hands them round by shuffle, so each coordinate is read from memory once per
// chunk pair and nothing is accumulated with atomics (results are bit-reproducible).
// 1 - f_C = sin^2(pi r / (2 R_Rc)) is used directly, which has no cancellation at short range.
//
// Replaces AniCharge / AniChargeGrad of the reference: gpu_featurizer/ani_charges.cpp:58-71,138-160
// (CPU) and gpu_featurizer/ani_charges_gpu.cu:70-128,197-260 (one block per molecule, one global
// atomicAdd per thread, and one per pair in the gradient).
#pragma once

#include "ani_common.cuh"

namespace ani {

constexpr float kChargeConstant = 0.529176917f;   // gpu_featurizer/parameters.h:10

template <typename T> __device__ __forceinline__ T damped_inverse_distance(T d2)
{
    // (1 - f_C(r, R_Rc)) / r with full-precision library math: the kernel is limited by memory
    // and latency, not by arithmetic
    const T r = sqrt(d2);
    if (!(r <= (T)kR_Rc)) return (T)1 / r;
    const T s = sin(r * (Num<T>::kPi / ((T)2 * (T)kR_Rc)));
    return s * s / r;
}

// phi of atom i0 + lane of the molecule [base, base + n); lanes past the end return 0.
template <typename T>
__device__ __forceinline__ T damped_potential(const T* __restrict__ xs, const T* __restrict__ ys,
                                              const T* __restrict__ zs, const T* __restrict__ qs,
                                              int base, int n, int i0)
{
    const int lane = lane_id();
    const int i = i0 + lane;
    const int gi = base + (i < n ? i : 0);
    const T xi = xs[gi], yi = ys[gi], zi = zs[gi];
    T phi = (T)0;
    for (int j0 = 0; j0 < n; j0 += kWarp) {
        const int j = j0 + lane;
        const int gj = base + (j < n ? j : 0);
        const T xj = xs[gj], yj = ys[gj], zj = zs[gj];
        const T qj = j < n ? qs[gj] : (T)0;
        const int cnt = min(kWarp, n - j0);
        for (int jj = 0; jj < cnt; jj++) {
            const T bx = __shfl_sync(kFull, xj, jj), by = __shfl_sync(kFull, yj, jj);
            const T bz = __shfl_sync(kFull, zj, jj), bq = __shfl_sync(kFull, qj, jj);
            const T dx = xi - bx, dy = yi - by, dz = zi - bz;
            if (j0 + jj != i) phi += bq * damped_inverse_distance<T>(dx * dx + dy * dy + dz * dz);
        }
    }
    return i < n ? phi : (T)0;
}

template <typename T, int NW>
__global__ void __launch_bounds__(NW* kWarp)
    charge_energy_kernel(const T* __restrict__ xs, const T* __restrict__ ys, const T* __restrict__ zs,
                         const T* __restrict__ qs, const int* __restrict__ mol_offsets,
                         const int* __restrict__ mol_counts, int n_mols, int n_atoms, T* __restrict__ energies)
{
    const int lane = lane_id();
    const int grid_warps = gridDim.x * NW;
    for (int m = blockIdx.x * NW + warp_id(); m < n_mols; m += grid_warps) {
        MolRange mol;
        T e = (T)0;
        if (load_molecule(mol_offsets, mol_counts, m, n_atoms, &mol)) {
            for (int i0 = 0; i0 < mol.n; i0 += kWarp) {
                const T phi = damped_potential<T>(xs, ys, zs, qs, mol.base, mol.n, i0);
                const int i = i0 + lane;
                e += i < mol.n ? qs[mol.base + i] * phi : (T)0;
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) e += __shfl_xor_sync(kFull, e, o);
        }
        if (lane == 0) energies[m] = (T)0.5 * (T)kChargeConstant * e;
    }
}

// q_grads must be zero-filled before the launch (atoms that belong to no molecule keep 0).
template <typename T, int NW>
__global__ void __launch_bounds__(NW* kWarp)
    charge_grad_kernel(const T* __restrict__ xs, const T* __restrict__ ys, const T* __restrict__ zs,
                       const T* __restrict__ qs, const int* __restrict__ mol_offsets,
                       const int* __restrict__ mol_counts, int n_mols, int n_atoms,
                       const T* __restrict__ energy_grads, T* __restrict__ q_grads)
{
    const int lane = lane_id();
    const int grid_warps = gridDim.x * NW;
    for (int m = blockIdx.x * NW + warp_id(); m < n_mols; m += grid_warps) {
        MolRange mol;
        if (!load_molecule(mol_offsets, mol_counts, m, n_atoms, &mol)) continue;
        const T g = energy_grads[m] * (T)kChargeConstant;
        for (int i0 = 0; i0 < mol.n; i0 += kWarp) {
            const T phi = damped_potential<T>(xs, ys, zs, qs, mol.base, mol.n, i0);
            const int i = i0 + lane;
            if (i < mol.n) q_grads[mol.base + i] = g * phi;
        }
    }
}

}  // namespace ani
