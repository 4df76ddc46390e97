// Jacobian-vector product of the featurizer: given a displacement v = (vx, vy, vz) of every
// atom, the directional derivative of every feature, written into the four per-element feature
// buffers.  This is the op behind FeaturizeGradInverse (gpu_featurizer/ani_op.cpp:224-330,
// kernel featurize_grad_inverse, gpu_featurizer/kernel_cpu.cpp:37-179), which TensorFlow calls
// when it differentiates through FeaturizeGrad (khan/training/trainer_multi_tower.py:64-91).
//
// The reference kernel reads the input vector at the ELEMENT ID of the central atom for all
// three atoms of every term (X_grads[g_atomic_num_i], kernel_cpu.cpp:111,118,155,162,169); since
// the derivatives with respect to i, j and k of a term sum to zero, its output vanishes up to
// rounding.  This kernel computes the mathematically meant product J v, with v indexed by the
// atom whose coordinate moves; it is the exact transpose of featurize_grad.
//
// One warp per central atom, lane = (theta, shift) for the angular part and lane = (half, radial
// shift) for the radial part; the neighbours are compacted into one shared-memory list in scan
// order and the pairs are walked by warp-uniform loops.  Every row is written exactly once.
#pragma once

#include "ani_common.cuh"

namespace ani {

constexpr int kJvpMaxNeighbors = 64;

template <typename T> struct JvpNeighbor {
    Vec4<T> u;     // (x_i - x_j) / r_ij, r_ij
    Vec4<T> w;     // v_i - v_j, and u . w = d r_ij along v
    T fc, dfc;     // f_C(r_ij, A_Rc) and derivative (valid when r_ij < A_Rc)
    T fcR, dfcR;   // f_C(r_ij, R_Rc) and derivative
    int type;
    int angular;   // r_ij < A_Rc
};

template <typename T> struct JvpWarpShared {
    JvpNeighbor<T> nb[kJvpMaxNeighbors];
};

// d/dr of exp(-R_eta (r - Rs)^2) f_C(r) for one radial shift.
template <typename T> __device__ __forceinline__ T radial_slope(T r, T fc, T dfc, T shift)
{
    const T d = r - shift;
    return Num<T>::exp_neg((T)kR_eta, d * d) * ((T)-2 * (T)kR_eta * d * fc + dfc);
}

// Directional derivative of the angular term (theta_t, shift_s) of one triplet.
template <typename T>
__device__ __forceinline__ T angular_jvp_term(T c, T sin2, T rj, T rk, T fj, T dfj, T fk, T dfk,
                                              T dcos, T drj, T drk, T ct, T st, T shift)
{
    const T s2 = Num<T>::min_((T)1, sin2);
    const bool bent = s2 > (T)1e-12;
    const T s = Num<T>::sqrt_(s2);
    const T cot = bent ? c * Num<T>::rsqrt_(s2) : (T)0;
    const T b = (T)1 + (c * ct + s * st);
    const T b2 = b * b, b4 = b2 * b2, b7 = b4 * b2 * b;
    const T a = b7 * b;
    const T a_c = bent ? (T)8 * b7 * (ct - st * cot) : (T)0;
    const T d = (T)0.5 * (rj + rk) - shift;
    const T e = Num<T>::exp_neg((T)kA_eta, d * d);
    const T through_rbar = -(T)kA_eta * d * e * fj * fk;
    const T pc = a_c * e * fj * fk;
    const T pj = a * (through_rbar + e * dfj * fk);
    const T pk = a * (through_rbar + e * fj * dfk);
    return (T)kA_pref * (pc * dcos + pj * drj + pk * drk);
}

template <typename T, int NW>
__global__ void __launch_bounds__(NW* kWarp)
    featurize_grad_inverse_kernel(const T* __restrict__ xs, const T* __restrict__ ys,
                                  const T* __restrict__ zs, const int* __restrict__ types,
                                  const int* __restrict__ mol_offsets,
                                  const int* __restrict__ mol_counts, int n_mols, int n_atoms, int slot_shift,
                                  const int* __restrict__ scatter, const T* __restrict__ vx,
                                  const T* __restrict__ vy, const T* __restrict__ vz, T* out_h,
                                  T* out_c, T* out_n, T* out_o, int acs0, int acs1, int acs2,
                                  int acs3)
{
    extern __shared__ __align__(128) unsigned char smem_raw[];
    using WarpShared = JvpWarpShared<T>;
    const int lane = lane_id(), warp = warp_id();
    WarpShared& ws = reinterpret_cast<WarpShared*>(smem_raw)[warp];

    __shared__ int cta_next_item;
    if (threadIdx.x == 0) cta_next_item = 0;
    __syncthreads();
    for (;;) {
        int m, slot;
        if (!next_work<NW>(&cta_next_item, n_mols, slot_shift & 31, (slot_shift & 32) != 0, &m, &slot)) break;
        if (slot >= mol_counts[m]) continue;
        MolRange mol;
        if (!load_molecule(mol_offsets, mol_counts, m, n_atoms, &mol)) continue;
        const int n = mol.n, base = mol.base;

        for (int i = slot; i < n; i += 1 << (slot_shift & 31)) {
            const int gi = base + i;
            const int ti = checked_type(types[gi]);
            const int srow = scatter[gi];
            const int cap = ti == 0 ? acs0 : (ti == 1 ? acs1 : (ti == 2 ? acs2 : acs3));
            if (srow < 0 || srow >= cap) {
                if (lane == 0) report(ANI_ERR_BAD_INDEX);
                continue;
            }
            T* row = (ti == 0 ? out_h : (ti == 1 ? out_c : (ti == 2 ? out_n : out_o))) + (size_t)srow * kTotal;
            const T xi = xs[gi], yi = ys[gi], zi = zs[gi];
            const T vxi = vx[gi], vyi = vy[gi], vzi = vz[gi];

            // ---- neighbour list (everything within R_Rc), scan order ----
            int n_nb = 0;
            for (int j0 = 0; j0 < n; j0 += kWarp) {
                const int j = j0 + lane;
                const bool live = j < n;
                const int gj = base + (live ? j : 0);
                const T dx = xi - xs[gj], dy = yi - ys[gj], dz = zi - zs[gj];
                T r, inv;
                length_and_inverse(dx * dx + dy * dy + dz * dz, &r, &inv);
                const bool in_rad = live && j != i && r < (T)kR_Rc;
                const unsigned mR = __ballot_sync(kFull, in_rad);
                if (in_rad) {
                    const int pos = n_nb + __popc(mR & lanemask_lt());
                    if (pos < kJvpMaxNeighbors) {
                        JvpNeighbor<T> e;
                        e.u = Vec4<T>{dx * inv, dy * inv, dz * inv, r};
                        const T wx = vxi - vx[gj], wy = vyi - vy[gj], wz = vzi - vz[gj];
                        e.w = Vec4<T>{wx, wy, wz, e.u.x * wx + e.u.y * wy + e.u.z * wz};
                        cutoff<T>(r, (T)kR_Rc, &e.fcR, &e.dfcR);
                        e.angular = r < (T)kA_Rc ? 1 : 0;
                        e.fc = (T)0;
                        e.dfc = (T)0;
                        if (e.angular) cutoff<T>(r, (T)kA_Rc, &e.fc, &e.dfc);
                        e.type = checked_type(types[gj]);
                        ws.nb[pos] = e;
                    }
                }
                n_nb += __popc(mR);
            }
            __syncwarp();
            if (n_nb > kJvpMaxNeighbors) {
                // Not supported by this kernel: more than 64 atoms within 4.6 A of one atom.
                if (lane == 0) report(ANI_ERR_TOO_MANY_ATOMS);
                for (int q = lane; q < kTotal; q += kWarp) row[q] = (T)0;
                continue;
            }

            // ---- radial block: lane = (half, shift) ----
            {
                const int half = lane >> 4;
                const T shift = (T)c_tab.R_Rs[lane & 15];
                T acc[kTypes] = {(T)0, (T)0, (T)0, (T)0};
                for (int p = half; p < n_nb; p += 2) {
                    const JvpNeighbor<T>& e = ws.nb[p];
                    const T val = radial_slope<T>(e.u.w, e.fcR, e.dfcR, shift) * e.w.w;
#pragma unroll
                    for (int g = 0; g < kTypes; g++) acc[g] += e.type == g ? val : (T)0;
                }
#pragma unroll
                for (int g = 0; g < kTypes; g++) acc[g] += __shfl_xor_sync(kFull, acc[g], 16);
                row[lane] = lane < 16 ? acc[0] : acc[1];
                row[32 + lane] = lane < 16 ? acc[2] : acc[3];
            }

            // ---- angular block: lane = (theta, shift), warp-uniform loops over pairs ----
            const T ct = (T)c_tab.cos_t[lane >> 2], st = (T)c_tab.sin_t[lane >> 2];
            const T shift = (T)c_tab.A_Rs[lane & 3];
            T acc[kPairBuckets];
#pragma unroll
            for (int b = 0; b < kPairBuckets; b++) acc[b] = (T)0;
            for (int a = 0; a < n_nb; a++) {
                const JvpNeighbor<T>& ea = ws.nb[a];
                if (!ea.angular) continue;
                const T ira = (T)1 / ea.u.w;
                for (int b = a + 1; b < n_nb; b++) {
                    const JvpNeighbor<T>& eb = ws.nb[b];
                    if (!eb.angular) continue;
                    T c = ea.u.x * eb.u.x + ea.u.y * eb.u.y + ea.u.z * eb.u.z;
                    c = Num<T>::max_((T)-1, Num<T>::min_((T)1, c));
                    const T s2 = sin2_from_cross<T>(ea.u.x, ea.u.y, ea.u.z, eb.u.x, eb.u.y, eb.u.z);
                    // d cos = [(u_b . w_a) - c (u_a . w_a)] / r_a + [(u_a . w_b) - c (u_b . w_b)] / r_b
                    const T ub_wa = eb.u.x * ea.w.x + eb.u.y * ea.w.y + eb.u.z * ea.w.z;
                    const T ua_wb = ea.u.x * eb.w.x + ea.u.y * eb.w.y + ea.u.z * eb.w.z;
                    const T irb = (T)1 / eb.u.w;
                    const T dcos = (ub_wa - c * ea.w.w) * ira + (ua_wb - c * eb.w.w) * irb;
                    const T val = angular_jvp_term<T>(c, s2, ea.u.w, eb.u.w, ea.fc, ea.dfc, eb.fc,
                                                      eb.dfc, dcos, ea.w.w, eb.w.w, ct, st, shift);
                    const int bk = pair_bucket(ea.type, eb.type);
#pragma unroll
                    for (int q = 0; q < kPairBuckets; q++) acc[q] += bk == q ? val : (T)0;
                }
            }
#pragma unroll
            for (int b = 0; b < kPairBuckets; b++) row[kRadial + b * kTS + lane] = acc[b];
            __syncwarp();
        }
    }
}

}  // namespace ani
