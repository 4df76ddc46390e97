// Forward kernel for batches of larger molecules (mean size above what the molecule-per-warp kernel
// takes; BASELINE's 64-256-atom molecules).
//
// Same decomposition as featurize_mol_kernel -- a CTA is one warp, a unit of work is a ROUND of up to
// four central atoms of one molecule, and passes T, B and C (group table, triplet factors with
// lane = slot over the groups of ALL central atoms of the round, contraction with lane = (theta,
// shift)) are the very same code, ani_featurize_round_passes.inl -- but the molecule does not fit the lanes,
// so the scan differs:
//   A. the molecule is read from global memory 32 candidates at a time, once per round; every lane
//      tests its candidate against the (up to) four central atoms, whose coordinates all lanes hold.
//      Radial neighbours go to the central atom's radial list in arrival order with their element,
//      angular neighbours to its angular list (32 at most);
//   S. each angular list is put into element order by one ballot sort (lane = entry), which is what
//      pass T needs; the per-element counts fall out of the same ballots;
//   R. radial features of the whole round, lane = (central atom, pair of shifts): every lane walks
//      the radial list of its central atom and adds to the sum of the neighbour's element.
// A central atom with more than 32 angular or 64 radial neighbours goes through the streaming
// routine of ani_featurize.cuh.  A CTA takes the rounds r, r + R0, r + 2 R0, ... of its molecule
// (R0 rounds per molecule in the grid, chosen by the host from the mean molecule size), so molecules
// of any size are covered.  Nothing is accumulated with atomics; rows need no zero fill by the caller.
//
// Computes what featurize_cpu of the reference computes (gpu_featurizer/kernel_cpu.cpp:406-537).
#pragma once

#include "ani_common.cuh"
#include "ani_device_math.cuh"
#include "ani_featurize.cuh"
#include "ani_featurize_mol.cuh"

namespace ani {

constexpr int kLargeCapR = 64;   // radial neighbours kept per central atom
constexpr int kLargeCapA = 32;   // angular neighbours kept per central atom (one ballot sort covers 32 entries)

template <typename T> struct LargeFwdWarpShared {
    MolAngularShared<T, kLargeCapA, kLargeCapR> ang;   // its radial lists are in arrival order
    unsigned char rad_t[kMolCentrals][kLargeCapR];   // element of that neighbour
    unsigned char ang_t[kMolCentrals * kLargeCapA];    // element of each angular neighbour before the sort
    int cnt_r[kMolCentrals];
};

template <typename T>
__global__ void __launch_bounds__(kWarp, sizeof(T) == 4 ? 32 : 1)
    featurize_large_kernel(const T* __restrict__ xs, const T* __restrict__ ys, const T* __restrict__ zs,
                           const int* __restrict__ types, const int* __restrict__ mol_offsets,
                           const int* __restrict__ mol_counts, int n_mols, int n_atoms, int rounds_in_grid,
                           const int* __restrict__ scatter, T* out_h, T* out_c, T* out_n, T* out_o,
                           int acs0, int acs1, int acs2, int acs3)
{
    __shared__ LargeFwdWarpShared<T> ws;
    using Granule = Vec4<float>;
    constexpr int kPerGranule = 16 / (int)sizeof(T);
    const int lane = lane_id();

    // round-major grid, as in featurize_mol_kernel: the first rounds of all molecules start first
    const int round0 = blockIdx.x / n_mols, m = blockIdx.x - round0 * n_mols;
    MolRange mol;
    if (!load_molecule(mol_offsets, mol_counts, m, n_atoms, &mol)) return;
    const int n = mol.n, base = mol.base;
    const int n_rounds = (n + kMolCentrals - 1) / kMolCentrals;

    for (int round = round0; round < n_rounds; round += rounds_in_grid) {
        // round r takes the central atoms r, r + R, r + 2 R, r + 3 R (R = rounds of the molecule)
        const int G = (n - round + n_rounds - 1) / n_rounds;
        __syncwarp();   // the previous round's readers are done
        if (lane == 0) {
            ws.ang.ang_u[0] = Vec4<T>{(T)1, (T)0, (T)0, (T)1};
            ws.ang.ang_fc[0] = (T)0;
        }
        if (lane < kMolCentrals * kTypes) ws.ang.cnt_a[lane] = 0;

        // ---- the central atoms: coordinates to all lanes, rows, zero fill of the angular blocks ----
        T xi[kMolCentrals], yi[kMolCentrals], zi[kMolCentrals];
        int ci[kMolCentrals];
        unsigned skip = 0;   // central atoms that are refused or finished by the streaming routine
#pragma unroll
        for (int g = 0; g < kMolCentrals; g++) {
            ci[g] = g < G ? round + g * n_rounds : -1;
            const int gi = base + (g < G ? ci[g] : 0);
            xi[g] = xs[gi]; yi[g] = ys[gi]; zi[g] = zs[gi];
            if (g < G) {
                const int ti = checked_type(types[gi]);
                const int srow = scatter[gi];
                const int cap = ti == 0 ? acs0 : (ti == 1 ? acs1 : (ti == 2 ? acs2 : acs3));
                if (srow < 0 || srow >= cap) {
                    if (lane == 0) report(ANI_ERR_BAD_INDEX);
                    skip |= 1u << g;
                } else {
                    T* row = element_buffer<T>(ti, out_h, out_c, out_n, out_o) + (size_t)srow * kTotal;
                    if (lane == 0) ws.ang.row[g] = row;
                    Granule* zero = reinterpret_cast<Granule*>(row + kRadial);
                    constexpr int kGranules = kAngular / kPerGranule;
#pragma unroll
                    for (int i = 0; i < (kGranules + kWarp - 1) / kWarp; i++)
                        if (i * kWarp + lane < kGranules) zero[i * kWarp + lane] = Granule{0.f, 0.f, 0.f, 0.f};
                }
            } else {
                skip |= 1u << g;
            }
        }

        // ---- A: scan, 32 candidates at a time against all central atoms of the round ----
        int cA[kMolCentrals] = {0, 0, 0, 0}, cR[kMolCentrals] = {0, 0, 0, 0};
        T qx, qy, qz;   // the next 32 candidates are requested before this chunk's arithmetic
        int qt;
        {
            const int gj = base + (lane < n ? lane : 0);
            qx = xs[gj]; qy = ys[gj]; qz = zs[gj];
            qt = types[gj];
        }
        for (int j0 = 0; j0 < n; j0 += kWarp) {
            const int j = j0 + lane;
            const bool live = j < n;
            const T px = qx, py = qy, pz = qz;
            const int tj = checked_type(qt);
            if (j0 + kWarp < n) {
                const int gj = base + (j + kWarp < n ? j + kWarp : 0);
                qx = xs[gj]; qy = ys[gj]; qz = zs[gj];
                qt = types[gj];
            }
#pragma unroll
            for (int g = 0; g < kMolCentrals; g++) {
                if ((skip >> g) & 1u) continue;   // warp-uniform
                const T dx = xi[g] - px, dy = yi[g] - py, dz = zi[g] - pz;
                T r, inv;
                length_and_inverse(dx * dx + dy * dy + dz * dz, &r, &inv);
                const bool in_rad = live && j != ci[g] && r < (T)kR_Rc;
                const bool in_ang = in_rad && r < (T)kA_Rc;
                const unsigned mR = __ballot_sync(kFull, in_rad);
                if (mR == 0) continue;
                const unsigned mA = __ballot_sync(kFull, in_ang);
                if (in_rad) {
                    const int pos = cR[g] + __popc(mR & lanemask_lt());
                    if (pos < kLargeCapR) {
                        ws.ang.rad[g][pos] = Vec2<T>{r, cutoff_value<T>(r, (T)kR_Rc)};
                        ws.rad_t[g][pos] = (unsigned char)tj;
                    }
                }
                if (in_ang) {
                    const int pos = cA[g] + __popc(mA & lanemask_lt());
                    if (pos < kLargeCapA) {
                        const int p = g * kLargeCapA + pos;
                        ws.ang.ang_u[p] = Vec4<T>{dx * inv, dy * inv, dz * inv, r};
                        ws.ang.ang_fc[p] = cutoff_value<T>(r, (T)kA_Rc);
                        ws.ang_t[p] = (unsigned char)tj;
                    }
                }
                cR[g] += __popc(mR);
                cA[g] += __popc(mA);
            }
        }
        __syncwarp();

        // ---- S: each angular list into element order; denser neighbourhoods stream ----
#pragma unroll
        for (int g = 0; g < kMolCentrals; g++) {
            if ((skip >> g) & 1u) continue;
            if (cA[g] > kLargeCapA || cR[g] > kLargeCapR) {
                featurize_atom_streaming<T>(xs, ys, zs, types, base, n, ci[g], ws.ang.row[g]);
                skip |= 1u << g;
                __syncwarp();
                continue;
            }
            const bool have = lane < cA[g];
            const int p = g * kLargeCapA + (have ? lane : 0);
            const Vec4<T> u = ws.ang.ang_u[p];
            const T fc = ws.ang.ang_fc[p];
            const int t = have ? ws.ang_t[p] : kTypes;
            const unsigned m0 = __ballot_sync(kFull, t == 0), m1 = __ballot_sync(kFull, t == 1),
                           m2 = __ballot_sync(kFull, t == 2), m3 = __ballot_sync(kFull, t == 3);
            const int c0 = __popc(m0), c1 = __popc(m1), c2 = __popc(m2);
            const unsigned mine = t == 0 ? m0 : (t == 1 ? m1 : (t == 2 ? m2 : m3));
            const int start = t == 0 ? 0 : (t == 1 ? c0 : (t == 2 ? c0 + c1 : c0 + c1 + c2));
            __syncwarp();   // every entry has been read
            if (have) {
                const int q = g * kLargeCapA + start + __popc(mine & lanemask_lt());
                ws.ang.ang_u[q] = u;
                ws.ang.ang_fc[q] = fc;
            }
            if (lane == 0)
                *reinterpret_cast<int4*>(&ws.ang.cnt_a[g * kTypes]) = make_int4(c0, c1, c2, __popc(m3));
        }
        if (lane < kMolCentrals) ws.cnt_r[lane] = 0;
        __syncwarp();
#pragma unroll
        for (int g = 0; g < kMolCentrals; g++)
            if (lane == 0 && !((skip >> g) & 1u)) ws.cnt_r[g] = cR[g];
        __syncwarp();

        // ---- R: radial features of the round, lane = (central atom, pair of shifts) ----
        {
            const int g = lane >> 3, sp = lane & 7;
            const T sh0 = (T)c_tab.R_Rs[2 * sp], sh1 = (T)c_tab.R_Rs[2 * sp + 1];
            const int cnt = ws.cnt_r[g];
            Pair<T> acc[kTypes];
#pragma unroll
            for (int t = 0; t < kTypes; t++) acc[t] = Pair<T>{(T)0, (T)0};
            for (int p = 0; p < cnt; p++) {
                const Vec2<T> e = ws.ang.rad[g][p];
                const int t = ws.rad_t[g][p];
                const Pair<T> d{e.x - sh0, e.x - sh1};
                const Pair<T> d2 = pmul(d, d);
                const Pair<T> v{Num<T>::exp_neg((T)kR_eta, d2.x) * e.y, Num<T>::exp_neg((T)kR_eta, d2.y) * e.y};
#pragma unroll
                for (int k = 0; k < kTypes; k++) {
                    acc[k].x += t == k ? v.x : (T)0;
                    acc[k].y += t == k ? v.y : (T)0;
                }
            }
            if (!((skip >> g) & 1u)) {
                T* row = ws.ang.row[g];
#pragma unroll
                for (int t = 0; t < kTypes; t++)
                    *reinterpret_cast<Vec2<T>*>(row + t * kNumRs + 2 * sp) = Vec2<T>{acc[t].x, acc[t].y};
            }
        }
        __syncwarp();

        constexpr int kRoundCapA = kLargeCapA;
#include "ani_featurize_round_passes.inl"
    }
}

}  // namespace ani
