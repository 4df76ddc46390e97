// Coordinate-gradient kernel for batches of small molecules (at most 32 atoms each).
//
// One CTA per molecule, NW warps.  The central atoms of the molecule, in element order (see
// load_sorted_molecule), are dealt to the warps in turn; a warp walks its share in ROUNDS of three
// atoms and keeps the molecule in registers, lane = atom.  Per round:
//   - the 384 upstream values of each of its central atoms are copied global -> shared memory
//     with asynchronous 16-byte copies (cp.async), all requested at the start of the round, so
//     the copies run under the arithmetic and cost three instructions per lane and row;
//   - A. per central atom c: one distance per lane; a lane whose atom j is within R_Rc contracts
//     the 16 upstream values of radial block type(j) with the radial derivatives and WRITES the
//     force on j into the molecule's force table part[c][j]; neighbours within A_Rc are
//     appended to the warp's neighbour list;
//   - B. when the list is full (or the round is in), the neighbour pairs of ALL central atoms in
//     the list are walked together in circulant order: the neighbours of a central atom with k
//     neighbours occupy k consecutive lanes, lane a handles the pair (a, a + d mod k) for
//     d = 1 .. k/2, keeps the force on a in registers and hands the force on b to its owner
//     with one shuffle.  Spare lanes run further offsets d at the same time;
//   - the lanes then add their neighbour's force to part[c][a].
// After one __syncthreads the molecule's gradient is column sum minus row sum of the table
// (every term depends on coordinate differences only, so the central atom gets minus what it
// handed out): each output value is written once, nothing is accumulated with atomics, the
// outputs need no zero fill and the result is bit-reproducible.
//
// A molecule with more than 32 atoms met by this kernel goes through the streaming routines
// (zero fill by its own CTA, then global atomics, all inside the CTA).
//
// Computes what featurize_grad_cpu of the reference computes
// (gpu_featurizer/kernel_cpu.cpp:217-366).
#pragma once

#include "ani_common.cuh"
#include "ani_featurize_mol.cuh"
#include "ani_grad.cuh"

namespace ani {

#ifndef ANI_MOL_GRAD_CLASSES
#define ANI_MOL_GRAD_CLASSES 1
#endif
constexpr int kMolGradClasses = ANI_MOL_GRAD_CLASSES;   // size classes of molecules (1 or 3), in the order in which their CTAs start
constexpr int kMolGradPitch = kMolMaxAtoms + 1;   // odd: rows and columns of the force table are both conflict-free

__device__ __forceinline__ void cp_async16(void* smem_dst, const void* gmem_src)
{
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(s), "l"(gmem_src) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait()
{
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// Central atoms per round = upstream rows a warp holds in shared memory.
template <typename T> struct MolGradCfg {
    static constexpr int kRowBufs = 3;
};

template <typename T> struct alignas(16) MolGradNeighbor {
    Vec4<T> u;         // (x_c - x_j) / r, r
    T inv_r, fc, dfc;  // 1 / r, f_C(r, A_Rc) and its derivative
    int info;          // element | lane of j << 2 | first list entry of its central atom << 7 |
                       // neighbours of that central atom << 12 | row buffer << 18 | lane of the central atom << 20
};

template <typename T> struct MolGradWarpShared {
    alignas(16) T g[MolGradCfg<T>::kRowBufs][kGradRowWords];   // upstream rows, blocks of 32 at stride 36
    MolGradNeighbor<T> nb[kWarp];
    MolSortShared sort;
};

template <typename T, int NW> constexpr size_t mol_grad_smem_bytes()
{
    return NW * sizeof(MolGradWarpShared<T>) + 3 * kMolMaxAtoms * kMolGradPitch * sizeof(T);
}

// Bucket of the element pair (ta, tb), four bits per entry of the 4 x 4 table.
constexpr unsigned long long kBucketLut =
    0x0ull | (0x1ull << 4) | (0x2ull << 8) | (0x3ull << 12) | (0x1ull << 16) | (0x4ull << 20) | (0x5ull << 24) |
    (0x6ull << 28) | (0x2ull << 32) | (0x5ull << 36) | (0x7ull << 40) | (0x8ull << 44) | (0x3ull << 48) |
    (0x6ull << 52) | (0x8ull << 56) | (0x9ull << 60);
__device__ __forceinline__ int bucket_of(int ta, int tb) { return (int)(kBucketLut >> (4 * (ta * kTypes + tb))) & 15; }

// Radial part of the gradient of one central atom of a LARGE molecule, with global atomics
// (the angular part is grad_atom_streaming of ani_grad.cuh).  g = upstream row in shared memory.
template <typename T>
__device__ __noinline__ void grad_atom_streaming_radial(const T* __restrict__ xs, const T* __restrict__ ys,
                                                        const T* __restrict__ zs, const int* __restrict__ types,
                                                        int base, int n, int i, const T* g, T* gx, T* gy, T* gz)
{
    const int lane = lane_id();
    const T xi = xs[base + i], yi = ys[base + i], zi = zs[base + i];
    T fix = (T)0, fiy = (T)0, fiz = (T)0;
    for (int j0 = 0; j0 < n; j0 += kWarp) {
        const int j = j0 + lane;
        if (j < n && j != i) {
            const T dx = xi - xs[base + j], dy = yi - ys[base + j], dz = zi - zs[base + j];
            T r, inv;
            length_and_inverse(dx * dx + dy * dy + dz * dz, &r, &inv);
            if (r < (T)kR_Rc) {
                T fc, dfc;
                cutoff<T>(r, (T)kR_Rc, &fc, &dfc);
                const T d = radial_vjp_dev<T>(r, fc, dfc, g + (types[base + j] & 3) * kNumRs);
                const T fx = d * dx * inv, fy = d * dy * inv, fz = d * dz * inv;
                fix += fx; fiy += fy; fiz += fz;
                atomicAdd(&gx[base + j], -fx);
                atomicAdd(&gy[base + j], -fy);
                atomicAdd(&gz[base + j], -fz);
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
        atomicAdd(&gx[base + i], fix);
        atomicAdd(&gy[base + i], fiy);
        atomicAdd(&gz[base + i], fiz);
    }
}

template <typename T, int NW>
__global__ void __launch_bounds__(NW* kWarp, sizeof(T) == 4 ? 20 / NW : 12 / NW)
    featurize_grad_mol_kernel(const T* __restrict__ xs, const T* __restrict__ ys, const T* __restrict__ zs,
                              const int* __restrict__ types, const int* __restrict__ mol_offsets,
                              const int* __restrict__ mol_counts, int n_mols, int n_atoms,
                              const int* __restrict__ scatter, const T* __restrict__ gh,
                              const T* __restrict__ gc, const T* __restrict__ gn, const T* __restrict__ go,
                              T* gx, T* gy, T* gz, int acs0, int acs1, int acs2, int acs3)
{
    constexpr int GR = MolGradCfg<T>::kRowBufs;   // central atoms per round
    extern __shared__ __align__(128) unsigned char smem_raw[];
    using WarpShared = MolGradWarpShared<T>;
    const int lane = lane_id(), warp = warp_id();
    WarpShared& ws = reinterpret_cast<WarpShared*>(smem_raw)[warp];
    T* part = reinterpret_cast<T*>(smem_raw + NW * sizeof(WarpShared));
    auto part_at = [part](int plane, int c, int j) -> T& {
        return part[(plane * kMolMaxAtoms + c) * kMolGradPitch + j];
    };

    // The grid has kMolGradClasses CTAs per molecule, class-major.  With 3 classes: first one CTA for
    // every molecule, of which only those of the largest molecules work (the others leave after one
    // load), then the same for the middle sizes, then for the small ones; CTAs start in index order, so
    // the expensive molecules start first and the cheap ones fill the SMs behind them.  Measured on
    // 1024-molecule batches: a kernel running alone ends 10 % sooner (shorter tail), but with several
    // batches in flight the extra CTAs cost 5 % of the throughput, so the default is one class.
    for (int item = blockIdx.x; item < n_mols * kMolGradClasses; item += gridDim.x) {
        const int cls = item / n_mols, m = item - cls * n_mols;
        MolRange mol;
        if (!load_molecule(mol_offsets, mol_counts, m, n_atoms, &mol)) continue;
        const int n = mol.n, base = mol.base;
        if (kMolGradClasses > 1 && cls != (n > 20 ? 0 : (n > 12 ? 1 : 2))) continue;

        if (n > kMolMaxAtoms) {   // a large molecule in a batch of small ones
            for (int j = threadIdx.x; j < n; j += NW * kWarp) {
                gx[base + j] = (T)0;
                gy[base + j] = (T)0;
                gz[base + j] = (T)0;
            }
            __syncthreads();
            for (int i = warp; i < n; i += NW) {
                const int gi = base + i;
                const int ti = checked_type(types[gi]);
                const int srow = scatter[gi];
                const int cap = ti == 0 ? acs0 : (ti == 1 ? acs1 : (ti == 2 ? acs2 : acs3));
                if (srow < 0 || srow >= cap) {
                    if (lane == 0) report(ANI_ERR_BAD_INDEX);
                    continue;
                }
                const T* grow = (ti == 0 ? gh : (ti == 1 ? gc : (ti == 2 ? gn : go))) + (size_t)srow * kTotal;
                T* g = ws.g[0];
                g[lane] = grow[lane];
                g[32 + lane] = grow[32 + lane];
                for (int bk = 0; bk < kPairBuckets; bk++)
                    g[kRadial + bk * kGradBucketStride + lane] = grow[kRadial + bk * kTS + lane];
                __syncwarp();
                grad_atom_streaming_radial<T>(xs, ys, zs, types, base, n, i, g, gx, gy, gz);
                grad_atom_streaming<T>(xs, ys, zs, types, base, n, i, g, gx, gy, gz);
                __syncwarp();
            }
            continue;
        }

        // every warp needs the sort for the last step, also one without a round of its own
        MolLanes<T> ml;
        load_sorted_molecule<T>(xs, ys, zs, types, scatter, base, n, &ws.sort, &ml);

        // Warp w takes the central atoms w, w + NW, w + 2 NW, ... (element order) and walks them in rounds
        // of GR: every warp gets the same number of atoms (no idle warps) AND the same mix of light and heavy
        // ones -- the cost of a central atom grows with the square of its neighbour count, and consecutive
        // atoms are of one element.  Which warp starts with atom 0 rotates with the molecule: a warp's
        // scheduler is fixed by its index, and the last warps have one atom less.
        const int w0 = (warp + m) % NW;
        const int K = w0 < n ? (n - w0 + NW - 1) / NW : 0;   // central atoms of this warp
        for (int k_first = 0; k_first < K; k_first += GR) {
            const int G = min(GR, K - k_first);
            // ---- upstream rows of the round: one commit group per row slot ----
#pragma unroll
            for (int g = 0; g < GR; g++) {
                const int c = min(w0 + (k_first + g) * NW, n - 1);
                const int ti = __shfl_sync(kFull, ml.type, c), sr = ws.sort.srow[c];
                const int cap = ti == 0 ? acs0 : (ti == 1 ? acs1 : (ti == 2 ? acs2 : acs3));
                if (g < G && sr >= 0 && sr < cap) {
                    const T* grow = (ti == 0 ? gh : (ti == 1 ? gc : (ti == 2 ? gn : go))) + (size_t)sr * kTotal;
                    T* dst = ws.g[g];
                    constexpr int V = 16 / (int)sizeof(T);   // values per 16-byte copy
#pragma unroll
                    for (int s = 0; s < kTotal / V / kWarp; s++) {
                        const int v = (lane + s * kWarp) * V;
                        const int d = v < kRadial
                                          ? v
                                          : kRadial + ((v - kRadial) >> 5) * kGradBucketStride + ((v - kRadial) & 31);
                        cp_async16(dst + d, grow + v);
                    }
                }
                cp_async_commit();
            }

            int g = 0;
            while (g < G) {
                // ---- A: scan central atoms into the neighbour list until it is full ----
                int used = 0, max_half = 0, taken = 0;
                while (g < G) {
                    const int c = w0 + (k_first + g) * NW;
                    const T xi = __shfl_sync(kFull, ml.x, c), yi = __shfl_sync(kFull, ml.y, c),
                            zi = __shfl_sync(kFull, ml.z, c);
                    const int ti = __shfl_sync(kFull, ml.type, c), sr = ws.sort.srow[c];
                    const int cap = ti == 0 ? acs0 : (ti == 1 ? acs1 : (ti == 2 ? acs2 : acs3));
                    const bool ok = sr >= 0 && sr < cap;
                    const T dx = xi - ml.x, dy = yi - ml.y, dz = zi - ml.z;
                    T r, inv;
                    length_and_inverse(dx * dx + dy * dy + dz * dz, &r, &inv);
                    const bool in_rad = ok && lane < n && lane != c && r < (T)kR_Rc;
                    const bool in_ang = in_rad && r < (T)kA_Rc;
                    const unsigned mA = __ballot_sync(kFull, in_ang);
                    const int nA = __popc(mA);
                    if (taken > 0 && used + nA > kWarp) break;   // this central atom opens the next pass

                    // row slot g has landed when at most GR - 1 - g younger groups are pending
                    if (g == 0) cp_async_wait<GR - 1>();
                    else if (g == 1) cp_async_wait<(GR > 2 ? GR - 2 : 0)>();
                    else if (g == 2) cp_async_wait<(GR > 3 ? GR - 3 : 0)>();
                    else cp_async_wait<0>();
                    __syncwarp();
                    if (!ok && lane == 0) report(ANI_ERR_BAD_INDEX);
                    const T* grow = ws.g[g];
                    const T ux = dx * inv, uy = dy * inv, uz = dz * inv;
                    T fx = (T)0, fy = (T)0, fz = (T)0;
                    if (in_rad) {
                        T fc, dfc;
                        cutoff<T>(r, (T)kR_Rc, &fc, &dfc);
                        T w[kNumRs];
#pragma unroll
                        for (int q = 0; q < kNumRs; q += 4) load4(grow + ml.type * kNumRs + q, w + q);
                        const T d = radial_vjp_dev<T>(r, fc, dfc, w);
                        fx = d * ux; fy = d * uy; fz = d * uz;
                    }
                    if (lane < n) {   // force on atom j from the radial terms of central atom c (0 out of range)
                        part_at(0, c, lane) = -fx;
                        part_at(1, c, lane) = -fy;
                        part_at(2, c, lane) = -fz;
                    }
                    if (in_ang) {
                        MolGradNeighbor<T> e;
                        e.u = Vec4<T>{ux, uy, uz, r};
                        e.inv_r = inv;
                        cutoff<T>(r, (T)kA_Rc, &e.fc, &e.dfc);
                        e.info = ml.type | (lane << 2) | (used << 7) | (nA << 12) | (g << 18) | (c << 20);
                        ws.nb[used + __popc(mA & lanemask_lt())] = e;
                    }
                    used += nA;
                    taken++;
                    max_half = max(max_half, nA >> 1);
                    g++;
                }
                __syncwarp();

                // ---- B: neighbour pairs of every central atom in the list, circulant order ----
                if (max_half > 0) {
#include "ani_grad_pair_pass.inl"
                    if (lane < used) {
                        const int cen = (ea.info >> 20) & 31, at = (ea.info >> 2) & 31;
                        part_at(0, cen, at) += fax;
                        part_at(1, cen, at) += fay;
                        part_at(2, cen, at) += faz;
                    }
                }
                __syncwarp();
            }
            cp_async_wait<0>();   // row slots of a short round are empty groups; nothing may stay pending
        }
        __syncthreads();
        // gradient of atom j = what the central atoms handed to j (column j) - what j handed out (row j)
        for (int plane = warp; plane < 3; plane += NW) {
            if (lane < n) {
                T col = (T)0, rw = (T)0;
                for (int c = 0; c < n; c++) col += part_at(plane, c, lane);
                for (int j = 0; j < n; j++) rw += part_at(plane, lane, j);
                T* dst = plane == 0 ? gx : (plane == 1 ? gy : gz);
                dst[base + ws.sort.src[lane]] = col - rw;
            }
        }
        __syncthreads();   // the table is reused by the next molecule of this CTA
    }
}

}  // namespace ani
