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
//      compacted (in scan order) into the warp's angular list;
//   B. walks the unordered neighbour pairs in CIRCULANT order.  With n angular neighbours,
//      lane (g, a) -- g = lane / n, a = lane % n -- owns neighbour a and, in a pass, handles the
//      pair (a, (a + d) mod n) for offset d = d0 + g.  Within a group every a and every
//      b = a + d is distinct, so the force on a is accumulated in the lane's own registers and
//      the force on b is handed to its owner with one shuffle: no atomics, no pair table.
//      Offsets 1 .. n/2 cover every unordered pair once (for even n, offset n/2 only for
//      a < n/2).  Per pair the 32 upstream values of block (type a, type b) are contracted
//      into dL/dcos, dL/dr_a, dL/dr_b, from which the two force vectors follow;
//   C. sums the per-group partial forces of each neighbour and adds them to the output; the
//      central atom gets minus the total, since every term depends on coordinate differences.
// Contributions of different central atoms to the same atom meet in the output arrays through
// floating-point atomic adds, so the outputs must be zero before the kernel starts and the
// summation order (hence the last bits) may differ between runs.
#pragma once

#include "ani_common.cuh"
#include "ani_device_math.cuh"

namespace ani {

constexpr int kGradBucketStride = 36;  // upstream values of one type pair, padded against bank conflicts
constexpr int kGradRowWords = kRadial + kPairBuckets * kGradBucketStride;
constexpr int kGradMaxNeighbors = 32;  // angular neighbours handled by the circulant passes

template <typename T> struct GradNeighbor {   // one angular neighbour
    Vec4<T> u;   // (x_i - x_j) / r_ij, r_ij
    T fc, dfc;   // f_C(r_ij, A_Rc) and its derivative
    int type;
    int atom;    // batch index of j
};

template <typename T> struct GradWarpShared {
    alignas(16) T g[kGradRowWords];  // upstream row: radial [0,64), then 10 blocks of 32 at stride 36
    GradNeighbor<T> nb[kGradMaxNeighbors];
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
                    angular_vjp_dev<T>(c, s2, rj, rk, fj, dfj, fk, dfk,
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

#ifndef ANI_GRAD_MIN_CTAS
#define ANI_GRAD_MIN_CTAS 8
#endif

template <typename T, int NW>
__global__ void __launch_bounds__(NW* kWarp, sizeof(T) == 4 ? ANI_GRAD_MIN_CTAS * 4 / NW : 1)
    featurize_grad_kernel(const T* __restrict__ xs, const T* __restrict__ ys,
                          const T* __restrict__ zs, const int* __restrict__ types,
                          const int* __restrict__ mol_offsets, const int* __restrict__ mol_counts,
                          int n_mols, int n_atoms, int slot_shift, const int* __restrict__ scatter,
                          const T* __restrict__ gh, const T* __restrict__ gc,
                          const T* __restrict__ gn, const T* __restrict__ go, T* gx, T* gy, T* gz,
                          int acs0, int acs1, int acs2, int acs3)
{
    extern __shared__ __align__(128) unsigned char smem_raw[];
    using WarpShared = GradWarpShared<T>;
    const int lane = lane_id(), warp = warp_id();
    WarpShared& ws = reinterpret_cast<WarpShared*>(smem_raw)[warp];

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
            const T* grow = (ti == 0 ? gh : (ti == 1 ? gc : (ti == 2 ? gn : go))) + (size_t)srow * kTotal;
            // upstream row -> shared memory (12 coalesced loads of 32 values)
            {
                T v[2 + kPairBuckets];
                v[0] = grow[lane];
                v[1] = grow[32 + lane];
#pragma unroll
                for (int bk = 0; bk < kPairBuckets; bk++) v[2 + bk] = grow[kRadial + bk * kTS + lane];
                ws.g[lane] = v[0];
                ws.g[32 + lane] = v[1];
#pragma unroll
                for (int bk = 0; bk < kPairBuckets; bk++)
                    ws.g[kRadial + bk * kGradBucketStride + lane] = v[2 + bk];
            }
            __syncwarp();
            T fix = (T)0, fiy = (T)0, fiz = (T)0;  // this lane's share of the force on atom i

            // ---- A: neighbour scan + radial part, lane = j ----
            int n_ang = 0;
            for (int j0 = 0; j0 < n; j0 += kWarp) {
                const int j = j0 + lane;
                const bool live = j < n;
                const int gj = base + (live ? j : 0);
                if (j0 > 0) {   // chunk 0 was requested above
                    px = xs[gj]; py = ys[gj]; pz = zs[gj];
                    pt = types[gj];
                }
                const T dx = xi - px, dy = yi - py, dz = zi - pz;
                const int tj = live ? checked_type(pt) : 0;
                T r, inv;
                length_and_inverse(dx * dx + dy * dy + dz * dz, &r, &inv);
                const bool in_rad = live && j != i && r < (T)kR_Rc;
                const bool in_ang = in_rad && r < (T)kA_Rc;
                const T ux = dx * inv, uy = dy * inv, uz = dz * inv;
                if (in_rad) {
                    T fc, dfc;
                    cutoff<T>(r, (T)kR_Rc, &fc, &dfc);
                    const T d = radial_vjp_dev<T>(r, fc, dfc, ws.g + tj * kNumRs);
                    const T fx = d * ux, fy = d * uy, fz = d * uz;
                    fix += fx; fiy += fy; fiz += fz;
                    atomicAdd(&gx[gj], -fx);
                    atomicAdd(&gy[gj], -fy);
                    atomicAdd(&gz[gj], -fz);
                }
                const unsigned mA = __ballot_sync(kFull, in_ang);
                if (in_ang) {
                    const int pos = n_ang + __popc(mA & lanemask_lt());
                    if (pos < kGradMaxNeighbors) {
                        GradNeighbor<T> e;
                        e.u = Vec4<T>{ux, uy, uz, r};
                        cutoff<T>(r, (T)kA_Rc, &e.fc, &e.dfc);
                        e.type = tj;
                        e.atom = gj;
                        ws.nb[pos] = e;
                    }
                }
                n_ang += __popc(mA);
            }
            __syncwarp();

            if (n_ang > kGradMaxNeighbors) {
                grad_atom_streaming<T>(xs, ys, zs, types, base, n, i, ws.g, gx, gy, gz);
            } else if (n_ang >= 2) {
                // ---- B: angular part, circulant pair order ----
                const int na = n_ang;
                const int groups = min(kWarp / na, 4);       // offsets handled per pass
                const int grp = lane / na;                    // 0 .. (32 / na)
                const int a = lane - grp * na;
                const bool owner = grp < groups;
                const GradNeighbor<T> ea = ws.nb[owner ? a : 0];
                T fax = (T)0, fay = (T)0, faz = (T)0;         // force on neighbour a (this group's share)
                const int half = na >> 1;
                const bool even = (na & 1) == 0;
                for (int d0 = 1; d0 <= half; d0 += groups) {
                    const int d = d0 + grp;
                    const bool valid = owner && d <= half && !(even && d == half && a >= half);
                    int b = a + d;
                    if (b >= na) b -= na;
                    T gbx = (T)0, gby = (T)0, gbz = (T)0;
                    if (valid) {
                        const GradNeighbor<T> eb = ws.nb[b];
                        T c = ea.u.x * eb.u.x + ea.u.y * eb.u.y + ea.u.z * eb.u.z;
                        c = Num<T>::max_((T)-1, Num<T>::min_((T)1, c));
                        const T s2 = sin2_from_cross<T>(ea.u.x, ea.u.y, ea.u.z, eb.u.x, eb.u.y, eb.u.z);
                        T gl[kTS];
                        const T* gsrc = ws.g + kRadial + pair_bucket(ea.type, eb.type) * kGradBucketStride;
#pragma unroll
                        for (int q = 0; q < kTS; q += 4) load4(gsrc + q, gl + q);
                        T dc, dra, drb;
                        angular_vjp_dev<T>(c, s2, ea.u.w, eb.u.w, ea.fc, ea.dfc, eb.fc, eb.dfc, gl, &dc,
                                          &dra, &drb);
                        T ra_inv, rb_inv, unused;
                        length_and_inverse(ea.u.w * ea.u.w, &unused, &ra_inv);
                        length_and_inverse(eb.u.w * eb.u.w, &unused, &rb_inv);
                        const T aa = -dc * ra_inv, ba = c * dc * ra_inv - dra;
                        const T ab = -dc * rb_inv, bb = c * dc * rb_inv - drb;
                        fax += aa * eb.u.x + ba * ea.u.x;
                        fay += aa * eb.u.y + ba * ea.u.y;
                        faz += aa * eb.u.z + ba * ea.u.z;
                        gbx = ab * ea.u.x + bb * eb.u.x;
                        gby = ab * ea.u.y + bb * eb.u.y;
                        gbz = ab * ea.u.z + bb * eb.u.z;
                    }
                    // hand the force on b to its owner in the same group: lane (grp, x) takes it
                    // from lane (grp, (x - d) mod na)
                    int src = a - d;
                    if (src < 0) src += na;
                    if (src < 0) src += na;   // d can exceed na only on lanes that are not valid
                    src = owner ? grp * na + src : lane;
                    fax += __shfl_sync(kFull, gbx, src);
                    fay += __shfl_sync(kFull, gby, src);
                    faz += __shfl_sync(kFull, gbz, src);
                }
                // ---- C: sum the groups, push the neighbour forces out ----
                for (int g = 1; g < groups; g++) {
                    const int src = lane + g * na < kWarp ? lane + g * na : lane;
                    const T ox = __shfl_sync(kFull, fax, src), oy = __shfl_sync(kFull, fay, src),
                            oz = __shfl_sync(kFull, faz, src);
                    if (lane < na) { fax += ox; fay += oy; faz += oz; }
                }
                if (lane < na) {
                    fix -= fax; fiy -= fay; fiz -= faz;
                    atomicAdd(&gx[ea.atom], fax);
                    atomicAdd(&gy[ea.atom], fay);
                    atomicAdd(&gz[ea.atom], faz);
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
