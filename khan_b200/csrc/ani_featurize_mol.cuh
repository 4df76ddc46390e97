// Forward kernel for batches of small molecules (at most 32 atoms each, the size range of the
// data sets khan trains on: its loaders drop larger molecules, data_utils.py:54,281-283).
//
// The central atoms of a molecule, in element order, are dealt to ROUNDS of at most four atoms
// (round r of R takes atoms r, r + R, ...), and a CTA is ONE WARP doing one round: a molecule has 8 CTAs (8 rounds, 32 atoms), a
// CTA whose round lies behind the end of the molecule leaves after one load.  No warp needs
// anything from another, every round gives its registers and shared memory back as soon as it
// is done, and the rounds of a large molecule spread over the SMs.  A warp keeps the whole
// molecule in registers, lane = atom:
//   0. every lane loads one atom; the atoms are ranked by element with four ballots and moved to
//      their rank by shuffles, so that lane order = element order and every neighbour list that
//      is compacted in lane order comes out sorted by element for free;
//   A. per central atom of the round (coordinates by shuffle): one distance per lane; (r, f_C)
//      of every atom of the molecule goes to a table (f_C = 0 beyond R_Rc), and the neighbours
//      within A_Rc, compacted by a ballot, to the list (unit vector, r, f_C) of this central atom;
//   R. the radial features of all central atoms of the round at once: lane = (central atom,
//      pair of radial shifts) walks the table of its central atom.  The table is in element
//      order for every central atom alike, so the loops over the four element runs are uniform
//      and the 2 x 4 sums of a lane stay in registers; four 8-byte stores per lane;
//   T. ONE table of all (central atom, element pair) groups of the round: start, size and list
//      bases of each group, every group padded to a multiple of four slots;
//   B. lane = slot, 32 slots at a time over the groups of ALL central atoms of the round (so the
//      lanes stay filled although one atom has only some 50 neighbour pairs): 8 theta factors and
//      4 radial factors of each triplet into shared memory.  A slot is decoded without a branch
//      and without a division: pairs of different elements are numbered row-major, pairs of
//      one element in circulant order (a, a + d), which is row-major in (d, a);
//   C. lane = (theta, shift): acc += A[theta][slot] * BF[shift][slot], four slots per pair of
//      16-byte loads; a 32-float block of a feature row is written when its group ends (the
//      ends inside a chunk come from one ballot).
// Nothing is accumulated with atomics and no row needs a zero fill by the caller; results do
// not depend on the launch shape.
//
// A molecule with more than 32 atoms met by this kernel (the host picks it from the MEAN
// molecule size) and a central atom with more than 24 neighbours within A_Rc go through the
// streaming routine of ani_featurize.cuh.
//
// Computes what featurize_cpu of the reference computes (gpu_featurizer/kernel_cpu.cpp:406-537).
#pragma once

#include "ani_common.cuh"
#include "ani_device_math.cuh"
#include "ani_featurize.cuh"

namespace ani {

constexpr int kMolMaxAtoms = 32;       // molecules up to this size take the fast path
constexpr int kMolCentrals = 4;        // central atoms per round
constexpr int kMolCapA = 24;           // angular neighbours kept per central atom
constexpr int kMolGroupStride = 16;    // group id = central slot * 16 + element-pair bucket
constexpr int kMolNoGroup = 0xff;      // id of the quads behind the last group
constexpr int kMolSlotsPerLane = 1;    // slots a lane evaluates per pass B (2 was measured: no gain)
constexpr int kMolChunk = kMolSlotsPerLane * kWarp;   // slots per pass B / C
constexpr int kMolChunkStride = kMolChunk + 4;        // + 4 words: keeps the 16-byte reads of pass C conflict-free
constexpr int kMolRounds = kMolMaxAtoms / kMolCentrals;   // rounds of the largest molecule of the fast path
// padded slots of one central atom: at most CapA (CapA - 1) / 2 pairs + 3 per bucket, in quads
constexpr int mol_quad_bytes(int cap_a)
{
    return ((kMolCentrals * ((cap_a * (cap_a - 1) / 2 + 3 * kPairBuckets) / 4 + 1) + 2 * (kMolChunk / 4) + 7) / 8) * 8;
}

struct alignas(16) MolGroupInfo {
    int off;         // first slot of the group (a multiple of 4)
    int cnt;         // triplets in the group
    int packed;      // list index of the first neighbour of element a | same for b << 8 | size of run b << 16 | a == b << 24
    unsigned recip;  // ceil(2^16 / size of run b): q / nb == (q * recip) >> 16 for every slot number q in use
};

// Per warp: what the element sort leaves behind for the rest of the molecule's work.
struct MolSortShared {
    alignas(16) unsigned tmask[kTypes];   // lanes of each element after the sort
    int srow[kMolMaxAtoms];               // scatter index of the atom in each lane
    unsigned char src[kMolMaxAtoms];      // index inside the molecule of the atom in each lane
};


// What the angular passes (T, B, C) of a round work on: the angular neighbour lists of the round's
// central atoms (element order inside each list), the group table, the factor chunks and the rows.
// CAPA = angular neighbours kept per central atom (at most 32: list indices are packed into 8 bits).
template <typename T, int CAPA, int CAPR> struct MolAngularShared {
    static constexpr int kCapA = CAPA;
    Vec4<T> ang_u[kMolCentrals * CAPA];   // (x_i - x_j) / r_ij and r_ij, element order, per central atom
    T ang_fc[kMolCentrals * CAPA];        // f_C(r_ij, A_Rc)
    Vec2<T> rad[kMolCentrals][CAPR];      // (r_ij, f_C(r_ij, R_Rc)) per central atom: the radial pass reads it, not T / B / C
    alignas(16) T A[kNumThetas][kMolChunkStride];
    alignas(16) T BF[kNumARs][kMolChunkStride];
    MolGroupInfo tab[kMolCentrals * kMolGroupStride];
    T* row[kMolCentrals];                     // feature row of each central atom of the round
    alignas(16) int cnt_a[kMolCentrals * kTypes];   // angular neighbours per element, per central atom
    alignas(8) unsigned char quad_gid[mol_quad_bytes(CAPA)];
};

template <typename T> struct MolFwdWarpShared {
    MolAngularShared<T, kMolCapA, kMolMaxAtoms> ang;   // its radial table: every atom j of the molecule, f_C = 0 out of range
    MolSortShared sort;
};

__device__ __forceinline__ unsigned low_lanes(int c) { return c >= 32 ? 0xffffffffu : ((1u << c) - 1u); }

// One molecule's atom per lane, moved into element order; lanes >= n hold copies of dead lanes.
// What is needed once per central atom only sits in the warp's shared memory instead.
template <typename T> struct MolLanes {
    T x, y, z;
    int type;          // 0..3 (4 on dead lanes)
};

template <typename T>
__device__ __forceinline__ void load_sorted_molecule(const T* __restrict__ xs, const T* __restrict__ ys,
                                                     const T* __restrict__ zs, const int* __restrict__ types,
                                                     const int* __restrict__ scatter, int base, int n,
                                                     MolSortShared* sh, MolLanes<T>* out)
{
    unsigned char* inv = sh->src;
    const int lane = lane_id();
    const bool live = lane < n;
    const int gj = base + (live ? lane : 0);
    const T x0 = xs[gj], y0 = ys[gj], z0 = zs[gj];
    const int s0 = scatter[gj];
    const int t0 = live ? checked_type(types[gj]) : kTypes;
    const unsigned m0 = __ballot_sync(kFull, t0 == 0), m1 = __ballot_sync(kFull, t0 == 1),
                   m2 = __ballot_sync(kFull, t0 == 2), m3 = __ballot_sync(kFull, t0 == 3);
    const int c0 = __popc(m0), c1 = __popc(m1), c2 = __popc(m2);
    const unsigned mine = t0 == 0 ? m0 : (t0 == 1 ? m1 : (t0 == 2 ? m2 : (t0 == 3 ? m3 : ~(m0 | m1 | m2 | m3))));
    const int start = t0 == 0 ? 0 : (t0 == 1 ? c0 : (t0 == 2 ? c0 + c1 : (t0 == 3 ? c0 + c1 + c2 : n)));
    const int rank = start + __popc(mine & lanemask_lt());
    __syncwarp();   // the previous molecule's readers are done
    inv[rank] = (unsigned char)lane;
    sh->srow[rank] = s0;
    if (lane == 0) {
        sh->tmask[0] = low_lanes(c0);
        sh->tmask[1] = low_lanes(c0 + c1) & ~low_lanes(c0);
        sh->tmask[2] = low_lanes(c0 + c1 + c2) & ~low_lanes(c0 + c1);
        sh->tmask[3] = low_lanes(n) & ~low_lanes(c0 + c1 + c2);
    }
    __syncwarp();
    const int src = inv[lane];
    out->x = __shfl_sync(kFull, x0, src);
    out->y = __shfl_sync(kFull, y0, src);
    out->z = __shfl_sync(kFull, z0, src);
    out->type = __shfl_sync(kFull, t0, src);
}

// Slot p of the round -> list indices (a, b) of its two neighbours.  Returns false for a
// padding slot (a and b then point at entry 0 of the list, which always holds finite values).
// Slot number q inside a group: different elements, q = ia * nb + ib; one element, q = (d - 1) * nb + a
// with b = a + d mod nb (d <= nb / 2; the last row of an even nb holds only a < nb / 2).
__device__ __forceinline__ bool decode_slot(const MolGroupInfo* tab, const unsigned char* quad_gid, int p,
                                            int* a, int* b)
{
    const int gid = quad_gid[p >> 2];
    const MolGroupInfo e = tab[gid == kMolNoGroup ? 0 : gid];
    const int q = p - e.off;
    const bool valid = gid != kMolNoGroup && q < e.cnt;
    const int nb = (e.packed >> 16) & 0xff;
    const bool same = (e.packed >> 24) != 0;
    const int hi = (int)(((unsigned)q * e.recip) >> 16);   // q / nb
    const int lo = q - hi * nb;                            // q % nb
    int wrap = lo + hi + 1;
    if (wrap >= nb) wrap -= nb;
    const int ia = same ? lo : hi, ib = same ? wrap : lo;
    *a = valid ? (e.packed & 0xff) + ia : 0;
    *b = valid ? ((e.packed >> 8) & 0xff) + ib : 0;
    return valid;
}

template <typename T>
__global__ void __launch_bounds__(kWarp, sizeof(T) == 4 ? 32 : 20)
    featurize_mol_kernel(const T* __restrict__ xs, const T* __restrict__ ys, const T* __restrict__ zs,
                         const int* __restrict__ types, const int* __restrict__ mol_offsets,
                         const int* __restrict__ mol_counts, int n_mols, int n_atoms,
                         const int* __restrict__ scatter, T* out_h, T* out_c, T* out_n, T* out_o,
                         int acs0, int acs1, int acs2, int acs3)
{
    __shared__ MolFwdWarpShared<T> ws;
    using Granule = Vec4<float>;                      // 16 bytes of zeros, whatever T is
    constexpr int kPerGranule = 16 / (int)sizeof(T);  // values in a granule
    const int lane = lane_id();

    // Round-major order of the grid: all first rounds (every molecule has one), then all second rounds, ...
    // so the work that exists starts first and is spread evenly over the SMs, and the CTAs of rounds that
    // most molecules do not have come last.
    const int round = blockIdx.x / n_mols, m = blockIdx.x - round * n_mols;
    MolRange mol;
    if (!load_molecule(mol_offsets, mol_counts, m, n_atoms, &mol)) return;
    const int n = mol.n, base = mol.base;

    if (n > kMolMaxAtoms) {   // a large molecule in a batch of small ones: its CTAs take one atom at a time
        for (int i = round; i < n; i += kMolRounds) {
            const int gi = base + i;
            const int ti = checked_type(types[gi]);
            const int srow = scatter[gi];
            const int cap = ti == 0 ? acs0 : (ti == 1 ? acs1 : (ti == 2 ? acs2 : acs3));
            if (srow < 0 || srow >= cap) {
                if (lane == 0) report(ANI_ERR_BAD_INDEX);
                continue;
            }
            featurize_atom_streaming<T>(xs, ys, zs, types, base, n, i,
                                        element_buffer<T>(ti, out_h, out_c, out_n, out_o) + (size_t)srow * kTotal);
            __syncwarp();
        }
        return;
    }
    // Round r of a molecule with R rounds takes the central atoms r, r + R, r + 2 R, r + 3 R: every round
    // gets the same mix of light and heavy atoms (atoms are in element order, and the cost of a central
    // atom grows with the square of its neighbour count), so the rounds of a molecule cost about the same.
    const int n_rounds = (n + kMolCentrals - 1) / kMolCentrals;
    if (round >= n_rounds) return;
    const int G = (n - round + n_rounds - 1) / n_rounds;

    MolLanes<T> ml;
    load_sorted_molecule<T>(xs, ys, zs, types, scatter, base, n, &ws.sort, &ml);

    // Padding slots read entry 0 of the angular list, possibly before anything was written there.
    if (lane == 0) {
        ws.ang.ang_u[0] = Vec4<T>{(T)1, (T)0, (T)0, (T)1};
        ws.ang.ang_fc[0] = (T)0;
    }
    if (lane < kMolCentrals * kTypes) ws.ang.cnt_a[lane] = 0;
    __syncwarp();

    // ---- A: scan, one central atom after another ----
    unsigned skip = 0;   // central atoms that are finished (streaming routine) or refused
    for (int g = 0; g < G; g++) {
        const int c = round + g * n_rounds;
        const T xi = __shfl_sync(kFull, ml.x, c), yi = __shfl_sync(kFull, ml.y, c), zi = __shfl_sync(kFull, ml.z, c);
        const int ti = __shfl_sync(kFull, ml.type, c);
        const int srow = ws.sort.srow[c];
        const int cap = ti == 0 ? acs0 : (ti == 1 ? acs1 : (ti == 2 ? acs2 : acs3));
        if (srow < 0 || srow >= cap) {
            if (lane == 0) report(ANI_ERR_BAD_INDEX);
            skip |= 1u << g;
            continue;
        }
        T* row = element_buffer<T>(ti, out_h, out_c, out_n, out_o) + (size_t)srow * kTotal;
        if (lane == 0) ws.ang.row[g] = row;

        const T dx = xi - ml.x, dy = yi - ml.y, dz = zi - ml.z;
        T r, inv;
        length_and_inverse(dx * dx + dy * dy + dz * dz, &r, &inv);
        const bool in_rad = lane < n && lane != c && r < (T)kR_Rc;
        const bool in_ang = in_rad && r < (T)kA_Rc;
        const unsigned mA = __ballot_sync(kFull, in_ang);
        if (__popc(mA) > kMolCapA) {   // denser than the list: the streaming routine does the whole row
            featurize_atom_streaming<T>(xs, ys, zs, types, base, n, ws.sort.src[c], row);
            skip |= 1u << g;
            __syncwarp();
            continue;
        }
        // the angular blocks start as zeros (16-byte stores: 2.5 per lane); pass C writes the blocks of
        // the element pairs that occur, after a __syncwarp, so the order of the two is fixed
        {
            Granule* zero = reinterpret_cast<Granule*>(row + kRadial);
            constexpr int kGranules = kAngular / kPerGranule;
#pragma unroll
            for (int i = 0; i < (kGranules + kWarp - 1) / kWarp; i++)
                if (i * kWarp + lane < kGranules) zero[i * kWarp + lane] = Granule{0.f, 0.f, 0.f, 0.f};
        }
        ws.ang.rad[g][lane] = Vec2<T>{r, in_rad ? cutoff_value<T>(r, (T)kR_Rc) : (T)0};
        if (in_ang) {
            const int p = g * kMolCapA + __popc(mA & lanemask_lt());
            ws.ang.ang_u[p] = Vec4<T>{dx * inv, dy * inv, dz * inv, r};
            ws.ang.ang_fc[p] = cutoff_value<T>(r, (T)kA_Rc);
        }
        if (lane < kTypes) ws.ang.cnt_a[g * kTypes + lane] = __popc(mA & ws.sort.tmask[lane]);
    }
    __syncwarp();

    // ---- R: radial features of the whole round, lane = (central atom, pair of shifts) ----
    {
        const int g = lane >> 3, sp = lane & 7;
        const Vec2<T>* list = ws.ang.rad[g];
        const T sh0 = (T)c_tab.R_Rs[2 * sp], sh1 = (T)c_tab.R_Rs[2 * sp + 1];
        const uint4 tmq = *reinterpret_cast<const uint4*>(ws.sort.tmask);
        const int run_end[kTypes] = {__popc(tmq.x), __popc(tmq.x | tmq.y), __popc(tmq.x | tmq.y | tmq.z), n};
        Pair<T> acc[kTypes];
        int p = 0;
#pragma unroll
        for (int t = 0; t < kTypes; t++) {
            acc[t] = Pair<T>{(T)0, (T)0};
            for (; p < run_end[t]; p++) {
                const Vec2<T> e = list[p];
                const Pair<T> d{e.x - sh0, e.x - sh1};
                const Pair<T> d2 = pmul(d, d);
                const Pair<T> v{Num<T>::exp_neg((T)kR_eta, d2.x), Num<T>::exp_neg((T)kR_eta, d2.y)};
                acc[t] = pfma(v, Pair<T>{e.y, e.y}, acc[t]);
            }
        }
        if (g < G && !((skip >> g) & 1u)) {
            T* row = ws.ang.row[g];
#pragma unroll
            for (int t = 0; t < kTypes; t++)
                *reinterpret_cast<Vec2<T>*>(row + t * kNumRs + 2 * sp) = Vec2<T>{acc[t].x, acc[t].y};
        }
    }

    constexpr int kRoundCapA = kMolCapA;
#include "ani_featurize_round_passes.inl"
}

}  // namespace ani
