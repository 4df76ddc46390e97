// TEST HELPER (host only).  Evaluates the per-pair / per-triplet formulas of
// khan_b200/csrc/ani_params.h -- the very header the CUDA kernels include -- in a naive
// double loop over every molecule, so that the formulas can be checked against the CPU oracle
// on a machine without a GPU.  It shares no orchestration with the kernels (no neighbour
// lists, no warps); it exists only to catch algebra mistakes in the shared math.
#include <vector>

#include "ani_params.h"

using namespace ani;

template <typename T>
static void featurize(const T* X, const T* Y, const T* Z, const int* A, const int* mo, const int* mac,
                      int n_mols, const int* si, T* const* out)
{
    for (int m = 0; m < n_mols; m++) {
        const int n = mac[m], base = mo[m];
        for (int i = 0; i < n; i++) {
            const int gi = base + i;
            T* row = out[A[gi]] + (size_t)si[gi] * kTotal;
            for (int q = 0; q < kTotal; q++) row[q] = (T)0;
            std::vector<T> ux, uy, uz, rr, fc;
            std::vector<int> tt;
            for (int j = 0; j < n; j++) {
                if (j == i) continue;
                const int gj = base + j;
                const T dx = X[gi] - X[gj], dy = Y[gi] - Y[gj], dz = Z[gi] - Z[gj];
                const T r = Num<T>::sqrt_(dx * dx + dy * dy + dz * dz);
                if (r < (T)kR_Rc) {
                    const T f = cutoff_value<T>(r, (T)kR_Rc);
                    for (int k = 0; k < kNumRs; k++) row[A[gj] * kNumRs + k] += radial_term<T>(r, f, k);
                }
                if (r < (T)kA_Rc) {
                    ux.push_back(dx / r); uy.push_back(dy / r); uz.push_back(dz / r);
                    rr.push_back(r); fc.push_back(cutoff_value<T>(r, (T)kA_Rc)); tt.push_back(A[gj]);
                }
            }
            for (size_t a = 0; a < rr.size(); a++)
                for (size_t b = a + 1; b < rr.size(); b++) {
                    T Av[kNumThetas], BF[kNumARs];
                    const T c = ux[a] * ux[b] + uy[a] * uy[b] + uz[a] * uz[b];
                    angular_factors<T>(c, (T)0.5 * (rr[a] + rr[b]), fc[a] * fc[b], Av, BF);
                    T* blk = row + kRadial + pair_bucket(tt[a], tt[b]) * kTS;
                    for (int t = 0; t < kNumThetas; t++)
                        for (int s = 0; s < kNumARs; s++) blk[t * kNumARs + s] += Av[t] * BF[s];
                }
        }
    }
}

template <typename T>
static void featurize_grad(const T* X, const T* Y, const T* Z, const int* A, const int* mo,
                           const int* mac, int n_mols, const int* si, const T* const* g, T* GX, T* GY,
                           T* GZ)
{
    for (int m = 0; m < n_mols; m++) {
        const int n = mac[m], base = mo[m];
        for (int i = 0; i < n; i++) {
            const int gi = base + i;
            const T* row = g[A[gi]] + (size_t)si[gi] * kTotal;
            std::vector<T> ux, uy, uz, rr, fc, dfc;
            std::vector<int> tt, idx;
            for (int j = 0; j < n; j++) {
                if (j == i) continue;
                const int gj = base + j;
                const T dx = X[gi] - X[gj], dy = Y[gi] - Y[gj], dz = Z[gi] - Z[gj];
                const T r = Num<T>::sqrt_(dx * dx + dy * dy + dz * dz);
                if (r < (T)kR_Rc) {
                    T f, df;
                    cutoff<T>(r, (T)kR_Rc, &f, &df);
                    const T d = radial_vjp<T, T>(r, f, df, row + A[gj] * kNumRs);
                    GX[gi] += d * dx / r; GY[gi] += d * dy / r; GZ[gi] += d * dz / r;
                    GX[gj] -= d * dx / r; GY[gj] -= d * dy / r; GZ[gj] -= d * dz / r;
                }
                if (r < (T)kA_Rc) {
                    T f, df;
                    cutoff<T>(r, (T)kA_Rc, &f, &df);
                    ux.push_back(dx / r); uy.push_back(dy / r); uz.push_back(dz / r);
                    rr.push_back(r); fc.push_back(f); dfc.push_back(df); tt.push_back(A[gj]);
                    idx.push_back(gj);
                }
            }
            for (size_t a = 0; a < rr.size(); a++)
                for (size_t b = a + 1; b < rr.size(); b++) {
                    T c = ux[a] * ux[b] + uy[a] * uy[b] + uz[a] * uz[b];
                    c = Num<T>::max_((T)-1, Num<T>::min_((T)1, c));
                    T dc, dra, drb;
                    const T s2 = sin2_from_cross<T>(ux[a], uy[a], uz[a], ux[b], uy[b], uz[b]);
                    angular_vjp<T, T>(c, s2, rr[a], rr[b], fc[a], dfc[a], fc[b], dfc[b],
                                      row + kRadial + pair_bucket(tt[a], tt[b]) * kTS, &dc, &dra, &drb);
                    const T aa = -dc / rr[a], ba = c * dc / rr[a] - dra;
                    const T ab = -dc / rr[b], bb = c * dc / rr[b] - drb;
                    const T gax = aa * ux[b] + ba * ux[a], gay = aa * uy[b] + ba * uy[a], gaz = aa * uz[b] + ba * uz[a];
                    const T gbx = ab * ux[a] + bb * ux[b], gby = ab * uy[a] + bb * uy[b], gbz = ab * uz[a] + bb * uz[b];
                    GX[idx[a]] += gax; GY[idx[a]] += gay; GZ[idx[a]] += gaz;
                    GX[idx[b]] += gbx; GY[idx[b]] += gby; GZ[idx[b]] += gbz;
                    GX[gi] -= gax + gbx; GY[gi] -= gay + gby; GZ[gi] -= gaz + gbz;
                }
        }
    }
}

#define EXPORT(T, SUF)                                                                              \
    extern "C" void hostmath_featurize_##SUF(const T* X, const T* Y, const T* Z, const int* A,     \
                                             const int* mo, const int* mac, int n_mols,              \
                                             const int* si, T* h, T* c, T* n, T* o)                  \
    {                                                                                                \
        T* out[4] = {h, c, n, o};                                                                    \
        featurize<T>(X, Y, Z, A, mo, mac, n_mols, si, out);                                          \
    }                                                                                                \
    extern "C" void hostmath_featurize_grad_##SUF(const T* X, const T* Y, const T* Z, const int* A,\
                                                  const int* mo, const int* mac, int n_mols,         \
                                                  const int* si, const T* h, const T* c, const T* n, \
                                                  const T* o, T* gx, T* gy, T* gz)                   \
    {                                                                                                \
        const T* g[4] = {h, c, n, o};                                                                \
        featurize_grad<T>(X, Y, Z, A, mo, mac, n_mols, si, g, gx, gy, gz);                           \
    }
EXPORT(float, f32)
EXPORT(double, f64)
