/*
 * TEST INFRASTRUCTURE ONLY.  CPU oracle for the ANI-1 atomic-environment-vector
 * path: a plain-C restatement of the reference's CPU algorithm, used by tests/,
 * by the smoke check and by the bench's cpu_baseline leg as the CHECKER.  No
 * product code path may link, load or call this file.
 *
 * What is restated, with the reference lines each part follows:
 *   oracle_ani_sort                    gpu_featurizer/ani_sort.cpp:41-62,90-113
 *   oracle_featurize_{f32,f64}         gpu_featurizer/kernel_cpu.cpp:406-537
 *   oracle_featurize_grad_{f32,f64}    gpu_featurizer/kernel_cpu.cpp:217-366
 *   oracle_featurize_grad_inverse_*    gpu_featurizer/kernel_cpu.cpp:37-179
 *   oracle_linearize                   gpu_featurizer/kernel_cpu.cpp:9-23
 *   oracle_fc / oracle_dist            gpu_featurizer/kernel_cpu.cpp:25-35
 *   constants                          gpu_featurizer/parameters.h:61-114
 *
 * Parity of this restatement is PINNED: tests/test_oracle.py checks it against
 * the reference's own known-answer vectors (sort indices of the 11-atom fixture,
 * gpu_featurizer/test_kernel.py:310-312) and against outputs of the reference's
 * kernel_cpu.cpp compiled unmodified (oracle/_ref, golden files under
 * tests/golden/).
 */

#include <math.h>
#include <stddef.h>
#include <stdlib.h>
#include <string.h>

#ifndef M_PI
#define M_PI 3.14159265358979323846
#endif

enum {
    ANI_MAX_TYPES = 4,
    ANI_NUM_R_RS = 16,
    ANI_NUM_A_THETAS = 8,
    ANI_NUM_A_RS = 4,
    ANI_RADIAL = ANI_MAX_TYPES * ANI_NUM_R_RS,                                             /* 64  */
    ANI_ANGULAR = ANI_NUM_A_RS * ANI_NUM_A_THETAS * (ANI_MAX_TYPES * (ANI_MAX_TYPES + 1) / 2), /* 320 */
    ANI_TOTAL = ANI_RADIAL + ANI_ANGULAR                                                   /* 384 */
};

/* gpu_featurizer/parameters.h:61-114 -- all single precision, also for the double build */
static const float kChargeConstant = 0.529176917f;   /* parameters.h:10 */
static const float kR_eta = 16.0f;
static const float kR_Rc = 4.6f;
static const float kA_Rc = 3.1f;
static const float kA_eta = 6.0f;
static const float kA_zeta = 8.0f;
static const float kR_Rs[ANI_NUM_R_RS] = {
    5.0000000e-01f, 7.5625000e-01f, 1.0125000e+00f, 1.2687500e+00f,
    1.5250000e+00f, 1.7812500e+00f, 2.0375000e+00f, 2.2937500e+00f,
    2.5500000e+00f, 2.8062500e+00f, 3.0625000e+00f, 3.3187500e+00f,
    3.5750000e+00f, 3.8312500e+00f, 4.0875000e+00f, 4.3437500e+00f};
static const float kA_thetas[ANI_NUM_A_THETAS] = {
    0.0000000e+00f, 7.8539816e-01f, 1.5707963e+00f, 2.3561945e+00f,
    3.1415927e+00f, 3.9269908e+00f, 4.7123890e+00f, 5.4977871e+00f};
static const float kA_Rs[ANI_NUM_A_RS] = {5.0000000e-01f, 1.1500000e+00f, 1.8000000e+00f, 2.4500000e+00f};

int oracle_feature_size(void) { return ANI_TOTAL; }

/* gpu_featurizer/kernel_cpu.cpp:9-23 */
int oracle_linearize(int i, int j, int k, int l)
{
    if (j < i) { int tmp = i; i = j; j = tmp; }
    const int N = ANI_MAX_TYPES;
    const int basis = N * (N - 1) / 2 - (N - i) * (N - i - 1) / 2 + j;
    return basis * ANI_NUM_A_THETAS * ANI_NUM_A_RS + k * ANI_NUM_A_RS + l;
}

/* gpu_featurizer/kernel_cpu.cpp:25-27 */
static double oracle_dist(double dx, double dy, double dz) { return sqrt(dx * dx + dy * dy + dz * dz); }

/* gpu_featurizer/kernel_cpu.cpp:29-35 */
static double oracle_fc(double r, double rc)
{
    if (r <= rc) return 0.5 * cos((M_PI * r) / rc) + 0.5;
    return 0.0;
}

/*
 * AniSort, gpu_featurizer/ani_sort.cpp:71-115: a stable sort of the whole batch by
 * element id.  scatter[i] = rank of atom i among atoms of its element (batch order),
 * gather[i] = position of atom i in the element-sorted concatenation, counts[4].
 * The reference sorts an index vector with std::stable_sort and inverts the
 * permutation; a stable counting sort yields the same three arrays.
 */
void oracle_ani_sort(const int *atomic_numbers, int n_atoms, int *scatter, int *gather, int *counts)
{
    int c[ANI_MAX_TYPES] = {0, 0, 0, 0};
    for (int i = 0; i < n_atoms; i++) {       /* ani_sort.cpp:95-100 */
        scatter[i] = c[atomic_numbers[i]];
        c[atomic_numbers[i]] += 1;
    }
    int start[ANI_MAX_TYPES];
    int acc = 0;
    for (int t = 0; t < ANI_MAX_TYPES; t++) { start[t] = acc; acc += c[t]; counts[t] = c[t]; }
    for (int i = 0; i < n_atoms; i++)         /* ani_sort.cpp:110-113 */
        gather[i] = start[atomic_numbers[i]] + scatter[i];
}

#define REAL float
#define SUFFIX f32
#define REAL_ACOS acosf
#define REAL_COS cosf
#define REAL_POW powf
#include "ani_oracle_impl.h"
#undef REAL
#undef SUFFIX
#undef REAL_ACOS
#undef REAL_COS
#undef REAL_POW

#define REAL double
#define SUFFIX f64
#define REAL_ACOS acos
#define REAL_COS cos
#define REAL_POW pow
#include "ani_oracle_impl.h"
#undef REAL
#undef SUFFIX
#undef REAL_ACOS
#undef REAL_COS
#undef REAL_POW

/* Work counters used to turn a timed run into flop/s: unordered radial pairs with
 * r < R_Rc and angular triplets (i; j<k) with r_ij, r_ik < A_Rc, using the same
 * float comparisons as the forward above. */
void oracle_count_work_f32(const float *X, const float *Y, const float *Z, const int *mol_offsets,
                           const int *mol_counts, int n_mols, long long *pairs, long long *triplets)
{
    long long P = 0, T = 0;
    for (int m = 0; m < n_mols; m++) {
        const int n = mol_counts[m], base = mol_offsets[m];
        for (int ii = 0; ii < n; ii++) {
            int nang = 0;
            for (int jj = 0; jj < n; jj++) {
                if (jj == ii) continue;
                const float dx = X[base + ii] - X[base + jj], dy = Y[base + ii] - Y[base + jj],
                            dz = Z[base + ii] - Z[base + jj];
                const float r = (float)oracle_dist(dx, dy, dz);
                if (r < kR_Rc && ii < jj) P++;
                if (r < kA_Rc) nang++;
            }
            T += (long long)nang * (nang - 1) / 2;
        }
    }
    *pairs = P; *triplets = T;
}
