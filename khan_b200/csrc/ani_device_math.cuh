// Per-pair and per-triplet arithmetic of the featurizer kernels in the form the device likes: the same
// formulas as in ani_params.h (which also compiles for the host and is what the CPU-side checks use),
// but with every constant as an immediate operand of a scalar instruction, packed pairs only for
// products of two computed values, and, in float64, all Gaussians of a pair from two exp() calls.
#pragma once

#include "ani_common.cuh"

namespace ani {

// ---- float64 only: the Gaussians of all shifts from TWO calls of exp() ------------------------------
// exp(-eta (r - s_k)^2) for equally spaced shifts s_k = s_0 + k D factorises into
//   exp(-eta x^2) * exp(2 eta D x)^k * exp(-eta D^2 k^2),   x = r - s_0,
// i.e. one exp for the first shift, one for the ratio, and a constant per shift.  The reference's
// shifts are single-precision literals promoted to double (gpu_featurizer/parameters.h:79-114), so
// they sit up to 1e-7 off the even grid; with e_k = (actual shift) - (grid point) the exact value is
// the grid value times exp(eta e_k (x_k + d_k)), x_k / d_k the distance to the grid point / to the
// actual shift, and that exponent is below 4e-6, so 1 + t + t^2 / 2 is exact to 1e-17.  In double a
// library exp() costs some 35 instructions; this replaces 14 of the 16 radial and 2 of the 4 angular
// ones of every pair.  (In float exp is one SFU instruction and nothing is gained.)
struct RadialGrid {
    static constexpr int kN = kNumRs;
    static constexpr double kEta = 16.0, kS0 = 0.5, kDelta = 0.25625;
    __device__ static double eps(int k)
    {
        constexpr double v[kN] = {0.00000000000000000e+00, 2.38418579323607105e-08, 4.76837158647214210e-08,
                                  -4.76837157536991185e-08, -2.38418578213384080e-08, 1.11022302462515654e-16,
                                  -9.53674315073982370e-08, 4.76837159757437234e-08, -4.76837156426768161e-08,
                                  9.53674318404651444e-08, 2.22044604925031308e-16, -9.53674313963759346e-08,
                                  4.76837160867660259e-08, -4.76837155316545136e-08, 9.53674319514874469e-08,
                                  3.33066907387546962e-16};
        return v[k];
    }
    __device__ static double grid_factor(int k)   // exp(-eta D^2 k^2)
    {
        constexpr double v[kN] = {1.0, 0.34971910635094079063, 0.014958134700577500195, 0.0000782481790297574252,
                                  5.0062180207670567999e-8, 3.9172744395097853607e-12, 3.7488404577454681545e-17,
                                  4.3878183249839540439e-23, 6.281148147606062409e-30, 1.0996846322891938883e-37,
                                  2.3547022296838610375e-46, 6.1665542139028671753e-56, 1.9750942872771476687e-66,
                                  7.7369863671725676252e-78, 3.7067607034345540139e-90, 2.1719808350408576127e-103};
        return v[k];
    }
    __device__ static double shift(int k) { return radial_shift<double>(k); }
};
struct AngularGrid {
    static constexpr int kN = kNumARs;
    static constexpr double kEta = 6.0, kS0 = 0.5, kDelta = 0.65;
    __device__ static double eps(int k)
    {
        constexpr double v[kN] = {0.00000000000000000e+00, -2.38418579323607105e-08, -4.76837158647214210e-08,
                                  4.76837157536991185e-08};
        return v[k];
    }
    __device__ static double grid_factor(int k)
    {
        constexpr double v[kN] = {1.0, 0.079261719264731553938, 0.000039468802825543528604, 1.2347282803234498325e-10};
        return v[k];
    }
    __device__ static double shift(int k) { return angular_shift<double>(k); }
};

// d[k] = r - shift_k (the actual, promoted-float shift) and e[k] = exp(-eta d[k]^2), k = 0 .. Grid::kN - 1.
template <typename Grid> __device__ __forceinline__ void gaussians_f64(double r, double* d, double* e)
{
    const double x0 = r - Grid::kS0;
    const double first = exp(-Grid::kEta * x0 * x0);
    const double ratio = exp(2.0 * Grid::kEta * Grid::kDelta * x0);
    double power = 1.0;
#pragma unroll
    for (int k = 0; k < Grid::kN; k++) {
        d[k] = r - Grid::shift(k);
        const double xk = x0 - k * Grid::kDelta;
        const double t = Grid::kEta * Grid::eps(k) * (xk + d[k]);
        e[k] = (first * Grid::grid_factor(k)) * power * (1.0 + t * (1.0 + 0.5 * t));
        power *= ratio;
    }
}

// The 8 theta factors and 4 radial factors of one triplet (see angular_factors in ani_params.h),
// arranged for the device: every constant is an immediate operand of a scalar instruction and
// only the squarings run as packed pairs.
template <typename T> __device__ __forceinline__ void angular_factors_dev(T cosv, T rbar, T fcprod, T* A, T* BF)
{
    const T c = Num<T>::max_((T)-1, Num<T>::min_((T)1, cosv));
    const T s = Num<T>::sqrt_(Num<T>::max_((T)0, (T)1 - c * c));
    T b[kNumThetas];
#pragma unroll
    for (int t = 0; t < kNumThetas; t++) b[t] = c * theta_cos<T>(t) + (s * theta_sin<T>(t) + (T)1);
#pragma unroll
    for (int t = 0; t < kNumThetas; t += 2) {
        const Pair<T> b1{b[t], b[t + 1]};
        const Pair<T> b2 = pmul(b1, b1);
        const Pair<T> b4 = pmul(b2, b2);
        const Pair<T> b8 = pmul(b4, b4);
        A[t] = b8.x;
        A[t + 1] = b8.y;
    }
    const T f = (T)kA_pref * fcprod;
    if constexpr (sizeof(T) == 8) {
        double d[kNumARs], e[kNumARs];
        gaussians_f64<AngularGrid>(rbar, d, e);
#pragma unroll
        for (int q = 0; q < kNumARs; q++) BF[q] = e[q] * f;
        return;
    }
    T d[kNumARs];
#pragma unroll
    for (int q = 0; q < kNumARs; q++) d[q] = rbar - angular_shift<T>(q);
#pragma unroll
    for (int q = 0; q < kNumARs; q += 2) {
        const Pair<T> dd{d[q], d[q + 1]};
        const Pair<T> d2 = pmul(dd, dd);
        const Pair<T> bf = pmul(Pair<T>{Num<T>::exp_neg((T)kA_eta, d2.x), Num<T>::exp_neg((T)kA_eta, d2.y)}, Pair<T>{f, f});
        BF[q] = bf.x;
        BF[q + 1] = bf.y;
    }
}

// radial_vjp and angular_vjp of ani_params.h, arranged for the device: the same arithmetic, but every
// constant (shift, cos / sin of a theta shift) is an immediate operand of a scalar instruction, and
// only products of two computed values run as packed pairs.  (A packed instruction takes its
// operands from register pairs, so a pair of constants would cost two moves per use.)
template <typename T> __device__ __forceinline__ T radial_vjp_dev(T rij, T fc, T dfc, const T* w)
{
    const T slope = (T)-2 * (T)kR_eta * fc;
    if constexpr (sizeof(T) == 8) {   // all 16 Gaussians from two exp() calls
        double d[kNumRs], e[kNumRs];
        gaussians_f64<RadialGrid>(rij, d, e);
        double sum = 0.0;
#pragma unroll
        for (int r = 0; r < kNumRs; r++) sum += w[r] * e[r] * (d[r] * slope + dfc);
        return sum;
    }
    const Pair<T> sl{slope, slope}, dd{dfc, dfc};
    Pair<T> acc{(T)0, (T)0};
#pragma unroll
    for (int r = 0; r < kNumRs; r += 2) {
        const Pair<T> d{rij - radial_shift<T>(r), rij - radial_shift<T>(r + 1)};
        const Pair<T> d2 = pmul(d, d);
        const Pair<T> e{Num<T>::exp_neg((T)kR_eta, d2.x), Num<T>::exp_neg((T)kR_eta, d2.y)};
        acc = pfma(pmul(Pair<T>{w[r], w[r + 1]}, e), pfma(d, sl, dd), acc);
    }
    return acc.x + acc.y;
}

template <typename T>
__device__ __forceinline__ void angular_vjp_dev(T cosv, T sin2, T rij, T rik, T fcj, T dfcj, T fck, T dfck,
                                                const T* g, T* dc, T* drj, T* drk)
{
    const T c = Num<T>::max_((T)-1, Num<T>::min_((T)1, cosv));
    const T s2 = Num<T>::min_((T)1, sin2);
    const T s = Num<T>::sqrt_(s2);
    const bool bent = s2 > (T)1e-12;  // sin(theta) > 1e-6
    const T cot = bent ? c * Num<T>::rsqrt_(s2) : (T)0;
    const T keep = bent ? (T)1 : (T)0;
    const T rbar = (T)0.5 * (rij + rik);

    Pair<T> e[kNumARs / 2], de[kNumARs / 2];   // exp(-eta d_q^2) and d_q exp(-eta d_q^2)
    if constexpr (sizeof(T) == 8) {
        double dq[kNumARs], eq[kNumARs];
        gaussians_f64<AngularGrid>(rbar, dq, eq);
#pragma unroll
        for (int q = 0; q < kNumARs; q += 2) {
            e[q / 2] = Pair<T>{eq[q], eq[q + 1]};
            de[q / 2] = Pair<T>{dq[q] * eq[q], dq[q + 1] * eq[q + 1]};
        }
    } else
#pragma unroll
    for (int q = 0; q < kNumARs; q += 2) {
        const Pair<T> d{rbar - angular_shift<T>(q), rbar - angular_shift<T>(q + 1)};
        const Pair<T> d2 = pmul(d, d);
        e[q / 2] = Pair<T>{Num<T>::exp_neg((T)kA_eta, d2.x), Num<T>::exp_neg((T)kA_eta, d2.y)};
        de[q / 2] = pmul(d, e[q / 2]);
    }
    T u[kNumThetas], v[kNumThetas];   // u[t] = sum_q g[t][q] e[q], v[t] = sum_q g[t][q] de[q]
#pragma unroll
    for (int t = 0; t < kNumThetas; t++) {
        const Pair<T> g01{g[t * kNumARs + 0], g[t * kNumARs + 1]}, g23{g[t * kNumARs + 2], g[t * kNumARs + 3]};
        const Pair<T> pu = pfma(g23, e[1], pmul(g01, e[0]));
        const Pair<T> pv = pfma(g23, de[1], pmul(g01, de[0]));
        u[t] = pu.x + pu.y;
        v[t] = pv.x + pv.y;
    }
    T b[kNumThetas];
#pragma unroll
    for (int t = 0; t < kNumThetas; t++) b[t] = c * theta_cos<T>(t) + (s * theta_sin<T>(t) + (T)1);
    Pair<T> s0p{(T)0, (T)0}, s2p{(T)0, (T)0};
    T sc = (T)0, ss = (T)0;
#pragma unroll
    for (int t = 0; t < kNumThetas; t += 2) {
        const Pair<T> b1{b[t], b[t + 1]}, ut{u[t], u[t + 1]}, vt{v[t], v[t + 1]};
        const Pair<T> b2 = pmul(b1, b1);
        const Pair<T> b4 = pmul(b2, b2);
        const Pair<T> b7 = pmul(pmul(b4, b2), b1);
        const Pair<T> a = pmul(b7, b1);
        s0p = pfma(a, ut, s0p);
        s2p = pfma(a, vt, s2p);
        const Pair<T> b7u = pmul(b7, ut);
        sc += b7u.x * theta_cos<T>(t) + b7u.y * theta_cos<T>(t + 1);
        ss += b7u.x * theta_sin<T>(t) + b7u.y * theta_sin<T>(t + 1);
    }
    const T s0 = s0p.x + s0p.y, s2sum = s2p.x + s2p.y;
    const T f = (T)kA_pref * fcj * fck;
    *dc = (T)8 * f * (keep * sc - cot * ss);                 // dA_t/dc = 8 b^7 (cos(theta_t) - sin(theta_t) c / s)
    const T common = -(T)kA_eta * f * s2sum;                  // through rbar: d rbar / d r = 1/2, d e/d rbar = -2 eta d e
    *drj = common + (T)kA_pref * dfcj * fck * s0;
    *drk = common + (T)kA_pref * fcj * dfck * s0;
}

}  // namespace ani
