// Fixed ANI-1 symmetry-function parameter set and the scalar math shared by every kernel.
//
// The parameter values are the live set of the reference's gpu_featurizer/parameters.h:61-114.
// They are single-precision literals there, also when the reference is instantiated for
// double, so the double variants below promote the float-rounded value instead of using the
// decimal literal (4.6f promoted is 4.599999904632568, not 4.6).
//
// Everything in this header compiles both as device code (nvcc) and as plain host C++ (g++),
// so that the per-pair / per-triplet formulas can be checked on a machine without a GPU.
#pragma once

#include <math.h>

#if defined(__CUDACC__)
#define ANI_HD __host__ __device__ __forceinline__
#else
#define ANI_HD inline
#endif

namespace ani {

constexpr int kTypes = 4;                       // H C N O, compacted ids 0..3
constexpr int kNumRs = 16;                      // radial shifts
constexpr int kNumThetas = 8;                   // angular theta shifts
constexpr int kNumARs = 4;                      // angular radial shifts
constexpr int kTS = kNumThetas * kNumARs;       // 32 (theta, shift) terms per type pair
constexpr int kRadial = kTypes * kNumRs;        // 64
constexpr int kPairBuckets = kTypes * (kTypes + 1) / 2;  // 10 unordered type pairs
constexpr int kAngular = kPairBuckets * kTS;    // 320
constexpr int kTotal = kRadial + kAngular;      // 384

constexpr float kR_eta = 16.0f;
constexpr float kR_Rc = 4.6f;
constexpr float kA_Rc = 3.1f;
constexpr float kA_eta = 6.0f;
// zeta = 8 is used as three squarings; 2^(1-zeta) = 1/128.
constexpr float kA_pref = 0.0078125f;

// Index of the unordered type pair (i, j) in the angular block: HH,HC,HN,HO,CC,CN,CO,NN,NO,OO.
// Same map as linearize() of the reference (gpu_featurizer/kernel_cpu.cpp:9-23) with N = 4.
ANI_HD int pair_bucket(int ti, int tj)
{
    const int lo = ti < tj ? ti : tj;
    const int hi = ti < tj ? tj : ti;
    return kTypes * (kTypes - 1) / 2 - (kTypes - lo) * (kTypes - lo - 1) / 2 + hi;
}

template <typename T> ANI_HD T radial_shift(int r)
{
    const float v[kNumRs] = {5.0000000e-01f, 7.5625000e-01f, 1.0125000e+00f, 1.2687500e+00f,
                             1.5250000e+00f, 1.7812500e+00f, 2.0375000e+00f, 2.2937500e+00f,
                             2.5500000e+00f, 2.8062500e+00f, 3.0625000e+00f, 3.3187500e+00f,
                             3.5750000e+00f, 3.8312500e+00f, 4.0875000e+00f, 4.3437500e+00f};
    return (T)v[r];
}

template <typename T> ANI_HD T angular_shift(int s)
{
    const float v[kNumARs] = {5.0000000e-01f, 1.1500000e+00f, 1.8000000e+00f, 2.4500000e+00f};
    return (T)v[s];
}

// cos / sin of the eight theta shifts.  The shifts are the float literals of the reference
// (0, 7.8539816e-01, 1.5707963, ... 5.4977871), which are NOT exact multiples of pi/4; the
// tables hold cos and sin of the float-rounded values, to 20 digits.
template <typename T> ANI_HD T theta_cos(int t)
{
    const double v[kNumThetas] = {1.0,
                                  0.70710676573223721282,
                                  7.5497899548918749969e-8,
                                  -0.70710678540262942905,
                                  -0.99999999999999617863,
                                  -0.70710683035554063407,
                                  1.1924880454806034642e-8,
                                  0.70710667863246853197};
    return (T)v[t];
}

template <typename T> ANI_HD T theta_sin(int t)
{
    const double v[kNumThetas] = {0.0,
                                  0.70710679664085749822,
                                  0.99999999999999715003,
                                  0.70710677697046559462,
                                  -8.7422780003724745258e-8,
                                  -0.70710673201755099574,
                                  -0.9999999999999999289,
                                  -0.70710688374061164307};
    return (T)v[t];
}

// ---------------------------------------------------------------------------------------
// Elementary functions.  float uses the SFU approximations on the device (ex2.approx,
// sin/cos.approx on an argument bounded by pi, rsqrt.approx); double uses full precision.
// ---------------------------------------------------------------------------------------
template <typename T> struct Num;

#if defined(__CUDACC__)
// Single SFU instructions, written as PTX so that the choice does not depend on compiler flags.
__device__ __forceinline__ float sfu_ex2(float x)
{
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float sfu_rsqrt(float x)
{
    float y;
    asm("rsqrt.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ float sfu_sqrt(float x)
{
    float y;
    asm("sqrt.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
#endif

// Two values processed by one instruction where the hardware can: Blackwell (sm_100) has packed
// single-precision fma / mul / add (fma.rn.f32x2 ...), which halves the instruction count of the
// multiply-add heavy loops.  Everywhere else (double, host) a pair is just two scalars.
template <typename T> struct Pair {
    T x, y;
};

template <typename T> ANI_HD Pair<T> pfma(Pair<T> a, Pair<T> b, Pair<T> c)
{
    return Pair<T>{a.x * b.x + c.x, a.y * b.y + c.y};
}
template <typename T> ANI_HD Pair<T> pmul(Pair<T> a, Pair<T> b) { return Pair<T>{a.x * b.x, a.y * b.y}; }
template <typename T> ANI_HD Pair<T> padd(Pair<T> a, Pair<T> b) { return Pair<T>{a.x + b.x, a.y + b.y}; }

#if defined(__CUDACC__)
__device__ __forceinline__ unsigned long long pack2(float x, float y)
{
    unsigned long long r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(x), "f"(y));
    return r;
}
__device__ __forceinline__ Pair<float> unpack2(unsigned long long r)
{
    Pair<float> p;
    asm("mov.b64 {%0, %1}, %2;" : "=f"(p.x), "=f"(p.y) : "l"(r));
    return p;
}
#endif

template <> ANI_HD Pair<float> pfma<float>(Pair<float> a, Pair<float> b, Pair<float> c)
{
#if defined(__CUDA_ARCH__)
    unsigned long long d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(pack2(a.x, a.y)), "l"(pack2(b.x, b.y)), "l"(pack2(c.x, c.y)));
    return unpack2(d);
#else
    return Pair<float>{a.x * b.x + c.x, a.y * b.y + c.y};
#endif
}
template <> ANI_HD Pair<float> pmul<float>(Pair<float> a, Pair<float> b)
{
#if defined(__CUDA_ARCH__)
    unsigned long long d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(pack2(a.x, a.y)), "l"(pack2(b.x, b.y)));
    return unpack2(d);
#else
    return Pair<float>{a.x * b.x, a.y * b.y};
#endif
}
template <> ANI_HD Pair<float> padd<float>(Pair<float> a, Pair<float> b)
{
#if defined(__CUDA_ARCH__)
    unsigned long long d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(pack2(a.x, a.y)), "l"(pack2(b.x, b.y)));
    return unpack2(d);
#else
    return Pair<float>{a.x + b.x, a.y + b.y};
#endif
}

template <> struct Num<float> {
    static constexpr float kPi = 3.14159265358979323846f;
    // exp(-eta * x2) for x2 >= 0 (a squared distance offset)
    static ANI_HD float exp_neg(float eta, float x2)
    {
#if defined(__CUDA_ARCH__)
        return sfu_ex2(x2 * (-eta * 1.4426950408889634f));
#else
        return expf(-eta * x2);
#endif
    }
    static ANI_HD void sincos_bounded(float a, float* s, float* c)  // |a| <= pi
    {
#if defined(__CUDA_ARCH__)
        *s = __sinf(a);
        *c = __cosf(a);
#else
        *s = sinf(a);
        *c = cosf(a);
#endif
    }
    static ANI_HD float sqrt_(float x)
    {
#if defined(__CUDA_ARCH__)
        return sfu_sqrt(x);
#else
        return sqrtf(x);
#endif
    }
    static ANI_HD float rsqrt_(float x)
    {
#if defined(__CUDA_ARCH__)
        return sfu_rsqrt(x);
#else
        return 1.0f / sqrtf(x);
#endif
    }
    static ANI_HD float max_(float a, float b) { return fmaxf(a, b); }
    static ANI_HD float min_(float a, float b) { return fminf(a, b); }
};

template <> struct Num<double> {
    static constexpr double kPi = 3.14159265358979323846;
    static ANI_HD double exp_neg(double eta, double x2) { return exp(-eta * x2); }
    static ANI_HD void sincos_bounded(double a, double* s, double* c)
    {
        *s = sin(a);
        *c = cos(a);
    }
    static ANI_HD double sqrt_(double x) { return sqrt(x); }
    static ANI_HD double rsqrt_(double x) { return 1.0 / sqrt(x); }
    static ANI_HD double max_(double a, double b) { return fmax(a, b); }
    static ANI_HD double min_(double a, double b) { return fmin(a, b); }
};

// Cosine cutoff f_C(r) = 0.5 cos(pi r / rc) + 0.5 and its derivative, for r already known
// to be below rc (gpu_featurizer/kernel_cpu.cpp:29-35).
template <typename T> ANI_HD void cutoff(T r, T rc, T* fc, T* dfc)
{
    T s, c;
    const T k = Num<T>::kPi / rc;
    Num<T>::sincos_bounded(r * k, &s, &c);
    *fc = (T)0.5 * c + (T)0.5;
    *dfc = (T)-0.5 * k * s;
}

template <typename T> ANI_HD T cutoff_value(T r, T rc)
{
    T fc, dfc;
    cutoff<T>(r, rc, &fc, &dfc);
    return fc;
}

// ---------------------------------------------------------------------------------------
// Radial terms of one (i, j) pair:  out[r] = exp(-R_eta (rij - R_Rs[r])^2) * fc(rij)
// (gpu_featurizer/kernel_cpu.cpp:479-487).
// ---------------------------------------------------------------------------------------
template <typename T> ANI_HD T radial_term(T rij, T fc, int r)
{
    const T d = rij - radial_shift<T>(r);
    return Num<T>::exp_neg((T)kR_eta, d * d) * fc;
}

// d/d rij of sum_r w[r] * radial_term(r): the scalar that multiplies the unit vector in the
// radial part of the coordinate gradient (gpu_featurizer/kernel_cpu.cpp:281-301).
template <typename T, typename W> ANI_HD T radial_vjp(T rij, T fc, T dfc, const W* w)
{
    Pair<T> acc{(T)0, (T)0};
    const Pair<T> rr{rij, rij}, slope{(T)-2 * (T)kR_eta * fc, (T)-2 * (T)kR_eta * fc}, dd{dfc, dfc};
#pragma unroll
    for (int r = 0; r < kNumRs; r += 2) {   // two radial shifts per packed instruction
        const Pair<T> neg_shift{-radial_shift<T>(r), -radial_shift<T>(r + 1)};
        const Pair<T> d = padd(rr, neg_shift);
        const Pair<T> d2 = pmul(d, d);
        const Pair<T> e{Num<T>::exp_neg((T)kR_eta, d2.x), Num<T>::exp_neg((T)kR_eta, d2.y)};
        const Pair<T> we = pmul(Pair<T>{(T)w[r], (T)w[r + 1]}, e);
        acc = pfma(we, pfma(d, slope, dd), acc);
    }
    return acc.x + acc.y;
}

// ---------------------------------------------------------------------------------------
// Angular factors of one triplet (i; j, k) (gpu_featurizer/kernel_cpu.cpp:513-531):
//   term(t, s) = A[t] * BF[s],
//   A[t]  = (1 + cos(theta - theta_t))^8, with cos(theta - theta_t) = c cos(theta_t) + s sin(theta_t)
//           evaluated from c = cos(theta) (clamped to [-1, 1]) and s = sqrt(1 - c^2) >= 0,
//           which is what acos() followed by cos() gives since theta is in [0, pi];
//   BF[s] = 2^-7 exp(-A_eta (rbar - A_Rs[s])^2) fc(rij) fc(rik).
// ---------------------------------------------------------------------------------------
template <typename T> ANI_HD void angular_factors(T cosv, T rbar, T fcprod, T* A, T* BF)
{
    const T c = Num<T>::max_((T)-1, Num<T>::min_((T)1, cosv));
    const T s = Num<T>::sqrt_(Num<T>::max_((T)0, (T)1 - c * c));
    const Pair<T> cc{c, c}, ss{s, s}, one{(T)1, (T)1};
#pragma unroll
    for (int t = 0; t < kNumThetas; t += 2) {   // two theta shifts per (packed) instruction
        const Pair<T> ct{theta_cos<T>(t), theta_cos<T>(t + 1)}, st{theta_sin<T>(t), theta_sin<T>(t + 1)};
        const Pair<T> b = pfma(cc, ct, pfma(ss, st, one));
        const Pair<T> b2 = pmul(b, b);
        const Pair<T> b4 = pmul(b2, b2);
        const Pair<T> b8 = pmul(b4, b4);
        A[t] = b8.x;
        A[t + 1] = b8.y;
    }
    const T f = (T)kA_pref * fcprod;
    const Pair<T> ff{f, f}, rr{rbar, rbar};
#pragma unroll
    for (int q = 0; q < kNumARs; q += 2) {
        const Pair<T> neg_shift{-angular_shift<T>(q), -angular_shift<T>(q + 1)};
        const Pair<T> d = padd(rr, neg_shift);
        const Pair<T> d2 = pmul(d, d);
        const Pair<T> e{Num<T>::exp_neg((T)kA_eta, d2.x), Num<T>::exp_neg((T)kA_eta, d2.y)};
        const Pair<T> bf = pmul(e, ff);
        BF[q] = bf.x;
        BF[q + 1] = bf.y;
    }
}

// |u x v|^2 = sin^2 of the angle between two unit vectors.  Used instead of 1 - cos^2 in the
// gradient, where the cancellation in 1 - cos^2 near a collinear triplet would be amplified
// by the 1/sin(theta) of d theta/d cos.
template <typename T> ANI_HD T sin2_from_cross(T ax, T ay, T az, T bx, T by, T bz)
{
    const T cx = ay * bz - az * by, cy = az * bx - ax * bz, cz = ax * by - ay * bx;
    return cx * cx + cy * cy + cz * cz;
}

// Reverse mode for one triplet.  g[t*4+s] is dL/d term(t, s) (the 32 upstream values of the
// central atom's row for this type pair); cosv and sin2 are cos(theta) and sin^2(theta) of
// the angle at the central atom.  Returns the three scalars
//   dc  = dL/dcos(theta),  drj = dL/dr_ij,  drk = dL/dr_ik
// from which the coordinate gradients follow by
//   dL/dx_j = -dc (u_k - c u_j)/r_ij - drj u_j,   dL/dx_k likewise,   dL/dx_i = -(sum),
// with u_j = (x_i - x_j)/r_ij.  Same derivative as the reference's expanded expressions at
// gpu_featurizer/kernel_cpu.cpp:335-353, but written with (1+cos)^7 sin(theta-theta_t) and
// d cos/dx, so nothing is divided by (1 + cos(theta - theta_t)); the remaining 1/sin(theta)
// is dropped (set to zero) for a numerically collinear triplet, where the reference
// returns Inf/NaN.
template <typename T, typename W>
ANI_HD void angular_vjp(T cosv, T sin2, T rij, T rik, T fcj, T dfcj, T fck, T dfck, const W* g,
                        T* dc, T* drj, T* drk)
{
    const T c = Num<T>::max_((T)-1, Num<T>::min_((T)1, cosv));
    const T s2 = Num<T>::min_((T)1, sin2);
    const T s = Num<T>::sqrt_(s2);
    const bool bent = s2 > (T)1e-12;  // sin(theta) > 1e-6
    const T cot = bent ? c * Num<T>::rsqrt_(s2) : (T)0;
    const T keep = bent ? (T)1 : (T)0;
    const T rbar = (T)0.5 * (rij + rik);

    // e[q] = exp(-eta d_q^2), de[q] = d_q e[q], two shifts per packed instruction
    Pair<T> e[kNumARs / 2], de[kNumARs / 2];
    const Pair<T> rr{rbar, rbar};
#pragma unroll
    for (int q = 0; q < kNumARs; q += 2) {
        const Pair<T> neg_shift{-angular_shift<T>(q), -angular_shift<T>(q + 1)};
        const Pair<T> d = padd(rr, neg_shift);
        const Pair<T> d2 = pmul(d, d);
        e[q / 2] = Pair<T>{Num<T>::exp_neg((T)kA_eta, d2.x), Num<T>::exp_neg((T)kA_eta, d2.y)};
        de[q / 2] = pmul(d, e[q / 2]);
    }
    // u[t] = sum_q g[t][q] e[q], v[t] = sum_q g[t][q] de[q]
    T u[kNumThetas], v[kNumThetas];
#pragma unroll
    for (int t = 0; t < kNumThetas; t++) {
        const Pair<T> g01{(T)g[t * kNumARs + 0], (T)g[t * kNumARs + 1]};
        const Pair<T> g23{(T)g[t * kNumARs + 2], (T)g[t * kNumARs + 3]};
        const Pair<T> pu = pfma(g23, e[1], pmul(g01, e[0]));
        const Pair<T> pv = pfma(g23, de[1], pmul(g01, de[0]));
        u[t] = pu.x + pu.y;
        v[t] = pv.x + pv.y;
    }
    Pair<T> s0p{(T)0, (T)0}, s2p{(T)0, (T)0}, scp{(T)0, (T)0}, ssp{(T)0, (T)0};
    const Pair<T> cc{c, c}, sn{s, s}, one{(T)1, (T)1};
#pragma unroll
    for (int t = 0; t < kNumThetas; t += 2) {   // two theta shifts per packed instruction
        const Pair<T> ct{theta_cos<T>(t), theta_cos<T>(t + 1)}, st{theta_sin<T>(t), theta_sin<T>(t + 1)};
        const Pair<T> ut{u[t], u[t + 1]}, vt{v[t], v[t + 1]};
        const Pair<T> b = pfma(cc, ct, pfma(sn, st, one));
        const Pair<T> b2 = pmul(b, b);
        const Pair<T> b4 = pmul(b2, b2);
        const Pair<T> b7 = pmul(pmul(b4, b2), b);
        const Pair<T> a = pmul(b7, b);
        s0p = pfma(a, ut, s0p);
        s2p = pfma(a, vt, s2p);
        const Pair<T> b7u = pmul(b7, ut);
        scp = pfma(b7u, ct, scp);
        ssp = pfma(b7u, st, ssp);
    }
    const T s0 = s0p.x + s0p.y, s2sum = s2p.x + s2p.y, sc = scp.x + scp.y, ss = ssp.x + ssp.y;
    const T f = (T)kA_pref * fcj * fck;
    // dA_t/dc = 8 b^7 (cos(theta_t) - sin(theta_t) c / s)
    *dc = (T)8 * f * (keep * sc - cot * ss);
    const T common = -(T)kA_eta * f * s2sum;  // through rbar: d rbar / d r = 1/2, d e/d rbar = -2 eta d e
    *drj = common + (T)kA_pref * dfcj * fck * s0;
    *drk = common + (T)kA_pref * fcj * dfck * s0;
}

}  // namespace ani
