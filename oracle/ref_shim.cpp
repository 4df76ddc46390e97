/*
 * TEST INFRASTRUCTURE ONLY.  extern "C" doors onto the reference's own CPU kernels.
 *
 * This file holds no algorithm.  It is compiled together with the reference's
 * gpu_featurizer/kernel_cpu.cpp, taken unmodified from the reference checkout at
 * build time (see the Makefile beside this file; no reference source is copied
 * into this repository), and forwards to the explicit template instantiations
 * that file provides (kernel_cpu.cpp:181-215, 369-403, 540-567).  The zero fill
 * that the reference does one layer up (gpu_featurizer/functor_op_cpu.cpp:31-34,
 * 70-72, 107-110) is left to the Python caller, which passes zeroed arrays.
 */
#include "kernel_cpu.h"   /* resolved with -I <reference>/gpu_featurizer */

#define DOORS(T, SUF)                                                                          \
    extern "C" void ref_featurize_##SUF(const T *x, const T *y, const T *z, const int *a,       \
                                        const int *mo, const int *mac, int n_mols,               \
                                        const int *si, T *h, T *c, T *n, T *o)                   \
    {                                                                                            \
        featurize_cpu<T>(x, y, z, a, mo, mac, n_mols, si, h, c, n, o);                           \
    }                                                                                            \
    extern "C" void ref_featurize_grad_##SUF(const T *x, const T *y, const T *z, const int *a,  \
                                             const int *mo, const int *mac, int n_mols,          \
                                             const int *si, const T *gh, const T *gc,            \
                                             const T *gn, const T *go, T *gx, T *gy, T *gz)      \
    {                                                                                            \
        featurize_grad_cpu<T>(x, y, z, a, mo, mac, n_mols, si, gh, gc, gn, go, gx, gy, gz);      \
    }                                                                                            \
    extern "C" void ref_featurize_grad_inverse_##SUF(                                            \
        const T *x, const T *y, const T *z, const int *a, const int *mo, const int *mac,         \
        int n_mols, const int *si, const T *vx, const T *vy, const T *vz, T *h, T *c, T *n,      \
        T *o)                                                                                    \
    {                                                                                            \
        featurize_grad_inverse<T>(x, y, z, a, mo, mac, n_mols, si, vx, vy, vz, h, c, n, o);      \
    }

DOORS(float, f32)
DOORS(double, f64)
