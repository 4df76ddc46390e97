/*
 * TEST INFRASTRUCTURE ONLY -- body of the CPU oracle, included twice by
 * ani_oracle.c (once with REAL=float, once with REAL=double).
 *
 * Each function restates, loop for loop, what the reference CPU kernels in
 * gpu_featurizer/kernel_cpu.cpp compute, but with the symbolic-algebra
 * gradient expressions of the reference factored by hand into
 * (value, d/dcos(theta), d/dr_ij, d/dr_ik) pieces.
 *
 * Precision notes (they matter for parity):
 *  - the symmetry-function parameters are `const float` in the reference even
 *    in its double instantiation (gpu_featurizer/parameters.h:61-114), so the
 *    double oracle uses the float-rounded constants promoted to double;
 *  - the reference stores intermediates in NumericType but calls libm through
 *    C++ overloads: pow(x, 2.0) / pow(x, int) / exp / f_C / dist_diff run in
 *    double, while acos(NumericType), cos(NumericType) and
 *    pow(NumericType, float) stay in NumericType
 *    (gpu_featurizer/kernel_cpu.cpp:25-35, 479-487, 513-527).  The forward
 *    below follows those types so that the float build rounds where the
 *    reference rounds.
 *  - the float gradient of the reference is not reproduced: it is non-finite
 *    on a large share of realistic triplets (0/0 when cos(theta_t-theta)+1
 *    rounds to zero, gpu_featurizer/kernel_cpu.cpp:335-353).  The float
 *    gradient here evaluates every term in double from the float inputs and
 *    rounds each accumulation to float.
 */

#ifndef REAL
#error "include from ani_oracle.c"
#endif

#define CAT_(a, b) a##_##b
#define CAT(a, b) CAT_(a, b)
#define FN(name) CAT(name, SUFFIX)

static REAL *FN(row_ptr)(int type, REAL *h, REAL *c, REAL *n, REAL *o)
{
    /* gpu_featurizer/kernel_cpu.cpp:438-447: element 0,1,2 -> H,C,N; anything else -> O */
    if (type == 0) return h;
    if (type == 1) return c;
    if (type == 2) return n;
    return o;
}

/* featurize_cpu, gpu_featurizer/kernel_cpu.cpp:406-537.  Outputs must be
 * zeroed by the caller (gpu_featurizer/functor_op_cpu.cpp:31-34 does so). */
void FN(oracle_featurize)(const REAL *X, const REAL *Y, const REAL *Z, const int *A,
                          const int *mol_offsets, const int *mol_counts, int n_mols,
                          const int *scatter, REAL *fH, REAL *fC_, REAL *fN, REAL *fO)
{
    for (int m = 0; m < n_mols; m++) {
        const int n = mol_counts[m];
        const int base = mol_offsets[m];
        for (int ii = 0; ii < n; ii++) {
            const int gi = base + ii;
            const int ti = A[gi];
            const REAL ix = X[gi], iy = Y[gi], iz = Z[gi];
            REAL *row_i = FN(row_ptr)(ti, fH, fC_, fN, fO) + (size_t)scatter[gi] * ANI_TOTAL;
            REAL *rad_i = row_i;
            REAL *ang_i = row_i + ANI_RADIAL;
            for (int jj = 0; jj < n; jj++) {
                const int gj = base + jj;
                const int tj = A[gj];
                const REAL dxj = ix - X[gj], dyj = iy - Y[gj], dzj = iz - Z[gj];
                const REAL rij = (REAL)oracle_dist((double)dxj, (double)dyj, (double)dzj);
                REAL *rad_j = FN(row_ptr)(tj, fH, fC_, fN, fO) + (size_t)scatter[gj] * ANI_TOTAL;

                if (rij < kR_Rc && ii < jj) { /* kernel_cpu.cpp:479 */
                    for (int r = 0; r < ANI_NUM_R_RS; r++) {
                        const REAL fc = (REAL)oracle_fc((double)rij, (double)kR_Rc);
                        const REAL dr = rij - kR_Rs[r];              /* NumericType - float */
                        const REAL lhs = (REAL)exp(-(double)kR_eta * ((double)dr * (double)dr));
                        const REAL summand = lhs * fc;
                        rad_i[tj * ANI_NUM_R_RS + r] += summand;
                        rad_j[ti * ANI_NUM_R_RS + r] += summand;
                    }
                }

                const REAL fc_ij = (REAL)oracle_fc((double)rij, (double)kA_Rc);
                if (rij < kA_Rc) { /* kernel_cpu.cpp:491 */
                    for (int kk = jj + 1; kk < n; kk++) {
                        if (ii == jj || ii == kk || jj == kk) continue;
                        const int gk = base + kk;
                        const int tk = A[gk];
                        const REAL dxk = ix - X[gk], dyk = iy - Y[gk], dzk = iz - Z[gk];
                        const REAL rik = (REAL)oracle_dist((double)dxk, (double)dyk, (double)dzk);
                        if (!(rik < kA_Rc)) continue;

                        REAL inner = (dxj * dxk + dyj * dyk + dzj * dzk) / (rij * rik);
                        inner = (REAL)fmax((double)inner, -1.0); /* kernel_cpu.cpp:514-516 */
                        inner = (REAL)fmin((double)inner, 1.0);
                        const REAL theta = REAL_ACOS(inner);
                        const REAL fc_ik = (REAL)oracle_fc((double)rik, (double)kA_Rc);
                        const REAL rbar = (rij + rik) / 2;
                        for (int t = 0; t < ANI_NUM_A_THETAS; t++) {
                            /* pow(NumericType, float) and cos(NumericType) stay in NumericType */
                            const REAL ang = REAL_POW((REAL)1 + REAL_COS(theta - (REAL)kA_thetas[t]),
                                                      (REAL)kA_zeta);
                            for (int s = 0; s < ANI_NUM_A_RS; s++) {
                                const REAL ds = rbar - kA_Rs[s];
                                const double summand = pow(2.0, 1 - (double)kA_zeta) * (double)ang *
                                    exp(-(double)kA_eta * ((double)ds * (double)ds)) *
                                    (double)fc_ij * (double)fc_ik;
                                ang_i[oracle_linearize(tj, tk, t, s)] += (REAL)summand;
                            }
                        }
                    }
                }
            }
        }
    }
}

/* One angular triplet (i; j, k): partial derivatives, in double, of
 *   F_ts = 2^(1-zeta) (1+cos(theta-theta_t))^zeta exp(-eta (rbar-Rs_s)^2) fc(rij) fc(rik)
 * with respect to cos(theta), r_ij and r_ik, for each of the 32 (t,s):
 *   pc[t*4+s] = dF_ts/dcos(theta), pj[..] = dF_ts/dr_ij, pk[..] = dF_ts/dr_ik.
 * Same factors as the sympy-expanded expressions at
 * gpu_featurizer/kernel_cpu.cpp:335-353 (theta is NOT clamped there, nor here). */
static void FN(triplet_partials)(double rij, double rik, double cosv,
                                 double *pc, double *pj, double *pk)
{
    const double theta = acos(cosv);
    const double sinv = sqrt(1.0 - cosv * cosv);
    const double Rc = (double)kA_Rc;
    const double fj = 0.5 * cos(M_PI * rij / Rc) + 0.5;
    const double fk = 0.5 * cos(M_PI * rik / Rc) + 0.5;
    const double dfj = -0.5 * M_PI * sin(M_PI * rij / Rc) / Rc;
    const double dfk = -0.5 * M_PI * sin(M_PI * rik / Rc) / Rc;
    const double pref = pow(2.0, 1.0 - (double)kA_zeta);
    const double rbar = 0.5 * rij + 0.5 * rik;
    for (int t = 0; t < ANI_NUM_A_THETAS; t++) {
        const double dth = theta - (double)kA_thetas[t];
        const double base = cos(dth) + 1.0;
        const double a = pow(base, (double)kA_zeta);
        /* d/dcos(theta) of base^zeta = zeta base^(zeta-1) sin(theta-theta_t) / sin(theta) */
        const double a_c = (double)kA_zeta * pow(base, (double)kA_zeta - 1.0) * sin(dth) / sinv;
        for (int s = 0; s < ANI_NUM_A_RS; s++) {
            const double ds = rbar - (double)kA_Rs[s];
            const double e = exp(-(double)kA_eta * ds * ds);
            const double radial_part = -(double)kA_eta * ds * e; /* (d e / d rbar) * 1/2 */
            pc[t * ANI_NUM_A_RS + s] = pref * a_c * e * fj * fk;
            pj[t * ANI_NUM_A_RS + s] = pref * a * (radial_part * fj * fk + e * dfj * fk);
            pk[t * ANI_NUM_A_RS + s] = pref * a * (radial_part * fj * fk + e * fj * dfk);
        }
    }
}

/* featurize_grad_cpu (vector-Jacobian product), gpu_featurizer/kernel_cpu.cpp:217-366.
 * Outputs must be zeroed by the caller (gpu_featurizer/functor_op_cpu.cpp:70-72). */
void FN(oracle_featurize_grad)(const REAL *X, const REAL *Y, const REAL *Z, const int *A,
                               const int *mol_offsets, const int *mol_counts, int n_mols,
                               const int *scatter, const REAL *gH, const REAL *gC, const REAL *gN,
                               const REAL *gO, REAL *GX, REAL *GY, REAL *GZ)
{
    for (int m = 0; m < n_mols; m++) {
        const int n = mol_counts[m];
        const int base = mol_offsets[m];
        for (int ii = 0; ii < n; ii++) {
            const int gi = base + ii;
            const int ti = A[gi];
            const double ix = X[gi], iy = Y[gi], iz = Z[gi];
            const REAL *row_i = FN(row_ptr)(ti, (REAL *)gH, (REAL *)gC, (REAL *)gN, (REAL *)gO) +
                                (size_t)scatter[gi] * ANI_TOTAL;
            const REAL *grad_rad = row_i;
            const REAL *grad_ang = row_i + ANI_RADIAL;
            for (int jj = 0; jj < n; jj++) {
                const int gj = base + jj;
                const int tj = A[gj];
                const double dxj = (REAL)(ix - X[gj]), dyj = (REAL)(iy - Y[gj]), dzj = (REAL)(iz - Z[gj]);
                const REAL rij_t = (REAL)oracle_dist(dxj, dyj, dzj);
                const double rij = rij_t;

                if (rij_t < kR_Rc && ii != jj) { /* kernel_cpu.cpp:281 */
                    const double Rc = (double)kR_Rc;
                    const double fc = 0.5 * cos(M_PI * rij / Rc) + 0.5;
                    const double dfc = -0.5 * M_PI * sin(M_PI * rij / Rc) / Rc;
                    for (int r = 0; r < ANI_NUM_R_RS; r++) {
                        const double w = grad_rad[tj * ANI_NUM_R_RS + r];
                        const double dr = rij - (double)kR_Rs[r];
                        const double e = exp(-(double)kR_eta * dr * dr);
                        const double dterm = e * (-2.0 * (double)kR_eta * dr * fc + dfc); /* d/dr */
                        const double ax = dterm * dxj / rij, ay = dterm * dyj / rij, az = dterm * dzj / rij;
                        GX[gi] += (REAL)(ax * w);  GY[gi] += (REAL)(ay * w);  GZ[gi] += (REAL)(az * w);
                        GX[gj] += (REAL)(-ax * w); GY[gj] += (REAL)(-ay * w); GZ[gj] += (REAL)(-az * w);
                    }
                }

                if (rij_t < kA_Rc) { /* kernel_cpu.cpp:304 */
                    for (int kk = jj + 1; kk < n; kk++) {
                        if (ii == jj || ii == kk || jj == kk) continue;
                        const int gk = base + kk;
                        const int tk = A[gk];
                        const double dxk = (REAL)(ix - X[gk]), dyk = (REAL)(iy - Y[gk]), dzk = (REAL)(iz - Z[gk]);
                        const REAL rik_t = (REAL)oracle_dist(dxk, dyk, dzk);
                        if (!(rik_t < kA_Rc)) continue;
                        /* the reference recomputes the distances in the gradient from the raw
                         * coordinates (kernel_cpu.cpp:330-332) */
                        const double dij = sqrt(dxj * dxj + dyj * dyj + dzj * dzj);
                        const double dik = sqrt(dxk * dxk + dyk * dyk + dzk * dzk);
                        const double dot = dxj * dxk + dyj * dyk + dzj * dzk;
                        const double cosv = dot / (dij * dik);
                        double pc[32], pj[32], pk[32];
                        FN(triplet_partials)(dij, dik, cosv, pc, pj, pk);
                        double dc = 0, drj = 0, drk = 0;
                        for (int t = 0; t < ANI_NUM_A_THETAS; t++)
                            for (int s = 0; s < ANI_NUM_A_RS; s++) {
                                const double w = grad_ang[oracle_linearize(tj, tk, t, s)];
                                dc += w * pc[t * ANI_NUM_A_RS + s];
                                drj += w * pj[t * ANI_NUM_A_RS + s];
                                drk += w * pk[t * ANI_NUM_A_RS + s];
                            }
                        /* d cos / d x_j = -(u_k - cos u_j)/r_ij ; d r_ij / d x_j = -u_j */
                        const double ujx = dxj / dij, ujy = dyj / dij, ujz = dzj / dij;
                        const double ukx = dxk / dik, uky = dyk / dik, ukz = dzk / dik;
                        const double jx = -dc * (ukx - cosv * ujx) / dij - drj * ujx;
                        const double jy = -dc * (uky - cosv * ujy) / dij - drj * ujy;
                        const double jz = -dc * (ukz - cosv * ujz) / dij - drj * ujz;
                        const double kx = -dc * (ujx - cosv * ukx) / dik - drk * ukx;
                        const double ky = -dc * (ujy - cosv * uky) / dik - drk * uky;
                        const double kz = -dc * (ujz - cosv * ukz) / dik - drk * ukz;
                        GX[gi] += (REAL)(-(jx + kx)); GY[gi] += (REAL)(-(jy + ky)); GZ[gi] += (REAL)(-(jz + kz));
                        GX[gj] += (REAL)jx; GY[gj] += (REAL)jy; GZ[gj] += (REAL)jz;
                        GX[gk] += (REAL)kx; GY[gk] += (REAL)ky; GZ[gk] += (REAL)kz;
                    }
                }
            }
        }
    }
}

/* featurize_grad_inverse, gpu_featurizer/kernel_cpu.cpp:37-179: the product of the
 * feature Jacobian with a coordinate-space vector v, accumulated into the per-element
 * feature buffers (pre-zeroed, gpu_featurizer/functor_op_cpu.cpp:107-110).
 *
 * mode 0: the mathematically correct J v (v indexed by the atom whose coordinate moves).
 * mode 1: bit-for-behaviour restatement of the reference, which reads the vector at the
 *         ELEMENT ID of the central atom for all three atoms of a term
 *         (X_grads[g_atomic_num_i], kernel_cpu.cpp:111,118,155,162,169).  Because the
 *         derivatives with respect to i, j and k of any term sum to zero, that makes
 *         every output vanish up to rounding. */
void FN(oracle_featurize_grad_inverse)(const REAL *X, const REAL *Y, const REAL *Z, const int *A,
                                       const int *mol_offsets, const int *mol_counts, int n_mols,
                                       const int *scatter, const REAL *VX, const REAL *VY,
                                       const REAL *VZ, REAL *oH, REAL *oC, REAL *oN, REAL *oO,
                                       int mode)
{
    for (int m = 0; m < n_mols; m++) {
        const int n = mol_counts[m];
        const int base = mol_offsets[m];
        for (int ii = 0; ii < n; ii++) {
            const int gi = base + ii;
            const int ti = A[gi];
            const double ix = X[gi], iy = Y[gi], iz = Z[gi];
            REAL *row_i = FN(row_ptr)(ti, oH, oC, oN, oO) + (size_t)scatter[gi] * ANI_TOTAL;
            REAL *out_rad = row_i;
            REAL *out_ang = row_i + ANI_RADIAL;
            const int vi = mode ? ti : gi;
            for (int jj = 0; jj < n; jj++) {
                const int gj = base + jj;
                const int tj = A[gj];
                const int vj = mode ? ti : gj;
                const double dxj = (REAL)(ix - X[gj]), dyj = (REAL)(iy - Y[gj]), dzj = (REAL)(iz - Z[gj]);
                const REAL rij_t = (REAL)oracle_dist(dxj, dyj, dzj);
                const double rij = rij_t;

                if (rij_t < kR_Rc && ii != jj) { /* kernel_cpu.cpp:105 */
                    const double Rc = (double)kR_Rc;
                    const double fc = 0.5 * cos(M_PI * rij / Rc) + 0.5;
                    const double dfc = -0.5 * M_PI * sin(M_PI * rij / Rc) / Rc;
                    for (int r = 0; r < ANI_NUM_R_RS; r++) {
                        const double dr = rij - (double)kR_Rs[r];
                        const double e = exp(-(double)kR_eta * dr * dr);
                        const double dterm = e * (-2.0 * (double)kR_eta * dr * fc + dfc);
                        const double ax = dterm * dxj / rij, ay = dterm * dyj / rij, az = dterm * dzj / rij;
                        out_rad[tj * ANI_NUM_R_RS + r] +=
                            (REAL)(ax * (double)VX[vi] + ay * (double)VY[vi] + az * (double)VZ[vi]);
                        out_rad[tj * ANI_NUM_R_RS + r] +=
                            (REAL)(-ax * (double)VX[vj] - ay * (double)VY[vj] - az * (double)VZ[vj]);
                    }
                }

                if (rij_t < kA_Rc) { /* kernel_cpu.cpp:123 */
                    for (int kk = jj + 1; kk < n; kk++) {
                        if (ii == jj || ii == kk || jj == kk) continue;
                        const int gk = base + kk;
                        const int tk = A[gk];
                        const int vk = mode ? ti : gk;
                        const double dxk = (REAL)(ix - X[gk]), dyk = (REAL)(iy - Y[gk]), dzk = (REAL)(iz - Z[gk]);
                        const REAL rik_t = (REAL)oracle_dist(dxk, dyk, dzk);
                        if (!(rik_t < kA_Rc)) continue;
                        const double dij = sqrt(dxj * dxj + dyj * dyj + dzj * dzj);
                        const double dik = sqrt(dxk * dxk + dyk * dyk + dzk * dzk);
                        const double cosv = (dxj * dxk + dyj * dyk + dzj * dzk) / (dij * dik);
                        const double ujx = dxj / dij, ujy = dyj / dij, ujz = dzj / dij;
                        const double ukx = dxk / dik, uky = dyk / dik, ukz = dzk / dik;
                        /* directional derivatives of cos(theta), r_ij, r_ik along v */
                        const double cjx = -(ukx - cosv * ujx) / dij, cjy = -(uky - cosv * ujy) / dij,
                                     cjz = -(ukz - cosv * ujz) / dij;
                        const double ckx = -(ujx - cosv * ukx) / dik, cky = -(ujy - cosv * uky) / dik,
                                     ckz = -(ujz - cosv * ukz) / dik;
                        const double dcos =
                            cjx * ((double)VX[vj] - (double)VX[vi]) + cjy * ((double)VY[vj] - (double)VY[vi]) +
                            cjz * ((double)VZ[vj] - (double)VZ[vi]) +
                            ckx * ((double)VX[vk] - (double)VX[vi]) + cky * ((double)VY[vk] - (double)VY[vi]) +
                            ckz * ((double)VZ[vk] - (double)VZ[vi]);
                        const double drij = ujx * ((double)VX[vi] - (double)VX[vj]) +
                                            ujy * ((double)VY[vi] - (double)VY[vj]) +
                                            ujz * ((double)VZ[vi] - (double)VZ[vj]);
                        const double drik = ukx * ((double)VX[vi] - (double)VX[vk]) +
                                            uky * ((double)VY[vi] - (double)VY[vk]) +
                                            ukz * ((double)VZ[vi] - (double)VZ[vk]);
                        double pc[32], pj[32], pk[32];
                        FN(triplet_partials)(dij, dik, cosv, pc, pj, pk);
                        for (int t = 0; t < ANI_NUM_A_THETAS; t++)
                            for (int s = 0; s < ANI_NUM_A_RS; s++) {
                                const int q = t * ANI_NUM_A_RS + s;
                                out_ang[oracle_linearize(tj, tk, t, s)] +=
                                    (REAL)(pc[q] * dcos + pj[q] * drij + pk[q] * drik);
                            }
                    }
                }
            }
        }
    }
}

/*
 * AniCharge, gpu_featurizer/ani_charges.cpp:58-71 (charge_energy) and :100-113 (the loop
 * over molecules): damped Coulomb energy of every molecule,
 *   E_m = sum_{i<j} k_e q_i q_j (1 - f_C(r_ij, R_Rc)) / r_ij .
 * Types follow the C++ expression: k_e is `const float` (parameters.h:10), so
 * k_e*q_i*q_j is evaluated in NumericType; (1 - f_C) is double, so the product, the
 * division and the addition to the NumericType accumulator run in double and are rounded
 * once per pair.  PARITY UNPINNED for the energy values: the reference has no golden numbers
 * for this op (its tests check only the gradient against finite differences,
 * gpu_featurizer/test_kernel.py:412-447, which tests/test_oracle_charge.py repeats here).
 */
void FN(oracle_charge)(const REAL *X, const REAL *Y, const REAL *Z, const REAL *Q,
                       const int *mol_offsets, const int *mol_counts, int n_mols, REAL *energies)
{
    for (int m = 0; m < n_mols; m++) {
        const int n = mol_counts[m], base = mol_offsets[m];
        REAL energy = 0;
        for (int i = 0; i < n; i++)
            for (int j = i + 1; j < n; j++) {
                const REAL dx = X[base + i] - X[base + j];
                const REAL dy = Y[base + i] - Y[base + j];
                const REAL dz = Z[base + i] - Z[base + j];
                const REAL r = (REAL)oracle_dist(dx, dy, dz);
                const REAL qq = (REAL)(kChargeConstant * Q[base + i]) * Q[base + j];
                energy = (REAL)((double)energy + (double)qq * (1 - oracle_fc(r, kR_Rc)) / (double)r);
            }
        energies[m] = energy;
    }
}

/*
 * AniChargeGrad, gpu_featurizer/ani_charges.cpp:138-160 (charge_grads) and :196-214:
 * q_grads = dL/dq given dL/dE_m per molecule; q_grads is zero-filled first (:194).
 * Atom i collects its j > i terms in a local NumericType accumulator that is added to
 * q_grads[i] afterwards; atom j's share is added to q_grads[j] directly.
 */
void FN(oracle_charge_grad)(const REAL *X, const REAL *Y, const REAL *Z, const REAL *Q,
                            const int *mol_offsets, const int *mol_counts, int n_mols, int n_atoms,
                            const REAL *energy_grads, REAL *q_grads)
{
    memset(q_grads, 0, (size_t)n_atoms * sizeof(REAL));
    for (int m = 0; m < n_mols; m++) {
        const int n = mol_counts[m], base = mol_offsets[m];
        const REAL g = energy_grads[m];
        for (int i = 0; i < n; i++) {
            REAL gi = 0;
            for (int j = i + 1; j < n; j++) {
                const REAL dx = X[base + i] - X[base + j];
                const REAL dy = Y[base + i] - Y[base + j];
                const REAL dz = Z[base + i] - Z[base + j];
                const REAL r = (REAL)oracle_dist(dx, dy, dz);
                const double damp = (1 - oracle_fc(r, kR_Rc)) / (double)r;
                const REAL kj = (REAL)((REAL)(g * kChargeConstant) * Q[base + j]);
                const REAL ki = (REAL)((REAL)(g * kChargeConstant) * Q[base + i]);
                gi = (REAL)((double)gi + (double)kj * damp);
                q_grads[base + j] = (REAL)((double)q_grads[base + j] + (double)ki * damp);
            }
            q_grads[base + i] += gi;
        }
    }
}

#undef FN
#undef CAT
#undef CAT_
