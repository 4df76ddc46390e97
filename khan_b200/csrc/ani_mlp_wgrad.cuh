// Weight and bias gradients of the per-element atomic networks on the Blackwell tensor cores:
//   dW1 = F^T dZ1 [384 x 128],  dW2 = A1^T dZ2 [128 x 128],  dW3 = A2^T dZ3 [128 x 64],
//   db_l = column sums of dZ_l,
// products whose long dimension is the ATOM index.  A CTA takes one range of atoms (sized on the
// host so that the whole grid is one wave) of
// one element and one 128-row block of one weight matrix (three blocks for W1, one each for W2
// and W3), accumulates its [128 x N] block in tensor memory over the range, and adds it to the
// output with 16-byte global reductions (the call ADDS to its outputs).  The CTA of the W3 block
// also does the output layer (dw4 = A3^T g, db4 = sum g) with plain loads.
// Both MMA operands are K-major with K = atom, so staging TRANSPOSES the row-major activations:
// a thread reads four consecutive columns of one atom and scatters them to four operand rows.
//
// Same mathematics as the weight part of tf.gradients through AtomNN (khan/model/nn.py:39-67
// under khan/training/trainer_multi_tower.py:396-397).
#pragma once

#include "ani_mlp_pipe.cuh"

namespace ani {

constexpr int kWgradBlocks = 5;    // W1 rows 0-127, 128-255, 256-383; W2; W3 (+ the output layer w4, b4)

struct MlpWgradParams {
    int count[kTypes];
    int range;                     // atoms per CTA, a multiple of 64 chosen so that the grid is one wave
    int range_start[kTypes + 1];   // prefix of ceil(count / range)
    const float* feat[kTypes];     // [count][384]
    const float* act1[kTypes];     // [count][128]
    const float* act2[kTypes];     // [count][128]
    const float* dz1[kTypes];      // [count][128]
    const float* dz2[kTypes];      // [count][128]
    const float* dz3[kTypes];      // [count][64]
    float* dw1[kTypes];            // [384][128]
    float* dw2[kTypes];            // [128][128]
    float* dw3[kTypes];            // [128][64]
    float* db1[kTypes];            // [128]
    float* db2[kTypes];            // [128]
    float* db3[kTypes];            // [64]
    const float* act3[kTypes];     // [count][64]
    const float* grad_energy[kTypes];   // [count]
    float* dw4[kTypes];            // [64]
    float* db4[kTypes];            // [1]
};

template <bool SPLIT>
__global__ void __launch_bounds__(kMlpAllThreads, 1) mlp_wgrad_kernel(const MlpWgradParams p)
{
    extern __shared__ unsigned char mlp_smem_raw[];
    MlpShared& sh = *reinterpret_cast<MlpShared*>(
        (reinterpret_cast<uintptr_t>(mlp_smem_raw) + 1023) & ~(uintptr_t)1023);
    const int tid = threadIdx.x, warp = tid >> 5;

    int e = 0;
#pragma unroll
    for (int t = 1; t < kTypes; t++) e += (int)blockIdx.x >= p.range_start[t] ? 1 : 0;
    const long long first = (long long)((int)blockIdx.x - p.range_start[e]) * p.range;
    const int n_here = (int)min((long long)p.range, (long long)p.count[e] - first);
    const int blk = blockIdx.y;

    // which product this CTA computes
    const float* a_src = blk < 3 ? p.feat[e] : (blk == 3 ? p.act1[e] : p.act2[e]);
    const int a_ld = blk < 3 ? kMlpIn : 128;
    const int a_col0 = blk < 3 ? blk * 128 : 0;
    const float* b_src = blk < 3 ? p.dz1[e] : (blk == 3 ? p.dz2[e] : p.dz3[e]);
    const int N = blk == 4 ? kMlpH3 : 128;
    float* out = blk < 3 ? p.dw1[e] + (size_t)blk * 128 * 128 : (blk == 3 ? p.dw2[e] : p.dw3[e]);
    float* bias_out = blk == 0 ? p.db1[e] : (blk == 3 ? p.db2[e] : (blk == 4 ? p.db3[e] : nullptr));

    if (warp == 0) tmem_alloc(&sh.tmem_base, kMlpTmemCols);
    if (tid == 0) {
        mbar_init(&sh.stage_bar[0], 1);
        mbar_init(&sh.stage_bar[1], 1);
        mbar_init(&sh.full_bar[0], kMlpThreads);
        mbar_init(&sh.full_bar[1], kMlpThreads);
        sh.failed = 0;
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem = sh.tmem_base;
    const int nchunks = (n_here + kPipeK - 1) / kPipeK;
    if (warp == kMlpThreads / 32) {
        IssueState is;
        pipe_issue<SPLIT>(sh, tmem, N, nchunks, true, is);
    } else {
        PipeState ps;
        const DirectShared<SPLIT> unused_sh{sh.act};
        // both operands are transposes with K = atom: A[m = in][k] = X[atom k][in m], B[n = out][k] = dZ[atom k][out n]
        Transposed<SPLIT> a_x{a_src, (size_t)a_ld, a_col0, 128, first, n_here, make_float4(0.f, 0.f, 0.f, 0.f)};
        Transposed<SPLIT> b_dz{b_src, (size_t)N, 0, N, first, n_here, make_float4(0.f, 0.f, 0.f, 0.f)};
        pipe_produce<SPLIT, false>(sh, nchunks, ps, a_x, unused_sh, b_dz);
        const bool ok = pipe_drain(sh, ps);
        const float4 bias_acc = b_dz.colsum;

        if (ok && n_here > 0) {
            // warp w: rows 32 (w % 4) .. of the weight block (TMEM lanes), columns 32 (w / 4) ..
            const int tile_row0 = (warp & 3) * 32, c0 = (warp >> 2) * 32;
            if (c0 < N) {
                float v[32];
                tmem_load32(tmem + ((unsigned)tile_row0 << 16) + c0, v);
                warp_tile_to_global<true>(warp_scratch(sh), v, out + (size_t)tile_row0 * N + c0, N, 32);
            }
            if (bias_out) {
                // this thread summed columns 4q .. 4q+3 of dZ over the atoms it staged
                const int q = transposed_quad(N);
                atomicAdd(bias_out + 4 * q + 0, bias_acc.x);
                atomicAdd(bias_out + 4 * q + 1, bias_acc.y);
                atomicAdd(bias_out + 4 * q + 2, bias_acc.z);
                atomicAdd(bias_out + 4 * q + 3, bias_acc.w);
            }
        } else if (!ok && tid == 0) {
            report(ANI_ERR_TIMEOUT);
        }
        if (blk == 4) {
            // output layer, done by the CTA with the lightest product: dw4 = A3^T g and db4 = sum g
            // over this range; no tensor cores involved
            const int q = tid & 15, a_in = tid >> 4;      // 16 column quads x 32 atoms per pass
            float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
            float gsum = 0.0f;
            for (int k = a_in; k < n_here; k += kMlpThreads / 16) {
                const float g = p.grad_energy[e][first + k];
                const float4 v = *reinterpret_cast<const float4*>(p.act3[e] + (size_t)(first + k) * kMlpH3 + 4 * q);
                acc.x += v.x * g; acc.y += v.y * g; acc.z += v.z * g; acc.w += v.w * g;
                gsum += q == 0 ? g : 0.0f;
            }
            atomicAdd(p.dw4[e] + 4 * q + 0, acc.x);
            atomicAdd(p.dw4[e] + 4 * q + 1, acc.y);
            atomicAdd(p.dw4[e] + 4 * q + 2, acc.z);
            atomicAdd(p.dw4[e] + 4 * q + 3, acc.w);
            if (q == 0) atomicAdd(p.db4[e], gsum);
        }
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, kMlpTmemCols);
}

}  // namespace ani
