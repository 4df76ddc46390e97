// Per-element atomic network 384-128-128-64-1, backward pass along the activations, fused into
// one kernel on the Blackwell tensor cores (same machinery as ani_mlp.cuh).
//
// Given g = dL/dE per atom and the activation derivatives D1, D2, D3 that the forward kernel
// saved, a CTA computes for its tile of 128 atoms of one element
//   dZ3 = (g w4^T) * D3                       (registers, thread = atom)
//   dZ2 = (dZ3 W3^T) * D2                     (MMA  M=128 N=128 K=64)
//   dZ1 = (dZ2 W2^T) * D1                     (MMA  M=128 N=128 K=128)
//   dF  =  dZ1 W1^T                           (MMA  M=128 N=3x128 K=128)
// and writes dZ1, dZ2, dZ3 (what the weight gradients A_{l-1}^T dZ_l need; those are plain
// GEMMs over all atoms of the element and are left to the caller) and dF = dL/d(features), the
// upstream of featurize_grad.  This is the part of the reference's tf.gradients through
// MoleculeNN (khan/model/nn.py:39-67,165-172; khan/training/trainer_multi_tower.py:350-419)
// that feeds the coordinate gradients.
//
// The weights are read in the reference's own layout W = [in][out]: for dA = dZ W^T the MMA's
// B operand is [N = in][K = out], which is W as stored.
#pragma once

#include "ani_mlp_pipe.cuh"

namespace ani {

struct MlpBackwardParams {
    const float* grad_energy[kTypes];   // [count]
    int count[kTypes];
    int tile_start[kTypes + 1];
    const float* w1[kTypes];     // [384][128]
    const float* w2[kTypes];     // [128][128]
    const float* w3[kTypes];     // [128][64]
    const float* w4[kTypes];     // [64]
    const float* dact1[kTypes];  // [count][128]
    const float* dact2[kTypes];  // [count][128]
    const float* dact3[kTypes];  // [count][64]
    float* dz1[kTypes];          // [count][128]
    float* dz2[kTypes];          // [count][128]
    float* dz3[kTypes];          // [count][64]
    float* grad_feat[kTypes];    // optional [count][384]
    const unsigned char* packed[kTypes];   // optional: the weights pre-packed by mlp_pack_kernel
};

template <bool SPLIT>
__global__ void __launch_bounds__(kMlpAllThreads, 1) mlp_backward_kernel(const MlpBackwardParams p)
{
    extern __shared__ unsigned char mlp_smem_raw[];
    MlpShared& sh = *reinterpret_cast<MlpShared*>(
        (reinterpret_cast<uintptr_t>(mlp_smem_raw) + 1023) & ~(uintptr_t)1023);
    const int tid = threadIdx.x, warp = tid >> 5;
    // this thread's accumulator row (TMEM lane = atom of the tile) and group of 32 columns
    const int erow = (warp & 3) * 32 + (tid & 31), ecg = warp >> 2;

    int e = 0;
#pragma unroll
    for (int t = 1; t < kTypes; t++) e += (int)blockIdx.x >= p.tile_start[t] ? 1 : 0;
    const int row0 = ((int)blockIdx.x - p.tile_start[e]) * kMlpTile;
    const int n_rows = min(kMlpTile, p.count[e] - row0);
    const bool live = erow < n_rows;
    const size_t atom = (size_t)(row0 + erow);

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
    const int step_k[2] = {kMlpH3, kMlpH2};
    const bool want_feat = p.grad_feat[e] != nullptr;

    if (warp == kMlpThreads / 32) {
        // ---- the MMA warp: the two products of the chain, then three for the feature gradient ----
        IssueState is;
        pipe_issue<SPLIT>(sh, tmem, 128, step_k[0] / kPipeK, true, is);
        pipe_issue<SPLIT>(sh, tmem, 128, step_k[1] / kPipeK, true, is);
        if (want_feat)
            for (int n0 = 0; n0 < kMlpIn; n0 += 128) pipe_issue<SPLIT>(sh, tmem, 128, kMlpH1 / kPipeK, true, is);
    } else {
        // ---- producers / epilogue warps ----
        const unsigned lane_addr = tmem + ((unsigned)((warp & 3) * 32) << 16);
        PipeState ps;
        const DirectShared<SPLIT> a_sh{sh.act};
        const int tile_row0 = (warp & 3) * 32;          // first row of this warp's 32 x 32 tiles
        const int tile_rows = n_rows - tile_row0;        // how many of them exist (may be <= 0)
        const size_t tile_atom0 = (size_t)(row0 + tile_row0);
        const int c0 = ecg * 32;
        float* scratch = warp_scratch(sh);

        // ---- dZ3 = g * w4 * D3 (64 columns: the warps of column groups 0 and 1); rows past the
        // end of the element are zero ----
        if (tid < kMlpH3) sh.vec[tid] = p.w4[e][tid];
        producer_sync();
        if (c0 < kMlpH3) {
            const float g = live ? p.grad_energy[e][atom] : 0.0f;
            float d[32], v[32];
            warp_tile_from_global(scratch, d, p.dact3[e] + tile_atom0 * kMlpH3 + c0, kMlpH3, tile_rows);
#pragma unroll
            for (int i = 0; i < 32; i++) {
                v[i] = g * sh.vec[c0 + i] * d[i];
                sh.act[erow * kMlpActStride + c0 + i] = v[i];
            }
            warp_tile_to_global<false>(scratch, v, p.dz3[e] + tile_atom0 * kMlpH3 + c0, kMlpH3, tile_rows);
        }
        producer_sync();

        // ---- dZ2 = (dZ3 W3^T) * D2 and dZ1 = (dZ2 W2^T) * D1 ----
        const float* step_w[2] = {p.w3[e], p.w2[e]};
        const float* step_d[2] = {p.dact2[e], p.dact1[e]};
        float* step_out[2] = {p.dz2[e], p.dz1[e]};
        bool ok = true;
#pragma unroll 1
        for (int s = 0; s < 2 && ok; s++) {
            // B[n = in][k = out] = W[n][k]: the weights as stored
            DirectGlobal<SPLIT> b_w{step_w[s], (size_t)step_k[s], 128, 128, 0};
            if (p.packed[e]) {
                PackedB b_packed{p.packed[e] + (size_t)(s == 0 ? kPackBwdS0 : kPackBwdS1) * kPackedChunkBytes};
                pipe_produce<SPLIT, true>(sh, step_k[s] / kPipeK, ps, b_w, a_sh, b_packed);
            } else {
                pipe_produce<SPLIT, true>(sh, step_k[s] / kPipeK, ps, b_w, a_sh, b_w);
            }
            ok = pipe_drain(sh, ps);
            if (!ok) break;
            {
                float v[32], d[32];
                tmem_load32(lane_addr + c0, v);
                warp_tile_from_global(scratch, d, step_d[s] + tile_atom0 * 128 + c0, 128, tile_rows);
#pragma unroll
                for (int i = 0; i < 32; i++) {
                    v[i] *= d[i];                      // d is zero on rows past the end
                    sh.act[erow * kMlpActStride + c0 + i] = v[i];
                }
                warp_tile_to_global<false>(scratch, v, step_out[s] + tile_atom0 * 128 + c0, 128, tile_rows);
            }
            tc_fence_before();
            producer_sync();
        }

        // ---- dF = dZ1 W1^T, 128 feature columns at a time ----
        if (ok && want_feat) {
#pragma unroll 1
            for (int n0 = 0; n0 < kMlpIn && ok; n0 += 128) {
                DirectGlobal<SPLIT> b_w{p.w1[e] + (size_t)n0 * kMlpH1, (size_t)kMlpH1, 128, 128, 0};
                if (p.packed[e]) {
                    PackedB b_packed{p.packed[e] + (size_t)(kPackBwdF + 4 * (n0 / 128)) * kPackedChunkBytes};
                    pipe_produce<SPLIT, true>(sh, kMlpH1 / kPipeK, ps, b_w, a_sh, b_packed);
                } else {
                    pipe_produce<SPLIT, true>(sh, kMlpH1 / kPipeK, ps, b_w, a_sh, b_w);
                }
                ok = pipe_drain(sh, ps);
                if (!ok) break;
                float v[32];
                tmem_load32(lane_addr + c0, v);
                warp_tile_to_global<false>(scratch, v, p.grad_feat[e] + tile_atom0 * kMlpIn + n0 + c0, kMlpIn, tile_rows);
                tc_fence_before();
                producer_sync();   // the accumulator and the scratch are overwritten by the next product
            }
        }
        if (!ok && tid == 0) report(ANI_ERR_TIMEOUT);
    }
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, kMlpTmemCols);
}

}  // namespace ani
