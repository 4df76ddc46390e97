// Per-element atomic network 384-128-128-64-1, forward pass, one kernel.
//
// What it computes is AtomNN of the reference (khan/model/nn.py:39-67): for the atoms of one
// element, A1 = act(F W1 + b1), A2 = act(A1 W2 + b2), A3 = act(A2 W3 + b3), E = A3 w4 + b4, with
// F the [n, 384] feature rows of that element.  MoleculeNN (khan/model/nn.py:165-172) runs four
// of these, one per element; here one launch covers all four (each CTA takes a tile of 128 atoms
// of one element).  A operand: the feature rows (layer 1) or the previous activations in shared
// memory; B operand: the transpose of the weights as stored ([in][out]).  The epilogue adds the
// bias, applies the activation, keeps the row in shared memory for the next layer and saves the
// activation and its derivative for the backward pass; the last layer (64 -> 1) is a dot product
// per atom from shared memory.
#pragma once

#include "ani_mlp_pipe.cuh"

namespace ani {

template <int ACT, bool SPLIT>
__global__ void __launch_bounds__(kMlpAllThreads, 1) mlp_forward_kernel(const MlpParams p)
{
    extern __shared__ unsigned char mlp_smem_raw[];
    // the launch asks for sizeof(MlpShared) + 1024 bytes so that the struct can be aligned here
    MlpShared& sh = *reinterpret_cast<MlpShared*>(
        (reinterpret_cast<uintptr_t>(mlp_smem_raw) + 1023) & ~(uintptr_t)1023);
    const int tid = threadIdx.x, warp = tid >> 5;
    // epilogue role of this thread: one accumulator row (TMEM lane), one group of 32 columns
    const int erow = (warp & 3) * 32 + (tid & 31), ecg = warp >> 2;

    int e = 0;
#pragma unroll
    for (int t = 1; t < kTypes; t++) e += (int)blockIdx.x >= p.tile_start[t] ? 1 : 0;
    const int row0 = ((int)blockIdx.x - p.tile_start[e]) * kMlpTile;
    const int n_rows = min(kMlpTile, p.count[e] - row0);

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
    const int layer_k[3] = {kMlpIn, kMlpH1, kMlpH2};
    const int layer_n[3] = {kMlpH1, kMlpH2, kMlpH3};

    if (warp == kMlpThreads / 32) {
        // ---- the MMA warp: one product per layer ----
        IssueState is;
#pragma unroll 1
        for (int layer = 0; layer < 3; layer++) pipe_issue<SPLIT>(sh, tmem, layer_n[layer], layer_k[layer] / kPipeK, true, is);
    } else {
        // ---- producers / epilogue warps ----
        PipeState ps;
        const float* layer_w[3] = {p.w1[e], p.w2[e], p.w3[e]};
        const float* layer_b[3] = {p.b1[e], p.b2[e], p.b3[e]};
        float* layer_out[3] = {p.act1[e], p.act2[e], p.act3[e]};
        float* layer_dout[3] = {p.dact1[e], p.dact2[e], p.dact3[e]};
        const DirectShared<SPLIT> a_sh{sh.act};
        bool ok = true;

#pragma unroll 1
        for (int layer = 0; layer < 3 && ok; layer++) {
            const int K = layer_k[layer], N = layer_n[layer];
            if (tid < N) sh.vec[tid] = layer_b[layer][tid];   // read in the epilogue, after the drain barrier
            DirectGlobal<SPLIT> a_feat{p.feat[e] + (size_t)row0 * kMlpIn, (size_t)kMlpIn, kMlpTile, n_rows, 0};
            // B[n = out][k = in] = W[k][n]: the weights are read as stored ([in][out]) and transposed
            Transposed<SPLIT> b_w{layer_w[layer], (size_t)N, 0, N, 0, K, make_float4(0.f, 0.f, 0.f, 0.f)};
            if (p.packed[e]) {      // pre-packed weights: one bulk copy per chunk instead of staging
                const int first_chunk = layer == 0 ? kPackFwdL1 : (layer == 1 ? kPackFwdL2 : kPackFwdL3);
                PackedB b_packed{p.packed[e] + (size_t)first_chunk * kPackedChunkBytes};
                if (layer == 0) pipe_produce<SPLIT, false>(sh, K / kPipeK, ps, a_feat, a_sh, b_packed);
                else pipe_produce<SPLIT, true>(sh, K / kPipeK, ps, a_feat, a_sh, b_packed);
            } else if (layer == 0) {
                pipe_produce<SPLIT, false>(sh, K / kPipeK, ps, a_feat, a_sh, b_w);
            } else {
                pipe_produce<SPLIT, true>(sh, K / kPipeK, ps, a_feat, a_sh, b_w);
            }
            ok = pipe_drain(sh, ps);
            if (!ok) break;
            // ---- epilogue: bias, activation and its derivative; the row goes back to shared
            // memory as the next layer's A operand (the last hidden layer included: the output
            // layer reads it from there) ----
            const int c0 = ecg * 32;
            if (c0 < N) {
                float v[32], d[32];
                tmem_load32(tmem + ((unsigned)((warp & 3) * 32) << 16) + c0, v);
#pragma unroll
                for (int i = 0; i < 32; i++) {
                    const float x = v[i] + sh.vec[c0 + i];
                    v[i] = mlp_activation<ACT>(x);
                    d[i] = mlp_activation_grad<ACT>(x, v[i]);
                    sh.act[erow * kMlpActStride + c0 + i] = v[i];
                }
                const int tile_row0 = (warp & 3) * 32;
                const size_t g0 = (size_t)(row0 + tile_row0) * N + c0;
                float* scratch = warp_scratch(sh);
                if (layer_out[layer]) warp_tile_to_global<false>(scratch, v, layer_out[layer] + g0, N, n_rows - tile_row0);
                if (layer_dout[layer]) warp_tile_to_global<false>(scratch, d, layer_dout[layer] + g0, N, n_rows - tile_row0);
            }
            tc_fence_before();
            producer_sync();
        }

        if (ok) {
            // ---- output layer 64 -> 1: one thread per atom, its last hidden row from shared memory ----
            if (tid < kMlpH3) sh.vec[tid] = p.w4[e][tid];
            producer_sync();
            if (tid < n_rows) {
                float acc = p.b4[e][0];
#pragma unroll 8
                for (int i = 0; i < kMlpH3; i++) acc += sh.act[tid * kMlpActStride + i] * sh.vec[i];
                p.energy[e][row0 + tid] = acc;
            }
        } else if (tid == 0) {
            report(ANI_ERR_TIMEOUT);
        }
    }
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, kMlpTmemCols);
}

}  // namespace ani
