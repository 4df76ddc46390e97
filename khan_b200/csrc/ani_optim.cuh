// One optimiser step over ALL weights as two launches on a flat parameter buffer.
//
// The reference applies, per step (khan/training/trainer_multi_tower.py:421-427):
//   grads <- clip_by_global_norm(grads, 5)            scale = c / max(||g||, c)
//   NadamOptimizer (Adam with Nesterov momentum):      m <- b1 m + (1-b1) g,  v <- b2 v + (1-b2) g^2,
//       w <- w - lr sqrt(1-b2^t)/(1-b1^t) * (b1 m + (1-b1) g) / (sqrt(v) + eps)
//   ExponentialMovingAverage(0.9999, global_step):     s <- s - (1-d)(s - w),  d = min(0.9999, (1+t)/(10+t))
// as ~150 small TensorFlow ops over 32 variables.  With the 296,452 weights in one buffer this
// is a sum of squares (launch 1) and one elementwise pass (launch 2); hyper-parameters and the
// step counter live in device memory so that the two launches can sit in a CUDA graph.
#pragma once

#include "ani_common.cuh"

namespace ani {

struct OptimState {     // 32 bytes of device memory, zero-initialised by the caller
    int step;           // updates applied so far
    unsigned blocks_done;
    float norm2[2];     // sum of squared gradients; slot (step & 1) is the one in use
    int pad[4];
};

struct OptimHyper {     // device memory, written by the host when a value changes
    float lr, beta1, beta2, eps, clip_norm, ema_decay;
};

constexpr int kOptimThreads = 256;

__global__ void __launch_bounds__(kOptimThreads)
    grad_sumsq_kernel(const float* __restrict__ g, long long n, OptimState* __restrict__ st)
{
    __shared__ float warp_sums[kOptimThreads / kWarp];
    float acc = 0.0f;
    const long long stride = (long long)gridDim.x * blockDim.x;
    const long long n4 = n >> 2;
    const float4* g4 = reinterpret_cast<const float4*>(g);
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += stride) {
        const float4 q = g4[i];
        acc += q.x * q.x + q.y * q.y + q.z * q.z + q.w * q.w;
    }
    for (long long i = (n4 << 2) + (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride)
        acc += g[i] * g[i];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(kFull, acc, o);
    if (lane_id() == 0) warp_sums[warp_id()] = acc;
    __syncthreads();
    if (warp_id() == 0) {
        acc = lane_id() < kOptimThreads / kWarp ? warp_sums[lane_id()] : 0.0f;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(kFull, acc, o);
        if (lane_id() == 0) atomicAdd(&st->norm2[st->step & 1], acc);
    }
}

__global__ void __launch_bounds__(kOptimThreads)
    nadam_update_kernel(float* __restrict__ w, const float* __restrict__ g, float* __restrict__ m,
                        float* __restrict__ v, float* __restrict__ ema, long long n,
                        const OptimHyper* __restrict__ hyper, OptimState* __restrict__ st)
{
    const OptimHyper h = *hyper;
    const int step = st->step;
    const float t = (float)(step + 1);
    const float norm = sqrtf(st->norm2[step & 1]);
    const float scale = h.clip_norm > 0.0f ? h.clip_norm / fmaxf(norm, h.clip_norm) : 1.0f;
    const float lr_t = h.lr * sqrtf(1.0f - powf(h.beta2, t)) / (1.0f - powf(h.beta1, t));
    const float decay = fminf(h.ema_decay, (1.0f + t) / (10.0f + t));
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += stride) {
        const float gi = g[i] * scale;
        const float mi = h.beta1 * m[i] + (1.0f - h.beta1) * gi;
        const float vi = h.beta2 * v[i] + (1.0f - h.beta2) * gi * gi;
        const float wi = w[i] - lr_t * (h.beta1 * mi + (1.0f - h.beta1) * gi) / (sqrtf(vi) + h.eps);
        m[i] = mi;
        v[i] = vi;
        w[i] = wi;
        if (ema) ema[i] -= (1.0f - decay) * (ema[i] - wi);
    }
    // the last block to finish advances the step and clears the slot the next step will use
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        if (atomicAdd(&st->blocks_done, 1u) == gridDim.x - 1) {
            st->norm2[(step + 1) & 1] = 0.0f;
            st->blocks_done = 0;
            __threadfence();
            st->step = step + 1;
        }
    }
}

// Max-norm constraint on the rows of the weight matrices: every row whose Euclidean norm
// exceeds max_norm is scaled back onto the sphere -- tf.clip_by_norm(w, 3.0, axes=1) over all
// weight matrices (khan/training/trainer_multi_tower.py:432-436), one launch over a row table
// instead of five small ops per matrix.  One warp per row.
__global__ void __launch_bounds__(kOptimThreads)
    clip_rows_kernel(float* __restrict__ w, const int* __restrict__ row_offsets, const int* __restrict__ row_lengths,
                     int n_rows, float max_norm)
{
    const int lane = lane_id();
    const int warps = gridDim.x * (kOptimThreads / kWarp);
    for (int r = blockIdx.x * (kOptimThreads / kWarp) + warp_id(); r < n_rows; r += warps) {
        float* row = w + row_offsets[r];
        const int len = row_lengths[r];
        float acc = 0.0f;
        for (int i = lane; i < len; i += kWarp) acc += row[i] * row[i];
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(kFull, acc, o);
        const float norm = sqrtf(acc);
        if (norm > max_norm) {
            const float scale = max_norm / norm;
            for (int i = lane; i < len; i += kWarp) row[i] *= scale;
        }
    }
}

// Gradient of the reference's training losses from the gradient of the mean squared error: with
// mse = mean(l2s) and rmse = sqrt(mse), d rmse = d mse / (2 rmse) and d exp(rmse) = exp(rmse) d mse / (2 rmse)
// (khan/training/trainer_multi_tower.py:390-396 minimises exp(rmse)).  Every block forms the mean of the
// n_mols squared errors itself (the same order in every block, so the same factor) and scales its part of
// the gradient buffer; block 0 also writes the rmse.  kind: 1 = rmse, 2 = exp(rmse).
__global__ void __launch_bounds__(kOptimThreads)
    loss_scale_kernel(float* __restrict__ grads, long long n, const float* __restrict__ l2s, int n_mols, int kind,
                      float* __restrict__ rmse_out)
{
    __shared__ float warp_sums[kOptimThreads / kWarp];
    __shared__ float factor_sh;
    float acc = 0.0f;
    for (int i = threadIdx.x; i < n_mols; i += kOptimThreads) acc += l2s[i];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) acc += __shfl_xor_sync(kFull, acc, o);
    if (lane_id() == 0) warp_sums[warp_id()] = acc;
    __syncthreads();
    if (threadIdx.x == 0) {
        float total = 0.0f;
        for (int w = 0; w < kOptimThreads / kWarp; w++) total += warp_sums[w];
        const float rmse = fmaxf(sqrtf(total / (float)max(n_mols, 1)), 1e-30f);
        factor_sh = (kind == 2 ? expf(rmse) : 1.0f) / (2.0f * rmse);
        if (blockIdx.x == 0 && rmse_out) *rmse_out = rmse;
    }
    __syncthreads();
    const float f = factor_sh;
    for (long long i = (long long)blockIdx.x * kOptimThreads + threadIdx.x; i < n; i += (long long)gridDim.x * kOptimThreads)
        grads[i] *= f;
}

}  // namespace ani
