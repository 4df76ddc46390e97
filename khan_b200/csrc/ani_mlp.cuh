// Shared pieces of the atomic-network kernels (per-element stacks 384-128-128-64-1 on the
// Blackwell tensor cores: tcgen05.mma kind::tf32, accumulators in tensor memory): parameter
// blocks, the shared-memory layout, PTX wrappers, activations and the epilogue helpers.
// The kernels are in ani_mlp_forward.cuh, ani_mlp_backward.cuh and ani_mlp_wgrad.cuh; the operand
// pipeline they share is in ani_mlp_pipe.cuh.
//
// Common structure of a CTA (512 + 32 threads, tile = 128 rows of the accumulator):
//   * operands are staged by all threads into shared memory in the K-major, no-swizzle
//     core-matrix layout that tcgen05.mma reads (8 rows x 16 bytes per core matrix), 32 values
//     of K per pipeline stage; weights are read in the reference's layout ([in][out]);
//   * a seventeenth warp does nothing but wait for a filled stage, issue its MMAs (M = 128,
//     N = 128 or 64, K = 8 per instruction) and commit them to the stage's mbarrier, so that the
//     producers never stall behind the tensor-core queue; every wait is bounded (on timeout the
//     kernel records an error, frees its tensor memory and returns);
//   * epilogues read the accumulator with tcgen05.ld (warp w: rows 32 (w % 4) .., columns
//     32 (w / 4) ..) and move 32 x 32 tiles to and from global memory through a per-warp
//     transposition scratch, so that every 16-byte access covers whole 128-byte row segments.
// With SPLIT = true every operand is staged as a high part (the value with its low 13 mantissa
// bits cleared, exact in tf32) and a low part (the remainder), and hi*hi + hi*lo + lo*hi are
// accumulated: three MMAs per step give products that are accurate to about 2^-21 instead of
// the 2^-10 of plain tf32.
#pragma once

#include "ani_common.cuh"

namespace ani {

constexpr int kMlpIn = 384, kMlpH1 = 128, kMlpH2 = 128, kMlpH3 = 64;
constexpr int kMlpTile = 128;             // atoms per CTA = MMA M
constexpr int kMlpThreads = 512;          // 16 producer / epilogue warps: warp w reads TMEM lanes 32 (w % 4) .., columns 32 (w / 4) ..
constexpr int kMlpAllThreads = kMlpThreads + 32;   // plus one warp that only issues the MMAs
constexpr int kMlpLbo = 128;              // bytes between core matrices adjacent in K
constexpr int kMlpOperandBytes = 32 * 1024;   // four of these make the 128 KiB operand area
constexpr int kMlpActStride = 129;        // floats per row of the activation buffer (bank-conflict free)
constexpr int kMlpTmemCols = 128;
constexpr unsigned kMlpSpinLimit = 1u << 24;

enum MlpActivation { kActCelu = 0, kActGaussian = 1, kActNormal = 2, kActSoftplus = 3 };

struct MlpParams {
    const float* feat[kTypes];   // [count][384]
    int count[kTypes];
    int tile_start[kTypes + 1];  // prefix of ceil(count / 128)
    const float* w1[kTypes];     // [384][128]  (the reference's layout, [in][out])
    const float* b1[kTypes];
    const float* w2[kTypes];     // [128][128]
    const float* b2[kTypes];
    const float* w3[kTypes];     // [128][64]
    const float* b3[kTypes];
    const float* w4[kTypes];     // [64]
    const float* b4[kTypes];     // [1]
    float* energy[kTypes];       // [count]
    float* act1[kTypes];         // optional [count][128] (saved for the backward pass)
    float* act2[kTypes];         // optional [count][128]
    float* act3[kTypes];         // optional [count][64]
    float* dact1[kTypes];        // optional [count][128]: derivative of the activation at the same place
    float* dact2[kTypes];        // optional [count][128]
    float* dact3[kTypes];        // optional [count][64]
    const unsigned char* packed[kTypes];   // optional: the weights pre-packed by mlp_pack_kernel
};

struct MlpShared {
    alignas(1024) unsigned char a_hi[kMlpOperandBytes];
    alignas(1024) unsigned char b_hi[kMlpOperandBytes];
    alignas(1024) unsigned char a_lo[kMlpOperandBytes];
    alignas(1024) unsigned char b_lo[kMlpOperandBytes];
    float act[kMlpTile * kMlpActStride];
    float vec[128];      // the layer's bias (forward) or the output weights w4 (backward)
    alignas(8) unsigned long long stage_bar[2];   // per operand stage: the MMAs that read it have finished
    alignas(8) unsigned long long full_bar[2];    // per operand stage: all 512 producers have filled it
    unsigned tmem_base;
    int failed;
};

// ------------------------------------------------------------------ PTX wrappers
__device__ __forceinline__ unsigned smem_u32(const void* p)
{
    return (unsigned)__cvta_generic_to_shared(p);
}
__device__ __forceinline__ void mbar_init(unsigned long long* bar, unsigned count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
}
// Bounded wait for the phase with the given parity; false on timeout.
__device__ __forceinline__ bool mbar_wait(unsigned long long* bar, unsigned parity)
{
    const unsigned addr = smem_u32(bar);
    for (unsigned spin = 0; spin < kMlpSpinLimit; spin++) {
        unsigned done;
        asm volatile(
            "{\n"
            ".reg .pred p;\n"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n"
            "selp.u32 %0, 1, 0, p;\n"
            "}\n"
            : "=r"(done)
            : "r"(addr), "r"(parity)
            : "memory");
        if (done) return true;
    }
    return false;
}
// Adds `bytes` to the transaction count that the current phase of the barrier waits for.
__device__ __forceinline__ void mbar_expect_tx(unsigned long long* bar, unsigned bytes)
{
    asm volatile("mbarrier.expect_tx.relaxed.cta.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// Bulk asynchronous copy (TMA, untiled) global -> shared memory; completion is reported to the
// barrier as `bytes` of its transaction count.  Addresses 16-byte aligned, size a multiple of 16.
__device__ __forceinline__ void bulk_copy_to_shared(void* dst_smem, const void* src_global, unsigned bytes,
                                                    unsigned long long* bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                     smem_u32(dst_smem)),
                 "l"(src_global), "r"(bytes), "r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void mbar_arrive(unsigned long long* bar)
{
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// Barrier among the 512 producer / epilogue threads only (the MMA warp does not take part).
__device__ __forceinline__ void producer_sync() { asm volatile("bar.sync 1, 512;" ::: "memory"); }
__device__ __forceinline__ void tmem_alloc(unsigned* dst_smem, unsigned cols)
{
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(dst_smem)),
                 "r"(cols)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(unsigned taddr, unsigned cols)
{
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void fence_async_smem()
{
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// Instruction descriptor for kind::tf32: D = f32, A = B = tf32, both K-major, M x N.
__device__ __forceinline__ unsigned instr_desc(int m, int n)
{
    return (1u << 4) | (2u << 7) | (2u << 10) | ((unsigned)(n >> 3) << 17) | ((unsigned)(m >> 4) << 24);
}
__device__ __forceinline__ void mma_tf32(unsigned d_tmem, unsigned long long a_desc, unsigned long long b_desc,
                                         unsigned idesc, bool accumulate)
{
    asm volatile(
        "{\n"
        ".reg .pred p;\n"
        "setp.ne.u32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, {%5, %6, %7, %8}, p;\n"
        "}\n" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"((unsigned)accumulate), "r"(0u), "r"(0u), "r"(0u), "r"(0u)
        : "memory");
}
__device__ __forceinline__ void mma_commit(unsigned long long* bar)
{
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}
// 32 consecutive accumulator columns of this thread's row (TMEM lane).
__device__ __forceinline__ void tmem_load32(unsigned taddr, float* v)
{
    unsigned r[32];
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]),
          "=r"(r[16]), "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]),
          "=r"(r[24]), "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
    for (int i = 0; i < 32; i++) v[i] = __uint_as_float(r[i]);
}

template <int ACT> __device__ __forceinline__ float mlp_activation(float x)
{
    if (ACT == kActCelu) return x >= 0.0f ? x : 0.1f * (expf(x * 10.0f) - 1.0f);   // activations.py:62-65
    if (ACT == kActGaussian) return expf(-x * x);                                  // activations.py:70-71
    if (ACT == kActNormal) return expf(-0.5f * x * x);                             // activations.py:67-68
    return (x > 20.0f ? x : log1pf(expf(x))) - 0.69314718056f;                      // activations.py:73-74
}

// d act / d x from the pre-activation x and the activation value a = act(x).
template <int ACT> __device__ __forceinline__ float mlp_activation_grad(float x, float a)
{
    if (ACT == kActCelu) return x >= 0.0f ? 1.0f : a * 10.0f + 1.0f;   // exp(x / 0.1)
    if (ACT == kActGaussian) return -2.0f * x * a;
    if (ACT == kActNormal) return -x * a;
    return 1.0f / (1.0f + expf(-x));
}

// Per-warp transposition scratch for the epilogues: 32 x 33 floats per warp, carved out of the
// operand buffers, which are idle while an epilogue runs (the MMAs that read them have finished
// and the next staging pass rewrites them).  a_hi, b_hi and a_lo are contiguous (96 KiB).
constexpr int kMlpScratchStride = 33;
__device__ __forceinline__ float* warp_scratch(MlpShared& sh)
{
    return reinterpret_cast<float*>(sh.a_hi) + (threadIdx.x >> 5) * (32 * kMlpScratchStride);
}

// A 32 x 32 tile that the warp holds as "lane = row, v[32] = columns" goes to global memory
// (row stride ld) with every 16-byte store instruction covering whole 128-byte row segments
// (4 rows x 8 lanes), instead of 32 different rows per instruction.  ADD = true adds with
// 16-byte reductions.  Rows >= rows_valid are skipped.
template <bool ADD>
__device__ __forceinline__ void warp_tile_to_global(float* scratch, const float* v, float* gbase, size_t ld,
                                                    int rows_valid)
{
    const int lane = threadIdx.x & 31;
#pragma unroll
    for (int i = 0; i < 32; i++) scratch[lane * kMlpScratchStride + i] = v[i];
    __syncwarp();
    const int sub = lane >> 3, c = 4 * (lane & 7);
#pragma unroll
    for (int r = 0; r < 32; r += 4) {
        const int rr = r + sub;
        const float* s = scratch + rr * kMlpScratchStride + c;
        const float4 q = make_float4(s[0], s[1], s[2], s[3]);
        if (rr < rows_valid) {
            float4* dst = reinterpret_cast<float4*>(gbase + (size_t)rr * ld + c);
            if (ADD) atomicAdd(dst, q); else *dst = q;
        }
    }
    __syncwarp();
}

// The inverse: a 32 x 32 tile of global memory into "lane = row, v[32] = columns"; rows past
// rows_valid read as zero.
__device__ __forceinline__ void warp_tile_from_global(float* scratch, float* v, const float* gbase, size_t ld,
                                                      int rows_valid)
{
    const int lane = threadIdx.x & 31;
    const int sub = lane >> 3, c = 4 * (lane & 7);
#pragma unroll
    for (int r = 0; r < 32; r += 4) {
        const int rr = r + sub;
        float4 q = make_float4(0.f, 0.f, 0.f, 0.f);
        if (rr < rows_valid) q = *reinterpret_cast<const float4*>(gbase + (size_t)rr * ld + c);
        float* s = scratch + rr * kMlpScratchStride + c;
        s[0] = q.x; s[1] = q.y; s[2] = q.z; s[3] = q.w;
    }
    __syncwarp();
#pragma unroll
    for (int i = 0; i < 32; i++) v[i] = scratch[lane * kMlpScratchStride + i];
    __syncwarp();
}

}  // namespace ani
