// Per-element atomic network 384-128-128-64-1, forward pass, fused into one kernel on the
// Blackwell tensor cores (tcgen05.mma, kind::tf32, accumulators in tensor memory).
//
// What it computes is AtomNN of the reference (khan/model/nn.py:39-67): for the atoms of one
// element, A1 = act(F W1 + b1), A2 = act(A1 W2 + b2), A3 = act(A2 W3 + b3), E = A3 w4 + b4, with
// F the [n, 384] feature rows of that element.  MoleculeNN (khan/model/nn.py:165-172) runs four
// of these, one per element; here one launch covers all four (each CTA takes a tile of 128 atoms
// of one element).
//
// Structure of one CTA (512 threads, tile = 128 atoms):
//   * operands are staged by all threads into shared memory in the K-major, no-swizzle
//     core-matrix layout that tcgen05.mma reads (8 rows x 16 bytes per core matrix), 64 values
//     of K at a time; weights are read in the reference's layout ([in][out]) and transposed
//     while they are staged;
//   * one thread issues the MMAs (M = 128, N = 128 or 64, K = 8 per instruction) and commits them
//     to an mbarrier; everybody waits on it (bounded spin: on timeout the kernel records an
//     error, frees its tensor memory and returns);
//   * the epilogue reads the accumulator with tcgen05.ld (warp w: rows 32 (w % 4) .., columns
//     32 (w / 4) ..), adds the bias, applies the activation and writes the values to shared
//     memory, where they become the A operand of the next layer; the last layer (64 -> 1) is a
//     dot product per atom from shared memory.
// With SPLIT = true every operand is staged as a high part (the value with its low 13 mantissa
// bits cleared, exact in tf32) and a low part (the remainder), and hi*hi + hi*lo + lo*hi are
// accumulated: three MMAs per step give products that are accurate to about 2^-21 instead of
// the 2^-10 of plain tf32.
#pragma once

#include "ani_common.cuh"

namespace ani {

constexpr int kMlpIn = 384, kMlpH1 = 128, kMlpH2 = 128, kMlpH3 = 64;
constexpr int kMlpTile = 128;             // atoms per CTA = MMA M
constexpr int kMlpThreads = 512;          // 16 warps: warp w reads TMEM lanes 32 (w % 4) .., columns 32 (w / 4) ..
constexpr int kMlpKChunk = 64;            // K values staged per step
constexpr int kMlpLbo = 128;              // bytes between core matrices adjacent in K
constexpr int kMlpSbo = (kMlpKChunk / 4) * 128;   // bytes between 8-row groups (2048)
constexpr int kMlpOperandBytes = kMlpTile * kMlpKChunk * 4;   // 32 KiB
constexpr int kMlpActStride = 129;        // floats per row of the activation buffer (bank-conflict free)
constexpr int kMlpTmemCols = 128;
constexpr int kMlpStageSteps = kMlpTile * (kMlpKChunk / 4) / kMlpThreads;   // staging slots per thread and chunk (4)
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
};

struct MlpShared {
    alignas(1024) unsigned char a_hi[kMlpOperandBytes];
    alignas(1024) unsigned char b_hi[kMlpOperandBytes];
    alignas(1024) unsigned char a_lo[kMlpOperandBytes];
    alignas(1024) unsigned char b_lo[kMlpOperandBytes];
    float act[kMlpTile * kMlpActStride];
    float vec[128];      // the layer's bias (forward) or the output weights w4 (backward)
    alignas(8) unsigned long long mbar;
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

// Shared-memory matrix descriptor: K-major, no swizzle, descriptor version 1.
__device__ __forceinline__ unsigned long long smem_desc(unsigned byte_addr)
{
    unsigned long long d = 0;
    d |= (unsigned long long)((byte_addr & 0x3ffff) >> 4);
    d |= (unsigned long long)(kMlpLbo >> 4) << 16;
    d |= (unsigned long long)(kMlpSbo >> 4) << 32;
    d |= 1ull << 46;
    return d;
}
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

// Position of element (row, k) of a staged chunk in the core-matrix layout, in bytes.
__device__ __forceinline__ int operand_offset(int row, int k)
{
    return (row >> 3) * kMlpSbo + (k >> 2) * kMlpLbo + (row & 7) * 16 + (k & 3) * 4;
}

// Stores four consecutive K values of one row as the high (tf32-exact) and low parts.
template <bool SPLIT>
__device__ __forceinline__ void stage4(unsigned char* hi, unsigned char* lo, int row, int k, float4 v)
{
    const int off = operand_offset(row, k);
    if (SPLIT) {
        float4 h, l;
        h.x = __uint_as_float(__float_as_uint(v.x) & 0xffffe000u);
        h.y = __uint_as_float(__float_as_uint(v.y) & 0xffffe000u);
        h.z = __uint_as_float(__float_as_uint(v.z) & 0xffffe000u);
        h.w = __uint_as_float(__float_as_uint(v.w) & 0xffffe000u);
        l.x = v.x - h.x; l.y = v.y - h.y; l.z = v.z - h.z; l.w = v.w - h.w;
        *reinterpret_cast<float4*>(hi + off) = h;
        *reinterpret_cast<float4*>(lo + off) = l;
    } else {
        *reinterpret_cast<float4*>(hi + off) = v;
    }
}

// (row, group of 4 K values) handled by thread `tid` in staging step `it`: 8 consecutive rows
// first (one 128-byte core matrix per 8 lanes, conflict-free), then 4 adjacent K groups.
__device__ __forceinline__ void staging_slot(int it, int tid, int* row, int* kgroup)
{
    const int q = it * kMlpThreads + tid;
    const int rest = q >> 5;
    *row = (rest >> 2) * 8 + (q & 7);
    *kgroup = (rest & 3) * 4 + ((q >> 3) & 3);
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

// 32 consecutive floats of one row, as eight 16-byte accesses.
__device__ __forceinline__ void store_row32(float* dst, const float* v)
{
#pragma unroll
    for (int i = 0; i < 32; i += 4)
        *reinterpret_cast<float4*>(dst + i) = make_float4(v[i], v[i + 1], v[i + 2], v[i + 3]);
}
__device__ __forceinline__ void load_row32(const float* src, float* v)
{
#pragma unroll
    for (int i = 0; i < 32; i += 4) {
        const float4 q = *reinterpret_cast<const float4*>(src + i);
        v[i] = q.x; v[i + 1] = q.y; v[i + 2] = q.z; v[i + 3] = q.w;
    }
}

// Stages the TRANSPOSE of src[r0 .. r0+63][col0 .. col0+rows-1] (row stride ld) as an operand
// chunk: operand row = column of src, operand k = row of src (an atom for the weight gradients,
// an input index for weights stored [in][out]).  Source rows past `n_valid` are zero.  A thread
// reads four consecutive columns of one source row and scatters them to four operand rows.
// Returns this thread's partial column sums over the source rows it touched (four columns).
// Column quad (four consecutive source columns) that this thread handles in stage_transposed
// for an operand of `rows` rows; the same in every pass.
__device__ __forceinline__ int transposed_quad(int rows)
{
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    return (warp % (rows >> 5)) * 8 + (lane >> 2);
}

// Lane mapping: a warp takes 8 column quads x 4 source rows, lane = (quad, source row).  Its
// loads are four 128-byte row segments; its stores are conflict-free because the bank of an
// operand element is 4 (row mod 8) + (k mod 4) and each store instruction writes 8 different
// (row mod 8) -- lanes rotate which of their four values they store -- times 4 different k.
template <bool SPLIT>
__device__ __forceinline__ float4 stage_transposed(unsigned char* hi, unsigned char* lo,
                                                   const float* __restrict__ src, int ld, int col0,
                                                   int rows, long long r0, int n_valid)
{
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int ksub = lane & 3, qsub = lane >> 2, rot = qsub >> 1;
    const int qblocks = rows >> 5;                        // 4 (128 rows) or 2 (64 rows)
    const int q = (warp % qblocks) * 8 + qsub;
    constexpr int kWarps = kMlpThreads / 32;
    constexpr int kMaxPasses = 4;
    const int passes = qblocks * (kMlpKChunk / 4) / kWarps;   // 4 or 2
    float4 colsum = make_float4(0.f, 0.f, 0.f, 0.f);
    float4 vs[kMaxPasses];
#pragma unroll
    for (int b = 0; b < kMaxPasses; b++) {                // all loads of the chunk in flight together
        const int k = ((b * kWarps + warp) / qblocks) * 4 + ksub;
        vs[b] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (b < passes && k < n_valid)
            vs[b] = *reinterpret_cast<const float4*>(src + (size_t)(r0 + k) * ld + col0 + 4 * q);
    }
#pragma unroll
    for (int b = 0; b < kMaxPasses; b++) {
        if (b >= passes) break;
        const int k = ((b * kWarps + warp) / qblocks) * 4 + ksub;
        const float4 v = vs[b];
        colsum.x += v.x; colsum.y += v.y; colsum.z += v.z; colsum.w += v.w;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int jj = (j + rot) & 3;
            const float val = jj == 0 ? v.x : (jj == 1 ? v.y : (jj == 2 ? v.z : v.w));
            const int off = operand_offset(4 * q + jj, k);
            if (SPLIT) {
                const float h = __uint_as_float(__float_as_uint(val) & 0xffffe000u);
                *reinterpret_cast<float*>(hi + off) = h;
                *reinterpret_cast<float*>(lo + off) = val - h;
            } else {
                *reinterpret_cast<float*>(hi + off) = val;
            }
        }
    }
    return colsum;
}

template <int ACT, bool SPLIT>
__global__ void __launch_bounds__(kMlpThreads, 1) mlp_forward_kernel(const MlpParams p)
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
        mbar_init(&sh.mbar, 1);
        sh.failed = 0;
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem = sh.tmem_base;
    unsigned parity = 0;
    bool ok = true;
    ANI_PHASE_DECL;

    const float* layer_w[3] = {p.w1[e], p.w2[e], p.w3[e]};
    const float* layer_b[3] = {p.b1[e], p.b2[e], p.b3[e]};
    float* layer_out[3] = {p.act1[e], p.act2[e], p.act3[e]};
    float* layer_dout[3] = {p.dact1[e], p.dact2[e], p.dact3[e]};
    const int layer_k[3] = {kMlpIn, kMlpH1, kMlpH2};
    const int layer_n[3] = {kMlpH1, kMlpH2, kMlpH3};

#pragma unroll 1
    for (int layer = 0; layer < 3; layer++) {
        const int K = layer_k[layer], N = layer_n[layer];
        const unsigned idesc = instr_desc(kMlpTile, N);
        if (tid < N) sh.vec[tid] = layer_b[layer][tid];   // read in the epilogue, after several barriers
#pragma unroll 1
        for (int kc = 0; kc < K; kc += kMlpKChunk) {
            // ---- stage the A chunk (128 atoms x 64) and the B chunk (N outputs x 64); all global
            // loads of the chunk are issued before any of them is used ----
            float4 av[kMlpStageSteps];
            int rows[kMlpStageSteps], kgs[kMlpStageSteps];
#pragma unroll
            for (int j = 0; j < kMlpStageSteps; j++) {
                staging_slot(j, tid, &rows[j], &kgs[j]);
                const int row = rows[j], kg = kgs[j];
                av[j] = make_float4(0.f, 0.f, 0.f, 0.f);
                if (layer == 0) {
                    if (row < n_rows)
                        av[j] = *reinterpret_cast<const float4*>(p.feat[e] + (size_t)(row0 + row) * kMlpIn + kc + kg * 4);
                } else {
                    const float* src = sh.act + row * kMlpActStride + kc + kg * 4;
                    av[j] = make_float4(src[0], src[1], src[2], src[3]);
                }
            }
            // B[n = out][k = in] = W[k][n]: the weights are read as stored ([in][out]) and transposed
            stage_transposed<SPLIT>(sh.b_hi, sh.b_lo, layer_w[layer], N, 0, N, kc, kMlpKChunk);
#pragma unroll
            for (int j = 0; j < kMlpStageSteps; j++) stage4<SPLIT>(sh.a_hi, sh.a_lo, rows[j], kgs[j] * 4, av[j]);
            ANI_PHASE(0);
            fence_async_smem();
            __syncthreads();
            ANI_PHASE(1);
            if (tid == 0) {
                tc_fence_after();
                const unsigned a_hi = smem_u32(sh.a_hi), b_hi = smem_u32(sh.b_hi);
                const unsigned a_lo = smem_u32(sh.a_lo), b_lo = smem_u32(sh.b_lo);
#pragma unroll
                for (int ks = 0; ks < kMlpKChunk / 8; ks++) {
                    const unsigned step = ks * 2 * kMlpLbo;
                    const bool first = kc == 0 && ks == 0;
                    mma_tf32(tmem, smem_desc(a_hi + step), smem_desc(b_hi + step), idesc, !first);
                    if (SPLIT) {
                        mma_tf32(tmem, smem_desc(a_hi + step), smem_desc(b_lo + step), idesc, true);
                        mma_tf32(tmem, smem_desc(a_lo + step), smem_desc(b_hi + step), idesc, true);
                    }
                }
                mma_commit(&sh.mbar);
            }
            // operands may be overwritten, and the accumulator read, only after the MMAs finish
            if (ok && !mbar_wait(&sh.mbar, parity)) ok = false;
            parity ^= 1u;
            if (!ok) sh.failed = 1;
            ANI_PHASE(2);
            __syncthreads();
            ANI_PHASE(3);
            if (sh.failed) break;
        }
        if (sh.failed) break;
        tc_fence_after();
        // ---- epilogue: bias, activation and its derivative; the row goes back to shared memory
        // as the next layer's A operand (the last hidden layer included: the output layer reads
        // it from there) ----
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
        ANI_PHASE(4);
        tc_fence_before();
        __syncthreads();
        ANI_PHASE(5);
    }
    ANI_PHASE_FLUSH;

    if (!sh.failed) {
        // ---- output layer 64 -> 1: one thread per atom, its last hidden row from shared memory ----
        if (tid < kMlpH3) sh.vec[tid] = p.w4[e][tid];
        __syncthreads();
        if (tid < n_rows) {
            float acc = p.b4[e][0];
#pragma unroll 8
            for (int i = 0; i < kMlpH3; i++) acc += sh.act[tid * kMlpActStride + i] * sh.vec[i];
            p.energy[e][row0 + tid] = acc;
        }
    } else if (tid == 0) {
        report(ANI_ERR_TIMEOUT);
    }
    __syncthreads();
    if (warp == 0) tmem_dealloc(tmem, kMlpTmemCols);
}

}  // namespace ani
