// Two-stage operand pipeline shared by the three atomic-network kernels.
//
// A product  acc[128 x N] (+)= A[128 x K] * B[N x K]^T  is cut into chunks of 32 values of K.  The
// 128 KiB operand area of MlpShared holds two stages (each: A hi, A lo, B hi, B lo, 16 KiB
// apiece); while the tensor core works on one stage the 512 producer threads fill the other, and
// the global loads of chunk c+1 are issued before chunk c is handed over, so that neither the MMAs
// nor the load latency sit on the critical path.  Hand-over is by mbarriers only: producers
// arrive on the stage's "full" barrier; the MMA warp waits for it, issues, and commits to the
// stage's "done" barrier, which the producers wait for before refilling.  All waits are bounded.
//
// Operand sources (where a chunk comes from and how it is laid out):
//   DirectGlobal   rows of a row-major global matrix, K along the row (16-byte loads and stores);
//   DirectShared   rows of the activation buffer in shared memory;
//   Transposed     the transpose of a row-major global matrix: operand row = source column,
//                  K = source row (weights stored [in][out]; activations with K = atom).
#pragma once

#include "ani_mlp.cuh"

namespace ani {

constexpr int kPipeK = 32;                                  // K values per stage
constexpr int kPipeSbo = (kPipeK / 4) * 128;                // 1024 bytes between 8-row groups
constexpr int kPipeOperandBytes = kMlpTile * kPipeK * 4;    // 16 KiB
constexpr int kPipeStageBytes = 4 * kPipeOperandBytes;      // A hi, A lo, B hi, B lo
static_assert(2 * kPipeStageBytes == 4 * kMlpOperandBytes, "two stages fill the operand area");

__device__ __forceinline__ int pipe_offset(int row, int k)
{
    return (row >> 3) * kPipeSbo + (k >> 2) * kMlpLbo + (row & 7) * 16 + (k & 3) * 4;
}
__device__ __forceinline__ unsigned long long pipe_desc(unsigned byte_addr)
{
    unsigned long long d = 0;
    d |= (unsigned long long)((byte_addr & 0x3ffff) >> 4);
    d |= (unsigned long long)(kMlpLbo >> 4) << 16;
    d |= (unsigned long long)(kPipeSbo >> 4) << 32;
    d |= 1ull << 46;
    return d;
}

template <bool SPLIT> __device__ __forceinline__ void pipe_store4(unsigned char* hi, unsigned char* lo, int off, float4 v)
{
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
template <bool SPLIT> __device__ __forceinline__ void pipe_store1(unsigned char* hi, unsigned char* lo, int off, float v)
{
    if (SPLIT) {
        const float h = __uint_as_float(__float_as_uint(v) & 0xffffe000u);
        *reinterpret_cast<float*>(hi + off) = h;
        *reinterpret_cast<float*>(lo + off) = v - h;
    } else {
        *reinterpret_cast<float*>(hi + off) = v;
    }
}

// (row, group of 4 K values) of direct-staging slot j of this thread: 8 consecutive rows first
// (one 128-byte core matrix per 8 lanes, conflict-free stores), then 4 adjacent K groups.
// 128 rows x 8 groups = 1024 slots, two per thread.
__device__ __forceinline__ void pipe_slot(int j, int* row, int* kgroup)
{
    const int q = j * kMlpThreads + (int)threadIdx.x;
    const int rest = q >> 5;
    *row = (rest >> 1) * 8 + (q & 7);
    *kgroup = (rest & 1) * 4 + ((q >> 3) & 3);
}

struct PipeRegs {
    float4 v[2];
};

// Rows [0, rows) of a row-major global matrix (row stride ld); rows >= rows_valid read as zero;
// chunk c covers columns k0 + 32 c .. + 31.
template <bool SPLIT> struct DirectGlobal {
    static constexpr bool kBulk = false;
    const float* base;
    size_t ld;
    int rows, rows_valid, k0;
    __device__ __forceinline__ void load(int c, PipeRegs& r) const
    {
#pragma unroll
        for (int j = 0; j < 2; j++) {
            int row, kg;
            pipe_slot(j, &row, &kg);
            r.v[j] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (row < rows_valid) r.v[j] = *reinterpret_cast<const float4*>(base + (size_t)row * ld + k0 + c * kPipeK + kg * 4);
        }
    }
    __device__ __forceinline__ void store(const PipeRegs& r, unsigned char* hi, unsigned char* lo)
    {
#pragma unroll
        for (int j = 0; j < 2; j++) {
            int row, kg;
            pipe_slot(j, &row, &kg);
            if (row < rows) pipe_store4<SPLIT>(hi, lo, pipe_offset(row, kg * 4), r.v[j]);
        }
    }
};

// All 128 rows of the activation buffer in shared memory (row stride kMlpActStride).
template <bool SPLIT> struct DirectShared {
    const float* act;
    __device__ __forceinline__ void load(int, PipeRegs&) const {}
    __device__ __forceinline__ void store_chunk(int c, unsigned char* hi, unsigned char* lo) const
    {
#pragma unroll
        for (int j = 0; j < 2; j++) {
            int row, kg;
            pipe_slot(j, &row, &kg);
            const float* src = act + row * kMlpActStride + c * kPipeK + kg * 4;
            pipe_store4<SPLIT>(hi, lo, pipe_offset(row, kg * 4), make_float4(src[0], src[1], src[2], src[3]));
        }
    }
};

// Column quad (four consecutive source columns) of this thread in a Transposed source with
// `rows` operand rows; the same for every chunk.
__device__ __forceinline__ int transposed_quad(int rows)
{
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    return (warp % (rows >> 5)) * 8 + (lane >> 2);
}

// The transpose of src[r0 + 32 c + k][col0 + row] (row stride ld): operand row = source column
// (rows = 128 or 64 of them), K = source row; source rows >= n_valid (counted from r0) are zero.
// Lane mapping: a warp takes 8 column quads x 4 source rows, lane = (quad, source row): loads are
// four 128-byte row segments; stores are conflict-free because the bank of an operand element
// is 4 (row mod 8) + (k mod 4) and each store instruction writes 8 different (row mod 8) -- lanes
// rotate which of their four values they store -- times 4 different k.
// colsum accumulates this thread's column sums (four columns) over everything it staged.
template <bool SPLIT> struct Transposed {
    static constexpr bool kBulk = false;
    const float* base;
    size_t ld;
    int col0, rows;
    long long r0;
    int n_valid;
    float4 colsum;
    __device__ __forceinline__ int passes() const { return (rows >> 5) * (kPipeK / 4) / (kMlpThreads / 32); }   // 2 or 1
    __device__ __forceinline__ int k_of(int b) const
    {
        const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
        return ((b * (kMlpThreads / 32) + warp) / (rows >> 5)) * 4 + (lane & 3);
    }
    __device__ __forceinline__ void load(int c, PipeRegs& r) const
    {
        const int q = transposed_quad(rows);
#pragma unroll
        for (int b = 0; b < 2; b++) {
            const int k = c * kPipeK + k_of(b);
            r.v[b] = make_float4(0.f, 0.f, 0.f, 0.f);
            if (b < passes() && k < n_valid)
                r.v[b] = *reinterpret_cast<const float4*>(base + (size_t)(r0 + k) * ld + col0 + 4 * q);
        }
    }
    __device__ __forceinline__ void store(const PipeRegs& r, unsigned char* hi, unsigned char* lo)
    {
        const int lane = threadIdx.x & 31;
        const int q = transposed_quad(rows), rot = lane >> 3;
#pragma unroll
        for (int b = 0; b < 2; b++) {
            if (b >= passes()) break;
            const int k = k_of(b);
            const float4 v = r.v[b];
            colsum.x += v.x; colsum.y += v.y; colsum.z += v.z; colsum.w += v.w;
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int jj = (j + rot) & 3;
                const float val = jj == 0 ? v.x : (jj == 1 ? v.y : (jj == 2 ? v.z : v.w));
                pipe_store1<SPLIT>(hi, lo, pipe_offset(4 * q + jj, k), val);
            }
        }
    }
};

// A B operand that was packed beforehand (mlp_pack_kernel): chunk c of the product is 32 KiB at
// base + c * 32 KiB, already split into high and low parts and laid out exactly as a stage wants
// it, so one thread moves it with ONE bulk asynchronous copy (TMA) that reports to the stage's
// "full" barrier; the other 511 producers spend nothing on B.
constexpr unsigned kPackedChunkBytes = 2 * kPipeOperandBytes;
struct PackedB {
    static constexpr bool kBulk = true;
    const unsigned char* base;
    __device__ __forceinline__ void load(int, PipeRegs&) const {}
    __device__ __forceinline__ void store(const PipeRegs&, unsigned char*, unsigned char*) const {}
};

// Packed layout of one element's weights: chunk indices of every product.
constexpr int kPackFwdL1 = 0, kPackFwdL2 = 12, kPackFwdL3 = 16;          // forward: W1 (12 chunks), W2 (4), W3 (4)
constexpr int kPackBwdS0 = 20, kPackBwdS1 = 22, kPackBwdF = 26;          // backward: W3 (2), W2 (4), W1 blocks (3 x 4)
constexpr int kPackChunks = 38;

struct PipeState {
    unsigned chunks = 0;          // chunks issued so far in this kernel (stage = chunks & 1)
    unsigned parity0 = 0, parity1 = 0;
    bool pending0 = false, pending1 = false;
    bool ok = true;
};

// Waits (bounded) for the MMAs that last read stage s, if any are outstanding.
__device__ __forceinline__ void pipe_wait_stage(MlpShared& sh, PipeState& ps, int s)
{
    bool& pending = s ? ps.pending1 : ps.pending0;
    unsigned& parity = s ? ps.parity1 : ps.parity0;
    if (!pending) return;
    if (ps.ok && !mbar_wait(&sh.stage_bar[s], parity)) {
        ps.ok = false;
        sh.failed = 1;
    }
    parity ^= 1u;
    pending = false;
}

// Producer side of  acc (+)= A * B^T  over `nchunks` chunks: fills stage after stage and
// signals each one.  ASHARED selects the activation buffer as the A source (a_sh) instead of
// a_src.  Never blocks without a bound; a timeout is reported by pipe_drain.
template <bool SPLIT, bool ASHARED, class ASrc, class BSrc>
__device__ __forceinline__ void pipe_produce(MlpShared& sh, int nchunks, PipeState& ps, ASrc& a_src,
                                             const DirectShared<SPLIT>& a_sh, BSrc& b_src)
{
    PipeRegs ra, rb;
    if (!ASHARED) a_src.load(0, ra);
    b_src.load(0, rb);
#pragma unroll 1
    for (int c = 0; c < nchunks; c++) {
        const int s = (int)(ps.chunks & 1u);
        unsigned char* stage = sh.a_hi + s * kPipeStageBytes;
        pipe_wait_stage(sh, ps, s);
        if (BSrc::kBulk) {
            if (threadIdx.x == 0) {      // registered before this thread's own arrival below
                mbar_expect_tx(&sh.full_bar[s], kPackedChunkBytes);
                bulk_copy_to_shared(stage + 2 * kPipeOperandBytes, b_src.base + (size_t)c * kPackedChunkBytes,
                                    kPackedChunkBytes, &sh.full_bar[s]);
            }
        } else {
            b_src.store(rb, stage + 2 * kPipeOperandBytes, stage + 3 * kPipeOperandBytes);
        }
        if (ASHARED) a_sh.store_chunk(c, stage, stage + kPipeOperandBytes);
        else a_src.store(ra, stage, stage + kPipeOperandBytes);
        if (c + 1 < nchunks) {           // the next chunk's loads fly while this one is consumed
            if (!ASHARED) a_src.load(c + 1, ra);
            b_src.load(c + 1, rb);
        }
        fence_async_smem();
        mbar_arrive(&sh.full_bar[s]);
        if (s) ps.pending1 = true; else ps.pending0 = true;
        ps.chunks++;
    }
}

// Packs the weights of the four elements into the stage layout (both products that read them:
// forward B[n = out][k = in] = W[k][n], backward B[n = in][k = out] = W[n][k]), high and low tf32
// parts.  grid = (kPackChunks, 4 elements); run once per weight update.
struct MlpPackParams {
    const float* w1[kTypes];   // [384][128]
    const float* w2[kTypes];   // [128][128]
    const float* w3[kTypes];   // [128][64]
    unsigned char* packed[kTypes];
};
__global__ void __launch_bounds__(kMlpThreads) mlp_pack_kernel(const MlpPackParams p)
{
    const int e = blockIdx.y, chunk = blockIdx.x;
    if (!p.packed[e]) return;
    const float* w;
    int ld, k0, n0, rows;
    bool transposed;   // true: operand (n, k) = W[k0 + k][n0 + n];  false: W[n0 + n][k0 + k]
    if (chunk < kPackFwdL2)      { w = p.w1[e]; ld = 128; transposed = true;  k0 = 32 * chunk;                n0 = 0; rows = 128; }
    else if (chunk < kPackFwdL3) { w = p.w2[e]; ld = 128; transposed = true;  k0 = 32 * (chunk - kPackFwdL2); n0 = 0; rows = 128; }
    else if (chunk < kPackBwdS0) { w = p.w3[e]; ld = 64;  transposed = true;  k0 = 32 * (chunk - kPackFwdL3); n0 = 0; rows = 64; }
    else if (chunk < kPackBwdS1) { w = p.w3[e]; ld = 64;  transposed = false; k0 = 32 * (chunk - kPackBwdS0); n0 = 0; rows = 128; }
    else if (chunk < kPackBwdF)  { w = p.w2[e]; ld = 128; transposed = false; k0 = 32 * (chunk - kPackBwdS1); n0 = 0; rows = 128; }
    else {
        const int c = chunk - kPackBwdF;
        w = p.w1[e]; ld = 128; transposed = false; k0 = 32 * (c & 3); n0 = 128 * (c >> 2); rows = 128;
    }
    unsigned char* hi = p.packed[e] + (size_t)chunk * kPackedChunkBytes;
    unsigned char* lo = hi + kPipeOperandBytes;
    for (int idx = threadIdx.x; idx < kMlpTile * kPipeK; idx += kMlpThreads) {
        const int n = idx / kPipeK, k = idx % kPipeK;
        float v = 0.0f;
        if (n < rows) v = transposed ? w[(size_t)(k0 + k) * ld + n0 + n] : w[(size_t)(n0 + n) * ld + k0 + k];
        const float h = __uint_as_float(__float_as_uint(v) & 0xffffe000u);
        const int off = pipe_offset(n, k);
        *reinterpret_cast<float*>(hi + off) = h;
        *reinterpret_cast<float*>(lo + off) = v - h;
    }
}

// MMA-warp side of the same product: waits (bounded) for each filled stage, issues its MMAs and
// commits them to the stage's barrier.  `fresh` = overwrite the accumulator with the first chunk.
struct IssueState {
    unsigned chunks = 0;
    unsigned parity0 = 0, parity1 = 0;
    bool ok = true;
};
template <bool SPLIT>
__device__ __forceinline__ void pipe_issue(MlpShared& sh, unsigned tmem, int N, int nchunks, bool fresh, IssueState& is)
{
    const unsigned idesc = instr_desc(kMlpTile, N);
    const int lane = threadIdx.x & 31;
#pragma unroll 1
    for (int c = 0; c < nchunks; c++) {
        const int s = (int)(is.chunks & 1u);
        unsigned& parity = s ? is.parity1 : is.parity0;
        if (is.ok && !mbar_wait(&sh.full_bar[s], parity)) {
            is.ok = false;
            sh.failed = 1;
        }
        parity ^= 1u;
        if (is.ok && lane == 0) {
            tc_fence_after();
            const unsigned a_hi = smem_u32(sh.a_hi + s * kPipeStageBytes), a_lo = a_hi + kPipeOperandBytes;
            const unsigned b_hi = a_hi + 2 * kPipeOperandBytes, b_lo = a_hi + 3 * kPipeOperandBytes;
#pragma unroll
            for (int ks = 0; ks < kPipeK / 8; ks++) {
                const unsigned step = ks * 2 * kMlpLbo;
                const bool first = fresh && c == 0 && ks == 0;
                mma_tf32(tmem, pipe_desc(a_hi + step), pipe_desc(b_hi + step), idesc, !first);
                if (SPLIT) {
                    mma_tf32(tmem, pipe_desc(a_hi + step), pipe_desc(b_lo + step), idesc, true);
                    mma_tf32(tmem, pipe_desc(a_lo + step), pipe_desc(b_hi + step), idesc, true);
                }
            }
            mma_commit(&sh.stage_bar[s]);
        }
        __syncwarp();
        is.chunks++;
    }
}

// Producers: waits for every outstanding MMA (before an epilogue reads the accumulator or reuses
// the operand area as scratch).  Returns false after a timeout (uniform across the producers).
__device__ __forceinline__ bool pipe_drain(MlpShared& sh, PipeState& ps)
{
    pipe_wait_stage(sh, ps, 0);
    pipe_wait_stage(sh, ps, 1);
    producer_sync();
    if (sh.failed) return false;
    tc_fence_after();
    return true;
}

}  // namespace ani
