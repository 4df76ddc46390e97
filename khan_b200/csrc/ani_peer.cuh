// Mean of one float buffer over the GPUs of a node, through peer memory, in ONE kernel launch per
// rank: the data-parallel average of the weight gradients (the reference concatenates the towers'
// gradients on the CPU and takes reduce_mean, khan/training/trainer_multi_tower.py:137-179).  One
// process per GPU; every rank owns a cudaMalloc'ed block [flags | staging 0 | staging 1] that the
// other ranks map with CUDA IPC.  A call on rank r, step s (parity = s & 1):
//   0. every block copies its part of the buffer into the rank's own staging[parity] (after this
//      the buffer itself is free: peers never read it);
//   1. the block that finishes the copy last publishes "rank r has arrived at step s + 1" in the flag
//      slot [r] of every peer (release store, system scope);
//   2. every block waits until all peers have arrived (acquire loads of the rank's own flag slots;
//      the wait is BOUNDED: when it runs out the kernel records ANI_ERR_TIMEOUT in the device status
//      word and goes on, so a missing rank costs a wrong step, not a hung GPU);
//   3. every block sums its part over the staging[parity] of all ranks (plain peer loads over
//      NVLink that bypass L1, 16 bytes each) and writes the mean back into the buffer.
// staging[parity] is rewritten two steps later, and a rank cannot get there before every peer has
// arrived at the step in between, i.e. has finished reading -- so one flag per (rank, peer) and two
// staging buffers are all the synchronisation there is.  The step number lives in device memory and
// is advanced by the kernel itself, so the launch can sit in a CUDA graph.  No NCCL call, plain
// peer mappings only; the grid is one block per SM at most, so that all blocks are resident while
// they wait.
//
// A second form (ani_peer_set_two_halves; the default above four ranks) moves fewer bytes: after the
// arrival round every rank forms the mean of ITS slice of the buffer only (1 / world of the bytes
// from each peer) and writes it to a second staging buffer; after a "slice ready" round of flags
// every rank fetches the other ranks' slices from there.  The same ordering argument covers both
// staging buffers.  Measured on four GPUs the second round of flags cost more than the bytes saved
// (0.253 against 0.243 ms per training step).
#pragma once

#include <cuda_runtime.h>

#include "ani_common.cuh"

namespace ani {

constexpr int kPeerMaxRanks = 8;
constexpr int kPeerFlagBytes = 256;          // flag area in front of the staging buffers
constexpr int kPeerThreads = 256;
#ifndef ANI_PEER_MAX_BLOCKS
#define ANI_PEER_MAX_BLOCKS 148
#endif
constexpr int kPeerMaxBlocks = ANI_PEER_MAX_BLOCKS;   // blocks of a call (one per SM at most)
constexpr unsigned kPeerSpinLimit = 1u << 18;   // tries of a microsecond or so each: a fraction of a second

struct PeerState {
    unsigned long long copied;   // blocks that have finished pass 0, over all launches
    unsigned long long reduced;  // blocks that have finished their part of the rank's slice (two-halves form)
    unsigned long long done;     // blocks that have finished the call, over all launches
    unsigned step;               // calls completed so far
    unsigned spin_limit;
};

struct PeerParams {
    float* buffer;                        // reduced in place
    long long n4;                         // 16-byte groups in the buffer
    long long stage_floats;               // floats per staging buffer
    int rank, world;
    float* stage[kPeerMaxRanks];          // staging area of every rank ([2][stage_floats]); [rank] is local
    unsigned* flags[kPeerMaxRanks];       // flag area of every rank ([world] slots); [rank] is local
    PeerState* state;                     // local
    float inv_world;
    int two_halves;                       // slice means + exchange of the slices instead of every rank summing everything
};

constexpr int kPeerReadySlot = kPeerMaxRanks;   // flag slots [0, 8): arrival; [8, 16): slice ready

__device__ __forceinline__ void store_release_sys(unsigned* p, unsigned v)
{
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ unsigned load_acquire_sys(const unsigned* p)
{
    unsigned v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ float4 load_peer16(const float4* p)
{
    return __ldcv(p);   // ld.global.cv: fetched again every time, never served from this SM's L1; loads may overlap
}

// Thread 0 of a block: counts the block in; the block that completes the count for this step publishes
// step + 1 in slot [slot0 + rank] of every peer's flag area; then waits (bounded) for the same from every
// peer.  Returns false when a wait ran out.
__device__ __forceinline__ bool peer_round(const PeerParams& p, unsigned long long* counter, int slot0, unsigned step)
{
    const unsigned long long before = atomicAdd(counter, 1ull);
    if (before + 1 == (unsigned long long)gridDim.x * (step + 1ull)) {
        __threadfence_system();
        for (int q = 0; q < p.world; q++)
            if (q != p.rank) store_release_sys(p.flags[q] + slot0 + p.rank, step + 1u);
    }
    const unsigned limit = p.state->spin_limit;
    bool ok = true;
    for (int q = 0; q < p.world; q++) {
        if (q == p.rank) continue;
        unsigned tries = 0;
        while ((int)(load_acquire_sys(p.flags[p.rank] + slot0 + q) - (step + 1u)) < 0) {
            if (++tries > limit) {
                ok = false;
                break;
            }
            __nanosleep(100);
        }
    }
    return ok;
}

// Mean over the ranks of 16-byte group i of the staging buffers at `off` (the same order on every rank).
__device__ __forceinline__ float4 peer_group_mean(const PeerParams& p, long long off, long long i)
{
    float4 v[kPeerMaxRanks];   // all loads of a group are in flight before the first is used
#pragma unroll
    for (int q = 0; q < kPeerMaxRanks; q++)
        if (q < p.world) v[q] = load_peer16(reinterpret_cast<const float4*>(p.stage[q] + off) + i);
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int q = 0; q < kPeerMaxRanks; q++)
        if (q < p.world) {
            acc.x += v[q].x; acc.y += v[q].y; acc.z += v[q].z; acc.w += v[q].w;
        }
    return make_float4(acc.x * p.inv_world, acc.y * p.inv_world, acc.z * p.inv_world, acc.w * p.inv_world);
}

__global__ void __launch_bounds__(kPeerThreads) peer_mean_kernel(const PeerParams p)
{
    __shared__ int timed_out;
    const unsigned step = *reinterpret_cast<volatile unsigned*>(&p.state->step);   // the same in every block of a launch
    const long long parity_off = (long long)(step & 1u) * p.stage_floats;
    const long long stride = (long long)gridDim.x * kPeerThreads;
    const long long first = (long long)blockIdx.x * kPeerThreads + threadIdx.x;

    // 0. this rank's contribution to its own staging buffer
    {
        const float4* src = reinterpret_cast<const float4*>(p.buffer);
        float4* dst = reinterpret_cast<float4*>(p.stage[p.rank] + parity_off);
        for (long long i = first; i < p.n4; i += stride) dst[i] = src[i];
    }
    __threadfence_system();
    __syncthreads();
    if (threadIdx.x == 0) {
        // 1 + 2. the last block to get here tells the peers; every block waits for all of them
        timed_out = peer_round(p, &p.state->copied, 0, step) ? 0 : 1;
    }
    __syncthreads();

    float4* out = reinterpret_cast<float4*>(p.buffer);
    if (!p.two_halves) {
        // 3. mean over the ranks (also after a timeout: the call must end like any other)
        for (long long i = first; i < p.n4; i += stride) out[i] = peer_group_mean(p, parity_off, i);
    } else {
        // 3a. the mean of this rank's slice, to the buffer and to the second staging buffer
        const long long per = (p.n4 + p.world - 1) / p.world;
        const long long out_off = (2 + (long long)(step & 1u)) * p.stage_floats;   // staging buffers 2, 3
        {
            const long long lo = per * p.rank, hi = min(p.n4, lo + per);
            float4* mine = reinterpret_cast<float4*>(p.stage[p.rank] + out_off);
            for (long long i = lo + first; i < hi; i += stride) {
                const float4 m = peer_group_mean(p, parity_off, i);
                mine[i] = m;
                out[i] = m;
            }
        }
        __threadfence_system();
        __syncthreads();
        if (threadIdx.x == 0 && !peer_round(p, &p.state->reduced, kPeerReadySlot, step)) timed_out = 1;
        __syncthreads();
        // 3b. the other ranks' slices
        for (long long i = first; i < p.n4; i += stride) {
            const int owner = (int)(i / per);
            if (owner != p.rank) out[i] = load_peer16(reinterpret_cast<const float4*>(p.stage[owner] + out_off) + i);
        }
    }
    if (threadIdx.x == 0 && timed_out) report(ANI_ERR_TIMEOUT);
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned long long before = atomicAdd(&p.state->done, 1ull);
        if (before + 1 == (unsigned long long)gridDim.x * (step + 1ull))
            *reinterpret_cast<volatile unsigned*>(&p.state->step) = step + 1u;   // the next launch sees it: launches are ordered
    }
}

}  // namespace ani
