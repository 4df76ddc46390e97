// C ABI of libani_b200.so: argument checks, launch configuration and the per-device scratch
// cache.  All kernels live in the .cuh files included below (one translation unit, so the
// device status word and the constant tables exist exactly once).
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>

#include <algorithm>
#include <initializer_list>
#include <new>
#include <mutex>
#include <vector>

#include "ani_common.cuh"

#include "ani_featurize.cuh"
#include "ani_featurize_mol.cuh"
#include "ani_featurize_large.cuh"
#include "ani_grad.cuh"
#include "ani_grad_mol.cuh"
#include "ani_grad_inverse.cuh"
#include "ani_mlp_forward.cuh"
#include "ani_mlp_backward.cuh"
#include "ani_mlp_wgrad.cuh"
#include "ani_charge.cuh"
#include "ani_optim.cuh"
#include "ani_energy.cuh"
#include "ani_sort.cuh"
#include "ani_host_pack.h"
#include "ani_feeder.h"
#include "ani_peer.cuh"

namespace {

using namespace ani;

thread_local cudaError_t t_last_error = cudaSuccess;

int cuda_fail(cudaError_t e)
{
    t_last_error = e;
    return ANI_ERR_CUDA;
}

#define ANI_CUDA(call)                                  \
    do {                                                \
        cudaError_t e_ = (call);                        \
        if (e_ != cudaSuccess) return cuda_fail(e_);    \
    } while (0)

constexpr int kMaxDevices = 64;

// Scratch of the large-batch sort (per-tile element counts), one buffer per (device, stream): two
// calls that overlap on the GPU are on different streams and so never share a buffer.  A buffer
// that has become too small is replaced but NEVER freed -- its address may be recorded in a CUDA
// graph that is replayed later -- so the old ones stay allocated until the process ends (they are
// a few KiB each and grow geometrically).
struct SortScratch {
    int dev;
    cudaStream_t stream;
    int* ptr;
    size_t bytes;
};
std::mutex g_scratch_mutex;
std::vector<SortScratch> g_sort_scratch;

// True when work given to `stream` is being recorded into a graph instead of run.
int stream_is_capturing(cudaStream_t stream, bool* capturing)
{
    cudaStreamCaptureStatus status = cudaStreamCaptureStatusNone;
    ANI_CUDA(cudaStreamIsCapturing(stream, &status));
    *capturing = status != cudaStreamCaptureStatusNone;
    return ANI_OK;
}

int sort_scratch(size_t bytes, cudaStream_t stream, int** out)
{
    int dev = 0;
    ANI_CUDA(cudaGetDevice(&dev));
    std::lock_guard<std::mutex> lock(g_scratch_mutex);
    SortScratch* slot = nullptr;
    for (SortScratch& s : g_sort_scratch)
        if (s.dev == dev && s.stream == stream) slot = &s;
    if (slot && slot->bytes >= bytes) {
        *out = slot->ptr;
        return ANI_OK;
    }
    // an allocation is not something a stream capture can record
    bool capturing = false;
    if (int rc = stream_is_capturing(stream, &capturing)) return rc;
    if (capturing) return ANI_ERR_CAPTURE;
    const size_t want = bytes < (1u << 16) ? (1u << 16) : bytes * 2;
    int* ptr = nullptr;
    ANI_CUDA(cudaMalloc(&ptr, want));
    if (slot) {
        slot->ptr = ptr;       // the previous buffer stays allocated (see above)
        slot->bytes = want;
    } else {
        g_sort_scratch.push_back(SortScratch{dev, stream, ptr, want});
    }
    *out = ptr;
    return ANI_OK;
}

// Fixed scratch for ani_sort_noalloc: per-tile element counts for batches of up to
// kSortStaticMaxAtoms atoms ((tiles + 1) x 4 ints = 64 KiB + 16 B).  It lives in the module's
// static device data, so every GPU that loads this library holds it until the process exits.
constexpr int kSortStaticMaxAtoms = 1 << 22;  // 4,194,304 atoms
constexpr int kSortStaticMaxTiles = kSortStaticMaxAtoms / kSortTile;
static __device__ __align__(256) int g_sort_static_scratch[(kSortStaticMaxTiles + 1) * kTypes];

// Device address of g_sort_static_scratch on each device, resolved on first use.  In host code
// the array's name is only a handle for the runtime, not a device address, so it is never
// passed to a kernel; the pointer obtained here is.
int* g_sort_static_ptr[kMaxDevices] = {};
std::mutex g_sort_static_mutex;

int sort_static_scratch(cudaStream_t stream, int** out)
{
    int dev = 0;
    ANI_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return ANI_ERR_BAD_SIZE;
    std::lock_guard<std::mutex> lock(g_sort_static_mutex);
    if (!g_sort_static_ptr[dev]) {
        // The look-up may load the module's data on this device: not something to do while the stream
        // is being captured.  Make the first call on a device outside any capture.
        bool capturing = false;
        if (int rc = stream_is_capturing(stream, &capturing)) return rc;
        if (capturing) return ANI_ERR_CAPTURE;
        int* ptr = nullptr;
        ANI_CUDA(cudaGetSymbolAddress((void**)&ptr, g_sort_static_scratch));  // current device = dev
        g_sort_static_ptr[dev] = ptr;
    }
    *out = g_sort_static_ptr[dev];
    return ANI_OK;
}

// Featurizer launch shapes: NW warps per CTA, (slots per molecule) / NW CTAs per molecule, one warp
// per central atom.  The capacities bound the neighbours of one element kept in shared memory
// per central atom (atoms with more take the streaming path).
#ifndef ANI_NW
#define ANI_NW 4
#endif
constexpr int kNW = ANI_NW;   // warps per CTA of the featurizer kernels (a power of two <= 32)
constexpr int kCapT = 24;  // angular (r < 3.1 A) neighbours per element
constexpr int kCapR = 48;  // radial (r < 4.6 A) neighbours per element

// Persistent grid: as many CTAs as fit on the device at once (rounded to a multiple of
// kSlotsPerMol / kNW so that the warp count is a multiple of kSlotsPerMol), or fewer when the
// batch is small.
template <typename K> int featurizer_grid(K kernel, size_t smem, int n_mols, int* grid)
{
    int dev = 0, sms = 0, per_sm = 0;
    ANI_CUDA(cudaGetDevice(&dev));
    ANI_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    ANI_CUDA(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kNW * kWarp, smem));
    constexpr int kGroup = kSlotsPerMol / kNW;
    long long resident = (long long)sms * (per_sm > 0 ? per_sm : 1);
    resident = (resident / kGroup) * kGroup;
    if (resident < kGroup) resident = kGroup;
    const long long needed = (long long)n_mols * kGroup;
    *grid = (int)(needed < resident ? needed : resident);
    return ANI_OK;
}

// Work list of a launch, packed into one kernel argument: bits 0-4 = log2 of the slots per
// molecule (the smallest power of two that is not below the mean atoms per molecule, between kNW
// and kSlotsPerMol: few empty items, and larger molecules simply give some slots a second atom);
// bit 5 = slot-major order, used when molecules are small (see next_work).
constexpr int kSlotMajorFlag = 32;
int pick_slot_shift(long long n_atoms, int n_mols)
{
    const long long mean = n_mols > 0 ? (n_atoms + n_mols - 1) / n_mols : 1;
    int shift = 0;
    while ((1 << shift) < kNW) shift++;   // at least one slot per warp of a CTA
    while ((1 << shift) < mean && (1 << shift) < kSlotsPerMol) shift++;
    return shift | (mean <= kSlotsPerMol ? kSlotMajorFlag : 0);
}

template <typename K> int set_smem(K kernel, size_t bytes)
{
    ANI_CUDA(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
    return ANI_OK;
}

// Batches whose MEAN molecule size is at most this take the one-CTA-per-molecule kernels (their
// fast path covers molecules of up to kMolMaxAtoms atoms; a larger molecule in such a batch is
// still handled, slowly).  Batches of larger molecules take featurize_large_kernel (rounds of four
// central atoms per warp, the molecule scanned from global memory) for the forward pass and the
// one-warp-per-atom kernel for the gradient; the one-warp-per-atom forward kernel remains for outputs
// that are not 16-byte aligned.  (A gradient kernel built like the large forward one was measured on
// 256 molecules of 64-256 atoms: 26 % fewer instructions and 104 instead of 139 us alone, but 99
// instead of 90 us per launch with four batches in flight, so it is not used.)
constexpr int kMolMeanLimit = 24;
#ifndef ANI_MOL_GRAD_WARPS
#define ANI_MOL_GRAD_WARPS 4
#endif
constexpr int kMolGradWarps = ANI_MOL_GRAD_WARPS;   // warps of a CTA (= molecule) of the small-molecule gradient kernel
bool small_molecules(long long n_atoms, int n_mols) { return n_mols > 0 && n_atoms <= (long long)n_mols * kMolMeanLimit; }

// True when every non-null pointer of the list is 16-byte aligned.
bool all_aligned16(std::initializer_list<const void*> ptrs)
{
    for (const void* q : ptrs)
        if (reinterpret_cast<uintptr_t>(q) & 15) return false;
    return true;
}

int check_acs(const int* acs_host, long long* n_atoms)
{
    if (!acs_host) return ANI_ERR_NULL_POINTER;
    long long n = 0;
    for (int t = 0; t < kTypes; t++) {
        if (acs_host[t] < 0) return ANI_ERR_BAD_SIZE;
        n += acs_host[t];
    }
    if (n > 0x7fffffffLL) return ANI_ERR_TOO_MANY_ATOMS;
    *n_atoms = n;
    return ANI_OK;
}

template <typename T, int CAPT = kCapT, int CAPR = kCapR>
int featurize_impl(const T* xs, const T* ys, const T* zs, const int* types, const int* mos,
                   const int* macs, int n_mols, const int* sis, T* oh, T* oc, T* on, T* oo,
                   const int* acs_host, void* stream)
{
    long long n_atoms = 0;
    if (int rc = check_acs(acs_host, &n_atoms)) return rc;
    if (n_mols < 0) return ANI_ERR_BAD_SIZE;
    if (n_mols == 0 || n_atoms == 0) return ANI_OK;
    if (!xs || !ys || !zs || !types || !mos || !macs || !sis) return ANI_ERR_NULL_POINTER;
    T* outs[kTypes] = {oh, oc, on, oo};
    for (int t = 0; t < kTypes; t++)
        if (acs_host[t] > 0 && !outs[t]) return ANI_ERR_NULL_POINTER;

    int dev = 0;
    ANI_CUDA(cudaGetDevice(&dev));
    // small molecules with outputs that take 16-byte stores: one warp (= one CTA) per round of four
    // central atoms
    if (small_molecules(n_atoms, n_mols) && all_aligned16({oh, oc, on, oo}) &&
        (long long)n_mols * kMolRounds <= 0x7fffffffLL) {
        featurize_mol_kernel<T><<<n_mols * kMolRounds, kWarp, 0, (cudaStream_t)stream>>>(
            xs, ys, zs, types, mos, macs, n_mols, (int)n_atoms, sis, oh, oc, on, oo, acs_host[0], acs_host[1],
            acs_host[2], acs_host[3]);
        ANI_CUDA(cudaGetLastError());
        return ANI_OK;
    }

    // larger molecules: the same rounds of four central atoms, the molecule scanned from global memory;
    // a CTA takes every rounds_in_grid-th round of its molecule
    if (n_mols > 0 && all_aligned16({oh, oc, on, oo})) {
        const long long mean_rounds = (n_atoms / n_mols + kMolCentrals) / kMolCentrals;
        const int rounds_in_grid = (int)std::min<long long>(std::max<long long>(mean_rounds, kMolRounds), 64);
        if ((long long)n_mols * rounds_in_grid <= 0x7fffffffLL) {
            featurize_large_kernel<T><<<n_mols * rounds_in_grid, kWarp, 0, (cudaStream_t)stream>>>(
                xs, ys, zs, types, mos, macs, n_mols, (int)n_atoms, rounds_in_grid, sis, oh, oc, on, oo, acs_host[0],
                acs_host[1], acs_host[2], acs_host[3]);
            ANI_CUDA(cudaGetLastError());
            return ANI_OK;
        }
    }

    auto kernel = featurize_kernel<T, kNW, CAPT, CAPR>;
    const size_t smem = kNW * sizeof(FeaturizeWarpShared<T, CAPT, CAPR>);
    static thread_local int configured_dev = -1;
    if (configured_dev != dev) {
        if (int rc = set_smem(kernel, smem)) return rc;
        configured_dev = dev;
    }
    static thread_local int cached_grid_dev = -1, cached_resident = 0;
    if (cached_grid_dev != dev) {
        if (int rc = featurizer_grid(kernel, smem, 1 << 24, &cached_resident)) return rc;
        cached_grid_dev = dev;
    }
    const int slot_shift = pick_slot_shift(n_atoms, n_mols);
    const long long needed = (long long)n_mols * ((1 << (slot_shift & 31)) / kNW);
    const int grid = (int)(needed < cached_resident ? needed : cached_resident);
    kernel<<<grid, kNW * kWarp, smem, (cudaStream_t)stream>>>(
        xs, ys, zs, types, mos, macs, n_mols, (int)n_atoms, slot_shift, sis, oh, oc, on, oo, acs_host[0],
        acs_host[1], acs_host[2], acs_host[3]);
    ANI_CUDA(cudaGetLastError());
    return ANI_OK;
}

template <typename T>
int featurize_grad_impl(const T* xs, const T* ys, const T* zs, const int* types, const int* mos,
                        const int* macs, int n_mols, const int* sis, const T* gh, const T* gc,
                        const T* gn, const T* go, T* gx, T* gy, T* gz, const int* acs_host,
                        void* stream)
{
    long long n_atoms = 0;
    if (int rc = check_acs(acs_host, &n_atoms)) return rc;
    if (n_mols < 0) return ANI_ERR_BAD_SIZE;
    if (n_atoms == 0) return ANI_OK;
    if (!gx || !gy || !gz) return ANI_ERR_NULL_POINTER;
    cudaStream_t st = (cudaStream_t)stream;
    const T* gin[kTypes] = {gh, gc, gn, go};
    // One CTA per molecule when the molecules are small and the upstream rows can be fetched with
    // 16-byte copies: writes every output itself, so no zero fill.
    if (n_mols > 0 && small_molecules(n_atoms, n_mols) && all_aligned16({gh, gc, gn, go}) &&
        (long long)n_mols * kMolGradClasses <= 0x7fffffffLL) {
        if (!xs || !ys || !zs || !types || !mos || !macs || !sis) return ANI_ERR_NULL_POINTER;
        for (int t = 0; t < kTypes; t++)
            if (acs_host[t] > 0 && !gin[t]) return ANI_ERR_NULL_POINTER;
        auto mol_kernel = featurize_grad_mol_kernel<T, kMolGradWarps>;
        const size_t mol_smem = mol_grad_smem_bytes<T, kMolGradWarps>();
        static thread_local int mol_configured_dev = -1;
        int dev = 0;
        ANI_CUDA(cudaGetDevice(&dev));
        if (mol_configured_dev != dev) {
            if (int rc = set_smem(mol_kernel, mol_smem)) return rc;
            mol_configured_dev = dev;
        }
        mol_kernel<<<n_mols * kMolGradClasses, kMolGradWarps * kWarp, mol_smem, st>>>(xs, ys, zs, types, mos, macs, n_mols, (int)n_atoms, sis, gh,
                                                          gc, gn, go, gx, gy, gz, acs_host[0], acs_host[1],
                                                          acs_host[2], acs_host[3]);
        ANI_CUDA(cudaGetLastError());
        return ANI_OK;
    }
    {
        const int threads = 256;
        long long blocks = (n_atoms + threads - 1) / threads;
        if (blocks > 1184) blocks = 1184;
        zero3_kernel<T><<<(int)blocks, threads, 0, st>>>(gx, gy, gz, (int)n_atoms);
        ANI_CUDA(cudaGetLastError());
    }
    if (n_mols == 0) return ANI_OK;
    if (!xs || !ys || !zs || !types || !mos || !macs || !sis) return ANI_ERR_NULL_POINTER;
    for (int t = 0; t < kTypes; t++)
        if (acs_host[t] > 0 && !gin[t]) return ANI_ERR_NULL_POINTER;

    auto kernel = featurize_grad_kernel<T, kNW>;
    const size_t smem = kNW * sizeof(GradWarpShared<T>);
    static thread_local int configured_dev = -1;
    int dev = 0;
    ANI_CUDA(cudaGetDevice(&dev));
    if (configured_dev != dev) {
        if (int rc = set_smem(kernel, smem)) return rc;
        configured_dev = dev;
    }
    static thread_local int cached_grid_dev = -1, cached_resident = 0;
    if (cached_grid_dev != dev) {
        if (int rc = featurizer_grid(kernel, smem, 1 << 24, &cached_resident)) return rc;
        cached_grid_dev = dev;
    }
    const int slot_shift = pick_slot_shift(n_atoms, n_mols);
    const long long needed = (long long)n_mols * ((1 << (slot_shift & 31)) / kNW);
    const int grid = (int)(needed < cached_resident ? needed : cached_resident);
    kernel<<<grid, kNW * kWarp, smem, st>>>(
        xs, ys, zs, types, mos, macs, n_mols, (int)n_atoms, slot_shift, sis, gh, gc, gn, go, gx, gy, gz,
        acs_host[0], acs_host[1], acs_host[2], acs_host[3]);
    ANI_CUDA(cudaGetLastError());
    return ANI_OK;
}

template <typename T>
int featurize_grad_inverse_impl(const T* xs, const T* ys, const T* zs, const int* types,
                                const int* mos, const int* macs, int n_mols, const int* sis,
                                const T* vx, const T* vy, const T* vz, T* oh, T* oc, T* on, T* oo,
                                const int* acs_host, void* stream)
{
    long long n_atoms = 0;
    if (int rc = check_acs(acs_host, &n_atoms)) return rc;
    if (n_mols < 0) return ANI_ERR_BAD_SIZE;
    if (n_mols == 0 || n_atoms == 0) return ANI_OK;
    if (!xs || !ys || !zs || !types || !mos || !macs || !sis || !vx || !vy || !vz)
        return ANI_ERR_NULL_POINTER;
    T* outs[kTypes] = {oh, oc, on, oo};
    for (int t = 0; t < kTypes; t++)
        if (acs_host[t] > 0 && !outs[t]) return ANI_ERR_NULL_POINTER;

    auto kernel = featurize_grad_inverse_kernel<T, kNW>;
    const size_t smem = kNW * sizeof(JvpWarpShared<T>);
    static thread_local int configured_dev = -1, cached_resident = 0;
    int dev = 0;
    ANI_CUDA(cudaGetDevice(&dev));
    if (configured_dev != dev) {
        if (int rc = set_smem(kernel, smem)) return rc;
        if (int rc = featurizer_grid(kernel, smem, 1 << 24, &cached_resident)) return rc;
        configured_dev = dev;
    }
    const int slot_shift = pick_slot_shift(n_atoms, n_mols);
    const long long needed = (long long)n_mols * ((1 << (slot_shift & 31)) / kNW);
    const int grid = (int)(needed < cached_resident ? needed : cached_resident);
    kernel<<<grid, kNW * kWarp, smem, (cudaStream_t)stream>>>(
        xs, ys, zs, types, mos, macs, n_mols, (int)n_atoms, slot_shift, sis, vx, vy, vz, oh, oc, on, oo,
        acs_host[0], acs_host[1], acs_host[2], acs_host[3]);
    ANI_CUDA(cudaGetLastError());
    return ANI_OK;
}

// Grid of the one-warp-per-molecule charge kernels: every molecule gets a warp, up to 16 CTAs per SM.
int charge_grid(int n_mols, int* grid)
{
    int dev = 0, sms = 0;
    ANI_CUDA(cudaGetDevice(&dev));
    ANI_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    const int needed = (n_mols + kNW - 1) / kNW;
    *grid = needed < sms * 16 ? needed : sms * 16;
    return ANI_OK;
}

template <typename T>
int charge_impl(const T* xs, const T* ys, const T* zs, const T* qs, const int* mos, const int* macs,
                int n_mols, int n_atoms, T* energies, void* stream)
{
    if (n_mols < 0 || n_atoms < 0) return ANI_ERR_BAD_SIZE;
    if (n_mols == 0) return ANI_OK;
    if (!mos || !macs || !energies) return ANI_ERR_NULL_POINTER;
    if (n_atoms > 0 && (!xs || !ys || !zs || !qs)) return ANI_ERR_NULL_POINTER;
    int grid = 0;
    if (int rc = charge_grid(n_mols, &grid)) return rc;
    charge_energy_kernel<T, kNW><<<grid, kNW * kWarp, 0, (cudaStream_t)stream>>>(
        xs, ys, zs, qs, mos, macs, n_mols, n_atoms, energies);
    ANI_CUDA(cudaGetLastError());
    return ANI_OK;
}

template <typename T>
int charge_grad_impl(const T* xs, const T* ys, const T* zs, const T* qs, const int* mos,
                     const int* macs, int n_mols, int n_atoms, const T* energy_grads, T* q_grads,
                     void* stream)
{
    if (n_mols < 0 || n_atoms < 0) return ANI_ERR_BAD_SIZE;
    if (n_atoms == 0) return ANI_OK;
    if (!xs || !ys || !zs || !qs || !q_grads) return ANI_ERR_NULL_POINTER;
    cudaStream_t st = (cudaStream_t)stream;
    ANI_CUDA(cudaMemsetAsync(q_grads, 0, (size_t)n_atoms * sizeof(T), st));
    if (n_mols == 0) return ANI_OK;
    if (!mos || !macs || !energy_grads) return ANI_ERR_NULL_POINTER;
    int grid = 0;
    if (int rc = charge_grid(n_mols, &grid)) return rc;
    charge_grad_kernel<T, kNW><<<grid, kNW * kWarp, 0, st>>>(xs, ys, zs, qs, mos, macs, n_mols, n_atoms,
                                                             energy_grads, q_grads);
    ANI_CUDA(cudaGetLastError());
    return ANI_OK;
}

template <int ACT, bool SPLIT> int mlp_launch(const MlpParams& p, int n_tiles, cudaStream_t st)
{
    auto kernel = mlp_forward_kernel<ACT, SPLIT>;
    const size_t smem = sizeof(MlpShared) + 1024;
    static thread_local int configured_dev = -1;
    int dev = 0;
    ANI_CUDA(cudaGetDevice(&dev));
    if (configured_dev != dev) {
        if (int rc = set_smem(kernel, smem)) return rc;
        configured_dev = dev;
    }
    kernel<<<n_tiles, kMlpAllThreads, smem, st>>>(p);
    ANI_CUDA(cudaGetLastError());
    return ANI_OK;
}

template <bool SPLIT> int mlp_backward_launch(const MlpBackwardParams& p, int n_tiles, cudaStream_t st)
{
    auto kernel = mlp_backward_kernel<SPLIT>;
    const size_t smem = sizeof(MlpShared) + 1024;
    static thread_local int configured_dev = -1;
    int dev = 0;
    ANI_CUDA(cudaGetDevice(&dev));
    if (configured_dev != dev) {
        if (int rc = set_smem(kernel, smem)) return rc;
        configured_dev = dev;
    }
    kernel<<<n_tiles, kMlpAllThreads, smem, st>>>(p);
    ANI_CUDA(cudaGetLastError());
    return ANI_OK;
}

template <bool SPLIT> int mlp_wgrad_launch(const MlpWgradParams& p, int n_ranges, cudaStream_t st)
{
    auto kernel = mlp_wgrad_kernel<SPLIT>;
    const size_t smem = sizeof(MlpShared) + 1024;
    static thread_local int configured_dev = -1;
    int dev = 0;
    ANI_CUDA(cudaGetDevice(&dev));
    if (configured_dev != dev) {
        if (int rc = set_smem(kernel, smem)) return rc;
        configured_dev = dev;
    }
    kernel<<<dim3(n_ranges, kWgradBlocks), kMlpAllThreads, smem, st>>>(p);
    ANI_CUDA(cudaGetLastError());
    return ANI_OK;
}

template <int ACT> int mlp_launch_act(const MlpParams& p, int n_tiles, bool split, cudaStream_t st)
{
    return split ? mlp_launch<ACT, true>(p, n_tiles, st) : mlp_launch<ACT, false>(p, n_tiles, st);
}

}  // namespace

extern "C" {

int ani_feature_size(void) { return ani::kTotal; }

const char* ani_status_string(int status)
{
    switch (status) {
        case ANI_OK: return "ok";
        case ANI_ERR_NULL_POINTER: return "a required pointer argument is NULL";
        case ANI_ERR_BAD_SIZE: return "negative or inconsistent size argument";
        case ANI_ERR_CUDA: return "CUDA runtime error (see ani_last_cuda_error)";
        case ANI_ERR_BAD_ELEMENT: return "element id outside 0..3 in atomic_numbers";
        case ANI_ERR_BAD_INDEX: return "molecule offset/count or scatter index out of range";
        case ANI_ERR_TOO_MANY_ATOMS: return "size beyond what this entry point supports";
        case ANI_ERR_TIMEOUT: return "a bounded device-side wait ran out";
        case ANI_ERR_MISALIGNED: return "a pointer that must be 16-byte aligned is not";
        case ANI_ERR_CAPTURE:
            return "first-use set-up (scratch allocation or address look-up) cannot run while the stream is being "
                   "captured: make the same call once outside the capture";
        default: return "unknown status";
    }
}

const char* ani_last_cuda_error(void) { return cudaGetErrorString(t_last_error); }

int ani_device_status(void* stream)
{
    ANI_CUDA(cudaStreamSynchronize((cudaStream_t)stream));
    int v = 0;
    ANI_CUDA(cudaMemcpyFromSymbol(&v, ani::g_status, sizeof(int)));
    if (v != 0) {
        const int zero = 0;
        ANI_CUDA(cudaMemcpyToSymbol(ani::g_status, &zero, sizeof(int)));
    }
    return v;
}

int ani_sort(const int* atomic_numbers, int n_atoms, int* scatter_idxs, int* gather_idxs,
             int* atom_counts, void* stream)
{
    if (n_atoms < 0) return ANI_ERR_BAD_SIZE;
    if (!atom_counts) return ANI_ERR_NULL_POINTER;
    cudaStream_t st = (cudaStream_t)stream;
    if (n_atoms == 0) {
        sort_empty_kernel<<<1, 32, 0, st>>>(atom_counts);
        ANI_CUDA(cudaGetLastError());
        return ANI_OK;
    }
    if (!atomic_numbers || !scatter_idxs || !gather_idxs) return ANI_ERR_NULL_POINTER;
    const int n_tiles = (n_atoms + kSortTile - 1) / kSortTile;
    if (n_atoms <= kSortSingleLaunchMax) {
        sort_single_kernel<<<n_tiles, kSortThreads, 0, st>>>(atomic_numbers, n_atoms, scatter_idxs,
                                                             gather_idxs, atom_counts);
        ANI_CUDA(cudaGetLastError());
        return ANI_OK;
    }
    int* scratch = nullptr;
    if (int rc = sort_scratch((size_t)(n_tiles + 1) * kTypes * sizeof(int), st, &scratch)) return rc;
    sort_histogram_kernel<<<n_tiles, kSortThreads, 0, st>>>(atomic_numbers, n_atoms, scratch);
    ANI_CUDA(cudaGetLastError());
    sort_scan_kernel<<<1, kSortThreads, 0, st>>>(scratch, n_tiles);
    ANI_CUDA(cudaGetLastError());
    sort_rank_kernel<<<n_tiles, kSortThreads, 0, st>>>(atomic_numbers, n_atoms, scratch, n_tiles,
                                                       scatter_idxs, gather_idxs, atom_counts);
    ANI_CUDA(cudaGetLastError());
    return ANI_OK;
}

int ani_sort_noalloc(const int* atomic_numbers, int n_atoms, int* scatter_idxs, int* gather_idxs,
                     int* atom_counts, void* stream)
{
    if (n_atoms < 0) return ANI_ERR_BAD_SIZE;
    if (n_atoms > kSortStaticMaxAtoms) return ANI_ERR_TOO_MANY_ATOMS;
    if (!atom_counts) return ANI_ERR_NULL_POINTER;
    cudaStream_t st = (cudaStream_t)stream;
    if (n_atoms == 0) {
        sort_empty_kernel<<<1, 32, 0, st>>>(atom_counts);
        ANI_CUDA(cudaGetLastError());
        return ANI_OK;
    }
    if (!atomic_numbers || !scatter_idxs || !gather_idxs) return ANI_ERR_NULL_POINTER;
    int* scratch = nullptr;
    if (int rc = sort_static_scratch(st, &scratch)) return rc;
    // Every scratch entry that is read is written first by the same call (the histogram kernel
    // fills entries [0, n_tiles), the scan kernel entry n_tiles), so nothing has to be cleared.
    const int n_tiles = (n_atoms + kSortTile - 1) / kSortTile;
    sort_histogram_kernel<<<n_tiles, kSortThreads, 0, st>>>(atomic_numbers, n_atoms, scratch);
    ANI_CUDA(cudaGetLastError());
    sort_scan_kernel<<<1, kSortThreads, 0, st>>>(scratch, n_tiles);
    ANI_CUDA(cudaGetLastError());
    sort_rank_kernel<<<n_tiles, kSortThreads, 0, st>>>(atomic_numbers, n_atoms, scratch, n_tiles,
                                                       scatter_idxs, gather_idxs, atom_counts);
    ANI_CUDA(cudaGetLastError());
    return ANI_OK;
}

int ani_sort_noalloc_max_atoms(void) { return kSortStaticMaxAtoms; }

int ani_featurize_f32(const float* xs, const float* ys, const float* zs, const int* atomic_numbers,
                      const int* mol_offsets, const int* mol_atom_counts, int n_mols,
                      const int* scatter_idxs, float* out_h, float* out_c, float* out_n,
                      float* out_o, const int* acs_host, void* stream)
{
    return featurize_impl<float>(xs, ys, zs, atomic_numbers, mol_offsets, mol_atom_counts, n_mols,
                                 scatter_idxs, out_h, out_c, out_n, out_o, acs_host, stream);
}

int ani_featurize_f64(const double* xs, const double* ys, const double* zs,
                      const int* atomic_numbers, const int* mol_offsets, const int* mol_atom_counts,
                      int n_mols, const int* scatter_idxs, double* out_h, double* out_c,
                      double* out_n, double* out_o, const int* acs_host, void* stream)
{
    return featurize_impl<double>(xs, ys, zs, atomic_numbers, mol_offsets, mol_atom_counts, n_mols,
                                  scatter_idxs, out_h, out_c, out_n, out_o, acs_host, stream);
}

int ani_featurize_grad_f32(const float* xs, const float* ys, const float* zs,
                           const int* atomic_numbers, const int* mol_offsets,
                           const int* mol_atom_counts, int n_mols, const int* scatter_idxs,
                           const float* grad_h, const float* grad_c, const float* grad_n,
                           const float* grad_o, float* x_grads, float* y_grads, float* z_grads,
                           const int* acs_host, void* stream)
{
    return featurize_grad_impl<float>(xs, ys, zs, atomic_numbers, mol_offsets, mol_atom_counts,
                                      n_mols, scatter_idxs, grad_h, grad_c, grad_n, grad_o,
                                      x_grads, y_grads, z_grads, acs_host, stream);
}

int ani_featurize_grad_f64(const double* xs, const double* ys, const double* zs,
                           const int* atomic_numbers, const int* mol_offsets,
                           const int* mol_atom_counts, int n_mols, const int* scatter_idxs,
                           const double* grad_h, const double* grad_c, const double* grad_n,
                           const double* grad_o, double* x_grads, double* y_grads,
                           double* z_grads, const int* acs_host, void* stream)
{
    return featurize_grad_impl<double>(xs, ys, zs, atomic_numbers, mol_offsets, mol_atom_counts,
                                       n_mols, scatter_idxs, grad_h, grad_c, grad_n, grad_o,
                                       x_grads, y_grads, z_grads, acs_host, stream);
}

int ani_featurize_grad_inverse_f32(const float* xs, const float* ys, const float* zs,
                                   const int* atomic_numbers, const int* mol_offsets,
                                   const int* mol_atom_counts, int n_mols, const int* scatter_idxs,
                                   const float* x_grads, const float* y_grads, const float* z_grads,
                                   float* out_h, float* out_c, float* out_n, float* out_o,
                                   const int* acs_host, void* stream)
{
    return featurize_grad_inverse_impl<float>(xs, ys, zs, atomic_numbers, mol_offsets,
                                              mol_atom_counts, n_mols, scatter_idxs, x_grads,
                                              y_grads, z_grads, out_h, out_c, out_n, out_o,
                                              acs_host, stream);
}

int ani_featurize_grad_inverse_f64(const double* xs, const double* ys, const double* zs,
                                   const int* atomic_numbers, const int* mol_offsets,
                                   const int* mol_atom_counts, int n_mols, const int* scatter_idxs,
                                   const double* x_grads, const double* y_grads,
                                   const double* z_grads, double* out_h, double* out_c,
                                   double* out_n, double* out_o, const int* acs_host, void* stream)
{
    return featurize_grad_inverse_impl<double>(xs, ys, zs, atomic_numbers, mol_offsets,
                                               mol_atom_counts, n_mols, scatter_idxs, x_grads,
                                               y_grads, z_grads, out_h, out_c, out_n, out_o,
                                               acs_host, stream);
}

int ani_mlp_forward_f32(const ani_mlp_args* a, const int* acs_host, int activation,
                        int split_precision, void* stream)
{
    long long n_atoms = 0;
    if (!a) return ANI_ERR_NULL_POINTER;
    if (int rc = check_acs(acs_host, &n_atoms)) return rc;
    if (activation < 0 || activation > 3) return ANI_ERR_BAD_SIZE;
    if (n_atoms == 0) return ANI_OK;
    MlpParams p;
    int tiles = 0;
    for (int t = 0; t < kTypes; t++) {
        p.tile_start[t] = tiles;
        p.count[t] = acs_host[t];
        tiles += (acs_host[t] + kMlpTile - 1) / kMlpTile;
        if (acs_host[t] > 0 && (!a->features[t] || !a->w1[t] || !a->b1[t] || !a->w2[t] || !a->b2[t] ||
                                !a->w3[t] || !a->b3[t] || !a->w4[t] || !a->b4[t] || !a->energy[t]))
            return ANI_ERR_NULL_POINTER;
        if (acs_host[t] > 0 && !all_aligned16({a->features[t], a->w1[t], a->w2[t], a->w3[t], a->act1[t], a->act2[t],
                                               a->act3[t], a->dact1[t], a->dact2[t], a->dact3[t]}))
            return ANI_ERR_MISALIGNED;
        p.feat[t] = a->features[t];
        p.w1[t] = a->w1[t]; p.b1[t] = a->b1[t];
        p.w2[t] = a->w2[t]; p.b2[t] = a->b2[t];
        p.w3[t] = a->w3[t]; p.b3[t] = a->b3[t];
        p.w4[t] = a->w4[t];   p.b4[t] = a->b4[t];
        p.energy[t] = a->energy[t];
        p.act1[t] = a->act1[t]; p.act2[t] = a->act2[t]; p.act3[t] = a->act3[t];
        p.dact1[t] = a->dact1[t]; p.dact2[t] = a->dact2[t]; p.dact3[t] = a->dact3[t];
        p.packed[t] = (const unsigned char*)a->packed[t];
        if (reinterpret_cast<uintptr_t>(a->packed[t]) & 15) return ANI_ERR_MISALIGNED;
    }
    p.tile_start[kTypes] = tiles;
    cudaStream_t st = (cudaStream_t)stream;
    const bool split = split_precision != 0;
    switch (activation) {
        case kActCelu: return mlp_launch_act<kActCelu>(p, tiles, split, st);
        case kActGaussian: return mlp_launch_act<kActGaussian>(p, tiles, split, st);
        case kActNormal: return mlp_launch_act<kActNormal>(p, tiles, split, st);
        default: return mlp_launch_act<kActSoftplus>(p, tiles, split, st);
    }
}

size_t ani_mlp_packed_bytes(void) { return (size_t)kPackChunks * kPackedChunkBytes; }

int ani_mlp_pack_weights_f32(const ani_mlp_pack_args* a, void* stream)
{
    if (!a) return ANI_ERR_NULL_POINTER;
    MlpPackParams p;
    bool any = false;
    for (int t = 0; t < kTypes; t++) {
        p.w1[t] = a->w1[t]; p.w2[t] = a->w2[t]; p.w3[t] = a->w3[t];
        p.packed[t] = (unsigned char*)a->packed[t];
        if (!a->packed[t]) continue;
        if (!a->w1[t] || !a->w2[t] || !a->w3[t]) return ANI_ERR_NULL_POINTER;
        if (reinterpret_cast<uintptr_t>(a->packed[t]) & 15) return ANI_ERR_MISALIGNED;
        any = true;
    }
    if (!any) return ANI_OK;
    mlp_pack_kernel<<<dim3(kPackChunks, kTypes), kMlpThreads, 0, (cudaStream_t)stream>>>(p);
    ANI_CUDA(cudaGetLastError());
    return ANI_OK;
}

int ani_mlp_backward_f32(const ani_mlp_backward_args* a, const int* acs_host, int split_precision,
                         void* stream)
{
    long long n_atoms = 0;
    if (!a) return ANI_ERR_NULL_POINTER;
    if (int rc = check_acs(acs_host, &n_atoms)) return rc;
    if (n_atoms == 0) return ANI_OK;
    MlpBackwardParams p;
    int tiles = 0;
    for (int t = 0; t < kTypes; t++) {
        p.tile_start[t] = tiles;
        p.count[t] = acs_host[t];
        tiles += (acs_host[t] + kMlpTile - 1) / kMlpTile;
        if (acs_host[t] > 0 && (!a->grad_energy[t] || !a->w1[t] || !a->w2[t] || !a->w3[t] || !a->w4[t] ||
                                !a->dact1[t] || !a->dact2[t] || !a->dact3[t] || !a->dz1[t] || !a->dz2[t] ||
                                !a->dz3[t]))
            return ANI_ERR_NULL_POINTER;
        if (acs_host[t] > 0 && !all_aligned16({a->w1[t], a->w2[t], a->w3[t], a->dact1[t], a->dact2[t], a->dact3[t],
                                               a->dz1[t], a->dz2[t], a->dz3[t], a->grad_features[t]}))
            return ANI_ERR_MISALIGNED;
        p.grad_energy[t] = a->grad_energy[t];
        p.w1[t] = a->w1[t]; p.w2[t] = a->w2[t]; p.w3[t] = a->w3[t]; p.w4[t] = a->w4[t];
        p.dact1[t] = a->dact1[t]; p.dact2[t] = a->dact2[t]; p.dact3[t] = a->dact3[t];
        p.dz1[t] = a->dz1[t]; p.dz2[t] = a->dz2[t]; p.dz3[t] = a->dz3[t];
        p.grad_feat[t] = a->grad_features[t];
        p.packed[t] = (const unsigned char*)a->packed[t];
        if (reinterpret_cast<uintptr_t>(a->packed[t]) & 15) return ANI_ERR_MISALIGNED;
    }
    p.tile_start[kTypes] = tiles;
    cudaStream_t st = (cudaStream_t)stream;
    return split_precision ? mlp_backward_launch<true>(p, tiles, st) : mlp_backward_launch<false>(p, tiles, st);
}

int ani_mlp_weight_grad_f32(const ani_mlp_weight_grad_args* a, const int* acs_host, int split_precision,
                            void* stream)
{
    long long n_atoms = 0;
    if (!a) return ANI_ERR_NULL_POINTER;
    if (int rc = check_acs(acs_host, &n_atoms)) return rc;
    if (n_atoms == 0) return ANI_OK;
    MlpWgradParams p;
    for (int t = 0; t < kTypes; t++) {
        p.count[t] = acs_host[t];
        if (acs_host[t] > 0 && (!a->features[t] || !a->act1[t] || !a->act2[t] || !a->dz1[t] || !a->dz2[t] ||
                                !a->dz3[t] || !a->dw1[t] || !a->dw2[t] || !a->dw3[t] || !a->db1[t] ||
                                !a->db2[t] || !a->db3[t] || !a->act3[t] || !a->grad_energy[t] ||
                                !a->dw4[t] || !a->db4[t]))
            return ANI_ERR_NULL_POINTER;
        if (acs_host[t] > 0) {
            const void* vec[] = {a->features[t], a->act1[t], a->act2[t], a->act3[t], a->dz1[t], a->dz2[t],
                                 a->dz3[t], a->dw1[t], a->dw2[t], a->dw3[t]};
            for (const void* ptr : vec)
                if (reinterpret_cast<uintptr_t>(ptr) & 15) return ANI_ERR_MISALIGNED;
        }
        p.feat[t] = a->features[t]; p.act1[t] = a->act1[t]; p.act2[t] = a->act2[t];
        p.dz1[t] = a->dz1[t]; p.dz2[t] = a->dz2[t]; p.dz3[t] = a->dz3[t];
        p.dw1[t] = a->dw1[t]; p.dw2[t] = a->dw2[t]; p.dw3[t] = a->dw3[t];
        p.db1[t] = a->db1[t]; p.db2[t] = a->db2[t]; p.db3[t] = a->db3[t];
        p.act3[t] = a->act3[t]; p.grad_energy[t] = a->grad_energy[t];
        p.dw4[t] = a->dw4[t]; p.db4[t] = a->db4[t];
    }
    // atoms per CTA: the smallest multiple of 64 for which the grid fits the SMs once (the
    // kernels run one CTA per SM, so a second partial wave would double the time)
    int dev = 0, sms = 0;
    ANI_CUDA(cudaGetDevice(&dev));
    ANI_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    int range = 256;
    for (;; range += 64) {
        long long ctas = 0;
        for (int t = 0; t < kTypes; t++) ctas += (acs_host[t] + range - 1) / range;
        if (ctas * kWgradBlocks <= sms || range >= (1 << 20)) break;
    }
    p.range = range;
    int ranges = 0;
    for (int t = 0; t < kTypes; t++) {
        p.range_start[t] = ranges;
        ranges += (acs_host[t] + range - 1) / range;
    }
    p.range_start[kTypes] = ranges;
    cudaStream_t st = (cudaStream_t)stream;
    return split_precision ? mlp_wgrad_launch<true>(p, ranges, st) : mlp_wgrad_launch<false>(p, ranges, st);
}

int ani_molecule_energy_f32(const float* atom_energy_sorted, const int* gather_idxs, const int* mol_offsets,
                            const int* mol_atom_counts, int n_mols, int n_atoms, const float* labels,
                            float grad_scale, float* mol_energy, float* l2s, float* grad_atom_energy_sorted,
                            void* stream)
{
    if (n_mols < 0 || n_atoms < 0) return ANI_ERR_BAD_SIZE;
    if (n_mols == 0) return ANI_OK;
    if (!mol_offsets || !mol_atom_counts || !mol_energy) return ANI_ERR_NULL_POINTER;
    if (n_atoms > 0 && (!atom_energy_sorted || !gather_idxs)) return ANI_ERR_NULL_POINTER;
    int grid = 0;
    if (int rc = charge_grid(n_mols, &grid)) return rc;
    molecule_energy_kernel<kNW><<<grid, kNW * kWarp, 0, (cudaStream_t)stream>>>(
        atom_energy_sorted, gather_idxs, mol_offsets, mol_atom_counts, n_mols, n_atoms, labels, grad_scale,
        mol_energy, l2s, grad_atom_energy_sorted);
    ANI_CUDA(cudaGetLastError());
    return ANI_OK;
}

int ani_nadam_step_f32(float* params, const float* grads, float* m, float* v, float* ema,
                       long long n, const float* hyper, void* state, void* stream)
{
    if (n < 0) return ANI_ERR_BAD_SIZE;
    if (n == 0) return ANI_OK;
    if (!params || !grads || !m || !v || !hyper || !state) return ANI_ERR_NULL_POINTER;
    int dev = 0, sms = 0;
    ANI_CUDA(cudaGetDevice(&dev));
    ANI_CUDA(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    const long long want = (n + 4 * kOptimThreads - 1) / (4 * kOptimThreads);
    const int grid = (int)(want < (long long)sms * 4 ? want : (long long)sms * 4);
    cudaStream_t st = (cudaStream_t)stream;
    grad_sumsq_kernel<<<grid, kOptimThreads, 0, st>>>(grads, n, (OptimState*)state);
    ANI_CUDA(cudaGetLastError());
    nadam_update_kernel<<<grid, kOptimThreads, 0, st>>>(params, grads, m, v, ema, n, (const OptimHyper*)hyper,
                                                        (OptimState*)state);
    ANI_CUDA(cudaGetLastError());
    return ANI_OK;
}

int ani_clip_rows_f32(float* params, const int* row_offsets, const int* row_lengths, int n_rows, float max_norm,
                      void* stream)
{
    if (n_rows < 0 || !(max_norm > 0.0f)) return ANI_ERR_BAD_SIZE;
    if (n_rows == 0) return ANI_OK;
    if (!params || !row_offsets || !row_lengths) return ANI_ERR_NULL_POINTER;
    const int per_block = kOptimThreads / kWarp;
    const int grid = (n_rows + per_block - 1) / per_block;
    clip_rows_kernel<<<grid, kOptimThreads, 0, (cudaStream_t)stream>>>(params, row_offsets, row_lengths, n_rows,
                                                                       max_norm);
    ANI_CUDA(cudaGetLastError());
    return ANI_OK;
}

int ani_scale_by_loss_f32(float* grads, long long n, const float* l2s, int n_mols, int kind, float* rmse_out,
                          void* stream)
{
    if (n < 0 || n_mols <= 0 || (kind != 1 && kind != 2)) return ANI_ERR_BAD_SIZE;
    if (!l2s || (n > 0 && !grads)) return ANI_ERR_NULL_POINTER;
    const long long blocks = std::max<long long>(1, std::min<long long>((n + kOptimThreads - 1) / kOptimThreads, 296));
    loss_scale_kernel<<<(int)blocks, kOptimThreads, 0, (cudaStream_t)stream>>>(grads, n, l2s, n_mols, kind, rmse_out);
    ANI_CUDA(cudaGetLastError());
    return ANI_OK;
}

int ani_charge_f32(const float* xs, const float* ys, const float* zs, const float* qs,
                   const int* mol_offsets, const int* mol_atom_counts, int n_mols, int n_atoms,
                   float* charge_energies, void* stream)
{
    return charge_impl<float>(xs, ys, zs, qs, mol_offsets, mol_atom_counts, n_mols, n_atoms,
                              charge_energies, stream);
}

int ani_charge_f64(const double* xs, const double* ys, const double* zs, const double* qs,
                   const int* mol_offsets, const int* mol_atom_counts, int n_mols, int n_atoms,
                   double* charge_energies, void* stream)
{
    return charge_impl<double>(xs, ys, zs, qs, mol_offsets, mol_atom_counts, n_mols, n_atoms,
                               charge_energies, stream);
}

int ani_charge_grad_f32(const float* xs, const float* ys, const float* zs, const float* qs,
                        const int* mol_offsets, const int* mol_atom_counts, int n_mols, int n_atoms,
                        const float* grads, float* q_grads, void* stream)
{
    return charge_grad_impl<float>(xs, ys, zs, qs, mol_offsets, mol_atom_counts, n_mols, n_atoms,
                                   grads, q_grads, stream);
}

int ani_charge_grad_f64(const double* xs, const double* ys, const double* zs, const double* qs,
                        const int* mol_offsets, const int* mol_atom_counts, int n_mols, int n_atoms,
                        const double* grads, double* q_grads, void* stream)
{
    return charge_grad_impl<double>(xs, ys, zs, qs, mol_offsets, mol_atom_counts, n_mols, n_atoms,
                                    grads, q_grads, stream);
}

int ani_host_pack_batch(const ani_host_pack_args* args)
{
    if (!args) return ANI_ERR_NULL_POINTER;
    return ani::host_pack_batch(*args);
}

struct ani_feeder {
    ani::Feeder impl;
    ani_feeder(int device, const ani_feeder_slot* slots, int n) : impl(device, slots, n) {}
};

int ani_feeder_create(int device, const ani_feeder_slot* slots, int n_slots, ani_feeder** out)
{
    if (!slots || !out) return ANI_ERR_NULL_POINTER;
    if (n_slots <= 0) return ANI_ERR_BAD_SIZE;
    for (int s = 0; s < n_slots; s++)
        if (!slots[s].host_arena || (device >= 0 && !slots[s].dev_arena)) return ANI_ERR_NULL_POINTER;
    ani_feeder* f = new (std::nothrow) ani_feeder(device, slots, n_slots);
    if (!f) return ANI_ERR_CUDA;
    if (int rc = f->impl.init()) {
        delete f;
        return rc;
    }
    *out = f;
    return ANI_OK;
}

int ani_feeder_begin(ani_feeder* f, const long long* order, long long n_order, int batch_size)
{
    return f ? f->impl.begin(order, n_order, batch_size) : ANI_ERR_NULL_POINTER;
}

int ani_feeder_next(ani_feeder* f, ani_feeder_batch* out)
{
    return f && out ? f->impl.next(out) : ANI_ERR_NULL_POINTER;
}

int ani_feeder_wait(ani_feeder* f, int slot, void* stream)
{
    return f ? f->impl.wait(slot, static_cast<cudaStream_t>(stream)) : ANI_ERR_NULL_POINTER;
}

int ani_feeder_release(ani_feeder* f, int slot, void* stream)
{
    return f ? f->impl.release(slot, static_cast<cudaStream_t>(stream)) : ANI_ERR_NULL_POINTER;
}

int ani_feeder_end(ani_feeder* f)
{
    if (!f) return ANI_ERR_NULL_POINTER;
    f->impl.end();
    return ANI_OK;
}

int ani_feeder_destroy(ani_feeder* f)
{
    if (!f) return ANI_OK;
    f->impl.end();
    const int rc = f->impl.drain();
    delete f;
    return rc;
}

struct ani_peer {
    int device = 0, rank = 0, world = 1, grid = 1;
    int two_halves = 0;                  // slice means + exchange (more than four ranks)
    long long capacity = 0;              // floats per staging buffer
    unsigned char* block = nullptr;      // local: [flags | staging 0 | staging 1]
    ani::PeerState* state = nullptr;     // local
    unsigned char* peer_block[ani::kPeerMaxRanks] = {};
    bool mapped[ani::kPeerMaxRanks] = {};   // opened through CUDA IPC (to be closed)
};

int ani_peer_create(int rank, int world, long long n_floats, ani_peer** out)
{
    if (!out) return ANI_ERR_NULL_POINTER;
    if (world < 1 || world > ani::kPeerMaxRanks || rank < 0 || rank >= world || n_floats <= 0) return ANI_ERR_BAD_SIZE;
    ani_peer* p = new (std::nothrow) ani_peer();
    if (!p) return ANI_ERR_CUDA;
    p->rank = rank;
    p->world = world;
    p->capacity = (n_floats + 3) / 4 * 4;
    cudaDeviceProp prop;
    cudaError_t e = cudaGetDevice(&p->device);
    if (e == cudaSuccess) e = cudaGetDeviceProperties(&prop, p->device);
    // [flags | staging 0, 1 (every rank's contribution) | staging 2, 3 (this rank's slice means)]
    const size_t bytes = ani::kPeerFlagBytes + 4 * (size_t)p->capacity * sizeof(float);
    if (e == cudaSuccess) e = cudaMalloc(&p->block, bytes);
    if (e == cudaSuccess) e = cudaMemset(p->block, 0, bytes);
    if (e == cudaSuccess) e = cudaMalloc(&p->state, sizeof(ani::PeerState));
    if (e == cudaSuccess) {
        ani::PeerState init{0ull, 0ull, 0ull, 0u, ani::kPeerSpinLimit};
        e = cudaMemcpy(p->state, &init, sizeof(init), cudaMemcpyHostToDevice);
    }
    if (e != cudaSuccess) {
        if (p->block) cudaFree(p->block);
        if (p->state) cudaFree(p->state);
        delete p;
        return cuda_fail(e);
    }
    const long long groups = p->capacity / 4;
    p->grid = (int)std::max<long long>(1, std::min<long long>((groups + ani::kPeerThreads - 1) / ani::kPeerThreads,
                                                               std::min(prop.multiProcessorCount, ani::kPeerMaxBlocks)));
    p->peer_block[rank] = p->block;
    p->two_halves = world > 4 ? 1 : 0;
    *out = p;
    return ANI_OK;
}

int ani_peer_handle(ani_peer* p, void* out64)
{
    if (!p || !out64) return ANI_ERR_NULL_POINTER;
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "the handle is exchanged as 64 bytes");
    cudaIpcMemHandle_t h;
    ANI_CUDA(cudaIpcGetMemHandle(&h, p->block));
    memcpy(out64, &h, sizeof(h));
    return ANI_OK;
}

int ani_peer_connect(ani_peer* p, int q, const void* handle64)
{
    if (!p || !handle64) return ANI_ERR_NULL_POINTER;
    if (q < 0 || q >= p->world || q == p->rank || p->peer_block[q]) return ANI_ERR_BAD_INDEX;
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, sizeof(h));
    void* ptr = nullptr;
    ANI_CUDA(cudaIpcOpenMemHandle(&ptr, h, cudaIpcMemLazyEnablePeerAccess));
    p->peer_block[q] = static_cast<unsigned char*>(ptr);
    p->mapped[q] = true;
    return ANI_OK;
}

int ani_peer_connect_raw(ani_peer* p, int q, void* block)
{
    if (!p || !block) return ANI_ERR_NULL_POINTER;
    if (q < 0 || q >= p->world || q == p->rank || p->peer_block[q]) return ANI_ERR_BAD_INDEX;
    p->peer_block[q] = static_cast<unsigned char*>(block);
    return ANI_OK;
}

void* ani_peer_block(ani_peer* p) { return p ? p->block : nullptr; }

int ani_peer_set_two_halves(ani_peer* p, int on)
{
    if (!p) return ANI_ERR_NULL_POINTER;
    p->two_halves = on ? 1 : 0;
    return ANI_OK;
}

int ani_peer_set_spin_limit(ani_peer* p, unsigned tries)
{
    if (!p) return ANI_ERR_NULL_POINTER;
    ANI_CUDA(cudaMemcpy(&p->state->spin_limit, &tries, sizeof(tries), cudaMemcpyHostToDevice));
    return ANI_OK;
}

int ani_peer_mean_f32(ani_peer* p, float* buffer, long long n, void* stream)
{
    if (!p || !buffer) return ANI_ERR_NULL_POINTER;
    if (n < 0 || n > p->capacity || (n & 3)) return ANI_ERR_BAD_SIZE;
    if (reinterpret_cast<uintptr_t>(buffer) & 15) return ANI_ERR_MISALIGNED;
    ani::PeerParams a{};
    a.buffer = buffer;
    a.n4 = n / 4;
    a.stage_floats = p->capacity;
    a.rank = p->rank;
    a.world = p->world;
    for (int q = 0; q < p->world; q++) {
        if (!p->peer_block[q]) return ANI_ERR_NULL_POINTER;   // a rank that was never connected
        a.flags[q] = reinterpret_cast<unsigned*>(p->peer_block[q]);
        a.stage[q] = reinterpret_cast<float*>(p->peer_block[q] + ani::kPeerFlagBytes);
    }
    a.state = p->state;
    a.inv_world = 1.0f / (float)p->world;
    a.two_halves = p->two_halves;
    ani::peer_mean_kernel<<<p->grid, ani::kPeerThreads, 0, (cudaStream_t)stream>>>(a);
    ANI_CUDA(cudaGetLastError());
    return ANI_OK;
}

int ani_peer_destroy(ani_peer* p)
{
    if (!p) return ANI_OK;
    cudaDeviceSynchronize();
    for (int q = 0; q < p->world; q++)
        if (p->mapped[q]) cudaIpcCloseMemHandle(p->peer_block[q]);
    cudaFree(p->block);
    cudaFree(p->state);
    delete p;
    return ANI_OK;
}

int ani_network_pass_f32(const ani_pass_args* a, void* stream)
{
    if (!a) return ANI_ERR_NULL_POINTER;
    long long n_atoms = 0;
    if (int rc = check_acs(a->acs_host, &n_atoms)) return rc;
    if (a->n_atoms < 0 || a->n_mols < 0 || n_atoms != a->n_atoms) return ANI_ERR_BAD_SIZE;
    const int* acs = a->acs_host;
    size_t start[kTypes];   // first row of each element
    size_t at = 0;
    for (int t = 0; t < kTypes; t++) {
        start[t] = at;
        at += (size_t)acs[t];
    }
    auto rows = [&](float* base, int t, int width) -> float* {
        return base && acs[t] > 0 ? base + start[t] * (size_t)width : nullptr;
    };
    if (a->phases & ANI_PASS_PACK) {
        ani_mlp_pack_args p;
        for (int t = 0; t < kTypes; t++) {
            p.w1[t] = a->w1[t]; p.w2[t] = a->w2[t]; p.w3[t] = a->w3[t];
            p.packed[t] = a->packed[t];
        }
        if (int rc = ani_mlp_pack_weights_f32(&p, stream)) return rc;
    }
    if (a->phases & ANI_PASS_FEATURIZE) {
        if (int rc = ani_sort(a->atomic_numbers, a->n_atoms, a->scatter_idxs, a->gather_idxs, a->atom_counts, stream))
            return rc;
        if (int rc = ani_featurize_f32(a->xs, a->ys, a->zs, a->atomic_numbers, a->mol_offsets, a->mol_atom_counts,
                                       a->n_mols, a->scatter_idxs, rows(a->features, 0, kTotal),
                                       rows(a->features, 1, kTotal), rows(a->features, 2, kTotal),
                                       rows(a->features, 3, kTotal), acs, stream))
            return rc;
    }
    if (a->phases & ANI_PASS_FORWARD) {
        ani_mlp_args f;
        for (int t = 0; t < kTypes; t++) {
            f.features[t] = rows(a->features, t, kTotal);
            f.w1[t] = a->w1[t]; f.b1[t] = a->b1[t]; f.w2[t] = a->w2[t]; f.b2[t] = a->b2[t];
            f.w3[t] = a->w3[t]; f.b3[t] = a->b3[t]; f.w4[t] = a->w4[t]; f.b4[t] = a->b4[t];
            f.energy[t] = rows(a->energy_sorted, t, 1);
            f.act1[t] = rows(a->act1, t, kMlpH1); f.act2[t] = rows(a->act2, t, kMlpH2); f.act3[t] = rows(a->act3, t, kMlpH3);
            f.dact1[t] = rows(a->dact1, t, kMlpH1); f.dact2[t] = rows(a->dact2, t, kMlpH2);
            f.dact3[t] = rows(a->dact3, t, kMlpH3);
            f.packed[t] = a->packed[t];
        }
        if (int rc = ani_mlp_forward_f32(&f, acs, a->activation, a->split_precision, stream)) return rc;
    }
    if (a->phases & ANI_PASS_ENERGY) {
        if (int rc = ani_molecule_energy_f32(a->energy_sorted, a->gather_idxs, a->mol_offsets, a->mol_atom_counts,
                                             a->n_mols, a->n_atoms, a->labels, a->grad_scale, a->mol_energy,
                                             a->labels ? a->l2s : nullptr,
                                             a->labels ? a->grad_energy_sorted : nullptr, stream))
            return rc;
    }
    if (a->phases & ANI_PASS_BACKWARD) {
        ani_mlp_backward_args b;
        for (int t = 0; t < kTypes; t++) {
            b.grad_energy[t] = rows(a->grad_energy_sorted, t, 1);
            b.w1[t] = a->w1[t]; b.w2[t] = a->w2[t]; b.w3[t] = a->w3[t]; b.w4[t] = a->w4[t];
            b.dact1[t] = rows(a->dact1, t, kMlpH1); b.dact2[t] = rows(a->dact2, t, kMlpH2);
            b.dact3[t] = rows(a->dact3, t, kMlpH3);
            b.dz1[t] = rows(a->dz1, t, kMlpH1); b.dz2[t] = rows(a->dz2, t, kMlpH2); b.dz3[t] = rows(a->dz3, t, kMlpH3);
            b.grad_features[t] = rows(a->feature_grads, t, kTotal);
            b.packed[t] = a->packed[t];
        }
        if (int rc = ani_mlp_backward_f32(&b, acs, a->split_precision, stream)) return rc;
    }
    if (a->phases & ANI_PASS_WEIGHT_GRAD) {
        if (a->zero_ptr && a->zero_bytes)
            ANI_CUDA(cudaMemsetAsync(a->zero_ptr, 0, a->zero_bytes, (cudaStream_t)stream));
        ani_mlp_weight_grad_args w;
        for (int t = 0; t < kTypes; t++) {
            w.features[t] = rows(a->features, t, kTotal);
            w.act1[t] = rows(a->act1, t, kMlpH1); w.act2[t] = rows(a->act2, t, kMlpH2); w.act3[t] = rows(a->act3, t, kMlpH3);
            w.dz1[t] = rows(a->dz1, t, kMlpH1); w.dz2[t] = rows(a->dz2, t, kMlpH2); w.dz3[t] = rows(a->dz3, t, kMlpH3);
            w.dw1[t] = a->dw1[t]; w.dw2[t] = a->dw2[t]; w.dw3[t] = a->dw3[t]; w.dw4[t] = a->dw4[t];
            w.db1[t] = a->db1[t]; w.db2[t] = a->db2[t]; w.db3[t] = a->db3[t]; w.db4[t] = a->db4[t];
            w.grad_energy[t] = rows(a->grad_energy_sorted, t, 1);
        }
        if (int rc = ani_mlp_weight_grad_f32(&w, acs, a->split_precision, stream)) return rc;
    }
    if (a->phases & ANI_PASS_COORD_GRAD) {
        if (int rc = ani_featurize_grad_f32(a->xs, a->ys, a->zs, a->atomic_numbers, a->mol_offsets, a->mol_atom_counts,
                                            a->n_mols, a->scatter_idxs, rows(a->feature_grads, 0, kTotal),
                                            rows(a->feature_grads, 1, kTotal), rows(a->feature_grads, 2, kTotal),
                                            rows(a->feature_grads, 3, kTotal), a->x_grads, a->y_grads, a->z_grads,
                                            acs, stream))
            return rc;
    }
    return ANI_OK;
}

}  // extern "C"
