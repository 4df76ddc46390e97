// Arithmetic-peak probe of bench.py: one kernel that does nothing but independent fused
// multiply-adds on every SM.  Timed by the caller, it gives the FP32 / FP64 peak that the
// featurizer kernels are compared with.  Built into libbench_probe.so beside bench.py; it is a
// measurement aid and not part of the library's C ABI.
#include <cuda_runtime.h>

namespace {

template <typename T> __global__ void __launch_bounds__(256) fma_probe_kernel(int iterations, T seed, T* sink)
{
    T a[8];
#pragma unroll
    for (int k = 0; k < 8; k++) a[k] = seed + (T)(threadIdx.x + k);
    const T m = (T)0.999, c = (T)1e-3;
    for (int it = 0; it < iterations; it++) {
#pragma unroll
        for (int k = 0; k < 8; k++) a[k] = a[k] * m + c;
    }
    T sum = (T)0;
#pragma unroll
    for (int k = 0; k < 8; k++) sum += a[k];
    if (sum == (T)-1) sink[0] = sum;   // never true; keeps the chains alive
}

}  // namespace

// Enqueues the probe on `stream` (precision_bits 32 or 64); *flops_host receives the number of
// floating-point operations it executes.  `sink` is any 8 bytes of device memory.  Returns 0, or
// a cudaError_t value.
extern "C" int bench_fma_probe(int precision_bits, int iterations, void* sink, long long* flops_host, void* stream)
{
    if (!sink || !flops_host || iterations < 0 || (precision_bits != 32 && precision_bits != 64)) return -1;
    int dev = 0, sms = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return -2;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return -2;
    const int blocks = sms * 8, threads = 256;
    if (precision_bits == 32)
        fma_probe_kernel<float><<<blocks, threads, 0, (cudaStream_t)stream>>>(iterations, 1.0f, (float*)sink);
    else
        fma_probe_kernel<double><<<blocks, threads, 0, (cudaStream_t)stream>>>(iterations, 1.0, (double*)sink);
    *flops_host = 2LL * 8 * iterations * (long long)blocks * threads;
    return (int)cudaGetLastError();
}
