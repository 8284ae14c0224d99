// Measurement helpers of the benchmark, built into their own small library
// (libdat_bench_probe.so); nothing here is part of the operator path or of its C ABI.
//
//   dat_probe_mufu: sustained MUFU ex2 throughput of the device, the denominator of the DAG
//     kernels' algorithmic roofline (one special-function result per (t, i->j) term of the
//     log-domain recursion).
//   dat_probe_ffma: sustained fp32 FMA throughput, the denominator for the work the shipped
//     probability-domain kernels actually execute.
#include <cuda_runtime.h>

namespace {

__global__ void __launch_bounds__(1024) mufu_probe_kernel(float *sink, int iters) {
    float x[8];
#pragma unroll
    for (int k = 0; k < 8; k++) x[k] = (threadIdx.x * 8 + k) * (1.0f / 8192.0f);
    for (int i = 0; i < iters; i++) {
#pragma unroll
        for (int k = 0; k < 8; k++) {
            float y;
            asm volatile("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x[k]));
            x[k] = y - 1.0f;  // stays in [0,1)
        }
    }
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < 8; k++) s += x[k];
    if (s == -1.0f) sink[0] = s;  // never true; keeps the chain alive
}

__global__ void __launch_bounds__(1024) ffma_probe_kernel(float *sink, int iters) {
    float x[16];
#pragma unroll
    for (int k = 0; k < 16; k++) x[k] = (threadIdx.x * 16 + k) * (1.0f / 16384.0f);
    const float a = 0.999f, c = 1.0e-4f;
    for (int i = 0; i < iters; i++) {
#pragma unroll
        for (int k = 0; k < 16; k++) x[k] = fmaf(x[k], a, c);
    }
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < 16; k++) s += x[k];
    if (s == -1.0f) sink[0] = s;
}

}  // namespace

// blocks CTAs of 1024 threads, 8 * iters dependent-chain ex2 per thread
extern "C" int dat_probe_mufu(int iters, int blocks, float *sink, void *stream) {
    if (iters <= 0 || blocks <= 0 || !sink) return 1;
    mufu_probe_kernel<<<blocks, 1024, 0, static_cast<cudaStream_t>(stream)>>>(sink, iters);
    return cudaGetLastError() == cudaSuccess ? 0 : 3;
}

// blocks CTAs of 1024 threads, 16 * iters fp32 FMAs per thread
extern "C" int dat_probe_ffma(int iters, int blocks, float *sink, void *stream) {
    if (iters <= 0 || blocks <= 0 || !sink) return 1;
    ffma_probe_kernel<<<blocks, 1024, 0, static_cast<cudaStream_t>(stream)>>>(sink, iters);
    return cudaGetLastError() == cudaSuccess ? 0 : 3;
}
