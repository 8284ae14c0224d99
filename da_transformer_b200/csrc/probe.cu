// Measurement helper: sustained MUFU ex2 throughput of the device, the denominator of the
// DAG kernels' roofline (one special-function result per (t, i->j) term of the log-domain
// recursion).  Not part of the operator path.
#include "dat_common.cuh"

namespace dat {

__global__ void __launch_bounds__(1024) mufu_probe_kernel(float *sink, int iters) {
    float x[8];
#pragma unroll
    for (int k = 0; k < 8; k++) x[k] = (threadIdx.x * 8 + k) * (1.0f / 8192.0f);
    for (int i = 0; i < iters; i++) {
#pragma unroll
        for (int k = 0; k < 8; k++) x[k] = ex2(x[k]) - 1.0f;  // stays in [0,1)
    }
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < 8; k++) s += x[k];
    if (s == -1.0f) sink[0] = s;  // never true; keeps the chain alive
}

}  // namespace dat

extern "C" int dat_probe_mufu(int iters, int blocks, float *sink, void *stream) {
    using namespace dat;
    DAT_REQUIRE(iters > 0 && blocks > 0 && sink, DAT_ERR_BAD_ARG, "dat_probe_mufu: bad argument");
    mufu_probe_kernel<<<blocks, 1024, 0, static_cast<cudaStream_t>(stream)>>>(sink, iters);
    return check_launch("dat_probe_mufu");
}
