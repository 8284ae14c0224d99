// dag_loss backward for sm_100a: grad_match_all and grad_links from the alpha / beta rows
// left by dat_dag_loss.  Replaces calculate_grad_match_all_kernel,
// calculate_grad_links_kernel and their host wrapper
// (fs_plugins/custom_ops/dag_loss.cu:378-401, 432-485, 518-571).
//
// Rows are stored in the log2 domain with per-row fp64 offsets, so each exponent is
// assembled as  (row value) + (row value) + float(offset_a + offset_b - log2 Z): every
// term that reaches the MUFU is O(10) in magnitude however long the sentence is.
// Both outputs are written completely, zeros included, so the caller may pass
// uninitialised buffers.
#include "dag_tiles.cuh"

namespace dat {

__host__ __device__ inline bool lengths_valid_g(long long ol, long long tl, int T, int L) {
    return tl >= 2 && ol >= 2 && ol >= tl && ol <= L && tl <= T;
}

// grad_match_all[b,t,j] = g[b] * 2^(alpha2 + beta2 - match*log2e - Z2)
__global__ void __launch_bounds__(256)
dag_grad_match_kernel(const float *__restrict__ grad_out, const float *__restrict__ alpha,
                      const float *__restrict__ beta, const double *__restrict__ offsets,
                      const float *__restrict__ match, const int64_t *__restrict__ output_length,
                      const int64_t *__restrict__ target_length, float *__restrict__ gmatch, int T,
                      int L) {
    const int b = blockIdx.z, t = blockIdx.y;
    const int j = blockIdx.x * blockDim.x + threadIdx.x;
    if (j >= L) return;
    const long long ol = output_length[b], tl = target_length[b];
    const double *offs = offsets + (size_t)b * (2 * T + 2);
    const size_t x = ((size_t)b * T + t) * L + j;
    float out = 0.f;
    if (lengths_valid_g(ol, tl, T, L) && t < tl) {
        const int W = (int)(ol - tl) + 1;
        const double z2 = offs[2 * T + 1];
        if (j >= t && j < t + W && z2 > -INFINITY && z2 < INFINITY) {
            const float mv = match[x];
            if (mv > -INFINITY && mv < INFINITY) {
                const float k = (float)(offs[t] + offs[T + t] - z2);
                const float e = (alpha[x] + beta[x]) + fmaf(-mv, kLog2e, k);
                out = grad_out[b] * ex2(e);
                if (!(out == out)) out = 0.f;
            }
        }
    }
    gmatch[x] = out;
}

// The same, four vertices per thread and kGmSteps target steps per CTA (grad_match_steps_vec, dag_tiles.cuh),
// for rows that start on 16-byte boundaries (prelen a multiple of 4).
__global__ void __launch_bounds__(256)
dag_grad_match_vec_kernel(const float *__restrict__ grad_out, const float *__restrict__ alpha,
                          const float *__restrict__ beta, const double *__restrict__ offsets,
                          const float *__restrict__ match, const int64_t *__restrict__ output_length,
                          const int64_t *__restrict__ target_length, float *__restrict__ gmatch, int T, int L) {
    grad_match_steps_vec(grad_out, alpha, beta, offsets, match, output_length, target_length, gmatch, T, L,
                         blockIdx.y, blockIdx.x * kGmSteps);
}

constexpr int kGlRows = 8;
constexpr int kGlThreads = 256;

// grad_links[b,i,d] = g[b] * sum_t 2^(alpha2[t,i] + beta2[t+1,i+d+1] + links*log2e + k_t)
// One CTA owns kGlRows consecutive vertices i and sweeps all their successors.
__global__ void __launch_bounds__(kGlThreads)
dag_grad_links_kernel(const float *__restrict__ grad_out, const float *__restrict__ alpha,
                      const float *__restrict__ beta, const double *__restrict__ offsets,
                      const float *__restrict__ links, const int64_t *__restrict__ output_length,
                      const int64_t *__restrict__ target_length, float *__restrict__ glinks,
                      const int *__restrict__ select, int B, int T, int L, int K) {
    extern __shared__ __align__(16) float a_s[];  // [T][kGlRows]: alpha2[t,i] + k_t, -inf when dead
    const int i0 = blockIdx.x * kGlRows;
    const int tid = threadIdx.x;
    // a CTA takes every gridDim.y-th sentence: with a selection mask most of them are skipped, and a grid of
    // one CTA per (row block, sentence) would spend its time launching CTAs that return at once
    if (select != nullptr) {   // nothing selected among this CTA's sentences (the usual case): one look at all of them
        bool any = false;
        for (int b = blockIdx.y + (int)gridDim.y * tid; b < B; b += gridDim.y * kGlThreads) any |= select[b] != 0;
        if (!__syncthreads_or(any)) return;
    }
    for (int b = blockIdx.y; b < B; b += gridDim.y) {
    if (select != nullptr && select[b] == 0) continue;  // done by the product-form kernel
    __syncthreads();   // the previous sentence's readers of a_s
    const long long oll = output_length[b], tll = target_length[b];
    const double *offs = offsets + (size_t)b * (2 * T + 2);
    float *out = glinks + (size_t)b * L * K;
    const int ncol = kGlRows - 1 + K;

    bool live = lengths_valid_g(oll, tll, T, L) && i0 < oll - 1;
    double z2 = 0.0;
    if (live) {
        z2 = offs[2 * T + 1];
        live = z2 > -INFINITY && z2 < INFINITY;
    }
    if (!live) {
        for (int e = tid; e < ncol; e += kGlThreads)
#pragma unroll
            for (int u = 0; u < kGlRows; u++) {
                const int d = e - u, i = i0 + u;
                if (d >= 0 && d < K && i < L) out[(size_t)i * K + d] = 0.f;
            }
        continue;
    }
    const int ol = (int)oll, tl = (int)tll;
    const int W = ol - tl + 1;
    const float g = grad_out[b];
    const float *al = alpha + (size_t)b * T * L;
    const float *be = beta + (size_t)b * T * L;
    const float *lk = links + (size_t)b * L * K;
    int thi = i0 + kGlRows - 1;  // alpha[t,i] is dead for t > i
    if (thi > tl - 2) thi = tl - 2;
    for (int x = tid; x < (thi + 1) * kGlRows; x += kGlThreads) {
        const int t = x / kGlRows, u = x - t * kGlRows;
        const int i = i0 + u;
        float v = -INFINITY;
        if (i < ol && i >= t && i < t + W)
            v = al[(size_t)t * L + i] + (float)(offs[t] + offs[T + t + 1] - z2);
        a_s[x] = v;
    }
    __syncthreads();

    for (int e = tid; e < ncol; e += kGlThreads) {
        const int j = i0 + 1 + e;
        float l2[kGlRows], acc[kGlRows];
#pragma unroll
        for (int u = 0; u < kGlRows; u++) {
            const int d = e - u, i = i0 + u;
            const bool ok = d >= 0 && d < K && i < ol && j < ol;
            l2[u] = ok ? __ldg(lk + (size_t)i * K + d) * kLog2e : -INFINITY;
            acc[u] = 0.f;
        }
        if (j < ol) {
            int tlo = j - W;
            if (tlo < 0) tlo = 0;
            int th = thi < j - 1 ? thi : j - 1;
            for (int t = tlo; t <= th; t++) {
                const float bj = __ldg(be + (size_t)(t + 1) * L + j);
                const float4 a0 = *reinterpret_cast<const float4 *>(a_s + t * kGlRows);
                const float4 a1 = *reinterpret_cast<const float4 *>(a_s + t * kGlRows + 4);
                const float av[kGlRows] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
#pragma unroll
                for (int u = 0; u < kGlRows; u++) acc[u] += ex2((av[u] + l2[u]) + bj);
            }
        }
#pragma unroll
        for (int u = 0; u < kGlRows; u++) {
            const int d = e - u, i = i0 + u;
            if (d >= 0 && d < K && i < L) {
                float v = g * acc[u];
                if (!(v == v)) v = 0.f;
                out[(size_t)i * K + d] = v;
            }
        }
    }
    }   // sentences
}

}  // namespace dat

namespace dat {

int launch_grad_match(const float *grad_output, const float *alpha, const float *beta,
                      const double *offsets, const float *match_all, const int64_t *output_length,
                      const int64_t *target_length, float *grad_match_all, int bsz, int tarlen,
                      int prelen, cudaStream_t st, const char *who) {
    const bool aligned = (prelen & 3) == 0 && ((reinterpret_cast<uintptr_t>(alpha) | reinterpret_cast<uintptr_t>(beta) |
                                                reinterpret_cast<uintptr_t>(match_all) |
                                                reinterpret_cast<uintptr_t>(grad_match_all)) & 15) == 0;
    if (aligned) {
        dim3 grid((tarlen + kGmSteps - 1) / kGmSteps, bsz);
        dag_grad_match_vec_kernel<<<grid, 256, 0, st>>>(grad_output, alpha, beta, offsets, match_all, output_length,
                                                        target_length, grad_match_all, tarlen, prelen);
    } else {
        dim3 grid((prelen + 255) / 256, tarlen, bsz);
        dag_grad_match_kernel<<<grid, 256, 0, st>>>(grad_output, alpha, beta, offsets, match_all,
                                                    output_length, target_length, grad_match_all, tarlen,
                                                    prelen);
    }
    return check_launch(who);
}

// exact grad_links; with a selection mask only the sentences whose entry is non-zero
int launch_exact_grad_links(const float *grad_output, const float *alpha, const float *beta,
                            const double *offsets, const float *links, const int64_t *output_length,
                            const int64_t *target_length, float *grad_links, const int *select, int bsz,
                            int tarlen, int prelen, int translen, cudaStream_t st, const char *who) {
    const size_t smem = (size_t)tarlen * kGlRows * sizeof(float);
    DAT_REQUIRE(tarlen <= kMaxTarlenGrad, DAT_ERR_UNSUPPORTED, "%s: tarlen=%d exceeds %d", who, tarlen,
                kMaxTarlenGrad);
    if (smem > 48 * 1024 &&
        cudaFuncSetAttribute(dag_grad_links_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                             (int)smem) != cudaSuccess)
        return check_launch(who);
    // with a selection mask few sentences are expected: 64 CTAs per row block share them out
    dim3 grid((prelen + kGlRows - 1) / kGlRows, select != nullptr && bsz > 64 ? 64 : bsz);
    dag_grad_links_kernel<<<grid, kGlThreads, smem, st>>>(grad_output, alpha, beta, offsets, links,
                                                         output_length, target_length, grad_links, select, bsz,
                                                         tarlen, prelen, translen);
    return check_launch(who);
}

}  // namespace dat

extern "C" {

int dat_dag_loss_backward(const float *grad_output, const float *alpha, const float *beta,
                          const double *offsets, const float *match_all, const float *links,
                          const int64_t *output_length, const int64_t *target_length,
                          float *grad_match_all, float *grad_links, int bsz, int tarlen,
                          int prelen, int translen, int config1, int config2, void *stream) {
    using namespace dat;
    (void)config1;
    (void)config2;
    DAT_REQUIRE(bsz >= 0 && tarlen >= 1 && prelen >= 1 && translen >= 1, DAT_ERR_BAD_ARG,
                "dat_dag_loss_backward: bad sizes bsz=%d tarlen=%d prelen=%d translen=%d", bsz,
                tarlen, prelen, translen);
    if (bsz == 0) return DAT_OK;
    DAT_REQUIRE(grad_output && alpha && beta && offsets && match_all && links && output_length &&
                    target_length && grad_match_all && grad_links,
                DAT_ERR_BAD_ARG, "dat_dag_loss_backward: null pointer");
    DAT_REQUIRE(bsz <= 65535 && tarlen <= 65535, DAT_ERR_UNSUPPORTED,
                "dat_dag_loss_backward: bsz and tarlen are limited to 65535");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (int rc = launch_grad_match(grad_output, alpha, beta, offsets, match_all, output_length,
                                   target_length, grad_match_all, bsz, tarlen, prelen, st,
                                   "dat_dag_loss_backward(grad_match)"))
        return rc;
    return launch_exact_grad_links(grad_output, alpha, beta, offsets, links, output_length,
                                   target_length, grad_links, nullptr, bsz, tarlen, prelen, translen, st,
                                   "dat_dag_loss_backward(grad_links)");
}

}  // extern "C"
