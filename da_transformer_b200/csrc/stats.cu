// Per-shard statistics of the criterion in one launch: what the reference computes with a dozen
// elementwise and reduction launches after dag_loss (fs_plugins/criterions/nat_dag_loss.py:190-194:
// sentences whose log-likelihood is inf/nan are zeroed and counted as invalid, the rest contribute
// loss / target_length) and then sums across ranks through its logging buffer.
//   stats[0] = sum_b clean_b / tl_b      stats[1] = sum_b tl_b
//   stats[2] = number of sentences       stats[3] = number of invalid sentences
// All in fp64, like the reference's all-reduce buffer.
// dat_sentence_mean additionally returns the criterion's differentiable scalar of the shard,
// -(clean / tl).mean() (nat_dag_loss.py:194), and its gradient with respect to every sentence's
// log-likelihood (-1 / (tl_b * B), 0 for the zeroed sentences), so that the backward pass is one
// multiplication by the incoming scalar gradient.
#include "dat_common.cuh"

namespace dat {

__global__ void __launch_bounds__(1024)
sentence_stats_kernel(const float *__restrict__ loss, const int64_t *__restrict__ target_length,
                      double *__restrict__ stats, float *__restrict__ mean_out,
                      float *__restrict__ grad_scale, int B) {
    __shared__ double part[3][32];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    double s_loss = 0.0, s_tl = 0.0, s_bad = 0.0;
    for (int b = tid; b < B; b += blockDim.x) {
        const float l = loss[b];
        const double tl = (double)target_length[b];
        const bool bad = !(l > -INFINITY && l < INFINITY);   // inf or nan
        s_loss += bad ? 0.0 : (double)l / tl;
        s_tl += tl;
        s_bad += bad ? 1.0 : 0.0;
        if (grad_scale) grad_scale[b] = bad ? 0.f : (float)(-1.0 / (tl * (double)B));
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        s_loss += __shfl_xor_sync(0xffffffffu, s_loss, o);
        s_tl += __shfl_xor_sync(0xffffffffu, s_tl, o);
        s_bad += __shfl_xor_sync(0xffffffffu, s_bad, o);
    }
    if (lane == 0) { part[0][warp] = s_loss; part[1][warp] = s_tl; part[2][warp] = s_bad; }
    __syncthreads();
    if (warp == 0) {
        const int nw = blockDim.x >> 5;
        double a = lane < nw ? part[0][lane] : 0.0, c = lane < nw ? part[1][lane] : 0.0,
               d = lane < nw ? part[2][lane] : 0.0;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            a += __shfl_xor_sync(0xffffffffu, a, o);
            c += __shfl_xor_sync(0xffffffffu, c, o);
            d += __shfl_xor_sync(0xffffffffu, d, o);
        }
        if (lane == 0) {
            stats[0] = a; stats[1] = c; stats[2] = (double)B; stats[3] = d;
            if (mean_out) *mean_out = B > 0 ? (float)(-a / (double)B) : 0.f;
        }
    }
}

}  // namespace dat

extern "C" int dat_sentence_stats(const float *loss, const int64_t *target_length, double *stats, int bsz,
                                  void *stream) {
    using namespace dat;
    DAT_REQUIRE(bsz >= 0 && stats && (bsz == 0 || (loss && target_length)), DAT_ERR_BAD_ARG,
                "dat_sentence_stats: bad argument");
    sentence_stats_kernel<<<1, 1024, 0, static_cast<cudaStream_t>(stream)>>>(loss, target_length, stats,
                                                                              nullptr, nullptr, bsz);
    return check_launch("dat_sentence_stats");
}

extern "C" int dat_sentence_mean(const float *loss, const int64_t *target_length, double *stats,
                                 float *mean_out, float *grad_scale, int bsz, void *stream) {
    using namespace dat;
    DAT_REQUIRE(bsz >= 0 && stats && mean_out && (bsz == 0 || (loss && target_length && grad_scale)),
                DAT_ERR_BAD_ARG, "dat_sentence_mean: bad argument");
    sentence_stats_kernel<<<1, 1024, 0, static_cast<cudaStream_t>(stream)>>>(loss, target_length, stats,
                                                                              mean_out, grad_scale, bsz);
    return check_launch("dat_sentence_mean");
}
