// dag_loss forward: alpha and beta recursions of the DAG log-likelihood for sm_100a.
//
// Replaces calculate_alpha_kernel / calculate_beta_kernel and their host wrapper
// (fs_plugins/custom_ops/dag_loss.cu:40-140, 178-274, 313-375).
//
// One CTA owns one (sentence, sweep) pair; no CTA ever waits for another one.  All
// arithmetic is fp32 in the log2 domain.  Only the reachable window is computed: at
// target step t the live vertices are j in [t, t+W), W = output_length - target_length
// + 1 (a vertex left of the window cannot have emitted t tokens yet, a vertex right of
// it cannot reach the last vertex in time).  In window coordinates the work of every
// step is the same triangle  { (r, c) : 0 <= r <= c < W, c - r < K },
//   alpha:  i = t-1+r  ->  j = t+c     link = band[i][c-r]
//   beta :  i = t+r    ->  j = t+1+c   link = band[i][c-r]
// Rows are stored shifted by a per-row offset (fp64, `offsets`) so that the stored fp32
// values stay O(10) whatever the length of the sentence.
//
// Layout of `offsets` per sentence (2*T+2 doubles): [0,T) alpha row offsets, [T,2T) beta
// row offsets, [2T] log2-likelihood from the alpha sweep, [2T+1] from the beta sweep.
#include "dag_tiles.cuh"

namespace dat {

// ---------------------------------------------------------------------------------
// alpha sweep
// ---------------------------------------------------------------------------------
__device__ void alpha_sweep(const float *__restrict__ match, const float *__restrict__ band,
                            float *__restrict__ alpha, double *__restrict__ offs, float *loss_out,
                            int ol, int tl, int T, int L, int K, unsigned char *raw) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int W = ol - tl + 1;
    const int ncb = (W + 31) >> 5;
    SweepSmem sm = carve(raw, L);
    __shared__ double off_s;
    __shared__ float delta_s;

    for (int x = tid; x < L + 32; x += kSweepThreads) sm.row[0][x] = -INFINITY;
    int my_lo, my_hi, cb_first;
    build_tile_plan(sm, W, K, my_lo, my_hi, cb_first);
    // warps without tiles sit between the first and last warp of a shared column block:
    // their merge slots must read as empty
#pragma unroll
    for (int which = 0; which < 2; which++) {
        float *p = sm.part + ((which * kSweepWarps + warp) * 2) * 32;
        p[lane] = kNegBig;
        p[32 + lane] = 0.f;
    }
    const float m00 = match[0] * kLog2e;
    if (tid == 0) {
        sm.row[0][0] = m00;
        alpha[0] = m00;
        offs[0] = 0.0;
        off_s = 0.0;
        for (int w = 0; w < kSweepWarps; w++) sm.wmax[w] = m00;  // row 0 has the single entry
    }
    // the rest of row 0 inside the window is unreachable
    for (int c = 1 + tid; c < W; c += kSweepThreads) alpha[c] = -INFINITY;
    __syncthreads();

    for (int t = 1; t < tl; t++) {
        const float *prev = sm.row[(t - 1) & 1];
        float *cur = sm.row[t & 1];
        // match of this thread's merge columns, requested early
        float mt[2];
#pragma unroll
        for (int q = 0; q < 2; q++) {
            int c = tid + q * kSweepThreads;
            mt[q] = (c < W) ? match[(size_t)t * L + t + c] : 0.f;
        }
        if (tid == 0) {
            float d = sm.wmax[((t - 1) & 1) * kSweepWarps];
            for (int w = 1; w < kSweepWarps; w++) d = fmaxf(d, sm.wmax[((t - 1) & 1) * kSweepWarps + w]);
            if (!(d > 0.5f * kNegBig)) d = 0.f;  // dead row
            delta_s = d;
            off_s += (double)d;
            offs[t] = off_s;
        }

        // ---- tile phase
        if (my_lo < my_hi) {
            int cb = cb_first;
            int rb = sm.rb_lo[cb] + (my_lo - sm.tile_start[cb]);
            bool owns_start = (my_lo == sm.tile_start[cb]);
            float m = kNegBig, s = 0.f;
            for (int tile = my_lo; tile < my_hi;) {
                const int c = 32 * cb + lane;
                int rmax = (c < W) ? c : -1;               // valid rows of this lane: [rmin, rmax]
                int rmin = c + 1 - K; rmin = rmin > 0 ? rmin : 0;
                const int r0 = 32 * rb;
                int r1 = r0 + 32;
                { int cap = 32 * cb + 32; cap = cap < W ? cap : W; if (r1 > cap) r1 = cap; }
                const float *bp = band + (size_t)(t - 1) * K + c;
                const int i0 = t - 1;
                for (int r = r0; r < r1; r += kChunk) {
                    float x[kChunk];
#pragma unroll
                    for (int u = 0; u < kChunk; u++) {
                        const int rr = r + u;
                        const bool ok = (rr >= rmin) && (rr <= rmax) && (rr < r1);
                        float lk = ok ? __ldg(bp + (size_t)rr * (K - 1)) : -INFINITY;
                        float pa = prev[i0 + (rr < r1 ? rr : r1 - 1)];
                        x[u] = fmaf(lk, kLog2e, pa);
                    }
                    float cm = x[0];
#pragma unroll
                    for (int u = 1; u < kChunk; u++) cm = fmaxf(cm, x[u]);
                    if (cm > m) {
                        s *= ex2(m - cm);
                        m = cm;
                    }
                    float acc = 0.f;
#pragma unroll
                    for (int u = 0; u < kChunk; u++) acc += ex2(x[u] - m);
                    s += acc;
                }
                tile++;
                rb++;
                if (rb > cb || tile == my_hi) {
                    const bool complete = owns_start && (rb > cb);
                    if (complete) {
                        if (c < W) { sm.fin_m[c] = m; sm.fin_s[c] = s; }
                    } else {
                        const int which = (cb == cb_first) ? 0 : 1;
                        float *p = sm.part + ((which * kSweepWarps + warp) * 2) * 32;
                        p[lane] = m;
                        p[32 + lane] = s;
                    }
                    cb++;
                    rb = sm.rb_lo[cb];
                    owns_start = true;
                    m = kNegBig;
                    s = 0.f;
                }
            }
        }
        __syncthreads();

        // ---- merge phase: one thread per window column
        const float delta = delta_s;
        float vmax = kNegBig;
#pragma unroll
        for (int q = 0; q < 2; q++) {
            const int c = tid + q * kSweepThreads;
            if (c < W) {
                const int cb = c >> 5, ln = c & 31;
                const int wa = sm.first_warp[cb], wb = sm.last_warp[cb];
                float m, s;
                if (wa == wb) {
                    m = sm.fin_m[c];
                    s = sm.fin_s[c];
                } else {
                    m = kNegBig;
                    s = 0.f;
                    for (int w = wa; w <= wb; w++) {
                        const int which = (sm.cb_first_of[w] == cb) ? 0 : 1;
                        const float *p = sm.part + ((which * kSweepWarps + w) * 2) * 32;
                        lse_merge(m, s, p[ln], p[32 + ln]);
                    }
                }
                float u = -INFINITY;
                if (s > 0.f) u = (m + lg2(s) - delta) + mt[q] * kLog2e;
                if (!(u > -INFINITY)) u = -INFINITY;  // also catches a NaN from +inf match
                const int j = t + c;
                cur[j] = u;
                alpha[(size_t)t * L + j] = u;
                vmax = fmaxf(vmax, u);
            }
        }
        vmax = warp_max(vmax);
        if (lane == 0) sm.wmax[(t & 1) * kSweepWarps + warp] = vmax;
        __syncthreads();
    }
    if (tid == 0) {
        float u = sm.row[(tl - 1) & 1][ol - 1];
        double z2 = (u > -INFINITY) ? (double)u + off_s : -INFINITY;
        offs[2 * T] = z2;
        if (loss_out) *loss_out = (float)(z2 * kLn2d);
    }
}

// ---------------------------------------------------------------------------------
// beta sweep: one warp per pair of window rows (r, W-1-r), lanes along the band row
// ---------------------------------------------------------------------------------
__device__ __forceinline__ void beta_row(const float *__restrict__ brow, const float *next_j,
                                         int len, int lane, float &m, float &s) {
    // log-sum-exp over e in [0,len) of next_j[e] + brow[e] * log2(e)
    m = kNegBig;
    s = 0.f;
    for (int e0 = 0; e0 < len; e0 += 32 * kChunk) {
        float x[kChunk];
#pragma unroll
        for (int u = 0; u < kChunk; u++) {
            const int e = e0 + u * 32 + lane;
            const bool ok = e < len;
            float lk = ok ? __ldg(brow + e) : -INFINITY;
            float nb = next_j[ok ? e : 0];
            x[u] = fmaf(lk, kLog2e, nb);
        }
        float cm = x[0];
#pragma unroll
        for (int u = 1; u < kChunk; u++) cm = fmaxf(cm, x[u]);
        if (cm > m) {
            s *= ex2(m - cm);
            m = cm;
        }
        float acc = 0.f;
#pragma unroll
        for (int u = 0; u < kChunk; u++) acc += ex2(x[u] - m);
        s += acc;
    }
    warp_lse(m, s);
}

__device__ void beta_sweep(const float *__restrict__ match, const float *__restrict__ band,
                           float *__restrict__ beta, double *__restrict__ offs, float *loss_out,
                           int ol, int tl, int T, int L, int K, unsigned char *raw) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int W = ol - tl + 1;
    SweepSmem sm = carve(raw, L);
    double *offb = offs + T;

    for (int x = tid; x < L + 32; x += kSweepThreads) {
        sm.row[0][x] = -INFINITY;
        sm.row[1][x] = -INFINITY;
    }
    __syncthreads();
    float mll = match[(size_t)(tl - 1) * L + (ol - 1)] * kLog2e;
    if (!(mll > -INFINITY)) mll = -INFINITY;
    if (tid == 0) {
        sm.row[(tl - 1) & 1][ol - 1] = mll;
        beta[(size_t)(tl - 1) * L + (ol - 1)] = mll;
        offb[tl - 1] = 0.0;
        for (int w = 0; w < kSweepWarps; w++) sm.wmax[((tl - 1) & 1) * kSweepWarps + w] = mll;
    }
    // the rest of row tl-1 inside the window is unreachable
    for (int c = tid; c < W - 1; c += kSweepThreads) beta[(size_t)(tl - 1) * L + (tl - 1) + c] = -INFINITY;
    double off = 0.0;  // thread 0 only
    __syncthreads();

    const int npairs = (W + 1) >> 1;
    for (int t = tl - 2; t >= 0; t--) {
        const float *next = sm.row[(t + 1) & 1];
        float *cur = sm.row[t & 1];
        float delta;
        {
            float d = (lane < kSweepWarps) ? sm.wmax[((t + 1) & 1) * kSweepWarps + lane] : kNegBig;
            d = warp_max(d);
            if (!(d > 0.5f * kNegBig)) d = 0.f;
            delta = d;
        }
        if (tid == 0) {
            off += (double)delta;
            offb[t] = off;
        }
        float vmax = kNegBig;
        for (int p = warp; p < npairs; p += kSweepWarps) {
#pragma unroll
            for (int h = 0; h < 2; h++) {
                const int r = h == 0 ? p : (W - 1 - p);
                if (h == 1 && r == p) break;
                const int i = t + r;
                int len = W - r;
                len = len < K ? len : K;
                const float mt = (lane == 0) ? match[(size_t)t * L + i] : 0.f;
                float m, s;
                beta_row(band + (size_t)i * K, next + t + 1 + r, len, lane, m, s);
                if (lane == 0) {
                    float u = -INFINITY;
                    if (s > 0.f) u = (m + lg2(s) - delta) + mt * kLog2e;
                    if (!(u > -INFINITY)) u = -INFINITY;
                    cur[i] = u;
                    beta[(size_t)t * L + i] = u;
                    vmax = fmaxf(vmax, u);
                }
            }
        }
        if (lane == 0) sm.wmax[(t & 1) * kSweepWarps + warp] = vmax;
        __syncthreads();
    }
    if (tid == 0) {
        float u = sm.row[0][0];
        double z2 = (u > -INFINITY) ? (double)u + off : -INFINITY;
        offs[2 * T + 1] = z2;
        if (loss_out) *loss_out = (float)(z2 * kLn2d);
    }
}

__global__ void __launch_bounds__(kSweepThreads)
dag_sweep_kernel(const float *__restrict__ match, const float *__restrict__ links,
                 const int64_t *__restrict__ output_length, const int64_t *__restrict__ target_length,
                 float *__restrict__ alpha, float *__restrict__ beta, double *__restrict__ offsets,
                 float *__restrict__ loss, int32_t *__restrict__ status, int nsweep, int T, int L,
                 int K) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int b = blockIdx.x / nsweep;
    const int sweep = blockIdx.x - b * nsweep;
    const long long ol = output_length[b], tl = target_length[b];
    double *offs = offsets + (size_t)b * (2 * T + 2);
    if (!lengths_valid(ol, tl, T, L)) {
        if (threadIdx.x == 0) {
            offs[2 * T + sweep] = -INFINITY;
            if (sweep == nsweep - 1) loss[b] = -INFINITY;
            if (status) atomicOr(status, DAT_STATUS_BAD_LENGTH);
        }
        return;
    }
    const float *mb = match + (size_t)b * T * L;
    const float *lb = links + (size_t)b * L * K;
    if (sweep == 0) {
        alpha_sweep(mb, lb, alpha + (size_t)b * T * L, offs, nsweep == 1 ? loss + b : nullptr,
                    (int)ol, (int)tl, T, L, K, smem_raw);
    } else {
        beta_sweep(mb, lb, beta + (size_t)b * T * L, offs, loss + b, (int)ol, (int)tl, T, L, K,
                   smem_raw);
    }
}

}  // namespace dat

extern "C" {

size_t dat_dag_loss_offsets_bytes(int bsz, int tarlen) {
    if (bsz < 0 || tarlen < 0) return 0;
    return (size_t)bsz * (2 * (size_t)tarlen + 2) * sizeof(double);
}

int dat_dag_loss(const float *match_all, const float *links, const int64_t *output_length,
                 const int64_t *target_length, int require_gradient, float *alpha, float *beta,
                 double *offsets, float *loss, int32_t *status, int bsz, int tarlen, int prelen,
                 int translen, int config, void *stream) {
    using namespace dat;
    (void)config;
    DAT_REQUIRE(bsz >= 0 && tarlen >= 1 && prelen >= 1 && translen >= 1, DAT_ERR_BAD_ARG,
                "dat_dag_loss: bad sizes bsz=%d tarlen=%d prelen=%d translen=%d", bsz, tarlen,
                prelen, translen);
    if (bsz == 0) return DAT_OK;
    DAT_REQUIRE(match_all && links && output_length && target_length && alpha && offsets && loss,
                DAT_ERR_BAD_ARG, "dat_dag_loss: null pointer");
    DAT_REQUIRE(!require_gradient || beta, DAT_ERR_BAD_ARG,
                "dat_dag_loss: beta workspace required when require_gradient");
    DAT_REQUIRE(prelen <= 2 * kSweepThreads, DAT_ERR_UNSUPPORTED,
                "dat_dag_loss: prelen=%d exceeds %d", prelen, 2 * kSweepThreads);
    DeviceInfo di;
    if (!device_info(&di)) return DAT_ERR_NO_DEVICE;
    const size_t smem = sweep_smem_bytes(prelen);
    DAT_REQUIRE(smem <= (size_t)di.max_smem_optin, DAT_ERR_UNSUPPORTED,
                "dat_dag_loss: prelen=%d needs %zu bytes of shared memory", prelen, smem);
    if (smem > 48 * 1024) {
        if (cudaFuncSetAttribute(dag_sweep_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)smem) != cudaSuccess)
            return check_launch("dat_dag_loss(attr)");
    }
    const int nsweep = require_gradient ? 2 : 1;
    dag_sweep_kernel<<<(unsigned)(bsz * nsweep), kSweepThreads, smem,
                       static_cast<cudaStream_t>(stream)>>>(
        match_all, links, output_length, target_length, alpha, beta, offsets, loss, status, nsweep,
        tarlen, prelen, translen);
    return check_launch("dat_dag_loss");
}

}  // extern "C"
