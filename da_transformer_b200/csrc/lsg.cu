// logsoftmax_gather forward / backward for sm_100a.
//
// Forward: one pass over each vocabulary row with an online (max, sum-exp) pair per
// thread, 128-bit streaming loads, fp32 math; only the gathered values and two row
// statistics are written.  Replaces the three-pass, scalar-load kernel of
// fs_plugins/custom_ops/logsoftmax_gather.cu:256-310.
// Backward: reads the logits and the row statistics and writes the dense gradient in
// place, once, rounded once from fp32 (the reference does mul_ + scatter_add_ in the
// logits dtype, fs_plugins/custom_ops/dag_loss.py:227-229).
//
// HBM-bound: algorithmic bytes are V*e per row forward and 2*V*e per row backward
// (e = element size), plus the small index / gathered-value traffic.
//
// Two things the criterion does around the gather ride on the same pass when asked for
// (dat_logsoftmax_gather_fused):
//   * the arg-max token of every row, which the glancing sampler takes with a separate full read of
//     the logits right before its gather (fs_plugins/criterions/nat_dag_loss.py:246), with
//     torch.argmax's result for ties (first index) and NaN (counts as the maximum);
//   * the forced alignment (nat_dag_loss.py:111-120): a target step that some vertex is forced to
//     emit keeps only that vertex (0 there, -inf at every other vertex), and no gradient flows
//     into the forced steps.  The reference builds three [B,T,L] temporaries for it.
#include <climits>

#include "dat_common.cuh"

namespace dat {

constexpr int kLsgThreads = 256;
constexpr int kLsgWarps = kLsgThreads / 32;
constexpr int kBwdUnroll = 4;   // 16-byte vectors in flight per thread in the backward
constexpr int kFwdStage = 512;  // selected logits staged per row in the forward
// six forward CTAs per SM (40 registers; five at the compiler's own choice of 44): more rows in flight cover the
// reductions at the end of a row.  The backward is left at its 64 registers (four CTAs): five or six were slower.
constexpr int kFwdMinCtas = 6;

struct Strides3 {
    int64_t b, l, s;
};

// Online update of (m, s) with `n` new values; m is the running maximum in the
// natural domain (exact), s = sum exp(x - m).
template <int N>
__device__ __forceinline__ void online_update(float &m, float &s, const float (&f)[N]) {
    float vmax = f[0];
#pragma unroll
    for (int i = 1; i < N; i++) vmax = fmaxf(vmax, f[i]);
    if (vmax > m) {
        s *= ex2((m - vmax) * kLog2e);
        m = vmax;
    }
    const float mneg = -m * kLog2e;
    float acc = 0.f;
#pragma unroll
    for (int i = 0; i < N; i++) acc += ex2(fmaf(f[i], kLog2e, mneg));
    s += acc;
}

__device__ __forceinline__ void online_update1(float &m, float &s, float v) {
    if (v > m) {
        s *= ex2((m - v) * kLog2e);
        m = v;
    }
    s += ex2((v - m) * kLog2e);
}

// Splits a row of V elements starting at `p` into a scalar head (up to the first
// 16-byte boundary), `nvec` aligned 16-byte vectors and a scalar tail.
template <typename T>
__device__ __forceinline__ void row_split(const T *p, int V, int &head, int &nvec) {
    constexpr int kVec = Elem<T>::kVec;
    int mis = (int)((reinterpret_cast<uintptr_t>(p) & 15u) / sizeof(T));
    head = mis ? (kVec - mis) : 0;
    if (head > V) head = V;
    nvec = (V - head) / kVec;
}

// Optional extras of the forward pass (all null for the plain gather).
struct LsgExtras {
    int64_t *argmax;             // [rows]: arg-max token of each row
    const int64_t *force_emit;   // [B, L] contiguous: target step vertex l is forced to emit, or -1
    const int32_t *forced_step;  // [B, S]: 1 where some vertex of the sentence is forced to emit step s
};

// (value, index) pair ordered like torch.argmax orders candidates: larger value first, then smaller index
__device__ __forceinline__ void arg_better(float &bm, int &bi, float v, int i) {
    if (v > bm || (v == bm && i < bi)) {
        bm = v;
        bi = i;
    }
}

template <typename T, bool kArgmax>
__global__ void __launch_bounds__(kLsgThreads, kFwdMinCtas)
lsg_fwd_kernel(const T *__restrict__ x, const int64_t *__restrict__ idx, Strides3 is,
               float *__restrict__ sel, Strides3 ss, float *__restrict__ stats,
               int32_t *__restrict__ status, LsgExtras ex, int64_t rows, int L, int S, int V) {
    constexpr int kVec = Elem<T>::kVec;
    __shared__ float red_m[2][kLsgWarps];
    __shared__ float red_s[2][kLsgWarps];
    __shared__ float arg_m[2][kLsgWarps];
    __shared__ int arg_i[2][kLsgWarps];
    __shared__ int arg_nan[2][kLsgWarps];
    __shared__ float xsel[2][kFwdStage];   // logits at the first kFwdStage selected positions
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    int par = 0;
    bool bad_index = false;
    for (int64_t row = blockIdx.x; row < rows; row += gridDim.x, par ^= 1) {
        const T *xr = x + row * (int64_t)V;
        const int64_t b = row / L, l = row - b * L;
        const int64_t *ir = idx + b * is.b + l * is.l;
        // The selected logits are fetched BEFORE the row is streamed: the sectors they pull in
        // from HBM are then hits for the streaming pass.  Fetched afterwards they miss (the
        // streaming loads do not keep the row in cache) and cost an extra ~12 % of traffic.
        for (int k = tid; k < S && k < kFwdStage; k += kLsgThreads) {
            const int64_t id = ir[(int64_t)k * is.s];
            const bool ok = id >= 0 && id < V;
            bad_index |= !ok;
            xsel[par][k] = ok ? Elem<T>::to_float(xr[id]) : __int_as_float(0x7fc00000);
        }
        int head, nvec;
        row_split(xr, V, head, nvec);
        const uint4 *xv = reinterpret_cast<const uint4 *>(xr + head);
        float m = kNegBig, s = 0.f;
        float bm = -INFINITY;   // arg-max candidate of this thread (kArgmax only)
        int bi = INT_MAX;
        int v = tid;
        for (; v + 3 * kLsgThreads < nvec; v += 4 * kLsgThreads) {
            uint4 u0 = ld_stream16(xv + v);
            uint4 u1 = ld_stream16(xv + v + kLsgThreads);
            uint4 u2 = ld_stream16(xv + v + 2 * kLsgThreads);
            uint4 u3 = ld_stream16(xv + v + 3 * kLsgThreads);
            float f[4 * kVec];
            Elem<T>::unpack(u0, f);
            Elem<T>::unpack(u1, f + kVec);
            Elem<T>::unpack(u2, f + 2 * kVec);
            Elem<T>::unpack(u3, f + 3 * kVec);
            if (kArgmax) {
                // a thread meets its elements in increasing index order, so a strictly larger
                // group maximum is the only way its candidate changes (rare after the first groups)
                float gm = f[0];
#pragma unroll
                for (int i = 1; i < 4 * kVec; i++) gm = fmaxf(gm, f[i]);
                if (gm > bm) {
                    bm = gm;
#pragma unroll
                    for (int i = 4 * kVec - 1; i >= 0; i--)
                        if (f[i] == gm) bi = head + (v + (i / kVec) * kLsgThreads) * kVec + (i % kVec);
                }
            }
            online_update<4 * kVec>(m, s, f);
        }
        if (v < nvec) {
            // the last one to three vectors of this thread, requested together; a vector that does not exist
            // is one of -inf elements (no contribution to the sum, never an arg-max candidate)
            const uint4 none = make_uint4(Elem<T>::kNegInfWord, Elem<T>::kNegInfWord, Elem<T>::kNegInfWord,
                                          Elem<T>::kNegInfWord);
            const bool p1 = v + kLsgThreads < nvec, p2 = v + 2 * kLsgThreads < nvec;
            uint4 u0 = ld_stream16(xv + v);
            uint4 u1 = p1 ? ld_stream16(xv + v + kLsgThreads) : none;
            uint4 u2 = p2 ? ld_stream16(xv + v + 2 * kLsgThreads) : none;
            float f[3 * kVec];
            Elem<T>::unpack(u0, f);
            Elem<T>::unpack(u1, f + kVec);
            Elem<T>::unpack(u2, f + 2 * kVec);
            if (kArgmax) {
#pragma unroll
                for (int i = 0; i < 3 * kVec; i++)
                    arg_better(bm, bi, f[i], head + (v + (i / kVec) * kLsgThreads) * kVec + (i % kVec));
            }
            online_update<3 * kVec>(m, s, f);
        }
        // scalar head and tail
        const int tail0 = head + nvec * kVec;
        if (tid < head) {
            const float xv0 = Elem<T>::to_float(xr[tid]);
            if (kArgmax) arg_better(bm, bi, xv0, tid);
            online_update1(m, s, xv0);
        }
        if (tail0 + tid < V) {
            const float xv0 = Elem<T>::to_float(xr[tail0 + tid]);
            if (kArgmax) arg_better(bm, bi, xv0, tail0 + tid);
            online_update1(m, s, xv0);
        }

        // block max (exact), then block sum of the rescaled partial sums
        float wm = warp_max(m);
        if (kArgmax) {
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, bm, o);
                const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
                arg_better(bm, bi, ov, oi);
            }
        }
        if (lane == 0) {
            red_m[par][warp] = wm;
            if (kArgmax) { arg_m[par][warp] = bm; arg_i[par][warp] = bi; }
        }
        __syncthreads();
        float M = red_m[par][0];
#pragma unroll
        for (int w = 1; w < kLsgWarps; w++) M = fmaxf(M, red_m[par][w]);
        float sc = s * ex2((m - M) * kLog2e);
        float ws = warp_sum(sc);
        if (lane == 0) red_s[par][warp] = ws;
        __syncthreads();
        float Ssum = 0.f;
#pragma unroll
        for (int w = 0; w < kLsgWarps; w++) Ssum += red_s[par][w];
        const float logS = lg2(Ssum) * kLn2;

        if (kArgmax) {
            float am = arg_m[par][0];
            int ai = arg_i[par][0];
#pragma unroll
            for (int w = 1; w < kLsgWarps; w++) arg_better(am, ai, arg_m[par][w], arg_i[par][w]);
            // A NaN or +inf logit, or a row of -inf, shows as a sum that is not a positive finite
            // number (fmaxf skips NaN, so the candidates above never saw it).  Such rows are scanned
            // again with torch.argmax's rules: the first NaN if there is one, else the first maximum.
            if (!(Ssum > 0.f && Ssum < INFINITY) || ai == INT_MAX) {   // block-uniform
                float sm2 = -INFINITY;
                int si = INT_MAX, sn = INT_MAX;
                for (int e = tid; e < V; e += kLsgThreads) {
                    const float xe = Elem<T>::to_float(xr[e]);
                    if (xe != xe) sn = e < sn ? e : sn;
                    else arg_better(sm2, si, xe, e);
                }
#pragma unroll
                for (int o = 16; o > 0; o >>= 1) {
                    const float ov = __shfl_xor_sync(0xffffffffu, sm2, o);
                    const int oi = __shfl_xor_sync(0xffffffffu, si, o);
                    const int on = __shfl_xor_sync(0xffffffffu, sn, o);
                    arg_better(sm2, si, ov, oi);
                    sn = on < sn ? on : sn;
                }
                __syncthreads();   // everybody has read the first reduction's slots
                if (lane == 0) { arg_m[par][warp] = sm2; arg_i[par][warp] = si; arg_nan[par][warp] = sn; }
                __syncthreads();
                am = arg_m[par][0];
                ai = arg_i[par][0];
                int an = arg_nan[par][0];
#pragma unroll
                for (int w = 1; w < kLsgWarps; w++) {
                    arg_better(am, ai, arg_m[par][w], arg_i[par][w]);
                    an = arg_nan[par][w] < an ? arg_nan[par][w] : an;
                }
                if (an != INT_MAX) ai = an;
                else if (ai == INT_MAX) ai = 0;
            }
            if (tid == 0) ex.argmax[row] = ai;
        }

        float *sr = sel + b * ss.b + l * ss.l;
        const int64_t fe = ex.force_emit ? ex.force_emit[row] : -1;
        const int32_t *forced = ex.forced_step ? ex.forced_step + b * S : nullptr;
        for (int k = tid; k < S; k += kLsgThreads) {
            float xv_k;
            if (k < kFwdStage) {
                xv_k = xsel[par][k];   // written by this same thread above
            } else {
                const int64_t id = ir[(int64_t)k * is.s];
                const bool ok = id >= 0 && id < V;
                bad_index |= !ok;
                xv_k = ok ? Elem<T>::to_float(xr[id]) : __int_as_float(0x7fc00000);
            }
            float out = (xv_k - M) - logS;
            if (forced && forced[k]) out = (fe == k) ? 0.f : -INFINITY;
            sr[(int64_t)k * ss.s] = out;
        }
        if (stats != nullptr && tid == 0) {
            stats[2 * row] = M;
            stats[2 * row + 1] = logS;
        }
    }
    if (bad_index && status) atomicOr(status, DAT_STATUS_BAD_INDEX);
}

// forced_step[b, s] = 1 if some vertex of sentence b is forced to emit target step s
// (the reference's matchmask.sum(-1) > 0, nat_dag_loss.py:114-116).  One CTA per sentence.
__global__ void __launch_bounds__(256)
lsg_forced_steps_kernel(const int64_t *__restrict__ force_emit, int32_t *__restrict__ forced_step,
                        int32_t *__restrict__ status, int L, int S) {
    extern __shared__ int32_t fs_s[];
    const int b = blockIdx.x;
    for (int k = threadIdx.x; k < S; k += blockDim.x) fs_s[k] = 0;
    __syncthreads();
    bool bad = false;
    for (int l = threadIdx.x; l < L; l += blockDim.x) {
        const int64_t t = force_emit[(int64_t)b * L + l];
        if (t >= 0 && t < S) fs_s[t] = 1;   // benign race: every writer stores 1
        else bad |= t >= S;
    }
    __syncthreads();
    for (int k = threadIdx.x; k < S; k += blockDim.x) forced_step[(int64_t)b * S + k] = fs_s[k];
    if (bad && status) atomicOr(status, DAT_STATUS_BAD_INDEX);
}

// Backward, in place.  Shared memory: S * (int + 3 float).
template <typename T>
__global__ void __launch_bounds__(kLsgThreads)
lsg_bwd_kernel(T *__restrict__ x, const int64_t *__restrict__ idx, Strides3 is,
               const float *__restrict__ g, Strides3 gs, const float *__restrict__ stats,
               const int32_t *__restrict__ forced_step, int64_t rows, int L, int S, int V) {
    constexpr int kVec = Elem<T>::kVec;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    int *idx_s = reinterpret_cast<int *>(smem_raw);
    float *g_s = reinterpret_cast<float *>(idx_s + S);
    float *x_s = g_s + S;
    float *tot_s = x_s + S;
    __shared__ float red[kLsgWarps];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
        T *xr = x + row * (int64_t)V;
        const int64_t b = row / L, l = row - b * L;
        const int64_t *ir = idx + b * is.b + l * is.l;
        const float *gr = g + b * gs.b + l * gs.l;
        __syncthreads();  // previous row's fix-ups are done with the staging arrays
        float gsum = 0.f;
        int nonzero = 0;
        const int32_t *forced = forced_step ? forced_step + b * S : nullptr;
        for (int k = tid; k < S; k += kLsgThreads) {
            int64_t id = ir[(int64_t)k * is.s];
            float gv = gr[(int64_t)k * gs.s];
            if (forced && forced[k]) gv = 0.f;   // a forced step's match value is a constant
            bool ok = id >= 0 && id < V;
            idx_s[k] = ok ? (int)id : -1;
            g_s[k] = ok ? gv : 0.f;
            x_s[k] = ok ? Elem<T>::to_float(xr[id]) : 0.f;
            gsum += gv;
            nonzero |= (gv != 0.f);
        }
        float ws = warp_sum(gsum);
        if (lane == 0) red[warp] = ws;
        const int any = __syncthreads_or(nonzero);
        float G = 0.f;
#pragma unroll
        for (int w = 0; w < kLsgWarps; w++) G += red[w];

        int head, nvec;
        row_split(xr, V, head, nvec);
        uint4 *xv = reinterpret_cast<uint4 *>(xr + head);
        const int tail0 = head + nvec * kVec;

        if (!any) {
            // no gradient flows into this row (padding): the result is all zeros, no read
            const uint4 z = make_uint4(0, 0, 0, 0);
            for (int v = tid; v < nvec; v += kLsgThreads) xv[v] = z;
            if (tid < head) xr[tid] = Elem<T>::from_float(0.f);
            if (tail0 + tid < V) xr[tail0 + tid] = Elem<T>::from_float(0.f);
            continue;
        }

        // total gradient arriving at each selected position (duplicates accumulate)
        for (int k = tid; k < S; k += kLsgThreads) {
            const int id = idx_s[k];
            float t = 0.f;
            for (int k2 = 0; k2 < S; k2++) t += (idx_s[k2] == id) ? g_s[k2] : 0.f;
            tot_s[k] = t;
        }

        const float M = stats[2 * row], logS = stats[2 * row + 1];
        const float c = -(M + logS) * kLog2e;
        const float nG = -G;
        int v = tid;
        for (; v + (kBwdUnroll - 1) * kLsgThreads < nvec; v += kBwdUnroll * kLsgThreads) {
            uint4 u[kBwdUnroll];
#pragma unroll
            for (int q = 0; q < kBwdUnroll; q++) u[q] = xv[v + q * kLsgThreads];
#pragma unroll
            for (int q = 0; q < kBwdUnroll; q++) {
                float f[kVec];
                Elem<T>::unpack(u[q], f);
#pragma unroll
                for (int i = 0; i < kVec; i++) f[i] = nG * ex2(fmaf(f[i], kLog2e, c));
                xv[v + q * kLsgThreads] = Elem<T>::pack(f);
            }
        }
        if (v < nvec) {   // the last one to three vectors of this thread, requested together
            const bool p1 = v + kLsgThreads < nvec, p2 = v + 2 * kLsgThreads < nvec;
            uint4 u[3];
            u[0] = xv[v];
            if (p1) u[1] = xv[v + kLsgThreads];
            if (p2) u[2] = xv[v + 2 * kLsgThreads];
#pragma unroll
            for (int q = 0; q < 3; q++) {
                if (q == 0 || (q == 1 ? p1 : p2)) {
                    float f[kVec];
                    Elem<T>::unpack(u[q], f);
#pragma unroll
                    for (int i = 0; i < kVec; i++) f[i] = nG * ex2(fmaf(f[i], kLog2e, c));
                    xv[v + q * kLsgThreads] = Elem<T>::pack(f);
                }
            }
        }
        if (tid < head)
            xr[tid] = Elem<T>::from_float(nG * ex2(fmaf(Elem<T>::to_float(xr[tid]), kLog2e, c)));
        if (tail0 + tid < V)
            xr[tail0 + tid] = Elem<T>::from_float(
                nG * ex2(fmaf(Elem<T>::to_float(xr[tail0 + tid]), kLog2e, c)));
        __syncthreads();  // the whole row is written before the selected positions are fixed up
        for (int k = tid; k < S; k += kLsgThreads) {
            const int id = idx_s[k];
            if (id >= 0) xr[id] = Elem<T>::from_float(fmaf(nG, ex2(fmaf(x_s[k], kLog2e, c)), tot_s[k]));
        }
    }
}

template <typename T, bool kArgmax>
static int launch_fwd_t(const void *x, const int64_t *idx, Strides3 is, float *sel, Strides3 ss,
                        float *stats, int32_t *status, const LsgExtras &ex, int64_t rows, int L, int S,
                        int V, cudaStream_t stream, const DeviceInfo &di, const char *who) {
    int per_sm = 0;
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, lsg_fwd_kernel<T, kArgmax>, kLsgThreads, 0);
    if (per_sm < 1) per_sm = 1;
    int64_t grid = (int64_t)di.sm_count * per_sm;
    if (grid > rows) grid = rows;
    lsg_fwd_kernel<T, kArgmax><<<(unsigned)grid, kLsgThreads, 0, stream>>>(
        static_cast<const T *>(x), idx, is, sel, ss, stats, status, ex, rows, L, S, V);
    return check_launch(who);
}

template <typename T>
static int launch_fwd(const void *x, const int64_t *idx, Strides3 is, float *sel, Strides3 ss,
                      float *stats, int32_t *status, const LsgExtras &ex, int64_t rows, int L, int S,
                      int V, cudaStream_t stream, const DeviceInfo &di, const char *who) {
    return ex.argmax ? launch_fwd_t<T, true>(x, idx, is, sel, ss, stats, status, ex, rows, L, S, V, stream, di, who)
                     : launch_fwd_t<T, false>(x, idx, is, sel, ss, stats, status, ex, rows, L, S, V, stream, di, who);
}

template <typename T>
static int launch_bwd(void *x, const int64_t *idx, Strides3 is, const float *g, Strides3 gs,
                      const float *stats, const int32_t *forced_step, int64_t rows, int L, int S, int V,
                      cudaStream_t stream, const DeviceInfo &di, const char *who) {
    size_t smem = (size_t)S * 16;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(lsg_bwd_kernel<T>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) {
            cudaGetLastError();
            set_error("%s: cannot reserve %zu bytes of shared memory", who, smem);
            return DAT_ERR_UNSUPPORTED;
        }
    }
    int per_sm = 0;
    cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, lsg_bwd_kernel<T>, kLsgThreads, smem);
    if (per_sm < 1) per_sm = 1;
    int64_t grid = (int64_t)di.sm_count * per_sm;
    if (grid > rows) grid = rows;
    lsg_bwd_kernel<T><<<(unsigned)grid, kLsgThreads, smem, stream>>>(
        static_cast<T *>(x), idx, is, g, gs, stats, forced_step, rows, L, S, V);
    return check_launch(who);
}

static int gather_forward(const void *word_ins_out, int dtype, const int64_t *select_idx, Strides3 is,
                          float *selected_result, Strides3 ss, float *row_stats, int32_t *status,
                          const LsgExtras &ex, int bsz, int prelen, int slen, int vocab,
                          cudaStream_t st, const char *who) {
    DAT_REQUIRE(bsz >= 0 && prelen >= 0 && slen >= 0 && vocab >= 1, DAT_ERR_BAD_ARG,
                "%s: bad sizes bsz=%d prelen=%d slen=%d vocab=%d", who, bsz, prelen, slen, vocab);
    if ((int64_t)bsz * prelen == 0) return DAT_OK;
    DAT_REQUIRE(word_ins_out && (slen == 0 || (select_idx && selected_result)), DAT_ERR_BAD_ARG,
                "%s: null pointer", who);
    DeviceInfo di;
    if (!device_info(&di)) return DAT_ERR_NO_DEVICE;
    const int64_t rows = (int64_t)bsz * prelen;
    switch (dtype) {
        case DAT_F32:
            return launch_fwd<float>(word_ins_out, select_idx, is, selected_result, ss, row_stats, status, ex,
                                     rows, prelen, slen, vocab, st, di, who);
        case DAT_F16:
            return launch_fwd<__half>(word_ins_out, select_idx, is, selected_result, ss, row_stats, status, ex,
                                      rows, prelen, slen, vocab, st, di, who);
        case DAT_BF16:
            return launch_fwd<__nv_bfloat16>(word_ins_out, select_idx, is, selected_result, ss, row_stats,
                                             status, ex, rows, prelen, slen, vocab, st, di, who);
        default:
            set_error("%s: unsupported dtype %d (fp32, fp16, bf16 only)", who, dtype);
            return DAT_ERR_UNSUPPORTED;
    }
}

static int gather_backward(void *word_ins_out, int dtype, const int64_t *select_idx, Strides3 is,
                           const float *grad_selected, Strides3 gs, const float *row_stats,
                           const int32_t *forced_step, int bsz, int prelen, int slen, int vocab,
                           cudaStream_t st, const char *who) {
    DAT_REQUIRE(bsz >= 0 && prelen >= 0 && slen >= 0 && vocab >= 1, DAT_ERR_BAD_ARG,
                "%s: bad sizes bsz=%d prelen=%d slen=%d vocab=%d", who, bsz, prelen, slen, vocab);
    if ((int64_t)bsz * prelen == 0) return DAT_OK;
    DAT_REQUIRE(word_ins_out && row_stats && (slen == 0 || (select_idx && grad_selected)), DAT_ERR_BAD_ARG,
                "%s: null pointer", who);
    DAT_REQUIRE(slen <= 4096, DAT_ERR_UNSUPPORTED, "%s: slen=%d exceeds 4096", who, slen);
    DeviceInfo di;
    if (!device_info(&di)) return DAT_ERR_NO_DEVICE;
    const int64_t rows = (int64_t)bsz * prelen;
    switch (dtype) {
        case DAT_F32:
            return launch_bwd<float>(word_ins_out, select_idx, is, grad_selected, gs, row_stats, forced_step,
                                     rows, prelen, slen, vocab, st, di, who);
        case DAT_F16:
            return launch_bwd<__half>(word_ins_out, select_idx, is, grad_selected, gs, row_stats, forced_step,
                                      rows, prelen, slen, vocab, st, di, who);
        case DAT_BF16:
            return launch_bwd<__nv_bfloat16>(word_ins_out, select_idx, is, grad_selected, gs, row_stats,
                                             forced_step, rows, prelen, slen, vocab, st, di, who);
        default:
            set_error("%s: unsupported dtype %d", who, dtype);
            return DAT_ERR_UNSUPPORTED;
    }
}

}  // namespace dat

extern "C" {

int dat_logsoftmax_gather(const void *word_ins_out, int dtype, const int64_t *select_idx,
                          int64_t idx_stride_b, int64_t idx_stride_l, int64_t idx_stride_s,
                          float *selected_result, int64_t sel_stride_b, int64_t sel_stride_l,
                          int64_t sel_stride_s, float *row_stats, int32_t *status, int bsz,
                          int prelen, int slen, int vocab, void *stream) {
    using namespace dat;
    const LsgExtras none{nullptr, nullptr, nullptr};
    return gather_forward(word_ins_out, dtype, select_idx, Strides3{idx_stride_b, idx_stride_l, idx_stride_s},
                          selected_result, Strides3{sel_stride_b, sel_stride_l, sel_stride_s}, row_stats,
                          status, none, bsz, prelen, slen, vocab, static_cast<cudaStream_t>(stream),
                          "dat_logsoftmax_gather");
}

int dat_logsoftmax_gather_fused(const void *word_ins_out, int dtype, const int64_t *select_idx,
                                int64_t idx_stride_b, int64_t idx_stride_l, int64_t idx_stride_s,
                                float *selected_result, int64_t sel_stride_b, int64_t sel_stride_l,
                                int64_t sel_stride_s, float *row_stats, int64_t *argmax,
                                const int64_t *force_emit, int32_t *forced_step, int32_t *status,
                                int bsz, int prelen, int slen, int vocab, void *stream) {
    using namespace dat;
    const char *who = "dat_logsoftmax_gather_fused";
    DAT_REQUIRE(!force_emit || forced_step, DAT_ERR_BAD_ARG,
                "%s: force_emit needs the forced_step workspace [bsz, slen]", who);
    DAT_REQUIRE(slen <= 8192, DAT_ERR_UNSUPPORTED, "%s: slen=%d exceeds 8192", who, slen);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (force_emit && (int64_t)bsz * prelen > 0 && slen > 0) {
        lsg_forced_steps_kernel<<<(unsigned)bsz, 256, (size_t)slen * sizeof(int32_t), st>>>(
            force_emit, forced_step, status, prelen, slen);
        if (int rc = check_launch(who)) return rc;
    }
    const LsgExtras ex{argmax, force_emit, force_emit ? forced_step : nullptr};
    return gather_forward(word_ins_out, dtype, select_idx, Strides3{idx_stride_b, idx_stride_l, idx_stride_s},
                          selected_result, Strides3{sel_stride_b, sel_stride_l, sel_stride_s}, row_stats,
                          status, ex, bsz, prelen, slen, vocab, st, who);
}

int dat_logsoftmax_gather_backward(void *word_ins_out, int dtype, const int64_t *select_idx,
                                   int64_t idx_stride_b, int64_t idx_stride_l,
                                   int64_t idx_stride_s, const float *grad_selected,
                                   int64_t g_stride_b, int64_t g_stride_l, int64_t g_stride_s,
                                   const float *row_stats, int bsz, int prelen, int slen,
                                   int vocab, void *stream) {
    using namespace dat;
    return gather_backward(word_ins_out, dtype, select_idx, Strides3{idx_stride_b, idx_stride_l, idx_stride_s},
                           grad_selected, Strides3{g_stride_b, g_stride_l, g_stride_s}, row_stats, nullptr,
                           bsz, prelen, slen, vocab, static_cast<cudaStream_t>(stream),
                           "dat_logsoftmax_gather_backward");
}

int dat_logsoftmax_gather_backward_fused(void *word_ins_out, int dtype, const int64_t *select_idx,
                                         int64_t idx_stride_b, int64_t idx_stride_l,
                                         int64_t idx_stride_s, const float *grad_selected,
                                         int64_t g_stride_b, int64_t g_stride_l, int64_t g_stride_s,
                                         const float *row_stats, const int32_t *forced_step, int bsz,
                                         int prelen, int slen, int vocab, void *stream) {
    using namespace dat;
    return gather_backward(word_ins_out, dtype, select_idx, Strides3{idx_stride_b, idx_stride_l, idx_stride_s},
                           grad_selected, Strides3{g_stride_b, g_stride_l, g_stride_s}, row_stats, forced_step,
                           bsz, prelen, slen, vocab, static_cast<cudaStream_t>(stream),
                           "dat_logsoftmax_gather_backward_fused");
}

}  // extern "C"
