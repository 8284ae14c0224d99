// dag_best_alignment for sm_100a: max-plus (Viterbi) sweep with trace, and the backtrace,
// in one launch.  Replaces calculate_maxalpha_kernel / calculate_backtrace_kernel and
// their host wrapper (fs_plugins/custom_ops/dag_best_alignment.cu:39-130, 170-189,
// 219-263) and the int32 -> int64 cast of fs_plugins/custom_ops/dag_loss.py:162.
//
// Values are the reference's own fp32 sums (alpha[t-1,i] + links[i,d-1], then + match[t,j]),
// so the maxima are bit-identical; the winner among equal candidates follows the
// reference's lane scan + shfl_down tree for TRANS_BLOCK_SIZE = 2^lg lanes
// (dag_best_alignment.cu:96-111): lane = (d-1) mod 2^lg, lanes preferred in bit-reversed
// order, then the smaller distance d.  That order is a total order on (value, rank), so any
// reduction tree gives the reference's answer.
//
// Layout: the band is first copied into a square, 16-byte aligned matrix Lsq[i][j] with
// -inf everywhere a transition does not exist (dag_align_prep_kernel).  In absolute vertex
// coordinates -inf replaces all masks (as 0 does in the probability-domain loss kernel), so
// a warp reads tiles of 16 rows x 128 columns with aligned 128-bit loads and no predicates;
// each lane owns 4 columns.  Per candidate the common path is 5 instructions (add, two
// compares, max, select); a chunk in which any lane saw an exact tie is redone with the full
// tie-break rule.  Warps merge their per-column winners through shared memory with a 64-bit
// atomicMax on (order-preserving value bits, inverted rank).
//
// One CTA owns one sentence; the trace (predecessor distances, uint16) stays in shared
// memory when it fits, and one thread walks it back at the end of the same launch.
#include "dag_tiles.cuh"

namespace dat {

constexpr int kAlignThreads = 512;
constexpr int kAlignWarps = kAlignThreads / 32;
constexpr int kRankNone = 0x7fffffff;
constexpr float kNoCand = -3.402823466e+38f;

__host__ __device__ inline int align_pitch(int L) { return (L + 127) & ~127; }
__host__ __device__ inline int align_rows(int L) { return (L + 15) & ~15; }

__device__ __forceinline__ int tie_rank(int d, int lg) {
    // bit-reversed lane in the high bits, distance in the low 20 bits
    const unsigned lane = (unsigned)(d - 1) & ((1u << lg) - 1u);
    const unsigned rev = __brev(lane) >> (32 - lg);
    return (int)((rev << 20) | (unsigned)d);
}

// order-preserving map float -> uint32 (larger float <=> larger unsigned)
__device__ __forceinline__ unsigned orderable(float v) {
    const unsigned u = __float_as_uint(v);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}
__device__ __forceinline__ float unorderable(unsigned o) {
    return __uint_as_float((o & 0x80000000u) ? (o & 0x7fffffffu) : ~o);
}
__device__ __forceinline__ unsigned long long pack_key(float v, int rank) {
    v += 0.0f;  // -0.0 and +0.0 compare equal in the reference
    return ((unsigned long long)orderable(v) << 32) | (unsigned long long)(0xffffffffu - (unsigned)rank);
}

// square copy of the band, natural-log values, -inf where no transition exists
__global__ void __launch_bounds__(256)
dag_align_prep_kernel(const float *__restrict__ links, const int64_t *__restrict__ output_length,
                      const int64_t *__restrict__ target_length, float *__restrict__ lsq_all, int T,
                      int L, int K, int rows, int pitch) {
    const int b = blockIdx.y;
    const int i = blockIdx.x * 8 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (i >= rows) return;
    const long long oll = output_length[b], tll = target_length[b];
    if (!lengths_valid(oll, tll, T, L)) return;
    const int ol = (int)oll;
    const float *brow = links + ((size_t)b * L + (i < L ? i : 0)) * K;
    float4 *erow = reinterpret_cast<float4 *>(lsq_all + ((size_t)b * rows + i) * pitch);
    for (int jv = lane; jv < pitch / 4; jv += 32) {
        float v[4];
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const int j = 4 * jv + k;
            const int d = j - i - 1;
            const bool ok = i < ol && j < ol && d >= 0 && d < K;
            v[k] = ok ? __ldg(brow + d) : -INFINITY;
        }
        erow[jv] = make_float4(v[0], v[1], v[2], v[3]);
    }
}

template <bool kTraceInSmem>
__global__ void __launch_bounds__(kAlignThreads, 1)
dag_align_kernel(const float *__restrict__ match_all, const float *__restrict__ lsq_all,
                 const int64_t *__restrict__ output_length, const int64_t *__restrict__ target_length,
                 int64_t *__restrict__ path_out, float *__restrict__ max_score,
                 uint16_t *__restrict__ trace_ws, int32_t *__restrict__ status, int T, int L, int K,
                 int lg, int rows, int pitch) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int b = blockIdx.x;
    int64_t *path = path_out + (size_t)b * L;
    for (int j = tid; j < L; j += kAlignThreads) path[j] = -1;
    const long long oll = output_length[b], tll = target_length[b];
    if (!lengths_valid(oll, tll, T, L)) {
        if (tid == 0) {
            if (max_score) max_score[b] = -INFINITY;
            if (status) atomicOr(status, DAT_STATUS_BAD_LENGTH);
        }
        return;
    }
    const int ol = (int)oll, tl = (int)tll;
    const int W = ol - tl + 1;
    const float *match = match_all + (size_t)b * T * L;
    const float *Lsq = lsq_all + (size_t)b * rows * pitch;
    const int rp = pitch + 32;
    unsigned long long *skey = reinterpret_cast<unsigned long long *>(smem_raw);  // [pitch]
    float *rbuf0 = reinterpret_cast<float *>(skey + pitch), *rbuf1 = rbuf0 + rp;
    // trace[t][c]: distance d of the chosen predecessor of window column c at step t (0 = none)
    uint16_t *trace = kTraceInSmem ? reinterpret_cast<uint16_t *>(rbuf1 + rp) : trace_ws + (size_t)b * T * L;
    const int tstride = kTraceInSmem ? W : L;
    const unsigned long long key_none = pack_key(-INFINITY, kRankNone);

    for (int x = tid; x < 2 * rp; x += kAlignThreads) rbuf0[x] = -INFINITY;
    for (int x = tid; x < pitch; x += kAlignThreads) skey[x] = key_none;
    __syncthreads();
    if (tid == 0) rbuf0[0] = match[0];
    __syncthreads();

    const int ncbmax = pitch >> 7;
    for (int t = 1; t < tl; t++) {
        const float *prev = ((t - 1) & 1) ? rbuf1 : rbuf0;  // absolute coordinates, -inf outside the window
        float *cur = (t & 1) ? rbuf1 : rbuf0;
        // live region: rows [t-1, t+W-2], columns [t, t+W-1]
        const int rt_lo = (t - 1) >> 4, rt_hi = (t + W - 2) >> 4;
        const int cb_lo = t >> 7;
        int cb_hi = (t + W - 1) >> 7;
        if (cb_hi > ncbmax - 1) cb_hi = ncbmax - 1;
        int total = 0;
        for (int cb = cb_lo; cb <= cb_hi; cb++) {
            int rf = 128 * cb - K; rf = rf > 0 ? (rf >> 4) : 0; rf = rf > rt_lo ? rf : rt_lo;
            int rl = 8 * cb + 7; rl = rl < rt_hi ? rl : rt_hi;
            total += rl >= rf ? rl - rf + 1 : 0;
        }
        const int my_lo = (warp * total) / kAlignWarps, my_hi = ((warp + 1) * total) / kAlignWarps;
        const bool reverse = t & 1;
        // match values of the columns this thread finalises, requested before the tile phase
        float mp[2];
#pragma unroll
        for (int q = 0; q < 2; q++) {
            const int j = 128 * cb_lo + tid + q * kAlignThreads, c = j - t;
            mp[q] = (c >= 0 && c < W) ? __ldg(match + (size_t)t * L + j) : 0.f;
        }
        int base = 0;
        for (int cbx = cb_lo; cbx <= cb_hi; cbx++) {
            const int cb = reverse ? (cb_hi - (cbx - cb_lo)) : cbx;
            int rf = 128 * cb - K; rf = rf > 0 ? (rf >> 4) : 0; rf = rf > rt_lo ? rf : rt_lo;
            int rl = 8 * cb + 7; rl = rl < rt_hi ? rl : rt_hi;
            const int n = rl >= rf ? rl - rf + 1 : 0;
            const int from = my_lo > base ? my_lo - base : 0;
            const int to = my_hi < base + n ? my_hi - base : n;
            base += n;
            if (from >= to) continue;
            const int col = 128 * cb + 4 * lane;
            // "nothing yet" is the most negative finite float rather than -inf, so that the
            // -inf of non-existent transitions never compares equal to it (no false ties)
            float bv[4] = {kNoCand, kNoCand, kNoCand, kNoCand};
            int bi[4] = {-1, -1, -1, -1};
            for (int q = from; q < to; q++) {
                const int rt = reverse ? (rl - q) : (rf + q);
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    const int i0 = 16 * rt + 8 * h;
                    const float4 *ep = reinterpret_cast<const float4 *>(Lsq + (size_t)i0 * pitch + col);
                    float4 e[8];
#pragma unroll
                    for (int r = 0; r < 8; r++) e[r] = __ldg(ep + (size_t)r * (pitch >> 2));
                    const float4 a0 = *reinterpret_cast<const float4 *>(prev + i0);
                    const float4 a1 = *reinterpret_cast<const float4 *>(prev + i0 + 4);
                    const float av[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
                    const float sv[4] = {bv[0], bv[1], bv[2], bv[3]};
                    const int si[4] = {bi[0], bi[1], bi[2], bi[3]};
                    bool tie = false;
#pragma unroll
                    for (int r = 0; r < 8; r++) {
                        const float v[4] = {__fadd_rn(av[r], e[r].x), __fadd_rn(av[r], e[r].y),
                                            __fadd_rn(av[r], e[r].z), __fadd_rn(av[r], e[r].w)};
#pragma unroll
                        for (int k = 0; k < 4; k++) {
                            tie |= (v[k] == bv[k]);
                            const bool up = v[k] > bv[k];
                            bv[k] = up ? v[k] : bv[k];
                            bi[k] = up ? (i0 + r) : bi[k];
                        }
                    }
                    if (__any_sync(0xffffffffu, tie)) {
                        // redo the chunk with the reference's full tie-break
#pragma unroll
                        for (int k = 0; k < 4; k++) { bv[k] = sv[k]; bi[k] = si[k]; }
#pragma unroll
                        for (int r = 0; r < 8; r++) {
                            const float v[4] = {__fadd_rn(av[r], e[r].x), __fadd_rn(av[r], e[r].y),
                                                __fadd_rn(av[r], e[r].z), __fadd_rn(av[r], e[r].w)};
#pragma unroll
                            for (int k = 0; k < 4; k++) {
                                const int j = col + k, i = i0 + r;
                                bool up = v[k] > bv[k];
                                if (!up && v[k] == bv[k] && v[k] > -INFINITY && j > i) {
                                    const int rnew = tie_rank(j - i, lg);
                                    const int rold = bi[k] >= 0 ? tie_rank(j - bi[k], lg) : kRankNone;
                                    up = rnew < rold;
                                }
                                if (up) { bv[k] = v[k]; bi[k] = i; }
                            }
                        }
                    }
                }
            }
#pragma unroll
            for (int k = 0; k < 4; k++) {
                const int rank = (bi[k] >= 0) ? tie_rank(col + k - bi[k], lg) : kRankNone;
                if (rank != kRankNone) atomicMax(skey + col + k, pack_key(bv[k], rank));
            }
        }
        __syncthreads();

        // finalisation: consume and clear every merge slot that may have been touched
        int fq = 0;
        for (int j = 128 * cb_lo + tid; j < 128 * (cb_hi + 1); j += kAlignThreads, fq++) {
            const unsigned long long key = skey[j];
            skey[j] = key_none;
            const int c = j - t;
            if (c >= 0 && c < W) {
                const float best = unorderable((unsigned)(key >> 32));
                const int rank = (int)(0xffffffffu - (unsigned)(key & 0xffffffffu));
                const float mt = fq == 0 ? mp[0] : (fq == 1 ? mp[1] : __ldg(match + (size_t)t * L + j));
                float v = __fadd_rn(best, mt);
                if (!(v > -INFINITY)) v = -INFINITY;
                cur[j] = v;
                const int d = (rank == kRankNone) ? 0 : (rank & 0xfffff);
                trace[(size_t)t * tstride + (kTraceInSmem ? c : j)] = (uint16_t)d;
            }
        }
        if (tid == 0) {  // entries of the recycled row buffer that left the window
            cur[t - 1] = -INFINITY;
            if (t >= 2) cur[t - 2] = -INFINITY;
        }
        __syncthreads();
    }

    // backtrace (dag_best_alignment.cu:185-188), one thread
    if (tid == 0) {
        const float score = (((tl - 1) & 1) ? rbuf1 : rbuf0)[ol - 1];
        if (max_score) max_score[b] = score;
        if (score > -INFINITY) {
            int pos = ol - 1;
            for (int t = tl - 1; t >= 0; t--) {
                path[pos] = t;
                if (t == 0) break;
                const int c = pos - t;
                if (c < 0 || c >= W) break;  // cannot happen on a finite path
                const int d = trace[(size_t)t * tstride + (kTraceInSmem ? c : pos)];
                if (d == 0 || d > pos) break;
                pos -= d;
            }
        } else if (status) {
            atomicOr(status, DAT_STATUS_NO_PATH);
        }
    }
}

static inline size_t align_base_smem(int L) {
    const int pitch = align_pitch(L);
    return (size_t)pitch * 8 + (size_t)2 * (pitch + 32) * 4;
}
static inline size_t align_lsq_bytes(int B, int L) {
    return (((size_t)B * align_rows(L) * align_pitch(L) * sizeof(float)) + 255) & ~(size_t)255;
}

}  // namespace dat

extern "C" {

size_t dat_dag_best_alignment_workspace_bytes(int bsz, int tarlen, int prelen) {
    if (bsz <= 0 || tarlen <= 0 || prelen <= 0) return 0;
    // square copy of the links + (only used when it does not fit in shared memory) the trace
    return dat::align_lsq_bytes(bsz, prelen) + (size_t)bsz * tarlen * prelen * sizeof(uint16_t) + 512;
}

int dat_dag_best_alignment(const float *match_all, const float *links,
                           const int64_t *output_length, const int64_t *target_length,
                           int64_t *path, float *max_score, void *workspace, int32_t *status,
                           int bsz, int tarlen, int prelen, int translen, int config,
                           void *stream) {
    using namespace dat;
    DAT_REQUIRE(bsz >= 0 && tarlen >= 1 && prelen >= 1 && translen >= 1, DAT_ERR_BAD_ARG,
                "dat_dag_best_alignment: bad sizes bsz=%d tarlen=%d prelen=%d translen=%d", bsz,
                tarlen, prelen, translen);
    DAT_REQUIRE(config >= 1 && config <= 4, DAT_ERR_BAD_ARG,
                "dat_dag_best_alignment: config should be 1~4 (got %d)", config);
    if (bsz == 0) return DAT_OK;
    DAT_REQUIRE(match_all && links && output_length && target_length && path && workspace,
                DAT_ERR_BAD_ARG, "dat_dag_best_alignment: null pointer");
    DAT_REQUIRE(prelen <= 65535, DAT_ERR_UNSUPPORTED,
                "dat_dag_best_alignment: prelen=%d exceeds 65535", prelen);
    DeviceInfo di;
    if (!device_info(&di)) return DAT_ERR_NO_DEVICE;
    const int lg = config + 1;  // 4, 8, 16, 32 lanes
    const int rows = align_rows(prelen), pitch = align_pitch(prelen);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const uintptr_t wbase = (reinterpret_cast<uintptr_t>(workspace) + 255) & ~(uintptr_t)255;
    float *lsq = reinterpret_cast<float *>(wbase);
    uint16_t *trace_ws = reinterpret_cast<uint16_t *>(wbase + align_lsq_bytes(bsz, prelen));
    {
        dim3 grid((rows + 7) / 8, bsz);
        dag_align_prep_kernel<<<grid, 256, 0, st>>>(links, output_length, target_length, lsq, tarlen,
                                                    prelen, translen, rows, pitch);
        if (int rc = check_launch("dat_dag_best_alignment(prep)")) return rc;
    }
    const size_t base = (align_base_smem(prelen) + 15) & ~(size_t)15;
    DAT_REQUIRE(base <= (size_t)di.max_smem_optin, DAT_ERR_UNSUPPORTED,
                "dat_dag_best_alignment: prelen=%d needs %zu bytes of shared memory", prelen, base);
    const size_t with_trace = base + (size_t)tarlen * prelen * sizeof(uint16_t);
    if (with_trace <= (size_t)di.max_smem_optin) {
        if (cudaFuncSetAttribute(dag_align_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)with_trace) != cudaSuccess)
            return check_launch("dat_dag_best_alignment(attr)");
        dag_align_kernel<true><<<(unsigned)bsz, kAlignThreads, with_trace, st>>>(
            match_all, lsq, output_length, target_length, path, max_score, nullptr, status, tarlen,
            prelen, translen, lg, rows, pitch);
    } else {
        if (cudaFuncSetAttribute(dag_align_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)base) != cudaSuccess)
            return check_launch("dat_dag_best_alignment(attr)");
        dag_align_kernel<false><<<(unsigned)bsz, kAlignThreads, base, st>>>(
            match_all, lsq, output_length, target_length, path, max_score, trace_ws, status, tarlen,
            prelen, translen, lg, rows, pitch);
    }
    return check_launch("dat_dag_best_alignment");
}

}  // extern "C"
