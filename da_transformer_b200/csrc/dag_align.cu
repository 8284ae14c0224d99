// dag_best_alignment for sm_100a: max-plus (Viterbi) sweep with trace, and the backtrace,
// in one launch.  Replaces calculate_maxalpha_kernel / calculate_backtrace_kernel and
// their host wrapper (fs_plugins/custom_ops/dag_best_alignment.cu:39-130, 170-189,
// 219-263) and the int32 -> int64 cast of fs_plugins/custom_ops/dag_loss.py:162.
//
// One CTA owns one sentence.  Values are the reference's own fp32 sums
// (alpha[t-1,i] + links[i,d-1], then + match[t,j]), so the maxima are bit-identical; the
// winner among equal candidates follows the reference's lane scan + shfl_down tree for
// TRANS_BLOCK_SIZE = 2^lg lanes (dag_best_alignment.cu:96-111): lane = (d-1) mod 2^lg,
// lanes preferred in bit-reversed order, then the smaller distance d.  That order is a
// total order on (value, rank), so any reduction tree gives the reference's answer.
#include "dag_tiles.cuh"

namespace dat {

constexpr int kRankNone = 0x7fffffff;

__device__ __forceinline__ int tie_rank(int d, int lg) {
    // bit-reversed lane in the high bits, distance in the low 20 bits
    const unsigned lane = (unsigned)(d - 1) & ((1u << lg) - 1u);
    const unsigned rev = __brev(lane) >> (32 - lg);
    return (int)((rev << 20) | (unsigned)d);
}

__device__ __forceinline__ void better(float &bv, int &br, float v, int r) {
    if (v > bv || (v == bv && r < br && v > -INFINITY)) {
        bv = v;
        br = r;
    }
}

template <bool kTraceInSmem>
__global__ void __launch_bounds__(kSweepThreads)
dag_align_kernel(const float *__restrict__ match_all, const float *__restrict__ links,
                 const int64_t *__restrict__ output_length, const int64_t *__restrict__ target_length,
                 int64_t *__restrict__ path_out, float *__restrict__ max_score,
                 uint16_t *__restrict__ trace_ws, int32_t *__restrict__ status, int T, int L, int K,
                 int lg) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int b = blockIdx.x;
    int64_t *path = path_out + (size_t)b * L;
    for (int j = tid; j < L; j += kSweepThreads) path[j] = -1;
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
    const float *band = links + (size_t)b * L * K;
    const SweepSmem sm = carve(smem_raw, L);
    // the partial-merge slots hold (value, rank) pairs here
    int *part_r = reinterpret_cast<int *>(sm.part);
    int *fin_r = reinterpret_cast<int *>(sm.fin_s);
    // trace[t][c]: distance d of the chosen predecessor of window column c at step t (0 = none)
    uint16_t *trace = kTraceInSmem
                          ? reinterpret_cast<uint16_t *>(smem_raw + ((sweep_smem_bytes(L) + 15) & ~(size_t)15))
                          : trace_ws + (size_t)b * T * L;
    const int tstride = kTraceInSmem ? W : L;

    const int pitch = sweep_row_pitch(L);
    for (int x = tid; x < 2 * pitch; x += kSweepThreads) sm.row0[x] = -INFINITY;  // row0 and row1
    int my_lo, my_hi, cb_first;
    build_tile_plan(sm, W, K, my_lo, my_hi, cb_first);
    // warps without tiles sit between the first and last warp of a shared column block:
    // their merge slots must read as empty
#pragma unroll
    for (int which = 0; which < 2; which++) {
        const int o = ((which * kSweepWarps + warp) * 2) * 32;
        sm.part[o + lane] = -INFINITY;
        part_r[o + 32 + lane] = kRankNone;
    }
    if (tid == 0) sm.row0[0] = match[0];
    __syncthreads();

    const unsigned stride = (unsigned)(K - 1);
    for (int t = 1; t < tl; t++) {
        const float *prev = (t & 1) ? sm.row0 : sm.row1;  // row of step t-1, window coordinates
        float *cur = (t & 1) ? sm.row1 : sm.row0;
        float mt[2];
#pragma unroll
        for (int q = 0; q < 2; q++) {
            int c = tid + q * kSweepThreads;
            mt[q] = (c < W) ? __ldg(match + (size_t)t * L + t + c) : 0.f;
        }
        if (my_lo < my_hi) {
            int cb = cb_first;
            int rb = sm.rb_lo[cb] + (my_lo - sm.tile_start[cb]);
            bool owns_start = (my_lo == sm.tile_start[cb]);
            float bv = -INFINITY;
            int br = kRankNone;
            const unsigned row_base = (unsigned)(t - 1) * (unsigned)K;
            for (int tile = my_lo; tile < my_hi;) {
                const TileGeom g = tile_geom(cb, rb, lane, W, K);
                const unsigned off0 = row_base + (unsigned)g.c;
                if (g.interior) {
#pragma unroll 1
                    for (int r = g.r0; r < g.r0 + 32; r += kChunk) {
                        const float4 p0 = *reinterpret_cast<const float4 *>(prev + r);
                        const float4 p1 = *reinterpret_cast<const float4 *>(prev + r + 4);
                        const float pa[kChunk] = {p0.x, p0.y, p0.z, p0.w, p1.x, p1.y, p1.z, p1.w};
                        const unsigned o = off0 + (unsigned)r * stride;
                        float x[kChunk];
#pragma unroll
                        for (int u = 0; u < kChunk; u++) x[u] = __ldg(band + (o + (unsigned)u * stride));
#pragma unroll
                        for (int u = 0; u < kChunk; u++) x[u] = __fadd_rn(pa[u], x[u]);
                        float cm = x[0];
#pragma unroll
                        for (int u = 1; u < kChunk; u++) cm = fmaxf(cm, x[u]);
                        if (cm >= bv && cm > -INFINITY) {  // some candidate of the chunk may win or tie
#pragma unroll
                            for (int u = 0; u < kChunk; u++)
                                if (x[u] >= bv) better(bv, br, x[u], tie_rank(g.c - (r + u) + 1, lg));
                        }
                    }
                } else {
#pragma unroll 1
                    for (int r = g.r0; r < g.r1; r += kChunk) {
                        float x[kChunk];
#pragma unroll
                        for (int u = 0; u < kChunk; u++) {
                            const int rr = r + u;
                            const bool ok = (rr >= g.rmin) && (rr <= g.rmax);
                            const float lk = ok ? __ldg(band + (off0 + (unsigned)rr * stride)) : -INFINITY;
                            x[u] = __fadd_rn(prev[rr], lk);  // rows past the window read the -inf padding
                        }
#pragma unroll
                        for (int u = 0; u < kChunk; u++)
                            if (x[u] >= bv && x[u] > -INFINITY)
                                better(bv, br, x[u], tie_rank(g.c - (r + u) + 1, lg));
                    }
                }
                tile++;
                rb++;
                if (rb > cb || tile == my_hi) {
                    const bool complete = owns_start && (rb > cb);
                    if (complete) {
                        if (g.c < W) { sm.fin_m[g.c] = bv; fin_r[g.c] = br; }
                    } else {
                        const int which = (cb == cb_first) ? 0 : 1;
                        const int o = ((which * kSweepWarps + warp) * 2) * 32;
                        sm.part[o + lane] = bv;
                        part_r[o + 32 + lane] = br;
                    }
                    cb++;
                    rb = sm.rb_lo[cb];
                    owns_start = true;
                    bv = -INFINITY;
                    br = kRankNone;
                }
            }
        }
        __syncthreads();
#pragma unroll
        for (int q = 0; q < 2; q++) {
            const int c = tid + q * kSweepThreads;
            if (c < W) {
                const int cb = c >> 5, ln = c & 31;
                const int wa = sm.first_warp[cb], wb = sm.last_warp[cb];
                float bv;
                int br;
                if (wa == wb) {
                    bv = sm.fin_m[c];
                    br = fin_r[c];
                } else {
                    bv = -INFINITY;
                    br = kRankNone;
                    for (int w = wa; w <= wb; w++) {
                        const int which = (sm.cb_first_of[w] == cb) ? 0 : 1;
                        const int o = ((which * kSweepWarps + w) * 2) * 32;
                        better(bv, br, sm.part[o + ln], part_r[o + 32 + ln]);
                    }
                }
                float v = __fadd_rn(bv, mt[q]);
                if (!(v > -INFINITY)) v = -INFINITY;  // keeps the -inf padding convention under NaN
                cur[c] = v;
                const int d = (br == kRankNone) ? 0 : (br & 0xfffff);
                trace[(size_t)t * tstride + (kTraceInSmem ? c : (t + c))] = (uint16_t)d;
            }
        }
        __syncthreads();
    }

    // backtrace (dag_best_alignment.cu:185-188), one thread
    if (tid == 0) {
        const float score = (((tl - 1) & 1) ? sm.row1 : sm.row0)[W - 1];
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

static inline size_t align_trace_smem(int T, int L) {
    // worst case window W = L - 2 + 1
    return (size_t)T * (size_t)L * sizeof(uint16_t);
}

}  // namespace dat

extern "C" {

size_t dat_dag_best_alignment_workspace_bytes(int bsz, int tarlen, int prelen) {
    if (bsz < 0 || tarlen < 0 || prelen < 0) return 0;
    return (size_t)bsz * tarlen * prelen * sizeof(uint16_t) + 16;
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
    DAT_REQUIRE(match_all && links && output_length && target_length && path, DAT_ERR_BAD_ARG,
                "dat_dag_best_alignment: null pointer");
    DAT_REQUIRE(prelen <= 2 * kSweepThreads, DAT_ERR_UNSUPPORTED,
                "dat_dag_best_alignment: prelen=%d exceeds %d", prelen, 2 * kSweepThreads);
    DeviceInfo di;
    if (!device_info(&di)) return DAT_ERR_NO_DEVICE;
    const int lg = config + 1;  // 4, 8, 16, 32 lanes
    const size_t base = (sweep_smem_bytes(prelen) + 15) & ~(size_t)15;
    const size_t with_trace = base + align_trace_smem(tarlen, prelen);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (with_trace <= (size_t)di.max_smem_optin) {
        if (cudaFuncSetAttribute(dag_align_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)with_trace) != cudaSuccess)
            return check_launch("dat_dag_best_alignment(attr)");
        dag_align_kernel<true><<<(unsigned)bsz, kSweepThreads, with_trace, st>>>(
            match_all, links, output_length, target_length, path, max_score, nullptr, status,
            tarlen, prelen, translen, lg);
    } else {
        DAT_REQUIRE(workspace != nullptr, DAT_ERR_BAD_ARG,
                    "dat_dag_best_alignment: workspace required for tarlen=%d prelen=%d", tarlen,
                    prelen);
        DAT_REQUIRE(base <= (size_t)di.max_smem_optin, DAT_ERR_UNSUPPORTED,
                    "dat_dag_best_alignment: prelen=%d too large", prelen);
        if (cudaFuncSetAttribute(dag_align_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)base) != cudaSuccess)
            return check_launch("dat_dag_best_alignment(attr)");
        uint16_t *ws = reinterpret_cast<uint16_t *>(
            (reinterpret_cast<uintptr_t>(workspace) + 15) & ~(uintptr_t)15);
        dag_align_kernel<false><<<(unsigned)bsz, kSweepThreads, base, st>>>(
            match_all, links, output_length, target_length, path, max_score, ws, status, tarlen,
            prelen, translen, lg);
    }
    return check_launch("dat_dag_best_alignment");
}

}  // extern "C"
