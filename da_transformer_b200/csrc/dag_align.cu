// dag_best_alignment for sm_100a: max-plus (Viterbi) sweep and the backtrace in one launch.
// Replaces calculate_maxalpha_kernel / calculate_backtrace_kernel and their host wrapper
// (fs_plugins/custom_ops/dag_best_alignment.cu:39-130, 170-189, 219-263) and the
// int32 -> int64 cast of fs_plugins/custom_ops/dag_loss.py:162.
//
// Values are the reference's own fp32 sums (alpha[t-1,i] + links[i,d-1], then + match[t,j]),
// so the maxima are bit-identical.  The reference records the winning predecessor of EVERY
// (t, j) during the sweep; only the tl-1 entries on the best path are ever read.  Here the
// sweep keeps just the row maxima (an add and a three-input max per two candidates) and keeps
// all rows; the backtrace then recomputes, for the one vertex per step that lies on the path,
// the candidates alpha[t-1,i] + links[i,pos] (the same fp32 additions, hence the same bits)
// and picks the winner among the maximal ones with the reference's rule: its lane scan +
// shfl_down tree for TRANS_BLOCK_SIZE = 2^lg lanes (dag_best_alignment.cu:96-111) prefers
// lane = (d-1) mod 2^lg in bit-reversed order, then the smaller distance d.  That is a total
// order on (value, rank), so one max-reduction over 64-bit keys gives the reference's answer.
//
// Layout: the band is first copied into a square, 16-byte aligned matrix Lsq[i][j] with
// -inf everywhere a transition does not exist (dag_align_prep_kernel).  In absolute vertex
// coordinates -inf replaces all masks (as 0 does in the probability-domain loss kernel), so
// a warp reads half-tiles of 8 rows x 128 columns with aligned 128-bit loads and no
// predicates; each lane owns 4 columns.  Warps merge their per-column maxima through shared
// memory with a 32-bit atomicMax on order-preserving value bits.
//
// One CTA owns one sentence; the rows stay in shared memory when they fit (else in the
// caller's workspace).
#include "dag_tiles.cuh"

namespace dat {

constexpr int kAlignThreads = 512;
constexpr int kAlignWarps = kAlignThreads / 32;

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

// Largest 64-bit key over the CTA, returned to every thread: hardware warp reductions on the
// two halves, one slot per warp, one CTA barrier.  `slots` alternates between two arrays from
// one call to the next, so a slot is rewritten only after every thread has passed the barrier
// that follows its last read.
__device__ __forceinline__ unsigned long long cta_max_key(unsigned long long key, unsigned long long *slots,
                                                          int lane, int warp) {
    const unsigned hi = (unsigned)(key >> 32);
    const unsigned mh = __reduce_max_sync(0xffffffffu, hi);
    const unsigned ml = __reduce_max_sync(0xffffffffu, hi == mh ? (unsigned)key : 0u);
    if (lane == 0) slots[warp] = ((unsigned long long)mh << 32) | ml;
    __syncthreads();
    const unsigned long long k = lane < kAlignWarps ? slots[lane] : 0ull;
    const unsigned kh = (unsigned)(k >> 32);
    const unsigned wh = __reduce_max_sync(0xffffffffu, kh);
    const unsigned wl = __reduce_max_sync(0xffffffffu, kh == wh ? (unsigned)k : 0u);
    return ((unsigned long long)wh << 32) | wl;
}

// kRowsInSmem: all tl rows live in shared memory in absolute vertex coordinates (stride
// pitch+32, -inf outside the reachable window).  Otherwise two row buffers ping-pong in shared
// memory and every finished row is also written to rows_ws[b][t][j] for the backtrace.
template <bool kRowsInSmem>
__global__ void __launch_bounds__(kAlignThreads, 1)
dag_align_kernel(const float *__restrict__ match_all, const float *__restrict__ lsq_all,
                 const int64_t *__restrict__ output_length, const int64_t *__restrict__ target_length,
                 int64_t *__restrict__ path_out, float *__restrict__ max_score,
                 float *rows_ws, int32_t *__restrict__ status, int T, int L, int K,
                 int lg, int rows, int pitch) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __shared__ unsigned long long bt_key[2][kAlignWarps];
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
    unsigned *skey = reinterpret_cast<unsigned *>(smem_raw);  // [pitch] per-column merge slots
    float *rbuf = reinterpret_cast<float *>(skey + pitch);    // tl rows, or 2 when the rows go to rows_ws
    float *grow = kRowsInSmem ? nullptr : rows_ws + (size_t)b * T * L;
    const unsigned key_none = orderable(-INFINITY);

    for (int x = tid; x < (kRowsInSmem ? tl : 2) * rp; x += kAlignThreads) rbuf[x] = -INFINITY;
    for (int x = tid; x < pitch; x += kAlignThreads) skey[x] = key_none;
    if (!kRowsInSmem)   // row 0 of the workspace copy: only vertex 0 is reachable
        for (int j = 1 + tid; j < W; j += kAlignThreads) grow[j] = -INFINITY;
    __syncthreads();
    if (tid == 0) {
        rbuf[0] = match[0];
        if (!kRowsInSmem) grow[0] = match[0];
    }
    __syncthreads();

    const int ncbmax = pitch >> 7;
    for (int t = 1; t < tl; t++) {
        // absolute coordinates, -inf outside the window
        const float *prev = rbuf + (size_t)(kRowsInSmem ? (t - 1) : ((t - 1) & 1)) * rp;
        float *cur = rbuf + (size_t)(kRowsInSmem ? t : (t & 1)) * rp;
        // live region: rows [t-1, t+W-2], columns [t, t+W-1]; work unit = 8 rows x 128 columns
        const int u_lo = (t - 1) >> 3, u_hi = (t + W - 2) >> 3;
        const int cb_lo = t >> 7;
        int cb_hi = (t + W - 1) >> 7;
        if (cb_hi > ncbmax - 1) cb_hi = ncbmax - 1;
        int total = 0;
        for (int cb = cb_lo; cb <= cb_hi; cb++) {
            int uf = 128 * cb - K; uf = uf > 0 ? (uf >> 3) : 0; uf = uf > u_lo ? uf : u_lo;
            int ul = 16 * cb + 15; ul = ul < u_hi ? ul : u_hi;
            total += ul >= uf ? ul - uf + 1 : 0;
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
            int uf = 128 * cb - K; uf = uf > 0 ? (uf >> 3) : 0; uf = uf > u_lo ? uf : u_lo;
            int ul = 16 * cb + 15; ul = ul < u_hi ? ul : u_hi;
            const int n = ul >= uf ? ul - uf + 1 : 0;
            const int from = my_lo > base ? my_lo - base : 0;
            const int to = my_hi < base + n ? my_hi - base : n;
            base += n;
            if (from >= to) continue;
            const int col = 128 * cb + 4 * lane;
            float bv[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll 2
            for (int q = from; q < to; q++) {
                const int i0 = 8 * (reverse ? (ul - q) : (uf + q));
                const float4 *ep = reinterpret_cast<const float4 *>(Lsq + (size_t)i0 * pitch + col);
                float4 e[8];
#pragma unroll
                for (int r = 0; r < 8; r++) e[r] = __ldg(ep + (size_t)r * (pitch >> 2));
                const float4 a0 = *reinterpret_cast<const float4 *>(prev + i0);
                const float4 a1 = *reinterpret_cast<const float4 *>(prev + i0 + 4);
                const float av[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
#pragma unroll
                for (int r = 0; r < 8; r += 2) {
                    bv[0] = max3(bv[0], __fadd_rn(av[r], e[r].x), __fadd_rn(av[r + 1], e[r + 1].x));
                    bv[1] = max3(bv[1], __fadd_rn(av[r], e[r].y), __fadd_rn(av[r + 1], e[r + 1].y));
                    bv[2] = max3(bv[2], __fadd_rn(av[r], e[r].z), __fadd_rn(av[r + 1], e[r + 1].z));
                    bv[3] = max3(bv[3], __fadd_rn(av[r], e[r].w), __fadd_rn(av[r + 1], e[r + 1].w));
                }
            }
#pragma unroll
            for (int k = 0; k < 4; k++)
                if (bv[k] > -INFINITY) atomicMax(skey + col + k, orderable(bv[k]));
        }
        __syncthreads();

        // finalisation: consume and clear every merge slot that may have been touched
        int fq = 0;
        for (int j = 128 * cb_lo + tid; j < 128 * (cb_hi + 1); j += kAlignThreads, fq++) {
            const unsigned key = skey[j];
            skey[j] = key_none;
            const int c = j - t;
            if (c >= 0 && c < W) {
                const float best = unorderable(key);
                const float mt = fq == 0 ? mp[0] : (fq == 1 ? mp[1] : __ldg(match + (size_t)t * L + j));
                float v = __fadd_rn(best, mt);
                if (!(v > -INFINITY)) v = -INFINITY;
                cur[j] = v;
                if (!kRowsInSmem) grow[(size_t)t * L + j] = v;
            }
        }
        if (!kRowsInSmem && tid == 0) {  // entries of the recycled row buffer that left the window
            cur[t - 1] = -INFINITY;
            if (t >= 2) cur[t - 2] = -INFINITY;
        }
        __syncthreads();
    }

    // backtrace (dag_best_alignment.cu:185-188).  At each step every thread re-evaluates one
    // candidate predecessor of the path vertex; the CTA keeps the largest (value, rank) key.
    const float score = rbuf[(size_t)(kRowsInSmem ? (tl - 1) : ((tl - 1) & 1)) * rp + (ol - 1)];
    if (tid == 0 && max_score) max_score[b] = score;
    if (!(score > -INFINITY)) {
        if (tid == 0 && status) atomicOr(status, DAT_STATUS_NO_PATH);
        return;
    }
    int pos = ol - 1;
    if (tid == 0) path[pos] = tl - 1;
    for (int t = tl - 1; t >= 1; t--) {
        int lo = pos - K; lo = lo > t - 1 ? lo : t - 1;
        int hi = t + W - 2; hi = hi < pos - 1 ? hi : pos - 1;
        unsigned long long key = 0ull;
        for (int i = lo + tid; i <= hi; i += kAlignThreads) {
            const float a = kRowsInSmem ? rbuf[(size_t)(t - 1) * rp + i] : grow[(size_t)(t - 1) * L + i];
            const float v = __fadd_rn(a, __ldg(Lsq + (size_t)i * pitch + pos));
            if (v > -INFINITY) {
                const unsigned long long kk = pack_key(v, tie_rank(pos - i, lg));
                key = kk > key ? kk : key;
            }
        }
        const unsigned long long win = cta_max_key(key, bt_key[t & 1], lane, warp);
        if (win == 0ull) break;                      // cannot happen on a finite path
        const int d = (int)((0xffffffffu - (unsigned)(win & 0xffffffffu)) & 0xfffffu);
        if (d <= 0 || d > pos) break;
        pos -= d;
        if (tid == 0) path[pos] = t - 1;
    }
}

// ---------------------------------------------------------------------------------------------
// Strip kernel.  The recursion only ever looks left (alpha[t][j] needs alpha[t-1][i], i < j), so the
// columns can be finished strip by strip, every target step of a strip before the next strip.
// A 32 x 32 block of the transition matrix is then used for ALL steps while it sits in the
// registers of one warp (lane = column, 32 rows per lane), and every transition is read from
// memory once per launch, straight from the band, instead of once per target step.
//
// Strips are 64 columns wide (two 32-column halves).  For strip S:
//   * blocks whose rows belong to an earlier strip have no dependency inside the strip: an item
//     (32 rows c, strip S, step t) is the maximum over the rows of alpha[t-1][32c+r] + link, for
//     both halves at once (64 registers of links per lane; the 32 row values come from shared
//     memory as broadcast loads, which is what bounds this kernel, so each loaded value feeds two
//     additions).  Items are dealt out to the 13 bulk warps in contiguous ranges and merged into
//     P[t][column] with a shared atomicMax.
//   * the three blocks on the diagonal depend on the strip's own previous step and are walked in
//     step order by three warps in a software pipeline, one named barrier per step:
//     warp 0 the triangular block of the left half (step t), warp 2 the square block from the
//     left half's rows to the right half's columns (step t, needs the left half at t-1), warp 1
//     the triangular block of the right half (step t-1, needs the square block at t-1).
// While the diagonal of strip S is walked, the bulk warps already do the items of strip S+1 whose
// rows lie in strips < S; the items whose rows are strip S follow in a short stage of their own.
// Two CTA barriers per strip instead of two per target step.
// ---------------------------------------------------------------------------------------------
constexpr int kStripDiagWarps = 3;

__device__ __forceinline__ void cp_async4(float *smem_dst, const float *gsrc) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void cp_async_wait_all() {
    asm volatile("cp.async.commit_group;\n\tcp.async.wait_group 0;" ::: "memory");
}
// barrier among the three diagonal warps only (also orders their shared-memory accesses)
__device__ __forceinline__ void diag_group_sync() {
    asm volatile("bar.sync 1, %0;" ::"n"(kStripDiagWarps * 32) : "memory");
}

// e[r] = link from vertex 32c+r to vertex 32h+lane (band entry d = j-i-1), -inf if it does not exist.
// Consecutive rows of one column lie K-1 floats apart in the band.  A block strictly left of the
// diagonal whose every transition exists (the common case) is read without masks.
__device__ __forceinline__ void strip_load_block(float (&e)[32], const float *__restrict__ links, int c,
                                                 int h, int lane, int K, int ol) {
    const int j = 32 * h + lane;
    const int d0 = j - 32 * c - 1;                         // band index in row 32c
    const bool full = h > c && 32 * (h - c) + 30 < K && 32 * h + 31 < ol;   // warp-uniform
    if (full) {
        const float *p = links + (size_t)(32 * c) * K + d0;
#pragma unroll
        for (int r = 0; r < 32; r++) e[r] = __ldg(p + (size_t)r * (K - 1));
    } else {
#pragma unroll
        for (int r = 0; r < 32; r++) {
            const int i = 32 * c + r, d = d0 - r;
            const bool ok = d >= 0 && d < K && j < ol;
            e[r] = ok ? __ldg(links + (size_t)i * K + d) : -INFINITY;
        }
    }
}

// max over the 32 rows of a block of arow[r] + e[r]; arow is read as broadcast 16-byte loads
__device__ __forceinline__ float strip_block_max(const float *arow, const float (&e)[32]) {
    float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
#pragma unroll
    for (int q = 0; q < 8; q += 2) {
        const float4 a = *reinterpret_cast<const float4 *>(arow + 4 * q);
        const float4 b = *reinterpret_cast<const float4 *>(arow + 4 * q + 4);
        float s0, s1, s2, s3, s4, s5, s6, s7;
        fadd2_rn(s0, s1, a.x, a.y, e[4 * q], e[4 * q + 1]);
        fadd2_rn(s2, s3, a.z, a.w, e[4 * q + 2], e[4 * q + 3]);
        fadd2_rn(s4, s5, b.x, b.y, e[4 * q + 4], e[4 * q + 5]);
        fadd2_rn(s6, s7, b.z, b.w, e[4 * q + 6], e[4 * q + 7]);
        m0 = max3(m0, s0, s1);
        m1 = max3(m1, s2, s3);
        m2 = max3(m2, s4, s5);
        m3 = max3(m3, s6, s7);
    }
    return fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
}

// the same for two blocks that share their rows (the two halves of a strip)
__device__ __forceinline__ void strip_block_max2(const float *arow, const float (&e0)[32],
                                                 const float (&e1)[32], float &r0, float &r1) {
    float m0 = -INFINITY, m1 = -INFINITY, n0 = -INFINITY, n1 = -INFINITY;
#pragma unroll
    for (int q = 0; q < 8; q++) {
        const float4 a = *reinterpret_cast<const float4 *>(arow + 4 * q);
        float s0, s1, s2, s3, u0, u1, u2, u3;
        fadd2_rn(s0, s1, a.x, a.y, e0[4 * q], e0[4 * q + 1]);
        fadd2_rn(s2, s3, a.z, a.w, e0[4 * q + 2], e0[4 * q + 3]);
        fadd2_rn(u0, u1, a.x, a.y, e1[4 * q], e1[4 * q + 1]);
        fadd2_rn(u2, u3, a.z, a.w, e1[4 * q + 2], e1[4 * q + 3]);
        m0 = max3(m0, s0, s1);
        m1 = max3(m1, s2, s3);
        n0 = max3(n0, u0, u1);
        n1 = max3(n1, u2, u3);
    }
    r0 = fmaxf(m0, m1);
    r1 = fmaxf(n0, n1);
}

// Items (32-row block c, step t) of strip S for c in [c_first, c_last]; bulk warp wb of kBulkWarps takes a
// contiguous share and merges its maxima into Pbuf[t][0..63].
template <int kBulkWarps>
__device__ __forceinline__ void strip_bulk(const float *__restrict__ links, const float *A, unsigned *Pbuf,
                                           int c_first, int c_last, int S, int wb, int lane, int K,
                                           int ol, int tl, int W, int rp) {
    int t0 = 64 * S - W + 1; t0 = t0 > 1 ? t0 : 1;
    int t1 = 64 * S + 63; t1 = t1 < tl - 1 ? t1 : tl - 1;
    int total = 0;
    for (int c = c_first; c <= c_last; c++) {
        int ta = 32 * c - W + 2; ta = ta > t0 ? ta : t0;
        int tb = 32 * c + 32; tb = tb < t1 ? tb : t1;
        total += tb >= ta ? tb - ta + 1 : 0;
    }
    const int lo = (wb * total) / kBulkWarps, hi = ((wb + 1) * total) / kBulkWarps;
    int base = 0;
    for (int c = c_first; c <= c_last; c++) {
        int ta = 32 * c - W + 2; ta = ta > t0 ? ta : t0;
        int tb = 32 * c + 32; tb = tb < t1 ? tb : t1;
        const int n = tb >= ta ? tb - ta + 1 : 0;
        const int from = lo > base ? lo - base : 0;
        const int to = hi < base + n ? hi - base : n;
        base += n;
        if (from >= to) continue;
        float e0[32], e1[32];
        strip_load_block(e0, links, c, 2 * S, lane, K, ol);
        strip_load_block(e1, links, c, 2 * S + 1, lane, K, ol);
#pragma unroll 2
        for (int q = from; q < to; q++) {
            const int t = ta + q;
            float m0, m1;
            strip_block_max2(A + (size_t)(t - 1) * rp + 32 * c, e0, e1, m0, m1);
            if (m0 > -INFINITY) atomicMax(Pbuf + t * 64 + lane, orderable(m0));
            if (m1 > -INFINITY) atomicMax(Pbuf + t * 64 + 32 + lane, orderable(m1));
        }
    }
}

// barrier among the first kWarps warps of the CTA (all of them: the sweep's warps)
template <int kWarps>
__device__ __forceinline__ void sweep_sync() {
    asm volatile("bar.sync 2, %0;" ::"n"(kWarps * 32) : "memory");
}

// The strip-ordered sweep of one sentence by warps 0 .. kWarps-1 of the CTA (3 diagonal warps, the others
// bulk): fills A[t][j] (absolute columns, -inf outside the window) for every step.
template <int kWarps>
__device__ __forceinline__ void align_strip_sweep(const float *__restrict__ match, const float *__restrict__ links,
                                                  float *A, unsigned *P, float *M, int ol, int tl, int W, int T,
                                                  int L, int K, int rp, int tid, int lane, int warp) {
    constexpr int kThreads = kWarps * 32, kBulk = kWarps - kStripDiagWarps;
    const unsigned key_none = orderable(-INFINITY);
    for (int x = tid; x < tl * rp; x += kThreads) A[x] = -INFINITY;
    for (int x = tid; x < 2 * T * 64; x += kThreads) P[x] = key_none;
    for (int x = tid; x < tl * 64; x += kThreads) {
        const int t = x >> 6, jj = x & 63;
        M[x] = jj < L ? match[(size_t)t * L + jj] : 0.f;
    }
    sweep_sync<kWarps>();
    if (tid == 0) A[0] = match[0];
    sweep_sync<kWarps>();

    const int nS = (ol + 63) >> 6;
    for (int S = 0; S < nS; S++) {
        unsigned *Pcur = P + (S & 1) * T * 64, *Pnext = P + ((S + 1) & 1) * T * 64;
        const float *Mcur = M + (S & 1) * T * 64;
        float *Mnext = M + ((S + 1) & 1) * T * 64;
        // ---- stage A: the items of strip S whose rows are strip S-1 (finished just now)
        for (int x = tid; x < tl * 64; x += kThreads) Pnext[x] = key_none;
        float ed[32];   // diagonal warps: their block, in flight across the barrier
        if (warp == 0) strip_load_block(ed, links, 2 * S, 2 * S, lane, K, ol);
        else if (warp == 1) strip_load_block(ed, links, 2 * S + 1, 2 * S + 1, lane, K, ol);
        else if (warp == 2) strip_load_block(ed, links, 2 * S, 2 * S + 1, lane, K, ol);
        else if (S >= 1)
            strip_bulk<kBulk>(links, A, Pcur, 2 * S - 2, 2 * S - 1, S, warp - kStripDiagWarps, lane, K, ol, tl, W, rp);
        sweep_sync<kWarps>();
        // ---- stage B: warps 0-2 walk the diagonal blocks of strip S; the others work ahead on strip S+1
        if (warp < kStripDiagWarps) {
            int t0 = 64 * S - W + 1; t0 = t0 > 1 ? t0 : 1;
            int t1 = 64 * S + 63; t1 = t1 < tl - 1 ? t1 : tl - 1;
            for (int tau = t0; tau <= t1 + 1; tau++) {
                if (warp == 0 && tau <= t1) {
                    const int t = tau, j = 64 * S + lane;
                    float best = strip_block_max(A + (size_t)(t - 1) * rp + 64 * S, ed);
                    best = fmaxf(best, unorderable(Pcur[t * 64 + lane]));
                    float v = __fadd_rn(best, Mcur[t * 64 + lane]);
                    if (!(v > -INFINITY) || j < t || j > t + W - 1) v = -INFINITY;
                    A[(size_t)t * rp + j] = v;
                } else if (warp == 2 && tau <= t1) {
                    const int t = tau;
                    const float m = strip_block_max(A + (size_t)(t - 1) * rp + 64 * S, ed);
                    // the bulk contributions to this strip are complete; only this warp writes here now
                    const unsigned o = orderable(m), p = Pcur[t * 64 + 32 + lane];
                    if (m > -INFINITY && o > p) Pcur[t * 64 + 32 + lane] = o;
                } else if (warp == 1 && tau > t0) {
                    const int t = tau - 1, j = 64 * S + 32 + lane;
                    float best = strip_block_max(A + (size_t)(t - 1) * rp + 64 * S + 32, ed);
                    best = fmaxf(best, unorderable(Pcur[t * 64 + 32 + lane]));
                    float v = __fadd_rn(best, Mcur[t * 64 + 32 + lane]);
                    if (!(v > -INFINITY) || j < t || j > t + W - 1) v = -INFINITY;
                    A[(size_t)t * rp + j] = v;
                }
                diag_group_sync();
            }
        } else if (S + 1 < nS) {
            for (int x = tid - 32 * kStripDiagWarps; x < tl * 64; x += kThreads - 32 * kStripDiagWarps) {
                const int t = x >> 6, jj = 64 * (S + 1) + (x & 63);
                if (jj < L) cp_async4(Mnext + x, match + (size_t)t * L + jj);
                else Mnext[x] = 0.f;
            }
            if (S >= 1) {
                int cmin = 2 * S + 1 - (K - 1) / 32;   // blocks further left hold no transition into strip S+1
                cmin = cmin > 0 ? cmin : 0;
                strip_bulk<kBulk>(links, A, Pnext, cmin, 2 * S - 1, S + 1, warp - kStripDiagWarps, lane, K, ol, tl, W, rp);
            }
            cp_async_wait_all();
        }
        sweep_sync<kWarps>();
    }
}

// The backtrace (dag_best_alignment.cu:185-188) by one warp.  At each step every lane re-evaluates its share of the
// candidate predecessors of the path vertex (the same additions as the sweep's, hence the same bits) and the warp
// keeps the largest (value, rank) key.  Sixteen candidates per lane are requested together, so a window of up to
// 512 vertices costs one round trip to the links in L2 per step.
// rows[t * pitch + j]: the finished rows, in global memory (kGlobalRows: written by other warps, read past L1) or
// in shared memory.
template <bool kGlobalRows>
__device__ __forceinline__ void warp_backtrace(const float *rows, int pitch, const float *__restrict__ links,
                                               int64_t *__restrict__ path, int ol, int tl, int K, int lg, int lane) {
    const int W = ol - tl + 1;
    int pos = ol - 1;
    if (lane == 0) path[pos] = tl - 1;
    for (int t = tl - 1; t >= 1; t--) {
        int lo = pos - K; lo = lo > t - 1 ? lo : t - 1;
        int hi = t + W - 2; hi = hi < pos - 1 ? hi : pos - 1;
        const float *arow = rows + (size_t)(t - 1) * pitch;
        unsigned long long key = 0ull;
        constexpr int kBtBatch = 16;
        for (int i0 = lo + lane; i0 <= hi; i0 += 32 * kBtBatch) {
            float a[kBtBatch], e[kBtBatch];
#pragma unroll
            for (int q = 0; q < kBtBatch; q++) {
                const int i = i0 + 32 * q;
                const bool ok = i <= hi;
                a[q] = ok ? (kGlobalRows ? __ldcg(arow + i) : arow[i]) : -INFINITY;
                e[q] = ok ? __ldg(links + (size_t)i * K + (pos - i - 1)) : -INFINITY;
            }
#pragma unroll
            for (int q = 0; q < kBtBatch; q++) {
                const float v = __fadd_rn(a[q], e[q]);
                if (v > -INFINITY) {
                    const unsigned long long kk = pack_key(v, tie_rank(pos - (i0 + 32 * q), lg));
                    key = kk > key ? kk : key;
                }
            }
        }
        const unsigned hi32 = (unsigned)(key >> 32);
        const unsigned mh = __reduce_max_sync(0xffffffffu, hi32);
        const unsigned ml = __reduce_max_sync(0xffffffffu, hi32 == mh ? (unsigned)key : 0u);
        if (mh == 0u && ml == 0u) break;             // cannot happen on a finite path
        const int d = (int)((0xffffffffu - ml) & 0xfffffu);
        if (d <= 0 || d > pos) break;
        pos -= d;
        if (lane == 0) path[pos] = t - 1;
    }
}

// One CTA per sentence: the sweep by all 16 warps, then the backtrace by all of them.
__global__ void __launch_bounds__(kAlignThreads, 1)
dag_align_strip_kernel(const float *__restrict__ match_all, const float *__restrict__ links_all,
                       const int64_t *__restrict__ output_length, const int64_t *__restrict__ target_length,
                       int64_t *__restrict__ path_out, float *__restrict__ max_score,
                       int32_t *__restrict__ status, int T, int L, int K, int lg, int rp) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __shared__ unsigned long long bt_key[2][kAlignWarps];
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
    const float *links = links_all + (size_t)b * L * K;
    float *A = reinterpret_cast<float *>(smem_raw);                    // [T][rp] rows, absolute columns
    unsigned *P = reinterpret_cast<unsigned *>(A + (size_t)T * rp);    // [2][T][64] merged maxima of a strip
    float *M = reinterpret_cast<float *>(P + 2 * T * 64);              // [2][T][64] match values of a strip
    align_strip_sweep<kAlignWarps>(match, links, A, P, M, ol, tl, W, T, L, K, rp, tid, lane, warp);

    const float score = A[(size_t)(tl - 1) * rp + (ol - 1)];
    if (tid == 0 && max_score) max_score[b] = score;
    if (!(score > -INFINITY)) {
        if (tid == 0 && status) atomicOr(status, DAT_STATUS_NO_PATH);
        return;
    }
    // the backtrace by the whole CTA: one candidate predecessor per thread and step, the CTA keeps the largest
    // (value, rank) key (quicker than warp_backtrace when nothing else runs on the SM: 0.5 against 0.8 us a step)
    int pos = ol - 1;
    if (tid == 0) path[pos] = tl - 1;
    for (int t = tl - 1; t >= 1; t--) {
        int lo = pos - K; lo = lo > t - 1 ? lo : t - 1;
        int hi = t + W - 2; hi = hi < pos - 1 ? hi : pos - 1;
        unsigned long long key = 0ull;
        for (int i = lo + tid; i <= hi; i += kAlignThreads) {
            const float v = __fadd_rn(A[(size_t)(t - 1) * rp + i], __ldg(links + (size_t)i * K + (pos - i - 1)));
            if (v > -INFINITY) {
                const unsigned long long kk = pack_key(v, tie_rank(pos - i, lg));
                key = kk > key ? kk : key;
            }
        }
        const unsigned long long win = cta_max_key(key, bt_key[t & 1], lane, warp);
        if (win == 0ull) break;                      // cannot happen on a finite path
        const int d = (int)((0xffffffffu - (unsigned)(win & 0xffffffffu)) & 0xfffffu);
        if (d <= 0 || d > pos) break;
        pos -= d;
        if (tid == 0) path[pos] = t - 1;
    }
}

// ---------------------------------------------------------------------------------------------
// Persistent form of the strip kernel for batches of more sentences than SMs.  The backtrace of a
// sentence is one chain of tl-1 dependent round trips to the links in L2 (the column of the path vertex is
// known only when the previous step is resolved) during which the SM does nothing else, about a fifth of
// the sentence's time.  Here a CTA stays on its SM and takes sentences from a counter, most expensive
// first; warps 0-14 sweep a sentence, copy its rows to the caller's workspace and go on to the next
// sentence, while warp 15 runs the backtrace of the one before from the workspace.  The two sides meet
// at two named barriers (rows handed over / backtrace finished), so the sweep is at most one sentence
// ahead; nothing spins.
// ---------------------------------------------------------------------------------------------
constexpr int kPersSweepWarps = kAlignWarps - 1;       // (a seventeenth warp would cap the registers at 96 per thread:
constexpr int kPersSweepThreads = 32 * kPersSweepWarps; //  five warps on one scheduler; the bulk warps need 128)
constexpr int kPersThreads = kPersSweepThreads + 32;   // + the backtrace warp

__device__ __forceinline__ void pers_bar_sync(int id) {
    asm volatile("bar.sync %0, %1;" ::"r"(id), "n"(kPersThreads) : "memory");
}
__device__ __forceinline__ void pers_bar_arrive(int id) {
    asm volatile("bar.arrive %0, %1;" ::"r"(id), "n"(kPersThreads) : "memory");
}
constexpr int kBarHandOver = 3, kBarBacktraced = 4;

// Sentences ranked by decreasing cost (tl-1) * W^2 and the work counter set to zero.  One CTA.
__global__ void __launch_bounds__(1024)
dag_align_order_kernel(const int64_t *__restrict__ output_length, const int64_t *__restrict__ target_length,
                       int *__restrict__ order, int *__restrict__ counter, int B, int T, int L) {
    extern __shared__ float align_cost_s[];
    if (threadIdx.x == 0) *counter = 0;
    for (int b = threadIdx.x; b < B; b += blockDim.x) {
        const long long ol = output_length[b], tl = target_length[b];
        float c = 0.f;
        if (lengths_valid(ol, tl, T, L)) {
            const float W = (float)(ol - tl + 1);
            c = (float)(tl - 1) * W * W;
        }
        align_cost_s[b] = c;
    }
    __syncthreads();
    for (int b = threadIdx.x; b < B; b += blockDim.x) {
        const float c = align_cost_s[b];
        int rank = 0;
        for (int o = 0; o < B; o++) {
            const float co = align_cost_s[o];
            rank += (co > c) || (co == c && o < b);
        }
        order[rank] = b;
    }
}

__global__ void __launch_bounds__(kPersThreads, 1)
dag_align_strip_persistent_kernel(const float *__restrict__ match_all, const float *__restrict__ links_all,
                                  const int64_t *__restrict__ output_length,
                                  const int64_t *__restrict__ target_length, const int *__restrict__ order,
                                  int *__restrict__ counter, int64_t *__restrict__ path_out,
                                  float *__restrict__ max_score, float *rows_ws, int32_t *__restrict__ status,
                                  int B, int T, int L, int K, int lg, int rp) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    __shared__ int mail[4];       // sentence handed to the backtrace warp (-1: no more), its lengths
    __shared__ int fetched[2];    // the counter's value, alternating slots
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;

    if (warp == kPersSweepWarps) {
        // ---- the backtrace warp (dag_best_alignment.cu:185-188): each lane re-evaluates its share of the candidate
        // predecessors of the path vertex; the warp keeps the largest (value, rank) key
        for (;;) {
            pers_bar_sync(kBarHandOver);
            const int b = mail[0], ol = mail[1], tl = mail[2];
            if (b < 0) break;
            const float *links = links_all + (size_t)b * L * K;
            const float *grow = rows_ws + (size_t)b * T * L;
            int64_t *path = path_out + (size_t)b * L;
            warp_backtrace<true>(grow, L, links, path, ol, tl, K, lg, lane);
            pers_bar_arrive(kBarBacktraced);
        }
        return;
    }

    // ---- the sweep warps
    float *A = reinterpret_cast<float *>(smem_raw);                    // [T][rp] rows, absolute columns
    unsigned *P = reinterpret_cast<unsigned *>(A + (size_t)T * rp);    // [2][T][64] merged maxima of a strip
    float *M = reinterpret_cast<float *>(P + 2 * T * 64);              // [2][T][64] match values of a strip
    int handed = 0;
    for (int round = 0;; round++) {
        if (tid == 0) fetched[round & 1] = atomicAdd(counter, 1);
        sweep_sync<kPersSweepWarps>();
        const int q = fetched[round & 1];
        if (q >= B) break;
        const int b = order ? order[q] : q;
        int64_t *path = path_out + (size_t)b * L;
        for (int j = tid; j < L; j += kPersSweepThreads) path[j] = -1;
        const long long oll = output_length[b], tll = target_length[b];
        if (!lengths_valid(oll, tll, T, L)) {
            if (tid == 0) {
                if (max_score) max_score[b] = -INFINITY;
                if (status) atomicOr(status, DAT_STATUS_BAD_LENGTH);
            }
            continue;
        }
        const int ol = (int)oll, tl = (int)tll;
        const int W = ol - tl + 1;
        const float *match = match_all + (size_t)b * T * L;
        const float *links = links_all + (size_t)b * L * K;
        align_strip_sweep<kPersSweepWarps>(match, links, A, P, M, ol, tl, W, T, L, K, rp, tid, lane, warp);
        const float score = A[(size_t)(tl - 1) * rp + (ol - 1)];
        if (tid == 0 && max_score) max_score[b] = score;
        if (!(score > -INFINITY)) {
            if (tid == 0 && status) atomicOr(status, DAT_STATUS_NO_PATH);
            sweep_sync<kPersSweepWarps>();   // everyone has read the score before the next sentence clears the rows
            continue;
        }
        // the rows the backtrace can ask for: steps 0 .. tl-2, the window of each
        float *grow = rows_ws + (size_t)b * T * L;
        for (int t = warp; t < tl - 1; t += kPersSweepWarps)
            for (int j = t + lane; j <= t + W - 1; j += 32) grow[(size_t)t * L + j] = A[(size_t)t * rp + j];
        __threadfence();
        if (handed) pers_bar_sync(kBarBacktraced);   // the backtrace warp is done with the sentence before
        if (tid == 0) {
            mail[0] = b;
            mail[1] = ol;
            mail[2] = tl;
        }
        __threadfence_block();
        pers_bar_arrive(kBarHandOver);
        handed = 1;
        sweep_sync<kPersSweepWarps>();   // (the rows are copied: the next sentence may clear them)
    }
    if (handed) pers_bar_sync(kBarBacktraced);
    if (tid == 0) mail[0] = -1;
    __threadfence_block();
    pers_bar_arrive(kBarHandOver);
}

}  // namespace dat

#include "dag_align_cluster.cuh"

namespace dat {

static inline size_t align_smem_bytes(int L, int nrows) {
    const int pitch = align_pitch(L);
    return ((size_t)pitch * 4 + (size_t)nrows * (pitch + 32) * 4 + 15) & ~(size_t)15;
}
static inline size_t align_rows_bytes(int B, int T, int L) {
    return (((size_t)B * T * L * sizeof(float)) + 255) & ~(size_t)255;
}
static inline size_t align_lsq_bytes(int B, int L) {
    return (((size_t)B * align_rows(L) * align_pitch(L) * sizeof(float)) + 255) & ~(size_t)255;
}

}  // namespace dat

extern "C" {

size_t dat_dag_best_alignment_workspace_bytes(int bsz, int tarlen, int prelen) {
    if (bsz <= 0 || tarlen <= 0 || prelen <= 0) return 0;
    // square copy of the links (tiled kernel only) + the rows (every kernel but the one-sentence-per-CTA strip
    // kernel) + the work counter and the order of the sentences (persistent strip kernel)
    return dat::align_lsq_bytes(bsz, prelen) + dat::align_rows_bytes(bsz, tarlen, prelen) +
           ((size_t)bsz + 64) * sizeof(int) + 512;
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
    float *rows_ws = reinterpret_cast<float *>(wbase + align_lsq_bytes(bsz, prelen));
    {
        // strip kernel: all rows plus the per-strip staging must fit in shared memory
        const int rp = (prelen + 63) & ~63;
        const size_t strip_smem = ((size_t)tarlen * rp + (size_t)4 * tarlen * 64) * sizeof(float);
        if (strip_smem + 512 <= (size_t)di.max_smem_optin && bsz > di.sm_count) {
            // more sentences than SMs: persistent CTAs, the backtrace of a sentence beside the sweep of the next
            int *counter = reinterpret_cast<int *>(wbase + align_lsq_bytes(bsz, prelen) +
                                                   align_rows_bytes(bsz, tarlen, prelen));
            int *order = counter + 64;
            const bool do_order = bsz <= 8192;
            if (do_order) {
                dag_align_order_kernel<<<1, 1024, (size_t)bsz * sizeof(float), st>>>(output_length, target_length, order,
                                                                                     counter, bsz, tarlen, prelen);
                if (int rc = check_launch("dat_dag_best_alignment(order)")) return rc;
            } else if (cudaMemsetAsync(counter, 0, sizeof(int), st) != cudaSuccess) {
                return check_launch("dat_dag_best_alignment(counter)");
            }
            if (cudaFuncSetAttribute(dag_align_strip_persistent_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     (int)strip_smem) != cudaSuccess)
                return check_launch("dat_dag_best_alignment(attr)");
            dag_align_strip_persistent_kernel<<<(unsigned)di.sm_count, kPersThreads, strip_smem, st>>>(
                match_all, links, output_length, target_length, do_order ? order : nullptr, counter, path, max_score,
                rows_ws, status, bsz, tarlen, prelen, translen, lg, rp);
            return check_launch("dat_dag_best_alignment");
        }
        if (strip_smem + 512 <= (size_t)di.max_smem_optin) {
            if (cudaFuncSetAttribute(dag_align_strip_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                     (int)strip_smem) != cudaSuccess)
                return check_launch("dat_dag_best_alignment(attr)");
            dag_align_strip_kernel<<<(unsigned)bsz, kAlignThreads, strip_smem, st>>>(
                match_all, links, output_length, target_length, path, max_score, status, tarlen, prelen,
                translen, lg, rp);
            return check_launch("dat_dag_best_alignment");
        }
    }
    {
        // rows that do not fit one SM: a cluster of 4, 8 or 16 CTAs per sentence, if the sentence's blocks of links
        // fit its registers and the device can co-schedule such a cluster
        int cl_ranks = 0;
        for (int r = 4; r <= kClMaxRanks && !cl_ranks; r *= 2)
            if (cluster_fits(prelen, r)) cl_ranks = r;
        const size_t csmem = align_cluster_smem_bytes(prelen);
        if (cl_ranks && csmem <= (size_t)di.max_smem_optin) {
            bool ok = true;
            if (csmem > 48 * 1024)
                ok = cudaFuncSetAttribute(dag_align_cluster_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          (int)csmem) == cudaSuccess;
            if (ok && cl_ranks > 8)
                ok = cudaFuncSetAttribute(dag_align_cluster_kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) ==
                     cudaSuccess;
            cudaLaunchConfig_t ccfg = {};
            cudaLaunchAttribute cattr[1];
            ccfg.gridDim = dim3((unsigned)bsz * (unsigned)cl_ranks);
            ccfg.blockDim = dim3(kClThreads);
            ccfg.dynamicSmemBytes = csmem;
            ccfg.stream = st;
            cattr[0].id = cudaLaunchAttributeClusterDimension;
            cattr[0].val.clusterDim.x = (unsigned)cl_ranks;
            cattr[0].val.clusterDim.y = 1;
            cattr[0].val.clusterDim.z = 1;
            ccfg.attrs = cattr;
            ccfg.numAttrs = 1;
            int nclusters = 0;
            if (ok) ok = cudaOccupancyMaxActiveClusters(&nclusters, dag_align_cluster_kernel, &ccfg) == cudaSuccess &&
                         nclusters >= 1;
            if (ok) {
                int *counter = reinterpret_cast<int *>(wbase + align_lsq_bytes(bsz, prelen) +
                                                       align_rows_bytes(bsz, tarlen, prelen));
                const int *order = nullptr;
                if (bsz > 1 && bsz <= 8192) {
                    dag_align_order_kernel<<<1, 1024, (size_t)bsz * sizeof(float), st>>>(output_length, target_length,
                                                                                         counter + 64, counter, bsz, tarlen,
                                                                                         prelen);
                    if (int rc = check_launch("dat_dag_best_alignment(order)")) return rc;
                    order = counter + 64;
                }
                if (cudaLaunchKernelEx(&ccfg, dag_align_cluster_kernel, match_all, links, output_length, target_length,
                                       order, path, max_score, rows_ws, status, tarlen, prelen, translen, lg) != cudaSuccess)
                    return check_launch("dat_dag_best_alignment(cluster)");
                return check_launch("dat_dag_best_alignment(cluster)");
            }
            cudaGetLastError();   // not an error of the call: the tiled kernel takes over
        }
    }
    {
        dim3 grid((rows + 7) / 8, bsz);
        dag_align_prep_kernel<<<grid, 256, 0, st>>>(links, output_length, target_length, lsq, tarlen,
                                                    prelen, translen, rows, pitch);
        if (int rc = check_launch("dat_dag_best_alignment(prep)")) return rc;
    }
    const size_t base = align_smem_bytes(prelen, 2);
    DAT_REQUIRE(base + 512 <= (size_t)di.max_smem_optin, DAT_ERR_UNSUPPORTED,
                "dat_dag_best_alignment: prelen=%d needs %zu bytes of shared memory", prelen, base);
    const size_t with_rows = align_smem_bytes(prelen, tarlen);
    if (with_rows + 512 <= (size_t)di.max_smem_optin) {  // 512: room for the kernel's static shared variables
        if (cudaFuncSetAttribute(dag_align_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)with_rows) != cudaSuccess)
            return check_launch("dat_dag_best_alignment(attr)");
        dag_align_kernel<true><<<(unsigned)bsz, kAlignThreads, with_rows, st>>>(
            match_all, lsq, output_length, target_length, path, max_score, nullptr, status, tarlen,
            prelen, translen, lg, rows, pitch);
    } else {
        if (cudaFuncSetAttribute(dag_align_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)base) != cudaSuccess)
            return check_launch("dat_dag_best_alignment(attr)");
        dag_align_kernel<false><<<(unsigned)bsz, kAlignThreads, base, st>>>(
            match_all, lsq, output_length, target_length, path, max_score, rows_ws, status, tarlen,
            prelen, translen, lg, rows, pitch);
    }
    return check_launch("dat_dag_best_alignment");
}

}  // extern "C"
