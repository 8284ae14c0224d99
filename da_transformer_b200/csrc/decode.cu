// Decode-side dynamic programmes over the SQUARE transition matrix (links[b,i,j] = log P(v_i -> v_j),
// -inf for j <= i), for sm_100a.  The training ops work on the band layout; decoding restores the
// square one first (restore_valid_links, fs_plugins/models/glat_decomposed_with_link.py:337-349).
//
//   dat_node_passing_prob: the probability that a path from vertex 0 passes through each vertex
//     (GlatDecomposedLink._analyze_graph, glat_decomposed_with_link.py:559-569).  The reference sums,
//     over path lengths s = 0..L-1, the probability of sitting on vertex j after exactly s
//     transitions (L-1 log-sum-exp products over the whole [L,L] matrix).  Edges only go left to
//     right, so that sum is the solution of the triangular system
//         pass[0] = 1,   pass[j] = sum_{i<j} pass[i] * exp(links[i][j]),
//     one sweep over the matrix.
//   dat_viterbi_decode: GlatDecomposedLink.inference_viterbi (glat_decomposed_with_link.py:720-777):
//     max-plus recursion over the number of emitted tokens with back-pointers, the length-normalised
//     choice of the best length, the back-trace and the collapse of repeated / pad tokens, all on the
//     device (the reference back-traces in Python lists on the host).  A step whose sums cannot be NaN (triangular
//     matrix without NaN or +inf, row without +inf or NaN) keeps its row's values instead of back-pointers; the
//     back-trace re-evaluates the candidates of the vertices on the path.
// One CTA per sentence; the matrix of a sentence (<= 4 MB) is served by L2 after its first read.  Graphs of up to
// 1024 vertices are decoded by a cluster per sentence with the matrix in its registers (viterbi_cluster_kernel);
// the one-CTA kernel then only takes the sentences whose matrix is not what decoding builds.
#include <climits>

#include "cluster_util.cuh"
#include "dat_common.cuh"

namespace dat {

constexpr int kDecThreads = 512;
constexpr int kDecWarps = kDecThreads / 32;

__global__ void __launch_bounds__(256)
node_pass_kernel(const float *__restrict__ links_all, float *__restrict__ pass_all, int L) {
    extern __shared__ float nsm[];
    float *pass = nsm;              // [Lp]
    float *part = nsm + ((L + 31) & ~31);   // [8][32]
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float *lk = links_all + (size_t)blockIdx.x * L * L;
    const int nblk = (L + 31) >> 5;
    for (int jb = 0; jb < nblk; jb++) {
        const int j = 32 * jb + lane;
        // what the finished vertices (i < 32 jb) send into this block of 32 columns
        float acc = 0.f;
        if (j < L)
            for (int i = warp; i < 32 * jb; i += 8) acc = fmaf(pass[i], ex2(__ldg(lk + (size_t)i * L + j) * kLog2e), acc);
        part[warp * 32 + lane] = acc;
        __syncthreads();
        if (warp == 0) {
            float v = 0.f;
#pragma unroll
            for (int w = 0; w < 8; w++) v += part[w * 32 + lane];
            if (jb == 0 && lane == 0) v = 1.f;
            // the block's own triangle, column by column: lane c receives pass[r] * E[r][c] from every r < c
            float e[32];
#pragma unroll
            for (int r = 0; r < 32; r++) {
                const int i = 32 * jb + r;
                e[r] = (r < lane && j < L) ? ex2(__ldg(lk + (size_t)i * L + j) * kLog2e) : 0.f;
            }
#pragma unroll
            for (int r = 0; r < 31; r++) {
                const float pr = __shfl_sync(0xffffffffu, v, r);   // final: every r' < r has been added
                v = fmaf(pr, e[r], v);
            }
            if (j < L) {
                pass[j] = v;
                pass_all[(size_t)blockIdx.x * L + j] = v;
            }
        }
        __syncthreads();
    }
}

// Candidate order of torch.max along a dimension: larger value first, then the smaller index.
__device__ __forceinline__ void vit_better(float &bv, int &bi, float v, int i) {
    if (v > bv || (v == bv && i < bi)) {
        bv = v;
        bi = i;
    }
}

__global__ void __launch_bounds__(kDecThreads)
viterbi_decode_kernel(const float *__restrict__ links_all, const float *__restrict__ logits_all,
                      const int64_t *__restrict__ tokens_all, const int64_t *__restrict__ output_length,
                      int32_t *__restrict__ trace_all, int64_t *__restrict__ out_tokens,
                      int64_t *__restrict__ out_length, int64_t *__restrict__ out_vertices,
                      float *__restrict__ out_score, int32_t *__restrict__ status,
                      const int *__restrict__ select, int L, int max_length, int joint, float beta, int64_t pad) {
    // select (optional): only the sentences with a non-zero word are decoded here (the cluster kernel has done the others)
    if (select != nullptr && select[blockIdx.x] == 0) return;
    extern __shared__ __align__(16) float vsm[];
    const int Lp = (L + 31) & ~31;
    float *a0 = vsm, *a1 = vsm + Lp;            // alpha of two consecutive steps
    float *lastcol = a1 + Lp;                    // links[j][ol-1]
    float *lg = lastcol + Lp;                    // token log-probabilities of the vertices
    float *part_v = lg + Lp;                     // [2][Lp] partial winners of a step's columns
    int *part_i = reinterpret_cast<int *>(part_v + 2 * Lp);
    unsigned char *step_plain = reinterpret_cast<unsigned char *>(part_i + 2 * Lp);   // [max_length] kind of a step
    __shared__ unsigned long long bt_slot[2][kDecWarps];
    __shared__ float red_v[kDecWarps];
    __shared__ int red_i[kDecWarps];
    __shared__ float best_score;
    __shared__ int best_len, best_vertex;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int b = blockIdx.x;
    const float *lk = links_all + (size_t)b * L * L;
    const float *logit = logits_all + (size_t)b * L;
    int32_t *trace = trace_all + (size_t)b * (max_length > 1 ? max_length - 1 : 1) * L;
    long long oll = output_length[b];
    if (oll < 1 || oll > L) {
        if (tid == 0) {
            if (status) atomicOr(status, DAT_STATUS_BAD_LENGTH);
            out_length[b] = 0;
            out_score[b] = -INFINITY;
        }
        for (int k = tid; k < max_length; k += kDecThreads) {
            out_tokens[(size_t)b * max_length + k] = pad;
            out_vertices[(size_t)b * max_length + k] = -1;
        }
        return;
    }
    const int last = (int)oll - 1;
    const float l0 = joint ? logit[0] : 0.f;
    for (int j = tid; j < L; j += kDecThreads) {
        lg[j] = logit[j];
        lastcol[j] = lk[(size_t)j * L + last];
        a0[j] = (lk[j] + l0) + logit[j];     // step 0: one transition out of vertex 0 (:727-732)
    }
    if (tid == 0) {
        best_score = -INFINITY;
        best_len = 0;
        best_vertex = 0;
    }
    // A transition matrix as decoding builds it has -inf on and below its diagonal; the recursion then
    // only needs the candidates i < j (checked once here: any other matrix takes all L candidates).
    bool dense = false, dirty = false;   // dirty: a NaN or +inf transition (a sum with it can be NaN)
    for (int i = warp; i < L; i += kDecWarps)
        for (int j = lane; j < L; j += 32) {
            const float e = __ldg(lk + (size_t)i * L + j);
            if (j <= i) dense |= !(e == -INFINITY);
            else dirty |= !(e < INFINITY);
        }
    const bool upper = !__syncthreads_or(dense);
    // A step is "plain" when the matrix is triangular and clean and the current row has no +inf or NaN: no sum can
    // be NaN then, torch.max is an ordinary maximum with the first index among equals, and the step keeps only the
    // VALUES of its row (in place of the back-pointers); the back-trace finds the predecessor of the one vertex per
    // step that lies on the path by re-evaluating its candidates (the same additions, the same bits).
    const bool clean = upper && !__syncthreads_or(dirty);
    for (int t = 0; t < max_length; t++) {
        const float *cur = (t & 1) ? a1 : a0;
        float *nxt = (t & 1) ? a0 : a1;
        // ---- score of stopping after t+1 tokens: max_j cur[j] + links[j][last], first maximum (:747-752)
        float sv = -INFINITY;
        int si = INT_MAX;
        bool odd = false;   // a +inf or NaN in the row (looked for in the same pass)
        for (int j = tid; j < L; j += kDecThreads) {
            const float v = cur[j] + lastcol[j];
            odd |= !(cur[j] < INFINITY);
            if (v != v) { sv = v; si = j < si ? j : si; }   // NaN counts as the maximum, like torch.max
            else if (!(sv != sv)) vit_better(sv, si, v, j);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, sv, o);
            const int oi = __shfl_xor_sync(0xffffffffu, si, o);
            if (ov != ov) { if (!(sv != sv) || oi < si) { sv = ov; si = oi; } }
            else if (!(sv != sv)) vit_better(sv, si, ov, oi);
        }
        if (lane == 0) { red_v[warp] = sv; red_i[warp] = si; }
        const bool any_odd = __syncthreads_or(odd);   // (also the barrier between the warps' results and their merge)
        if (tid == 0) {
            float v = red_v[0];
            int i = red_i[0];
            for (int w = 1; w < kDecWarps; w++) {
                const float ov = red_v[w];
                const int oi = red_i[w];
                if (ov != ov) { if (!(v != v) || oi < i) { v = ov; i = oi; } }
                else if (!(v != v)) vit_better(v, i, ov, oi);
            }
            if (i == INT_MAX) i = 0;
            const float sc = v / powf((float)(t + 1), beta);
            // first maximum over the lengths (:754)
            if (t == 0 || sc > best_score || (sc != sc && !(best_score != best_score))) {
                best_score = sc;
                best_len = t + 1;
                best_vertex = i;
            }
        }
        if (t + 1 == max_length) break;
        // ---- next step: nxt[j] = max_i cur[i] + links[i][j], first maximum (:737-742).  With an upper
        // triangular matrix the candidates i >= j are -inf + cur[i]: they never win, unless cur[i] is +inf or
        // NaN (the sum is NaN then, and torch.max returns the first NaN), so such a step takes all L.
        const bool tri = upper && !any_odd;
        const bool plain = tri && clean;
        if (tid == 0) step_plain[t] = plain ? 1 : 0;
        // The matrix is walked in 32 x 32 tiles (lane = destination j, 32 sources per tile, all of a tile's
        // loads in flight together, two tiles at a time).  Column block c has c + 1 tiles when the matrix is
        // triangular, so blocks c and nb-1-c form a pair of nb + 1 tiles, and the two warps of a warp pair
        // take half of a pair's tiles each: equal work for all 16 warps.  A column's candidates then come
        // from at most two warps, in index order; part_v / part_i hold the two partial winners.
        {
            const int nb = (L + 31) >> 5, npairs = (nb + 1) >> 1;
            const int wp = warp & (kDecWarps / 2 - 1), hf = warp / (kDecWarps / 2);
            for (int p = wp; p < npairs; p += kDecWarps / 2) {
                const int cbA = p, cbB = nb - 1 - p;
                const int nA = tri ? cbA + 1 : nb, nB = cbB != cbA ? (tri ? cbB + 1 : nb) : 0;
                const int tot = nA + nB, cut = (tot + 1) >> 1;
                const int q0 = hf ? cut : 0, q1 = hf ? tot : cut;
#pragma unroll 1
                for (int side = 0; side < 2; side++) {
                    const int cb = side ? cbB : cbA;
                    if (side && cbB == cbA) break;
                    int r0 = side ? q0 - nA : q0, r1 = side ? q1 - nA : q1;   // this warp's row blocks of cb
                    const int nside = side ? nB : nA;
                    r0 = r0 < 0 ? 0 : r0;
                    r1 = r1 > nside ? nside : r1;
                    const int j = 32 * cb + lane;
                    float bv = -INFINITY;
                    int bi = INT_MAX;
                    bool nan = false;
                    const float *col = lk + (j < L ? j : 0);
                    if (plain) {   // values only: an add and half a three-input maximum per candidate
                        for (int rb = r0; rb < r1; rb += 2) {
                            float v[64];
                            const bool two = rb + 1 < r1;
#pragma unroll
                            for (int u = 0; u < 32; u++) {
                                const int i = 32 * rb + u;
                                v[u] = (i < L && j < L && i < j) ? __ldg(col + (size_t)i * L) : -INFINITY;
                            }
#pragma unroll
                            for (int u = 0; u < 32; u++) {
                                const int i = 32 * (rb + 1) + u;
                                v[32 + u] = (two && i < L && j < L && i < j) ? __ldg(col + (size_t)i * L) : -INFINITY;
                            }
                            const float *crow = cur + 32 * rb;   // (the row buffer is padded to a multiple of 32 with
                            float m0 = -INFINITY, m1 = -INFINITY;   //  -inf and has 32 more floats behind it)
#pragma unroll
                            for (int q = 0; q < 16; q++) {
                                const float4 a = *reinterpret_cast<const float4 *>(crow + 4 * q);
                                float s0, s1, s2, s3;
                                fadd2_rn(s0, s1, a.x, a.y, v[4 * q], v[4 * q + 1]);
                                fadd2_rn(s2, s3, a.z, a.w, v[4 * q + 2], v[4 * q + 3]);
                                m0 = max3(m0, s0, s1);
                                m1 = max3(m1, s2, s3);
                            }
                            bv = max3(bv, m0, m1);
                        }
                        if (j < L) part_v[hf * Lp + j] = bv;
                        continue;
                    }
                    for (int rb = r0; rb < r1; rb += 2) {
                        float v[64];
                        const bool two = rb + 1 < r1;
#pragma unroll
                        for (int u = 0; u < 32; u++) {
                            const int i = 32 * rb + u;
                            v[u] = (i < L && j < L && (!tri || i < j)) ? __ldg(col + (size_t)i * L) : -INFINITY;
                        }
                        if (two) {
#pragma unroll
                            for (int u = 0; u < 32; u++) {
                                const int i = 32 * (rb + 1) + u;
                                v[32 + u] = (i < L && j < L && (!tri || i < j)) ? __ldg(col + (size_t)i * L) : -INFINITY;
                            }
                        }
                        const int nu = two ? 64 : 32;
#pragma unroll
                        for (int u = 0; u < 64; u++) {
                            if (u < nu) {
                                const int i = 32 * rb + u;
                                const float w = cur[i < L ? i : 0] + v[u];
                                if (w != w) { if (!nan) { nan = true; bv = w; bi = i; } }
                                else if (!nan && w > bv) { bv = w; bi = i; }
                            }
                        }
                    }
                    if (j < L) {
                        part_v[hf * Lp + j] = bv;
                        part_i[hf * Lp + j] = bi;
                    }
                }
            }
        }
        __syncthreads();
        if (plain) {
            float *rowvals = reinterpret_cast<float *>(trace + (size_t)t * L);
            for (int j = tid; j < L; j += kDecThreads) {
                const float bv = fmaxf(part_v[j], part_v[Lp + j]);
                rowvals[j] = cur[j];                 // what the back-trace needs of this step
                nxt[j] = joint ? bv + lg[j] : bv;
            }
            __syncthreads();
            continue;
        }
        for (int j = tid; j < L; j += kDecThreads) {
            float bv = part_v[j];
            int bi = part_i[j];
            const float ov = part_v[Lp + j];
            const int oi = part_i[Lp + j];
            // the second partial holds the later indices: it wins only with a strictly larger value, or with
            // the first NaN
            if (!(bv != bv) && (ov != ov || ov > bv)) { bv = ov; bi = oi; }
            if (bi == INT_MAX) bi = 0;          // every candidate is -inf: torch returns index 0
            trace[(size_t)t * L + j] = bi;
            nxt[j] = joint ? bv + lg[j] : bv;
        }
        __syncthreads();
    }
    __syncthreads();
    // ---- back-trace and token collapse by one thread (<= max_length steps; :757-771)
    const int len = best_len;
    int64_t *vert = out_vertices + (size_t)b * max_length;
    {
        // back-trace.  A step that kept back-pointers is one lookup; a plain step kept its row, and the predecessor
        // of vertex j is the first index of the maximum of row[i] + links[i][j] over all i (torch.max's order:
        // larger value, then smaller index; -0 and +0 are equal), found by the whole CTA.
        int j = best_vertex;
        for (int k = len - 1; k >= 0; k--) {
            if (tid == 0) vert[k] = j;
            if (k == 0) break;
            if (!step_plain[k - 1]) {
                j = trace[(size_t)(k - 1) * L + j];
                continue;
            }
            const float *rowvals = reinterpret_cast<const float *>(trace + (size_t)(k - 1) * L);
            unsigned long long key = 0ull;
            for (int i = tid; i < L; i += kDecThreads) {
                float w = rowvals[i] + __ldg(lk + (size_t)i * L + j);
                w += 0.0f;
                const unsigned u = __float_as_uint(w);
                const unsigned ord = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
                const unsigned long long kk = ((unsigned long long)ord << 32) | (0xffffffffu - (unsigned)i);
                key = kk > key ? kk : key;
            }
            const unsigned hi = (unsigned)(key >> 32);
            const unsigned mh = __reduce_max_sync(0xffffffffu, hi);
            const unsigned ml = __reduce_max_sync(0xffffffffu, hi == mh ? (unsigned)key : 0u);
            unsigned long long *slots = bt_slot[k & 1];
            if (lane == 0) slots[warp] = ((unsigned long long)mh << 32) | ml;
            __syncthreads();
            const unsigned long long kw = lane < kDecWarps ? slots[lane] : 0ull;
            const unsigned kh = (unsigned)(kw >> 32);
            const unsigned wh = __reduce_max_sync(0xffffffffu, kh);
            const unsigned wl = __reduce_max_sync(0xffffffffu, kh == wh ? (unsigned)kw : 0u);
            j = (int)(0xffffffffu - wl);
        }
    }
    __syncthreads();
    if (tid == 0) {
        int64_t *tok = out_tokens + (size_t)b * max_length;
        const int64_t *tokens = tokens_all + (size_t)b * L;
        for (int k = len; k < max_length; k++) vert[k] = -1;
        // walk from the end: a token is kept unless it is pad or equals the token that follows it;
        // the final token is always kept.  Kept tokens are written right-aligned, then shifted left.
        int64_t lastt = tokens[vert[len - 1]];
        int w = max_length - 1;
        tok[w--] = lastt;
        for (int k = len - 2; k >= 0; k--) {
            const int64_t now = tokens[vert[k]];
            if (now != pad && now != lastt) tok[w--] = now;
            lastt = now;
        }
        const int n = max_length - 1 - w;
        for (int k = 0; k < n; k++) tok[k] = tok[w + 1 + k];
        for (int k = n; k < max_length; k++) tok[k] = pad;
        out_length[b] = n;
        out_score[b] = best_score;
    }
}


// ---------------------------------------------------------------------------------------------
// Viterbi decoding of one sentence by a thread-block cluster.  The general kernel above reads the whole
// upper triangle of the matrix from L2 once per emitted token; here the triangle sits in the registers of a
// cluster of 4, 8 or 16 CTAs (32 x 32 blocks, lane = destination, up to three blocks per warp, destination
// blocks dealt to the CTAs in pairs of equal work: the layout of the training kernels for long sentences) and
// is read once per call.  A step: every warp takes the maximum over the 32 sources of each of its blocks
// (the current row lies in every CTA's shared memory), one warp per owned destination block merges them,
// adds the token score and hands the new 32 values to every CTA (st.async onto the receivers' transaction
// barriers) and to the workspace; every CTA waits for its own copy of the row.  Only VALUES are kept; the
// back-trace re-evaluates the candidates of the vertices on the path (first index of the maximum, like
// torch.max).  That is valid when no sum can be NaN: matrix -inf on and below the diagonal, no NaN or +inf
// above it, no +inf or NaN in any row.  The kernel checks all three while it runs and raises the sentence's
// word in `redo` otherwise; the general kernel then decodes that sentence again with torch's NaN rules.
// ---------------------------------------------------------------------------------------------
__host__ __device__ inline size_t viterbi_cluster_smem_bytes(int L) {
    const int Lp = (L + 31) & ~31;
    return (size_t)(3 * Lp + kClMaxBlocks * 32 + kClMaxDest * 32 + 2 * kClMaxBlocks + 2 * kClMaxDest) * sizeof(float) + 64;
}

__device__ __forceinline__ float vit_block_max(const float *arow, const float (&e)[32]) {
    float m0 = -INFINITY, m1 = -INFINITY, m2 = -INFINITY, m3 = -INFINITY;
#pragma unroll
    for (int q = 0; q < 8; q += 2) {
        const float4 a = *reinterpret_cast<const float4 *>(arow + 4 * q);
        const float4 c = *reinterpret_cast<const float4 *>(arow + 4 * q + 4);
        float s0, s1, s2, s3, s4, s5, s6, s7;
        fadd2_rn(s0, s1, a.x, a.y, e[4 * q], e[4 * q + 1]);
        fadd2_rn(s2, s3, a.z, a.w, e[4 * q + 2], e[4 * q + 3]);
        fadd2_rn(s4, s5, c.x, c.y, e[4 * q + 4], e[4 * q + 5]);
        fadd2_rn(s6, s7, c.z, c.w, e[4 * q + 6], e[4 * q + 7]);
        m0 = max3(m0, s0, s1);
        m1 = max3(m1, s2, s3);
        m2 = max3(m2, s4, s5);
        m3 = max3(m3, s6, s7);
    }
    return fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
}

__global__ void __launch_bounds__(kClThreads, 1)
viterbi_cluster_kernel(const float *__restrict__ links_all, const float *__restrict__ logits_all,
                       const int64_t *__restrict__ tokens_all, const int64_t *__restrict__ output_length,
                       float *rows_all, int *redo, int64_t *__restrict__ out_tokens,
                       int64_t *__restrict__ out_length, int64_t *__restrict__ out_vertices,
                       float *__restrict__ out_score, int32_t *__restrict__ status, int L, int max_length, int joint,
                       float beta, int64_t pad) {
    extern __shared__ __align__(16) float vcs[];
    __shared__ __align__(8) uint64_t rowbar[2];
    __shared__ int gaveup;
    __shared__ unsigned long long bt_slot[2][kClWarps];
    __shared__ float best_score;
    __shared__ int best_len, best_vertex;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    int nranks;
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(nranks));
    const int rank = (int)(blockIdx.x % nranks), b = (int)(blockIdx.x / nranks);
    const float *lk = links_all + (size_t)b * L * L;
    const float *logit = logits_all + (size_t)b * L;
    float *rows = rows_all + (size_t)b * (max_length > 1 ? max_length - 1 : 1) * L;
    const long long oll = output_length[b];
    if (oll < 1 || oll > L) {   // the same for every CTA of the cluster: nobody reaches a cluster barrier
        if (rank == 0) {
            if (tid == 0) {
                if (status) atomicOr(status, DAT_STATUS_BAD_LENGTH);
                out_length[b] = 0;
                out_score[b] = -INFINITY;
                redo[b] = 0;
            }
            for (int k = tid; k < max_length; k += kClThreads) {
                out_tokens[(size_t)b * max_length + k] = pad;
                out_vertices[(size_t)b * max_length + k] = -1;
            }
        }
        return;
    }
    const int last = (int)oll - 1;
    const int Lp = (L + 31) & ~31, nsub = Lp >> 5;
    float *row = vcs;                                   // [2][Lp] current / next row (-inf past L)
    float *lastcol = row + 2 * Lp;                      // [Lp] links[j][last] (used by the first CTA)
    float *slot = lastcol + Lp;                         // [kClMaxBlocks][32] maxima of this CTA's blocks
    float *lgs = slot + kClMaxBlocks * 32;              // [kClMaxDest][32] token scores of the owned destinations
    int *tab_c = reinterpret_cast<int *>(lgs + kClMaxDest * 32);
    int *tab_d = tab_c + kClMaxBlocks;
    int *dlist = tab_d + kClMaxBlocks;
    int *dbase = dlist + kClMaxDest;

    int nd = 0, nblk = 0;
    for (int p = rank; 2 * p < nsub; p += nranks) {
        for (int side = 0; side < 2; side++) {
            const int d = side ? nsub - 1 - p : p;
            if (side && d == p) break;
            if (tid == 0) {
                dlist[nd] = d;
                dbase[nd] = nblk;
                for (int c = 0; c <= d; c++) {
                    tab_c[nblk + c] = c;
                    tab_d[nblk + c] = d;
                }
            }
            nd++;
            nblk += d + 1;
        }
    }
    if (tid == 0) {
        cluster_mbar_init(&rowbar[0], 1);
        cluster_mbar_init(&rowbar[1], 1);
        gaveup = 0;
        best_score = -INFINITY;
        best_len = 0;
        best_vertex = 0;
        if (rank == 0) redo[b] = 0;
    }
    __syncthreads();

    // this warp's blocks, read once; anything but a finite number or -inf above the diagonal spoils the plain maximum
    bool bad = false;
    float eb[kClPerWarp][32];
    int kc[kClPerWarp], kd[kClPerWarp];
#pragma unroll
    for (int q = 0; q < kClPerWarp; q++) {
        const int k = warp + q * kClWarps;
        kc[q] = -1;
        kd[q] = -1;
        if (k < nblk) {
            kc[q] = tab_c[k];
            kd[q] = tab_d[k];
            const int j = 32 * kd[q] + lane;
#pragma unroll
            for (int r = 0; r < 32; r++) {
                const int i = 32 * kc[q] + r;
                float e = -INFINITY;
                if (i < L && j < L && i < j) {
                    e = __ldg(lk + (size_t)i * L + j);
                    bad |= !(e < INFINITY);
                }
                eb[q][r] = e;
            }
        }
    }
    // on and below the diagonal everything must be -inf (rows dealt to the CTAs and warps in turn)
    for (int i = rank * kClWarps + warp; i < L; i += nranks * kClWarps)
        for (int j = lane; j <= i; j += 32) bad |= !(__ldg(lk + (size_t)i * L + j) == -INFINITY);
    // step 0 (one transition out of vertex 0, :727-732): every CTA builds its own copy
    const float l0 = joint ? logit[0] : 0.f;
    for (int j = tid; j < Lp; j += kClThreads) {
        float v = -INFINITY, lc = -INFINITY;
        if (j < L) {
            v = (lk[j] + l0) + logit[j];
            lc = lk[(size_t)j * L + last];
            bad |= !(v < INFINITY);
            if (rank == 0 && max_length > 1) rows[j] = v;
        }
        row[j] = v;
        row[Lp + j] = -INFINITY;
        lastcol[j] = lc;
    }
    for (int x = tid; x < nd * 32; x += kClThreads) {
        const int u = 32 * dlist[x >> 5] + (x & 31);
        lgs[x] = u < L ? logit[u] : 0.f;
    }
    __syncthreads();
    cluster_barrier();   // every CTA is set up (and the sentence's word in `redo` is cleared) before anyone writes
    if (bad) atomicOr(redo + b, 1);

    const uint32_t row_bytes = (uint32_t)nsub * 128u;
    const int npairs = (nsub + 1) >> 1, nown = npairs < nranks ? npairs : nranks;
    // the score of stopping after t+1 tokens (:747-754) is followed by the last warp of the first CTA
    float bs_score = -INFINITY;
    int bs_len = 0, bs_vertex = 0;
    for (int t = 0; t < max_length && rank < nown; t++) {
        const float *cur = row + (t & 1) * Lp;
        float *nxt = row + ((t + 1) & 1) * Lp;
        if (rank == 0 && warp == kClWarps - 1) {
            float sv = -INFINITY;
            int si = INT_MAX;
            for (int j = lane; j < L; j += 32) vit_better(sv, si, cur[j] + lastcol[j], j);
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ov = __shfl_xor_sync(0xffffffffu, sv, o);
                const int oi = __shfl_xor_sync(0xffffffffu, si, o);
                vit_better(sv, si, ov, oi);
            }
            if (si == INT_MAX) si = 0;
            const float sc = sv / powf((float)(t + 1), beta);
            if (t == 0 || sc > bs_score) {   // first maximum over the lengths
                bs_score = sc;
                bs_len = t + 1;
                bs_vertex = si;
            }
        }
        if (t + 1 == max_length) break;
        uint64_t *bar = &rowbar[(t + 1) & 1];
        if (tid == 0) cluster_mbar_expect(bar, row_bytes);
#pragma unroll
        for (int q = 0; q < kClPerWarp; q++) {
            if (kc[q] < 0) continue;   // warp-uniform
            slot[(warp + q * kClWarps) * 32 + lane] = vit_block_max(cur + 32 * kc[q], eb[q]);
        }
        __syncthreads();
        if (gaveup) break;   // (set during a wait, read after the barrier every thread passes next: the same for all)
        if (warp < nd) {
            const int d = dlist[warp], base = dbase[warp], u = 32 * d + lane;
            float best = -INFINITY;
            for (int c = 0; c <= d; c++) best = fmaxf(best, slot[(base + c) * 32 + lane]);
            float v = joint ? best + lgs[warp * 32 + lane] : best;
            if (u >= L) v = -INFINITY;
            if (!(v < INFINITY)) atomicOr(redo + b, 1);   // +inf or NaN: the general kernel takes the sentence
            for (int r = 0; r < nown; r++)
                cluster_st_async_b32(cluster_map(nxt + u, r), __float_as_uint(v), cluster_map(bar, r));
            if (u < L && t + 1 < max_length - 1) rows[(size_t)(t + 1) * L + u] = v;
        }
        const int s = t + 1;   // (this step's barrier has been through (s + 1) / 2 - 1 phases before this one)
        if (!cluster_mbar_wait(bar, (uint32_t)((((s + 1) >> 1) + 1) & 1))) gaveup = 1;
    }
    if (rank == 0 && warp == kClWarps - 1 && lane == 0) {
        best_score = bs_score;
        best_len = bs_len;
        best_vertex = bs_vertex;
    }
    __syncthreads();
    if (gaveup && tid == 0) atomicOr(redo + b, 1);   // cannot happen
    __threadfence();
    cluster_barrier();   // every row is in the workspace; nobody leaves while a neighbour may still write here
    if (rank != 0) return;
    if (__ldcg(redo + b) != 0) return;   // the general kernel decodes this sentence

    const int len = best_len;
    int64_t *vert = out_vertices + (size_t)b * max_length;
    {
        int j = best_vertex;
        for (int k = len - 1; k >= 0; k--) {
            if (tid == 0) vert[k] = j;
            if (k == 0) break;
            const float *rowvals = rows + (size_t)(k - 1) * L;
            unsigned long long key = 0ull;
            for (int i = tid; i < L; i += kClThreads) {
                float w = __ldcg(rowvals + i) + __ldg(lk + (size_t)i * L + j);
                w += 0.0f;
                const unsigned u = __float_as_uint(w);
                const unsigned ord = (u & 0x80000000u) ? ~u : (u | 0x80000000u);
                const unsigned long long kk = ((unsigned long long)ord << 32) | (0xffffffffu - (unsigned)i);
                key = kk > key ? kk : key;
            }
            const unsigned hi = (unsigned)(key >> 32);
            const unsigned mh = __reduce_max_sync(0xffffffffu, hi);
            const unsigned ml = __reduce_max_sync(0xffffffffu, hi == mh ? (unsigned)key : 0u);
            unsigned long long *slots = bt_slot[k & 1];
            if (lane == 0) slots[warp] = ((unsigned long long)mh << 32) | ml;
            __syncthreads();
            const unsigned long long kw = lane < kClWarps ? slots[lane] : 0ull;
            const unsigned kh = (unsigned)(kw >> 32);
            const unsigned wh = __reduce_max_sync(0xffffffffu, kh);
            const unsigned wl = __reduce_max_sync(0xffffffffu, kh == wh ? (unsigned)kw : 0u);
            j = (int)(0xffffffffu - wl);
        }
    }
    __syncthreads();
    if (tid == 0) {
        int64_t *tok = out_tokens + (size_t)b * max_length;
        const int64_t *tokens = tokens_all + (size_t)b * L;
        for (int k = len; k < max_length; k++) vert[k] = -1;
        // (the collapse of repeated / pad tokens, as in the general kernel)
        int64_t lastt = tokens[vert[len - 1]];
        int w = max_length - 1;
        tok[w--] = lastt;
        for (int k = len - 2; k >= 0; k--) {
            const int64_t now = tokens[vert[k]];
            if (now != pad && now != lastt) tok[w--] = now;
            lastt = now;
        }
        const int n = max_length - 1 - w;
        for (int k = 0; k < n; k++) tok[k] = tok[w + 1 + k];
        for (int k = n; k < max_length; k++) tok[k] = pad;
        out_length[b] = n;
        out_score[b] = best_score;
    }
}

}  // namespace dat

extern "C" {

int dat_node_passing_prob(const float *links_square, float *node_pass, int bsz, int prelen, void *stream) {
    using namespace dat;
    DAT_REQUIRE(bsz >= 0 && prelen >= 1, DAT_ERR_BAD_ARG, "dat_node_passing_prob: bad sizes bsz=%d prelen=%d",
                bsz, prelen);
    if (bsz == 0) return DAT_OK;
    DAT_REQUIRE(links_square && node_pass, DAT_ERR_BAD_ARG, "dat_node_passing_prob: null pointer");
    DAT_REQUIRE(prelen <= 8192, DAT_ERR_UNSUPPORTED, "dat_node_passing_prob: prelen=%d exceeds 8192", prelen);
    const size_t smem = ((size_t)((prelen + 31) & ~31) + 8 * 32) * sizeof(float);
    node_pass_kernel<<<(unsigned)bsz, 256, smem, static_cast<cudaStream_t>(stream)>>>(links_square, node_pass,
                                                                                    prelen);
    return check_launch("dat_node_passing_prob");
}

size_t dat_viterbi_decode_workspace_bytes(int bsz, int prelen, int max_length) {
    if (bsz <= 0 || prelen <= 0 || max_length <= 0) return 0;
    // per sentence and step the back-pointers or the row's values, then one word per sentence (decoded by the
    // cluster kernel / left to the general kernel)
    return (size_t)bsz * (size_t)(max_length > 1 ? max_length - 1 : 1) * prelen * sizeof(int32_t) +
           ((size_t)bsz + 64) * sizeof(int);
}

int dat_viterbi_decode(const float *links_square, const float *unreduced_logits,
                       const int64_t *unreduced_tokens, const int64_t *output_length, void *workspace,
                       int64_t *out_tokens, int64_t *out_length, int64_t *out_vertices, float *out_score,
                       int32_t *status, int bsz, int prelen, int max_length, int joint, float beta,
                       int64_t pad_index, void *stream) {
    using namespace dat;
    const char *who = "dat_viterbi_decode";
    DAT_REQUIRE(bsz >= 0 && prelen >= 1 && max_length >= 1, DAT_ERR_BAD_ARG,
                "%s: bad sizes bsz=%d prelen=%d max_length=%d", who, bsz, prelen, max_length);
    if (bsz == 0) return DAT_OK;
    DAT_REQUIRE(links_square && unreduced_logits && unreduced_tokens && output_length && workspace &&
                    out_tokens && out_length && out_vertices && out_score,
                DAT_ERR_BAD_ARG, "%s: null pointer", who);
    DAT_REQUIRE(prelen <= 4096, DAT_ERR_UNSUPPORTED, "%s: prelen=%d exceeds 4096", who, prelen);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const size_t smem = (size_t)8 * ((prelen + 31) & ~31) * sizeof(float) + (((size_t)max_length + 15) & ~(size_t)15);
    if (smem > 48 * 1024 &&
        cudaFuncSetAttribute(viterbi_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
            cudaSuccess)
        return check_launch(who);
    // graphs of up to 1024 vertices: a cluster per sentence with the matrix in its registers; the general kernel
    // afterwards decodes only the sentences the cluster kernel left (matrices that are not clean and triangular)
    int *redo = reinterpret_cast<int *>(static_cast<char *>(workspace) +
                                        (size_t)bsz * (size_t)(max_length > 1 ? max_length - 1 : 1) * prelen * sizeof(int32_t));
    const int *select = nullptr;
    DeviceInfo di;
    if (!device_info(&di)) return DAT_ERR_NO_DEVICE;
    int cl_ranks = 0;
    for (int r = 4; r <= kClMaxRanks && !cl_ranks; r *= 2)
        if (cluster_fits(prelen, r)) cl_ranks = r;
    const size_t csmem = viterbi_cluster_smem_bytes(prelen);
    if (cl_ranks && csmem <= (size_t)di.max_smem_optin) {
        bool ok = true;
        if (csmem > 48 * 1024)
            ok = cudaFuncSetAttribute(viterbi_cluster_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)csmem) ==
                 cudaSuccess;
        if (ok && cl_ranks > 8)
            ok = cudaFuncSetAttribute(viterbi_cluster_kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) ==
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
        if (ok) ok = cudaOccupancyMaxActiveClusters(&nclusters, viterbi_cluster_kernel, &ccfg) == cudaSuccess &&
                     nclusters >= 1;
        if (ok) {
            if (cudaLaunchKernelEx(&ccfg, viterbi_cluster_kernel, links_square, unreduced_logits, unreduced_tokens,
                                   output_length, static_cast<float *>(workspace), redo, out_tokens, out_length,
                                   out_vertices, out_score, status, prelen, max_length, joint, beta,
                                   pad_index) != cudaSuccess)
                return check_launch("dat_viterbi_decode(cluster)");
            if (int rc = check_launch("dat_viterbi_decode(cluster)")) return rc;
            select = redo;
        } else {
            cudaGetLastError();   // not an error of the call: the general kernel decodes everything
        }
    }
    viterbi_decode_kernel<<<(unsigned)bsz, kDecThreads, smem, st>>>(
        links_square, unreduced_logits, unreduced_tokens, output_length, static_cast<int32_t *>(workspace),
        out_tokens, out_length, out_vertices, out_score, status, select, prelen, max_length, joint, beta, pad_index);
    return check_launch(who);
}

}  // extern "C"
