// Transition scores -> band links, forward and backward, for sm_100a.
//
// Replaces the tail of GlatDecomposedLink.extract_links
// (fs_plugins/models/glat_decomposed_with_link.py:380-404, with extract_valid_links :319-335):
// from the per-head scores  content[b,i,j,h]  (log_multi_content, [B,L,L,H] fp32) and the
// per-vertex head log-probabilities  log_gates[b,i,h]  it produces the band
//     links[b,i,d] = logsumexp_h( log_softmax_j(content[b,i,.,h])[j] + log_gates[b,i,h] ),  j = i+d+1,
// where the softmax runs over the valid successors of i inside the band (j in (i, i+K], j < L,
// column allowed by the mask); invalid entries and vertices without any successor are -inf.
// The reference materialises [B,L,K,H] three times on the way (gather, log_softmax, + gates).
// Here one warp owns one vertex (b,i) (head counts that are 4, 8, 16 or 32; a CTA per vertex with the
// scores staged in shared memory otherwise): it streams the H x (valid successors) scores, reduces per
// head, streams them again from L2 and writes the K band entries; nothing else touches HBM.
//
// HBM-bound.  Algorithmic bytes: forward reads the upper triangle of content once
// (~ B*L*L*H*4 / 2) and writes B*L*K*4; backward reads the same triangle plus the band gradient and
// writes the dense [B,L,L,H] gradient once (zeros included, like autograd's result).
#include "dat_common.cuh"

namespace dat {

constexpr int kLinksThreads = 128;   // 256 and 64 threads per vertex row were slower (0.25 / 0.26 against 0.22 ms forward)

struct LinksMask {
    const int64_t *bound_end;      // [B, L]: successors j <= bound_end[b,i] (decoding), or null
    const unsigned char *nonpad;   // [B, L]: successor j allowed iff nonpad[b,j] != 0 (training), or null
};

// first / last successor of vertex i inside the band and the graph: j in [i+1, jhi]
__device__ __forceinline__ int links_jhi(int i, int L, int K, const LinksMask &mk, int64_t row) {
    int jhi = i + K < L - 1 ? i + K : L - 1;
    if (mk.bound_end) {
        const int64_t be = mk.bound_end[row];
        jhi = be < jhi ? (int)be : jhi;
    }
    return jhi;
}

// Stages content[b,i,j,:] for j in [i+1, jhi] into sm[(j-i-1)*H + h]; masked columns become -inf.
__device__ __forceinline__ void links_stage_row(const float *__restrict__ crow, float *sm, int i, int jhi,
                                                int H, const unsigned char *np_row) {
    const int n = (jhi - i) * H;   // may be <= 0
    const float *src = crow + (size_t)(i + 1) * H;
    if ((H & 3) == 0) {
        const float4 *s4 = reinterpret_cast<const float4 *>(src);
        float4 *d4 = reinterpret_cast<float4 *>(sm);
        for (int x = threadIdx.x; x < n / 4; x += kLinksThreads) {
            float4 v = __ldg(s4 + x);
            if (np_row && !np_row[i + 1 + (4 * x) / H]) v = make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
            d4[x] = v;
        }
    } else {
        for (int x = threadIdx.x; x < n; x += kLinksThreads) {
            float v = __ldg(src + x);
            if (np_row && !np_row[i + 1 + x / H]) v = -INFINITY;
            sm[x] = v;
        }
    }
}

// Per-head log-sum-exp (natural log) over the staged successors.  Thread (h = tid % H, part = tid / H)
// walks the successors part, part + P, ...; partial (max, sum) pairs meet in shared memory.
// Result in lse_s[h] (-inf when the head sees no finite score).  Needs H <= kLinksThreads.
__device__ __forceinline__ void links_head_lse(const float *sm, int nj, int H, float *part_m, float *part_s,
                                               float *lse_s) {
    const int tid = threadIdx.x;
    const int P = kLinksThreads / H;
    const int h = tid % H, part = tid / H;
    float m = kNegBig, s = 0.f;
    if (part < P) {
        for (int j = part; j < nj; j += P) {
            const float v = sm[j * H + h] * kLog2e;
            if (v > m) {
                s *= ex2(m - v);
                m = v;
            }
            s += ex2(v - m);
        }
        part_m[part * H + h] = m;
        part_s[part * H + h] = s;
    }
    __syncthreads();
    if (tid < H) {
        float M = kNegBig, S = 0.f;
        for (int p = 0; p < P; p++) lse_merge(M, S, part_m[p * H + tid], part_s[p * H + tid]);
        lse_s[tid] = (S > 0.f && M > 0.5f * kNegBig) ? (M + lg2(S)) * kLn2 : -INFINITY;
    }
    __syncthreads();
}

__global__ void __launch_bounds__(kLinksThreads)
links_fwd_kernel(const float *__restrict__ content, const float *__restrict__ log_gates, LinksMask mk,
                 float *__restrict__ links, float *__restrict__ head_lse, int L, int H, int K) {
    extern __shared__ __align__(16) float lsm[];
    const int64_t row = blockIdx.x;          // b * L + i
    const int i = (int)(row % L);
    const int64_t b = row / L;
    const int tid = threadIdx.x;
    float *sm = lsm;                          // [(L-1) * H] staged scores
    float *part_m = sm + (size_t)(L - 1) * H; // [P * H]
    float *part_s = part_m + kLinksThreads;
    float *lse_s = part_s + kLinksThreads;    // [H]
    float *gate_s = lse_s + H;                // [H]
    const int jhi = links_jhi(i, L, K, mk, row);
    const int nj = jhi - i > 0 ? jhi - i : 0;
    const unsigned char *np_row = mk.nonpad ? mk.nonpad + b * L : nullptr;
    links_stage_row(content + row * (size_t)L * H, sm, i, jhi, H, np_row);
    if (tid < H) gate_s[tid] = log_gates[row * H + tid];
    __syncthreads();
    links_head_lse(sm, nj, H, part_m, part_s, lse_s);
    if (head_lse && tid < H) head_lse[row * H + tid] = lse_s[tid];
    // per head, what is added to a score: (gate - lse) in log2 units; a head whose every score is -inf
    // (lse = -inf) takes no part
    if (tid < H) gate_s[tid] = lse_s[tid] > -INFINITY ? (gate_s[tid] - lse_s[tid]) * kLog2e : -INFINITY;
    __syncthreads();
    float *out = links + row * (size_t)K;
    for (int d = tid; d < K; d += kLinksThreads) {
        float v = -INFINITY;
        if (d < nj) {
            // max over the heads first, then the sum: no rescaling and no branches inside the loops
            float m = -INFINITY;
            for (int h = 0; h < H; h++) m = fmaxf(m, fmaf(sm[d * H + h], kLog2e, gate_s[h]));
            if (m > -INFINITY) {
                float s = 0.f;
                for (int h = 0; h < H; h++) s += ex2(fmaf(sm[d * H + h], kLog2e, gate_s[h]) - m);
                v = (m + lg2(s)) * kLn2;
            }
        }
        out[d] = v;
    }
}

// Backward.  With z[j,h] = c[j,h] - lse_h + g_h, links[j] = logsumexp_h z[j,h], G[j] the incoming
// gradient and p[j,h] = exp(z[j,h] - links[j]):
//     S_h          = sum_j G[j] p[j,h]                          = d / d log_gates[h]
//     d / d c[j,h] = G[j] p[j,h] - exp(c[j,h] - lse_h) * S_h
// grad_content is written for the whole [L,H] row (zeros outside the valid successors); it may alias
// content (a CTA has its row in shared memory before it writes).
__global__ void __launch_bounds__(kLinksThreads)
links_bwd_kernel(const float *__restrict__ grad_links, const float *content,
                 const float *__restrict__ log_gates, const float *__restrict__ links,
                 const float *__restrict__ head_lse, LinksMask mk, float *grad_content,
                 float *__restrict__ grad_log_gates, int L, int H, int K) {
    extern __shared__ __align__(16) float lsm[];
    const int64_t row = blockIdx.x;
    const int i = (int)(row % L);
    const int64_t b = row / L;
    const int tid = threadIdx.x;
    float *sm = lsm;                           // [(L-1) * H]
    float *gl_s = sm + (size_t)(L - 1) * H;    // [L-1] incoming gradient per successor
    float *lk_s = gl_s + (L - 1);              // [L-1] forward value per successor
    float *part = lk_s + (L - 1);              // [kLinksThreads]
    float *lse_s = part + kLinksThreads;       // [H]
    float *gate_s = lse_s + H;                 // [H]
    float *S_s = gate_s + H;                   // [H]
    const int jhi = links_jhi(i, L, K, mk, row);
    const int nj = jhi - i > 0 ? jhi - i : 0;
    const unsigned char *np_row = mk.nonpad ? mk.nonpad + b * L : nullptr;
    links_stage_row(content + row * (size_t)L * H, sm, i, jhi, H, np_row);
    for (int d = tid; d < nj; d += kLinksThreads) {
        gl_s[d] = grad_links[row * (size_t)K + d];
        lk_s[d] = links[row * (size_t)K + d];
    }
    if (tid < H) {
        gate_s[tid] = log_gates[row * H + tid];
        lse_s[tid] = head_lse[row * H + tid];
    }
    __syncthreads();
    // S_h: thread (h, part) sums over its successors
    const int P = kLinksThreads / H;
    const int h = tid % H, pt = tid / H;
    float acc = 0.f;
    if (pt < P) {
        const float k = (gate_s[h] - lse_s[h]) * kLog2e;
        if (lse_s[h] > -INFINITY)
            for (int j = pt; j < nj; j += P) {
                const float lk = lk_s[j];
                if (lk > -INFINITY) acc += gl_s[j] * ex2(fmaf(sm[j * H + h], kLog2e, k) - lk * kLog2e);
            }
        part[pt * H + h] = acc;
    }
    __syncthreads();
    if (tid < H) {
        float S = 0.f;
        for (int p = 0; p < P; p++) S += part[p * H + tid];
        S_s[tid] = S;
        grad_log_gates[row * H + tid] = S;
    }
    __syncthreads();
    // the dense gradient row: zeros for j <= i and past the valid successors
    float *grow = grad_content + row * (size_t)L * H;
    const int total = L * H;
    for (int x = tid; x < total; x += kLinksThreads) {
        const int j = x / H, hh = x - j * H;
        float v = 0.f;
        const int d = j - i - 1;
        if (d >= 0 && d < nj) {
            const float c = sm[d * H + hh], lse = lse_s[hh], lk = lk_s[d];
            if (c > -INFINITY && lse > -INFINITY) {
                const float soft = ex2((c - lse) * kLog2e);
                float pg = 0.f;
                if (lk > -INFINITY) pg = gl_s[d] * ex2(((c - lse) + gate_s[hh] - lk) * kLog2e);
                v = pg - soft * S_s[hh];
            }
        }
        grow[x] = v;
    }
}

// ---------------------------------------------------------------------------------------------------
// One WARP per vertex row, no shared memory, no CTA barrier: the row's scores are streamed twice with
// 128-bit loads (the second pass hits L2: a row is at most a few KB), first for the per-head
// log-sum-exp (or, backward, the per-head sums S_h), then for the outputs.  A 16-byte vector holds four
// heads of one successor, and with H/4 a power of two a lane always meets the same four heads, so the
// per-head state lives in registers and is merged across the lanes by shuffles.  Used when H is a
// multiple of 4 with H/4 in {1, 2, 4, 8}; other head counts take the kernels above.  Rows are dealt so
// that the warps of a CTA alternate between long and short rows (vertex i and vertex L-1-i).
// ---------------------------------------------------------------------------------------------------
constexpr int kLwWarps = 4;
constexpr int kLwMaxGroups = 8;   // H / 4

__device__ __forceinline__ int links_row_of_slot(int q, int L) { return (q & 1) ? L - 1 - (q >> 1) : (q >> 1); }

template <int G>   // G = H / 4 vectors per successor
__global__ void __launch_bounds__(kLwWarps * 32)
links_fwd_warp_kernel(const float *__restrict__ content, const float *__restrict__ log_gates, LinksMask mk,
                      float *__restrict__ links, float *__restrict__ head_lse, int B, int L, int K) {
    constexpr int H = 4 * G;
    constexpr int U = 8;   // vectors a lane has in flight
    const int lane = threadIdx.x & 31;
    const int64_t slot = (int64_t)blockIdx.x * kLwWarps + (threadIdx.x >> 5);
    if (slot >= (int64_t)B * L) return;
    const int64_t b = slot / L;
    const int i = links_row_of_slot((int)(slot - b * L), L);
    const int64_t row = b * L + i;
    const int jhi = links_jhi(i, L, K, mk, row);
    const int nj = jhi - i > 0 ? jhi - i : 0;
    const unsigned char *np = mk.nonpad ? mk.nonpad + b * L + i + 1 : nullptr;
    const float4 *src = reinterpret_cast<const float4 *>(content + (row * L + i + 1) * (int64_t)H);
    const int nvec = nj * G;                      // vectors of the row
    const int g = lane & (G - 1);                 // this lane's head group: heads 4g .. 4g+3
    const float4 ninf = make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
    // ---- pass 1: per-head log-sum-exp over the successors (log2 units), U vectors requested at a time
    float m[4] = {kNegBig, kNegBig, kNegBig, kNegBig}, sum[4] = {0.f, 0.f, 0.f, 0.f};
    for (int v0 = lane; v0 < nvec; v0 += 32 * U) {
        float4 c4[U];
#pragma unroll
        for (int u = 0; u < U; u++) {
            const int v = v0 + 32 * u;
            c4[u] = (v < nvec && !(np && !np[v / G])) ? __ldg(src + v) : ninf;
        }
        // one new maximum per head and batch (one rescaling instead of one per element), then one ex2 per element
        float bm[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
        for (int u = 0; u < U; u++) {
            bm[0] = fmaxf(bm[0], c4[u].x);
            bm[1] = fmaxf(bm[1], c4[u].y);
            bm[2] = fmaxf(bm[2], c4[u].z);
            bm[3] = fmaxf(bm[3], c4[u].w);
        }
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const float b2 = bm[k] * kLog2e;
            if (b2 > m[k]) {
                sum[k] *= ex2(m[k] - b2);
                m[k] = b2;
            }
        }
#pragma unroll
        for (int u = 0; u < U; u++) {
            float t0 = -m[0], t1 = -m[1], t2 = -m[2], t3 = -m[3];
            ffma2_rn(t0, t1, c4[u].x, c4[u].y, kLog2e, kLog2e);
            ffma2_rn(t2, t3, c4[u].z, c4[u].w, kLog2e, kLog2e);
            fadd2_rn(sum[0], sum[1], sum[0], sum[1], ex2(t0), ex2(t1));
            fadd2_rn(sum[2], sum[3], sum[2], sum[3], ex2(t2), ex2(t3));
        }
    }
#pragma unroll
    for (int o = G; o < 32; o <<= 1) {   // lanes with the same head group
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const float m2 = __shfl_xor_sync(0xffffffffu, m[k], o), s2 = __shfl_xor_sync(0xffffffffu, sum[k], o);
            lse_merge(m[k], sum[k], m2, s2);
        }
    }
    // lse (natural log) and what a head adds to a score, (gate - lse) in log2 units (-inf: the head takes no part)
    float kh[4];
#pragma unroll
    for (int k = 0; k < 4; k++) {
        const float lse = (sum[k] > 0.f && m[k] > 0.5f * kNegBig) ? (m[k] + lg2(sum[k])) * kLn2 : -INFINITY;
        const int h = 4 * g + k;
        if (head_lse && lane < G) head_lse[row * H + h] = lse;
        kh[k] = lse > -INFINITY ? (__ldg(log_gates + row * H + h) - lse) * kLog2e : -INFINITY;
    }
    // every lane needs all heads' terms: head group gg from lane gg
    float ka[H];
#pragma unroll
    for (int gg = 0; gg < G; gg++) {
#pragma unroll
        for (int k = 0; k < 4; k++) ka[4 * gg + k] = __shfl_sync(0xffffffffu, kh[k], gg);
    }
    // ---- pass 2: links[d] = logsumexp_h(score[d][h] + gate_h - lse_h), one successor per lane and round,
    // U2 rounds requested at a time (the scores come from L2 now)
    constexpr int U2 = G >= 4 ? 2 : 4;
    float *out = links + row * (int64_t)K;
    for (int d0 = lane; d0 < K; d0 += 32 * U2) {
        float4 c4[U2][G];
#pragma unroll
        for (int u = 0; u < U2; u++) {
            const int d = d0 + 32 * u;
            const bool live = d < nj && !(np && !np[d]);
#pragma unroll
            for (int gg = 0; gg < G; gg++) c4[u][gg] = live ? __ldg(src + d * G + gg) : ninf;
        }
#pragma unroll
        for (int u = 0; u < U2; u++) {
            const int d = d0 + 32 * u;
            if (d >= K) break;
            if (d >= nj) {   // no such successor
                out[d] = -INFINITY;
                continue;
            }
            float z[H];
            float mx = -INFINITY;
#pragma unroll
            for (int gg = 0; gg < G; gg++) {
#pragma unroll
                for (int k = 0; k < 4; k++) z[4 * gg + k] = ka[4 * gg + k];
                ffma2_rn(z[4 * gg], z[4 * gg + 1], c4[u][gg].x, c4[u][gg].y, kLog2e, kLog2e);
                ffma2_rn(z[4 * gg + 2], z[4 * gg + 3], c4[u][gg].z, c4[u][gg].w, kLog2e, kLog2e);
                mx = max3(mx, z[4 * gg], z[4 * gg + 1]);
                mx = max3(mx, z[4 * gg + 2], z[4 * gg + 3]);
            }
            float v = -INFINITY;
            if (mx > -INFINITY) {
                float s0 = 0.f, s1 = 0.f;
#pragma unroll
                for (int k = 0; k < H; k += 2) {
                    float t0, t1;
                    fadd2_rn(t0, t1, z[k], z[k + 1], -mx, -mx);
                    fadd2_rn(s0, s1, s0, s1, ex2(t0), ex2(t1));
                }
                v = (mx + lg2(s0 + s1)) * kLn2;
            }
            out[d] = v;
        }
    }
}

// Backward, same layout of the work.  grad_content may alias content: a warp has finished reading its row
// for the sums before it writes, and every element is read by the lane that overwrites it.
template <int G>
__global__ void __launch_bounds__(kLwWarps * 32)
links_bwd_warp_kernel(const float *__restrict__ grad_links, const float *content, const float *__restrict__ log_gates,
                      const float *__restrict__ links, const float *__restrict__ head_lse, LinksMask mk,
                      float *grad_content, float *__restrict__ grad_log_gates, int B, int L, int K) {
    constexpr int H = 4 * G;
    constexpr int U = 4;   // vectors a lane has in flight
    const int lane = threadIdx.x & 31;
    const int64_t slot = (int64_t)blockIdx.x * kLwWarps + (threadIdx.x >> 5);
    if (slot >= (int64_t)B * L) return;
    const int64_t b = slot / L;
    const int i = links_row_of_slot((int)(slot - b * L), L);
    const int64_t row = b * L + i;
    const int jhi = links_jhi(i, L, K, mk, row);
    const int nj = jhi - i > 0 ? jhi - i : 0;
    const unsigned char *np = mk.nonpad ? mk.nonpad + b * L + i + 1 : nullptr;
    const float4 *src = reinterpret_cast<const float4 *>(content + (row * L + i + 1) * (int64_t)H);
    float4 *dst = reinterpret_cast<float4 *>(grad_content + (row * L + i + 1) * (int64_t)H);
    const float *gl = grad_links + row * (int64_t)K, *lk = links + row * (int64_t)K;
    const int nvec = nj * G;
    const int g = lane & (G - 1);
    const float4 ninf = make_float4(-INFINITY, -INFINITY, -INFINITY, -INFINITY);
    float lse2[4], kq[4];   // lse_h and (gate_h - lse_h), log2 units; -inf: the head takes no part
#pragma unroll
    for (int k = 0; k < 4; k++) {
        const float lse = __ldg(head_lse + row * H + 4 * g + k);
        lse2[k] = lse * kLog2e;
        kq[k] = lse > -INFINITY ? (__ldg(log_gates + row * H + 4 * g + k) - lse) * kLog2e : -INFINITY;
    }
    // ---- pass 1: S_h = sum_j G[j] p[j,h],  p[j,h] = exp(c[j,h] - lse_h + gate_h - links[j])
    float S[4] = {0.f, 0.f, 0.f, 0.f};
    for (int v0 = lane; v0 < nvec; v0 += 32 * U) {
        float4 c4[U];
        float l2[U], gd[U];
#pragma unroll
        for (int u = 0; u < U; u++) {
            const int v = v0 + 32 * u, d = v / G;
            const bool live = v < nvec && !(np && !np[d]);
            c4[u] = live ? __ldg(src + v) : ninf;
            l2[u] = live ? __ldg(lk + d) * kLog2e : -INFINITY;
            gd[u] = live ? __ldg(gl + d) : 0.f;
        }
#pragma unroll
        for (int u = 0; u < U; u++) {
            if (!(l2[u] > -INFINITY)) continue;
            // (a head that takes no part has kq = -inf: its term is ex2(-inf) = 0; two-lane arithmetic throughout)
            float t0, t1, t2, t3;
            fadd2_rn(t0, t1, kq[0], kq[1], -l2[u], -l2[u]);
            fadd2_rn(t2, t3, kq[2], kq[3], -l2[u], -l2[u]);
            ffma2_rn(t0, t1, c4[u].x, c4[u].y, kLog2e, kLog2e);
            ffma2_rn(t2, t3, c4[u].z, c4[u].w, kLog2e, kLog2e);
            ffma2_rn(S[0], S[1], ex2(t0), ex2(t1), gd[u], gd[u]);
            ffma2_rn(S[2], S[3], ex2(t2), ex2(t3), gd[u], gd[u]);
        }
    }
#pragma unroll
    for (int o = G; o < 32; o <<= 1) {
#pragma unroll
        for (int k = 0; k < 4; k++) S[k] += __shfl_xor_sync(0xffffffffu, S[k], o);
    }
    if (lane < G) {
#pragma unroll
        for (int k = 0; k < 4; k++) grad_log_gates[row * H + 4 * g + k] = S[k];
    }
    // ---- pass 2: d/dc[j,h] = G[j] p[j,h] - exp(c[j,h] - lse_h) S_h; zeros in the rest of the dense row
    float nl[4], nS[4];
#pragma unroll
    for (int k = 0; k < 4; k++) {
        nl[k] = kq[k] > -INFINITY ? -lse2[k] : -INFINITY;
        nS[k] = -S[k];
    }
    for (int v0 = lane; v0 < nvec; v0 += 32 * U) {
        float4 c4[U];
        float l2[U], gd[U];
        bool live[U];
#pragma unroll
        for (int u = 0; u < U; u++) {
            const int v = v0 + 32 * u, d = v / G;
            live[u] = v < nvec && !(np && !np[d]);
            c4[u] = live[u] ? src[v] : ninf;
            l2[u] = live[u] ? __ldg(lk + d) * kLog2e : -INFINITY;
            gd[u] = live[u] ? __ldg(gl + d) : 0.f;
        }
#pragma unroll
        for (int u = 0; u < U; u++) {
            const int v = v0 + 32 * u;
            if (v >= nvec) break;
            // soft = exp(c - lse_h) (0 for a masked score or a head that takes no part: nl = -inf there),
            // o = G p - soft S, in two-lane arithmetic
            float a0 = nl[0], a1 = nl[1], a2 = nl[2], a3 = nl[3];
            ffma2_rn(a0, a1, c4[u].x, c4[u].y, kLog2e, kLog2e);
            ffma2_rn(a2, a3, c4[u].z, c4[u].w, kLog2e, kLog2e);
            float o0 = 0.f, o1 = 0.f, o2 = 0.f, o3 = 0.f;
            if (l2[u] > -INFINITY) {
                float t0, t1, t2, t3;
                fadd2_rn(t0, t1, kq[0], kq[1], -l2[u], -l2[u]);
                fadd2_rn(t2, t3, kq[2], kq[3], -l2[u], -l2[u]);
                ffma2_rn(t0, t1, c4[u].x, c4[u].y, kLog2e, kLog2e);
                ffma2_rn(t2, t3, c4[u].z, c4[u].w, kLog2e, kLog2e);
                fmul2_rn(o0, o1, ex2(t0), ex2(t1), gd[u], gd[u]);
                fmul2_rn(o2, o3, ex2(t2), ex2(t3), gd[u], gd[u]);
            }
            ffma2_rn(o0, o1, ex2(a0), ex2(a1), nS[0], nS[1]);
            ffma2_rn(o2, o3, ex2(a2), ex2(a3), nS[2], nS[3]);
            dst[v] = make_float4(o0, o1, o2, o3);
        }
    }
    // the rest of the row: successors up to and including i, and those past jhi
    float4 *rowv = reinterpret_cast<float4 *>(grad_content + row * (int64_t)L * H);
    const int head = (i + 1) * G, tail0 = (i + 1 + nj) * G, total = L * G;
    for (int v = lane; v < head; v += 32) rowv[v] = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int v = tail0 + lane; v < total; v += 32) rowv[v] = make_float4(0.f, 0.f, 0.f, 0.f);
}

static bool links_warp_form(int H, const void *a, const void *b) {
    const int G = H / 4;
    return H % 4 == 0 && (G == 1 || G == 2 || G == 4 || G == 8) &&
           ((reinterpret_cast<uintptr_t>(a) | reinterpret_cast<uintptr_t>(b)) & 15) == 0;
}

static size_t links_smem_fwd(int L, int H) {
    return ((size_t)(L - 1) * H + 2 * kLinksThreads + 2 * H) * sizeof(float) + 16;
}
static size_t links_smem_bwd(int L, int H) {
    return ((size_t)(L - 1) * H + 2 * (size_t)(L - 1) + kLinksThreads + 3 * H) * sizeof(float) + 16;
}

}  // namespace dat

extern "C" {

int dat_links_from_heads(const float *content, const float *log_gates, const int64_t *bound_end,
                         const unsigned char *nonpad, float *links, float *head_lse, int bsz,
                         int prelen, int heads, int translen, void *stream) {
    using namespace dat;
    const char *who = "dat_links_from_heads";
    DAT_REQUIRE(bsz >= 0 && prelen >= 1 && heads >= 1 && translen >= 1, DAT_ERR_BAD_ARG,
                "%s: bad sizes bsz=%d prelen=%d heads=%d translen=%d", who, bsz, prelen, heads, translen);
    if (bsz == 0) return DAT_OK;
    DAT_REQUIRE(content && log_gates && links, DAT_ERR_BAD_ARG, "%s: null pointer", who);
    DAT_REQUIRE(heads <= kLinksThreads, DAT_ERR_UNSUPPORTED, "%s: heads=%d exceeds %d", who, heads,
                kLinksThreads);
    DeviceInfo di;
    if (!device_info(&di)) return DAT_ERR_NO_DEVICE;
    if (links_warp_form(heads, content, content)) {
        const LinksMask mkw{bound_end, nonpad};
        const int64_t rows = (int64_t)bsz * prelen;
        const unsigned grid = (unsigned)((rows + kLwWarps - 1) / kLwWarps);
        cudaStream_t st = static_cast<cudaStream_t>(stream);
        switch (heads / 4) {
            case 1: links_fwd_warp_kernel<1><<<grid, kLwWarps * 32, 0, st>>>(content, log_gates, mkw, links, head_lse, bsz, prelen, translen); break;
            case 2: links_fwd_warp_kernel<2><<<grid, kLwWarps * 32, 0, st>>>(content, log_gates, mkw, links, head_lse, bsz, prelen, translen); break;
            case 4: links_fwd_warp_kernel<4><<<grid, kLwWarps * 32, 0, st>>>(content, log_gates, mkw, links, head_lse, bsz, prelen, translen); break;
            default: links_fwd_warp_kernel<8><<<grid, kLwWarps * 32, 0, st>>>(content, log_gates, mkw, links, head_lse, bsz, prelen, translen); break;
        }
        return check_launch(who);
    }
    const size_t smem = links_smem_fwd(prelen, heads);
    DAT_REQUIRE(smem <= (size_t)di.max_smem_optin, DAT_ERR_UNSUPPORTED,
                "%s: prelen*heads = %d*%d needs %zu bytes of shared memory", who, prelen, heads, smem);
    if (smem > 48 * 1024 &&
        cudaFuncSetAttribute(links_fwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
            cudaSuccess)
        return check_launch(who);
    const LinksMask mk{bound_end, nonpad};
    links_fwd_kernel<<<(unsigned)((size_t)bsz * prelen), kLinksThreads, smem, static_cast<cudaStream_t>(stream)>>>(
        content, log_gates, mk, links, head_lse, prelen, heads, translen);
    return check_launch(who);
}

int dat_links_from_heads_backward(const float *grad_links, const float *content, const float *log_gates,
                                  const float *links, const float *head_lse, const int64_t *bound_end,
                                  const unsigned char *nonpad, float *grad_content,
                                  float *grad_log_gates, int bsz, int prelen, int heads, int translen,
                                  void *stream) {
    using namespace dat;
    const char *who = "dat_links_from_heads_backward";
    DAT_REQUIRE(bsz >= 0 && prelen >= 1 && heads >= 1 && translen >= 1, DAT_ERR_BAD_ARG,
                "%s: bad sizes bsz=%d prelen=%d heads=%d translen=%d", who, bsz, prelen, heads, translen);
    if (bsz == 0) return DAT_OK;
    DAT_REQUIRE(grad_links && content && log_gates && links && head_lse && grad_content && grad_log_gates,
                DAT_ERR_BAD_ARG, "%s: null pointer", who);
    DAT_REQUIRE(heads <= kLinksThreads, DAT_ERR_UNSUPPORTED, "%s: heads=%d exceeds %d", who, heads,
                kLinksThreads);
    DeviceInfo di;
    if (!device_info(&di)) return DAT_ERR_NO_DEVICE;
    if (links_warp_form(heads, content, grad_content)) {
        const LinksMask mkw{bound_end, nonpad};
        const int64_t rows = (int64_t)bsz * prelen;
        const unsigned grid = (unsigned)((rows + kLwWarps - 1) / kLwWarps);
        cudaStream_t st = static_cast<cudaStream_t>(stream);
#define DAT_LINKS_BWD(G_) links_bwd_warp_kernel<G_><<<grid, kLwWarps * 32, 0, st>>>(grad_links, content, log_gates, links, head_lse, mkw, grad_content, grad_log_gates, bsz, prelen, translen)
        switch (heads / 4) {
            case 1: DAT_LINKS_BWD(1); break;
            case 2: DAT_LINKS_BWD(2); break;
            case 4: DAT_LINKS_BWD(4); break;
            default: DAT_LINKS_BWD(8); break;
        }
#undef DAT_LINKS_BWD
        return check_launch(who);
    }
    const size_t smem = links_smem_bwd(prelen, heads);
    DAT_REQUIRE(smem <= (size_t)di.max_smem_optin, DAT_ERR_UNSUPPORTED,
                "%s: prelen*heads = %d*%d needs %zu bytes of shared memory", who, prelen, heads, smem);
    if (smem > 48 * 1024 &&
        cudaFuncSetAttribute(links_bwd_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem) !=
            cudaSuccess)
        return check_launch(who);
    const LinksMask mk{bound_end, nonpad};
    links_bwd_kernel<<<(unsigned)((size_t)bsz * prelen), kLinksThreads, smem, static_cast<cudaStream_t>(stream)>>>(
        grad_links, content, log_gates, links, head_lse, mk, grad_content, grad_log_gates, prelen, heads,
        translen);
    return check_launch(who);
}

}  // extern "C"
