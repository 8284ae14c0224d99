// dag_best_alignment for one sentence by a cluster of 4, 8 or 16 CTAs (included by dag_align.cu after the
// strip kernel, whose block loader, block maximum and backtrace helpers it uses).
//
// The strip kernel keeps every row of a sentence in one SM's shared memory; a sentence whose rows do not
// fit went to the tiled kernel, which reads a square copy of the links from L2 once per target step.  Here
// the upper triangle of the link matrix sits in the registers of a cluster instead (32 x 32 blocks, lane =
// destination vertex, 32 sources per lane, up to three blocks per warp; destination blocks d and nsub-1-d
// form a pair of equal work and the pairs are dealt to the CTAs in turn, as in the cluster sweep of
// dag_loss), so every link is read once per launch.  A step of the max-plus recursion
//     a_t[j] = match[t][j] + max_{i < j} (a_{t-1}[i] + links[i][j])
// has no dependency inside the step:
//   1. every warp takes the maximum over the 32 sources of each of its blocks (the previous row lies in
//      every CTA's shared memory) and leaves it in a slot;
//   2. (CTA barrier) one warp per owned destination block merges the slots, adds match, and stores the new
//      row segment into the next-row buffer of every CTA of the cluster through distributed shared memory
//      (st.async: the store counts its bytes on a transaction barrier in the destination CTA) and into the rows
//      workspace in global memory;
//   3. every CTA waits until the bytes of a whole row have arrived in its own buffer: no barrier among the CTAs,
//      no release fence on the senders.
// The additions are the reference's: one rounding per candidate (link + previous value) and one for the
// match value, and a maximum, so the rows are bit-identical to those of the other kernels.  The backtrace is
// the tiled kernel's, run by the cluster's first CTA on the rows workspace and the band itself.
#pragma once

#include "cluster_util.cuh"

namespace dat {

__host__ __device__ inline size_t align_cluster_smem_bytes(int prelen) {
    const int Lp = ((prelen + 31) / 32) * 32;
    return (size_t)(2 * Lp + kClMaxBlocks * 32 + kClMRing * kClMaxDest * 32 + 2 * kClMaxBlocks + 2 * kClMaxDest) *
               sizeof(float) + 64;
}

__global__ void __launch_bounds__(kClThreads, 1)
dag_align_cluster_kernel(const float *__restrict__ match_all, const float *__restrict__ links_all,
                         const int64_t *__restrict__ output_length, const int64_t *__restrict__ target_length,
                         const int *__restrict__ order, int64_t *__restrict__ path_out,
                         float *__restrict__ max_score, float *rows_ws, int32_t *__restrict__ status, int T, int L,
                         int K, int lg) {
    static_assert(kClThreads == kAlignThreads, "the backtrace's CTA-wide maximum assumes the alignment CTA size");
    extern __shared__ __align__(16) float acsm[];
    __shared__ unsigned long long bt_key[2][kAlignWarps];
    __shared__ __align__(8) uint64_t rowbar[2];   // transaction barriers of the rows of odd and even steps
    __shared__ int gaveup;                        // a wait for a row ran out (in rank 0: in any CTA of the cluster)
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    int nranks;
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(nranks));
    const int rank = (int)(blockIdx.x % nranks), cid = (int)(blockIdx.x / nranks);
    const int b = order ? order[cid] : cid;   // most expensive sentences first: the clusters run in waves
    int64_t *path = path_out + (size_t)b * L;
    if (rank == 0)
        for (int j = tid; j < L; j += kClThreads) path[j] = -1;
    const long long oll = output_length[b], tll = target_length[b];
    if (!lengths_valid(oll, tll, T, L)) {   // the same for every CTA of the cluster: nobody reaches a cluster barrier
        if (tid == 0 && rank == 0) {
            if (max_score) max_score[b] = -INFINITY;
            if (status) atomicOr(status, DAT_STATUS_BAD_LENGTH);
        }
        return;
    }
    const int ol = (int)oll, tl = (int)tll;
    const int W = ol - tl + 1;
    const int nsub = (ol + 31) >> 5, Lp = ((L + 31) >> 5) << 5;
    const float *match = match_all + (size_t)b * T * L;
    const float *links = links_all + (size_t)b * L * K;
    float *grow = rows_ws + (size_t)b * T * L;
    float *row = acsm;                                    // [2][Lp] previous / next row, -inf outside the window
    float *slot = row + 2 * Lp;                           // [kClMaxBlocks][32] maxima of this CTA's blocks
    float *M = slot + kClMaxBlocks * 32;                  // [kClMRing][kClMaxDest][32] match values
    int *tab_c = reinterpret_cast<int *>(M + kClMRing * kClMaxDest * 32);   // [kClMaxBlocks] source block of a slot
    int *tab_d = tab_c + kClMaxBlocks;                    // [kClMaxBlocks] destination block of a slot
    int *dlist = tab_d + kClMaxBlocks;                    // [kClMaxDest] owned destination blocks
    int *dbase = dlist + kClMaxDest;                      // [kClMaxDest] their first slot

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
    for (int x = tid; x < 2 * Lp; x += kClThreads) row[x] = -INFINITY;
    if (tid == 0) {
        cluster_mbar_init(&rowbar[0], 1);
        cluster_mbar_init(&rowbar[1], 1);
        gaveup = 0;
    }
    __syncthreads();

    // this warp's blocks of the link matrix, read once
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
            strip_load_block(eb[q], links, kc[q], kd[q], lane, K, ol);
        }
    }

    // match values of the owned destination blocks, half a ring of steps at a time
    const auto stage_match = [&](int t_first) {
        for (int x = tid; x < (kClMRing / 2) * nd * 32; x += kClThreads) {
            const int t = t_first + x / (nd * 32), rem = x % (nd * 32), q = rem >> 5, u = 32 * dlist[q] + (rem & 31);
            if (t >= tl) break;
            float *dst = M + ((t & (kClMRing - 1)) * kClMaxDest + q) * 32 + (rem & 31);
            if (u < ol) cp_async4(dst, match + (size_t)t * L + u);
            else *dst = -INFINITY;
        }
    };
    stage_match(0);
    stage_match(kClMRing / 2);
    asm volatile("cp.async.commit_group;" ::: "memory");

    // row 0: only vertex 0 is reachable
    if (tid == 0) {
        const float m0 = match[0];
        row[0] = m0;
        if (rank == 0) grow[0] = m0;
    }
    if (rank == 0)
        for (int j = 1 + tid; j < W; j += kClThreads) grow[j] = -INFINITY;
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();
    cluster_barrier();   // every CTA of the cluster is set up before anyone writes into its shared memory

    // Every destination block has one owner, and an owner sends all 32 values of a block to every CTA at every step:
    // a CTA receives nsub * 128 bytes per step.  Steps alternate between two barriers, so bytes of step t + 2 (whose
    // senders have seen this CTA's segments of step t + 1, hence this CTA past its wait for step t) never meet a
    // phase that is still open for step t.
    // Only the CTAs that own blocks take part (a short sentence in a long batch leaves some without): the others
    // have nothing to read or send, and nobody would wait for them.
    const uint32_t row_bytes = (uint32_t)nsub * 128u;
    const int npairs = (nsub + 1) >> 1, nown = npairs < nranks ? npairs : nranks;
    for (int t = 1; t < tl && rank < nown; t++) {
        const float *rowc = row + ((t - 1) & 1) * Lp;
        float *rown = row + (t & 1) * Lp;
        uint64_t *bar = &rowbar[t & 1];
        if (tid == 0) cluster_mbar_expect(bar, row_bytes);
        if ((t & (kClMRing / 2 - 1)) == 0) {   // match values half a ring ahead; the half before them has landed
            stage_match(t + kClMRing / 2);
            asm volatile("cp.async.commit_group;\n\tcp.async.wait_group 1;" ::: "memory");
        }
        // sources [t-1, t+W-2] can be finite, destinations [t, t+W-1] are wanted
        const int c_lo = (t - 1) >> 5, c_hi = (t + W - 2) >> 5;
        // ---- 1. maxima of this warp's blocks
#pragma unroll
        for (int q = 0; q < kClPerWarp; q++) {
            const int k = warp + q * kClWarps;
            if (kc[q] < 0) continue;   // warp-uniform
            const int c = kc[q], d = kd[q];
            const bool live = 32 * d + 31 >= t && 32 * d <= t + W - 1 && c >= c_lo && c <= c_hi;
            if (live) slot[k * 32 + lane] = strip_block_max(rowc + 32 * c, eb[q]);
        }
        __syncthreads();
        if (gaveup) break;   // (set during a wait, read after the barrier every thread passes next: the same for all)
        // ---- 2. the owned destination blocks, one warp each
        float o_v = -INFINITY;
        bool o_inside = false;
        int o_u = 0;
        if (warp < nd) {
            const int d = dlist[warp], base = dbase[warp], u = 32 * d + lane;
            const bool reach = 32 * d + 31 >= t && 32 * d <= t + W - 1;
            const bool inside = u >= t && u <= t + W - 1;
            float v = -INFINITY;
            if (reach) {
                float best = -INFINITY;
                const int ce = c_hi < d ? c_hi : d;
                for (int c = c_lo; c <= ce; c++) best = fmaxf(best, slot[(base + c) * 32 + lane]);
                v = __fadd_rn(best, M[((t & (kClMRing - 1)) * kClMaxDest + warp) * 32 + lane]);
                if (!(v > -INFINITY) || !inside) v = -INFINITY;
            }
            for (int r = 0; r < nown; r++)
                cluster_st_async_b32(cluster_map(rown + u, r), __float_as_uint(v), cluster_map(bar, r));
            o_v = v;
            o_inside = inside;
            o_u = u;
        }
        if (o_inside) grow[(size_t)t * L + o_u] = o_v;
        // ---- 3. the next row is complete here (every CTA waits for its own copy only)
        // (the barrier of this step's parity has been through (t + 1) / 2 - 1 phases before this one)
        if (!cluster_mbar_wait(bar, (uint32_t)((((t + 1) >> 1) + 1) & 1))) gaveup = 1;
    }
    __syncthreads();
    if (gaveup && tid == 0 && rank != 0) cluster_st_s32(cluster_map(&gaveup, 0), 1);
    __threadfence();
    cluster_barrier();   // every row is in the workspace; nobody leaves while a neighbour may still write here
    if (rank != 0) return;
    if (gaveup) {   // cannot happen: a wait for a row ran out somewhere in the cluster; the sentence gets no path
        if (tid == 0) {
            if (max_score) max_score[b] = -INFINITY;
            if (status) atomicOr(status, DAT_STATUS_NO_PATH);
        }
        return;
    }

    // backtrace (dag_best_alignment.cu:185-188): at each step every thread re-evaluates one candidate
    // predecessor of the path vertex; the CTA keeps the largest (value, rank) key
    const float score = row[((tl - 1) & 1) * Lp + (ol - 1)];
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
        for (int i = lo + tid; i <= hi; i += kClThreads) {
            const float v = __fadd_rn(__ldcg(grow + (size_t)(t - 1) * L + i), __ldg(links + (size_t)i * K + (pos - i - 1)));
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

}  // namespace dat
