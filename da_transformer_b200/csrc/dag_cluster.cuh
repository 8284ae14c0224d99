// dag_loss forward, probability-domain sweep of one sentence and direction by a cluster of 4, 8 or 16 CTAs
// (included by dag_fast.cu after dag_strip.cuh, whose block loaders and scaling helpers it uses).
//
// alpha_s[u] = exp(match_s[u]) * sum_{u' < u} alpha_{s-1}[u'] * E[u'][u] has no dependency inside a step:
// a step is one product of the previous row with the triangular matrix E = exp(links).  The strip sweep
// (dag_strip.cuh) orders the work by vertex group so that one SM can keep every block of E it needs in
// registers, at the price of a long chain of small steps.  Here the whole upper triangle of E sits in the
// registers of a CLUSTER instead: 32 x 32 blocks (lane = destination, 32 sources per lane), two or three per
// warp, 16 warps per CTA, as many CTAs as that takes; every link is still read and exponentiated once per sweep, and a
// sweep is tl - 1 steps instead of (tl + 3) per group of 128 vertices.  A step:
//   1. every warp multiplies the previous row's 32-vertex source segments with its blocks (the row lies in
//      every CTA's shared memory) and leaves each partial sum, with its magnitude, in a slot;
//   2. (CTA barrier) the destination blocks a CTA owns (blocks d and nsub-1-d form a pair of equal work,
//      pairs are dealt to the CTAs in turn, so all slots of a destination are in its owner's shared memory)
//      are finished by one warp each: the partial sums are added in a unit chosen from their magnitudes,
//      multiplied by exp(match), renormalised to one power-of-two exponent per 32 vertices, written to the
//      output (log2 value relative to a row offset known before the step) and to the next-row buffer of all
//      CTAs of the cluster through distributed shared memory (st.async: a store counts its bytes on a
//      transaction barrier in the destination CTA);
//   3. every CTA waits until the bytes of a whole row have arrived in its own buffers, then the next step: no
//      barrier among the CTAs, no release fence on the senders.
// Numerics and outputs are those of the strip sweep: fp32 mantissas with one exponent per sub-strip and step,
// units within 2^64 of the largest term, inputs below 2^-120 and holes reported through the sentence's
// flag word, log2 maxima per (step, sub-strip) and per step for dag_fast_check_kernel.  Nothing waits on a
// flag: the synchronisation is the hardware barrier of the CTA and the transaction barriers of the rows (bounded
// waits; a sentence whose wait ran out would go to the exact kernels).
// A step here costs about as much time as the strip sweep's four iterations for the same step and occupies
// several SMs, so on sentences whose rows fit in one SM's shared memory the strip sweep has twice the
// throughput (1.3 against 6.7 ms for 512 sentences of 512 vertices).  This kernel is for the sentences that
// do not fit: long graphs with many target steps, usually few per batch, where the alternative is the
// tiled sweep with its row-wide scaling (which such sentences fail) and then the exact kernels.
#pragma once

#include "cluster_util.cuh"

namespace dat {

struct ClusterSmem {
    float *row;      // [2][Lp]      mantissas of the previous / next row (every CTA holds the whole row)
    int *ex;         // [2][kClMaxSub] exponent of a sub-strip (kExpNone: all zero)
    float *mx;       // [2][2][kClMaxSub] log2 maxima of a sub-strip's entries, with and without exp(match)
    float *slot;     // [kClMaxBlocks][32] partial sums of this CTA's blocks
    int *slotmag;    // [kClMaxBlocks]  exponent of a partial sum's largest entry, in absolute terms (or kExpNone)
    float *M;        // [kClMRing][kClMaxDest][32] match values of the owned destination blocks
    int *tab_c, *tab_d;   // [kClMaxBlocks] source / destination block of a slot
    int *dlist, *dbase;   // [kClMaxDest] owned destination blocks and their first slot
};
__host__ __device__ inline size_t cluster_smem_bytes(int prelen) {
    const int Lp = ((prelen + 31) / 32) * 32;
    return (size_t)(2 * Lp + 2 * kClMaxSub + 4 * kClMaxSub + kClMaxBlocks * 32 + kClMaxBlocks +
                    kClMRing * kClMaxDest * 32 + 2 * kClMaxBlocks + 2 * kClMaxDest) * sizeof(float) + 64;
}

__global__ void __launch_bounds__(kClThreads, 1)
dag_cluster_sweep_kernel(const float *__restrict__ match_all, const float *__restrict__ links_all,
                         const int64_t *__restrict__ output_length, const int64_t *__restrict__ target_length,
                         const int *__restrict__ order, float *__restrict__ alpha_all, float *__restrict__ beta_all,
                         double *__restrict__ offsets_all, float *__restrict__ chk_all, float *__restrict__ sub_all,
                         int *__restrict__ flag, float *__restrict__ loss, int32_t *__restrict__ status, int T, int L,
                         int K, int nH) {
    extern __shared__ __align__(16) float csm[];
    __shared__ __align__(8) uint64_t rowbar[2];   // transaction barriers of the rows of odd and even steps
    __shared__ int gaveup;                        // a wait for a row ran out
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    int nranks;
    asm volatile("mov.u32 %0, %%cluster_nctarank;" : "=r"(nranks));
    const int rank = (int)(blockIdx.x % nranks), cid = (int)(blockIdx.x / nranks);
    const bool rev = cid & 1;   // odd clusters: the beta recursion (reversed graph)
    const int b = order ? order[cid >> 1] : (cid >> 1);
    const long long oll = output_length[b], tll = target_length[b];
    double *offs = offsets_all + (size_t)b * (2 * T + 2);
    if (!lengths_valid(oll, tll, T, L)) {   // the same for every CTA of the cluster: nobody reaches a cluster barrier
        if (tid == 0 && rank == 0) {
            offs[2 * T + (rev ? 1 : 0)] = -INFINITY;
            if (rev) loss[b] = -INFINITY;
            if (status) atomicOr(status, DAT_STATUS_BAD_LENGTH);
        }
        return;
    }
    const int ol = (int)oll, tl = (int)tll;
    const int W = ol - tl + 1;
    const int nsub = (ol + 31) >> 5, Lp = ((L + 31) >> 5) << 5;
    const float *match = match_all + (size_t)b * T * L;
    const float *links = links_all + (size_t)b * L * K;
    float *out = (rev ? beta_all : alpha_all) + (size_t)b * T * L;
    float *chk = chk_all + (size_t)b * 2 * T + (rev ? T : 0);
    float *sub = sub_all + ((size_t)b * 2 + (rev ? 1 : 0)) * T * nH;
    ClusterSmem sm;
    sm.row = csm;
    sm.ex = reinterpret_cast<int *>(sm.row + 2 * Lp);
    sm.mx = reinterpret_cast<float *>(sm.ex + 2 * kClMaxSub);
    sm.slot = sm.mx + 4 * kClMaxSub;
    sm.slotmag = reinterpret_cast<int *>(sm.slot + kClMaxBlocks * 32);
    sm.M = reinterpret_cast<float *>(sm.slotmag + kClMaxBlocks);
    sm.tab_c = reinterpret_cast<int *>(sm.M + kClMRing * kClMaxDest * 32);
    sm.tab_d = sm.tab_c + kClMaxBlocks;
    sm.dlist = sm.tab_d + kClMaxBlocks;
    sm.dbase = sm.dlist + kClMaxDest;

    // ---- this CTA's destination blocks and slots (the same arithmetic in every thread)
    int nd = 0, nblk = 0;
    for (int p = rank; 2 * p < nsub; p += nranks) {
        for (int side = 0; side < 2; side++) {
            const int d = side ? nsub - 1 - p : p;
            if (side && d == p) break;
            if (tid == 0) {
                sm.dlist[nd] = d;
                sm.dbase[nd] = nblk;
                for (int c = 0; c <= d; c++) {
                    sm.tab_c[nblk + c] = c;
                    sm.tab_d[nblk + c] = d;
                }
            }
            nd++;
            nblk += d + 1;
        }
    }
    for (int x = tid; x < 2 * Lp; x += kClThreads) sm.row[x] = 0.f;
    for (int x = tid; x < 2 * kClMaxSub; x += kClThreads) sm.ex[x] = kExpNone;
    for (int x = tid; x < 4 * kClMaxSub; x += kClThreads) sm.mx[x] = -INFINITY;
    if (tid == 0) {
        cluster_mbar_init(&rowbar[0], 1);
        cluster_mbar_init(&rowbar[1], 1);
        gaveup = 0;
    }
    __syncthreads();

    // ---- this warp's blocks of E, read and exponentiated once
    StripInputRange ir;
    ir.fin = INFINITY;
    ir.all = K < ol - 1 ? -INFINITY : INFINITY;   // a band narrower than the graph: vertex pairs without a link
    float eb[kClPerWarp][32];
    int kc[kClPerWarp], kd[kClPerWarp];
#pragma unroll
    for (int q = 0; q < kClPerWarp; q++) {
        const int k = warp + q * kClWarps;
        kc[q] = -1;
        kd[q] = -1;
        if (k < nblk) {
            kc[q] = sm.tab_c[k];
            kd[q] = sm.tab_d[k];
            strip_load_raw(eb[q], links, kc[q], kd[q], lane, K, ol, rev);
        }
    }
#pragma unroll
    for (int q = 0; q < kClPerWarp; q++)
        if (kc[q] >= 0) strip_exp_block(eb[q], kc[q], kd[q], lane, K, ol, ir);

    // match values of the owned destination blocks, kClMRing steps at a time
    const auto stage_match = [&](int s_first) {   // steps [s_first, s_first + kClMRing / 2)
        for (int x = tid; x < (kClMRing / 2) * nd * 32; x += kClThreads) {
            const int s = s_first + x / (nd * 32), rem = x % (nd * 32), q = rem >> 5, u = 32 * sm.dlist[q] + (rem & 31);
            if (s >= tl) break;
            float *dst = sm.M + ((s & (kClMRing - 1)) * kClMaxDest + q) * 32 + (rem & 31);
            if (u < ol)
                strip_cp_async4(dst, rev ? match + (size_t)(tl - 1 - s) * L + (ol - 1 - u) : match + (size_t)s * L + u);
            else *dst = -INFINITY;
        }
    };
    stage_match(0);
    stage_match(kClMRing / 2);
    asm volatile("cp.async.commit_group;" ::: "memory");

    // ---- step 0: only canonical vertex 0, value exp(match) = 2^m0; every CTA fills its own copy
    if (tid == 0) {
        const float m0 = (rev ? match[(size_t)(tl - 1) * L + (ol - 1)] : match[0]) * kLog2e;
        if (rank == 0) strip_note_finite(ir, m0);
        float y0 = 0.f;
        int e0 = kExpNone;
        if (m0 > -INFINITY && m0 < INFINITY) {
            const float fl = floorf(m0);
            y0 = ex2(m0 - fl);
            e0 = (int)fl;
        }
        sm.row[0] = y0;
        sm.ex[0] = e0;
        const float l0 = e0 != kExpNone ? lg2(y0) + (float)e0 : -INFINITY;
        sm.mx[0] = l0;                   // [buffer 0][with match][sub-strip 0]
        sm.mx[kClMaxSub] = l0;           // [buffer 0][without match][0] (step 0: the same)
        if (rank == 0) {
            const int t = rev ? tl - 1 : 0;
            const int off = e0 != kExpNone ? e0 : 0;
            offs[(rev ? T : 0) + t] = (double)off;
            out[(size_t)t * L + (rev ? ol - 1 : 0)] = e0 != kExpNone ? lg2(y0) + (float)(e0 - off) : -INFINITY;
            chk[t] = l0;
            for (int h = 0; h < nH; h++) sub[(size_t)t * nH + h] = h == 0 ? l0 : -INFINITY;
        }
    }
    if (rank == 0) {   // the rest of row 0's window: nothing there yet
        const int t = rev ? tl - 1 : 0, uhi = W - 1 < ol - 1 ? W - 1 : ol - 1;
        for (int u = 1 + tid; u <= uhi; u += kClThreads) out[(size_t)t * L + (rev ? ol - 1 - u : u)] = -INFINITY;
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();
    cluster_barrier();   // every CTA of the cluster is set up before anyone writes into its shared memory

    // Every destination block has one owner, which sends the block's 32 values and three words (exponent, two
    // maxima) to every CTA that takes part, at every step: nsub * 140 bytes per CTA and step, counted by a
    // transaction barrier of the receiving CTA; steps alternate between two barriers.  Only the CTAs that own blocks
    // take part (a short sentence in a long batch leaves some without).
    const uint32_t row_bytes = (uint32_t)nsub * 140u;
    const int npairs = (nsub + 1) >> 1, nown = npairs < nranks ? npairs : nranks;
    for (int s = 1; s < tl && rank < nown; s++) {
        const int cur = (s - 1) & 1, nxt = s & 1;
        const float *rowc = sm.row + cur * Lp;
        const int *exc = sm.ex + cur * kClMaxSub;
        uint64_t *bar = &rowbar[s & 1];
        if (tid == 0) cluster_mbar_expect(bar, row_bytes);
        if ((s & (kClMRing / 2 - 1)) == 0) {   // match values half a ring ahead; the half before them has landed
            stage_match(s + kClMRing / 2);
            asm volatile("cp.async.commit_group;\n\tcp.async.wait_group 1;" ::: "memory");
        }
        // the row offset of step s: the largest exponent of the previous row (the same in every CTA)
        const int offe = __reduce_max_sync(0xffffffffu, lane < nsub ? exc[lane] : kExpNone);
        // what the finished step left behind for the check: row maxima over the sub-strips (one step late)
        if (rank == 0 && warp == kClWarps - 1) {
            const int sp = s - 1, tp = rev ? tl - 1 - sp : sp;
            float ry = -INFINITY, rv = -INFINITY;
            for (int h = lane; h < nsub; h += 32) {
                ry = fmaxf(ry, sm.mx[(cur * 2 + 0) * kClMaxSub + h]);
                rv = fmaxf(rv, sm.mx[(cur * 2 + 1) * kClMaxSub + h]);
            }
            ry = warp_max(ry);
            rv = warp_max(rv);
            if (lane == 0 && sp > 0) chk[tp] = rev ? rv : ry;
        }
        // ---- 1. partial sums of this warp's blocks
#pragma unroll
        for (int q = 0; q < kClPerWarp; q++) {
            const int k = warp + q * kClWarps;
            if (kc[q] < 0) continue;   // warp-uniform
            const int c = kc[q], d = kd[q], ec = exc[c];
            // the destination block is reachable at step s: [32 d, 32 d + 31] meets [s, s + W - 1]
            const bool live = ec != kExpNone && 32 * d + 31 >= s && 32 * d <= s + W - 1;
            float p = 0.f;
            if (live) p = strip_block_dot(rowc + 32 * c, eb[q]);
            const unsigned pb = __reduce_max_sync(0xffffffffu, __float_as_uint(p));
            sm.slot[k * 32 + lane] = p;
            if (lane == 0) sm.slotmag[k] = (live && pb != 0u) ? exponent_of_bits(pb) + ec : kExpNone;
        }
        __syncthreads();
        if (gaveup) break;   // (set during a wait, read after the barrier every thread passes next: the same for all)
        // ---- 2. the owned destination blocks, one warp each
        float o_val = 0.f, o_hyv = 0.f;
        bool o_inside = false;
        int o_off = 0, o_d = 0;
        if (warp < nd) {
            const int d = sm.dlist[warp], base = sm.dbase[warp], u = 32 * d + lane;
            const bool reach = 32 * d + 31 >= s && 32 * d <= s + W - 1;
            // lane c looks at slot c (a sentence has at most 32 sub-strips): the largest magnitude decides the unit,
            // and every slot's scale 2^(exponent of its source - unit) is prepared as two exact factors
            // (scale2's rule) by its lane and handed round by shuffles
            const int mg = lane <= d ? sm.slotmag[base + lane] : kExpNone;
            const int est = __reduce_max_sync(0xffffffffu, mg);
            float y = 0.f, val = 0.f;
            int U = kExpNone;
            const bool inside = u >= s && u <= s + W - 1 && u < ol;
            if (est != kExpNone && reach) {
                U = est - kTargetExp;
                float f1 = 0.f, f2 = 0.f;
                if (mg != kExpNone) {
                    int k = exc[lane] - U;
                    if (k >= -252) {
                        k = k > 254 ? 254 : k;
                        const int k1 = (k >= -126 && k <= 127) ? k : k / 2;
                        f1 = __int_as_float((k1 + 127) << 23);
                        f2 = __int_as_float((k - k1 + 127) << 23);
                    }
                }
                for (int c = 0; c <= d; c++) {
                    const float g1 = __shfl_sync(0xffffffffu, f1, c), g2 = __shfl_sync(0xffffffffu, f2, c);
                    val += (sm.slot[(base + c) * 32 + lane] * g1) * g2;
                }
                const float m2 = sm.M[((s & (kClMRing - 1)) * kClMaxDest + warp) * 32 + lane] * kLog2e;
                ir.fin = fminf(ir.fin, (inside && m2 > -INFINITY) ? m2 : INFINITY);
                y = inside ? val * ex2(m2) : 0.f;
            }
            const unsigned yb = __reduce_max_sync(0xffffffffu, __float_as_uint(y));
            const unsigned vb = __reduce_max_sync(0xffffffffu, __float_as_uint(inside ? val : 0.f));
            // renormalise: the block's largest entry back to about 2^kTargetExp
            int e = kExpNone;
            if (yb != 0u && U != kExpNone && yb < 0x7f800000u) {
                const int sh = kTargetExp - exponent_of_bits(yb);
                y = scale2(y, sh);
                e = U - sh;
            } else if (yb >= 0x7f800000u) {
                e = U;   // inf / NaN from bad inputs: carried along, the check rejects the sentence
            }
            const float hy = e != kExpNone ? lg2(__uint_as_float(yb)) + (float)U : -INFINITY;
            const float hv = (vb != 0u && U != kExpNone) ? lg2(__uint_as_float(vb)) + (float)U : -INFINITY;
            // next row, exponent and maxima into every CTA of the cluster
            float *rown = sm.row + nxt * Lp + u;
            // (lanes 0, 1, 2 carry the block's exponent and its two maxima: one store per CTA for the three)
            const void *meta = lane == 0 ? (const void *)(sm.ex + nxt * kClMaxSub + d)
                             : lane == 1 ? (const void *)(sm.mx + (nxt * 2 + 0) * kClMaxSub + d)
                                         : (const void *)(sm.mx + (nxt * 2 + 1) * kClMaxSub + d);
            const int metav = lane == 0 ? e : lane == 1 ? __float_as_int(hy) : __float_as_int(hv);
            for (int r = 0; r < nown; r++) {
                const uint32_t rbar = cluster_map(bar, r);
                cluster_st_async_b32(cluster_map(rown, r), __float_as_uint(y), rbar);
                if (lane < 3) cluster_st_async_b32(cluster_map(meta, r), (uint32_t)metav, rbar);
            }
            // the output row: log2 values relative to the row offset
            o_off = offe != kExpNone ? offe : 0;
            o_val = (y > 0.f || y != y) ? lg2(y) + (float)(e - o_off) : -INFINITY;
            o_inside = inside;
            o_hyv = rev ? hv : hy;
            o_d = d;
        }
        if (warp < nd) {
            const int t = rev ? tl - 1 - s : s, u = 32 * o_d + lane;
            if (o_inside) out[(size_t)t * L + (rev ? ol - 1 - u : u)] = o_val;
            if (lane == 0) {
                sub[(size_t)t * nH + o_d] = o_hyv;
                if (o_d == 0) offs[(rev ? T : 0) + t] = (double)o_off;   // (block 0 belongs to rank 0)
            }
        }
        // ---- 3. the next row is complete here (every CTA waits for its own copy only)
        if (!cluster_mbar_wait(bar, (uint32_t)((((s + 1) >> 1) + 1) & 1))) gaveup = 1;
    }
    __syncthreads();
    if (gaveup && tid == 0) atomicOr(flag + b, kFlagTiny);   // cannot happen; the exact kernels take the sentence
    // ---- the last step's maxima, the sub-strips nobody owns, the likelihood
    {
        const int last = (tl - 1) & 1;
        if (rank == 0 && warp == kClWarps - 1 && tl > 1) {
            const int tp = rev ? 0 : tl - 1;
            float ry = -INFINITY, rv = -INFINITY;
            for (int h = lane; h < nsub; h += 32) {
                ry = fmaxf(ry, sm.mx[(last * 2 + 0) * kClMaxSub + h]);
                rv = fmaxf(rv, sm.mx[(last * 2 + 1) * kClMaxSub + h]);
            }
            ry = warp_max(ry);
            rv = warp_max(rv);
            if (lane == 0) chk[tp] = rev ? rv : ry;
        }
        if (rank == 0)
            for (int x = tid; x < (tl - 1) * (nH - nsub); x += kClThreads) {   // columns of sub past the graph
                const int s = 1 + x / (nH - nsub), h = nsub + x % (nH - nsub);
                sub[(size_t)(rev ? tl - 1 - s : s) * nH + h] = -INFINITY;
            }
        if (rank == 0 && tid == 0) {
            const float y = sm.row[last * Lp + (ol - 1)];
            const int e = sm.ex[last * kClMaxSub + ((ol - 1) >> 5)];
            const double z2 = (y > 0.f && e != kExpNone) ? (double)lg2(y) + (double)e : (y != y ? (double)y : -INFINITY);
            offs[2 * T + (rev ? 1 : 0)] = z2;
            if (rev) loss[b] = (float)(z2 * kLn2d);
        }
    }
    if (ir.fin < kMinLog2Input) atomicOr(flag + b, kFlagTiny);
    if (ir.all == -INFINITY) atomicOr(flag + b, kFlagHole);
    cluster_barrier();   // nobody leaves while a neighbour may still write into its shared memory
}

}  // namespace dat
