// dag_loss forward, strip-ordered probability-domain sweep (included by dag_fast.cu).
//
// Both recursions only ever look one way: alpha[t][j] needs alpha[t-1][i] with i < j, and beta is
// the same recursion on the reversed graph (vertex u = ol-1-i, step s = tl-1-t).  So a sweep can
// finish its vertices group by group, every target step of a group before the next group, and a
// 32 x 32 block of E = exp(links) then serves ALL steps while it sits in the registers of one warp
// (lane = destination vertex, 32 source vertices per lane).  Every link is read, and
// exponentiated, once per sweep, straight from the band: no square copy, no re-read per step.
//
// One CTA per (sentence, direction).  In canonical coordinates (u, s) the row of step s is
// y[s][u] * 2^sc[s][u/32]: fp32 mantissas with one power-of-two exponent per 32-vertex sub-strip,
// all rows resident in shared memory.  Vertices are taken in groups of four sub-strips (128):
//   phase 1 (tensor cores, tcgen05): what the finished groups send into this group.  For each
//     finished 32-vertex source block c this is, over all steps at once, the product
//     [128 x 32] x [32 x steps] of the tile of E (transposed: destinations are the rows) with the rows
//     y[s-1][32c..32c+31] (scaled to the step's common unit 2^g[s-1]); the [128 x steps] sum lives in
//     tensor memory and the diagonal blocks read their column of it step by step; see strip_bulk_umma.
//   phase 2 (10 warps, one CTA barrier per iteration): the ten blocks inside the group, one per
//     warp, walked as a pipeline.  In iteration tau the triangular block of sub-strip k does step
//     tau - k, and the square block from sub-strip ks to kd does step tau - ks: its sources were
//     finished one iteration earlier, and its sum (a ring accumulator with its own exponent) is
//     complete when the destination's triangular block needs it.  A group therefore takes
//     (steps + 3) iterations instead of 4 x steps.
// A triangular step combines its three terms at a unit chosen from magnitudes that are known
// before its own sum is (see strip_diag_step), multiplies by exp(match) and stores the entry; the
// maxima it leaves behind are taken off the step-to-step chain.
// At the end the rows are written out exactly like the other paths write them: log2 values
// relative to one fp64 offset per row, plus the row maxima dag_fast_check_kernel needs.
// Anything that underflows is 2^-126 below the unit it is added in, which sits within 2^64 of the
// largest term, i.e. inside what the check's bound covers; inputs below 2^-120 flag the sentence
// as in the tiled kernel.
#pragma once

#include "umma.cuh"

namespace dat {

// defined in dag_fast.cu: the a-posteriori check of one sentence, run by the sentence's sweep CTA that finishes second
__device__ __forceinline__ void fast_check_sentence(int b, int bits, const double *__restrict__ offsets_all,
                                                    const float *__restrict__ chk_all, const float *__restrict__ sub_all,
                                                    int nH, long long ol, long long tl, int *__restrict__ flag,
                                                    int32_t *__restrict__ status, int T, int tid, int nthreads);

constexpr int kStripThreads = 512;
constexpr int kStripWarps = kStripThreads / 32;
constexpr int kExpNone = -(1 << 28);   // exponent of a half-strip that is entirely zero

// 2^k as a float; 0 when it would be subnormal or when an operand was kExpNone
__device__ __forceinline__ float pow2_flush(int k) {
    if (k < -126) return 0.f;
    k = k > 127 ? 127 : k;
    return __int_as_float((k + 127) << 23);
}
// floor(log2(x)) for a positive normal float given by its bits
__device__ __forceinline__ int exponent_of_bits(unsigned bits) { return (int)(bits >> 23) - 127; }

__device__ __forceinline__ void strip_cp_async4(float *smem_dst, const float *gsrc) {
    const unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(d), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void strip_cp_async_wait_all() {
    asm volatile("cp.async.commit_group;\n\tcp.async.wait_group 0;" ::: "memory");
}
// l[r] = link (natural log) from canonical vertex 32c+r to canonical vertex 32h+lane, -inf if it
// does not exist.  Forward: links[u'][u-u'-1]; reversed: the link of the original graph from
// ol-1-u to ol-1-u', i.e. links[ol-1-u][u-u'-1].  A block strictly before the diagonal whose every
// link exists (the common case) is read without masks, all 32 loads in flight together.
__device__ __forceinline__ void strip_load_raw(float (&l)[32], const float *__restrict__ links, int c, int h,
                                               int lane, int K, int ol, bool rev) {
    const int u = 32 * h + lane;
    const int d0 = u - 32 * c - 1;
    const bool full = h > c && 32 * (h - c) + 30 < K && 32 * h + 31 < ol;   // warp-uniform
    const float *p = rev ? links + (size_t)(ol - 1 - (u < ol ? u : ol - 1)) * K + d0
                         : links + (size_t)(32 * c) * K + d0;
    const long long stride = rev ? -1 : (long long)(K - 1);
    if (full) {
#pragma unroll
        for (int r = 0; r < 32; r++) l[r] = __ldg(p + r * stride);
    } else {
#pragma unroll
        for (int r = 0; r < 32; r++) {
            const int d = d0 - r;
            l[r] = (d >= 0 && d < K && u < ol) ? __ldg(p + r * stride) : -INFINITY;
        }
    }
}
// What the sweep remembers about the size of its inputs (log2 units), one pair per thread:
//   fin: the smallest FINITE link or in-window match it used (below kMinLog2Input: "tiny");
//   all: the smallest link between two vertices of the graph that the band reaches (-inf: a "hole").
// Both are looked at where the values are consumed, so that the loads stay in flight until then.
struct StripInputRange {
    float fin, all;
};
__device__ __forceinline__ void strip_note_finite(StripInputRange &ir, float l2) {
    ir.fin = fminf(ir.fin, l2 > -INFINITY ? l2 : INFINITY);
}
// in place: e[r] = exp(l[r]) for the block strip_load_raw fetched (same c, h)
__device__ __forceinline__ void strip_exp_block(float (&e)[32], int c, int h, int lane, int K, int ol,
                                                StripInputRange &ir) {
    const int u = 32 * h + lane;
    const int d0 = u - 32 * c - 1;
    const bool full = h > c && 32 * (h - c) + 30 < K && 32 * h + 31 < ol;   // warp-uniform, as in strip_load_raw
#pragma unroll
    for (int r = 0; r < 32; r++) {
        const float l2 = e[r] * kLog2e;
        strip_note_finite(ir, l2);
        const int d = d0 - r;
        ir.all = fminf(ir.all, (full || (d >= 0 && d < K && u < ol)) ? l2 : INFINITY);
        e[r] = ex2(l2);
    }
}
// (two-lane multiply-adds: the same fused operations in half the issue slots)
__device__ __forceinline__ float strip_block_dot(const float *yrow, const float (&e)[32]) {
    float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll
    for (int q = 0; q < 8; q++) {
        const float4 a = *reinterpret_cast<const float4 *>(yrow + 4 * q);
        ffma2_rn(s0, s1, a.x, a.y, e[4 * q], e[4 * q + 1]);
        ffma2_rn(s2, s3, a.z, a.w, e[4 * q + 2], e[4 * q + 3]);
    }
    return (s0 + s1) + (s2 + s3);
}

constexpr int kGroupSubs = 4;                  // 32-vertex sub-strips per group
constexpr int kGroupCols = 32 * kGroupSubs;    // 128
constexpr int kRing = 8;                       // steps an in-group accumulator can be alive (> kGroupSubs)
constexpr int kMRing = 32;                     // steps of match values staged ahead
constexpr int kUmmaPolls = 1 << 22;            // bound of a wait for the tensor core (never reached)
__host__ __device__ inline int strip_step_pad(int T) { return (T + 15) & ~15; }   // N of the tensor-core product

struct StripSmem {
    float *Y;       // [T][rp]            mantissas of the rows, canonical vertices
    float *Ea;      // [2][128 x 32]      tf32 high / low parts of the E tile (destinations x sources), tensor-core layout
    float *Yb;      // [2][Tpad x 32]     tf32 high / low parts of the scaled rows (steps x sources), same layout
    float *M;       // [kMRing][kGroupCols] match values (natural log) of the current group, ring over steps
    float *Pr;      // [kGroupSubs][kRing][32] what the group's earlier sub-strips send, ring over steps
    int *Pe;        // [kGroupSubs][kRing]     and the exponent of each such accumulator
    int *sc;        // [T][nH]   exponent of each 32-vertex sub-strip (kExpNone: nothing there)
    int *g;         // [T]       largest exponent over the finished groups
    unsigned *mxy;  // [T][nH]   largest entry of a sub-strip, as float bits, in the sub-strip's unit
    unsigned *mxv;  // [T][nH]   the same before the multiplication by exp(match)
    uint64_t *mbar; // completion barrier of the tensor-core products
    uint32_t *tmem; // base address of the accumulator in tensor memory
};
__host__ __device__ inline size_t strip_smem_floats(int T, int rp) {
    const int nH = rp / 32;
    return (size_t)T * rp + (size_t)2 * kGroupCols * 32 + (size_t)2 * strip_step_pad(T) * 32 +
           (size_t)kMRing * kGroupCols + (size_t)kGroupSubs * kRing * 32 + kGroupSubs * kRing + (size_t)T * nH +
           T + (size_t)2 * T * nH + 8;
}

// x * 2^k for k in [-252, 254] as two exact power-of-two multiplications; 0 below that range
// (also for k derived from kExpNone)
__device__ __forceinline__ float scale2(float x, int k) {
    if (k >= -126 && k <= 127) return x * __int_as_float((k + 127) << 23);   // the usual case: one factor
    if (k < -252) return 0.f;
    k = k > 254 ? 254 : k;
    const int k1 = k / 2, k2 = k - k1;
    return (x * __int_as_float((k1 + 127) << 23)) * __int_as_float((k2 + 127) << 23);
}

// The tensor core reads the upper 19 bits of an fp32 operand (sign, exponent, 10 mantissa bits), so the
// high part of a split is the value itself with the low mantissa bits masked off; the rounding
// conversion instruction would run on the 16-lane special-function unit.
__device__ __forceinline__ float tf32_high(float x) { return __uint_as_float(__float_as_uint(x) & 0xffffe000u); }
__device__ __forceinline__ void tf32_split4(const float (&v)[4], float4 &hi, float4 &lo) {
    hi = make_float4(tf32_high(v[0]), tf32_high(v[1]), tf32_high(v[2]), tf32_high(v[3]));
    lo = make_float4(v[0] - hi.x, v[1] - hi.y, v[2] - hi.z, v[3] - hi.w);
}

// phase 1: what the finished groups send into the current group, as matrix products on the tensor
// cores (tcgen05.mma, accumulator in tensor memory).  For one 32-vertex source block c and all steps
// at once
//     F[j][s] += sum_r E[32c + r][32 h0 + j] * (y[s-1][32c + r] * 2^(sc[s-1][c] - g[s-1])),  j < 128,
// i.e. [128 x 32] x [32 x steps], summed over c: D = A * B^T with A = the E tile (row = destination j,
// K = source r) and B = the scaled rows (row = step s, K = source r), both staged by all threads in
// the K-major layout of umma.cuh, one thread issuing the instructions.  fp32 accuracy comes from
// splitting both operands into two tf32 numbers and adding the three leading products
// (hi*hi + hi*lo + lo*hi) into the same fp32 accumulator.  The [128 lanes x steps] accumulator stays
// in tensor memory; lane j, column s is what strip_diag_step of sub-strip j / 32 reads at step s.
// The operand tiles are single-buffered: the products of block c must have finished (mbarrier) before
// block c + 1 is staged; the links of block c + 1 are in flight meanwhile.
// Returns false if a wait for the tensor core ran out (the caller then hands the sentence to the
// exact kernels).
__device__ __forceinline__ bool strip_bulk_umma(const float *__restrict__ links, const StripSmem &sm, int h0,
                                                int t0, int t1, int tid, int K, int ol, int rp, int nH,
                                                int Tpad, bool rev, uint32_t tmem_base, uint32_t &mbar_phase,
                                                StripInputRange &ir) {
    const int lane = tid & 31, warp = tid >> 5;
    int cmin = h0 - (K - 1) / 32 - 1;   // blocks further back hold no link into the group
    cmin = cmin > 0 ? cmin : 0;
    bool ok_all = true;
    // E tile: a thread owns one destination m and the K chunks kq0, kq0 + 4 (four sources each).  The
    // lanes of a quarter-warp always hold eight consecutive destinations with the same chunk, so their
    // 16-byte stores fall into distinct banks; beyond that the lanes run along whatever is contiguous in
    // memory: the destinations in the forward sweep (a band row holds the links of one source), the
    // chunks in the reversed sweep (a band row holds the links INTO one canonical destination).
    const int m = rev ? 8 * warp + (lane & 7) : tid & (kGroupCols - 1);
    const int kq0 = rev ? lane >> 3 : tid >> 7;
    const int u = 32 * h0 + m;
    const auto tile_load = [&](int c, float (&v)[8]) {
#pragma unroll
        for (int q = 0; q < 8; q++) {
            const int r = 4 * (kq0 + 4 * (q >> 2)) + (q & 3);
            const int up = 32 * c + r, d = u - up - 1;   // d >= 0: c < h0
            const bool ok = d < K && u < ol;
            const float *p = rev ? links + (size_t)(ol - 1 - (u < ol ? u : ol - 1)) * K + d
                                 : links + (size_t)up * K + d;
            v[q] = ok ? __ldg(p) : -INFINITY;
        }
    };
    char *ea_hi = reinterpret_cast<char *>(sm.Ea), *ea_lo = ea_hi + kGroupCols * 32 * sizeof(float);
    char *yb_hi = reinterpret_cast<char *>(sm.Yb), *yb_lo = yb_hi + (size_t)Tpad * 32 * sizeof(float);
    const uint32_t idesc_full = umma::instr_desc_tf32(kGroupCols, Tpad > 256 ? 256 : Tpad);
    float cur[8], nxt[8];
    tile_load(cmin, cur);
    for (int c = cmin; c < h0; c++) {
        if (c + 1 < h0) tile_load(c + 1, nxt);   // in flight while block c is staged and multiplied
        if (c > cmin) {   // the products of block c - 1 have read the tiles
            if (ok_all && !umma::mbar_wait(sm.mbar, mbar_phase, kUmmaPolls)) ok_all = false;
            mbar_phase ^= 1u;
        }
        // ---- E tile of block c
#pragma unroll
        for (int half = 0; half < 2; half++) {
            float e[4];
#pragma unroll
            for (int q = 0; q < 4; q++) {
                const float l2 = cur[4 * half + q] * kLog2e;
                strip_note_finite(ir, l2);
                const int r = 4 * (kq0 + 4 * half) + q;
                ir.all = fminf(ir.all, ((u - 32 * c - r - 1 < K) && u < ol) ? l2 : INFINITY);
                e[q] = ex2(l2);
            }
            float4 hi, lo;
            tf32_split4(e, hi, lo);
            const int off = umma::tile_unit_offset(m, kq0 + 4 * half);
            *reinterpret_cast<float4 *>(ea_hi + off) = hi;
            *reinterpret_cast<float4 *>(ea_lo + off) = lo;
        }
        // ---- scaled rows of block c: row (= step) 8 rg + lane % 8, K chunk kq
        {
            const int kq = (lane >> 3) + 4 * (warp & 1);
            for (int rg = warp >> 1; 8 * rg < Tpad; rg += kStripWarps / 2) {
                const int sx = 8 * rg + (lane & 7);
                float y[4] = {0.f, 0.f, 0.f, 0.f};
                if (sx >= t0 && sx <= t1) {
                    const int ex = sm.sc[(sx - 1) * nH + c];
                    const int kx = ex - sm.g[sx - 1];   // <= 0
                    if (ex != kExpNone && kx >= -252) {
                        // 2^kx as two exact factors (the second is 1 in the usual case): an entry only
                        // vanishes when it is really below 2^-126 in the step's unit
                        const int k1 = kx >= -126 ? kx : kx / 2;
                        const float f1 = __int_as_float((k1 + 127) << 23), f2 = __int_as_float((kx - k1 + 127) << 23);
                        const float4 yv = *reinterpret_cast<const float4 *>(sm.Y + (size_t)(sx - 1) * rp + 32 * c + 4 * kq);
                        y[0] = (yv.x * f1) * f2;
                        y[1] = (yv.y * f1) * f2;
                        y[2] = (yv.z * f1) * f2;
                        y[3] = (yv.w * f1) * f2;
                    }
                }
                float4 hi, lo;
                tf32_split4(y, hi, lo);
                const int off = umma::tile_unit_offset(sx, kq);
                *reinterpret_cast<float4 *>(yb_hi + off) = hi;
                *reinterpret_cast<float4 *>(yb_lo + off) = lo;
            }
        }
        umma::fence_smem_to_async();
        __syncthreads();
        if (tid == 4 * 32) {   // one thread of a warp that owns no diagonal block issues the products
            umma::fence_after_sync();
            const uint32_t a_hi = umma::smem_u32(ea_hi), a_lo = umma::smem_u32(ea_lo);
            for (int n0 = 0; n0 < Tpad; n0 += 256) {   // at most 256 steps per instruction
                const int nn = Tpad - n0 < 256 ? Tpad - n0 : 256;
                const uint32_t idesc = nn == 256 || Tpad <= 256 ? idesc_full : umma::instr_desc_tf32(kGroupCols, nn);
                const uint32_t b_hi = umma::smem_u32(yb_hi) + (n0 >> 3) * umma::kRowGroupBytes;
                const uint32_t b_lo = umma::smem_u32(yb_lo) + (n0 >> 3) * umma::kRowGroupBytes;
                const uint32_t d = tmem_base + (uint32_t)n0;
#pragma unroll
                for (int kk = 0; kk < umma::kTileK / 8; kk++) {
                    const uint32_t o = kk * umma::kStepBytes;
                    umma::mma_tf32(d, umma::smem_desc(a_hi + o), umma::smem_desc(b_hi + o), idesc, c > cmin || kk > 0);
                    umma::mma_tf32(d, umma::smem_desc(a_hi + o), umma::smem_desc(b_lo + o), idesc, true);
                    umma::mma_tf32(d, umma::smem_desc(a_lo + o), umma::smem_desc(b_hi + o), idesc, true);
                }
            }
            umma::commit(sm.mbar);
        }
#pragma unroll
        for (int q = 0; q < 8; q++) cur[q] = nxt[q];
    }
    // the last block's products: the accumulator is complete
    if (ok_all && !umma::mbar_wait(sm.mbar, mbar_phase, kUmmaPolls)) ok_all = false;
    mbar_phase ^= 1u;
    umma::fence_after_sync();
    return ok_all;
}

// State a diagonal block carries from one step of its sub-strip to the next.
struct StripCarry {
    int eo;            // exponent of the sub-strip at the previous step (kExpNone: nothing there)
    unsigned ybits;    // largest entry of the previous step, as float bits
    unsigned vbits;    // the same before the multiplication by exp(match)
    int sprev;         // the previous step (-1: none yet), for the delayed store of the two maxima
    float far_next;    // what the finished groups send at the next step (requested from tensor memory)
};

// One step of a diagonal (triangular) block: sub-strip h = h0 + k of the group, step s.  Three
// terms meet here, each with its own unit: the block's own sum (unit 2^eo), what the finished
// groups sent (phase-1 accumulator, unit 2^g[s-1]) and what the group's earlier sub-strips sent (ring accumulator
// with its own exponent).  Their magnitudes are known before the own sum is: the maximum of this
// sub-strip one step ago and warp maxima of the other two, all taken while the own sum is being
// computed.  The new unit puts the largest of the three near 2^kTargetExp, so that the only
// things on the step-to-step chain are the shared loads of the previous row, the 32
// multiply-adds, two scalings and the store; nothing overflows, and what is flushed is 2^-190
// below the largest term.
// far_col: tensor-memory address of this warp's 32 lanes of the phase-1 accumulator, column 0 (only
// meaningful when has_far: the group has finished predecessors); the column of step s + 1 is requested
// here, at step s.
__device__ __forceinline__ void strip_diag_step(const StripSmem &sm, const float (&ed)[32], int h, int k, int s,
                                                int lane, int ol, int W, int rp, int nH, bool want_v,
                                                bool has_far, uint32_t far_col, int t1, StripCarry &cy,
                                                StripInputRange &ir) {
    const int u = 32 * h + lane, pc = 32 * k + lane, ring = (k * kRing + (s & (kRing - 1)));
    // ---- independent of the previous step's result
    const int U = sm.g[s - 1];
    const int en = sm.Pe[ring];
    float far = 0.f;
    if (has_far) {   // warp-uniform
        umma::tmem_ld_wait(cy.far_next);
        far = cy.far_next;
        if (s < t1) umma::tmem_ld_col(cy.far_next, far_col + (uint32_t)(s + 1));
    }
    const float near = sm.Pr[ring * 32 + lane];
    sm.Pr[ring * 32 + lane] = 0.f;      // and the ring entry for the step kRing later
    __syncwarp();
    if (lane == 0) sm.Pe[ring] = kExpNone;
    const float m2 = sm.M[(s & (kMRing - 1)) * kGroupCols + pc] * kLog2e;
    const bool inside = u >= s && u <= s + W - 1 && u < ol;
    ir.fin = fminf(ir.fin, (inside && m2 > -INFINITY) ? m2 : INFINITY);
    const float pm = inside ? ex2(m2) : 0.f;
    // values are >= 0 (or inf/NaN from bad inputs, which order above every finite float as bits)
    const unsigned fbits = __reduce_max_sync(0xffffffffu, __float_as_uint(far));
    const unsigned nbits = __reduce_max_sync(0xffffffffu, __float_as_uint(near));
    if (lane == 0 && cy.sprev >= 0) {   // maxima of the previous step, stored off the chain
        sm.mxy[cy.sprev * nH + h] = cy.ybits;
        sm.mxv[cy.sprev * nH + h] = cy.vbits;
    }
    const int eo = cy.eo;
    int est = (cy.ybits != 0u && eo != kExpNone) ? exponent_of_bits(cy.ybits) + eo + 5 : kExpNone;
    if (fbits != 0u && U != kExpNone) { const int x = exponent_of_bits(fbits) + U; est = x > est ? x : est; }
    if (nbits != 0u && en != kExpNone) { const int x = exponent_of_bits(nbits) + en; est = x > est ? x : est; }
    const int sn = est != kExpNone ? est - kTargetExp : kExpNone;
    if (lane == 0) sm.sc[s * nH + h] = sn;
    const float rest = est != kExpNone ? scale2(far, U - sn) + scale2(near, en - sn) : 0.f;
    // multipliers of the own sum: 2^(eo - sn) as two exact factors (0 when it does not count)
    float a1 = 0.f, a2 = 0.f;
    if (eo != kExpNone && est != kExpNone && eo - sn >= -252) {
        int kk = eo - sn; kk = kk > 254 ? 254 : kk;
        const int k1 = (kk >= -126 && kk <= 127) ? kk : kk / 2;   // the usual case: one factor, the other is 1
        a1 = __int_as_float((k1 + 127) << 23);
        a2 = __int_as_float((kk - k1 + 127) << 23);
    }
    // ---- the chain: previous row -> own sum -> entry
    const float own = eo != kExpNone ? strip_block_dot(sm.Y + (size_t)(s - 1) * rp + 32 * h, ed) : 0.f;
    const float val = (own * a1) * a2 + rest;
    const float y = val * pm;
    sm.Y[(size_t)s * rp + u] = y;
    // ---- for the next step (the reductions overlap its loads and multiply-adds)
    cy.ybits = __reduce_max_sync(0xffffffffu, __float_as_uint(y));
    cy.vbits = want_v ? __reduce_max_sync(0xffffffffu, __float_as_uint(inside ? val : 0.f)) : 0u;
    cy.eo = sn;
    cy.sprev = s;
}

// One step of an in-group square block: sources sub-strip h0+ks at step s-1, destinations
// sub-strip h0+kd at step s.  The sum joins the ring accumulator of (kd, s), whose exponent
// follows the largest source exponent seen so far.  Only one block touches a given accumulator
// in one iteration; the CTA barrier orders the iterations.
__device__ __forceinline__ void strip_cross_step(const StripSmem &sm, const float (&ex)[32], int h0, int ks,
                                                 int kd, int s, int lane, int rp, int nH) {
    const int en = sm.sc[(s - 1) * nH + h0 + ks];
    if (en == kExpNone) return;   // warp-uniform
    const int ring = kd * kRing + (s & (kRing - 1));
    const int pe = sm.Pe[ring];
    const float acc = sm.Pr[ring * 32 + lane];
    const float dot = strip_block_dot(sm.Y + (size_t)(s - 1) * rp + 32 * (h0 + ks), ex);
    float out;
    int ne;
    if (pe == kExpNone || en >= pe) {
        out = (pe == kExpNone ? 0.f : acc * pow2_flush(pe - en)) + dot;
        ne = en;
    } else {
        out = acc + dot * pow2_flush(en - pe);
        ne = pe;
    }
    sm.Pr[ring * 32 + lane] = out;
    __syncwarp();
    if (lane == 0) sm.Pe[ring] = ne;
}

__global__ void __launch_bounds__(kStripThreads, 1)
dag_strip_sweep_kernel(const float *__restrict__ match_all, const float *__restrict__ links_all,
                       const int64_t *__restrict__ output_length, const int64_t *__restrict__ target_length,
                       const int *__restrict__ order, float *__restrict__ alpha_all,
                       float *__restrict__ beta_all, double *__restrict__ offsets_all,
                       float *__restrict__ chk_all, float *__restrict__ sub_all, int *__restrict__ flag,
                       float *__restrict__ loss, int32_t *__restrict__ status, int T, int L, int K, int rp) {
    extern __shared__ __align__(16) float ssm[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const bool rev = blockIdx.x & 1;   // odd CTAs: the beta recursion (reversed graph)
    const int b = order ? order[blockIdx.x >> 1] : (int)(blockIdx.x >> 1);
    const long long oll = output_length[b], tll = target_length[b];
    double *offs = offsets_all + (size_t)b * (2 * T + 2);
    if (!lengths_valid(oll, tll, T, L)) {
        if (tid == 0) {
            offs[2 * T + (rev ? 1 : 0)] = -INFINITY;
            if (rev) loss[b] = -INFINITY;
            if (status) atomicOr(status, DAT_STATUS_BAD_LENGTH);
        }
        return;
    }
    const int ol = (int)oll, tl = (int)tll;
    const int W = ol - tl + 1;
    const int nH = rp / 32;
    const float *match = match_all + (size_t)b * T * L;
    const float *links = links_all + (size_t)b * L * K;
    float *out = (rev ? beta_all : alpha_all) + (size_t)b * T * L;
    float *chk = chk_all + (size_t)b * 2 * T + (rev ? T : 0);
    StripSmem sm;
    sm.Y = ssm;
    const int Tpad = strip_step_pad(T);
    sm.Ea = sm.Y + (size_t)T * rp;
    sm.Yb = sm.Ea + 2 * kGroupCols * 32;
    sm.M = sm.Yb + (size_t)2 * Tpad * 32;
    sm.Pr = sm.M + kMRing * kGroupCols;
    sm.Pe = reinterpret_cast<int *>(sm.Pr + kGroupSubs * kRing * 32);
    sm.sc = sm.Pe + kGroupSubs * kRing;
    sm.g = sm.sc + T * nH;
    sm.mxy = reinterpret_cast<unsigned *>(sm.g + T);
    sm.mxv = sm.mxy + T * nH;
    sm.mbar = reinterpret_cast<uint64_t *>((reinterpret_cast<uintptr_t>(sm.mxv + T * nH) + 7) & ~(uintptr_t)7);
    sm.tmem = reinterpret_cast<uint32_t *>(sm.mbar + 1);

    // tensor memory for the phase-1 accumulator: 128 lanes x Tpad columns (a power of two >= 32 is allocated)
    int tmem_cols = 32;
    while (tmem_cols < Tpad) tmem_cols <<= 1;
    if (warp == 0) umma::tmem_alloc(sm.tmem, tmem_cols);
    if (tid == 0) umma::mbar_init(sm.mbar, 1);
    for (int x = tid; x < tl * rp; x += kStripThreads) sm.Y[x] = 0.f;
    for (int x = tid; x < kGroupSubs * kRing * 32; x += kStripThreads) sm.Pr[x] = 0.f;
    for (int x = tid; x < kGroupSubs * kRing; x += kStripThreads) sm.Pe[x] = kExpNone;
    for (int x = tid; x < T * nH; x += kStripThreads) {
        sm.sc[x] = kExpNone;
        sm.mxy[x] = 0u;
        sm.mxv[x] = 0u;
    }
    for (int x = tid; x < T; x += kStripThreads) sm.g[x] = kExpNone;
    umma::fence_before_sync();
    __syncthreads();
    umma::fence_after_sync();
    const uint32_t tmem_base = *sm.tmem;   // lane 0, column 0 of the accumulator
    uint32_t mbar_phase = 0;   // parity of the next completion of the tensor-core barrier
    bool tc_ok = true;         // no wait for the tensor core has run out
    StripInputRange ir;
    ir.fin = INFINITY;
    ir.all = K < ol - 1 ? -INFINITY : INFINITY;   // a band narrower than the graph: vertex pairs without a link
    if (tid == 0) {
        // step 0: only canonical vertex 0, value exp(match) = 2^m0
        const float m0 = (rev ? match[(size_t)(tl - 1) * L + (ol - 1)] : match[0]) * kLog2e;
        strip_note_finite(ir, m0);
        if (m0 > -INFINITY && m0 < INFINITY) {
            const float fl = floorf(m0);
            sm.Y[0] = ex2(m0 - fl);
            sm.sc[0] = (int)fl;
            sm.mxy[0] = __float_as_uint(sm.Y[0]);
        }
    }
    __syncthreads();

    const int nsub = (ol + 31) >> 5;
    for (int h0 = 0; h0 < nsub; h0 += kGroupSubs) {
        const int gs = nsub - h0 < kGroupSubs ? nsub - h0 : kGroupSubs;   // sub-strips in this group
        int t0 = 32 * h0 - W + 1; t0 = t0 > 1 ? t0 : 1;                  // steps at which the group is reachable
        int t1 = 32 * (h0 + gs) - 1; t1 = t1 < tl - 1 ? t1 : tl - 1;
        // match values of the first steps (the rest follows in the ring, two batches ahead)
        const auto stage_match = [&](int s_first) {   // steps [s_first, s_first + 8)
            for (int x = tid; x < 8 * kGroupCols; x += kStripThreads) {
                const int s = s_first + x / kGroupCols, pc = x % kGroupCols, u = 32 * h0 + pc;
                if (s > t1) break;
                float *dst = sm.M + (s & (kMRing - 1)) * kGroupCols + pc;
                if (u < ol)
                    strip_cp_async4(dst, rev ? match + (size_t)(tl - 1 - s) * L + (ol - 1 - u)
                                             : match + (size_t)s * L + u);
                else *dst = -INFINITY;
            }
        };
        stage_match(t0);
        stage_match(t0 + 8);
        // ---- the group's own blocks: sub-strip pairs (ks <= kd); warp w takes block number w of the
        // list D_0 .. D_{gs-1}, then the square blocks row by row.  Its links are requested now and
        // exponentiated after phase 1, which hides their latency.
        static_assert(kGroupSubs * (kGroupSubs + 1) / 2 <= kStripWarps, "one block per warp");
        float eb0[32];
        int ks0 = -1, kd0 = -1;
        {
            int idx = 0;
            for (int kd = 0; kd < gs; kd++, idx++)
                if (idx == warp) { ks0 = kd; kd0 = kd; }
            for (int kd = 1; kd < gs; kd++)
                for (int ks = 0; ks < kd; ks++, idx++)
                    if (idx == warp) { ks0 = ks; kd0 = kd; }
        }
        if (kd0 >= 0) strip_load_raw(eb0, links, h0 + ks0, h0 + kd0, lane, K, ol, rev);
        // ---- phase 1: everything the finished groups send into this group
        if (h0 > 0)
            tc_ok &= strip_bulk_umma(links, sm, h0, t0, t1, tid, K, ol, rp, nH, Tpad, rev, tmem_base, mbar_phase, ir);
        if (kd0 >= 0) strip_exp_block(eb0, h0 + ks0, h0 + kd0, lane, K, ol, ir);
        strip_cp_async_wait_all();
        __syncthreads();
        // ---- phase 2: pipelined walk.  In iteration tau the diagonal block of sub-strip k does step
        // tau - k and a square block with sources ks does step tau - ks (its sources were finished
        // in iteration tau - 1, its destination needs the sum in iteration tau - ks + kd).
        StripCarry cy;
        cy.eo = kExpNone; cy.ybits = 0u; cy.vbits = 0u; cy.sprev = -1; cy.far_next = 0.f;
        uint32_t far_col = 0u;   // this warp's lanes of the phase-1 accumulator (diagonal warp k = warp k: lanes 32k..)
        const bool has_far = h0 > 0 && t0 <= t1;
        if (kd0 >= 0 && ks0 == kd0) {   // this sub-strip at step t0-1 (non-zero only at step 0)
            const int h = h0 + kd0;
            cy.eo = sm.sc[(t0 - 1) * nH + h];
            cy.ybits = __reduce_max_sync(0xffffffffu, __float_as_uint(sm.Y[(size_t)(t0 - 1) * rp + 32 * h + lane]));
            if (has_far) {
                umma::fence_after_sync();
                far_col = tmem_base + ((uint32_t)(32 * kd0) << 16);
                umma::tmem_ld_col(cy.far_next, far_col + (uint32_t)t0);
            }
        }
        for (int tau = t0; tau <= t1 + gs - 1; tau++) {
            if (((tau - t0) & 7) == 0) {   // match values two batches ahead; the batch before them has landed
                stage_match(tau + 16);
                asm volatile("cp.async.commit_group;\n\tcp.async.wait_group 1;" ::: "memory");
            }
            if (kd0 >= 0) {
                const int s = tau - ks0;
                if (s >= t0 && s <= t1) {
                    if (ks0 == kd0) strip_diag_step(sm, eb0, h0 + kd0, kd0, s, lane, ol, W, rp, nH, rev, has_far, far_col, t1, cy, ir);
                    else strip_cross_step(sm, eb0, h0, ks0, kd0, s, lane, rp, nH);
                }
            }
            __syncthreads();
        }
        if (kd0 >= 0 && ks0 == kd0 && lane == 0 && cy.sprev >= 0) {   // maxima of the last step
            sm.mxy[cy.sprev * nH + h0 + kd0] = cy.ybits;
            sm.mxv[cy.sprev * nH + h0 + kd0] = cy.vbits;
        }
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        umma::fence_before_sync();   // the accumulator has been read; the next group's products may overwrite it
        __syncthreads();
        // the group's exponents join the running maxima
        for (int s = t0 - 1 + tid; s <= t1; s += kStripThreads) {
            int m = sm.g[s];
            for (int k = 0; k < gs; k++) {
                const int a = sm.sc[s * nH + h0 + k];
                m = a > m ? a : m;
            }
            sm.g[s] = m;
        }
        __syncthreads();
    }
    if (ir.fin < kMinLog2Input || !tc_ok) atomicOr(flag + b, kFlagTiny);   // either way: redone by the exact kernels
    if (ir.all == -INFINITY) atomicOr(flag + b, kFlagHole);

    // ---- write the rows out: log2 values relative to one fp64 offset per row
    float *sub = sub_all + ((size_t)b * 2 + (rev ? 1 : 0)) * T * nH;   // log2 maxima per (step, sub-strip)
    for (int s = warp; s < tl; s += kStripWarps) {
        float ry = -INFINITY, rv = -INFINITY;
        for (int h = lane; h < nH; h += 32) {
            const unsigned yb = sm.mxy[s * nH + h], vb = sm.mxv[s * nH + h];
            const float e = (float)sm.sc[s * nH + h];
            float hy = -INFINITY, hv = -INFINITY;
            if (yb != 0u) hy = lg2(__uint_as_float(yb)) + e;
            if (vb != 0u) hv = lg2(__uint_as_float(vb)) + e;
            ry = fmaxf(ry, hy);
            rv = fmaxf(rv, hv);
            sub[(rev ? tl - 1 - s : s) * nH + h] = rev ? hv : hy;   // canonical sub-strip index
        }
        ry = warp_max(ry);
        rv = warp_max(rv);
        const int t = rev ? tl - 1 - s : s;
        const int off = (ry > -INFINITY && ry < INFINITY) ? (int)floorf(ry) : 0;
        if (lane == 0) {
            offs[(rev ? T : 0) + t] = (double)off;
            chk[t] = rev ? rv : ry;
        }
        int uhi = s + W - 1; uhi = uhi < ol - 1 ? uhi : ol - 1;
        for (int u = s + lane; u <= uhi; u += 32) {
            const float y = sm.Y[(size_t)s * rp + u];
            const float v = lg2(y) + (float)(sm.sc[s * nH + (u >> 5)] - off);
            out[(size_t)t * L + (rev ? ol - 1 - u : u)] = (y > 0.f || y != y) ? v : -INFINITY;
        }
    }
    if (tid == 0) {
        const float y = sm.Y[(size_t)(tl - 1) * rp + (ol - 1)];
        const int e = sm.sc[(tl - 1) * nH + ((ol - 1) >> 5)];
        const double z2 = (y > 0.f && e != kExpNone) ? (double)lg2(y) + (double)e : (y != y ? (double)y : -INFINITY);
        offs[2 * T + (rev ? 1 : 0)] = z2;
        if (rev) loss[b] = (float)(z2 * kLn2d);
    }
    if (warp == 0) {   // every read of the accumulator finished before the last barrier of the group loop
        __syncwarp();
        umma::tmem_dealloc(tmem_base, tmem_cols);
    }
    // ---- the check of the sentence, by whichever of its two CTAs finishes second: the arrival count sits
    // above the flag bits of the sentence's word (cleared before the launch)
    __shared__ int arrived_before;
    __threadfence();   // this CTA's rows, maxima and offsets are visible before its arrival is
    __syncthreads();
    if (tid == 0) arrived_before = atomicAdd(flag + b, kFlagArrival);
    __syncthreads();
    if (arrived_before >= kFlagArrival) {
        __threadfence();
        fast_check_sentence(b, arrived_before & kFlagBits, offsets_all, chk_all, sub_all, nH, oll, tll, flag, status, T, tid,
                            kStripThreads);
    }
}

}  // namespace dat
