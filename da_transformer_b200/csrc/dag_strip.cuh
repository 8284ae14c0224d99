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
//   phase 1 (16 warps, tensor cores): what the finished groups send into this group.  For each
//     finished 32-vertex source block c this is, over all steps at once, the product
//     [steps x 32] x [32 x 128] of the rows y[s-1][32c..32c+31] (scaled to the step's common unit
//     2^g[s-1]) with the tile of E; see strip_bulk_mma.  No dependency between source blocks.
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

namespace dat {

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
__device__ __forceinline__ float strip_block_dot(const float *yrow, const float (&e)[32]) {
    float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
#pragma unroll
    for (int q = 0; q < 8; q++) {
        const float4 a = *reinterpret_cast<const float4 *>(yrow + 4 * q);
        s0 = fmaf(a.x, e[4 * q], s0);
        s1 = fmaf(a.y, e[4 * q + 1], s1);
        s2 = fmaf(a.z, e[4 * q + 2], s2);
        s3 = fmaf(a.w, e[4 * q + 3], s3);
    }
    return (s0 + s1) + (s2 + s3);
}

constexpr int kGroupSubs = 4;                  // 32-vertex sub-strips per group
constexpr int kGroupCols = 32 * kGroupSubs;    // 128
constexpr int kRing = 8;                       // steps an in-group accumulator can be alive (> kGroupSubs)
constexpr int kMRing = 32;                     // steps of match values staged ahead
constexpr int kEtPitch = kGroupCols + 8;       // the tensor-core operand loads of a tile hit 32 distinct banks

struct StripSmem {
    float *Y;       // [T][rp]            mantissas of the rows, canonical vertices
    float *Pf;      // [T][kGroupCols]    what the finished groups send to the current group, unit 2^g[s-1]
    float *M;       // [kMRing][kGroupCols] match values (natural log) of the current group, ring over steps
    float *Pr;      // [kGroupSubs][kRing][32] what the group's earlier sub-strips send, ring over steps
    float *Et;      // [32][kEtPitch]     exp(links) from one finished 32-vertex block into the whole group
    int *Pe;        // [kGroupSubs][kRing]     and the exponent of each such accumulator
    int *sc;        // [T][nH]   exponent of each 32-vertex sub-strip (kExpNone: nothing there)
    int *g;         // [T]       largest exponent over the finished groups
    unsigned *mxy;  // [T][nH]   largest entry of a sub-strip, as float bits, in the sub-strip's unit
    unsigned *mxv;  // [T][nH]   the same before the multiplication by exp(match)
};
__host__ __device__ inline size_t strip_smem_floats(int T, int rp) {
    const int nH = rp / 32;
    return (size_t)T * rp + (size_t)T * kGroupCols + (size_t)kMRing * kGroupCols +
           (size_t)kGroupSubs * kRing * 32 + 32 * kEtPitch + kGroupSubs * kRing + (size_t)T * nH + T +
           (size_t)2 * T * nH;
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

// The tensor core reads the upper 19 bits of an fp32 operand (sign, exponent, 10 mantissa bits).
// Splitting by masking costs one logic operation; the rounding conversion instruction runs on
// the 16-lane special-function unit and was the bottleneck of this phase.
__device__ __forceinline__ unsigned to_tf32(float x) { return __float_as_uint(x) & 0xffffe000u; }
__device__ __forceinline__ void mma_tf32(float (&d)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// phase 1: what the finished groups send into the current group, as a matrix product on the
// tensor cores.  For one 32-vertex source block c and all steps at once
//     Pf[s][j] += sum_r (y[s-1][32c + r] * 2^(sc[s-1][c] - g[s-1])) * E[32c + r][32 h0 + j],  j < 128,
// i.e. [steps x 32] x [32 x 128], summed over c.  The CTA loads and exponentiates the
// [32 x 128] tile of E once per c (the loads of the next tile are in flight while this one is
// used); warp w owns destination sub-strip w % 4 and the 16 steps t0 + 16 (w / 4) .. (+64 per
// further pass), keeps its [16 x 32] result in registers over all c and stores it once: no atomics.
// fp32 accuracy comes from splitting both operands into two tf32 numbers and adding the three
// leading products (hi*hi + hi*lo + lo*hi) in fp32.
// Fragment layout of mma.m16n8k8 (g8 = lane / 4, t4 = lane % 4): A rows g8, g8+8, columns t4, t4+4;
// B rows t4, t4+4, column g8; C rows g8, g8+8, columns 2 t4, 2 t4 + 1.
__device__ __forceinline__ void strip_bulk_mma(const float *__restrict__ links, const StripSmem &sm, int h0,
                                               int gs, int t0, int t1, int tid, int K, int ol, int rp,
                                               int nH, bool rev, StripInputRange &ir) {
    const int lane = tid & 31, warp = tid >> 5;
    const int k = warp & 3, mt = warp >> 2, g8 = lane >> 2, t4 = lane & 3;
    int cmin = h0 - (K - 1) / 32 - 1;   // blocks further back hold no link into the group
    cmin = cmin > 0 ? cmin : 0;
    // tile element q of this thread: forward rows are contiguous along the destination, reversed
    // ones along the source, so the lanes run along that index
    const auto tile_rc = [&](int q, int &r, int &col) {
        if (rev) { r = lane; col = warp + kStripWarps * q; }
        else { r = (tid >> 7) + 4 * q; col = tid & 127; }
    };
    const auto tile_load = [&](int c, float (&v)[8]) {
#pragma unroll
        for (int q = 0; q < 8; q++) {
            int r, col;
            tile_rc(q, r, col);
            const int up = 32 * c + r, u = 32 * h0 + col, d = u - up - 1;   // d >= 0: c < h0
            const bool ok = d < K && u < ol;
            const float *p = rev ? links + (size_t)(ol - 1 - (u < ol ? u : ol - 1)) * K + d
                                 : links + (size_t)up * K + d;
            v[q] = ok ? __ldg(p) : -INFINITY;
        }
    };
    for (int sbase = t0; sbase <= t1; sbase += 64) {   // same trip count in every warp: barriers inside
        const int s0 = sbase + 16 * mt;
        float acc[4][4];
#pragma unroll
        for (int nn = 0; nn < 4; nn++)
#pragma unroll
            for (int q = 0; q < 4; q++) acc[nn][q] = 0.f;
        float nxt[8];
        tile_load(cmin, nxt);
        for (int c = cmin; c < h0; c++) {
#pragma unroll
            for (int q = 0; q < 8; q++) {
                int r, col;
                tile_rc(q, r, col);
                const float l2 = nxt[q] * kLog2e;
                strip_note_finite(ir, l2);
                const int u = 32 * h0 + col;
                ir.all = fminf(ir.all, ((u - 32 * c - r - 1 < K) && u < ol) ? l2 : INFINITY);
                sm.Et[r * kEtPitch + col] = ex2(l2);
            }
            __syncthreads();
            if (c + 1 < h0) tile_load(c + 1, nxt);
            // scale of the two A rows this lane holds (steps s0 + g8 and s0 + g8 + 8): 2^(sc - g), applied
            // as two exact power-of-two factors so that an entry only vanishes when it is really below
            // 2^-126 in the step's unit, i.e. 2^-190 below the largest entry of the finished groups
            // (the second factor is 1 in the usual case)
            float as1[2], as2[2];
#pragma unroll
            for (int q = 0; q < 2; q++) {
                const int sx = s0 + g8 + 8 * q;
                float f1 = 0.f, f2 = 0.f;
                if (k < gs && sx <= t1) {
                    const int e = sm.sc[(sx - 1) * nH + c];
                    int kx = e - sm.g[sx - 1];   // <= 0
                    if (e != kExpNone && kx >= -252) {
                        const int k1 = kx >= -126 ? kx : kx / 2;
                        f1 = __int_as_float((k1 + 127) << 23);
                        f2 = __int_as_float((kx - k1 + 127) << 23);
                    }
                }
                as1[q] = f1;
                as2[q] = f2;
            }
            if (__any_sync(0xffffffffu, as1[0] != 0.f || as1[1] != 0.f)) {
#pragma unroll
                for (int kk = 0; kk < 4; kk++) {
                    unsigned ahi[4], alo[4];
#pragma unroll
                    for (int q = 0; q < 4; q++) {   // (row g8 + 8 (q & 1), source t4 + 4 (q >> 1))
                        const int sx = s0 + g8 + 8 * (q & 1);
                        float a = 0.f;
                        if (as1[q & 1] != 0.f)
                            a = (sm.Y[(size_t)(sx - 1) * rp + 32 * c + 8 * kk + t4 + 4 * (q >> 1)] * as1[q & 1]) * as2[q & 1];
                        ahi[q] = to_tf32(a);
                        alo[q] = to_tf32(a - __uint_as_float(ahi[q]));
                    }
#pragma unroll
                    for (int nn = 0; nn < 4; nn++) {
                        const float b0 = sm.Et[(8 * kk + t4) * kEtPitch + 32 * k + 8 * nn + g8];
                        const float b1 = sm.Et[(8 * kk + t4 + 4) * kEtPitch + 32 * k + 8 * nn + g8];
                        const unsigned bh0 = to_tf32(b0), bh1 = to_tf32(b1);
                        const unsigned bl0 = to_tf32(b0 - __uint_as_float(bh0));
                        const unsigned bl1 = to_tf32(b1 - __uint_as_float(bh1));
                        mma_tf32(acc[nn], alo, bh0, bh1);
                        mma_tf32(acc[nn], ahi, bl0, bl1);
                        mma_tf32(acc[nn], ahi, bh0, bh1);
                    }
                }
            }
            __syncthreads();   // the tile is overwritten in the next round
        }
        if (k < gs) {
#pragma unroll
            for (int nn = 0; nn < 4; nn++)
#pragma unroll
                for (int q = 0; q < 4; q++) {   // (row g8 + 8 (q >> 1), column 2 t4 + (q & 1))
                    const int sx = s0 + g8 + 8 * (q >> 1);
                    if (sx <= t1) sm.Pf[sx * kGroupCols + 32 * k + 8 * nn + 2 * t4 + (q & 1)] = acc[nn][q];
                }
        }
    }
}

// State a diagonal block carries from one step of its sub-strip to the next.
struct StripCarry {
    int eo;            // exponent of the sub-strip at the previous step (kExpNone: nothing there)
    unsigned ybits;    // largest entry of the previous step, as float bits
    unsigned vbits;    // the same before the multiplication by exp(match)
    int sprev;         // the previous step (-1: none yet), for the delayed store of the two maxima
};

// One step of a diagonal (triangular) block: sub-strip h = h0 + k of the group, step s.  Three
// terms meet here, each with its own unit: the block's own sum (unit 2^eo), what the finished
// groups sent (Pf, unit 2^g[s-1]) and what the group's earlier sub-strips sent (ring accumulator
// with its own exponent).  Their magnitudes are known before the own sum is: the maximum of this
// sub-strip one step ago and warp maxima of the other two, all taken while the own sum is being
// computed.  The new unit puts the largest of the three near 2^kTargetExp, so that the only
// things on the step-to-step chain are the shared loads of the previous row, the 32
// multiply-adds, two scalings and the store; nothing overflows, and what is flushed is 2^-190
// below the largest term.
__device__ __forceinline__ void strip_diag_step(const StripSmem &sm, const float (&ed)[32], int h, int k, int s,
                                                int lane, int ol, int W, int rp, int nH, bool want_v,
                                                StripCarry &cy, StripInputRange &ir) {
    const int u = 32 * h + lane, pc = 32 * k + lane, ring = (k * kRing + (s & (kRing - 1)));
    // ---- independent of the previous step's result
    const int U = sm.g[s - 1];
    const int en = sm.Pe[ring];
    const float far = sm.Pf[s * kGroupCols + pc];
    sm.Pf[s * kGroupCols + pc] = 0.f;   // consumed: clean for the next group
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
    sm.Pf = sm.Y + (size_t)T * rp;
    sm.M = sm.Pf + (size_t)T * kGroupCols;
    sm.Pr = sm.M + kMRing * kGroupCols;
    sm.Et = sm.Pr + kGroupSubs * kRing * 32;
    sm.Pe = reinterpret_cast<int *>(sm.Et + 32 * kEtPitch);
    sm.sc = sm.Pe + kGroupSubs * kRing;
    sm.g = sm.sc + T * nH;
    sm.mxy = reinterpret_cast<unsigned *>(sm.g + T);
    sm.mxv = sm.mxy + T * nH;

    for (int x = tid; x < tl * rp; x += kStripThreads) sm.Y[x] = 0.f;
    for (int x = tid; x < T * kGroupCols; x += kStripThreads) sm.Pf[x] = 0.f;
    for (int x = tid; x < kGroupSubs * kRing * 32; x += kStripThreads) sm.Pr[x] = 0.f;
    for (int x = tid; x < kGroupSubs * kRing; x += kStripThreads) sm.Pe[x] = kExpNone;
    for (int x = tid; x < T * nH; x += kStripThreads) {
        sm.sc[x] = kExpNone;
        sm.mxy[x] = 0u;
        sm.mxv[x] = 0u;
    }
    for (int x = tid; x < T; x += kStripThreads) sm.g[x] = kExpNone;
    __syncthreads();
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
        if (h0 > 0) strip_bulk_mma(links, sm, h0, gs, t0, t1, tid, K, ol, rp, nH, rev, ir);
        if (kd0 >= 0) strip_exp_block(eb0, h0 + ks0, h0 + kd0, lane, K, ol, ir);
        strip_cp_async_wait_all();
        __syncthreads();
        // ---- phase 2: pipelined walk.  In iteration tau the diagonal block of sub-strip k does step
        // tau - k and a square block with sources ks does step tau - ks (its sources were finished
        // in iteration tau - 1, its destination needs the sum in iteration tau - ks + kd).
        StripCarry cy;
        cy.eo = kExpNone; cy.ybits = 0u; cy.vbits = 0u; cy.sprev = -1;
        if (kd0 >= 0 && ks0 == kd0) {   // this sub-strip at step t0-1 (non-zero only at step 0)
            const int h = h0 + kd0;
            cy.eo = sm.sc[(t0 - 1) * nH + h];
            cy.ybits = __reduce_max_sync(0xffffffffu, __float_as_uint(sm.Y[(size_t)(t0 - 1) * rp + 32 * h + lane]));
        }
        for (int tau = t0; tau <= t1 + gs - 1; tau++) {
            if (((tau - t0) & 7) == 0) {   // match values two batches ahead; the batch before them has landed
                stage_match(tau + 16);
                asm volatile("cp.async.commit_group;\n\tcp.async.wait_group 1;" ::: "memory");
            }
            if (kd0 >= 0) {
                const int s = tau - ks0;
                if (s >= t0 && s <= t1) {
                    if (ks0 == kd0) strip_diag_step(sm, eb0, h0 + kd0, kd0, s, lane, ol, W, rp, nH, rev, cy, ir);
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
    if (ir.fin < kMinLog2Input) atomicOr(flag + b, kFlagTiny);
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
}

}  // namespace dat
