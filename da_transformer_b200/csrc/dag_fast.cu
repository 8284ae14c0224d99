// dag_loss forward, fast path.  When all rows of a sentence fit in shared memory the
// strip-ordered sweep of dag_strip.cuh runs (one CTA per direction); otherwise the tiled kernel of
// this file, described next: both recursions of a sentence in ONE CTA, in the linear
// (probability) domain with per-row power-of-two rescaling, sharing every load of the
// transition matrix between the alpha and the beta step.
//
// Why it is faster than the log-domain sweep (dag_sweep.cu): a log-sum-exp term costs an
// exp each time it is used, i.e. (tl-1) times per link.  Here E[i][j] = exp(links[i][j])
// is computed ONCE per call into a zero-padded, 16-byte aligned square matrix
// (dag_fast_prep_kernel) and a term becomes a single FFMA:
//     alpha:  s_a[j] += a_{t-1}[i] * E[i][j]        beta:  s_b[i] += E[i][j] * b_{t+1}[j]
// In absolute vertex coordinates zeros replace all masks (E is 0 below the diagonal, past
// the band and past output_length; the rows a, b are 0 outside their windows), so tiles of
// 16 rows x 128 columns are read with aligned 128-bit loads and no predicates.  Alpha step
// k and beta step tl-1-k touch almost the same tiles, so the CTA walks the union once and
// does both FMAs per element; tile order alternates direction every step so that what is
// left in L1 from the previous step is hit first.
//
// What it costs: dynamic range.  A row is rescaled so that its maximum sits near 2^37..2^64;
// anything below 2^-126 (2^-149 with denormals) in those units is flushed.  Sentences that
// contain a finite link or an in-window match below 2^-120 are sent to the exact kernel up
// front (their exp() would flush by itself), so what can be lost is a quantity below 2^-150
// of its row's maximum, and the likelihood mass it could carry is bounded by
//     2^-150 * max_j alpha_t[j] * max_j betahat_t[j]      (betahat = beta without match)
// dag_fast_check_kernel evaluates R_t = log2(max alpha_t * max betahat_t / Z) for every
// step from the row maxima the sweep leaves behind and flags the sentence unless every
// R_t <= 100 and Z is finite; flagged sentences are recomputed by the exact log-domain
// kernel (dag_sweep_kernel with a selection mask) in the same call.  On the flagged=0 path
// the relative mass lost is below 2^-50 * (T*L^2) < 2^-26 -- far inside the 1e-5 tolerance.
//
// The rows are stored exactly like the log-domain sweep stores them (log2 values plus fp64
// row offsets), so the backward kernels do not care which path produced them.
#include <mutex>

#include "dag_tiles.cuh"

namespace dat {

constexpr int kFastThreads = 512;
constexpr int kFastWarps = kFastThreads / 32;
constexpr int kTargetExp = 64;   // rows are rescaled with 2^-(floor(log2 max) - kTargetExp)
constexpr float kMaxSpread = 100.f;        // row-wide spread (bits) a sentence may have when the flush is row-relative
constexpr float kMaxSpreadLocal = 140.f;   // spread inside a 32-vertex sub-strip (the flush there is 2^-190 relative)
constexpr float kMaxSpreadBackward = 200.f;   // row-wide spread up to which grad_links may use the product form
constexpr float kMinLog2Input = -120.f;  // finite links / matches below this go to the exact kernel
// The tiled sweep scales a whole row by one power of two, and the row-wide spread it may have (kMaxSpread)
// is used up by the length of the target alone: on diffuse graphs the spread grows by about 0.75 bits per
// target step (132 steps: 96 bits, 255 steps: 190-200 bits; peaky graphs need more), so a sentence with more
// steps than this is not swept at all but handed to the exact kernels up front, which would redo it anyway.
constexpr int kTiledMaxSteps = 128;
// Per-sentence word in the scratch.  The sweeps OR in what they saw; dag_fast_check_kernel turns it
// into the verdict the later launches read.
constexpr int kFlagTiny = 1;            // in: a finite link or in-window match below 2^kMinLog2Input
constexpr int kFlagHole = 4;            // in: two vertices of the graph without a (finite) link between them
constexpr int kFlagRedo = 1;            // out: forward and backward by the exact log-domain kernels
constexpr int kFlagExactBackward = 2;   // out: forward kept, grad_links by the exact kernel
constexpr int kFlagBits = 0xffff;        // the kFlag* bits of a sentence's word
constexpr int kFlagArrival = 1 << 16;    // above them: how many strip-sweep CTAs of the sentence have finished

}  // namespace dat
#include "dag_strip.cuh"
namespace dat {

__host__ __device__ inline int fast_pitch(int L) { return (L + 127) & ~127; }
__host__ __device__ inline int fast_rows(int L) { return (L + 15) & ~15; }

struct FastScratch {
    float *esq;   // [B][rows][pitch]   E = exp(links), square layout, zero padded (tiled path only)
    float *chk;   // [B][2][T]          log2 row maxima: alpha rows, betahat rows
    float *sub;   // [B][2][T][nH]      the same per 32-vertex sub-strip (strip path only)
    int *flag;    // [B]                kFlag* bits, then the verdict
    int *order;   // [B]                sentences sorted by decreasing cost
    float *hk;    // [B][T + 32]        backward: half the log2 scale of the step's factor product
    int4 *sel;    // [B]                backward: snapshot of the verdicts (and lengths) the product-form kernel works from
};

__host__ __device__ inline int strip_row_pitch_hd(int prelen) { return ((prelen + 63) & ~63) + 4; }
__host__ __device__ inline int fast_sub_strips(int L) { return strip_row_pitch_hd(L) / 32; }


// the square matrix comes last so that a caller that does not need it (strip sweep) can leave it out
__host__ __device__ inline size_t fast_scratch_bytes(int B, int T, int L, bool with_esq) {
    size_t e = with_esq ? (size_t)B * fast_rows(L) * fast_pitch(L) * sizeof(float) : 0;
    size_t c = (size_t)B * 2 * T * sizeof(float);
    size_t f = (size_t)B * sizeof(int) * 2;
    size_t u = (size_t)B * 2 * T * fast_sub_strips(L) * sizeof(float);
    size_t h = (((size_t)B * (T + 32) * sizeof(float) + 15) & ~(size_t)15) + (size_t)B * sizeof(int4);
    return ((e + 255) & ~(size_t)255) + ((c + 255) & ~(size_t)255) + ((f + 255) & ~(size_t)255) +
           ((u + 255) & ~(size_t)255) + ((h + 255) & ~(size_t)255) + 256;
}

static inline FastScratch carve_fast(void *scratch, int B, int T, int L) {
    uintptr_t p = (reinterpret_cast<uintptr_t>(scratch) + 255) & ~(uintptr_t)255;
    FastScratch s;
    s.chk = reinterpret_cast<float *>(p);
    p += (((size_t)B * 2 * T * sizeof(float)) + 255) & ~(size_t)255;
    s.flag = reinterpret_cast<int *>(p);
    s.order = s.flag + B;
    p += (((size_t)B * sizeof(int) * 2) + 255) & ~(size_t)255;
    s.sub = reinterpret_cast<float *>(p);
    p += (((size_t)B * 2 * T * fast_sub_strips(L) * sizeof(float)) + 255) & ~(size_t)255;
    s.hk = reinterpret_cast<float *>(p);
    s.sel = reinterpret_cast<int4 *>(p + (((size_t)B * (T + 32) * sizeof(float) + 15) & ~(size_t)15));
    p += ((((size_t)B * (T + 32) * sizeof(float) + 15) & ~(size_t)15) + (size_t)B * sizeof(int4) + 255) & ~(size_t)255;
    s.esq = reinterpret_cast<float *>(p);   // only present (and only touched) on the tiled path
    return s;
}

// ---------------------------------------------------------------------------------------
// E = exp(links) in square layout.  One warp per row; reads the band row (contiguous),
// writes the square row with 128-bit stores.  Every entry of the [rows][pitch] matrix is
// written, so the previous contents of the scratch never matter.
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(256)
dag_fast_prep_kernel(const float *__restrict__ links, const int64_t *__restrict__ output_length,
                     const int64_t *__restrict__ target_length, float *__restrict__ esq_all,
                     int *__restrict__ flag, int T, int L, int K, int rows, int pitch) {
    const int b = blockIdx.y;
    const int i = blockIdx.x * 8 + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (i >= rows) return;
    const long long oll = output_length[b], tll = target_length[b];
    if (!lengths_valid(oll, tll, T, L) || tll > kTiledMaxSteps) return;  // the sweep never reads this sentence
    const int ol = (int)oll;
    const float *brow = links + ((size_t)b * L + (i < L ? i : 0)) * K;
    float4 *erow = reinterpret_cast<float4 *>(esq_all + ((size_t)b * rows + i) * pitch);
    bool tiny = false;
    for (int jv = lane; jv < pitch / 4; jv += 32) {
        float v[4];
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const int j = 4 * jv + k;
            const int d = j - i - 1;
            const bool ok = i < ol && j < ol && d >= 0 && d < K;
            const float l2 = ok ? __ldg(brow + d) * kLog2e : -INFINITY;
            tiny |= (l2 < kMinLog2Input) && (l2 > -INFINITY);
            v[k] = ex2(l2);
        }
        erow[jv] = make_float4(v[0], v[1], v[2], v[3]);
    }
    if (tiny) flag[b] = 1;  // benign race: every writer stores the same value
}

// Sentences sorted by decreasing cost (tl-1) * W^2, so the long ones start first and the
// tail of the grid is made of short ones.  One CTA; O(B^2 / 1024) per thread.
__global__ void __launch_bounds__(1024)
dag_fast_order_kernel(const int64_t *__restrict__ output_length, const int64_t *__restrict__ target_length,
                      int *__restrict__ order, int *__restrict__ flag, int B, int T, int L,
                      int do_order) {
    extern __shared__ float cost_s[];
    for (int b = threadIdx.x; b < B; b += blockDim.x) flag[b] = 0;
    if (!do_order) return;
    for (int b = threadIdx.x; b < B; b += blockDim.x) {
        const long long ol = output_length[b], tl = target_length[b];
        float c = 0.f;
        if (lengths_valid(ol, tl, T, L)) {
            const float W = (float)(ol - tl + 1);
            c = (float)(tl - 1) * W * W;
        }
        cost_s[b] = c;
    }
    __syncthreads();
    for (int b = threadIdx.x; b < B; b += blockDim.x) {
        const float c = cost_s[b];
        int rank = 0;
        for (int o = 0; o < B; o++) {
            const float co = cost_s[o];
            rank += (co > c) || (co == c && o < b);
        }
        order[rank] = b;
    }
}

// exact 2^e as a float, e clamped to the normal range
__device__ __forceinline__ float pow2i(int e) {
    e = e < -126 ? -126 : (e > 127 ? 127 : e);
    return __int_as_float((e + 127) << 23);
}

// floor(log2(x)) - kTargetExp for a positive normal x, 0 for anything else
__device__ __forceinline__ int row_shift(float mx) {
    const int bits = __float_as_int(mx);
    const int ex = (bits >> 23) & 0xff;
    if (!(mx > 0.f) || ex == 0 || ex == 255) return 0;
    return ex - 127 - kTargetExp;
}

// Sum the 8 per-lane values v[0..7] over the 32 lanes of the warp; afterwards every lane
// holds, in the return value, the total of v[(lane >> 2) & 7].
__device__ __forceinline__ float reduce8_transposed(const float (&v)[8], int lane) {
    float w4[4], w2[2], w1;
    {
        const bool hi = lane & 16;
#pragma unroll
        for (int q = 0; q < 4; q++) {
            const float send = hi ? v[q] : v[q + 4];
            const float keep = hi ? v[q + 4] : v[q];
            w4[q] = keep + __shfl_xor_sync(0xffffffffu, send, 16);
        }
    }
    {
        const bool hi = lane & 8;
#pragma unroll
        for (int q = 0; q < 2; q++) {
            const float send = hi ? w4[q] : w4[q + 2];
            const float keep = hi ? w4[q + 2] : w4[q];
            w2[q] = keep + __shfl_xor_sync(0xffffffffu, send, 8);
        }
    }
    {
        const bool hi = lane & 4;
        const float send = hi ? w2[0] : w2[1];
        const float keep = hi ? w2[1] : w2[0];
        w1 = keep + __shfl_xor_sync(0xffffffffu, send, 4);
    }
    w1 += __shfl_xor_sync(0xffffffffu, w1, 2);
    w1 += __shfl_xor_sync(0xffffffffu, w1, 1);
    return w1;
}

__global__ void __launch_bounds__(kFastThreads, 1)
dag_fast_sweep_kernel(const float *__restrict__ match_all, const float *__restrict__ esq_all,
                      const int64_t *__restrict__ output_length, const int64_t *__restrict__ target_length,
                      const int *__restrict__ order, float *__restrict__ alpha_all,
                      float *__restrict__ beta_all, double *__restrict__ offsets_all,
                      float *__restrict__ chk_all, int *__restrict__ flag, float *__restrict__ loss,
                      int32_t *__restrict__ status, int T, int L, int K, int rows, int pitch) {
    extern __shared__ __align__(16) float fsm[];
    __shared__ float wmax_a[2][kFastWarps], wmax_b[2][kFastWarps], wmax_bb[2][kFastWarps];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int b = order ? order[blockIdx.x] : blockIdx.x;
    const long long oll = output_length[b], tll = target_length[b];
    double *offs = offsets_all + (size_t)b * (2 * T + 2);
    if (!lengths_valid(oll, tll, T, L)) {
        if (tid == 0) {
            offs[2 * T] = -INFINITY;
            offs[2 * T + 1] = -INFINITY;
            loss[b] = -INFINITY;
            if (status) atomicOr(status, DAT_STATUS_BAD_LENGTH);
        }
        return;
    }
    const int ol = (int)oll, tl = (int)tll;
    if (tl > kTiledMaxSteps) {   // its row-wide spread would not pass the check: straight to the exact kernels
        if (tid == 0) atomicOr(flag + b, kFlagTiny);
        return;
    }
    const int W = ol - tl + 1;
    const int rp = pitch + 32;                // row buffers carry 32 floats of zero padding
    float *abuf0 = fsm, *abuf1 = fsm + rp, *bbuf0 = fsm + 2 * rp, *bbuf1 = fsm + 3 * rp;
    float *sa = fsm + 4 * rp, *sb = sa + pitch;
    const float *match = match_all + (size_t)b * T * L;
    const float *E = esq_all + (size_t)b * rows * pitch;
    float *alpha = alpha_all + (size_t)b * T * L;
    float *beta = beta_all + (size_t)b * T * L;
    float *chk_a = chk_all + (size_t)b * 2 * T, *chk_bb = chk_a + T;

    for (int x = tid; x < 4 * rp + 2 * pitch; x += kFastThreads) fsm[x] = 0.f;
    __syncthreads();
    float m00 = match[0] * kLog2e;
    float mll = match[(size_t)(tl - 1) * L + (ol - 1)] * kLog2e;
    const bool dead = !(m00 > -INFINITY && m00 < INFINITY && mll > -INFINITY && mll < INFINITY);
    if (dead) { m00 = 0.f; mll = 0.f; }       // everything stays 0; the check flags the sentence
    if (tid == 0) {
        abuf0[0] = dead ? 0.f : 1.f;
        (((tl - 1) & 1) ? bbuf1 : bbuf0)[ol - 1] = dead ? 0.f : 1.f;
        alpha[0] = dead ? -INFINITY : 0.f;
        beta[(size_t)(tl - 1) * L + (ol - 1)] = dead ? -INFINITY : 0.f;
        offs[0] = (double)m00;
        offs[T + tl - 1] = (double)mll;
    }
    if (tid < kFastWarps) {
        wmax_a[0][tid] = dead ? 0.f : 1.f;
        wmax_b[(tl - 1) & 1][tid] = dead ? 0.f : 1.f;
        wmax_bb[0][tid] = 0.f;
        wmax_bb[1][tid] = 0.f;
    }
    for (int c = 1 + tid; c < W; c += kFastThreads) alpha[c] = -INFINITY;
    for (int c = tid; c < W - 1; c += kFastThreads) beta[(size_t)(tl - 1) * L + (tl - 1) + c] = -INFINITY;
    double offa = (double)m00, offb = (double)mll, offb_prev = 0.0;  // thread 0 only
    __syncthreads();

    const int ncbmax = pitch >> 7;
    bool tiny = false;
    for (int k = 1; k < tl; k++) {
        const int ta = k, tb = tl - 1 - k;
        const float *a_prev = ((ta - 1) & 1) ? abuf1 : abuf0;
        float *a_cur = (ta & 1) ? abuf1 : abuf0;
        const float *b_next = ((tb + 1) & 1) ? bbuf1 : bbuf0;
        float *b_cur = (tb & 1) ? bbuf1 : bbuf0;

        // ---- row scales from the maxima of the rows computed one step ago
        const float mxa = warp_max(lane < kFastWarps ? wmax_a[(ta - 1) & 1][lane] : 0.f);
        const float mxb = warp_max(lane < kFastWarps ? wmax_b[(tb + 1) & 1][lane] : 0.f);
        const float mxbb = warp_max(lane < kFastWarps ? wmax_bb[(tb + 1) & 1][lane] : 0.f);
        const int sha = row_shift(mxa), shb = row_shift(mxb);
        if (tid == 0) {
            chk_a[ta - 1] = lg2(mxa) + (float)offa;
            if (k >= 2) chk_bb[tb + 1] = lg2(mxbb) + (float)offb_prev;
            offa += (double)sha;
            offs[ta] = offa;
            offb_prev = offb;
            offb += (double)shb;
            offs[T + tb] = offb;
        }

        // ---- fused tile phase over the union of the two live regions
        const int xa = ta - 1, xb = tb;                       // region x: rows [x, x+W-1], cols [x+1, x+W]
        const int xlo = xa < xb ? xa : xb, xhi = xa < xb ? xb : xa;
        const int rt_lo = xlo >> 4, rt_hi = (xhi + W - 1) >> 4;
        const int cb_lo = (xlo + 1) >> 7;
        int cb_hi = (xhi + W) >> 7;
        if (cb_hi > ncbmax - 1) cb_hi = ncbmax - 1;
        int total = 0;
        for (int cb = cb_lo; cb <= cb_hi; cb++) {
            int rf = 128 * cb - K; rf = rf > 0 ? (rf >> 4) : 0; rf = rf > rt_lo ? rf : rt_lo;
            int rl = 8 * cb + 7; rl = rl < rt_hi ? rl : rt_hi;
            total += rl >= rf ? rl - rf + 1 : 0;
        }
        const int my_lo = (warp * total) / kFastWarps, my_hi = ((warp + 1) * total) / kFastWarps;
        const bool reverse = k & 1;
        // match values of the entries this thread finalises, requested before the tile phase
        float mpa[2], mpb[2];
#pragma unroll
        for (int q = 0; q < 2; q++) {
            const int j = 128 * cb_lo + tid + q * kFastThreads, c = j - ta;
            mpa[q] = (c >= 0 && c < W) ? __ldg(match + (size_t)ta * L + j) : 0.f;
            const int i = 16 * rt_lo + tid + q * kFastThreads, r = i - tb;
            mpb[q] = (r >= 0 && r < W) ? __ldg(match + (size_t)tb * L + i) : 0.f;
        }
        int base = 0;
        for (int cbx = cb_lo; cbx <= cb_hi; cbx++) {
            // walk column blocks in the same direction as the rows so the whole order flips
            const int cb = reverse ? (cb_hi - (cbx - cb_lo)) : cbx;
            int rf = 128 * cb - K; rf = rf > 0 ? (rf >> 4) : 0; rf = rf > rt_lo ? rf : rt_lo;
            int rl = 8 * cb + 7; rl = rl < rt_hi ? rl : rt_hi;
            const int n = rl >= rf ? rl - rf + 1 : 0;
            int from = my_lo > base ? my_lo - base : 0;
            int to = my_hi < base + n ? my_hi - base : n;
            base += n;
            if (from >= to) continue;
            const int col = 128 * cb + 4 * lane;
            const float4 b4 = *reinterpret_cast<const float4 *>(b_next + col);
            float acc0 = 0.f, acc1 = 0.f, acc2 = 0.f, acc3 = 0.f;
            // does this column block meet the alpha / beta region at all (warp-uniform)
            const bool cols_a = (128 * cb + 127 >= xa + 1) && (128 * cb <= xa + W);
            const bool cols_b = (128 * cb + 127 >= xb + 1) && (128 * cb <= xb + W);
            for (int q = from; q < to; q++) {
                const int rt = reverse ? (rl - q) : (rf + q);
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    const int i0 = 16 * rt + 8 * h;
                    // a half-tile outside a sweep's region only multiplies zeros for that sweep
                    const bool live_a = cols_a && (i0 + 7 >= xa) && (i0 <= xa + W - 1);
                    const bool live_b = cols_b && (i0 + 7 >= xb) && (i0 <= xb + W - 1);
                    if (!live_a && !live_b) continue;
                    const float4 *ep = reinterpret_cast<const float4 *>(E + (size_t)i0 * pitch + col);
                    float4 e[8];
#pragma unroll
                    for (int r = 0; r < 8; r++) e[r] = __ldg(ep + (size_t)r * (pitch >> 2));
                    if (live_a) {
                        const float4 a0 = *reinterpret_cast<const float4 *>(a_prev + i0);
                        const float4 a1 = *reinterpret_cast<const float4 *>(a_prev + i0 + 4);
                        const float av[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
#pragma unroll
                        for (int r = 0; r < 8; r++) {
                            acc0 = fmaf(av[r], e[r].x, acc0);
                            acc1 = fmaf(av[r], e[r].y, acc1);
                            acc2 = fmaf(av[r], e[r].z, acc2);
                            acc3 = fmaf(av[r], e[r].w, acc3);
                        }
                    }
                    if (live_b) {
                        float rpart[8];
#pragma unroll
                        for (int r = 0; r < 8; r++)
                            rpart[r] = fmaf(e[r].w, b4.w, fmaf(e[r].z, b4.z, fmaf(e[r].y, b4.y, e[r].x * b4.x)));
                        const float tot = reduce8_transposed(rpart, lane);
                        if ((lane & 3) == 0) atomicAdd(sb + i0 + ((lane >> 2) & 7), tot);
                    }
                }
            }
            atomicAdd(sa + col, acc0);
            atomicAdd(sa + col + 1, acc1);
            atomicAdd(sa + col + 2, acc2);
            atomicAdd(sa + col + 3, acc3);
        }
        __syncthreads();

        // ---- finalisation: every accumulator touched this step is consumed and cleared
        const float sca = pow2i(-sha), scb = pow2i(-shb);
        float vmax_a = 0.f, vmax_b = 0.f, vmax_bb = 0.f;
        int fq = 0;
        for (int j = 128 * cb_lo + tid; j < 128 * (cb_hi + 1); j += kFastThreads, fq++) {
            const float s = sa[j];
            sa[j] = 0.f;
            const int c = j - ta;
            if (c >= 0 && c < W) {
                const float mt = fq == 0 ? mpa[0] : (fq == 1 ? mpa[1] : __ldg(match + (size_t)ta * L + j));
                const float m2 = mt * kLog2e;
                tiny |= (m2 < kMinLog2Input) && (m2 > -INFINITY);
                const float pm = ex2(m2);
                const float a = (s * sca) * pm;
                a_cur[j] = a;
                alpha[(size_t)ta * L + j] = lg2(a);
                vmax_a = fmaxf(vmax_a, a);
            }
        }
        fq = 0;
        for (int i = 16 * rt_lo + tid; i < 16 * (rt_hi + 1); i += kFastThreads, fq++) {
            const float s = sb[i];
            sb[i] = 0.f;
            const int r = i - tb;
            if (r >= 0 && r < W) {
                const float mt = fq == 0 ? mpb[0] : (fq == 1 ? mpb[1] : __ldg(match + (size_t)tb * L + i));
                const float m2 = mt * kLog2e;
                tiny |= (m2 < kMinLog2Input) && (m2 > -INFINITY);
                const float pm = ex2(m2);
                const float bv = (s * scb) * pm;
                b_cur[i] = bv;
                beta[(size_t)tb * L + i] = lg2(bv);
                vmax_b = fmaxf(vmax_b, bv);
                vmax_bb = fmaxf(vmax_bb, s);
            }
        }
        if (tid == 0) {  // entries of the recycled row buffers that left the window
            a_cur[ta - 1] = 0.f;
            if (ta >= 2) a_cur[ta - 2] = 0.f;
            b_cur[tb + W] = 0.f;
            b_cur[tb + W + 1] = 0.f;
        }
        vmax_a = warp_max(vmax_a);
        vmax_b = warp_max(vmax_b);
        vmax_bb = warp_max(vmax_bb);
        if (lane == 0) {
            wmax_a[ta & 1][warp] = vmax_a;
            wmax_b[tb & 1][warp] = vmax_b;
            wmax_bb[tb & 1][warp] = vmax_bb;
        }
        __syncthreads();
    }
    if (tiny) flag[b] = 1;  // benign race: every writer stores the same value
    if (tid == 0) {
        const float al = (((tl - 1) & 1) ? abuf1 : abuf0)[ol - 1];
        const float be = bbuf0[0];
        const double z2a = (al > 0.f) ? (double)lg2(al) + offa : -INFINITY;
        const double z2b = (be > 0.f) ? (double)lg2(be) + offb : -INFINITY;
        offs[2 * T] = z2a;
        offs[2 * T + 1] = z2b;
        loss[b] = (float)(z2b * kLn2d);
        float mxbb = wmax_bb[0][0];
        for (int w = 1; w < kFastWarps; w++) mxbb = fmaxf(mxbb, wmax_bb[0][w]);
        chk_bb[0] = lg2(mxbb) + (float)offb_prev;
    }
}

// One small CTA per sentence: the verdict on what the probability-domain sweeps left behind.
// What they can lose is what underflowed in the unit it was added in.  Two bounds cover it:
//  * everything is within 2^-190 of the largest entry of its own 32-vertex sub-strip at that step
//    (rows, in-group sums), so with R_sub = max over (t, sub-strip) of
//        log2(max_{j in sub-strip} alpha_t[j] * max_{j in sub-strip} betahat_t[j] / Z) <= kMaxSpreadLocal
//    a lost quantity could have carried at most 2^(-190 + kMaxSpreadLocal) = 2^-50 of the likelihood;
//  * what finished vertex groups send forward is scaled to ONE unit per step, the largest entry of the
//    finished vertices.  An entry 2^-190 below that unit vanishes.  If every pair of vertices is
//    linked with a probability above 2^kMinLog2Input (no hole, nothing tiny), the largest finished
//    entry itself reaches every later vertex with at least 2^kMinLog2Input of its size, so what
//    vanished is below 2^(-190 - kMinLog2Input) = 2^-70 of what arrived.  With holes in the graph
//    that argument fails and the row-wide spread R_t = log2(max alpha_t * max betahat_t / Z) must
//    stay below kMaxSpread instead (the tiled sweep, whose rows have a single unit, always needs that).
// The product form of grad_links multiplies factors of size 2^(R_t / 2); beyond kMaxSpreadBackward its
// factors would underflow where they matter, so those sentences get the exact grad_links kernel.
constexpr int kCheckThreads = 128;
// The check of one sentence by all `nthreads` threads of a CTA (a multiple of 32, at most 512); every thread of
// the CTA must call it.  `bits`: the kFlag* bits the sweeps left.
__device__ __forceinline__ void fast_check_sentence(int b, int bits, const double *__restrict__ offsets_all,
                                                    const float *__restrict__ chk_all, const float *__restrict__ sub_all,
                                                    int nH, long long ol, long long tl, int *__restrict__ flag,
                                                    int32_t *__restrict__ status, int T, int tid, int nthreads) {
    __shared__ float row_s[16];
    if (bits & kFlagTiny) {  // set by the prep or a sweep kernel: an input below 2^kMinLog2Input
        if (tid == 0) {
            flag[b] = kFlagRedo;
            if (status) atomicOr(status, DAT_STATUS_FAST_FALLBACK);
        }
        return;
    }
    const double *offs = offsets_all + (size_t)b * (2 * T + 2);
    const float *chk_a = chk_all + (size_t)b * 2 * T, *chk_bb = chk_a + T;
    const double z2a = __ldcg(offs + 2 * T), z2b = __ldcg(offs + 2 * T + 1);
    bool bad = !(z2a > -INFINITY && z2a < INFINITY && z2b > -INFINITY && z2b < INFINITY);
    if (!bad) bad = !(fabs(z2a - z2b) <= 1e-3 * (1.0 + fabs(z2b)));
    const float z2 = (float)z2b;
    float r_row = -INFINITY;
    for (int t = tid; t + 1 < (int)tl; t += nthreads) {
        const float r = __ldcg(chk_a + t) + __ldcg(chk_bb + t) - z2;
        if (!(r <= 1e30f)) bad = true;   // NaN / inf
        r_row = fmaxf(r_row, r);
    }
    r_row = warp_max(r_row);
    if ((tid & 31) == 0) row_s[tid >> 5] = r_row;
    const bool local = sub_all != nullptr && !(bits & kFlagHole);   // the sub-strip bound applies
    if (local) {
        const float *sa = sub_all + (size_t)b * 2 * T * nH, *sb = sa + (size_t)T * nH;
        const int nsub = ((int)ol + 31) >> 5;
        const int pairs = ((int)tl - 1) * nsub;
        for (int x = tid; x < pairs; x += nthreads) {
            const int t = x / nsub, h = x - t * nsub;
            const float a = __ldcg(sa + t * nH + h);
            if (!(a > -INFINITY)) continue;
            // vertices 32h .. 32h+31 are the reversed sweep's canonical vertices ol-1-32h-31 .. ol-1-32h
            int ulo = (int)ol - 32 - 32 * h, uhi = (int)ol - 1 - 32 * h;
            ulo = ulo > 0 ? ulo : 0;
            const float bb = fmaxf(__ldcg(sb + t * nH + (ulo >> 5)), __ldcg(sb + t * nH + (uhi >> 5)));
            if (!(a + bb - z2 <= kMaxSpreadLocal)) bad = true;
        }
    }
    bad = __syncthreads_or(bad);
    if (tid == 0) {
        r_row = row_s[0];
        for (int w = 1; w < nthreads / 32; w++) r_row = fmaxf(r_row, row_s[w]);
        if (!local) bad |= !(r_row <= kMaxSpread);
        int verdict = 0;
        if (bad) verdict = kFlagRedo;
        else if (!(r_row <= kMaxSpreadBackward)) verdict = kFlagExactBackward;
        flag[b] = verdict;
        if (verdict == kFlagRedo && status) atomicOr(status, DAT_STATUS_FAST_FALLBACK);
    }
}

// One CTA per sentence: the check after the tiled sweep (the strip sweep runs it itself, in the CTA of a
// sentence that finishes second).
__global__ void __launch_bounds__(kCheckThreads)
dag_fast_check_kernel(const double *__restrict__ offsets_all, const float *__restrict__ chk_all,
                                      const float *__restrict__ sub_all, int nH,
                                      const int64_t *__restrict__ output_length,
                                      const int64_t *__restrict__ target_length, int *__restrict__ flag,
                                      int32_t *__restrict__ status, int B, int T, int L) {
    const int b = blockIdx.x, tid = threadIdx.x;
    const long long ol = output_length[b], tl = target_length[b];
    if (!lengths_valid(ol, tl, T, L)) {
        if (tid == 0) flag[b] = 0;  // nothing to recompute: the loss is -inf by definition
        return;
    }
    const int bits = flag[b] & kFlagBits;
    __syncthreads();
    fast_check_sentence(b, bits, offsets_all, chk_all, sub_all, nH, ol, tl, flag, status, T, tid, kCheckThreads);
}

}  // namespace dat
#include "dag_cluster.cuh"
#include "dag_grad_umma.cuh"
namespace dat {

// count[0]: sentences the forward handed to the exact kernels; count[1]: sentences whose forward was
// kept but whose grad_links goes to the exact kernel
__global__ void dag_fast_flagged_kernel(const int *__restrict__ flag, int32_t *__restrict__ count, int B) {
    int n = 0, m = 0;
    for (int b = threadIdx.x; b < B; b += blockDim.x) {
        n += flag[b] == kFlagRedo;
        m += flag[b] == kFlagExactBackward;
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        n += __shfl_xor_sync(0xffffffffu, n, o);
        m += __shfl_xor_sync(0xffffffffu, m, o);
    }
    __shared__ int part[2][32];
    if ((threadIdx.x & 31) == 0) { part[0][threadIdx.x >> 5] = n; part[1][threadIdx.x >> 5] = m; }
    __syncthreads();
    if (threadIdx.x == 0) {
        int t = 0, u = 0;
        for (int w = 0; w < (int)(blockDim.x >> 5); w++) { t += part[0][w]; u += part[1][w]; }
        count[0] = t;
        count[1] = u;
    }
}

// defined in dag_sweep.cu
int launch_exact_sweeps(const float *match_all, const float *links, const int64_t *output_length,
                        const int64_t *target_length, const int *select, float *alpha, float *beta,
                        double *offsets, float *loss, int32_t *status, int bsz, int tarlen, int prelen,
                        int translen, int nsweep, cudaStream_t stream, const char *who);

// defined in dag_grad.cu
int launch_grad_match(const float *grad_output, const float *alpha, const float *beta,
                      const double *offsets, const float *match_all, const int64_t *output_length,
                      const int64_t *target_length, float *grad_match_all, int bsz, int tarlen,
                      int prelen, cudaStream_t st, const char *who);
int launch_exact_grad_links(const float *grad_output, const float *alpha, const float *beta,
                            const double *offsets, const float *links, const int64_t *output_length,
                            const int64_t *target_length, float *grad_links, const int *select, int bsz,
                            int tarlen, int prelen, int translen, cudaStream_t st, const char *who);

// The strip-ordered sweep keeps every row of a sentence in shared memory; when that fits it is the
// forward path, and the square exp(links) copy is only built by the backward pass that reads it.
// + 4: the tensor-core operand loads of 8 consecutive rows then hit distinct banks
static inline int strip_row_pitch(int prelen) { return strip_row_pitch_hd(prelen); }
static inline bool strip_applicable(int tarlen, int prelen, const DeviceInfo &di) {
    // all rows in shared memory, and the [128 x steps] accumulator of the tensor-core phase within the 512
    // columns of tensor memory
    return strip_step_pad(tarlen) <= 512 &&
           strip_smem_floats(tarlen, strip_row_pitch(prelen)) * sizeof(float) + 512 <= (size_t)di.max_smem_optin;
}

}  // namespace dat

extern "C" {

int dat_dag_loss_backward_fast(const float *grad_output, const float *alpha, const float *beta,
                               const double *offsets, const float *match_all, const float *links,
                               const int64_t *output_length, const int64_t *target_length,
                               float *grad_match_all, float *grad_links, const void *scratch, int bsz,
                               int tarlen, int prelen, int translen, void *stream) {
    using namespace dat;
    DAT_REQUIRE(bsz >= 0 && tarlen >= 1 && prelen >= 1 && translen >= 1, DAT_ERR_BAD_ARG,
                "dat_dag_loss_backward_fast: bad sizes bsz=%d tarlen=%d prelen=%d translen=%d", bsz,
                tarlen, prelen, translen);
    if (bsz == 0) return DAT_OK;
    DAT_REQUIRE(grad_output && alpha && beta && offsets && match_all && links && output_length &&
                    target_length && grad_match_all && grad_links && scratch,
                DAT_ERR_BAD_ARG, "dat_dag_loss_backward_fast: null pointer");
    DAT_REQUIRE(bsz <= 65535 && tarlen <= 8192, DAT_ERR_UNSUPPORTED,
                "dat_dag_loss_backward_fast: bsz is limited to 65535 and tarlen to 8192");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const FastScratch sc = carve_fast(const_cast<void *>(scratch), bsz, tarlen, prelen);
    DeviceInfo di;
    if (!device_info(&di)) return DAT_ERR_NO_DEVICE;
    // grad_match rides in the prep kernel of grad_links when its tensors allow 128-bit accesses
    const bool match_vec = (prelen & 3) == 0 &&
                           ((reinterpret_cast<uintptr_t>(alpha) | reinterpret_cast<uintptr_t>(beta) |
                             reinterpret_cast<uintptr_t>(match_all) | reinterpret_cast<uintptr_t>(grad_match_all)) & 15) == 0;
    {
        // grad_links, product form on the tensor cores, for the sentences whose forward passed the check
        if (cudaFuncSetAttribute(dag_grad_links_umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)kGuSmemBytes) != cudaSuccess)
            return check_launch("dat_dag_loss_backward_fast(attr)");
        const int nC = gu_classes(prelen, translen), nJw = ((kGuTile - 1 + translen) / kGuTile) + 1;
        DAT_REQUIRE((long long)bsz * nC < (1ll << 30), DAT_ERR_UNSUPPORTED,
                    "dat_dag_loss_backward_fast: too many tiles (bsz=%d, prelen=%d)", bsz, prelen);
        const int ntiles = bsz * nC;
        const int grid = ntiles < di.sm_count ? ntiles : di.sm_count;
        if (!match_vec)
            if (int rc = launch_grad_match(grad_output, alpha, beta, offsets, match_all, output_length,
                                           target_length, grad_match_all, bsz, tarlen, prelen, st,
                                           "dat_dag_loss_backward_fast(grad_match)"))
                return rc;
        dag_grad_links_prep_kernel<<<dim3((tarlen + kGmSteps - 1) / kGmSteps, bsz), 256, 0, st>>>(
            grad_output, alpha, beta, offsets, match_all, sc.flag, output_length, target_length, grad_match_all,
            sc.hk, sc.sel, grad_links, tarlen, prelen, translen, match_vec ? 1 : 0);
        if (int rc = check_launch("dat_dag_loss_backward_fast(prep)")) return rc;
        dag_grad_links_umma_kernel<<<grid, kGuThreads, kGuSmemBytes, st>>>(
            alpha, beta, sc.hk, links, sc.sel, sc.flag, grad_links, tarlen, prelen, translen, nC, nJw,
            ntiles);
        if (int rc = check_launch("dat_dag_loss_backward_fast(grad_links)")) return rc;
    }
    // sentences the forward handed to the exact kernels get the exact backward as well
    return launch_exact_grad_links(grad_output, alpha, beta, offsets, links, output_length,
                                   target_length, grad_links, sc.flag, bsz, tarlen, prelen, translen, st,
                                   "dat_dag_loss_backward_fast(exact)");
}

int dat_dag_loss_fast_flagged(const void *scratch, int32_t *count, int bsz, int tarlen, int prelen,
                              void *stream) {
    using namespace dat;
    DAT_REQUIRE(scratch && count && bsz >= 1 && tarlen >= 1 && prelen >= 1, DAT_ERR_BAD_ARG,
                "dat_dag_loss_fast_flagged: bad argument");
    const FastScratch sc = carve_fast(const_cast<void *>(scratch), bsz, tarlen, prelen);
    dag_fast_flagged_kernel<<<1, 256, 0, static_cast<cudaStream_t>(stream)>>>(sc.flag, count, bsz);
    return check_launch("dat_dag_loss_fast_flagged");
}

size_t dat_dag_loss_fast_scratch_bytes(int bsz, int tarlen, int prelen) {
    if (bsz <= 0 || tarlen <= 0 || prelen <= 0) return 0;
    // the square exp(links) matrix is only needed when the tiled sweep runs on the current device
    dat::DeviceInfo di;
    const bool with_esq = !dat::device_info(&di) || !dat::strip_applicable(tarlen, prelen, di);
    return dat::fast_scratch_bytes(bsz, tarlen, prelen, with_esq);
}

int dat_dag_loss_fast(const float *match_all, const float *links, const int64_t *output_length,
                      const int64_t *target_length, float *alpha, float *beta, double *offsets,
                      float *loss, int32_t *status, void *scratch, int bsz, int tarlen, int prelen,
                      int translen, void *stream) {
    using namespace dat;
    DAT_REQUIRE(bsz >= 0 && tarlen >= 1 && prelen >= 1 && translen >= 1, DAT_ERR_BAD_ARG,
                "dat_dag_loss_fast: bad sizes bsz=%d tarlen=%d prelen=%d translen=%d", bsz, tarlen,
                prelen, translen);
    if (bsz == 0) return DAT_OK;
    DAT_REQUIRE(match_all && links && output_length && target_length && alpha && beta && offsets &&
                    loss && scratch,
                DAT_ERR_BAD_ARG, "dat_dag_loss_fast: null pointer");
    DAT_REQUIRE(prelen <= kMaxPrelen, DAT_ERR_UNSUPPORTED,
                "dat_dag_loss_fast: prelen=%d exceeds %d", prelen, kMaxPrelen);
    DAT_REQUIRE(tarlen <= kMaxTarlenGrad, DAT_ERR_UNSUPPORTED,
                "dat_dag_loss_fast: tarlen=%d exceeds %d (limit of the backward)", tarlen, kMaxTarlenGrad);
    DeviceInfo di;
    if (!device_info(&di)) return DAT_ERR_NO_DEVICE;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int rows = fast_rows(prelen), pitch = fast_pitch(prelen);
    const FastScratch sc = carve_fast(scratch, bsz, tarlen, prelen);

    // clears the per-sentence flags and (for batches it can rank in one CTA) sorts by cost
    const int do_order = bsz <= 8192;
    dag_fast_order_kernel<<<1, 1024, do_order ? (size_t)bsz * sizeof(float) : 0, st>>>(
        output_length, target_length, sc.order, sc.flag, bsz, tarlen, prelen, do_order);
    if (int rc = check_launch("dat_dag_loss_fast(order)")) return rc;
    const int *order = do_order ? sc.order : nullptr;
    const int strip_rp = strip_row_pitch(prelen);
    const size_t strip_smem = strip_smem_floats(tarlen, strip_rp) * sizeof(float);
    // Rows that do not fit in shared memory: a cluster of 4, 8 or 16 CTAs per direction, if the sentence's blocks
    // of exp(links) fit its registers and the device can co-schedule such a cluster
    int cl_ranks = 0;
    cudaLaunchConfig_t ccfg = {};
    cudaLaunchAttribute cattr[1];
    const size_t csmem = cluster_smem_bytes(prelen);
    if (!strip_applicable(tarlen, prelen, di)) {
        for (int r = 4; r <= kClMaxRanks && !cl_ranks; r *= 2)
            if (cluster_fits(prelen, r)) cl_ranks = r;
        if (cl_ranks) {
            bool ok = csmem <= (size_t)di.max_smem_optin;
            if (ok && csmem > 48 * 1024)
                ok = cudaFuncSetAttribute(dag_cluster_sweep_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                          (int)csmem) == cudaSuccess;
            if (ok && cl_ranks > 8)
                ok = cudaFuncSetAttribute(dag_cluster_sweep_kernel, cudaFuncAttributeNonPortableClusterSizeAllowed, 1) ==
                     cudaSuccess;
            ccfg.gridDim = dim3(2u * (unsigned)bsz * (unsigned)cl_ranks);
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
            if (ok) ok = cudaOccupancyMaxActiveClusters(&nclusters, dag_cluster_sweep_kernel, &ccfg) == cudaSuccess &&
                         nclusters >= 1;
            if (!ok) {
                cudaGetLastError();   // not an error of the call: the tiled sweep takes over
                cl_ranks = 0;
            }
        }
    }
    if (cl_ranks) {
        if (cudaLaunchKernelEx(&ccfg, dag_cluster_sweep_kernel, match_all, links, output_length, target_length, order,
                               alpha, beta, offsets, sc.chk, sc.sub, sc.flag, loss, status, tarlen, prelen, translen,
                               fast_sub_strips(prelen)) != cudaSuccess)
            return check_launch("dat_dag_loss_fast(cluster sweep)");
        if (int rc = check_launch("dat_dag_loss_fast(cluster sweep)")) return rc;
    } else if (strip_applicable(tarlen, prelen, di)) {
        // all rows of a sentence fit in shared memory: strip-ordered sweep, one CTA per direction
        if (cudaFuncSetAttribute(dag_strip_sweep_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)strip_smem) != cudaSuccess)
            return check_launch("dat_dag_loss_fast(attr)");
        dag_strip_sweep_kernel<<<2u * (unsigned)bsz, kStripThreads, strip_smem, st>>>(
            match_all, links, output_length, target_length, order, alpha, beta, offsets, sc.chk, sc.sub,
            sc.flag, loss, status, tarlen, prelen, translen, strip_rp);
        if (int rc = check_launch("dat_dag_loss_fast(strip sweep)")) return rc;
    } else {
        {
            dim3 grid((rows + 7) / 8, bsz);
            dag_fast_prep_kernel<<<grid, 256, 0, st>>>(links, output_length, target_length, sc.esq, sc.flag,
                                                       tarlen, prelen, translen, rows, pitch);
            if (int rc = check_launch("dat_dag_loss_fast(prep)")) return rc;
        }
        const size_t smem = (size_t)(4 * (pitch + 32) + 2 * pitch) * sizeof(float);
        DAT_REQUIRE(smem <= (size_t)di.max_smem_optin, DAT_ERR_UNSUPPORTED,
                    "dat_dag_loss_fast: prelen=%d needs %zu bytes of shared memory", prelen, smem);
        if (smem > 48 * 1024 &&
            cudaFuncSetAttribute(dag_fast_sweep_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)smem) != cudaSuccess)
            return check_launch("dat_dag_loss_fast(attr)");
        dag_fast_sweep_kernel<<<(unsigned)bsz, kFastThreads, smem, st>>>(
            match_all, sc.esq, output_length, target_length, order, alpha, beta, offsets, sc.chk, sc.flag,
            loss, status, tarlen, prelen, translen, rows, pitch);
        if (int rc = check_launch("dat_dag_loss_fast(sweep)")) return rc;
    }
    if (!strip_applicable(tarlen, prelen, di)) {   // (the strip sweep's CTAs run the check themselves)
        dag_fast_check_kernel<<<(unsigned)bsz, kCheckThreads, 0, st>>>(offsets, sc.chk, cl_ranks ? sc.sub : nullptr,
                                                                       fast_sub_strips(prelen),
                                                                       output_length, target_length, sc.flag, status, bsz,
                                                                       tarlen, prelen);
        if (int rc = check_launch("dat_dag_loss_fast(check)")) return rc;
    }
    // flagged sentences only; all other CTAs return at once
    return launch_exact_sweeps(match_all, links, output_length, target_length, sc.flag, alpha, beta,
                               offsets, loss, status, bsz, tarlen, prelen, translen, 2, st,
                               "dat_dag_loss_fast(exact)");
}

}  // extern "C"
