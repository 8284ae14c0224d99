// dag_loss forward: alpha and beta recursions of the DAG log-likelihood for sm_100a.
//
// Replaces calculate_alpha_kernel / calculate_beta_kernel and their host wrapper
// (fs_plugins/custom_ops/dag_loss.cu:40-140, 178-274, 313-375).
//
// One CTA owns one (sentence, sweep) pair; no CTA ever waits for another one.  All
// arithmetic is fp32 in the log2 domain.  Only the reachable window is computed: at
// target step t the live vertices are j in [t, t+W), W = output_length - target_length
// + 1 (a vertex left of the window cannot have emitted t tokens yet, a vertex right of
// it cannot reach the last vertex in time).  In window coordinates the work of every
// step is the same triangle  { (r, c) : 0 <= r <= c < W, c - r < K },
//   alpha:  i = t-1+r  ->  j = t+c     link = band[i][c-r]
//   beta :  i = t+r    ->  j = t+1+c   link = band[i][c-r]
// Rows are stored shifted by a per-row offset (fp64, `offsets`) so that the stored fp32
// values stay O(10) whatever the length of the sentence.
//
// Layout of `offsets` per sentence (2*T+2 doubles): [0,T) alpha row offsets, [T,2T) beta
// row offsets, [2T] log2-likelihood from the alpha sweep, [2T+1] from the beta sweep.
//
// The band of one sentence (<= 4 MB) is re-read at every target step and is served by
// L2; per term the inner loops issue one coalesced 4-byte load, a quarter of a 128-bit
// shared-memory broadcast, one FFMA, one FMNMX, two FADD and one MUFU.EX2.
#include <mutex>

#include "dag_tiles.cuh"

namespace dat {

// One chunk of kChunk rows for 32 columns: online log-sum-exp update of (m, s).
__device__ __forceinline__ void lse_chunk(float &m, float &s, const float (&x)[kChunk]) {
    float cm = x[0];
#pragma unroll
    for (int u = 1; u < kChunk; u++) cm = fmaxf(cm, x[u]);
    if (cm > m) {
        s *= ex2(m - cm);
        m = cm;
    }
    float acc = 0.f;
#pragma unroll
    for (int u = 0; u < kChunk; u++) acc += ex2(x[u] - m);
    s += acc;
}

// ---------------------------------------------------------------------------------
// alpha sweep
// ---------------------------------------------------------------------------------
__device__ void alpha_sweep(const float *__restrict__ match, const float *__restrict__ band,
                            float *__restrict__ alpha, double *__restrict__ offs, float *loss_out,
                            int ol, int tl, int T, int L, int K, unsigned char *raw) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int W = ol - tl + 1;
    const SweepSmem sm = carve(raw, L);
    const int pitch = sweep_row_pitch(L);
    __shared__ double off_s;
    __shared__ float delta_s;

    for (int x = tid; x < 2 * pitch; x += kSweepThreads) sm.row0[x] = -INFINITY;  // row0 and row1
    int my_lo, my_hi, cb_first;
    build_tile_plan(sm, W, K, my_lo, my_hi, cb_first);
    // warps without tiles sit between the first and last warp of a shared column block:
    // their merge slots must read as empty
#pragma unroll
    for (int which = 0; which < 2; which++) {
        float *p = sm.part + ((which * kSweepWarps + warp) * 2) * 32;
        p[lane] = kNegBig;
        p[32 + lane] = 0.f;
    }
    const float m00 = match[0] * kLog2e;
    if (tid == 0) {
        sm.row0[0] = m00;
        alpha[0] = m00;
        offs[0] = 0.0;
        off_s = 0.0;
        for (int w = 0; w < kSweepWarps; w++) sm.wmax[w] = m00;  // row 0 has the single entry
    }
    // the rest of row 0 inside the window is unreachable
    for (int c = 1 + tid; c < W; c += kSweepThreads) alpha[c] = -INFINITY;
    __syncthreads();

    const unsigned stride = (unsigned)(K - 1);
    for (int t = 1; t < tl; t++) {
        const float *prev = (t & 1) ? sm.row0 : sm.row1;  // row of step t-1
        float *cur = (t & 1) ? sm.row1 : sm.row0;
        // match of this thread's merge columns, requested early
        float mt[kMergeCols];
#pragma unroll
        for (int q = 0; q < kMergeCols; q++) {
            int c = tid + q * kSweepThreads;
            mt[q] = (c < W) ? ld_early(match + (size_t)t * L + t + c) : 0.f;
        }
        if (tid == 0) {
            const float *wm = sm.wmax + ((t - 1) & 1) * kSweepWarps;
            float d = wm[0];
            for (int w = 1; w < kSweepWarps; w++) d = fmaxf(d, wm[w]);
            if (!(d > 0.5f * kNegBig)) d = 0.f;  // dead row
            delta_s = d;
            off_s += (double)d;
            offs[t] = off_s;
        }

        // ---- tile phase
        if (my_lo < my_hi) {
            int cb = cb_first;
            int rb = sm.rb_lo[cb] + (my_lo - sm.tile_start[cb]);
            bool owns_start = (my_lo == sm.tile_start[cb]);
            float m = kNegBig, s = 0.f;
            const unsigned row_base = (unsigned)(t - 1) * (unsigned)K;
            for (int tile = my_lo; tile < my_hi;) {
                const TileGeom g = tile_geom(cb, rb, lane, W, K);
                // element (r, c) sits at band[(t-1+r)*K + (c-r)] = band[row_base + c + r*(K-1)]
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
                        for (int u = 0; u < kChunk; u++) x[u] = fmaf(x[u], kLog2e, pa[u]);
                        lse_chunk(m, s, x);
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
                            x[u] = fmaf(lk, kLog2e, prev[rr]);  // rows past the window read the -inf padding
                        }
                        lse_chunk(m, s, x);
                    }
                }
                tile++;
                rb++;
                if (rb > cb || tile == my_hi) {
                    const bool complete = owns_start && (rb > cb);
                    if (complete) {
                        if (g.c < W) { sm.fin_m[g.c] = m; sm.fin_s[g.c] = s; }
                    } else {
                        const int which = (cb == cb_first) ? 0 : 1;
                        float *p = sm.part + ((which * kSweepWarps + warp) * 2) * 32;
                        p[lane] = m;
                        p[32 + lane] = s;
                    }
                    cb++;
                    rb = sm.rb_lo[cb];
                    owns_start = true;
                    m = kNegBig;
                    s = 0.f;
                }
            }
        }
        __syncthreads();

        // ---- merge phase: one thread per window column
        const float delta = delta_s;
        float vmax = kNegBig;
#pragma unroll
        for (int q = 0; q < kMergeCols; q++) {
            const int c = tid + q * kSweepThreads;
            if (c < W) {
                const int cb = c >> 5, ln = c & 31;
                const int wa = sm.first_warp[cb], wb = sm.last_warp[cb];
                float m, s;
                if (wa == wb) {
                    m = sm.fin_m[c];
                    s = sm.fin_s[c];
                } else {
                    m = kNegBig;
                    s = 0.f;
                    for (int w = wa; w <= wb; w++) {
                        const int which = (sm.cb_first_of[w] == cb) ? 0 : 1;
                        const float *p = sm.part + ((which * kSweepWarps + w) * 2) * 32;
                        lse_merge(m, s, p[ln], p[32 + ln]);
                    }
                }
                float u = -INFINITY;
                if (s > 0.f) u = (m + lg2(s) - delta) + mt[q] * kLog2e;
                if (!(u > -INFINITY)) u = -INFINITY;  // also catches a NaN from +inf match
                cur[c] = u;
                alpha[(size_t)t * L + t + c] = u;
                vmax = fmaxf(vmax, u);
            }
        }
        vmax = warp_max(vmax);
        if (lane == 0) sm.wmax[(t & 1) * kSweepWarps + warp] = vmax;
        __syncthreads();
    }
    if (tid == 0) {
        const float *last = ((tl - 1) & 1) ? sm.row1 : sm.row0;
        float u = last[W - 1];
        double z2 = (u > -INFINITY) ? (double)u + off_s : -INFINITY;
        offs[2 * T] = z2;
        if (loss_out) *loss_out = (float)(z2 * kLn2d);
    }
}

// ---------------------------------------------------------------------------------
// beta sweep: one warp per window row, lanes along the band row (coalesced), per-lane
// online accumulators reduced once per row
// ---------------------------------------------------------------------------------
template <int NS, bool kMasked>
__device__ __forceinline__ void beta_chunk(const float *__restrict__ brow, const float *next_c, int e0,
                                           int len, int lane, float &m, float &s) {
    float x[NS];
#pragma unroll
    for (int u = 0; u < NS; u++) {
        const int e = e0 + u * 32 + lane;
        if (kMasked) {
            const bool ok = e < len;
            const float lk = ok ? __ldg(brow + e) : -INFINITY;
            x[u] = fmaf(lk, kLog2e, next_c[ok ? e : 0]);
        } else {
            x[u] = fmaf(__ldg(brow + e), kLog2e, next_c[e]);
        }
    }
    float cm = x[0];
#pragma unroll
    for (int u = 1; u < NS; u++) cm = fmaxf(cm, x[u]);
    if (cm > m) {
        s *= ex2(m - cm);
        m = cm;
    }
    float acc = 0.f;
#pragma unroll
    for (int u = 0; u < NS; u++) acc += ex2(x[u] - m);
    s += acc;
}

// log2-sum-exp2 over e in [0,len) of next_c[e] + brow[e]*log2(e); returns (m, s) reduced
// over the warp.
__device__ __forceinline__ void beta_row(const float *__restrict__ brow, const float *next_c, int len,
                                         int lane, float &m, float &s) {
    m = kNegBig;
    s = 0.f;
    int e0 = 0;
    for (; e0 + 256 <= len; e0 += 256) beta_chunk<8, false>(brow, next_c, e0, len, lane, m, s);
    const int rem = len - e0;
    if (rem > 128) beta_chunk<8, true>(brow, next_c, e0, len, lane, m, s);
    else if (rem > 64) beta_chunk<4, true>(brow, next_c, e0, len, lane, m, s);
    else if (rem > 32) beta_chunk<2, true>(brow, next_c, e0, len, lane, m, s);
    else if (rem > 0) beta_chunk<1, true>(brow, next_c, e0, len, lane, m, s);
    const float M = warp_max(m);
    s = warp_sum(s * ex2(m - M));
    m = M;
}

__device__ void beta_sweep(const float *__restrict__ match, const float *__restrict__ band,
                           float *__restrict__ beta, double *__restrict__ offs, float *loss_out,
                           int ol, int tl, int T, int L, int K, unsigned char *raw) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int W = ol - tl + 1;
    const SweepSmem sm = carve(raw, L);
    const int pitch = sweep_row_pitch(L);
    double *offb = offs + T;

    for (int x = tid; x < 2 * pitch; x += kSweepThreads) sm.row0[x] = -INFINITY;
    __syncthreads();
    float mll = match[(size_t)(tl - 1) * L + (ol - 1)] * kLog2e;
    if (!(mll > -INFINITY)) mll = -INFINITY;
    if (tid == 0) {
        float *last = ((tl - 1) & 1) ? sm.row1 : sm.row0;
        last[W - 1] = mll;
        beta[(size_t)(tl - 1) * L + (ol - 1)] = mll;
        offb[tl - 1] = 0.0;
        for (int w = 0; w < kSweepWarps; w++) sm.wmax[((tl - 1) & 1) * kSweepWarps + w] = mll;
    }
    // the rest of row tl-1 inside the window is unreachable
    for (int c = tid; c < W - 1; c += kSweepThreads) beta[(size_t)(tl - 1) * L + (tl - 1) + c] = -INFINITY;
    double off = 0.0;  // thread 0 only
    __syncthreads();

    for (int t = tl - 2; t >= 0; t--) {
        const float *next = ((t + 1) & 1) ? sm.row1 : sm.row0;
        float *cur = (t & 1) ? sm.row1 : sm.row0;
        float delta;
        {
            float d = (lane < kSweepWarps) ? sm.wmax[((t + 1) & 1) * kSweepWarps + lane] : kNegBig;
            d = warp_max(d);
            if (!(d > 0.5f * kNegBig)) d = 0.f;
            delta = d;
        }
        if (tid == 0) {
            off += (double)delta;
            offb[t] = off;
        }
        float vmax = kNegBig;
        // rows are dealt in snake order (w, 31-w, 32+w, 63-w, ...) so that every warp gets
        // the same mix of long and short rows
        for (int p = 0; p < ((W + 31) >> 5) * 2; p++) {
            const int r = (p >> 1) * 32 + ((p & 1) ? (31 - warp) : warp);
            if (r >= W) continue;
            const int i = t + r;
            int len = W - r;
            len = len < K ? len : K;
            const float mt = (lane == 0) ? __ldg(match + (size_t)t * L + i) : 0.f;
            float m, s;
            beta_row(band + (size_t)i * K, next + r, len, lane, m, s);
            if (lane == 0) {
                float u = -INFINITY;
                if (s > 0.f) u = (m + lg2(s) - delta) + mt * kLog2e;
                if (!(u > -INFINITY)) u = -INFINITY;
                cur[r] = u;
                beta[(size_t)t * L + i] = u;
                vmax = fmaxf(vmax, u);
            }
        }
        if (lane == 0) sm.wmax[(t & 1) * kSweepWarps + warp] = vmax;
        __syncthreads();
    }
    if (tid == 0) {
        float u = sm.row0[0];
        double z2 = (u > -INFINITY) ? (double)u + off : -INFINITY;
        offs[2 * T + 1] = z2;
        if (loss_out) *loss_out = (float)(z2 * kLn2d);
    }
}

__global__ void __launch_bounds__(kSweepThreads)
dag_sweep_kernel(const float *__restrict__ match, const float *__restrict__ links,
                 const int64_t *__restrict__ output_length, const int64_t *__restrict__ target_length,
                 float *__restrict__ alpha, float *__restrict__ beta, double *__restrict__ offsets,
                 float *__restrict__ loss, int32_t *__restrict__ status,
                 const int *__restrict__ select, int nsweep, int T, int L, int K) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int b = blockIdx.x / nsweep;
    const int sweep = blockIdx.x - b * nsweep;
    if (select != nullptr && select[b] != 1) return;  // only the sentences the fast path gave up on (verdict 1)
    const long long ol = output_length[b], tl = target_length[b];
    double *offs = offsets + (size_t)b * (2 * T + 2);
    if (!lengths_valid(ol, tl, T, L)) {
        if (threadIdx.x == 0) {
            offs[2 * T + sweep] = -INFINITY;
            if (sweep == nsweep - 1) loss[b] = -INFINITY;
            if (status) atomicOr(status, DAT_STATUS_BAD_LENGTH);
        }
        return;
    }
    const float *mb = match + (size_t)b * T * L;
    const float *lb = links + (size_t)b * L * K;
    if (sweep == 0) {
        alpha_sweep(mb, lb, alpha + (size_t)b * T * L, offs, nsweep == 1 ? loss + b : nullptr,
                    (int)ol, (int)tl, T, L, K, smem_raw);
    } else {
        beta_sweep(mb, lb, beta + (size_t)b * T * L, offs, loss + b, (int)ol, (int)tl, T, L, K,
                   smem_raw);
    }
}

// Launches the log-domain sweeps (nsweep = 1: alpha only, 2: alpha and beta).  With a
// selection mask only the sentences whose entry is non-zero are computed.
int launch_exact_sweeps(const float *match_all, const float *links, const int64_t *output_length,
                        const int64_t *target_length, const int *select, float *alpha, float *beta,
                        double *offsets, float *loss, int32_t *status, int bsz, int tarlen, int prelen,
                        int translen, int nsweep, cudaStream_t stream, const char *who) {
    DeviceInfo di;
    if (!device_info(&di)) return DAT_ERR_NO_DEVICE;
    const size_t smem = sweep_smem_bytes(prelen);
    DAT_REQUIRE(smem <= (size_t)di.max_smem_optin, DAT_ERR_UNSUPPORTED,
                "%s: prelen=%d needs %zu bytes of shared memory", who, prelen, smem);
    if (smem > 48 * 1024) {
        if (cudaFuncSetAttribute(dag_sweep_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)smem) != cudaSuccess)
            return check_launch(who);
    }
    dag_sweep_kernel<<<(unsigned)(bsz * nsweep), kSweepThreads, smem, stream>>>(
        match_all, links, output_length, target_length, alpha, beta, offsets, loss, status, select,
        nsweep, tarlen, prelen, translen);
    return check_launch(who);
}

}  // namespace dat

extern "C" {

size_t dat_dag_loss_offsets_bytes(int bsz, int tarlen) {
    if (bsz < 0 || tarlen < 0) return 0;
    return (size_t)bsz * (2 * (size_t)tarlen + 2) * sizeof(double);
}

int dat_dag_loss(const float *match_all, const float *links, const int64_t *output_length,
                 const int64_t *target_length, int require_gradient, float *alpha, float *beta,
                 double *offsets, float *loss, int32_t *status, int bsz, int tarlen, int prelen,
                 int translen, int config, void *stream) {
    using namespace dat;
    (void)config;
    DAT_REQUIRE(bsz >= 0 && tarlen >= 1 && prelen >= 1 && translen >= 1, DAT_ERR_BAD_ARG,
                "dat_dag_loss: bad sizes bsz=%d tarlen=%d prelen=%d translen=%d", bsz, tarlen,
                prelen, translen);
    if (bsz == 0) return DAT_OK;
    DAT_REQUIRE(match_all && links && output_length && target_length && alpha && offsets && loss,
                DAT_ERR_BAD_ARG, "dat_dag_loss: null pointer");
    DAT_REQUIRE(!require_gradient || beta, DAT_ERR_BAD_ARG,
                "dat_dag_loss: beta workspace required when require_gradient");
    DAT_REQUIRE(prelen <= kMaxPrelen, DAT_ERR_UNSUPPORTED,
                "dat_dag_loss: prelen=%d exceeds %d", prelen, kMaxPrelen);
    DAT_REQUIRE(!require_gradient || tarlen <= kMaxTarlenGrad, DAT_ERR_UNSUPPORTED,
                "dat_dag_loss: tarlen=%d exceeds %d (limit of the backward)", tarlen, kMaxTarlenGrad);
    DAT_REQUIRE((long long)prelen * translen < (1ll << 31), DAT_ERR_UNSUPPORTED,
                "dat_dag_loss: prelen*translen too large");
    return launch_exact_sweeps(match_all, links, output_length, target_length, nullptr, alpha, beta,
                               offsets, loss, status, bsz, tarlen, prelen, translen,
                               require_gradient ? 2 : 1, static_cast<cudaStream_t>(stream),
                               "dat_dag_loss");
}

}  // extern "C"

// ---------------------------------------------------------------------------------------
// Likelihood without any allocation by anybody: the recursion workspace lives in the
// library image.
// ---------------------------------------------------------------------------------------
namespace dat {

constexpr size_t kStaticRowFloats = (size_t)1 << 21;      // 8 MiB of recursion rows
constexpr size_t kStaticOffsetDoubles = (size_t)1 << 16;  // 512 KiB of row offsets

// One copy per GPU that loads the library, resident until the process exits.  In host code
// these names are only handles; the device addresses are fetched with cudaGetSymbolAddress.
static __device__ __align__(256) float g_static_rows[kStaticRowFloats];
static __device__ __align__(256) double g_static_offsets[kStaticOffsetDoubles];

struct StaticScratch {
    float *rows;
    double *offsets;
    bool ready;
};

// Device addresses of the static scratch for the CURRENT device (looked up once per device).
static int static_scratch(StaticScratch *out) {
    constexpr int kMaxDev = 64;
    static StaticScratch cache[kMaxDev] = {};
    static std::mutex mu;
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDev) {
        cudaGetLastError();
        set_error("dat_dag_loss_static: no current CUDA device");
        return DAT_ERR_NO_DEVICE;
    }
    std::lock_guard<std::mutex> lock(mu);
    if (!cache[dev].ready) {
        void *rows = nullptr, *offs = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&rows, g_static_rows);
        if (e == cudaSuccess) e = cudaGetSymbolAddress(&offs, g_static_offsets);
        if (e != cudaSuccess || !rows || !offs) {
            cudaGetLastError();
            set_error("dat_dag_loss_static: cudaGetSymbolAddress failed on device %d: %s", dev,
                      cudaGetErrorString(e));
            return DAT_ERR_LAUNCH;
        }
        cache[dev].rows = static_cast<float *>(rows);
        cache[dev].offsets = static_cast<double *>(offs);
        cache[dev].ready = true;
    }
    *out = cache[dev];
    return DAT_OK;
}

}  // namespace dat

extern "C" int dat_dag_loss_static(const float *match_all, const float *links,
                                   const int64_t *output_length, const int64_t *target_length,
                                   float *loss, int32_t *status, int bsz, int tarlen, int prelen,
                                   int translen, void *stream) {
    using namespace dat;
    DAT_REQUIRE(bsz >= 0 && tarlen >= 1 && prelen >= 1 && translen >= 1, DAT_ERR_BAD_ARG,
                "dat_dag_loss_static: bad sizes bsz=%d tarlen=%d prelen=%d translen=%d", bsz, tarlen,
                prelen, translen);
    if (bsz == 0) return DAT_OK;
    DAT_REQUIRE(match_all && links && output_length && target_length && loss, DAT_ERR_BAD_ARG,
                "dat_dag_loss_static: null pointer");
    const size_t need_rows = (size_t)bsz * tarlen * prelen;
    const size_t need_offs = (size_t)bsz * (2 * (size_t)tarlen + 2);
    DAT_REQUIRE(need_rows <= kStaticRowFloats && need_offs <= kStaticOffsetDoubles, DAT_ERR_UNSUPPORTED,
                "dat_dag_loss_static: bsz*tarlen*prelen = %zu exceeds the built-in workspace of %zu "
                "floats (or bsz*(2*tarlen+2) = %zu exceeds %zu); use dat_dag_loss with caller-provided "
                "workspaces for larger batches",
                need_rows, kStaticRowFloats, need_offs, kStaticOffsetDoubles);
    DAT_REQUIRE(prelen <= kMaxPrelen, DAT_ERR_UNSUPPORTED,
                "dat_dag_loss_static: prelen=%d exceeds %d", prelen, kMaxPrelen);
    DAT_REQUIRE((long long)prelen * translen < (1ll << 31), DAT_ERR_UNSUPPORTED,
                "dat_dag_loss_static: prelen*translen too large");
    DeviceInfo di;
    if (!device_info(&di)) return DAT_ERR_NO_DEVICE;
    StaticScratch sc;
    if (int rc = static_scratch(&sc)) return rc;
    const size_t smem = sweep_smem_bytes(prelen);
    DAT_REQUIRE(smem <= (size_t)di.max_smem_optin, DAT_ERR_UNSUPPORTED,
                "dat_dag_loss_static: prelen=%d needs %zu bytes of shared memory", prelen, smem);
    if (smem > 48 * 1024) {
        if (cudaFuncSetAttribute(dag_sweep_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                 (int)smem) != cudaSuccess)
            return check_launch("dat_dag_loss_static(attr)");
    }
    // alpha sweep only; every row it reads it has written in this launch, so nothing of the
    // previous call's contents has to be cleared
    dag_sweep_kernel<<<(unsigned)bsz, kSweepThreads, smem, static_cast<cudaStream_t>(stream)>>>(
        match_all, links, output_length, target_length, sc.rows, nullptr, sc.offsets, loss, status,
        /*select=*/nullptr, /*nsweep=*/1, tarlen, prelen, translen);
    return check_launch("dat_dag_loss_static");
}
