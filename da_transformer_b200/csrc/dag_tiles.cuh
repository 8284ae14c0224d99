// Work decomposition shared by the alpha sweep and the best-alignment sweep.
//
// In window coordinates (see dag_sweep.cu) every step reduces, for each column c, over the
// rows r of the triangle { 0 <= r <= c < W, c - r < K }.  The triangle is cut into tiles of
// 32 rows x 32 columns, enumerated column-block major, and the enumeration is split into
// contiguous ranges of (almost) equal length, one per warp.  A warp keeps one accumulator
// per lane (= column) while it walks the tiles of a column block; a column block shared by
// several warps is merged through shared memory.
//
// Recursion rows live in shared memory in WINDOW coordinates (entry r of the row of step t
// is vertex t + r), so the 4 / 8 consecutive rows a chunk needs are one or two aligned
// 128-bit broadcast loads.
#pragma once

#include "dat_common.cuh"

namespace dat {

constexpr int kSweepThreads = 512;
constexpr int kSweepWarps = kSweepThreads / 32;
constexpr int kChunk = 8;
// Window columns one thread of the alpha sweep finalises per step; bounds the graph length.
constexpr int kMergeCols = 4;
constexpr int kMaxPrelen = kMergeCols * kSweepThreads;   // 2048 vertices
// The exact grad_links kernel stages tarlen x 8 floats in shared memory (opt-in limit 227 KB).
constexpr int kMaxTarlenGrad = 7168;

__host__ __device__ inline bool lengths_valid(long long ol, long long tl, int T, int L) {
    return tl >= 2 && ol >= 2 && ol >= tl && ol <= L && tl <= T;
}

// Shared-memory carve-up (plain pointers: a struct indexed at run time would live in
// local memory).
struct SweepSmem {
    float *row0, *row1;  // recursion rows, window coordinates, padded with -inf
    float *fin_m;        // per window column: merged running max / sum
    float *fin_s;
    float *part;         // [2][warps][2][32] partial (m, s) of column blocks shared by warps
    float *wmax;         // [2][warps] per-warp maxima of the row just written
    int *rb_lo;          // [ncb+1] first row block of a column block (band limit)
    int *tile_start;     // [ncb+1] prefix sum of tiles per column block
    int *first_warp;     // [ncb]
    int *last_warp;      // [ncb]
    int *cb_first_of;    // [warps]
};

__host__ __device__ inline int sweep_row_pitch(int L) { return (L + 63) & ~31; }

__host__ __device__ inline size_t sweep_smem_bytes(int L) {
    int lp = sweep_row_pitch(L);
    int ncb = (L + 31) / 32 + 1;
    size_t f = (size_t)4 * lp + 2 * kSweepWarps * 2 * 32 + 2 * kSweepWarps;
    size_t i = (size_t)4 * ncb + 2 + kSweepWarps;
    return (f + i) * 4 + 64;
}

__device__ inline SweepSmem carve(unsigned char *raw, int L) {
    SweepSmem s;
    int lp = sweep_row_pitch(L);
    int ncb = (L + 31) / 32 + 1;
    float *f = reinterpret_cast<float *>(raw);
    s.row0 = f; f += lp;
    s.row1 = f; f += lp;
    s.fin_m = f; f += lp;
    s.fin_s = f; f += lp;
    s.part = f; f += 2 * kSweepWarps * 2 * 32;
    s.wmax = f; f += 2 * kSweepWarps;
    int *i = reinterpret_cast<int *>(f);
    s.rb_lo = i; i += ncb;
    s.tile_start = i; i += ncb + 1;
    s.first_warp = i; i += ncb;
    s.last_warp = i; i += ncb;
    s.cb_first_of = i;
    return s;
}

// Builds the tile plan in shared memory and returns this warp's tile range [my_lo, my_hi)
// and the column block its range starts in.  Contains two __syncthreads().
__device__ inline void build_tile_plan(const SweepSmem &sm, int W, int K, int &my_lo, int &my_hi,
                                       int &cb_first) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int ncb = (W + 31) >> 5;
    if (tid == 0) {
        int acc = 0;
        for (int cb = 0; cb < ncb; cb++) {
            int lo = 32 * cb + 1 - K;
            lo = lo > 0 ? (lo >> 5) : 0;
            sm.rb_lo[cb] = lo;
            sm.tile_start[cb] = acc;
            acc += cb - lo + 1;
        }
        sm.tile_start[ncb] = acc;
        sm.rb_lo[ncb] = 0;
    }
    __syncthreads();
    const int ntiles = sm.tile_start[ncb];
    my_lo = (int)(((long long)warp * ntiles) / kSweepWarps);
    my_hi = (int)(((long long)(warp + 1) * ntiles) / kSweepWarps);
    cb_first = 0;
    while (cb_first + 1 < ncb && sm.tile_start[cb_first + 1] <= my_lo) cb_first++;
    if (lane == 0) sm.cb_first_of[warp] = cb_first;
    if (tid < ncb) {
        int a = sm.tile_start[tid], b = sm.tile_start[tid + 1] - 1;
        int fw = 0, lw = 0;
        for (int w = 0; w < kSweepWarps; w++) {
            int lo = (int)(((long long)w * ntiles) / kSweepWarps);
            int hi = (int)(((long long)(w + 1) * ntiles) / kSweepWarps);
            if (a >= lo && a < hi) fw = w;
            if (b >= lo && b < hi) lw = w;
        }
        sm.first_warp[tid] = fw;
        sm.last_warp[tid] = lw;
    }
    __syncthreads();
}

// Geometry of one tile for one lane.
struct TileGeom {
    int c;        // window column of this lane
    int r0, r1;   // row range of the tile (r1 exclusive, clipped to the triangle)
    int rmin, rmax;  // valid rows of this lane (band limit, diagonal); rmax < rmin if none
    bool interior;   // every (row, lane) pair of the tile is a valid, in-bounds term
};

__device__ __forceinline__ TileGeom tile_geom(int cb, int rb, int lane, int W, int K) {
    TileGeom g;
    g.c = 32 * cb + lane;
    g.rmax = (g.c < W) ? g.c : -1;
    int rmin = g.c + 1 - K;
    g.rmin = rmin > 0 ? rmin : 0;
    g.r0 = 32 * rb;
    int cap = 32 * cb + 32;
    cap = cap < W ? cap : W;
    g.r1 = (g.r0 + 32 < cap) ? g.r0 + 32 : cap;
    // strictly below the diagonal block, the whole 32x32 square inside the band, and the
    // lanes past W (last column block) still address valid memory: c - r < K
    g.interior = (rb < cb) && (32 * cb + 31 - g.r0 < K);
    return g;
}

// grad_match_all[b, t, j] = g[b] * 2^(alpha2 + beta2 - match * log2e - Z2) for the steps t0 .. t0 + kGmSteps - 1
// of sentence b, zeros outside the window: called by all 256 threads of a CTA, four vertices per thread;
// rows must start on 16-byte boundaries (prelen a multiple of 4, aligned tensors).
constexpr int kGmSteps = 4;
__device__ __forceinline__ void grad_match_steps_vec(const float *__restrict__ grad_out, const float *__restrict__ alpha,
                                                     const float *__restrict__ beta, const double *__restrict__ offsets,
                                                     const float *__restrict__ match,
                                                     const int64_t *__restrict__ output_length,
                                                     const int64_t *__restrict__ target_length,
                                                     float *__restrict__ gmatch, int T, int L, int b, int t0) {
    const long long ol = output_length[b], tl = target_length[b];
    const double *offs = offsets + (size_t)b * (2 * T + 2);
    bool live = lengths_valid(ol, tl, T, L);
    double z2 = 0.0;
    if (live) {
        z2 = offs[2 * T + 1];
        live = z2 > -INFINITY && z2 < INFINITY;
    }
    const float g = live ? grad_out[b] : 0.f;
    const int W = (int)(ol - tl) + 1, nv = L >> 2;
    for (int x = threadIdx.x; x < kGmSteps * nv; x += 256) {
        const int r = x / nv, j = (x - r * nv) << 2, t = t0 + r;
        if (t >= T) break;
        const size_t at = ((size_t)b * T + t) * L + j;
        float4 out = make_float4(0.f, 0.f, 0.f, 0.f);
        if (live && t < tl && j + 3 >= t && j < t + W) {
            const float k = (float)(offs[t] + offs[T + t] - z2);
            const float4 a = __ldg(reinterpret_cast<const float4 *>(alpha + at));
            const float4 bb = __ldg(reinterpret_cast<const float4 *>(beta + at));
            const float4 m = __ldg(reinterpret_cast<const float4 *>(match + at));
            const float av[4] = {a.x, a.y, a.z, a.w}, bv[4] = {bb.x, bb.y, bb.z, bb.w}, mv[4] = {m.x, m.y, m.z, m.w};
            float o[4];
#pragma unroll
            for (int c = 0; c < 4; c++) {
                o[c] = 0.f;
                if (j + c >= t && j + c < t + W && mv[c] > -INFINITY && mv[c] < INFINITY) {
                    o[c] = g * ex2((av[c] + bv[c]) + fmaf(-mv[c], kLog2e, k));
                    if (!(o[c] == o[c])) o[c] = 0.f;
                }
            }
            out = make_float4(o[0], o[1], o[2], o[3]);
        }
        *reinterpret_cast<float4 *>(gmatch + at) = out;
    }
}

}  // namespace dat
