// grad_links in product form on the tensor cores (included by dag_fast.cu).
//
//     grad_links[i][j-i-1] = g * E[i][j] * sum_t A'[t][i] * B'[t][j],
//     A'[t][i] = 2^(u_a[t,i] + h_t),  B'[t][j] = 2^(u_b[t+1,j] + h_t),  h_t = (off_a[t] + off_b[t+1] - log2 Z) / 2
// is, per 128 x 128 tile of (i, j), the product of the [128 x steps] factor A'^T with the [steps x 128]
// factor B': M = i, N = j, K = target step.  One exp per stored factor entry instead of one per
// (t, i, j) term, and the multiply-adds on the tensor cores.  Only sentences that passed the forward's
// dynamic-range check take this path (A' * B' <= 2^100 there, so neither factor overflows and a factor
// that underflows belongs to a posterior below 2^-60); the others are left to the exact kernel.
//
// One persistent CTA per SM (a kernel that allocates tensor memory gets one CTA per SM), each with a
// contiguous range of the tiles, two groups of eight warps that only meet through mbarriers:
//   producers  exponentiate the factors on their way into shared memory (K-major core-matrix layout,
//     32 steps per chunk, two operand stages), each as a tf32 high part and the fp32 remainder; one
//     thread issues tcgen05.mma kind::tf32 (hi*hi + hi*lo + lo*hi: fp32-level accuracy) into one of two
//     [128 x 128] accumulators in tensor memory and commits to the stage's and the accumulator's barrier;
//   consumers  read a finished accumulator column by column (the product is formed transposed, M = j, so
//     that the accumulator's lanes, i.e. a warp's threads, run along j like the band's memory does),
//     multiply by g * exp(link) and store with coalesced accesses.  A tile's links wait in shared
//     memory: each thread copies the link of its next tile's entry asynchronously into the slot it has
//     just used up, so their latency is covered by a whole tile of work.
// Every band entry of a sentence that takes this path is written, zeros included: the tiles write the
// entries that are links of the sentence's graph, dag_grad_links_prep_kernel (which also prepares h_t and
// a snapshot of the per-sentence decisions) fills the rest of every band row with zeros beforehand.
// All waits are bounded.  A group whose wait gives up stops using the
// tensor core, tells the other group through shared memory, and the sentences that are then left
// incomplete are handed to the exact kernel (which runs after this one and rewrites all of their
// entries) through their flag; which sentences this kernel works on is read from a snapshot of the
// flags, so that both groups always agree on the tiles.
#pragma once

#include "umma.cuh"

namespace dat {

constexpr int kGuTile = 128;
constexpr int kGuGroup = 256;                        // threads per group
constexpr int kGuThreads = 2 * kGuGroup;
constexpr int kGuOperand = kGuTile * umma::kTileK;   // floats of one operand chunk (128 rows x 32 steps)
constexpr int kGuPolls = 1 << 20;
constexpr int kGuBatch = 8;   // entries a consumer thread works on together (16 and 32 were slower: 316 and 389 us against 259)
constexpr size_t kGuSmemBytes =
    (size_t)(2 * 4 * kGuOperand + kGuTile * kGuTile + 2 * kGuOperand) * sizeof(float) + 6 * sizeof(uint64_t) + 16;

// Before the product kernel, kGmSteps target steps and a share of the band rows of a sentence per CTA:
// grad_match of those steps (when the tensors allow the vector form; the caller launches the plain
// kernel otherwise), h_t of every step (zero past the last one, rows padded so that a 32-step chunk may
// read past T), the snapshot of the verdicts with what a tile needs to know about its sentence, and zeros
// in every band entry that is not a link of the graph (j >= ol; whole rows from ol - 1 on; everything when
// there is nothing to add up).  The zeros are pure stores and the gradient of the match mostly loads, so
// the two share the memory system better in one kernel than one after the other.
constexpr int kGuHkPad = umma::kTileK;
__global__ void __launch_bounds__(256)
dag_grad_links_prep_kernel(const float *__restrict__ grad_out, const float *__restrict__ alpha,
                           const float *__restrict__ beta, const double *__restrict__ offsets_all,
                           const float *__restrict__ match, const int *__restrict__ flag,
                           const int64_t *__restrict__ output_length, const int64_t *__restrict__ target_length,
                           float *__restrict__ gmatch, float *__restrict__ hk_all, int4 *__restrict__ sel,
                           float *__restrict__ glinks, int T, int L, int K, int with_match) {
    const int b = blockIdx.y;
    const long long oll = output_length[b], tll = target_length[b];
    const double *offs = offsets_all + (size_t)b * (2 * T + 2);
    const bool live = lengths_valid(oll, tll, T, L);
    const double z2 = live ? offs[2 * T + 1] : 0.0;
    const bool fin = live && z2 > -INFINITY && z2 < INFINITY;
    const int verdict = flag[b];
    if (blockIdx.x == 0) {
        for (int t = threadIdx.x; t < T + kGuHkPad; t += blockDim.x)
            hk_all[(size_t)b * (T + kGuHkPad) + t] =
                (fin && t <= tll - 2) ? 0.5f * (float)(offs[t] + offs[T + t + 1] - z2) : 0.f;
        // x = 0: the product kernel's sentence, 1: the exact kernel's, 2: nothing to add up; y, z: lengths;
        // w: the sentence's incoming gradient
        if (threadIdx.x == 0)
            sel[b] = make_int4(verdict != 0 ? 1 : (fin ? 0 : 2), fin ? (int)oll : 0, fin ? (int)tll : 0,
                               __float_as_int(grad_out[b]));
    }
    if (verdict == 0) {   // (the exact kernel writes every entry of the other sentences)
        const int ol = fin ? (int)oll : 0;
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
        const int per = (L + (int)gridDim.x - 1) / (int)gridDim.x;
        const int iend = per * ((int)blockIdx.x + 1) < L ? per * ((int)blockIdx.x + 1) : L;
        for (int i = per * (int)blockIdx.x + warp; i < iend; i += 8) {
            int d0 = ol - 1 - i;   // first entry that is not a link
            d0 = d0 < 0 ? 0 : d0;
            float *row = glinks + ((size_t)b * L + i) * K;
            // scalar head up to a 16-byte boundary, then 128-bit stores, then the scalar tail
            int d1 = d0 + (int)(((16u - (unsigned)(reinterpret_cast<uintptr_t>(row + d0) & 15u)) & 15u) >> 2);
            d1 = d1 < K ? d1 : K;
            for (int d = d0 + lane; d < d1; d += 32) row[d] = 0.f;
            const int nv = (K - d1) >> 2;
            float4 *rv = reinterpret_cast<float4 *>(row + d1);
            for (int q = lane; q < nv; q += 32) rv[q] = make_float4(0.f, 0.f, 0.f, 0.f);
            for (int d = d1 + 4 * nv + lane; d < K; d += 32) row[d] = 0.f;
        }
    }
    if (with_match)
        grad_match_steps_vec(grad_out, alpha, beta, offsets_all, match, output_length, target_length, gmatch, T, L, b,
                             (int)blockIdx.x * kGmSteps);
}

__device__ __forceinline__ void gu_split4(const float (&v)[4], float4 &hi, float4 &lo) {
    hi.x = __uint_as_float(__float_as_uint(v[0]) & 0xffffe000u);
    hi.y = __uint_as_float(__float_as_uint(v[1]) & 0xffffe000u);
    hi.z = __uint_as_float(__float_as_uint(v[2]) & 0xffffe000u);
    hi.w = __uint_as_float(__float_as_uint(v[3]) & 0xffffe000u);
    lo.x = v[0] - hi.x;
    lo.y = v[1] - hi.y;
    lo.z = v[2] - hi.z;
    lo.w = v[3] - hi.w;
}
// barrier of one group (ids 1 and 2; 0 is the CTA's), returning the OR of a predicate over the group
__device__ __forceinline__ bool gu_group_or(int id, bool p) {
    uint32_t r;
    asm volatile(
        "{\n\t.reg .pred a, b;\n\tsetp.ne.b32 a, %2, 0;\n\tbarrier.red.or.pred b, %1, %3, a;\n\tselp.u32 %0, 1, 0, b;\n\t}"
        : "=r"(r)
        : "r"(id), "r"((uint32_t)p), "r"(kGuGroup)
        : "memory");
    return r != 0u;
}
__device__ __forceinline__ void gu_mbar_arrive(uint64_t *mbar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(umma::smem_u32(mbar)) : "memory");
}
__device__ __forceinline__ void gu_cp_async4(uint32_t smem_dst, const float *gsrc) {
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(smem_dst), "l"(gsrc) : "memory");
}
__device__ __forceinline__ void gu_cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void gu_cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

// What both groups derive, identically, for a tile.
struct GuTileInfo {
    int b, i0, j0, ol, W, tlo, thi;
    bool work;   // the tile holds links of a sentence this kernel computes
    bool real;   // ... and nothing else: every (i, j) of the tile is a link of the graph
    float g;     // the sentence's incoming gradient
};
// Tiles are numbered sentence by sentence; within a sentence only the (ib, q) classes that can hold a link
// at all (j0 < L, inside the band) are counted: gu_classes of them.
__host__ __device__ inline int gu_class_width(int ib, int L, int nJw) {   // j-tiles of row block ib
    const int w = (L - ib * kGuTile + kGuTile - 1) / kGuTile;
    return w < nJw ? w : nJw;
}
__host__ __device__ inline int gu_classes(int L, int K) {
    const int nI = (L + kGuTile - 1) / kGuTile, nJw = (kGuTile - 1 + K) / kGuTile + 1;
    int n = 0;
    for (int ib = 0; ib < nI; ib++) n += gu_class_width(ib, L, nJw);
    return n;
}
__device__ __forceinline__ GuTileInfo gu_tile_info(int tile, int nC, int nJw, const int4 *__restrict__ sel,
                                                   int L, int K) {
    GuTileInfo ti;
    ti.b = tile / nC;
    int c = tile - ti.b * nC, ib = 0;
    for (int w = gu_class_width(0, L, nJw); c >= w; w = gu_class_width(ib, L, nJw)) {
        c -= w;
        ib++;
    }
    const int q = c;
    ti.i0 = ib * kGuTile;
    ti.j0 = ti.i0 + q * kGuTile;
    ti.W = 0; ti.tlo = 0; ti.thi = -1;
    ti.work = false; ti.real = false;
    const int4 si = __ldg(sel + ti.b);
    ti.g = __int_as_float(si.w);
    ti.ol = si.y;
    const int ol = si.y, tl = si.z, W = ol - tl + 1;
    if (si.x != 0 || !(ti.i0 < ol - 1 && ti.j0 < ol) || ti.j0 - (ti.i0 + kGuTile - 1) - 1 >= K) return ti;
    int tlo = ti.j0 - W;
    if (ti.i0 - W + 1 > tlo) tlo = ti.i0 - W + 1;
    if (tlo < 0) tlo = 0;
    int thi = tl - 2;
    if (ti.i0 + kGuTile - 1 < thi) thi = ti.i0 + kGuTile - 1;
    if (ti.j0 + kGuTile - 2 < thi) thi = ti.j0 + kGuTile - 2;
    ti.W = W; ti.tlo = tlo; ti.thi = thi;
    ti.work = true;   // (an empty step range leaves zeros in the accumulator's place: see the consumers)
    ti.real = q >= 1 && ti.j0 + kGuTile - 1 - ti.i0 - 1 < K && ti.j0 + kGuTile - 1 < ol;
    return ti;
}

// The consumers' pass over one tile: entries (i0 + 64 half + e, j0 + jl), e = 0..63, of a thread.
//   HAVE   the accumulator holds the tile's sums (otherwise the entries are zero: no step contributes)
//   REAL   every entry of the tile is a link (no tests); NREAL the same for the next tile, whose links
//          are copied into the slots this pass uses up
template <bool HAVE, bool REAL, bool NREAL>
__device__ __forceinline__ void gu_consume(const GuTileInfo &cur, const GuTileInfo &nxt, bool nwork, uint32_t ta,
                                           float *Lk, int half, int jl, float *__restrict__ glinks,
                                           const float *__restrict__ links_all, int L, int K) {
    const int il0 = 64 * half;
    // entry (i, j) sits at element (i K + j - i - 1) of the sentence's band: K - 1 further for the next i
    int eo = (cur.i0 + il0) * K + (cur.j0 + jl) - (cur.i0 + il0) - 1;
    float *out = glinks + (size_t)cur.b * L * K;
    // the next tile's entries sit `shift` elements away from this tile's in their own sentence's band
    const long long shift = (long long)(nxt.i0 + il0) * K + (nxt.j0 + jl) - (nxt.i0 + il0) - 1 - eo;
    const float *nsrc = links_all + (size_t)nxt.b * L * K + shift;
    uint32_t slot = umma::smem_u32(Lk + il0 * kGuTile + jl);
    float *lslot = Lk + il0 * kGuTile + jl;
    const float g = cur.g;
    // which of this thread's entries e = 0..63 (i = i0 + il0 + e) are links: 0 <= j-i-1 < K, i < ol, j < ol,
    // i.e. e in [lo, lo + n)
    int c_lo = 0, c_n = 0, n_lo = 0, n_n = 0;
    if (!REAL) {
        const int j = cur.j0 + jl, i = cur.i0 + il0;
        int lo = j - i - K, hi = j - i - 1;        // lo <= e <= hi
        lo = lo > 0 ? lo : 0;
        hi = hi < 63 ? hi : 63;
        hi = hi < cur.ol - 1 - i ? hi : cur.ol - 1 - i;
        c_lo = lo;
        c_n = (j < cur.ol && hi >= lo) ? hi - lo + 1 : 0;
    }
    if (!NREAL) {
        const int j = nxt.j0 + jl, i = nxt.i0 + il0;
        int lo = j - i - K, hi = j - i - 1;
        lo = lo > 0 ? lo : 0;
        hi = hi < 63 ? hi : 63;
        hi = hi < nxt.ol - 1 - i ? hi : nxt.ol - 1 - i;
        n_lo = lo;
        n_n = (nwork && j < nxt.ol && hi >= lo) ? hi - lo + 1 : 0;
    }
    // Batches of kGuBatch entries, each in four sweeps (loads, arithmetic, stores, copies): the asynchronous
    // copy is a compiler barrier for memory accesses, and entry by entry it would keep the next load from
    // starting; the sums of the batch after the one at hand are requested a batch ahead.
    constexpr int NB = kGuBatch / 8;
    float an[NB][8];
    if (HAVE) {
#pragma unroll
        for (int h = 0; h < NB; h++) umma::tmem_ld_col8(an[h], ta + 8 * h);
    }
#pragma unroll 1
    for (int bt = 0; bt < 64 / kGuBatch; bt++) {
        float a[NB][8];
        if (HAVE) {
#pragma unroll
            for (int h = 0; h < NB; h++) {
                umma::tmem_ld_wait8(an[h]);
#pragma unroll
                for (int k = 0; k < 8; k++) a[h][k] = an[h][k];
            }
            if (bt + 1 < 64 / kGuBatch) {
#pragma unroll
                for (int h = 0; h < NB; h++) umma::tmem_ld_col8(an[h], ta + kGuBatch * (bt + 1) + 8 * h);
            }
        }
        float v[kGuBatch];
#pragma unroll
        for (int k = 0; k < kGuBatch; k++) v[k] = HAVE ? lslot[(kGuBatch * bt + k) * kGuTile] : 0.f;
        if (HAVE) {
#pragma unroll
            for (int k = 0; k < kGuBatch; k++) {
                v[k] = g * a[k >> 3][k & 7] * ex2(v[k] * kLog2e);
                if (!(v[k] == v[k])) v[k] = 0.f;
            }
        }
#pragma unroll
        for (int k = 0; k < kGuBatch; k++) {
            const int e = kGuBatch * bt + k;
            if (REAL || (unsigned)(e - c_lo) < (unsigned)c_n) out[eo + k * (K - 1)] = v[k];
        }
#pragma unroll
        for (int k = 0; k < kGuBatch; k++) {
            const int e = kGuBatch * bt + k;
            if (NREAL || (unsigned)(e - n_lo) < (unsigned)n_n) gu_cp_async4(slot + e * kGuTile * 4, nsrc + eo + k * (K - 1));
            else lslot[e * kGuTile] = -INFINITY;
        }
        eo += kGuBatch * (K - 1);
    }
}

__global__ void __launch_bounds__(kGuThreads, 1)
dag_grad_links_umma_kernel(const float *__restrict__ alpha_all, const float *__restrict__ beta_all,
                           const float *__restrict__ hk_all, const float *__restrict__ links_all,
                           const int4 *__restrict__ sel, int *flag, float *__restrict__ glinks, int T, int L, int K,
                           int nC, int nJw, int ntiles) {
    extern __shared__ __align__(128) unsigned char gu_raw[];
    float *opnd = reinterpret_cast<float *>(gu_raw);          // [stage][A' hi, A' lo, B' hi, B' lo][kGuOperand]
    float *Lk = opnd + 2 * 4 * kGuOperand;                    // [128 i][128 j] links of the consumers' tile
    float *rawA = Lk + kGuTile * kGuTile;                     // [32 t][128 i] u_a rows of the producers' next chunk
    float *rawB = rawA + kGuOperand;                          // [32 t][128 j] u_b rows
    uint64_t *opfree = reinterpret_cast<uint64_t *>(rawB + kGuOperand);   // [2] products that read a stage are done
    uint64_t *full = opfree + 2;                              // [2] an accumulator is complete
    uint64_t *empty = full + 2;                               // [2] an accumulator has been read out (8 warps arrive)
    uint32_t *tslot = reinterpret_cast<uint32_t *>(empty + 2);
    volatile int *dead = reinterpret_cast<volatile int *>(tslot + 1);   // a wait gave up somewhere in the CTA
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    // a contiguous range of tiles per CTA: whole sentences, so every CTA gets the same mix of tile classes
    const int tile_lo = (int)((long long)ntiles * blockIdx.x / gridDim.x),
              tile_hi = (int)((long long)ntiles * (blockIdx.x + 1) / gridDim.x);

    if (warp == 0) umma::tmem_alloc(tslot, 2 * kGuTile);
    if (tid == 32) {
        for (int k = 0; k < 4; k++) umma::mbar_init(&opfree[k], 1);
        umma::mbar_init(&empty[0], kGuGroup / 32);
        umma::mbar_init(&empty[1], kGuGroup / 32);
        *dead = 0;
    }
    umma::fence_before_sync();
    __syncthreads();
    umma::fence_after_sync();
    const uint32_t tmem = *tslot;

    if (warp < kGuGroup / 32) {
        // =========================== producers ===========================
        const uint32_t idesc = umma::instr_desc_tf32(kGuTile, kGuTile);
        uint32_t ph_op0 = 0u, ph_op1 = 0u, ph_e0 = 0u, ph_e1 = 0u;
        int chunk = 0, nprod = 0;   // operand chunks and product tiles so far
        bool go = true;             // the issuing thread's own: false once it gave up on an accumulator
        const int row = tid & (kGuTile - 1), kq0 = tid >> 7;   // this thread's vertex of a tile; its K chunks kq0 + 2 u
        // The raw rows of a chunk (32 steps x 128 vertices of u_a and of u_b) are copied asynchronously into
        // rawA / rawB one chunk ahead; every thread copies exactly the entries it converts itself.
        float *myA = rawA + row, *myB = rawB + row;
        struct Chunk {
            GuTileInfo ti;
            int tile, c, nchunks;
            bool valid;
        };
        auto advance = [&](Chunk &k) {   // to the next chunk of a tile with a product, in tile order
            if (k.valid && k.c + 1 < k.nchunks) {
                k.c++;
                return;
            }
            for (int t = k.tile + 1; t < tile_hi; t++) {
                const GuTileInfo ti = gu_tile_info(t, nC, nJw, sel, L, K);
                if (ti.work && ti.thi >= ti.tlo) {
                    k.ti = ti;
                    k.tile = t;
                    k.c = 0;
                    k.nchunks = (ti.thi - ti.tlo + umma::kTileK) / umma::kTileK;
                    k.valid = true;
                    return;
                }
            }
            k.valid = false;
            k.tile = tile_hi;
        };
        // A'[t][i] exists for i in [t, t+W), i.e. t in (i-W, i]; B'[t][j] for j in [t+1, t+W], i.e. t in [j-W, j-1]
        struct Masks {
            int a_lo, a_hi, b_lo, b_hi;
        };
        auto masks_of = [&](const GuTileInfo &ti) {
            const int vi = ti.i0 + row, vj = ti.j0 + row;
            Masks m;
            m.a_lo = vi - ti.W + 1;
            m.a_hi = vi < L ? (vi < ti.thi ? vi : ti.thi) : -1;
            m.b_lo = vj - ti.W;
            m.b_hi = vj < L ? (vj - 1 < ti.thi ? vj - 1 : ti.thi) : -1;
            return m;
        };
        float hv[4][4], hvn[4][4];
        auto request = [&](const Chunk &k) {   // the chunk's raw entries and h_t
            const Masks m = masks_of(k.ti);
            const int t0 = k.ti.tlo + umma::kTileK * k.c;
            const float *al = alpha_all + (size_t)k.ti.b * T * L + k.ti.i0 + row;
            const float *be = beta_all + ((size_t)k.ti.b * T + 1) * L + k.ti.j0 + row;
            const float *hk = hk_all + (size_t)k.ti.b * (T + kGuHkPad);
#pragma unroll
            for (int u = 0; u < 4; u++) {
#pragma unroll
                for (int cc = 0; cc < 4; cc++) {
                    const int tl_ = 4 * (kq0 + 2 * u) + cc, t = t0 + tl_;
                    hvn[u][cc] = __ldg(hk + t);
                    if (t >= m.a_lo && t <= m.a_hi) gu_cp_async4(umma::smem_u32(myA + tl_ * kGuTile), al + (size_t)t * L);
                    if (t >= m.b_lo && t <= m.b_hi) gu_cp_async4(umma::smem_u32(myB + tl_ * kGuTile), be + (size_t)t * L);
                }
            }
            gu_cp_async_commit();
        };
        Chunk cu;
        cu.valid = false;
        cu.tile = tile_lo - 1;
        cu.c = 0;
        cu.nchunks = 0;
        advance(cu);
        if (cu.valid) request(cu);
        Chunk pf = cu;
        if (pf.valid) advance(pf);
        bool ok = true;
        int acc = 0;
        while (cu.valid) {
            const GuTileInfo &ti = cu.ti;
            const int c = cu.c;
            if (c == 0) {
                acc = nprod & 1;
                nprod++;
                if (gu_group_or(1, *dead != 0 || !ok)) break;   // no tensor-core work any more
            }
            const int s = chunk & 1, t0 = ti.tlo + umma::kTileK * c;
            float *st = opnd + s * 4 * kGuOperand;
            const Masks m = masks_of(ti);
            // this chunk's raw entries (copied while the previous chunk was converted) into registers ...
            gu_cp_async_wait_all();
            float ra[4][4], rb[4][4];
#pragma unroll
            for (int u = 0; u < 4; u++) {
#pragma unroll
                for (int cc = 0; cc < 4; cc++) {
                    const int tl_ = 4 * (kq0 + 2 * u) + cc, t = t0 + tl_;
                    hv[u][cc] = hvn[u][cc];
                    ra[u][cc] = (t >= m.a_lo && t <= m.a_hi) ? myA[tl_ * kGuTile] : -INFINITY;
                    rb[u][cc] = (t >= m.b_lo && t <= m.b_hi) ? myB[tl_ * kGuTile] : -INFINITY;
                }
            }
            // ... and the next chunk's on their way
            if (pf.valid) request(pf);
            if (chunk >= 2) {   // the products of the chunk before last read this stage
                if (ok && !umma::mbar_wait(&opfree[s], s ? ph_op1 : ph_op0, kGuPolls)) ok = false;
                if (s) ph_op1 ^= 1u; else ph_op0 ^= 1u;
            }
#pragma unroll
            for (int u = 0; u < 4; u++) {
                const int o = umma::tile_unit_offset(row, kq0 + 2 * u);
                float va[4], vb[4];
#pragma unroll
                for (int cc = 0; cc < 4; cc++) {
                    va[cc] = ex2(ra[u][cc] + hv[u][cc]);
                    vb[cc] = ex2(rb[u][cc] + hv[u][cc]);
                }
                float4 hi, lo4;
                gu_split4(va, hi, lo4);
                *reinterpret_cast<float4 *>(reinterpret_cast<char *>(st) + o) = hi;
                *reinterpret_cast<float4 *>(reinterpret_cast<char *>(st + kGuOperand) + o) = lo4;
                gu_split4(vb, hi, lo4);
                *reinterpret_cast<float4 *>(reinterpret_cast<char *>(st + 2 * kGuOperand) + o) = hi;
                *reinterpret_cast<float4 *>(reinterpret_cast<char *>(st + 3 * kGuOperand) + o) = lo4;
            }
            umma::fence_smem_to_async();
            if (gu_group_or(1, !ok)) break;   // also the barrier between the staging and the products
            if (tid == 0) {
                umma::fence_after_sync();
                if (go && c == 0 && nprod > 2) {   // the accumulator's previous tile has been read out
                    go = umma::mbar_wait(&empty[acc], acc ? ph_e1 : ph_e0, kGuPolls);
                    if (acc) ph_e1 ^= 1u; else ph_e0 ^= 1u;
                    umma::fence_after_sync();
                }
                if (go) {
                    // D[j][i] += B'^T A': the factor along j is the M operand
                    const uint32_t d = tmem + (uint32_t)(acc * kGuTile);
                    const uint32_t n_hi = umma::smem_u32(st), n_lo = umma::smem_u32(st + kGuOperand);
                    const uint32_t m_hi = umma::smem_u32(st + 2 * kGuOperand), m_lo = umma::smem_u32(st + 3 * kGuOperand);
                    int nk = (ti.thi - t0 + 8) >> 3;   // K steps of 8 that hold a real target step
                    nk = nk > umma::kTileK / 8 ? umma::kTileK / 8 : nk;
                    for (int kk = 0; kk < nk; kk++) {
                        const uint32_t o = kk * umma::kStepBytes;
                        umma::mma_tf32(d, umma::smem_desc(m_hi + o), umma::smem_desc(n_hi + o), idesc, c > 0 || kk > 0);
                        umma::mma_tf32(d, umma::smem_desc(m_hi + o), umma::smem_desc(n_lo + o), idesc, true);
                        umma::mma_tf32(d, umma::smem_desc(m_lo + o), umma::smem_desc(n_hi + o), idesc, true);
                    }
                    umma::commit(&opfree[s]);
                    if (c == cu.nchunks - 1) umma::commit(&full[acc]);
                } else {
                    *dead = 1;   // seen by this group before its next tile, by the consumers when their wait ends
                }
            }
            chunk++;
            cu = pf;
            if (pf.valid) advance(pf);
        }
        if (cu.valid && tid == 0) *dead = 1;   // left the loop early
        gu_cp_async_wait_all();
    } else {
        // =========================== consumers ===========================
        // thread = column j0 + jl of the tile (a lane of the accumulator), rows i0 + 64 half .. + 63
        const int ctid = tid - kGuGroup, cw = warp - kGuGroup / 32;
        const int jl = 32 * (cw & 3) + lane, half = cw >> 2;
        uint32_t ph_f0 = 0u, ph_f1 = 0u;
        int nprod = 0;
        bool off = false;   // group-uniform
        GuTileInfo none;
        none.b = 0; none.i0 = 0; none.j0 = 0; none.ol = 0; none.W = 0; none.tlo = 0; none.thi = -1;
        none.work = false; none.real = false; none.g = 0.f;
        int tile = tile_lo;
        GuTileInfo cur = none;
        if (tile < tile_hi) cur = gu_tile_info(tile, nC, nJw, sel, L, K);
        // the first tile's links (the pass over a tile that is not there only fetches)
        gu_consume<false, false, false>(none, cur, cur.work, 0u, Lk, half, jl, glinks, links_all, L, K);
        gu_cp_async_commit();
        for (; tile < tile_hi; tile++) {
            const int next = tile + 1;
            GuTileInfo nxt = none;
            if (next < tile_hi) nxt = gu_tile_info(next, nC, nJw, sel, L, K);
            bool have = false;   // the accumulator holds this tile's sums
            const int acc = nprod & 1;
            if (cur.work && cur.thi >= cur.tlo) {
                nprod++;
                bool ok = !off && *dead == 0;
                if (ok && cw == 0) ok = umma::mbar_wait(&full[acc], acc ? ph_f1 : ph_f0, kGuPolls);   // one warp polls
                if (acc) ph_f1 ^= 1u; else ph_f0 ^= 1u;
                if (!off && gu_group_or(2, !ok)) {
                    off = true;
                    if (ctid == 0) *dead = 1;
                }
                if (off) {
                    if (ctid == 0) flag[cur.b] = kFlagExactBackward;   // the exact kernel takes the whole sentence
                } else {
                    umma::fence_after_sync();
                    have = true;
                }
            }
            gu_cp_async_wait_all();   // this thread's links of the tile are in their slots
            const uint32_t ta = tmem + ((uint32_t)(32 * (cw & 3)) << 16) + (uint32_t)(acc * kGuTile + 64 * half);
            const bool nreal = nxt.work && nxt.real;
            if (have) {
                if (cur.real) {
                    if (nreal) gu_consume<true, true, true>(cur, nxt, true, ta, Lk, half, jl, glinks, links_all, L, K);
                    else gu_consume<true, true, false>(cur, nxt, nxt.work, ta, Lk, half, jl, glinks, links_all, L, K);
                } else {
                    if (nreal) gu_consume<true, false, true>(cur, nxt, true, ta, Lk, half, jl, glinks, links_all, L, K);
                    else gu_consume<true, false, false>(cur, nxt, nxt.work, ta, Lk, half, jl, glinks, links_all, L, K);
                }
                umma::fence_before_sync();
                __syncwarp();
                if (lane == 0) gu_mbar_arrive(&empty[acc]);
            } else if (cur.work && !(cur.thi >= cur.tlo)) {
                // links without a step that passes through them: zeros
                gu_consume<false, false, false>(cur, nxt, nxt.work, ta, Lk, half, jl, glinks, links_all, L, K);
            } else {
                gu_consume<false, false, false>(none, nxt, nxt.work, ta, Lk, half, jl, glinks, links_all, L, K);
            }
            gu_cp_async_commit();
            cur = nxt;
        }
        gu_cp_async_wait_all();
    }
    umma::fence_before_sync();
    __syncthreads();
    if (warp == 0) umma::tmem_dealloc(tmem, 2 * kGuTile);
}

}  // namespace dat
