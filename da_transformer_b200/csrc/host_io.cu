// Host-to-device transfer of band links that moves only the entries a graph can have.
//
// links[b,i,d] is the transition i -> i+d+1, so row i of a graph with n vertices has n-1-i real
// entries; the rest of the [L,K] band (about half of it when K = L-1) is -inf padding that no kernel
// of this library ever reads (every link access is guarded by "destination < output_length").  A
// caller that feeds the ops from HOST memory (the reference's host-side callers never do: its model
// produces the links on the device) pays PCIe time for that padding.  dat_upload_links moves only the
// real entries.  When the host buffer is page-locked (and therefore mapped into the device's address
// space) a small kernel PULLS them: one warp per band row reads the row's real prefix straight from
// host memory in 16-byte units (512 contiguous bytes per warp instruction) and stores it to the device
// copy (measured: 268 MB of ragged rows at ~38 GB/s, against ~41 GB/s x 284 MB for the copy engines'
// staircase below and 55 GB/s x 535 MB for the whole band; splitting the rows between the two made no
// difference).  What does help is to keep BOTH kinds of PCIe reads going: the first rows of a sentence are nearly
// full (row i of n has n-1-i real entries of translen), so rows 0 .. head-1, those at least three quarters real,
// go as one contiguous block per sentence through the copy engine on a helper stream (padding included, 55 GB/s)
// while the kernel pulls the ragged rest; the call's stream waits for both (46 GB/s over the whole transfer).
// For pageable memory it falls back to the staircase of kRowBlock-row blocks, each block one strided 3-D copy over
// all sentences, cut at the longest row of the block.
#include "dat_common.cuh"

#include <mutex>

namespace dat {
constexpr int kRowBlock = 32;
constexpr int kPullThreads = 256;
constexpr int kPullBlocks = 96;

// One warp per band row (b, i), i < n - 1: copies the 16-byte units that cover the row's n - 1 - i real
// entries (at most translen).  src and dst have the same alignment modulo 16; the units may reach a few
// bytes into the padding on either side of the prefix, which is copied like everything else.
__global__ void __launch_bounds__(kPullThreads)
upload_links_pull_kernel(const float *__restrict__ src, float *__restrict__ dst, int B, int L, int K, int n,
                         int row_begin) {
    const int lane = threadIdx.x & 31;
    const long long nwarps = (long long)gridDim.x * (kPullThreads / 32);
    const int per = n - 1 - row_begin;   // rows with a successor that this kernel moves, in every sentence
    const long long rows = (long long)B * per;
    const uintptr_t base = reinterpret_cast<uintptr_t>(src);
    const uintptr_t total = (uintptr_t)B * L * K * sizeof(float);
    const ptrdiff_t shift = reinterpret_cast<const char *>(dst) - reinterpret_cast<const char *>(src);
    for (long long w = (long long)blockIdx.x * (kPullThreads / 32) + (threadIdx.x >> 5); w < rows; w += nwarps) {
        const int b = (int)(w / per), i = row_begin + (int)(w - (long long)b * per);
        int len = n - 1 - i;
        len = len < K ? len : K;
        const uintptr_t lo = ((uintptr_t)b * L + i) * (uintptr_t)K * sizeof(float);
        uintptr_t a0 = (base + lo) & ~(uintptr_t)15;
        uintptr_t a1 = (base + lo + (uintptr_t)len * sizeof(float) + 15) & ~(uintptr_t)15;
        if (a0 < base) a0 = base;                    // base itself is 16-byte aligned (checked by the caller)
        if (a1 > base + total) a1 = base + total;
        const int units = (int)((a1 - a0) >> 4);     // <= translen / 4 + 2
        // every lane requests all its units before it stores any of them
        uint4 v[4];
        int k = lane;
        for (; k + 96 < units; k += 128) {
#pragma unroll
            for (int q = 0; q < 4; q++) v[q] = ld_stream16(reinterpret_cast<const void *>(a0 + ((uintptr_t)(k + 32 * q) << 4)));
#pragma unroll
            for (int q = 0; q < 4; q++)
                *reinterpret_cast<uint4 *>(reinterpret_cast<char *>(a0 + ((uintptr_t)(k + 32 * q) << 4)) + shift) = v[q];
        }
#pragma unroll
        for (int q = 0; q < 4; q++)
            if (k + 32 * q < units) v[q] = ld_stream16(reinterpret_cast<const void *>(a0 + ((uintptr_t)(k + 32 * q) << 4)));
#pragma unroll
        for (int q = 0; q < 4; q++)
            if (k + 32 * q < units)
                *reinterpret_cast<uint4 *>(reinterpret_cast<char *>(a0 + ((uintptr_t)(k + 32 * q) << 4)) + shift) = v[q];
    }
}
// rows of a sentence that go through the copy engine whole: those with at least 3/4 of translen real entries
__host__ inline int upload_head_rows(int n, int translen) {
    int h = n - 1 - (3 * translen) / 4;
    h = h < 0 ? 0 : h;
    return h < n - 1 ? h : n - 1;
}

struct UploadSide {
    cudaStream_t stream = nullptr;
    cudaEvent_t fork = nullptr, join = nullptr;
};
// helper stream and events of the current device (created on first use, kept for the life of the process)
// (the caller holds g_upload_mutex from here until it has made its own stream wait for `join`: the events are
// shared by all callers of a device, and a wait refers to an event's latest record)
static std::mutex g_upload_mutex;
static bool upload_side(UploadSide *out) {
    static UploadSide side[64];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return false;
    UploadSide &s = side[dev];
    if (!s.stream) {
        UploadSide t;
        if (cudaStreamCreateWithFlags(&t.stream, cudaStreamNonBlocking) != cudaSuccess ||
            cudaEventCreateWithFlags(&t.fork, cudaEventDisableTiming) != cudaSuccess ||
            cudaEventCreateWithFlags(&t.join, cudaEventDisableTiming) != cudaSuccess) {
            cudaGetLastError();
            return false;
        }
        s = t;
    }
    *out = s;
    return true;
}
}  // namespace dat

extern "C" {

int dat_upload_links_head_rows(int prelen, int translen, int max_output_length) {
    if (prelen <= 0 || translen <= 0) return 0;
    const int n = max_output_length < prelen ? max_output_length : prelen;
    return n < 2 ? 0 : dat::upload_head_rows(n, translen);
}

size_t dat_upload_links_bytes(int bsz, int prelen, int translen, int max_output_length) {
    using namespace dat;
    if (bsz <= 0 || prelen <= 0 || translen <= 0) return 0;
    int n = max_output_length < prelen ? max_output_length : prelen;
    size_t total = 0;
    for (int r0 = 0; r0 < n - 1; r0 += kRowBlock) {
        int rows = n - 1 - r0 < kRowBlock ? n - 1 - r0 : kRowBlock;
        int cols = n - 1 - r0 < translen ? n - 1 - r0 : translen;
        total += (size_t)rows * cols * sizeof(float);
    }
    return total * (size_t)bsz;
}

int dat_upload_links(const float *host_links, float *dev_links, int bsz, int prelen, int translen,
                     int max_output_length, void *stream) {
    using namespace dat;
    DAT_REQUIRE(bsz >= 0 && prelen >= 1 && translen >= 1 && max_output_length >= 0, DAT_ERR_BAD_ARG,
                "dat_upload_links: bad sizes bsz=%d prelen=%d translen=%d max_output_length=%d", bsz, prelen,
                translen, max_output_length);
    if (bsz == 0) return DAT_OK;
    DAT_REQUIRE(host_links && dev_links, DAT_ERR_BAD_ARG, "dat_upload_links: null pointer");
    const int n = max_output_length < prelen ? max_output_length : prelen;
    if (n < 2) return DAT_OK;
    {
        // page-locked host memory is visible to kernels: pull the rows' real prefixes
        void *mapped = nullptr;
        const bool pinned = cudaHostGetDevicePointer(&mapped, const_cast<float *>(host_links), 0) == cudaSuccess &&
                            mapped != nullptr;
        if (!pinned) cudaGetLastError();
        if (pinned && (reinterpret_cast<uintptr_t>(mapped) & 15) == 0 &&
            (reinterpret_cast<uintptr_t>(dev_links) & 15) == 0) {
            cudaStream_t st = static_cast<cudaStream_t>(stream);
            int head = upload_head_rows(n, translen);
            cudaStreamCaptureStatus cap = cudaStreamCaptureStatusNone;
            // (not while the stream is being captured: the helper stream belongs to no graph)
            if (head > 0 && (cudaStreamIsCapturing(st, &cap) != cudaSuccess || cap != cudaStreamCaptureStatusNone)) {
                cudaGetLastError();
                head = 0;
            }
            std::unique_lock<std::mutex> lock(g_upload_mutex, std::defer_lock);
            UploadSide side;
            if (head > 0) {
                lock.lock();
                if (!upload_side(&side)) {
                    lock.unlock();
                    head = 0;
                }
            }
            if (head > 0) {
                const size_t sentence = (size_t)prelen * translen * sizeof(float);
                bool ok = cudaEventRecord(side.fork, st) == cudaSuccess &&
                          cudaStreamWaitEvent(side.stream, side.fork, 0) == cudaSuccess &&
                          cudaMemcpy2DAsync(dev_links, sentence, host_links, sentence,
                                            (size_t)head * translen * sizeof(float), (size_t)bsz, cudaMemcpyHostToDevice,
                                            side.stream) == cudaSuccess &&
                          cudaEventRecord(side.join, side.stream) == cudaSuccess;
                if (!ok) return check_launch("dat_upload_links(copy)");
            }
            if (head < n - 1)
                upload_links_pull_kernel<<<kPullBlocks, kPullThreads, 0, st>>>(static_cast<const float *>(mapped), dev_links,
                                                                             bsz, prelen, translen, n, head);
            if (int rc = check_launch("dat_upload_links")) return rc;
            if (head > 0 && cudaStreamWaitEvent(st, side.join, 0) != cudaSuccess) return check_launch("dat_upload_links(join)");
            return DAT_OK;
        }
    }
    const size_t pitch = (size_t)translen * sizeof(float);
    for (int r0 = 0; r0 < n - 1; r0 += kRowBlock) {
        const int rows = n - 1 - r0 < kRowBlock ? n - 1 - r0 : kRowBlock;
        const int cols = n - 1 - r0 < translen ? n - 1 - r0 : translen;   // row r0 is the longest of the block
        cudaMemcpy3DParms p = {};
        p.srcPtr = make_cudaPitchedPtr(const_cast<float *>(host_links), pitch, pitch, (size_t)prelen);
        p.dstPtr = make_cudaPitchedPtr(dev_links, pitch, pitch, (size_t)prelen);
        p.srcPos = make_cudaPos(0, (size_t)r0, 0);
        p.dstPos = make_cudaPos(0, (size_t)r0, 0);
        p.extent = make_cudaExtent((size_t)cols * sizeof(float), (size_t)rows, (size_t)bsz);
        p.kind = cudaMemcpyHostToDevice;
        cudaError_t e = cudaMemcpy3DAsync(&p, static_cast<cudaStream_t>(stream));
        if (e != cudaSuccess) {
            cudaGetLastError();
            set_error("dat_upload_links: cudaMemcpy3DAsync failed at row %d: %s", r0, cudaGetErrorString(e));
            return DAT_ERR_LAUNCH;
        }
    }
    return DAT_OK;
}

}  // extern "C"
