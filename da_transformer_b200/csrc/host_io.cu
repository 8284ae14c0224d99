// Host-to-device transfer of band links that moves only the entries a graph can have.
//
// links[b,i,d] is the transition i -> i+d+1, so row i of a graph with n vertices has n-1-i real
// entries; the rest of the [L,K] band (about half of it when K = L-1) is -inf padding that no kernel
// of this library ever reads (every link access is guarded by "destination < output_length").  A
// caller that feeds the ops from HOST memory (the reference's host-side callers never do: its model
// produces the links on the device) pays PCIe time for that padding.  dat_upload_links copies the
// staircase that covers the real entries instead: rows in blocks of kRowBlock, each block as one
// strided 3-D copy over all sentences, cut at the longest row of the block.
#include "dat_common.cuh"

namespace dat {
constexpr int kRowBlock = 32;
}

extern "C" {

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
