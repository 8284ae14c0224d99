// Error reporting, version and device queries of the C ABI.
#include <cstdarg>
#include <cstdio>
#include <mutex>

#include "dat_common.cuh"

namespace dat {

static thread_local char g_error[512] = "";

void set_error(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

int check_launch(const char *what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        set_error("%s: CUDA error %d (%s)", what, (int)e, cudaGetErrorString(e));
        return DAT_ERR_LAUNCH;
    }
    return DAT_OK;
}

bool device_info(DeviceInfo *out) {
    constexpr int kMaxDev = 64;
    static DeviceInfo cache[kMaxDev];
    static bool have[kMaxDev] = {};
    static std::mutex mu;
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDev) {
        cudaGetLastError();
        set_error("no current CUDA device");
        return false;
    }
    std::lock_guard<std::mutex> lock(mu);
    if (!have[dev]) {
        DeviceInfo d;
        d.device = dev;
        bool ok = cudaDeviceGetAttribute(&d.sm_count, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess &&
                  cudaDeviceGetAttribute(&d.max_smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev) == cudaSuccess &&
                  cudaDeviceGetAttribute(&d.cc_major, cudaDevAttrComputeCapabilityMajor, dev) == cudaSuccess;
        if (!ok) {
            cudaGetLastError();
            set_error("cannot query CUDA device %d", dev);
            return false;
        }
        cache[dev] = d;
        have[dev] = true;
    }
    *out = cache[dev];
    return true;
}

}  // namespace dat

extern "C" {

int dat_version(void) { return DAT_B200_VERSION; }

const char *dat_last_error(void) { return dat::g_error; }

const char *dat_status_string(int code) {
    switch (code) {
        case DAT_OK: return "ok";
        case DAT_ERR_BAD_ARG: return "bad argument";
        case DAT_ERR_UNSUPPORTED: return "unsupported dtype or size";
        case DAT_ERR_LAUNCH: return "CUDA launch failure";
        case DAT_ERR_NO_DEVICE: return "no usable CUDA device";
        default: return "unknown status";
    }
}

}  // extern "C"
