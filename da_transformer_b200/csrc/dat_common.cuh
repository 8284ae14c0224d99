// Shared helpers of the sm_100a kernels: error reporting for the C ABI, MUFU wrappers,
// warp/block reductions, 128-bit streaming loads.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/dat_b200.h"

namespace dat {

constexpr float kLog2e = 1.4426950408889634f;
constexpr float kLn2 = 0.6931471805599453f;
constexpr double kLn2d = 0.6931471805599453094172321;
constexpr double kLog2ed = 1.4426950408889634073599247;
// "minus infinity" of the online log-sum-exp accumulators: finite, so that
// (-inf) - kNegBig stays -inf (exp2 -> 0) instead of producing NaN.
constexpr float kNegBig = -1.0e30f;

void set_error(const char *fmt, ...);
int check_launch(const char *what);

#define DAT_REQUIRE(cond, code, ...)      \
    do {                                  \
        if (!(cond)) {                    \
            ::dat::set_error(__VA_ARGS__); \
            return (code);                \
        }                                 \
    } while (0)

__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ float lg2(float x) {
    float y;
    asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// Two-lane fp32 arithmetic of sm_100: one issue slot for two operations, each rounded like its scalar form.
// (x, y) = (a0 + b0, a1 + b1), round to nearest like __fadd_rn
__device__ __forceinline__ void fadd2_rn(float &x, float &y, float a0, float a1, float b0, float b1) {
    asm("{\n\t.reg .b64 ra, rb, rc;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\t"
        "add.rn.f32x2 rc, ra, rb;\n\tmov.b64 {%0, %1}, rc;\n\t}"
        : "=f"(x), "=f"(y)
        : "f"(a0), "f"(a1), "f"(b0), "f"(b1));
}
// (x, y) = (a0 * b0 + x, a1 * b1 + y), fused and rounded to nearest like fmaf
__device__ __forceinline__ void ffma2_rn(float &x, float &y, float a0, float a1, float b0, float b1) {
    asm("{\n\t.reg .b64 ra, rb, rc;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\tmov.b64 rc, {%0, %1};\n\t"
        "fma.rn.f32x2 rc, ra, rb, rc;\n\tmov.b64 {%0, %1}, rc;\n\t}"
        : "+f"(x), "+f"(y)
        : "f"(a0), "f"(a1), "f"(b0), "f"(b1));
}
// (x, y) = (a0 * b0, a1 * b1), round to nearest
__device__ __forceinline__ void fmul2_rn(float &x, float &y, float a0, float a1, float b0, float b1) {
    asm("{\n\t.reg .b64 ra, rb, rc;\n\tmov.b64 ra, {%2, %3};\n\tmov.b64 rb, {%4, %5};\n\t"
        "mul.rn.f32x2 rc, ra, rb;\n\tmov.b64 {%0, %1}, rc;\n\t}"
        : "=f"(x), "=f"(y)
        : "f"(a0), "f"(a1), "f"(b0), "f"(b1));
}
// three-input maximum of sm_100 (NaN operands are ignored, as by fmaxf)
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Merge two online log-sum-exp states (m = running max in the log2 domain, s = sum of
// 2^(x-m)).  Safe for empty states (m = kNegBig, s = 0).
__device__ __forceinline__ void lse_merge(float &m, float &s, float m2, float s2) {
    float mn = fmaxf(m, m2);
    s = s * ex2(m - mn) + s2 * ex2(m2 - mn);
    m = mn;
}

__device__ __forceinline__ void warp_lse(float &m, float &s) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        float m2 = __shfl_xor_sync(0xffffffffu, m, o);
        float s2 = __shfl_xor_sync(0xffffffffu, s, o);
        lse_merge(m, s, m2, s2);
    }
}

// 16-byte read-only streaming load that does not allocate in L1.
__device__ __forceinline__ uint4 ld_stream16(const void *p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

// A 4-byte read-only load the compiler will not move down to its first use: issued where it
// is written, so that its latency overlaps the work in between.
__device__ __forceinline__ float ld_early(const float *p) {
    float v;
    asm volatile("ld.global.nc.f32 %0, [%1];" : "=f"(v) : "l"(p));
    return v;
}

template <typename T>
struct Elem;

template <>
struct Elem<float> {
    static constexpr int kVec = 4;
    static constexpr uint32_t kNegInfWord = 0xff800000u;   // a 32-bit word full of -inf elements
    __device__ static __forceinline__ float to_float(float v) { return v; }
    __device__ static __forceinline__ float from_float(float v) { return v; }
    __device__ static __forceinline__ void unpack(const uint4 &u, float *f) {
        f[0] = __uint_as_float(u.x);
        f[1] = __uint_as_float(u.y);
        f[2] = __uint_as_float(u.z);
        f[3] = __uint_as_float(u.w);
    }
    __device__ static __forceinline__ uint4 pack(const float *f) {
        return make_uint4(__float_as_uint(f[0]), __float_as_uint(f[1]), __float_as_uint(f[2]),
                          __float_as_uint(f[3]));
    }
};

template <>
struct Elem<__half> {
    static constexpr int kVec = 8;
    static constexpr uint32_t kNegInfWord = 0xfc00fc00u;
    __device__ static __forceinline__ float to_float(__half v) { return __half2float(v); }
    __device__ static __forceinline__ __half from_float(float v) { return __float2half_rn(v); }
    __device__ static __forceinline__ void unpack(const uint4 &u, float *f) {
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int i = 0; i < 4; i++) {
            __half2 h = *reinterpret_cast<const __half2 *>(&w[i]);
            float2 p = __half22float2(h);
            f[2 * i] = p.x;
            f[2 * i + 1] = p.y;
        }
    }
    __device__ static __forceinline__ uint4 pack(const float *f) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            __half2 h = __floats2half2_rn(f[2 * i], f[2 * i + 1]);
            w[i] = *reinterpret_cast<uint32_t *>(&h);
        }
        return make_uint4(w[0], w[1], w[2], w[3]);
    }
};

template <>
struct Elem<__nv_bfloat16> {
    static constexpr int kVec = 8;
    static constexpr uint32_t kNegInfWord = 0xff80ff80u;
    __device__ static __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }
    __device__ static __forceinline__ __nv_bfloat16 from_float(float v) { return __float2bfloat16_rn(v); }
    __device__ static __forceinline__ void unpack(const uint4 &u, float *f) {
        // a bf16 is the upper half of an fp32
        const uint32_t w[4] = {u.x, u.y, u.z, u.w};
#pragma unroll
        for (int i = 0; i < 4; i++) {
            f[2 * i] = __uint_as_float(w[i] << 16);
            f[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
    __device__ static __forceinline__ uint4 pack(const float *f) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; i++) {
            __nv_bfloat162 h = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
            w[i] = *reinterpret_cast<uint32_t *>(&h);
        }
        return make_uint4(w[0], w[1], w[2], w[3]);
    }
};

struct DeviceInfo {
    int device;
    int sm_count;
    int max_smem_optin;
    int cc_major;
};
// Properties of the current device (cached per device).  Returns false on failure.
bool device_info(DeviceInfo *out);

}  // namespace dat
