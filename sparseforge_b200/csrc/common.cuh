// Shared host/device helpers for the sparseforge_b200 kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>

#include "../../include/sparseforge_b200.h"

namespace sf {

// ---- error reporting -----------------------------------------------------------------
// One message per host thread; sf_last_error_string() hands it out.
char* last_error_buffer();
int fail(int code, const char* fmt, ...);

#define SF_CHECK_ARG(cond, ...)                             \
    do {                                                    \
        if (!(cond)) return sf::fail(SF_ERR_BAD_ARG, __VA_ARGS__); \
    } while (0)

#define SF_CHECK_CUDA(expr)                                                              \
    do {                                                                                 \
        cudaError_t _e = (expr);                                                         \
        if (_e != cudaSuccess)                                                           \
            return sf::fail(SF_ERR_CUDA, "%s failed: %s", #expr, cudaGetErrorString(_e)); \
    } while (0)

inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// Number of SMs of the current device (cached per thread; 148 on B200).
int sm_count();

// ---- device helpers ------------------------------------------------------------------
__device__ __forceinline__ float bf16_round(float x) {
    return __bfloat162float(__float2bfloat16_rn(x));
}

// Ordering used by every top-2-of-4 selection: descending by value, NaN counts as the
// largest value, equal values keep their column order (lower index first).
__device__ __forceinline__ bool gt_desc(float a, float b) {
    return (a > b) || (a != a && b == b);
}
__device__ __forceinline__ bool eq_desc(float a, float b) {
    return (a == b) || (a != a && b != b);
}

// rank[i] = position of element i in the stable descending order of the group.
__device__ __forceinline__ void rank4(const float (&x)[4], int (&rank)[4]) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        int r = 0;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            if (j == i) continue;
            r += gt_desc(x[j], x[i]) ? 1 : 0;
            if (j < i) r += eq_desc(x[j], x[i]) ? 1 : 0;
        }
        rank[i] = r;
    }
}

// 2:4 metadata nibble of a keep pattern (exactly two bits of `keep` set):
// i0 | (i1 << 2), i0 < i1 the kept column offsets inside the group.
__device__ __forceinline__ uint32_t nibble_of_keep(uint32_t keep) {
    uint32_t i0 = __ffs(keep) - 1;
    uint32_t i1 = 31 - __clz(keep);
    return i0 | (i1 << 2);
}

// keep bitmask (bit i = column i kept) of the stable top-2 of a group.
__device__ __forceinline__ uint32_t top2_keep(const float (&x)[4]) {
    int r[4];
    rank4(x, r);
    uint32_t k = 0;
#pragma unroll
    for (int i = 0; i < 4; ++i) k |= (r[i] < 2 ? 1u : 0u) << i;
    return k;
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ double warp_sum(double v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// Streaming 16-byte global accesses (data is touched once per pass).
__device__ __forceinline__ uint4 ld_stream16(const void* p) {
    return __ldcs(reinterpret_cast<const uint4*>(p));
}
__device__ __forceinline__ void st_stream16(void* p, uint4 v) {
    __stcs(reinterpret_cast<uint4*>(p), v);
}
__device__ __forceinline__ uint2 ld_stream8(const void* p) {
    return __ldcs(reinterpret_cast<const uint2*>(p));
}
__device__ __forceinline__ void st_stream8(void* p, uint2 v) {
    __stcs(reinterpret_cast<uint2*>(p), v);
}

// 8 consecutive elements of a float / bf16 tensor <-> 8 floats.
template <typename T>
struct Vec8;
template <>
struct Vec8<float> {
    static __device__ __forceinline__ void load(const float* p, float (&x)[8]) {
        uint4 a = ld_stream16(p), b = ld_stream16(p + 4);
        x[0] = __uint_as_float(a.x); x[1] = __uint_as_float(a.y);
        x[2] = __uint_as_float(a.z); x[3] = __uint_as_float(a.w);
        x[4] = __uint_as_float(b.x); x[5] = __uint_as_float(b.y);
        x[6] = __uint_as_float(b.z); x[7] = __uint_as_float(b.w);
    }
    static __device__ __forceinline__ void store(float* p, const float (&x)[8]) {
        st_stream16(p, make_uint4(__float_as_uint(x[0]), __float_as_uint(x[1]),
                                  __float_as_uint(x[2]), __float_as_uint(x[3])));
        st_stream16(p + 4, make_uint4(__float_as_uint(x[4]), __float_as_uint(x[5]),
                                      __float_as_uint(x[6]), __float_as_uint(x[7])));
    }
    // Rounding a value to the storage type and back (identity for fp32).
    static __device__ __forceinline__ float round(float x) { return x; }
};
template <>
struct Vec8<__nv_bfloat16> {
    static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&x)[8]) {
        uint4 a = ld_stream16(p);
        uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            x[2 * i] = __uint_as_float(w[i] << 16);
            x[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, const float (&x)[8]) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            __nv_bfloat162 h = __floats2bfloat162_rn(x[2 * i], x[2 * i + 1]);
            w[i] = *reinterpret_cast<uint32_t*>(&h);
        }
        st_stream16(p, make_uint4(w[0], w[1], w[2], w[3]));
    }
    static __device__ __forceinline__ float round(float x) { return bf16_round(x); }
};

}  // namespace sf
