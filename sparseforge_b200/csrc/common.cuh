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

// ---- cheap arithmetic for the HBM-bound passes ------------------------------------------
// The passes must stay under ~60 instructions per element to keep up with HBM, so division,
// square root and exp use the 1-2 ulp hardware approximations (relative error < 5e-7, far
// inside the 1e-5 parity bar) instead of the IEEE-exact sequences.
__device__ __forceinline__ float fast_rcp(float x) {
    float r;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}
__device__ __forceinline__ float fast_sqrt(float x) {
    float r;
    asm("sqrt.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}
__device__ __forceinline__ float fast_ex2(float x) {
    float r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(x));
    return r;
}
// Round-to-nearest-even to bf16 precision with integer ops (keeps the conversion pipe free).
__device__ __forceinline__ float bf16_round_int(float x) {
    uint32_t u = __float_as_uint(x);
    u = (u + 0x7fffu + ((u >> 16) & 1u)) & 0xffff0000u;
    return __uint_as_float(u);
}

// Stable top-2 of a group of four without NaN handling: six comparisons, "a >= b" lets the
// lower index win a tie. rank[i] as in rank4 for NaN-free input.
__device__ __forceinline__ void rank4_fast(const float (&x)[4], int (&rank)[4]) {
    const int c01 = x[0] >= x[1], c02 = x[0] >= x[2], c03 = x[0] >= x[3];
    const int c12 = x[1] >= x[2], c13 = x[1] >= x[3], c23 = x[2] >= x[3];
    rank[0] = 3 - c01 - c02 - c03;
    rank[1] = c01 + 2 - c12 - c13;
    rank[2] = c02 + c12 + 1 - c23;
    rank[3] = c03 + c13 + c23;
}
__device__ __forceinline__ uint32_t top2_keep_fast(const float (&x)[4]) {
    int r[4];
    rank4_fast(x, r);
    return (r[0] < 2 ? 1u : 0u) | (r[1] < 2 ? 2u : 0u) | (r[2] < 2 ? 4u : 0u) | (r[3] < 2 ? 8u : 0u);
}

// The same stable top-2 as lane masks: keep[i] is all ones if column i is kept, else zero.
// b_ij = (x_i >= x_j) says "i beats j" (the lower index wins a tie); column i is kept when at
// most one other column beats it, which is a majority vote over three of the six comparisons.
__device__ __forceinline__ uint32_t set_ge(float a, float b) {
    uint32_t d;
    asm("set.ge.u32.f32 %0, %1, %2;" : "=r"(d) : "f"(a), "f"(b));
    return d;
}
__device__ __forceinline__ uint32_t maj3(uint32_t a, uint32_t b, uint32_t c) { return (a & b) | (a & c) | (b & c); }
__device__ __forceinline__ void top2_keep_masks(const float (&x)[4], uint32_t (&keep)[4]) {
    const uint32_t b01 = set_ge(x[0], x[1]), b02 = set_ge(x[0], x[2]), b03 = set_ge(x[0], x[3]);
    const uint32_t b12 = set_ge(x[1], x[2]), b13 = set_ge(x[1], x[3]), b23 = set_ge(x[2], x[3]);
    keep[0] = maj3(b01, b02, b03);
    keep[1] = maj3(~b01, b12, b13);
    keep[2] = maj3(~b02, ~b12, b23);
    keep[3] = maj3(~b03, ~b13, ~b23);
}
__device__ __forceinline__ uint32_t keep_bits(const uint32_t (&keep)[4]) {
    return (keep[0] & 1u) | (keep[1] & 2u) | (keep[2] & 4u) | (keep[3] & 8u);
}
// Second largest of four values (the 2:4 group threshold), seven min/max.
__device__ __forceinline__ float second_largest4(const float (&x)[4]) {
    const float lo1 = fminf(x[0], x[1]), hi1 = fmaxf(x[0], x[1]);
    const float lo2 = fminf(x[2], x[3]), hi2 = fmaxf(x[2], x[3]);
    return fmaxf(fminf(hi1, hi2), fmaxf(lo1, lo2));
}
// Metadata nibble from keep bits with exactly two set: keep >> 1 is unique per pattern (1..6).
__device__ __forceinline__ uint32_t nibble_of_keep_lut(uint32_t keep) {
    constexpr uint32_t lut = (4u << 4) | (8u << 8) | (9u << 12) | (12u << 16) | (13u << 20) | (14u << 24);
    return (lut >> ((keep & 0xEu) << 1)) & 0xFu;
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
// 32-byte streaming accesses (eight fp32 at once, sm_100): one memory instruction where the 16-byte
// form needs two. The address must be 32-byte aligned.
__device__ __forceinline__ void ld_stream32(const float* p, float (&x)[8]) {
    asm volatile("ld.global.cs.v8.f32 {%0,%1,%2,%3,%4,%5,%6,%7}, [%8];"
                 : "=f"(x[0]), "=f"(x[1]), "=f"(x[2]), "=f"(x[3]), "=f"(x[4]), "=f"(x[5]), "=f"(x[6]), "=f"(x[7])
                 : "l"(p));
}
__device__ __forceinline__ void st_stream32(float* p, const float (&x)[8]) {
    asm volatile("st.global.cs.v8.f32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8};"
                 ::"l"(p), "f"(x[0]), "f"(x[1]), "f"(x[2]), "f"(x[3]), "f"(x[4]), "f"(x[5]), "f"(x[6]), "f"(x[7])
                 : "memory");
}
__host__ __device__ inline bool aligned32(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 31u) == 0; }

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
    // Raw storage of 8 elements, and p <- raw * round(f) element by element.
    struct Raw { uint4 a, b; };
    static __device__ __forceinline__ Raw load_raw(const float* p) { return Raw{ld_stream16(p), ld_stream16(p + 4)}; }
    static __device__ __forceinline__ void unpack(const Raw& r, float (&x)[8]) {
        x[0] = __uint_as_float(r.a.x); x[1] = __uint_as_float(r.a.y); x[2] = __uint_as_float(r.a.z); x[3] = __uint_as_float(r.a.w);
        x[4] = __uint_as_float(r.b.x); x[5] = __uint_as_float(r.b.y); x[6] = __uint_as_float(r.b.z); x[7] = __uint_as_float(r.b.w);
    }
    static __device__ __forceinline__ void square(const Raw& r, float (&x)[8]) {
        unpack(r, x);
#pragma unroll
        for (int i = 0; i < 8; ++i) x[i] = __fmul_rn(x[i], x[i]);
    }
    static __device__ __forceinline__ void round8(float (&)[8]) {}
    // The storage form of 8 values, and its store.
    static __device__ __forceinline__ Raw pack(const float (&x)[8]) {
        return Raw{make_uint4(__float_as_uint(x[0]), __float_as_uint(x[1]), __float_as_uint(x[2]), __float_as_uint(x[3])),
                   make_uint4(__float_as_uint(x[4]), __float_as_uint(x[5]), __float_as_uint(x[6]), __float_as_uint(x[7]))};
    }
    static __device__ __forceinline__ void store_raw(float* p, const Raw& r) {
        st_stream16(p, r.a);
        st_stream16(p + 4, r.b);
    }
    static __device__ __forceinline__ void store_product(float* p, const Raw& r, const float (&f)[8]) {
        st_stream16(p, make_uint4(__float_as_uint(__fmul_rn(__uint_as_float(r.a.x), f[0])),
                                  __float_as_uint(__fmul_rn(__uint_as_float(r.a.y), f[1])),
                                  __float_as_uint(__fmul_rn(__uint_as_float(r.a.z), f[2])),
                                  __float_as_uint(__fmul_rn(__uint_as_float(r.a.w), f[3]))));
        st_stream16(p + 4, make_uint4(__float_as_uint(__fmul_rn(__uint_as_float(r.b.x), f[4])),
                                      __float_as_uint(__fmul_rn(__uint_as_float(r.b.y), f[5])),
                                      __float_as_uint(__fmul_rn(__uint_as_float(r.b.z), f[6])),
                                      __float_as_uint(__fmul_rn(__uint_as_float(r.b.w), f[7]))));
    }
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
    static __device__ __forceinline__ float round(float x) { return bf16_round_int(x); }
    // Raw storage of 8 elements, and p <- raw * round(f): the factors are packed to bf16 pairs and
    // multiplied pairwise (one rounding of the exact product, as a bf16 tensor multiply does).
    struct Raw { uint4 a; };
    static __device__ __forceinline__ Raw load_raw(const __nv_bfloat16* p) { return Raw{ld_stream16(p)}; }
    static __device__ __forceinline__ void unpack(const Raw& r, float (&x)[8]) {
        const uint32_t w[4] = {r.a.x, r.a.y, r.a.z, r.a.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            x[2 * i] = __uint_as_float(w[i] << 16);
            x[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
    static __device__ __forceinline__ Raw pack(const float (&x)[8]) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            __nv_bfloat162 h = __floats2bfloat162_rn(x[2 * i], x[2 * i + 1]);
            w[i] = *reinterpret_cast<uint32_t*>(&h);
        }
        return Raw{make_uint4(w[0], w[1], w[2], w[3])};
    }
    static __device__ __forceinline__ void store_raw(__nv_bfloat16* p, const Raw& r) { st_stream16(p, r.a); }
    // Rounds eight values to the storage type and back, two per conversion.
    static __device__ __forceinline__ void round8(float (&x)[8]) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const __nv_bfloat162 h = __floats2bfloat162_rn(x[2 * i], x[2 * i + 1]);
            const uint32_t u = *reinterpret_cast<const uint32_t*>(&h);
            x[2 * i] = __uint_as_float(u << 16);
            x[2 * i + 1] = __uint_as_float(u & 0xffff0000u);
        }
    }
    // x <- round(raw * raw): the packed multiply rounds the exact product once, as the tensor op does
    static __device__ __forceinline__ void square(const Raw& r, float (&x)[8]) {
        const uint32_t w[4] = {r.a.x, r.a.y, r.a.z, r.a.w};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const __nv_bfloat162 v = *reinterpret_cast<const __nv_bfloat162*>(&w[i]);
            const __nv_bfloat162 sq = __hmul2(v, v);
            const uint32_t u = *reinterpret_cast<const uint32_t*>(&sq);
            x[2 * i] = __uint_as_float(u << 16);
            x[2 * i + 1] = __uint_as_float(u & 0xffff0000u);
        }
    }
    static __device__ __forceinline__ void store_product(__nv_bfloat16* p, const Raw& r, const float (&f)[8]) {
        const uint32_t w[4] = {r.a.x, r.a.y, r.a.z, r.a.w};
        uint32_t o[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            const __nv_bfloat162 e = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
            const __nv_bfloat162 prod = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&w[i]), e);
            o[i] = *reinterpret_cast<const uint32_t*>(&prod);
        }
        st_stream16(p, make_uint4(o[0], o[1], o[2], o[3]));
    }
};


// ---- warp-span decomposition of the streaming passes ------------------------------------
// A warp walks the tensor in spans of 256 consecutive elements. Lane l owns two 2:4 groups of
// the span: elements [4l, 4l+4) and [128+4l, 128+4l+4). Every warp-wide access is then one
// contiguous run (512 B for fp32, 256 B for bf16, 128 B for int8): full sectors, no sector is
// touched by two instructions. x[0..3] is the first group, x[4..7] the second.
struct SpanPos {
    int64_t a, b;  // element index of the lane's first / second group
    bool va, vb;   // the group lies inside the tensor (n is a multiple of 8)
};
__device__ __forceinline__ SpanPos span_pos(int64_t span, int lane, int64_t n) {
    SpanPos p;
    p.a = span * 256 + 4 * lane;
    p.b = p.a + 128;
    p.va = p.a + 4 <= n;
    p.vb = p.b + 4 <= n;
    return p;
}
#define SF_SPAN_LOOP(span, n)                                                                   \
    for (int64_t span = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5),           \
                 _spans = ((n) + 255) / 256, _step = (int64_t)gridDim.x * (blockDim.x >> 5);    \
         span < _spans; span += _step)

template <typename T>
struct Span8;
template <>
struct Span8<float> {
    static __device__ __forceinline__ void load(const float* p, const SpanPos& s, float (&x)[8]) {
        uint4 a = s.va ? ld_stream16(p + s.a) : make_uint4(0, 0, 0, 0);
        uint4 b = s.vb ? ld_stream16(p + s.b) : make_uint4(0, 0, 0, 0);
        x[0] = __uint_as_float(a.x); x[1] = __uint_as_float(a.y);
        x[2] = __uint_as_float(a.z); x[3] = __uint_as_float(a.w);
        x[4] = __uint_as_float(b.x); x[5] = __uint_as_float(b.y);
        x[6] = __uint_as_float(b.z); x[7] = __uint_as_float(b.w);
    }
    static __device__ __forceinline__ void store(float* p, const SpanPos& s, const float (&x)[8]) {
        if (s.va) st_stream16(p + s.a, make_uint4(__float_as_uint(x[0]), __float_as_uint(x[1]),
                                                   __float_as_uint(x[2]), __float_as_uint(x[3])));
        if (s.vb) st_stream16(p + s.b, make_uint4(__float_as_uint(x[4]), __float_as_uint(x[5]),
                                                   __float_as_uint(x[6]), __float_as_uint(x[7])));
    }
    static __device__ __forceinline__ float round(float x) { return x; }
};
template <>
struct Span8<__nv_bfloat16> {
    static __device__ __forceinline__ void load(const __nv_bfloat16* p, const SpanPos& s, float (&x)[8]) {
        uint2 a = s.va ? ld_stream8(p + s.a) : make_uint2(0, 0);
        uint2 b = s.vb ? ld_stream8(p + s.b) : make_uint2(0, 0);
        const uint32_t w[4] = {a.x, a.y, b.x, b.y};
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            x[2 * i] = __uint_as_float(w[i] << 16);
            x[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
        }
    }
    static __device__ __forceinline__ void store(__nv_bfloat16* p, const SpanPos& s, const float (&x)[8]) {
        uint32_t w[4];
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            __nv_bfloat162 h = __floats2bfloat162_rn(x[2 * i], x[2 * i + 1]);
            w[i] = *reinterpret_cast<uint32_t*>(&h);
        }
        if (s.va) st_stream8(p + s.a, make_uint2(w[0], w[1]));
        if (s.vb) st_stream8(p + s.b, make_uint2(w[2], w[3]));
    }
    static __device__ __forceinline__ float round(float x) { return bf16_round_int(x); }
};
// +1 / -1 probes stored as int8: the float is built from the sign bit.
template <>
struct Span8<int8_t> {
    static __device__ __forceinline__ void load(const int8_t* p, const SpanPos& s, float (&x)[8]) {
        const uint32_t a = s.va ? __ldcs(reinterpret_cast<const uint32_t*>(p + s.a)) : 0u;
        const uint32_t b = s.vb ? __ldcs(reinterpret_cast<const uint32_t*>(p + s.b)) : 0u;
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            x[i] = __uint_as_float(0x3f800000u | (((a >> (8 * i)) & 0x80u) << 24));
            x[4 + i] = __uint_as_float(0x3f800000u | (((b >> (8 * i)) & 0x80u) << 24));
        }
    }
};
// Eight +-1 probe signs held as int8 in one 8-byte load (only the sign bit is read).
template <>
struct Vec8<int8_t> {
    // The sign bit of each of 8 values (+1 / -1 probes), moved to the float sign position.
    static __device__ __forceinline__ void load_signs(const int8_t* p, uint32_t (&sb)[8]) {
        const uint2 r = __ldcs(reinterpret_cast<const uint2*>(p));
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            sb[i] = (r.x << (24 - 8 * i)) & 0x80000000u;
            sb[4 + i] = (r.y << (24 - 8 * i)) & 0x80000000u;
        }
    }
    static __device__ __forceinline__ void load(const int8_t* p, float (&x)[8]) {
        const uint2 r = __ldcs(reinterpret_cast<const uint2*>(p));
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            x[i] = __uint_as_float(0x3f800000u | (((r.x >> (8 * i)) & 0x80u) << 24));
            x[4 + i] = __uint_as_float(0x3f800000u | (((r.y >> (8 * i)) & 0x80u) << 24));
        }
    }
};
// Packed 2:4 metadata of a span: byte j of the tensor holds groups 2j (low nibble) and 2j+1.
// Lanes 2j and 2j+1 hold those two groups; the even lane writes the byte of the first halves,
// the odd lane the byte of the second halves. Must be called by the whole warp.
__device__ __forceinline__ void store_meta_span(uint8_t* meta, const SpanPos& s, uint32_t nib_a, uint32_t nib_b) {
    const uint32_t pa = __shfl_xor_sync(0xffffffffu, nib_a, 1);
    const uint32_t pb = __shfl_xor_sync(0xffffffffu, nib_b, 1);
    if (((threadIdx.x & 1) == 0)) {
        if (s.va) meta[s.a >> 3] = (uint8_t)(nib_a | (pa << 4));
    } else {
        if (s.vb) meta[s.b >> 3] = (uint8_t)(pb | (nib_b << 4));
    }
}

}  // namespace sf
