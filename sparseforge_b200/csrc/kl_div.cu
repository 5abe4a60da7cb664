// Distillation KL loss over a large vocabulary, one pass per direction.
//
// Reference: Distill_Model.kl_loss, legacy/sparse_modeling.py:1749-1828. Per token row, with
// a = clamp(student, -L, L) / Temp and b = clamp(teacher, -L, L) / Temp:
//     KL_row = sum_v softmax(b)_v (log_softmax(b)_v - log_softmax(a)_v)
//            = [sum_v e^{b_v - lse_b} (b_v - a_v)] - lse_b + lse_a
// so one sweep with running maxima gives lse_a, lse_b and the weighted sum together; the
// reference makes about ten passes over [chunk, vocab] fp32 temporaries.
// Backward (student only): dKL_row/ds_v = (softmax(a)_v - softmax(b)_v) / Temp where |s_v| < L
// (the clamp passes no gradient outside).
#include "common.cuh"

namespace sf {

constexpr int kKlThreads = 256;

struct RowAcc {
    float max_a, sum_a;  // running maximum and sum of e^{a - max_a}
    float max_b, sum_b;  // the same for b
    float wsum;          // sum of e^{b - max_b} (b - a)
};

// clamp that keeps NaN (fminf / fmaxf would return the bound), as the tensor clamp does
__device__ __forceinline__ float clamp_keep_nan(float x, float lim) {
    float y;
    asm("max.NaN.f32 %0, %1, %2;\n\tmin.NaN.f32 %0, %0, %3;" : "=&f"(y) : "f"(x), "f"(-lim), "f"(lim));
    return y;
}
__device__ __forceinline__ float ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ void acc_init(RowAcc& r) {
    r.max_a = -INFINITY; r.sum_a = 0.f; r.max_b = -INFINITY; r.sum_b = 0.f; r.wsum = 0.f;
}
__device__ __forceinline__ void acc_add(RowAcc& r, float a, float b) {
    if (a > r.max_a) { r.sum_a *= __expf(r.max_a - a); r.max_a = a; }
    r.sum_a += __expf(a - r.max_a);  // a NaN logit never becomes the maximum but makes the sum NaN
    if (b > r.max_b) {
        const float sc = __expf(r.max_b - b);
        r.sum_b *= sc; r.wsum *= sc; r.max_b = b;
    }
    const float e = __expf(b - r.max_b);
    r.sum_b += e;
    r.wsum = fmaf(e, b - a, r.wsum);
}
// Eight logits of each tensor at once: the running maxima move at most once per chunk, so the
// common case is one subtraction, one ex2 and one addition per logit. Internally the exponent is
// taken in base 2 (logits scaled by log2 e); max_a / max_b are kept in natural units.
__device__ __forceinline__ void acc_add8(RowAcc& r, const float (&a)[8], const float (&b)[8], float max_logit,
                                         float inv_temp) {
    constexpr float kLog2e = 1.4426950408889634f;
    float x[8], y[8];
    float mx = -INFINITY, my = -INFINITY;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        x[i] = clamp_keep_nan(a[i], max_logit) * inv_temp;
        y[i] = clamp_keep_nan(b[i], max_logit) * inv_temp;
        mx = fmaxf(mx, x[i]);
        my = fmaxf(my, y[i]);
    }
    if (mx > r.max_a) { r.sum_a *= ex2((r.max_a - mx) * kLog2e); r.max_a = mx; }
    if (my > r.max_b) {
        const float sc = ex2((r.max_b - my) * kLog2e);
        r.sum_b *= sc; r.wsum *= sc; r.max_b = my;
    }
    const float ma2 = r.max_a * kLog2e, mb2 = r.max_b * kLog2e;
    float sa = 0.f, sb = 0.f, ws = 0.f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        sa += ex2(fmaf(x[i], kLog2e, -ma2));  // NaN logits make the sums NaN (they never become the maximum)
        const float e = ex2(fmaf(y[i], kLog2e, -mb2));
        sb += e;
        ws = fmaf(e, y[i] - x[i], ws);
    }
    r.sum_a += sa; r.sum_b += sb; r.wsum += ws;
}

__device__ __forceinline__ void acc_merge(RowAcc& r, const RowAcc& o) {
    const float ma = fmaxf(r.max_a, o.max_a);
    r.sum_a = r.sum_a * (r.max_a == -INFINITY ? 0.f : __expf(r.max_a - ma)) +
              o.sum_a * (o.max_a == -INFINITY ? 0.f : __expf(o.max_a - ma));
    r.max_a = ma;
    const float mb = fmaxf(r.max_b, o.max_b);
    const float s1 = r.max_b == -INFINITY ? 0.f : __expf(r.max_b - mb);
    const float s2 = o.max_b == -INFINITY ? 0.f : __expf(o.max_b - mb);
    r.sum_b = r.sum_b * s1 + o.sum_b * s2;
    r.wsum = r.wsum * s1 + o.wsum * s2;
    r.max_b = mb;
}
__device__ __forceinline__ RowAcc acc_shfl_xor(const RowAcc& r, int o) {
    RowAcc t;
    t.max_a = __shfl_xor_sync(0xffffffffu, r.max_a, o);
    t.sum_a = __shfl_xor_sync(0xffffffffu, r.sum_a, o);
    t.max_b = __shfl_xor_sync(0xffffffffu, r.max_b, o);
    t.sum_b = __shfl_xor_sync(0xffffffffu, r.sum_b, o);
    t.wsum = __shfl_xor_sync(0xffffffffu, r.wsum, o);
    return t;
}

// One block per token row (grid-stride over rows). row_kl[row] = KL of the row (before the
// Temp^2 / tokens factor); lse[2 row] = lse_a, lse[2 row + 1] = lse_b for the backward pass.
template <typename T>
__global__ void __launch_bounds__(kKlThreads)
kl_div_fwd_kernel(const T* __restrict__ student, const T* __restrict__ teacher, int64_t rows, int64_t vocab,
                  float inv_temp, float max_logit, float* __restrict__ row_kl, float* __restrict__ lse) {
    __shared__ RowAcc part[kKlThreads / 32];
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    const int64_t chunks = vocab / 8;
    for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const T* s = student + row * vocab;
        const T* t = teacher + row * vocab;
        RowAcc r;
        acc_init(r);
        for (int64_t c = threadIdx.x; c < chunks; c += kKlThreads) {
            float a[8], b[8];
            Vec8<T>::load(s + c * 8, a);
            Vec8<T>::load(t + c * 8, b);
            acc_add8(r, a, b, max_logit, inv_temp);
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) acc_merge(r, acc_shfl_xor(r, o));
        if (lane == 0) part[wid] = r;
        __syncthreads();
        if (wid == 0) {
            RowAcc q;
            if (lane < kKlThreads / 32) q = part[lane]; else acc_init(q);
#pragma unroll
            for (int o = 4; o > 0; o >>= 1) acc_merge(q, acc_shfl_xor(q, o));
            if (lane == 0) {
                const float lse_a = q.max_a + logf(q.sum_a);
                const float lse_b = q.max_b + logf(q.sum_b);
                row_kl[row] = q.wsum / q.sum_b - lse_b + lse_a;
                lse[2 * row] = lse_a;
                lse[2 * row + 1] = lse_b;
            }
        }
        __syncthreads();
    }
}

// grad[row, v] = row_scale[row] * (softmax(a)_v - softmax(b)_v) * inv_temp inside the clamp, else 0.
// row_scale already holds upstream gradient * Temp^2 / tokens, or 0 for a row of a skipped chunk.
template <typename T>
__global__ void __launch_bounds__(kKlThreads)
kl_div_bwd_kernel(const T* __restrict__ student, const T* __restrict__ teacher, const float* __restrict__ lse,
                  const float* __restrict__ row_scale, int64_t rows, int64_t vocab, float inv_temp, float max_logit,
                  T* __restrict__ grad) {
    const int64_t chunks = vocab / 8;
    for (int64_t row = blockIdx.x; row < rows; row += gridDim.x) {
        const T* s = student + row * vocab;
        const T* t = teacher + row * vocab;
        T* g = grad + row * vocab;
        const float lse_a = lse[2 * row], lse_b = lse[2 * row + 1];
        const float scale = row_scale[row] * inv_temp;
        for (int64_t c = threadIdx.x; c < chunks; c += kKlThreads) {
            float a[8], b[8], o[8];
            Vec8<T>::load(s + c * 8, a);
            Vec8<T>::load(t + c * 8, b);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const bool inside = a[i] > -max_logit && a[i] < max_logit;
                const float av = clamp_keep_nan(a[i], max_logit) * inv_temp;
                const float bv = clamp_keep_nan(b[i], max_logit) * inv_temp;
                // a dropped row (scale 0) gets exact zeros even if its logits hold NaN
                o[i] = (inside && scale != 0.0f) ? scale * (__expf(av - lse_a) - __expf(bv - lse_b)) : 0.0f;
            }
            Vec8<T>::store(g + c * 8, o);
        }
    }
}

static int kl_grid(int64_t rows) {
    const int64_t cap = 148 * 8;
    return (int)(rows < cap ? rows : cap);
}

}  // namespace sf

using namespace sf;

extern "C" {

int sf_kl_div_fwd(const void* student, const void* teacher, int dtype, int64_t rows, int64_t vocab, double temperature,
                  double max_logit, float* row_kl, float* lse, void* stream) {
    SF_CHECK_ARG(student && teacher && row_kl && lse, "sf_kl_div_fwd: student, teacher, row_kl, lse must be non-null");
    SF_CHECK_ARG(rows > 0 && vocab > 0 && vocab % 8 == 0, "sf_kl_div_fwd: vocab=%lld must be a positive multiple of 8", (long long)vocab);
    SF_CHECK_ARG(dtype == SF_F32 || dtype == SF_BF16, "sf_kl_div_fwd: dtype must be SF_F32 or SF_BF16");
    SF_CHECK_ARG(temperature > 0.0, "sf_kl_div_fwd: temperature must be positive");
    if (!aligned16(student) || !aligned16(teacher)) return fail(SF_ERR_ALIGNMENT, "sf_kl_div_fwd: logits must be 16-byte aligned");
    cudaStream_t st = (cudaStream_t)stream;
    const float it = (float)(1.0 / temperature), ml = (float)max_logit;
    if (dtype == SF_F32)
        kl_div_fwd_kernel<float><<<kl_grid(rows), kKlThreads, 0, st>>>((const float*)student, (const float*)teacher, rows, vocab, it, ml, row_kl, lse);
    else
        kl_div_fwd_kernel<__nv_bfloat16><<<kl_grid(rows), kKlThreads, 0, st>>>((const __nv_bfloat16*)student, (const __nv_bfloat16*)teacher,
                                                                              rows, vocab, it, ml, row_kl, lse);
    SF_CHECK_CUDA(cudaGetLastError());
    return SF_OK;
}

int sf_kl_div_bwd(const void* student, const void* teacher, int dtype, const float* lse, const float* row_scale,
                  int64_t rows, int64_t vocab, double temperature, double max_logit, void* grad, void* stream) {
    SF_CHECK_ARG(student && teacher && lse && row_scale && grad, "sf_kl_div_bwd: all pointers must be non-null");
    SF_CHECK_ARG(rows > 0 && vocab > 0 && vocab % 8 == 0, "sf_kl_div_bwd: vocab=%lld must be a positive multiple of 8", (long long)vocab);
    SF_CHECK_ARG(dtype == SF_F32 || dtype == SF_BF16, "sf_kl_div_bwd: dtype must be SF_F32 or SF_BF16");
    SF_CHECK_ARG(temperature > 0.0, "sf_kl_div_bwd: temperature must be positive");
    if (!aligned16(student) || !aligned16(teacher) || !aligned16(grad))
        return fail(SF_ERR_ALIGNMENT, "sf_kl_div_bwd: logits and grad must be 16-byte aligned");
    cudaStream_t st = (cudaStream_t)stream;
    const float it = (float)(1.0 / temperature), ml = (float)max_logit;
    if (dtype == SF_F32)
        kl_div_bwd_kernel<float><<<kl_grid(rows), kKlThreads, 0, st>>>((const float*)student, (const float*)teacher, lse, row_scale, rows,
                                                                       vocab, it, ml, (float*)grad);
    else
        kl_div_bwd_kernel<__nv_bfloat16><<<kl_grid(rows), kKlThreads, 0, st>>>((const __nv_bfloat16*)student, (const __nv_bfloat16*)teacher,
                                                                              lse, row_scale, rows, vocab, it, ml, (__nv_bfloat16*)grad);
    SF_CHECK_CUDA(cudaGetLastError());
    return SF_OK;
}

}  // extern "C"
