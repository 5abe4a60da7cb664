// HBM-bound passes of the SparseLinear hot path: Hutchinson accumulate + score,
// 2:4 soft-mask update + hard projection + masked-weight emit, mask-aware AdamW,
// mask statistics, bias gradient. Each thread owns 8 consecutive elements (two 2:4
// groups) and moves them with 16-byte streaming accesses; grids are sized from the
// SM count and walk the tensor with a grid-stride loop.
#include <mutex>
#include <unordered_map>

#include "common.cuh"

namespace sf {

static thread_local char g_err[512];
char* last_error_buffer() { return g_err; }

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

int sm_count() {
    static thread_local int cached_dev = -1;
    static thread_local int cached = 0;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 148;
    if (dev != cached_dev) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
            n = 148;
        cached = n;
        cached_dev = dev;
    }
    return cached;
}

constexpr int kThreads = 256;
constexpr int kMaxPartialBlocks = 2048;

// Blocks for a grid-stride pass over `chunks` 8-element chunks: a multiple of the SM count.
static inline int grid_for(int64_t chunks, int blocks_per_sm) {
    int64_t need = (chunks + kThreads - 1) / kThreads;
    int64_t cap = (int64_t)sm_count() * blocks_per_sm;
    if (need < 1) need = 1;
    return (int)(need < cap ? need : cap);
}

// Grid of exactly one resident wave of `kernel` (SMs x blocks that fit per SM), so the
// grid-stride loop gives every block the same share and there is no partial last wave.
static int grid_one_wave(const void* kernel, int64_t chunks) {
    static std::mutex mu;
    static std::unordered_map<const void*, int> cache;
    int per_sm = 0;
    {
        std::lock_guard<std::mutex> lock(mu);
        auto it = cache.find(kernel);
        if (it != cache.end()) per_sm = it->second;
    }
    if (per_sm == 0) {
        if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kThreads, 0) != cudaSuccess || per_sm <= 0)
            per_sm = 4;
        std::lock_guard<std::mutex> lock(mu);
        cache[kernel] = per_sm;
    }
    return grid_for(chunks, per_sm);
}

// ---------------------------------------------------------------------------------------
// Hutchinson accumulate + score + partial sums
// ---------------------------------------------------------------------------------------
constexpr int kMetricNone = -1;

template <typename TW, typename TV, int METRIC, bool ACCUM>
__global__ void __launch_bounds__(kThreads)
hutch_score_kernel(const TW* __restrict__ hvp, const TV* __restrict__ v, float* __restrict__ H,
                   const TW* __restrict__ W, const TW* __restrict__ aux, float aux_scalar,
                   float* __restrict__ score, double* __restrict__ partials, int64_t chunks,
                   float beta, float one_minus_beta) {
    double acc_s = 0.0, acc_s2 = 0.0;
    const float eps = 1e-8f;
    const int64_t n = chunks * 8;
    SF_SPAN_LOOP(span, n) {
        const SpanPos pos = span_pos(span, threadIdx.x & 31, n);
        constexpr bool SCORE = METRIC != kMetricNone;  // kMetricNone: update H only
        float w[8], h[8], s[8];
        if (SCORE) Span8<TW>::load(W, pos, w);
        constexpr bool NEED_H = (METRIC == SF_METRIC_HESSIAN_OBD || METRIC == SF_METRIC_HESSIAN_RATIO ||
                                 METRIC == SF_METRIC_HESSIAN) || ACCUM;
        if (NEED_H) Span8<float>::load(H, pos, h);
        if (ACCUM) {
            float hv[8], sg[8];
            Span8<TW>::load(hvp, pos, hv);
            Span8<TV>::load(v, pos, sg);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                // diag_est = clamp(hvp*v, min=0) in the weight dtype; H.mul_(beta).add_(d, alpha=1-beta)
                float d = fmaxf(Vec8<TW>::round(__fmul_rn(hv[i], sg[i])), 0.0f);
                h[i] = __fmaf_rn(one_minus_beta, d, __fmul_rn(h[i], beta));
            }
            Span8<float>::store(H, pos, h);
        }
        if (!SCORE) continue;
        if (METRIC == SF_METRIC_MOVEMENT) {
            float g[8];
            Span8<TW>::load(aux, pos, g);
#pragma unroll
            for (int i = 0; i < 8; ++i)
                s[i] = Vec8<TW>::round(__fdiv_rn(fabsf(Vec8<TW>::round(__fmul_rn(w[i], g[i]))), aux_scalar));
        } else {
            if (METRIC == SF_METRIC_HESSIAN_OBD) {
                // round(w * w) in the weight dtype, two per conversion
#pragma unroll
                for (int i = 0; i < 8; ++i) w[i] = __fmul_rn(w[i], w[i]);
                Vec8<TW>::round8(w);
            }
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                if (METRIC == SF_METRIC_HESSIAN_OBD) {
                    s[i] = __fmul_rn(__fadd_rn(h[i], eps), w[i]);
                } else if (METRIC == SF_METRIC_HESSIAN_RATIO) {
                    s[i] = __fdiv_rn(fabsf(w[i]), __fsqrt_rn(__fadd_rn(h[i], eps)));
                } else if (METRIC == SF_METRIC_HESSIAN) {
                    s[i] = h[i];
                } else {
                    s[i] = fabsf(w[i]);
                }
            }
        }
        Span8<float>::store(score, pos, s);
        // eight values are summed in fp32, the running totals are kept in fp64
        float ps = 0.0f, ps2 = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            ps += s[i];
            ps2 = fmaf(s[i], s[i], ps2);
        }
        acc_s += (double)ps;
        acc_s2 += (double)ps2;
    }
    if (METRIC == kMetricNone) return;
    __shared__ double red[2][kThreads / 32];
    acc_s = warp_sum(acc_s);
    acc_s2 = warp_sum(acc_s2);
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    if (lane == 0) { red[0][wid] = acc_s; red[1][wid] = acc_s2; }
    __syncthreads();
    if (threadIdx.x == 0) {
        double a = 0.0, b = 0.0;
#pragma unroll
        for (int i = 0; i < kThreads / 32; ++i) { a += red[0][i]; b += red[1][i]; }
        partials[2 * blockIdx.x] = a;
        partials[2 * blockIdx.x + 1] = b;
    }
}

// out = a + b (the joint score of a gate / up pair) with this block's partial sums of out and out^2.
__global__ void __launch_bounds__(kThreads)
score_sum_kernel(const float* __restrict__ a, const float* __restrict__ b, float* __restrict__ out,
                 double* __restrict__ partials, int64_t chunks) {
    double acc_s = 0.0, acc_s2 = 0.0;
    for (int64_t c = (int64_t)blockIdx.x * kThreads + threadIdx.x; c < chunks; c += (int64_t)gridDim.x * kThreads) {
        float x[8], y[8];
        Vec8<float>::load(a + c * 8, x);
        Vec8<float>::load(b + c * 8, y);
        float ps = 0.0f, ps2 = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            x[i] = __fadd_rn(x[i], y[i]);
            ps += x[i];
            ps2 = fmaf(x[i], x[i], ps2);
        }
        Vec8<float>::store(out + c * 8, x);
        acc_s += (double)ps;
        acc_s2 += (double)ps2;
    }
    __shared__ double red[2][kThreads / 32];
    acc_s = warp_sum(acc_s);
    acc_s2 = warp_sum(acc_s2);
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    if (lane == 0) { red[0][wid] = acc_s; red[1][wid] = acc_s2; }
    __syncthreads();
    if (threadIdx.x == 0) {
        double sa = 0.0, sb = 0.0;
#pragma unroll
        for (int i = 0; i < kThreads / 32; ++i) { sa += red[0][i]; sb += red[1][i]; }
        partials[2 * blockIdx.x] = sa;
        partials[2 * blockIdx.x + 1] = sb;
    }
}

// ---------------------------------------------------------------------------------------
// WANDA: per-input-channel activation energy and the score |W| * sqrt(scaler_row + eps)
// ---------------------------------------------------------------------------------------
__device__ __forceinline__ float to_float(float x) { return x; }
__device__ __forceinline__ float to_float(__nv_bfloat16 x) { return __bfloat162float(x); }
template <typename T> __device__ __forceinline__ T from_float(float x);
template <> __device__ __forceinline__ float from_float<float>(float x) { return x; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float x) { return __float2bfloat16_rn(x); }

constexpr int kWandaRowLanes = 8;                      // row lanes per block
constexpr int kWandaColsPerBlock = (kThreads / kWandaRowLanes) * 8;  // 32 threads x 8 columns
constexpr int kWandaMaxRowBlocks = 64;

// partial[blockIdx.y][c] = sum over this block's rows of x[r, c]^2 (fp32, rows in a fixed order)
template <typename TX>
__global__ void __launch_bounds__(kThreads)
wanda_colsumsq_kernel(const TX* __restrict__ x, int64_t rows, int64_t cols, float* __restrict__ partial) {
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const int64_t c0 = (int64_t)blockIdx.x * kWandaColsPerBlock + tx * 8;
    float acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = 0.f;
    if (c0 < cols)
        for (int64_t r = (int64_t)blockIdx.y * kWandaRowLanes + ty; r < rows; r += (int64_t)gridDim.y * kWandaRowLanes) {
            float v[8];
            Vec8<TX>::load(x + r * cols + c0, v);
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] = fmaf(v[i], v[i], acc[i]);
        }
    __shared__ float red[kWandaRowLanes][kWandaColsPerBlock + 8];
#pragma unroll
    for (int i = 0; i < 8; ++i) red[ty][tx * 8 + i] = acc[i];
    __syncthreads();
    const int64_t c = (int64_t)blockIdx.x * kWandaColsPerBlock + threadIdx.x;
    if (threadIdx.x < kWandaColsPerBlock && c < cols) {
        float s = 0.f;
#pragma unroll
        for (int j = 0; j < kWandaRowLanes; ++j) s += red[j][threadIdx.x];
        partial[(int64_t)blockIdx.y * cols + c] = s;
    }
}

// scaler_row <- round(scaler_row * keep) then round(scaler_row + norm2(x[:, c])^2 / denom), the two
// in-place tensor operations of add_batch (the norm is a square root that is squared again).
template <typename TS>
__global__ void __launch_bounds__(kThreads)
wanda_scaler_update_kernel(const float* __restrict__ partial, int row_blocks, int64_t cols, float keep, float denom,
                           TS* __restrict__ scaler) {
    const int64_t c = (int64_t)blockIdx.x * kThreads + threadIdx.x;
    if (c >= cols) return;
    float s = 0.f;
    for (int j = 0; j < row_blocks; ++j) s += partial[(int64_t)j * cols + c];
    const float nrm = __fsqrt_rn(s);
    const float add = __fdiv_rn(__fmul_rn(nrm, nrm), denom);
    float cur = to_float(scaler[c]);
    cur = Vec8<TS>::round(__fmul_rn(cur, keep));
    cur = Vec8<TS>::round(__fadd_rn(cur, add));
    scaler[c] = from_float<TS>(cur);
}

// score = |W| * sqrt(scaler_row + eps) in the dtypes torch would use (bf16 arithmetic rounds after
// every operation; a bf16 weight times an fp32 scaler is an fp32 product), with partial sums.
template <typename TW, typename TS>
__global__ void __launch_bounds__(kThreads)
wanda_score_kernel(const TW* __restrict__ W, const TS* __restrict__ scaler, int64_t cols, float eps,
                   float* __restrict__ score, double* __restrict__ partials, int64_t chunks) {
    constexpr bool kRoundProduct = sizeof(TW) == 2 && sizeof(TS) == 2;
    double acc_s = 0.0, acc_s2 = 0.0;
    for (int64_t c = (int64_t)blockIdx.x * kThreads + threadIdx.x; c < chunks; c += (int64_t)gridDim.x * kThreads) {
        float w[8], sc[8], s[8];
        Vec8<TW>::load(W + c * 8, w);
        const int64_t col = (c * 8) % cols;
#pragma unroll
        for (int i = 0; i < 8; ++i) sc[i] = to_float(scaler[col + i]);
        float ps = 0.0f, ps2 = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float root = Vec8<TS>::round(__fsqrt_rn(Vec8<TS>::round(__fadd_rn(sc[i], eps))));
            const float prod = __fmul_rn(fabsf(w[i]), root);
            s[i] = kRoundProduct ? Vec8<TW>::round(prod) : prod;
            ps += s[i];
            ps2 = fmaf(s[i], s[i], ps2);
        }
        Vec8<float>::store(score + c * 8, s);
        acc_s += (double)ps;
        acc_s2 += (double)ps2;
    }
    __shared__ double red[2][kThreads / 32];
    acc_s = warp_sum(acc_s);
    acc_s2 = warp_sum(acc_s2);
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    if (lane == 0) { red[0][wid] = acc_s; red[1][wid] = acc_s2; }
    __syncthreads();
    if (threadIdx.x == 0) {
        double sa = 0.0, sb = 0.0;
#pragma unroll
        for (int i = 0; i < kThreads / 32; ++i) { sa += red[0][i]; sb += red[1][i]; }
        partials[2 * blockIdx.x] = sa;
        partials[2 * blockIdx.x + 1] = sb;
    }
}

// Summary of one soft mask for logging: twelve sums (count, sum m, sum m^2, entropy with the
// reference's fp32 clamp, counts below 0.5 / 0.1 / 0.01 and above 0.9 / 0.99 / 0.5, sums of the
// entries below and above 0.5), added to `out` with atomics.
__global__ void __launch_bounds__(kThreads)
mask_summary_kernel(const float* __restrict__ mask, int64_t n, float clamp_lo, float clamp_hi, double* __restrict__ out) {
    double acc[12];
#pragma unroll
    for (int i = 0; i < 12; ++i) acc[i] = 0.0;
    // eight elements at a time are summed in fp32 (entropy with fp32 logarithms: each term is good
    // to an fp32 ulp, which is what a logging statistic needs), the running totals are fp64
    for (int64_t i0 = ((int64_t)blockIdx.x * kThreads + threadIdx.x) * 8; i0 < n; i0 += (int64_t)gridDim.x * kThreads * 8) {
        float p[12];
#pragma unroll
        for (int i = 0; i < 12; ++i) p[i] = 0.f;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            if (i0 + e >= n) break;
            const float m = __ldcs(mask + i0 + e);
            p[0] += 1.f;
            p[1] += m;
            p[2] = fmaf(m, m, p[2]);
            const float mm = fminf(fmaxf(m, clamp_lo), clamp_hi);
            p[3] += -(mm * logf(mm)) - ((1.0f - mm) * logf(1.0f - mm));
            p[4] += m < 0.5f ? 1.f : 0.f;
            p[5] += m < 0.1f ? 1.f : 0.f;
            p[6] += m < 0.01f ? 1.f : 0.f;
            p[7] += m > 0.9f ? 1.f : 0.f;
            p[8] += m > 0.99f ? 1.f : 0.f;
            p[9] += m > 0.5f ? 1.f : 0.f;
            p[10] += m < 0.5f ? m : 0.f;
            p[11] += m > 0.5f ? m : 0.f;
        }
#pragma unroll
        for (int i = 0; i < 12; ++i) acc[i] += (double)p[i];
    }
    __shared__ double red[12][kThreads / 32];
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
#pragma unroll
    for (int i = 0; i < 12; ++i) {
        const double v = warp_sum(acc[i]);
        if (lane == 0) red[i][wid] = v;
    }
    __syncthreads();
    if (threadIdx.x < 12) {
        double a = 0.0;
#pragma unroll
        for (int i = 0; i < kThreads / 32; ++i) a += red[threadIdx.x][i];
        atomicAdd(&out[threadIdx.x], a);
    }
}

// Histogram of mask[idx[j]] over `bins` equal bins of [0, 1] (torch.histc: bin = trunc(x * bins),
// x = 1 in the last bin, values outside [0, 1] dropped), added to `hist`.
__global__ void __launch_bounds__(kThreads)
mask_sample_hist_kernel(const float* __restrict__ mask, const int64_t* __restrict__ idx, int64_t take, int bins,
                        double* __restrict__ hist) {
    for (int64_t j = (int64_t)blockIdx.x * kThreads + threadIdx.x; j < take; j += (int64_t)gridDim.x * kThreads) {
        const float x = mask[idx[j]];
        if (x >= 0.0f && x <= 1.0f) {
            int pos = (int)(__fmul_rn(__fdiv_rn(x, 1.0f), (float)bins));
            if (pos > bins - 1) pos = bins - 1;
            atomicAdd(&hist[pos], 1.0);
        }
    }
}

// One block folds the per-block partial sums in a fixed order (deterministic) and writes
// mean and population std + 1e-6 as fp32.
__global__ void __launch_bounds__(kThreads)
score_norm_finalize_kernel(double* __restrict__ partials, int nblocks, double n,
                           float* __restrict__ norm) {
    __shared__ double red[2][kThreads];
    double a = 0.0, b = 0.0;
    for (int i = threadIdx.x; i < nblocks; i += kThreads) { a += partials[2 * i]; b += partials[2 * i + 1]; }
    red[0][threadIdx.x] = a;
    red[1][threadIdx.x] = b;
    __syncthreads();
    for (int s = kThreads / 2; s > 0; s >>= 1) {
        if (threadIdx.x < s) {
            red[0][threadIdx.x] += red[0][threadIdx.x + s];
            red[1][threadIdx.x] += red[1][threadIdx.x + s];
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        double mean = red[0][0] / n;
        double var = red[1][0] / n - mean * mean;
        if (var < 0.0) var = 0.0;
        norm[0] = (float)mean;
        norm[1] = __fadd_rn((float)sqrt(var), 1e-6f);
        // the raw sums stay available to callers that combine several shards of one layer
        partials[0] = red[0][0];
        partials[1] = red[1][0];
    }
}

__global__ void score_norm_from_sums_kernel(const double* __restrict__ sums, double n, float* __restrict__ norm) {
    if (threadIdx.x == 0 && blockIdx.x == 0) {
        double mean = sums[0] / n;
        double var = sums[1] / n - mean * mean;
        if (var < 0.0) var = 0.0;
        norm[0] = (float)mean;
        norm[1] = __fadd_rn((float)sqrt(var), 1e-6f);
    }
}

template <typename TW, typename TV, bool ACCUM>
static int launch_hutch_score(int metric, const void* hvp, const void* v, float* H, const void* W,
                              const void* aux, float aux_scalar, float* score, double* scratch,
                              int64_t chunks, double beta_d, int& grid, cudaStream_t st) {
    const float beta = (float)beta_d;
    const float omb = (float)(1.0 - beta_d);
#define SF_LAUNCH_HS(M)                                                                          \
    do {                                                                                         \
        auto kern = hutch_score_kernel<TW, TV, M, ACCUM>;                                        \
        grid = grid_one_wave((const void*)kern, chunks);                                         \
        if (grid > kMaxPartialBlocks) grid = kMaxPartialBlocks;                                  \
        kern<<<grid, kThreads, 0, st>>>((const TW*)hvp, (const TV*)v, H, (const TW*)W, (const TW*)aux, aux_scalar, \
                                        score, scratch, chunks, beta, omb);                      \
    } while (0)
    switch (score == nullptr ? kMetricNone : metric) {
        case kMetricNone: SF_LAUNCH_HS(kMetricNone); break;
        case SF_METRIC_HESSIAN_OBD: SF_LAUNCH_HS(SF_METRIC_HESSIAN_OBD); break;
        case SF_METRIC_HESSIAN_RATIO: SF_LAUNCH_HS(SF_METRIC_HESSIAN_RATIO); break;
        case SF_METRIC_MAGNITUDE: SF_LAUNCH_HS(SF_METRIC_MAGNITUDE); break;
        case SF_METRIC_HESSIAN: SF_LAUNCH_HS(SF_METRIC_HESSIAN); break;
        case SF_METRIC_MOVEMENT: SF_LAUNCH_HS(SF_METRIC_MOVEMENT); break;
        default: return fail(SF_ERR_BAD_ARG, "sf_hutch_score: unknown metric %d", metric);
    }
#undef SF_LAUNCH_HS
    return SF_OK;
}

// ---------------------------------------------------------------------------------------
// Gradient EMA (movement metric) and the g^2 Hessian proxy in one pass over the gradient:
//   grad_ema.mul_(b).add_(g, alpha = 1 - b)           in the weight dtype
//   H.mul_(b).add_(g * g, alpha = 1 - b)              H fp32, g * g rounded to the gradient dtype
// ---------------------------------------------------------------------------------------
template <typename TW>
__global__ void __launch_bounds__(kThreads)
grad_hessian_ema_kernel(const TW* __restrict__ g, TW* __restrict__ grad_ema, float* __restrict__ H, int64_t n,
                        float beta, float one_minus_beta) {
    SF_SPAN_LOOP(span, n) {
        const SpanPos pos = span_pos(span, threadIdx.x & 31, n);
        float gv[8], e[8];
        Span8<TW>::load(g, pos, gv);
        Span8<TW>::load(grad_ema, pos, e);
#pragma unroll
        for (int i = 0; i < 8; ++i)
            e[i] = __fmaf_rn(one_minus_beta, gv[i], Vec8<TW>::round(__fmul_rn(e[i], beta)));
        Span8<TW>::store(grad_ema, pos, e);
        if (H != nullptr) {
            float h[8];
            Span8<float>::load(H, pos, h);
#pragma unroll
            for (int i = 0; i < 8; ++i)
                h[i] = __fmaf_rn(one_minus_beta, Vec8<TW>::round(__fmul_rn(gv[i], gv[i])), __fmul_rn(h[i], beta));
            Span8<float>::store(H, pos, h);
        }
    }
}

// ---------------------------------------------------------------------------------------
// 2:4 soft-mask update + projection + masked weight + metadata + stats
// ---------------------------------------------------------------------------------------
struct MaskUpdateParams {
    float neg_log2e_over_t;  // -log2(e) / (T + 1e-8)
    float a, one_minus_a;
    float pen;
    int penalty_mode;
    float beta_s, one_minus_beta_s;
    float bin_lo, bin_hi;  // 1-d, 1+d
    int binarize;
    float hx, one_minus_hx;
    int soft_only;  // hx >= 1 - 1e-6: effective mask = soft mask
    int structured_exact;
    int score_bf16;
    const float* tau;  // unstructured gate: threshold in normalised-score units (device); null = 2:4 gate
    const float* pen_mask;  // mask the penalty pull is taken from (GLU joint update); null = the updated mask
    int metric;             // FROM_W instantiations: which score to form from W and H
    // freeze bands: flags (fp32 0 / 1, updated in place) of entries that no longer follow the gate;
    // entries at or below freeze_low snap to 0, entries at or above freeze_high to 1 (when enabled)
    float* frozen;
    float freeze_low, freeze_high;
    int freeze_high_on;
};

__device__ __forceinline__ float effective_mask_value(float m, bool kept, const MaskUpdateParams& P) {
    if (P.soft_only) return m;
    return __fadd_rn(__fmul_rn(P.hx, m), kept ? P.one_minus_hx : 0.0f);
}

struct GroupStats {
    float sum_m = 0.f, sum_m1m = 0.f, sum_top2 = 0.f, sum_bot2 = 0.f;
    int flips = 0, lt_half = 0;
};

__device__ __forceinline__ void block_reduce_stats(const GroupStats& g, double* __restrict__ stats) {
    __shared__ double red[6][kThreads / 32];
    double v[6] = {(double)g.flips, (double)g.sum_m, (double)g.sum_m1m,
                   (double)g.sum_top2, (double)g.sum_bot2, (double)g.lt_half};
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
#pragma unroll
    for (int k = 0; k < 6; ++k) {
        v[k] = warp_sum(v[k]);
        if (lane == 0) red[k][wid] = v[k];
    }
    __syncthreads();
    if (threadIdx.x < 6) {
        double a = 0.0;
#pragma unroll
        for (int i = 0; i < kThreads / 32; ++i) a += red[threadIdx.x][i];
        atomicAdd(&stats[threadIdx.x], a);
    }
}

// PLAIN: no bf16 score rounding, no exact gate, no beta mixing, no penalty, no binarise push
// (the tempering recipe of the benchmark); the general instantiation tests those at run time.
// FROM_W: the score is not read but formed again from the weight and the Hessian diagonal with the
// arithmetic of the score kernels (so it equals what they would have written); `score` then holds H.
// WIDE: the fp32 tensors are 32-byte aligned and are moved with 32-byte accesses.
template <typename TW, bool EMIT_WM, bool EMIT_META, bool PLAIN, bool FROM_W = false, bool WIDE = false>
__global__ void __launch_bounds__(kThreads)
mask_update_nm24_kernel(const float* __restrict__ score, const float* __restrict__ norm,
                        float* __restrict__ mask, const TW* __restrict__ W, TW* __restrict__ wm,
                        uint8_t* __restrict__ meta, double* __restrict__ stats, int64_t chunks,
                        MaskUpdateParams P) {
    const float mu = norm[0];
    const float inv_sigma = __fdiv_rn(1.0f, norm[1]);
    const bool unstructured = P.tau != nullptr;
    const float tau_global = unstructured ? *P.tau : 0.0f;
    const bool score_bf16 = !PLAIN && P.score_bf16;
    const bool exact = !PLAIN && P.structured_exact && !unstructured;
    const bool mix = !PLAIN && P.beta_s > 0.0f;
    const bool penalty = !PLAIN && P.pen != 0.0f;
    const bool binarize = !PLAIN && P.binarize;
    const bool freeze = !PLAIN && !FROM_W && P.frozen != nullptr;
    const uint32_t omhx_bits = P.soft_only ? 0u : __float_as_uint(P.one_minus_hx);
    const float hx = P.soft_only ? 1.0f : P.hx;
    GroupStats gs;
    for (int64_t c = (int64_t)blockIdx.x * kThreads + threadIdx.x; c < chunks;
         c += (int64_t)gridDim.x * kThreads) {
        const int64_t e = c * 8;
        float sc[8], m[8], eff[8];
        typename Vec8<TW>::Raw wraw;
        if (!FROM_W || P.metric != SF_METRIC_MAGNITUDE) {
            if (WIDE) ld_stream32(score + e, sc); else Vec8<float>::load(score + e, sc);
        }
        if (WIDE) ld_stream32(mask + e, m); else Vec8<float>::load(mask + e, m);
        if (EMIT_WM || FROM_W) wraw = Vec8<TW>::load_raw(W + e);
        if (FROM_W) {
            float w[8];
            if (P.metric == SF_METRIC_HESSIAN_OBD) {
                Vec8<TW>::square(wraw, w);  // round(w * w) in the weight dtype
#pragma unroll
                for (int i = 0; i < 8; ++i) sc[i] = __fmul_rn(__fadd_rn(sc[i], 1e-8f), w[i]);
            } else {
                Vec8<TW>::unpack(wraw, w);
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    const float h = sc[i];
                    if (P.metric == SF_METRIC_HESSIAN_RATIO) sc[i] = __fdiv_rn(fabsf(w[i]), __fsqrt_rn(__fadd_rn(h, 1e-8f)));
                    else if (P.metric == SF_METRIC_MAGNITUDE) sc[i] = fabsf(w[i]);
                }
            }
        }
        float fz[8];
        if (freeze) Vec8<float>::load(P.frozen + e, fz);
        uint32_t kp8 = 0, kn8 = 0;
#pragma unroll
        for (int g = 0; g < 2; ++g) {
            float s[4], G[4], mp[4], mn[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                s[i] = __fmul_rn(__fsub_rn(sc[4 * g + i], mu), inv_sigma);
                if (score_bf16) s[i] = bf16_round_int(s[i]);
                mp[i] = m[4 * g + i];
            }
            const float tau = unstructured ? tau_global : second_largest4(s);
            uint32_t ks[4] = {0u, 0u, 0u, 0u};
            if (exact || mix) top2_keep_masks(s, ks);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                float gi;
                if (exact) gi = __uint_as_float(ks[i] & 0x3f800000u);
                else {
                    // sigmoid(z) = 1 / (1 + 2^(-z log2 e)), z = (s_i - tau) / (T + 1e-8)
                    gi = fast_rcp(1.0f + fast_ex2(__fmul_rn(__fsub_rn(s[i], tau), P.neg_log2e_over_t)));
                    if (score_bf16) gi = bf16_round_int(gi);
                }
                if (mix) {
                    const float t = __uint_as_float(ks[i] & __float_as_uint(P.beta_s));
                    gi = __fadd_rn(__fmul_rn(P.one_minus_beta_s, gi), t);
                    if (score_bf16) gi = bf16_round_int(gi);
                }
                // a frozen entry's gate is its own value: the pull toward the score is switched off
                if (freeze && fz[4 * g + i] != 0.0f) gi = mp[i];
                G[i] = gi;
            }
            if (penalty) {
                float pm[4] = {mp[0], mp[1], mp[2], mp[3]};
                if (P.pen_mask != nullptr) {
                    const float4 t = __ldcs(reinterpret_cast<const float4*>(P.pen_mask + e + 4 * g));
                    pm[0] = t.x; pm[1] = t.y; pm[2] = t.z; pm[3] = t.w;
                }
                if (P.penalty_mode == SF_PENALTY_TOPN) {
                    uint32_t kg[4];
                    top2_keep_masks(G, kg);
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        float delta = __fsub_rn(pm[i], __uint_as_float(kg[i] & 0x3f800000u));
                        G[i] = __fsub_rn(G[i], __fmul_rn(P.pen, delta));
                    }
                } else if (P.penalty_mode == SF_PENALTY_MID) {
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        float pg = __fsub_rn(1.0f, __fmul_rn(2.0f, pm[i]));
                        G[i] = __fsub_rn(G[i], __fmul_rn(P.pen, pg));
                    }
                }
#pragma unroll
                for (int i = 0; i < 4; ++i) G[i] = fminf(fmaxf(G[i], 0.0f), 1.0f);
            }
            if (binarize) {
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    if (G[i] < 0.5f) G[i] = __fmul_rn(G[i], P.bin_lo);
                    else if (G[i] > 0.5f) G[i] = __fmul_rn(G[i], P.bin_hi);
                }
            }
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                // clamp((1-a) mask + a G, 0, 1): the clamp rides on the multiply-add
                mn[i] = __saturatef(__fmaf_rn(P.a, G[i], __fmul_rn(mp[i], P.one_minus_a)));
                if (freeze) {
                    const bool low = mn[i] <= P.freeze_low;
                    const bool high = P.freeze_high_on && mn[i] >= P.freeze_high;
                    if (low) mn[i] = 0.0f;
                    if (high) mn[i] = 1.0f;
                    if (low || high) fz[4 * g + i] = fmaxf(fz[4 * g + i], 1.0f);
                }
                m[4 * g + i] = mn[i];
            }
            uint32_t kp[4], kn[4];
            top2_keep_masks(mp, kp);
            top2_keep_masks(mn, kn);
            kp8 |= keep_bits(kp) << (4 * g);
            kn8 |= keep_bits(kn) << (4 * g);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const float mv = mn[i];
                gs.sum_m += mv;
                gs.sum_m1m += __fmaf_rn(-mv, mv, mv);
                gs.sum_top2 += __uint_as_float(kn[i] & __float_as_uint(mv));
                gs.lt_half += mv < 0.5f ? 1 : 0;
                // hx * mask + (1 - hx) * hard, two roundings as the reference's tensor expression
                if (EMIT_WM) eff[4 * g + i] = __fadd_rn(__fmul_rn(hx, mv), __uint_as_float(kn[i] & omhx_bits));
            }
        }
        gs.flips += __popc(kp8 ^ kn8);
        if (WIDE) st_stream32(mask + e, m); else Vec8<float>::store(mask + e, m);
        if (freeze) Vec8<float>::store(P.frozen + e, fz);
        if (EMIT_WM) Vec8<TW>::store_product(wm + e, wraw, eff);
        if (EMIT_META) meta[c] = (uint8_t)(nibble_of_keep_lut(kn8 & 0xFu) | (nibble_of_keep_lut(kn8 >> 4) << 4));
    }
    gs.sum_bot2 = gs.sum_m - gs.sum_top2;
    block_reduce_stats(gs, stats);
}

// ---------------------------------------------------------------------------------------
// hard projection (generic strides and tails)
// ---------------------------------------------------------------------------------------
template <typename T>
__device__ __forceinline__ float load_scalar(const T* p);
template <>
__device__ __forceinline__ float load_scalar<float>(const float* p) { return *p; }
template <>
__device__ __forceinline__ float load_scalar<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <typename T>
__device__ __forceinline__ void store_scalar(T* p, float v);
template <>
__device__ __forceinline__ void store_scalar<float>(float* p, float v) { *p = v; }
template <>
__device__ __forceinline__ void store_scalar<__nv_bfloat16>(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

// One thread per 8 columns of one row. FAST: full chunks, 16-byte aligned rows.
template <typename TI, typename TO, bool FAST>
__global__ void __launch_bounds__(kThreads)
project_nm24_kernel(const TI* __restrict__ soft, int64_t ld_soft, TO* __restrict__ hard,
                    int64_t ld_hard, uint8_t* __restrict__ meta, int64_t rows, int64_t cols,
                    int64_t chunks_per_row) {
    const int64_t total = rows * chunks_per_row;
    const int64_t full_cols = (cols / 4) * 4;
    for (int64_t t = (int64_t)blockIdx.x * kThreads + threadIdx.x; t < total;
         t += (int64_t)gridDim.x * kThreads) {
        const int64_t row = t / chunks_per_row, ch = t - row * chunks_per_row;
        const int64_t col0 = ch * 8;
        float x[8], h[8];
        if (FAST) {
            Vec8<TI>::load(soft + row * ld_soft + col0, x);
        } else {
#pragma unroll
            for (int i = 0; i < 8; ++i)
                x[i] = (col0 + i < cols) ? load_scalar<TI>(soft + row * ld_soft + col0 + i) : 0.0f;
        }
        uint32_t mb = 0;
#pragma unroll
        for (int g = 0; g < 2; ++g) {
            float s[4] = {x[4 * g], x[4 * g + 1], x[4 * g + 2], x[4 * g + 3]};
            const bool in_core = FAST || (col0 + 4 * g + 4 <= full_cols);
            uint32_t k = in_core ? top2_keep(s) : 0xFu;
#pragma unroll
            for (int i = 0; i < 4; ++i) h[4 * g + i] = ((k >> i) & 1u) ? 1.0f : 0.0f;
            if (in_core) mb |= nibble_of_keep(k) << (4 * g);
        }
        if (hard != nullptr) {
            if (FAST) {
                Vec8<TO>::store(hard + row * ld_hard + col0, h);
            } else {
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    if (col0 + i < cols) store_scalar<TO>(hard + row * ld_hard + col0 + i, h[i]);
            }
        }
        if (meta != nullptr) meta[row * chunks_per_row + ch] = (uint8_t)mb;
    }
}

// ---------------------------------------------------------------------------------------
// effective masked weight (no mask update)
// ---------------------------------------------------------------------------------------
template <typename TW>
__global__ void __launch_bounds__(kThreads)
effective_weight_kernel(const TW* __restrict__ W, const float* __restrict__ mask, TW* __restrict__ wm,
                        uint8_t* __restrict__ meta, int64_t chunks, MaskUpdateParams P, float scale) {
    for (int64_t c = (int64_t)blockIdx.x * kThreads + threadIdx.x; c < chunks;
         c += (int64_t)gridDim.x * kThreads) {
        const int64_t e = c * 8;
        float w[8], m[8], o[8];
        Vec8<TW>::load(W + e, w);
        Vec8<float>::load(mask + e, m);
        uint32_t mb = 0;
#pragma unroll
        for (int g = 0; g < 2; ++g) {
            float s[4] = {m[4 * g], m[4 * g + 1], m[4 * g + 2], m[4 * g + 3]};
            uint32_t k = top2_keep_fast(s);
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                float eff = Vec8<TW>::round(effective_mask_value(s[i], (k >> i) & 1u, P));
                float v = Vec8<TW>::round(__fmul_rn(w[4 * g + i], eff));
                o[4 * g + i] = scale != 1.0f ? __fmul_rn(v, scale) : v;
            }
            mb |= nibble_of_keep(k) << (4 * g);
        }
        Vec8<TW>::store(wm + e, o);
        if (meta != nullptr) meta[c] = (uint8_t)mb;
    }
}

// ---------------------------------------------------------------------------------------
// mask-aware AdamW
// ---------------------------------------------------------------------------------------
struct AdamParams {
    float c_wd;       // 1 - lr*wd
    float decay;
    float beta1, one_minus_beta1, beta2, one_minus_beta2;
    float inv_sqrt_bc2, eps, step_size, lr, l1;
    int has_mask;
    void* vmax;  // AMSGrad: running maximum of the second moment (weight dtype), else unused
};

template <typename TW>
struct HutchArgs {
    const TW* hvp;          // NULL: H is read only
    const int8_t* probe_i8; // exactly one of the two probes is set when hvp is
    const TW* probe_w;
    float beta, one_minus_beta;
};

// SCORE: also writes the importance score of the updated (stored) weight and this block's partial
// sums of score and score^2, so the mask update that follows needs no separate score pass.
// AMS: the AMSGrad variant (legacy/adamw.py:142-156): the denominator uses the running maximum of the
// stored second moment.
template <typename TW, bool EMIT_WM, bool SCORE, bool AMS = false, bool WIDE = false>
__global__ void __launch_bounds__(kThreads)
adamw_masked_kernel(TW* __restrict__ p, const TW* __restrict__ g, const float* __restrict__ mask,
                    TW* __restrict__ m, TW* __restrict__ v, TW* __restrict__ wm, int64_t chunks,
                    AdamParams A, MaskUpdateParams P, float* __restrict__ H, float* __restrict__ score,
                    double* __restrict__ partials, int metric, HutchArgs<TW> hu) {
    double acc_s = 0.0, acc_s2 = 0.0;
    for (int64_t c = (int64_t)blockIdx.x * kThreads + threadIdx.x; c < chunks;
         c += (int64_t)gridDim.x * kThreads) {
        const int64_t e = c * 8;
        float pw[8], gr[8], mk[8], em[8], ev[8], o[8];
        Vec8<TW>::load(p + e, pw);
        Vec8<TW>::load(g + e, gr);
        Vec8<TW>::load(m + e, em);
        Vec8<TW>::load(v + e, ev);
        if (A.has_mask) {
            if (WIDE) ld_stream32(mask + e, mk); else Vec8<float>::load(mask + e, mk);
        }
        float vx[8];
        if (AMS) Vec8<TW>::load(static_cast<const TW*>(A.vmax) + e, vx);
        // p.mul_(1 - lr*wd) rounds to the storage type; the moments and the update are carried in
        // fp32 and rounded once when stored (the reference rounds after every in-place op, which
        // differs by at most one storage ulp)
        float pd[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) pd[i] = __fmul_rn(pw[i], A.c_wd);
        Vec8<TW>::round8(pd);
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const float p1 = pd[i];
            float g1 = gr[i];
            if (A.has_mask)
                g1 = __fmaf_rn(A.decay, __fmul_rn(p1, __fsub_rn(1.0f, mk[i])), g1);
            float m1 = __fmaf_rn(A.one_minus_beta1, g1, __fmul_rn(em[i], A.beta1));
            float v1 = __fmaf_rn(A.one_minus_beta2, __fmul_rn(g1, g1), __fmul_rn(ev[i], A.beta2));
            float vden = v1;
            if (AMS) {
                vx[i] = fmaxf(vx[i], Vec8<TW>::round(v1));
                vden = vx[i];
            }
            float denom = __fmaf_rn(fast_sqrt(vden), A.inv_sqrt_bc2, A.eps);
            const float inv_denom = fast_rcp(denom);
            float p2 = __fsub_rn(p1, __fmul_rn(A.step_size, __fmul_rn(m1, inv_denom)));
            if (A.l1 > 0.0f && A.has_mask) {
                float sgn = (p2 > 0.0f) ? 1.0f : ((p2 < 0.0f) ? -1.0f : 0.0f);
                p2 = __fsub_rn(p2, __fmul_rn(A.lr, __fmul_rn(__fmul_rn(A.l1, sgn), inv_denom)));
            }
            pw[i] = p2; em[i] = m1; ev[i] = v1;
        }
        const typename Vec8<TW>::Raw praw = Vec8<TW>::pack(pw);  // the weight as stored
        Vec8<TW>::store_raw(p + e, praw);
        Vec8<TW>::store(m + e, em);
        Vec8<TW>::store(v + e, ev);
        if (AMS) Vec8<TW>::store(static_cast<TW*>(A.vmax) + e, vx);
        if (SCORE) {
            float h[8], sc[8];
            if (metric != SF_METRIC_MAGNITUDE || hu.hvp != nullptr) {
                if (WIDE) ld_stream32(H + e, h); else Vec8<float>::load(H + e, h);
            }
            if (hu.hvp != nullptr) {
                // the Hutchinson sample of this step is folded into H before the score reads it
                float hv[8];
                Vec8<TW>::load(hu.hvp + e, hv);
                if (hu.probe_i8) {
                    // a +1 / -1 probe only flips the sign: the product is exact in the weight dtype
                    uint32_t sb[8];
                    Vec8<int8_t>::load_signs(hu.probe_i8 + e, sb);
#pragma unroll
                    for (int i = 0; i < 8; ++i) hv[i] = __uint_as_float(__float_as_uint(hv[i]) ^ sb[i]);
                } else {
                    float sg[8];
                    Vec8<TW>::load(hu.probe_w + e, sg);
#pragma unroll
                    for (int i = 0; i < 8; ++i) hv[i] = __fmul_rn(hv[i], sg[i]);
                    Vec8<TW>::round8(hv);
                }
#pragma unroll
                for (int i = 0; i < 8; ++i)
                    h[i] = __fmaf_rn(hu.one_minus_beta, fmaxf(hv[i], 0.0f), __fmul_rn(h[i], hu.beta));
                if (WIDE) st_stream32(H + e, h); else Vec8<float>::store(H + e, h);
            }
            float ps = 0.0f, ps2 = 0.0f;
            float ws[8];  // the stored weight, or for the OBD score its square rounded to the weight dtype
            if (metric == SF_METRIC_HESSIAN_OBD) Vec8<TW>::square(praw, ws); else Vec8<TW>::unpack(praw, ws);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                float sv;
                if (metric == SF_METRIC_HESSIAN_OBD) sv = __fmul_rn(__fadd_rn(h[i], 1e-8f), ws[i]);
                else if (metric == SF_METRIC_HESSIAN_RATIO) sv = __fdiv_rn(fabsf(ws[i]), __fsqrt_rn(__fadd_rn(h[i], 1e-8f)));
                else if (metric == SF_METRIC_HESSIAN) sv = h[i];
                else sv = fabsf(ws[i]);
                sc[i] = sv;
                ps += sv;
                ps2 = fmaf(sv, sv, ps2);
            }
            if (score != nullptr) Vec8<float>::store(score + e, sc);
            acc_s += (double)ps;
            acc_s2 += (double)ps2;
        }
        if (EMIT_WM) {
#pragma unroll
            for (int g2 = 0; g2 < 2; ++g2) {
                float s[4] = {mk[4 * g2], mk[4 * g2 + 1], mk[4 * g2 + 2], mk[4 * g2 + 3]};
                uint32_t k = P.soft_only ? 0u : top2_keep_fast(s);
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    float eff = Vec8<TW>::round(effective_mask_value(s[i], (k >> i) & 1u, P));
                    o[4 * g2 + i] = __fmul_rn(Vec8<TW>::round(pw[4 * g2 + i]), eff);  // the weight as stored
                }
            }
            Vec8<TW>::store(wm + e, o);
        }
    }
    if (SCORE) {
        __shared__ double red[2][kThreads / 32];
        acc_s = warp_sum(acc_s);
        acc_s2 = warp_sum(acc_s2);
        const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
        if (lane == 0) { red[0][wid] = acc_s; red[1][wid] = acc_s2; }
        __syncthreads();
        if (threadIdx.x == 0) {
            double a = 0.0, b = 0.0;
#pragma unroll
            for (int i = 0; i < kThreads / 32; ++i) { a += red[0][i]; b += red[1][i]; }
            partials[2 * blockIdx.x] = a;
            partials[2 * blockIdx.x + 1] = b;
        }
    }
}

// ---------------------------------------------------------------------------------------
// mask statistics
// ---------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreads)
mask_stats_kernel(const float* __restrict__ mask, double* __restrict__ stats, int64_t groups) {
    GroupStats gs;
    for (int64_t c = (int64_t)blockIdx.x * kThreads + threadIdx.x; c < groups;
         c += (int64_t)gridDim.x * kThreads) {
        uint4 a = ld_stream16(mask + c * 4);
        float s[4] = {__uint_as_float(a.x), __uint_as_float(a.y), __uint_as_float(a.z), __uint_as_float(a.w)};
        int r[4];
        rank4(s, r);
#pragma unroll
        for (int i = 0; i < 4; ++i) {
            gs.sum_m += s[i];
            gs.sum_m1m += s[i] * (1.0f - s[i]);
            if (r[i] < 2) gs.sum_top2 += s[i]; else gs.sum_bot2 += s[i];
            gs.lt_half += s[i] < 0.5f ? 1 : 0;
        }
    }
    block_reduce_stats(gs, stats);
}

// ---------------------------------------------------------------------------------------
// bias gradient: column sums of dy[T, out]
// ---------------------------------------------------------------------------------------
template <typename T>
__global__ void __launch_bounds__(kThreads)
bias_grad_kernel(const T* __restrict__ dy, float* __restrict__ db, int64_t rows, int64_t cols,
                 int64_t rows_per_block) {
    // block = 32 columns x 8 row lanes
    const int cx = threadIdx.x & 31, ry = threadIdx.x >> 5;
    const int64_t col = (int64_t)blockIdx.x * 32 + cx;
    const int64_t r0 = (int64_t)blockIdx.y * rows_per_block;
    int64_t r1 = r0 + rows_per_block;
    if (r1 > rows) r1 = rows;
    float acc = 0.0f;
    if (col < cols)
        for (int64_t r = r0 + ry; r < r1; r += 8) acc += load_scalar<T>(dy + r * cols + col);
    __shared__ float red[8][33];
    red[ry][cx] = acc;
    __syncthreads();
    if (ry == 0 && col < cols) {
        float s = 0.0f;
#pragma unroll
        for (int i = 0; i < 8; ++i) s += red[i][cx];
        atomicAdd(&db[col], s);
    }
}

}  // namespace sf

using namespace sf;

extern "C" {

int sf_version(void) { return 100; }

const char* sf_last_error_string(void) { return sf::last_error_buffer(); }

int64_t sf_hutch_score_scratch_doubles(int64_t n) {
    (void)n;
    return 2 * (int64_t)kMaxPartialBlocks;
}

int sf_hutch_score(const void* hvp, const void* v, int v_dtype, float* H, const void* W, int w_dtype,
                   const void* aux, double aux_scalar_d, float* score, float* norm, double* scratch,
                   int64_t n, double beta_d, int metric, void* stream) {
    float aux_scalar = (float)aux_scalar_d;
    const float beta = (float)beta_d;
    SF_CHECK_ARG(W != nullptr || score == nullptr, "sf_hutch_score: W must be non-null");
    SF_CHECK_ARG(score == nullptr ? hvp != nullptr : (norm && scratch),
                 "sf_hutch_score: give score, norm and scratch, or score = NULL with hvp to update H only");
    SF_CHECK_ARG(n > 0 && n % 8 == 0, "sf_hutch_score: n=%lld must be a positive multiple of 8", (long long)n);
    SF_CHECK_ARG(w_dtype == SF_F32 || w_dtype == SF_BF16, "sf_hutch_score: w_dtype must be SF_F32 or SF_BF16");
    const bool accum = hvp != nullptr;
    if (accum) {
        SF_CHECK_ARG(v != nullptr && H != nullptr, "sf_hutch_score: hvp given without v or H");
        SF_CHECK_ARG(v_dtype == SF_I8 || v_dtype == w_dtype, "sf_hutch_score: v_dtype must be SF_I8 or w_dtype");
    }
    const bool need_h = score != nullptr && (metric == SF_METRIC_HESSIAN_OBD || metric == SF_METRIC_HESSIAN_RATIO ||
                                             metric == SF_METRIC_HESSIAN);
    SF_CHECK_ARG(!need_h || H != nullptr, "sf_hutch_score: metric %d needs H", metric);
    SF_CHECK_ARG(score == nullptr || metric != SF_METRIC_MOVEMENT || aux != nullptr, "sf_hutch_score: movement metric needs aux=grad_ema");
    if (!(aligned16(W) && aligned16(score) && aligned16(H) && aligned16(hvp) && aligned16(aux)) ||
        (reinterpret_cast<uintptr_t>(v) & 7u))
        return fail(SF_ERR_ALIGNMENT, "sf_hutch_score: buffers must be 16-byte aligned (v: 8-byte)");
    cudaStream_t st = (cudaStream_t)stream;
    const int64_t chunks = n / 8;
    int grid = grid_for(chunks, 8);
    if (grid > kMaxPartialBlocks) grid = kMaxPartialBlocks;
    if (metric == SF_METRIC_MOVEMENT && aux_scalar < 1e-8f) aux_scalar = 1e-8f;
    int rc = SF_OK;
#define SF_HS(TW, TV, ACC) \
    rc = launch_hutch_score<TW, TV, ACC>(metric, hvp, v, H, W, aux, aux_scalar, score, scratch, chunks, beta_d, grid, st)
    if (w_dtype == SF_F32) {
        if (!accum) SF_HS(float, float, false);
        else if (v_dtype == SF_I8) SF_HS(float, int8_t, true);
        else SF_HS(float, float, true);
    } else {
        if (!accum) SF_HS(__nv_bfloat16, __nv_bfloat16, false);
        else if (v_dtype == SF_I8) SF_HS(__nv_bfloat16, int8_t, true);
        else SF_HS(__nv_bfloat16, __nv_bfloat16, true);
    }
#undef SF_HS
    if (rc != SF_OK) return rc;
    SF_CHECK_CUDA(cudaGetLastError());
    if (score == nullptr) return SF_OK;
    score_norm_finalize_kernel<<<1, kThreads, 0, st>>>(scratch, grid, (double)n, norm);
    SF_CHECK_CUDA(cudaGetLastError());
    return SF_OK;
}

int sf_grad_hessian_ema(const void* g, void* grad_ema, int dtype, float* H, int64_t n, double beta, void* stream) {
    SF_CHECK_ARG(g != nullptr && grad_ema != nullptr, "sf_grad_hessian_ema: g and grad_ema must be non-null");
    SF_CHECK_ARG(n > 0 && n % 8 == 0, "sf_grad_hessian_ema: n=%lld must be a positive multiple of 8", (long long)n);
    SF_CHECK_ARG(dtype == SF_F32 || dtype == SF_BF16, "sf_grad_hessian_ema: dtype must be SF_F32 or SF_BF16");
    if (!(aligned16(g) && aligned16(grad_ema) && aligned16(H)))
        return fail(SF_ERR_ALIGNMENT, "sf_grad_hessian_ema: buffers must be 16-byte aligned");
    cudaStream_t st = (cudaStream_t)stream;
    const float b = (float)beta, omb = (float)(1.0 - beta);
    if (dtype == SF_F32) {
        auto kern = grad_hessian_ema_kernel<float>;
        kern<<<grid_one_wave((const void*)kern, n / 8), kThreads, 0, st>>>((const float*)g, (float*)grad_ema, H, n, b, omb);
    } else {
        auto kern = grad_hessian_ema_kernel<__nv_bfloat16>;
        kern<<<grid_one_wave((const void*)kern, n / 8), kThreads, 0, st>>>((const __nv_bfloat16*)g, (__nv_bfloat16*)grad_ema,
                                                                          H, n, b, omb);
    }
    SF_CHECK_CUDA(cudaGetLastError());
    return SF_OK;
}

int sf_score_norm_from_sums(const double* sums, double n, float* norm, void* stream) {
    SF_CHECK_ARG(sums && norm, "sf_score_norm_from_sums: sums and norm must be non-null");
    SF_CHECK_ARG(n > 0, "sf_score_norm_from_sums: n must be positive");
    score_norm_from_sums_kernel<<<1, 32, 0, (cudaStream_t)stream>>>(sums, n, norm);
    SF_CHECK_CUDA(cudaGetLastError());
    return SF_OK;
}

static MaskUpdateParams make_mask_params(double temperature, double mask_lr, double pen, int penalty_mode,
                                         double beta_s, double binarize_decay, double hx, int structured_exact,
                                         int score_bf16) {
    MaskUpdateParams P;
    P.neg_log2e_over_t = (float)(-1.4426950408889634 / (double)((float)temperature + 1e-8f));
    P.a = (float)mask_lr;
    P.one_minus_a = (float)(1.0 - mask_lr);
    P.pen = (float)pen;
    P.penalty_mode = penalty_mode;
    P.beta_s = (float)beta_s;
    P.one_minus_beta_s = (float)(1.0 - beta_s);
    P.bin_lo = (float)(1.0 - binarize_decay);
    P.bin_hi = (float)(1.0 + binarize_decay);
    P.binarize = binarize_decay != 0.0;
    P.hx = (float)hx;
    P.one_minus_hx = (float)(1.0 - hx);
    P.soft_only = hx >= 1.0 - 1e-6;
    P.structured_exact = structured_exact;
    P.score_bf16 = score_bf16;
    P.tau = nullptr;
    P.pen_mask = nullptr;
    P.metric = SF_METRIC_HESSIAN_OBD;
    P.frozen = nullptr;
    P.freeze_low = 0.0f;
    P.freeze_high = 1.0f;
    P.freeze_high_on = 0;
    return P;
}

struct FreezeBands {
    float* flags = nullptr;
    double low = 0.0, high = 1.0;
    int high_on = 0;
};

static int mask_update_impl(const float* score, const float* norm, const float* tau, const float* pen_mask,
                            float* mask, const void* W, int w_dtype, void* wm, uint8_t* meta, double* stats,
                            int64_t rows, int64_t cols, double temperature, double mask_lr, double pen,
                            int penalty_mode, double beta_s, double binarize_decay, double hx, int structured_exact,
                            int score_bf16, void* stream, const FreezeBands& fb = FreezeBands());

int sf_mask_update_nm24(const float* score, const float* norm, const float* tau, float* mask, const void* W,
                        int w_dtype, void* wm, uint8_t* meta, double* stats, int64_t rows, int64_t cols,
                        double temperature, double mask_lr, double pen, int penalty_mode, double beta_s,
                        double binarize_decay, double hx, int structured_exact, int score_bf16,
                        void* stream) {
    return mask_update_impl(score, norm, tau, nullptr, mask, W, w_dtype, wm, meta, stats, rows, cols, temperature,
                            mask_lr, pen, penalty_mode, beta_s, binarize_decay, hx, structured_exact, score_bf16, stream);
}

int sf_mask_update_nm24_joint(const float* score, const float* norm, const float* tau, const float* pen_mask,
                              float* mask, const void* W, int w_dtype, void* wm, uint8_t* meta, double* stats,
                              int64_t rows, int64_t cols, double temperature, double mask_lr, double pen,
                              int penalty_mode, double beta_s, double binarize_decay, double hx,
                              int structured_exact, int score_bf16, void* stream) {
    if (pen_mask != nullptr && !aligned16(pen_mask))
        return fail(SF_ERR_ALIGNMENT, "sf_mask_update_nm24_joint: pen_mask must be 16-byte aligned");
    return mask_update_impl(score, norm, tau, pen_mask, mask, W, w_dtype, wm, meta, stats, rows, cols, temperature,
                            mask_lr, pen, penalty_mode, beta_s, binarize_decay, hx, structured_exact, score_bf16, stream);
}

int sf_mask_update_nm24_frozen(const float* score, const float* norm, const float* tau, float* frozen_flags,
                               double freeze_low, double freeze_high, int apply_high, float* mask, const void* W,
                               int w_dtype, void* wm, uint8_t* meta, double* stats, int64_t rows, int64_t cols,
                               double temperature, double mask_lr, double pen, int penalty_mode, double beta_s,
                               double binarize_decay, double hx, int structured_exact, int score_bf16, void* stream) {
    SF_CHECK_ARG(frozen_flags != nullptr, "sf_mask_update_nm24_frozen: frozen_flags must be non-null");
    if (!aligned16(frozen_flags))
        return fail(SF_ERR_ALIGNMENT, "sf_mask_update_nm24_frozen: frozen_flags must be 16-byte aligned");
    FreezeBands fb;
    fb.flags = frozen_flags;
    fb.low = freeze_low;
    fb.high = freeze_high;
    fb.high_on = apply_high ? 1 : 0;
    return mask_update_impl(score, norm, tau, nullptr, mask, W, w_dtype, wm, meta, stats, rows, cols, temperature,
                            mask_lr, pen, penalty_mode, beta_s, binarize_decay, hx, structured_exact, score_bf16, stream,
                            fb);
}

int sf_score_sum(const float* a, const float* b, float* out, float* norm, double* scratch, int64_t n, void* stream) {
    SF_CHECK_ARG(a && b && out && norm && scratch, "sf_score_sum: a, b, out, norm, scratch must be non-null");
    SF_CHECK_ARG(n > 0 && n % 8 == 0, "sf_score_sum: n=%lld must be a positive multiple of 8", (long long)n);
    if (!(aligned16(a) && aligned16(b) && aligned16(out)))
        return fail(SF_ERR_ALIGNMENT, "sf_score_sum: buffers must be 16-byte aligned");
    cudaStream_t st = (cudaStream_t)stream;
    const int64_t chunks = n / 8;
    int grid = grid_one_wave((const void*)score_sum_kernel, chunks);
    if (grid > kMaxPartialBlocks) grid = kMaxPartialBlocks;
    score_sum_kernel<<<grid, kThreads, 0, st>>>(a, b, out, scratch, chunks);
    SF_CHECK_CUDA(cudaGetLastError());
    score_norm_finalize_kernel<<<1, kThreads, 0, st>>>(scratch, grid, (double)n, norm);
    SF_CHECK_CUDA(cudaGetLastError());
    return SF_OK;
}

int64_t sf_wanda_scratch_floats(int64_t cols) { return cols > 0 ? cols * kWandaMaxRowBlocks : 0; }

int sf_wanda_add_batch(const void* x, int x_dtype, int64_t rows, int64_t cols, void* scaler_row, int s_dtype,
                       double keep, double denom, float* scratch, void* stream) {
    SF_CHECK_ARG(x && scaler_row && scratch, "sf_wanda_add_batch: x, scaler_row, scratch must be non-null");
    SF_CHECK_ARG(rows > 0 && cols > 0 && cols % 8 == 0, "sf_wanda_add_batch: rows=%lld, cols=%lld (cols a multiple of 8)",
                 (long long)rows, (long long)cols);
    SF_CHECK_ARG((x_dtype == SF_F32 || x_dtype == SF_BF16) && (s_dtype == SF_F32 || s_dtype == SF_BF16),
                 "sf_wanda_add_batch: dtypes must be SF_F32 or SF_BF16");
    SF_CHECK_ARG(denom > 0.0, "sf_wanda_add_batch: denom must be positive");
    if (!aligned16(x)) return fail(SF_ERR_ALIGNMENT, "sf_wanda_add_batch: x must be 16-byte aligned");
    cudaStream_t st = (cudaStream_t)stream;
    const int col_blocks = (int)((cols + kWandaColsPerBlock - 1) / kWandaColsPerBlock);
    int64_t row_blocks = (4 * (int64_t)sm_count() + col_blocks - 1) / col_blocks;
    const int64_t by_rows = (rows + kWandaRowLanes - 1) / kWandaRowLanes;
    if (row_blocks > by_rows) row_blocks = by_rows;
    if (row_blocks > kWandaMaxRowBlocks) row_blocks = kWandaMaxRowBlocks;
    if (row_blocks < 1) row_blocks = 1;
    const dim3 grid((unsigned)col_blocks, (unsigned)row_blocks);
    if (x_dtype == SF_BF16)
        wanda_colsumsq_kernel<__nv_bfloat16><<<grid, kThreads, 0, st>>>((const __nv_bfloat16*)x, rows, cols, scratch);
    else
        wanda_colsumsq_kernel<float><<<grid, kThreads, 0, st>>>((const float*)x, rows, cols, scratch);
    SF_CHECK_CUDA(cudaGetLastError());
    const int ub = (int)((cols + kThreads - 1) / kThreads);
    if (s_dtype == SF_BF16)
        wanda_scaler_update_kernel<__nv_bfloat16><<<ub, kThreads, 0, st>>>(scratch, (int)row_blocks, cols, (float)keep,
                                                                            (float)denom, (__nv_bfloat16*)scaler_row);
    else
        wanda_scaler_update_kernel<float><<<ub, kThreads, 0, st>>>(scratch, (int)row_blocks, cols, (float)keep,
                                                                    (float)denom, (float*)scaler_row);
    SF_CHECK_CUDA(cudaGetLastError());
    return SF_OK;
}

int sf_wanda_score(const void* W, int w_dtype, const void* scaler_row, int s_dtype, int64_t rows, int64_t cols,
                   double eps, float* score, float* norm, double* scratch, void* stream) {
    SF_CHECK_ARG(W && scaler_row && score && norm && scratch,
                 "sf_wanda_score: W, scaler_row, score, norm, scratch must be non-null");
    SF_CHECK_ARG(rows > 0 && cols > 0 && cols % 8 == 0, "sf_wanda_score: cols=%lld must be a positive multiple of 8",
                 (long long)cols);
    SF_CHECK_ARG((w_dtype == SF_F32 || w_dtype == SF_BF16) && (s_dtype == SF_F32 || s_dtype == SF_BF16),
                 "sf_wanda_score: dtypes must be SF_F32 or SF_BF16");
    if (!(aligned16(W) && aligned16(score))) return fail(SF_ERR_ALIGNMENT, "sf_wanda_score: W and score must be 16-byte aligned");
    cudaStream_t st = (cudaStream_t)stream;
    const int64_t n = rows * cols, chunks = n / 8;
    int grid = 0;
#define SF_LAUNCH_WS(TW, TS)                                                                                     \
    do {                                                                                                         \
        auto kern = wanda_score_kernel<TW, TS>;                                                                  \
        grid = grid_one_wave((const void*)kern, chunks);                                                         \
        if (grid > kMaxPartialBlocks) grid = kMaxPartialBlocks;                                                  \
        kern<<<grid, kThreads, 0, st>>>((const TW*)W, (const TS*)scaler_row, cols, (float)eps, score, scratch, chunks); \
    } while (0)
    if (w_dtype == SF_BF16 && s_dtype == SF_BF16) SF_LAUNCH_WS(__nv_bfloat16, __nv_bfloat16);
    else if (w_dtype == SF_BF16) SF_LAUNCH_WS(__nv_bfloat16, float);
    else if (s_dtype == SF_BF16) SF_LAUNCH_WS(float, __nv_bfloat16);
    else SF_LAUNCH_WS(float, float);
#undef SF_LAUNCH_WS
    SF_CHECK_CUDA(cudaGetLastError());
    score_norm_finalize_kernel<<<1, kThreads, 0, st>>>(scratch, grid, (double)n, norm);
    SF_CHECK_CUDA(cudaGetLastError());
    return SF_OK;
}

int sf_mask_update_nm24_from_weight(const void* W, int w_dtype, const float* H, int metric, const float* norm,
                                    const float* tau, float* mask, void* wm, uint8_t* meta, double* stats,
                                    int64_t rows, int64_t cols, double temperature, double mask_lr, double pen,
                                    int penalty_mode, double beta_s, double binarize_decay, double hx,
                                    int structured_exact, void* stream) {
    SF_CHECK_ARG(W && norm && mask && wm && meta && stats,
                 "sf_mask_update_nm24_from_weight: W, norm, mask, wm, meta, stats must be non-null");
    SF_CHECK_ARG(metric == SF_METRIC_HESSIAN_OBD || metric == SF_METRIC_HESSIAN_RATIO || metric == SF_METRIC_MAGNITUDE ||
                     metric == SF_METRIC_HESSIAN,
                 "sf_mask_update_nm24_from_weight: metric %d cannot be formed from W and H", metric);
    SF_CHECK_ARG(metric == SF_METRIC_MAGNITUDE || H != nullptr, "sf_mask_update_nm24_from_weight: metric %d needs H", metric);
    SF_CHECK_ARG(rows > 0 && cols > 0 && cols % 8 == 0,
                 "sf_mask_update_nm24_from_weight: cols=%lld must be a positive multiple of 8", (long long)cols);
    SF_CHECK_ARG(penalty_mode >= SF_PENALTY_NONE && penalty_mode <= SF_PENALTY_MID,
                 "sf_mask_update_nm24_from_weight: unknown penalty_mode %d", penalty_mode);
    SF_CHECK_ARG(w_dtype == SF_F32 || w_dtype == SF_BF16, "sf_mask_update_nm24_from_weight: w_dtype must be SF_F32 or SF_BF16");
    if (!(aligned16(H) && aligned16(mask) && aligned16(W) && aligned16(wm)))
        return fail(SF_ERR_ALIGNMENT, "sf_mask_update_nm24_from_weight: buffers must be 16-byte aligned");
    cudaStream_t st = (cudaStream_t)stream;
    MaskUpdateParams P = make_mask_params(temperature, mask_lr, pen, penalty_mode, beta_s, binarize_decay, hx,
                                          structured_exact, 0);
    P.tau = tau;
    P.metric = metric;
    const int64_t chunks = rows * cols / 8;
    SF_CHECK_CUDA(cudaMemsetAsync(stats, 0, SF_MSTAT_COUNT * sizeof(double), st));
    const bool plain = !structured_exact && !(beta_s > 0.0) && pen == 0.0 && binarize_decay == 0.0;
    const bool wide = aligned32(mask) && aligned32(H);
#define SF_MUW(TW, PL, WD)                                                                       \
    do {                                                                                         \
        auto kern = mask_update_nm24_kernel<TW, true, true, PL, true, WD>;                       \
        kern<<<grid_one_wave((const void*)kern, chunks), kThreads, 0, st>>>(                     \
            H, norm, mask, (const TW*)W, (TW*)wm, meta, stats, chunks, P);                       \
    } while (0)
#define SF_MUW_W(TW, PL) do { if (wide) SF_MUW(TW, PL, true); else SF_MUW(TW, PL, false); } while (0)
    if (w_dtype == SF_F32) { if (plain) SF_MUW_W(float, true); else SF_MUW_W(float, false); }
    else { if (plain) SF_MUW_W(__nv_bfloat16, true); else SF_MUW_W(__nv_bfloat16, false); }
#undef SF_MUW_W
#undef SF_MUW
    SF_CHECK_CUDA(cudaGetLastError());
    return SF_OK;
}

static int mask_update_impl(const float* score, const float* norm, const float* tau, const float* pen_mask,
                            float* mask, const void* W, int w_dtype, void* wm, uint8_t* meta, double* stats,
                            int64_t rows, int64_t cols, double temperature, double mask_lr, double pen,
                            int penalty_mode, double beta_s, double binarize_decay, double hx, int structured_exact,
                            int score_bf16, void* stream, const FreezeBands& fb) {
    SF_CHECK_ARG(score && norm && mask && stats, "sf_mask_update_nm24: score, norm, mask, stats must be non-null");
    SF_CHECK_ARG(rows > 0 && cols > 0, "sf_mask_update_nm24: rows=%lld cols=%lld must be positive",
                 (long long)rows, (long long)cols);
    SF_CHECK_ARG(cols % 8 == 0, "sf_mask_update_nm24: cols=%lld must be a multiple of 8 (2:4 groups, packed metadata)",
                 (long long)cols);
    SF_CHECK_ARG(penalty_mode >= SF_PENALTY_NONE && penalty_mode <= SF_PENALTY_MID,
                 "sf_mask_update_nm24: unknown penalty_mode %d", penalty_mode);
    SF_CHECK_ARG((wm == nullptr) || (W != nullptr), "sf_mask_update_nm24: wm requested without W");
    SF_CHECK_ARG(w_dtype == SF_F32 || w_dtype == SF_BF16, "sf_mask_update_nm24: w_dtype must be SF_F32 or SF_BF16");
    if (!(aligned16(score) && aligned16(mask) && aligned16(W) && aligned16(wm)))
        return fail(SF_ERR_ALIGNMENT, "sf_mask_update_nm24: buffers must be 16-byte aligned");
    cudaStream_t st = (cudaStream_t)stream;
    MaskUpdateParams P = make_mask_params(temperature, mask_lr, pen, penalty_mode, beta_s, binarize_decay,
                                          hx, structured_exact, score_bf16);
    P.tau = tau;
    P.pen_mask = pen_mask;
    P.frozen = fb.flags;
    P.freeze_low = (float)fb.low;
    P.freeze_high = (float)fb.high;
    P.freeze_high_on = fb.high_on;
    const int64_t chunks = rows * cols / 8;
    SF_CHECK_CUDA(cudaMemsetAsync(stats, 0, SF_MSTAT_COUNT * sizeof(double), st));
    const bool plain = !score_bf16 && !structured_exact && !(beta_s > 0.0) && pen == 0.0 && binarize_decay == 0.0 &&
                       fb.flags == nullptr;
#define SF_MU_K(TW, EW, EM, PL)                                                                  \
    do {                                                                                         \
        auto kern = mask_update_nm24_kernel<TW, EW, EM, PL>;                                     \
        kern<<<grid_one_wave((const void*)kern, chunks), kThreads, 0, st>>>(                     \
            score, norm, mask, (const TW*)W, (TW*)wm, meta, stats, chunks, P);                   \
    } while (0)
#define SF_MU(TW, EW, EM)                                                                        \
    do {                                                                                         \
        if (plain) SF_MU_K(TW, EW, EM, true); else SF_MU_K(TW, EW, EM, false);                   \
    } while (0)
    // the layer path (masked weight and metadata wanted, no freeze flags): 32-byte fp32 accesses where aligned
    const bool wide = wm && meta && fb.flags == nullptr && aligned32(score) && aligned32(mask);
#define SF_MU_WIDE(TW)                                                                           \
    do {                                                                                         \
        if (plain) {                                                                             \
            auto kern = mask_update_nm24_kernel<TW, true, true, true, false, true>;              \
            kern<<<grid_one_wave((const void*)kern, chunks), kThreads, 0, st>>>(                 \
                score, norm, mask, (const TW*)W, (TW*)wm, meta, stats, chunks, P);               \
        } else {                                                                                 \
            auto kern = mask_update_nm24_kernel<TW, true, true, false, false, true>;             \
            kern<<<grid_one_wave((const void*)kern, chunks), kThreads, 0, st>>>(                 \
                score, norm, mask, (const TW*)W, (TW*)wm, meta, stats, chunks, P);               \
        }                                                                                        \
    } while (0)
#define SF_MU_T(TW)                                       \
    do {                                                  \
        if (wide) SF_MU_WIDE(TW);                         \
        else if (wm && meta) SF_MU(TW, true, true);       \
        else if (wm) SF_MU(TW, true, false);              \
        else if (meta) SF_MU(TW, false, true);            \
        else SF_MU(TW, false, false);                     \
    } while (0)
    if (w_dtype == SF_F32) SF_MU_T(float); else SF_MU_T(__nv_bfloat16);
#undef SF_MU_T
#undef SF_MU_WIDE
#undef SF_MU_K
#undef SF_MU
    SF_CHECK_CUDA(cudaGetLastError());
    return SF_OK;
}

int sf_project_nm24(const void* soft, int in_dtype, int64_t ld_soft, void* hard, int out_dtype,
                    int64_t ld_hard, uint8_t* meta, int64_t rows, int64_t cols, void* stream) {
    SF_CHECK_ARG(soft != nullptr, "sf_project_nm24: soft must be non-null");
    SF_CHECK_ARG(hard != nullptr || meta != nullptr, "sf_project_nm24: nothing to write (hard and meta both null)");
    SF_CHECK_ARG(rows >= 0 && cols >= 0, "sf_project_nm24: negative shape");
    SF_CHECK_ARG(ld_soft >= cols && (hard == nullptr || ld_hard >= cols), "sf_project_nm24: row stride smaller than cols");
    SF_CHECK_ARG(in_dtype == SF_F32 || in_dtype == SF_BF16, "sf_project_nm24: in_dtype must be SF_F32 or SF_BF16");
    SF_CHECK_ARG(hard == nullptr || out_dtype == SF_F32 || out_dtype == SF_BF16,
                 "sf_project_nm24: out_dtype must be SF_F32 or SF_BF16");
    if (rows == 0 || cols == 0) return SF_OK;
    cudaStream_t st = (cudaStream_t)stream;
    const int64_t cpr = (cols + 7) / 8;
    const bool fast = (cols % 8 == 0) && (ld_soft % 8 == 0) && aligned16(soft) &&
                      (hard == nullptr || ((ld_hard % 8 == 0) && aligned16(hard)));
    const int grid = grid_for(rows * cpr, 8);
#define SF_PJ(TI, TO, F) \
    project_nm24_kernel<TI, TO, F><<<grid, kThreads, 0, st>>>((const TI*)soft, ld_soft, (TO*)hard, ld_hard, meta, rows, cols, cpr)
#define SF_PJ_F(TI, TO) do { if (fast) SF_PJ(TI, TO, true); else SF_PJ(TI, TO, false); } while (0)
    const int od = hard ? out_dtype : SF_F32;
    if (in_dtype == SF_F32 && od == SF_F32) SF_PJ_F(float, float);
    else if (in_dtype == SF_F32) SF_PJ_F(float, __nv_bfloat16);
    else if (od == SF_F32) SF_PJ_F(__nv_bfloat16, float);
    else SF_PJ_F(__nv_bfloat16, __nv_bfloat16);
#undef SF_PJ_F
#undef SF_PJ
    SF_CHECK_CUDA(cudaGetLastError());
    return SF_OK;
}

int sf_effective_weight(const void* W, int w_dtype, const float* mask, void* wm, uint8_t* meta,
                        int64_t rows, int64_t cols, double hx, int finalized, double scale_d, void* stream) {
    const float scale = (float)scale_d;
    SF_CHECK_ARG(W && mask && wm, "sf_effective_weight: W, mask, wm must be non-null");
    SF_CHECK_ARG(rows > 0 && cols > 0 && cols % 8 == 0, "sf_effective_weight: cols=%lld must be a positive multiple of 8",
                 (long long)cols);
    SF_CHECK_ARG(w_dtype == SF_F32 || w_dtype == SF_BF16, "sf_effective_weight: w_dtype must be SF_F32 or SF_BF16");
    if (!(aligned16(W) && aligned16(mask) && aligned16(wm)))
        return fail(SF_ERR_ALIGNMENT, "sf_effective_weight: buffers must be 16-byte aligned");
    cudaStream_t st = (cudaStream_t)stream;
    MaskUpdateParams P = make_mask_params(1.0, 0.0, 0.0, 0, 0.0, 0.0, finalized ? 1.0 : hx, 0, 0);
    const int64_t chunks = rows * cols / 8;
    const int grid = w_dtype == SF_F32 ? grid_one_wave((const void*)effective_weight_kernel<float>, chunks)
                                       : grid_one_wave((const void*)effective_weight_kernel<__nv_bfloat16>, chunks);
    if (w_dtype == SF_F32)
        effective_weight_kernel<float><<<grid, kThreads, 0, st>>>((const float*)W, mask, (float*)wm, meta, chunks, P, scale);
    else
        effective_weight_kernel<__nv_bfloat16><<<grid, kThreads, 0, st>>>((const __nv_bfloat16*)W, mask,
                                                                          (__nv_bfloat16*)wm, meta, chunks, P, scale);
    SF_CHECK_CUDA(cudaGetLastError());
    return SF_OK;
}

static int adamw_impl(void* p, const void* g, const float* mask, void* m, void* v, int w_dtype, int64_t n,
                      double lr, double beta1, double beta2, double eps, double weight_decay, double decay,
                      double bc1, double bc2, double adaptive_l1, void* wm, double hx, int64_t cols,
                      float* H, float* score, float* norm, double* scratch, int metric, const void* hvp,
                      const void* probe, int v_dtype, double beta_h, void* stream, void* vmax = nullptr) {
    SF_CHECK_ARG(p && g && m && v, "sf_adamw_masked: p, g, m, v must be non-null");
    SF_CHECK_ARG(n > 0 && n % 8 == 0, "sf_adamw_masked: n=%lld must be a positive multiple of 8", (long long)n);
    SF_CHECK_ARG(w_dtype == SF_F32 || w_dtype == SF_BF16, "sf_adamw_masked: w_dtype must be SF_F32 or SF_BF16");
    SF_CHECK_ARG(bc1 > 0.0 && bc2 > 0.0, "sf_adamw_masked: bias corrections must be positive (step >= 1)");
    if (wm != nullptr) {
        SF_CHECK_ARG(mask != nullptr, "sf_adamw_masked: wm requested without mask");
        SF_CHECK_ARG(cols > 0 && cols % 8 == 0 && n % cols == 0,
                     "sf_adamw_masked: wm needs cols=%lld a multiple of 8 dividing n", (long long)cols);
    }
    if (!(aligned16(p) && aligned16(g) && aligned16(m) && aligned16(v) && aligned16(mask) && aligned16(wm)))
        return fail(SF_ERR_ALIGNMENT, "sf_adamw_masked: buffers must be 16-byte aligned");
    cudaStream_t st = (cudaStream_t)stream;
    AdamParams A;
    A.c_wd = (float)(1.0 - lr * weight_decay);
    A.decay = (float)decay;
    A.beta1 = (float)beta1; A.one_minus_beta1 = (float)(1.0 - beta1);
    A.beta2 = (float)beta2; A.one_minus_beta2 = (float)(1.0 - beta2);
    A.inv_sqrt_bc2 = (float)(1.0 / sqrt(bc2));
    A.eps = (float)eps;
    A.step_size = (float)(lr / bc1);
    A.lr = (float)lr;
    A.l1 = (float)adaptive_l1;
    A.has_mask = mask != nullptr;
    A.vmax = vmax;
    MaskUpdateParams P = make_mask_params(1.0, 0.0, 0.0, 0, 0.0, 0.0, hx, 0, 0);
    const int64_t chunks = n / 8;
    int grid = 0;
#define SF_AD(TW, EW, SC, ...)                                                                   \
    do {                                                                                         \
        auto kern = adamw_masked_kernel<TW, EW, SC, ##__VA_ARGS__>;                              \
        grid = grid_one_wave((const void*)kern, chunks);                                         \
        if (grid > kMaxPartialBlocks) grid = kMaxPartialBlocks;                                  \
        HutchArgs<TW> hu;                                                                        \
        hu.hvp = (const TW*)hvp;                                                                 \
        hu.probe_i8 = (hvp && v_dtype == SF_I8) ? (const int8_t*)probe : nullptr;                \
        hu.probe_w = (hvp && v_dtype != SF_I8) ? (const TW*)probe : nullptr;                     \
        hu.beta = (float)beta_h;                                                                 \
        hu.one_minus_beta = (float)(1.0 - beta_h);                                               \
        kern<<<grid, kThreads, 0, st>>>((TW*)p, (const TW*)g, mask, (TW*)m, (TW*)v, (TW*)wm, chunks, A, P, H, score, \
                                        scratch, metric, hu);                                    \
    } while (0)
    if (vmax != nullptr) {
        if (w_dtype == SF_F32) SF_AD(float, false, false, true); else SF_AD(__nv_bfloat16, false, false, true);
    } else if (norm != nullptr) {
        // the fp32 mask and Hessian move in 32-byte accesses where their addresses allow it
        const bool wide = (mask == nullptr || aligned32(mask)) && (H == nullptr || aligned32(H)) && score == nullptr;
        if (w_dtype == SF_F32) { if (wide) SF_AD(float, false, true, false, true); else SF_AD(float, false, true); }
        else { if (wide) SF_AD(__nv_bfloat16, false, true, false, true); else SF_AD(__nv_bfloat16, false, true); }
    } else if (w_dtype == SF_F32) { if (wm) SF_AD(float, true, false); else SF_AD(float, false, false); }
    else { if (wm) SF_AD(__nv_bfloat16, true, false); else SF_AD(__nv_bfloat16, false, false); }
#undef SF_AD
    SF_CHECK_CUDA(cudaGetLastError());
    if (norm != nullptr) {
        score_norm_finalize_kernel<<<1, kThreads, 0, st>>>(scratch, grid, (double)n, norm);
        SF_CHECK_CUDA(cudaGetLastError());
    }
    return SF_OK;
}

int sf_adamw_masked(void* p, const void* g, const float* mask, void* m, void* v, int w_dtype, int64_t n,
                    double lr, double beta1, double beta2, double eps, double weight_decay, double decay,
                    double bc1, double bc2, double adaptive_l1, void* wm, double hx, int64_t cols,
                    void* stream) {
    return adamw_impl(p, g, mask, m, v, w_dtype, n, lr, beta1, beta2, eps, weight_decay, decay, bc1, bc2, adaptive_l1,
                      wm, hx, cols, nullptr, nullptr, nullptr, nullptr, 0, nullptr, nullptr, 0, 0.0, stream);
}

int sf_adamw_masked_amsgrad(void* p, const void* g, const float* mask, void* m, void* v, void* v_max, int w_dtype,
                            int64_t n, double lr, double beta1, double beta2, double eps, double weight_decay,
                            double decay, double bc1, double bc2, double adaptive_l1, void* stream) {
    SF_CHECK_ARG(v_max != nullptr, "sf_adamw_masked_amsgrad: v_max must be non-null");
    if (!aligned16(v_max)) return fail(SF_ERR_ALIGNMENT, "sf_adamw_masked_amsgrad: v_max must be 16-byte aligned");
    return adamw_impl(p, g, mask, m, v, w_dtype, n, lr, beta1, beta2, eps, weight_decay, decay, bc1, bc2, adaptive_l1,
                      nullptr, 1.0, 0, nullptr, nullptr, nullptr, nullptr, 0, nullptr, nullptr, 0, 0.0, stream, v_max);
}

int sf_adamw_masked_score(void* p, const void* g, const float* mask, void* m, void* v, int w_dtype, int64_t n,
                          double lr, double beta1, double beta2, double eps, double weight_decay, double decay,
                          double bc1, double bc2, double adaptive_l1, const void* hvp, const void* probe,
                          int v_dtype, double beta_h, float* H, float* score, float* norm, double* scratch,
                          int metric, void* stream) {
    if (hvp != nullptr) {
        SF_CHECK_ARG(probe != nullptr && H != nullptr, "sf_adamw_masked_score: hvp given without probe or H");
        SF_CHECK_ARG(v_dtype == SF_I8 || v_dtype == w_dtype, "sf_adamw_masked_score: v_dtype must be SF_I8 or w_dtype");
        if (!aligned16(hvp) || (reinterpret_cast<uintptr_t>(probe) & 7u))
            return fail(SF_ERR_ALIGNMENT, "sf_adamw_masked_score: hvp must be 16-byte, probe 8-byte aligned");
    }
    SF_CHECK_ARG(norm && scratch, "sf_adamw_masked_score: norm and scratch must be non-null");
    SF_CHECK_ARG(metric == SF_METRIC_HESSIAN_OBD || metric == SF_METRIC_HESSIAN_RATIO || metric == SF_METRIC_MAGNITUDE ||
                     metric == SF_METRIC_HESSIAN,
                 "sf_adamw_masked_score: metric %d is not available fused (use sf_hutch_score)", metric);
    SF_CHECK_ARG(metric == SF_METRIC_MAGNITUDE || H != nullptr, "sf_adamw_masked_score: metric %d needs H", metric);
    if (!(aligned16(H) && aligned16(score)))
        return fail(SF_ERR_ALIGNMENT, "sf_adamw_masked_score: buffers must be 16-byte aligned");
    return adamw_impl(p, g, mask, m, v, w_dtype, n, lr, beta1, beta2, eps, weight_decay, decay, bc1, bc2, adaptive_l1,
                      nullptr, 1.0, 0, H, score, norm, scratch, metric, hvp, probe, v_dtype, beta_h, stream);
}

int sf_mask_stats(const float* mask, double* stats, int64_t rows, int64_t cols, void* stream) {
    SF_CHECK_ARG(mask && stats, "sf_mask_stats: mask and stats must be non-null");
    SF_CHECK_ARG(rows > 0 && cols > 0 && cols % 4 == 0, "sf_mask_stats: cols=%lld must be a positive multiple of 4",
                 (long long)cols);
    if (!aligned16(mask)) return fail(SF_ERR_ALIGNMENT, "sf_mask_stats: mask must be 16-byte aligned");
    cudaStream_t st = (cudaStream_t)stream;
    SF_CHECK_CUDA(cudaMemsetAsync(stats, 0, SF_MSTAT_COUNT * sizeof(double), st));
    const int64_t groups = rows * cols / 4;
    mask_stats_kernel<<<grid_for(groups, 8), kThreads, 0, st>>>(mask, stats, groups);
    SF_CHECK_CUDA(cudaGetLastError());
    return SF_OK;
}

int sf_mask_summary(const float* mask, int64_t n, double eps, double* out, void* stream) {
    SF_CHECK_ARG(mask && out, "sf_mask_summary: mask and out must be non-null");
    SF_CHECK_ARG(n > 0, "sf_mask_summary: n must be positive");
    // the clamp bounds are formed in fp32 as the tensor op forms them (1 - 1e-8 is 1 in fp32)
    const float lo = (float)eps, hi = (float)(1.0 - eps);
    int64_t blocks = (n + kThreads * 16 - 1) / (kThreads * 16);
    if (blocks > 148 * 4) blocks = 148 * 4;
    if (blocks < 1) blocks = 1;
    mask_summary_kernel<<<(int)blocks, kThreads, 0, (cudaStream_t)stream>>>(mask, n, lo, hi, out);
    SF_CHECK_CUDA(cudaGetLastError());
    return SF_OK;
}

int sf_mask_sample_hist(const float* mask, const int64_t* idx, int64_t take, int bins, double* hist, void* stream) {
    SF_CHECK_ARG(mask && idx && hist, "sf_mask_sample_hist: mask, idx, hist must be non-null");
    SF_CHECK_ARG(take > 0 && bins > 0, "sf_mask_sample_hist: take and bins must be positive");
    int64_t blocks = (take + kThreads - 1) / kThreads;
    if (blocks > 148 * 4) blocks = 148 * 4;
    mask_sample_hist_kernel<<<(int)blocks, kThreads, 0, (cudaStream_t)stream>>>(mask, idx, take, bins, hist);
    SF_CHECK_CUDA(cudaGetLastError());
    return SF_OK;
}

int sf_bias_grad(const void* dy, int dtype, float* db, int64_t T, int64_t out, void* stream) {
    SF_CHECK_ARG(dy && db, "sf_bias_grad: dy and db must be non-null");
    SF_CHECK_ARG(T > 0 && out > 0, "sf_bias_grad: T and out must be positive");
    SF_CHECK_ARG(dtype == SF_F32 || dtype == SF_BF16, "sf_bias_grad: dtype must be SF_F32 or SF_BF16");
    cudaStream_t st = (cudaStream_t)stream;
    SF_CHECK_CUDA(cudaMemsetAsync(db, 0, out * sizeof(float), st));
    const int64_t col_blocks = (out + 31) / 32;
    int64_t row_blocks = ((int64_t)sm_count() * 8 + col_blocks - 1) / col_blocks;
    if (row_blocks < 1) row_blocks = 1;
    if (row_blocks > (T + 7) / 8) row_blocks = (T + 7) / 8;
    const int64_t rpb = (T + row_blocks - 1) / row_blocks;
    dim3 grid((unsigned)col_blocks, (unsigned)row_blocks);
    if (dtype == SF_F32) bias_grad_kernel<float><<<grid, kThreads, 0, st>>>((const float*)dy, db, T, out, rpb);
    else bias_grad_kernel<__nv_bfloat16><<<grid, kThreads, 0, st>>>((const __nv_bfloat16*)dy, db, T, out, rpb);
    SF_CHECK_CUDA(cudaGetLastError());
    return SF_OK;
}

}  // extern "C"

// ---------------------------------------------------------------------------------------
// sf_hutch_score_static: the same pass with the partial-sum scratch held inside the library
// ---------------------------------------------------------------------------------------
// For callers that may not allocate device memory where they need the score: a hook in the
// middle of a training step while a caching allocator holds all free memory, code that must
// avoid the device-wide synchronisation that cudaMalloc and cudaFree imply, a process with a
// fixed device-memory budget. The scratch of the score pass lives in the file-scope array
// below instead of a caller buffer: 32 KiB on every GPU that loads the library, held until
// the process exits. The entry point itself allocates nothing.
namespace sf {
constexpr int64_t kStaticScratchDoubles = 2 * (int64_t)kMaxPartialBlocks;
static __device__ __align__(256) double g_static_score_scratch[kStaticScratchDoubles];

constexpr int kMaxDevices = 64;
static double* g_static_scratch_ptr[kMaxDevices];  // device address of the array, per device
static std::mutex g_static_scratch_mu;

// Device address of g_static_score_scratch on the current device. In host code the name of a
// __device__ array is only a handle; the address a kernel can use comes from the runtime.
static int static_scratch_address(double** out) {
    int dev = 0;
    SF_CHECK_CUDA(cudaGetDevice(&dev));
    if (dev < 0 || dev >= kMaxDevices) return fail(SF_ERR_UNSUPPORTED, "sf_hutch_score_static: device index %d beyond %d", dev, kMaxDevices);
    std::lock_guard<std::mutex> lock(g_static_scratch_mu);
    if (g_static_scratch_ptr[dev] == nullptr) {
        void* p = nullptr;
        SF_CHECK_CUDA(cudaGetSymbolAddress(&p, g_static_score_scratch));
        g_static_scratch_ptr[dev] = static_cast<double*>(p);
    }
    *out = g_static_scratch_ptr[dev];
    return SF_OK;
}
}  // namespace sf

extern "C" {

int64_t sf_hutch_score_static_max_n(void) { return SF_HUTCH_SCORE_STATIC_MAX_N; }

int sf_hutch_score_static(const void* hvp, const void* v, int v_dtype, float* H, const void* W, int w_dtype,
                          const void* aux, double aux_scalar, float* score, float* norm, int64_t n, double beta,
                          int metric, void* stream) {
    if (n > SF_HUTCH_SCORE_STATIC_MAX_N)
        return sf::fail(SF_ERR_UNSUPPORTED,
                        "sf_hutch_score_static: n=%lld exceeds the built-in scratch limit of %lld elements; "
                        "use sf_hutch_score with caller-provided scratch",
                        (long long)n, (long long)SF_HUTCH_SCORE_STATIC_MAX_N);
    double* scratch = nullptr;
    int rc = sf::static_scratch_address(&scratch);
    if (rc != SF_OK) return rc;
    // Every partial-sum slot the kernels read is written earlier in the same call, so nothing
    // has to be cleared between calls; calls that overlap on the GPU would mix their partials.
    return sf_hutch_score(hvp, v, v_dtype, H, W, w_dtype, aux, aux_scalar, score, norm, scratch, n, beta, metric,
                          stream);
}

}  // extern "C"
