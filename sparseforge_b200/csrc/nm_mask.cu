// mask_type / hard_mask_type 'structured' with a general N:M (legacy/sparse_modeling.py:720-735,
// :1164-1185): groups of M consecutive entries along the input dimension keep their N largest.
// The 2:4 case has kernels of its own (eight entries per thread, metadata for the sparse tensor
// cores); this file covers every other N < M with M in {2, 4, 8, 16, 32}.
//
// One thread owns one group (two or four groups for M = 4, 2): it holds the scores, the previous mask values
// and the new ones in registers and ranks every group with M (M - 1) / 2 comparisons (stable descending
// order: ties go to the lower column). The hard projection alone also orders NaN (largest, as a stable sort
// of the group does). The passes are bound by HBM for M <= 8 and by the comparisons above that.
#include "common.cuh"

namespace sf {

constexpr int kNmThreads = 256;

struct NmUpdateParams {
    int n_keep;
    float neg_log2e_over_t;  // -log2(e) / (T + 1e-8)
    float a, one_minus_a;
    float pen;
    int penalty_mode;  // 0 none, SF_PENALTY_TOPN, SF_PENALTY_MID
    float beta_s, one_minus_beta_s;
    float bin_lo, bin_hi;
    int binarize;
    float hx, one_minus_hx;
    int soft_only;
    int structured_exact;
    int score_bf16;
    const float* tau;       // unstructured gate threshold (device scalar) or null
    const float* pen_mask;  // mask the penalty pull is taken from (GLU joint update); null = the layer's own
    int hard_threshold;     // hard view = (mask > 0.5) instead of the top N of every group ('unstructured')
};

// M consecutive values -> floats, with the widest accesses the run allows (the run starts on a
// multiple of its own size, the tensors on 16 bytes). Every tensor is read and written once per pass:
// streaming (evict-first) accesses.
template <int M>
__device__ __forceinline__ void load_run(const float* __restrict__ p, float (&x)[M]) {
    if constexpr (M == 2) {
        const float2 t = __ldcs(reinterpret_cast<const float2*>(p));
        x[0] = t.x; x[1] = t.y;
    } else {
#pragma unroll
        for (int i = 0; i < M / 4; ++i) {
            const float4 t = __ldcs(reinterpret_cast<const float4*>(p + 4 * i));
            x[4 * i] = t.x; x[4 * i + 1] = t.y; x[4 * i + 2] = t.z; x[4 * i + 3] = t.w;
        }
    }
}
template <int M>
__device__ __forceinline__ void store_run(float* __restrict__ p, const float (&x)[M]) {
    if constexpr (M == 2) {
        __stcs(reinterpret_cast<float2*>(p), make_float2(x[0], x[1]));
    } else {
#pragma unroll
        for (int i = 0; i < M / 4; ++i)
            __stcs(reinterpret_cast<float4*>(p + 4 * i), make_float4(x[4 * i], x[4 * i + 1], x[4 * i + 2], x[4 * i + 3]));
    }
}
// M bf16 values as M / 2 packed pairs
template <int M>
__device__ __forceinline__ void load_pairs(const __nv_bfloat16* __restrict__ p, uint32_t (&w)[M / 2]) {
    if constexpr (M == 2) {
        w[0] = __ldcs(reinterpret_cast<const uint32_t*>(p));
    } else if constexpr (M == 4) {
        const uint2 t = __ldcs(reinterpret_cast<const uint2*>(p));
        w[0] = t.x; w[1] = t.y;
    } else {
#pragma unroll
        for (int i = 0; i < M / 8; ++i) {
            const uint4 t = __ldcs(reinterpret_cast<const uint4*>(p + 8 * i));
            w[4 * i] = t.x; w[4 * i + 1] = t.y; w[4 * i + 2] = t.z; w[4 * i + 3] = t.w;
        }
    }
}
template <int M>
__device__ __forceinline__ void store_pairs(__nv_bfloat16* __restrict__ p, const uint32_t (&w)[M / 2]) {
    if constexpr (M == 2) {
        __stcs(reinterpret_cast<uint32_t*>(p), w[0]);
    } else if constexpr (M == 4) {
        __stcs(reinterpret_cast<uint2*>(p), make_uint2(w[0], w[1]));
    } else {
#pragma unroll
        for (int i = 0; i < M / 8; ++i)
            __stcs(reinterpret_cast<uint4*>(p + 8 * i), make_uint4(w[4 * i], w[4 * i + 1], w[4 * i + 2], w[4 * i + 3]));
    }
}
// wm = W * cast(eff): the product is rounded once, in the weight's type, as `weight * mask` is in
// the reference (legacy/sparse_modeling.py:74-81)
template <int M>
__device__ __forceinline__ void store_product_run(float* __restrict__ wm, const float* __restrict__ W, const float (&eff)[M]) {
    float w[M], o[M];
    load_run<M>(W, w);
#pragma unroll
    for (int i = 0; i < M; ++i) o[i] = __fmul_rn(w[i], eff[i]);
    store_run<M>(wm, o);
}
template <int M>
__device__ __forceinline__ void store_product_run(__nv_bfloat16* __restrict__ wm, const __nv_bfloat16* __restrict__ W,
                                                  const float (&eff)[M]) {
    uint32_t w[M / 2];
    load_pairs<M>(W, w);
#pragma unroll
    for (int i = 0; i < M / 2; ++i) {
        const __nv_bfloat162 e = __floats2bfloat162_rn(eff[2 * i], eff[2 * i + 1]);
        const __nv_bfloat162 r = __hmul2(*reinterpret_cast<const __nv_bfloat162*>(&w[i]), e);
        w[i] = *reinterpret_cast<const uint32_t*>(&r);
    }
    store_pairs<M>(wm, w);
}

// bit i set = entry i is among the n largest of the group (stable descending order)
template <int M>
__device__ __forceinline__ uint32_t topn_keep(const float (&x)[M], int n) {
    uint32_t keep = 0;
#pragma unroll
    for (int i = 0; i < M; ++i) {
        int r = 0;
#pragma unroll
        for (int j = 0; j < M; ++j) {
            if (j == i) continue;
            // j sorts before i: strictly larger, or equal and to the left
            const bool before = j < i ? !gt_desc(x[i], x[j]) : gt_desc(x[j], x[i]);
            r += before ? 1 : 0;
        }
        keep |= (r < n ? 1u : 0u) << i;
    }
    return keep;
}

// The update pass ranks NaN-free values (normalised scores, gates and masks in [0, 1]), so every pair is
// compared once: c = (x_i >= x_j) for i < j puts i before j (the lower column wins a tie); rank_i starts at
// the number of later columns and loses one for each of them it beats, rank_j gains one. x points at the M
// values of the group inside a register array (all indices are compile-time constants after unrolling).
template <int M>
__device__ __forceinline__ void ranks_pairwise(const float* x, int (&rank)[M]) {
#pragma unroll
    for (int i = 0; i < M; ++i) rank[i] = M - 1 - i;
#pragma unroll
    for (int i = 0; i < M; ++i)
#pragma unroll
        for (int j = i + 1; j < M; ++j) {
            const int c = (int)set_ge(x[i], x[j]);  // -1 when i sorts before j, else 0
            rank[i] += c;
            rank[j] -= c;
        }
}
template <int M>
__device__ __forceinline__ uint32_t keep_fast(const float* x, int n) {
    int rank[M];
    ranks_pairwise<M>(x, rank);
    uint32_t keep = 0;
#pragma unroll
    for (int i = 0; i < M; ++i) keep |= (rank[i] < n ? 1u : 0u) << i;
    return keep;
}
template <int M>
__device__ __forceinline__ uint32_t keep_tau_fast(const float* x, int n, float& tau) {
    int rank[M];
    ranks_pairwise<M>(x, rank);
    uint32_t keep = 0;
    tau = x[0];
#pragma unroll
    for (int i = 0; i < M; ++i) {
        keep |= (rank[i] < n ? 1u : 0u) << i;
        if (rank[i] == n - 1) tau = x[i];
    }
    return keep;
}

template <int M>
__device__ __forceinline__ uint32_t above_half(const float* x) {
    uint32_t keep = 0;
#pragma unroll
    for (int i = 0; i < M; ++i) keep |= (x[i] > 0.5f ? 1u : 0u) << i;
    return keep;
}

struct NmStats {
    float sum_m = 0.f, sum_m1m = 0.f, sum_top = 0.f;
    int flips = 0, lt_half = 0;
};

__device__ __forceinline__ void nm_reduce_stats(const NmStats& g, double* __restrict__ stats) {
    __shared__ double red[5][kNmThreads / 32];
    double v[5] = {(double)g.flips, (double)g.sum_m, (double)g.sum_m1m, (double)g.sum_top, (double)g.lt_half};
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
#pragma unroll
    for (int k = 0; k < 5; ++k) {
        v[k] = warp_sum(v[k]);
        if (lane == 0) red[k][wid] = v[k];
    }
    __syncthreads();
    if (threadIdx.x < 5) {
        double a = 0.0;
#pragma unroll
        for (int i = 0; i < kNmThreads / 32; ++i) a += red[threadIdx.x][i];
        // slots: flips, sum m, sum m(1-m), sum of kept, [sum of dropped: finalize], count < 0.5
        const int slot = threadIdx.x < 4 ? threadIdx.x : 5;
        atomicAdd(&stats[slot], a);
        if (threadIdx.x == 1) atomicAdd(&stats[4], a);   // dropped = sum m - sum kept
        if (threadIdx.x == 3) atomicAdd(&stats[4], -a);
    }
}

// E = GPT * M consecutive entries per thread: GPT groups of M (32 bytes of each fp32 tensor per thread
// for M <= 8, which the memory system likes better than 8 or 16).
template <typename TW, int M, int GPT>
__global__ void __launch_bounds__(kNmThreads)
mask_update_nm_kernel(const float* __restrict__ score, const float* __restrict__ norm, float* __restrict__ mask,
                      const TW* __restrict__ W, TW* __restrict__ wm, double* __restrict__ stats, int64_t chunks,
                      NmUpdateParams P) {
    constexpr int E = GPT * M;
    const float mu = norm[0];
    const float inv_sigma = __fdiv_rn(1.0f, norm[1]);
    const bool unstructured = P.tau != nullptr;
    const float tau_global = unstructured ? *P.tau : 0.0f;
    const bool exact = P.structured_exact && !unstructured;
    const bool mix = P.beta_s > 0.0f;
    const int n = P.n_keep;
    NmStats gs;
    for (int64_t c = (int64_t)blockIdx.x * kNmThreads + threadIdx.x; c < chunks; c += (int64_t)gridDim.x * kNmThreads) {
        const int64_t e = c * E;
        float s[E], mp[E], G[E], pm[E];
        load_run<E>(score + e, s);
        load_run<E>(mask + e, mp);
        if (P.pen != 0.0f && P.pen_mask != nullptr) load_run<E>(P.pen_mask + e, pm);
#pragma unroll
        for (int i = 0; i < E; ++i) {
            s[i] = __fmul_rn(__fsub_rn(s[i], mu), inv_sigma);
            if (P.score_bf16) s[i] = bf16_round_int(s[i]);
        }
        uint32_t kn_all = 0;
#pragma unroll
        for (int g = 0; g < GPT; ++g) {
            const int o = g * M;
            float tau = tau_global;
            uint32_t ks = 0;
            if (!unstructured || mix) {
                float t;
                ks = keep_tau_fast<M>(s + o, n, t);
                if (!unstructured) tau = t;
            }
#pragma unroll
            for (int i = 0; i < M; ++i) {
                const float top = ((ks >> i) & 1u) ? 1.0f : 0.0f;
                float gi;
                if (exact) gi = top;
                else {
                    gi = fast_rcp(1.0f + fast_ex2(__fmul_rn(__fsub_rn(s[o + i], tau), P.neg_log2e_over_t)));
                    if (P.score_bf16) gi = bf16_round_int(gi);
                }
                if (mix) {
                    gi = __fadd_rn(__fmul_rn(P.one_minus_beta_s, gi), __fmul_rn(P.beta_s, top));
                    if (P.score_bf16) gi = bf16_round_int(gi);
                }
                G[o + i] = gi;
            }
            if (P.pen != 0.0f) {
                if (P.penalty_mode == SF_PENALTY_TOPN) {
                    const uint32_t kg = keep_fast<M>(G + o, n);
#pragma unroll
                    for (int i = 0; i < M; ++i) {
                        const float from = P.pen_mask != nullptr ? pm[o + i] : mp[o + i];
                        G[o + i] = __fsub_rn(G[o + i], __fmul_rn(P.pen, __fsub_rn(from, ((kg >> i) & 1u) ? 1.0f : 0.0f)));
                    }
                } else if (P.penalty_mode == SF_PENALTY_MID) {
#pragma unroll
                    for (int i = 0; i < M; ++i) {
                        const float from = P.pen_mask != nullptr ? pm[o + i] : mp[o + i];
                        G[o + i] = __fsub_rn(G[o + i], __fmul_rn(P.pen, __fsub_rn(1.0f, __fmul_rn(2.0f, from))));
                    }
                }
#pragma unroll
                for (int i = 0; i < M; ++i) G[o + i] = fminf(fmaxf(G[o + i], 0.0f), 1.0f);
            }
            if (P.binarize) {
#pragma unroll
                for (int i = 0; i < M; ++i) {
                    if (G[o + i] < 0.5f) G[o + i] = __fmul_rn(G[o + i], P.bin_lo);
                    else if (G[o + i] > 0.5f) G[o + i] = __fmul_rn(G[o + i], P.bin_hi);
                }
            }
            const uint32_t kp = P.hard_threshold ? above_half<M>(mp + o) : keep_fast<M>(mp + o, n);
            // the new mask takes the place of the gate
#pragma unroll
            for (int i = 0; i < M; ++i)
                G[o + i] = __saturatef(__fmaf_rn(P.a, G[o + i], __fmul_rn(mp[o + i], P.one_minus_a)));
            const uint32_t kn = P.hard_threshold ? above_half<M>(G + o) : keep_fast<M>(G + o, n);
            gs.flips += __popc(kp ^ kn);
            kn_all |= kn << (o & 31);
        }
        store_run<E>(mask + e, G);
#pragma unroll
        for (int i = 0; i < E; ++i) {
            const float mv = G[i];
            const bool top = (kn_all >> i) & 1u;
            gs.sum_m += mv;
            gs.sum_m1m += __fmaf_rn(-mv, mv, mv);
            gs.sum_top += top ? mv : 0.0f;
            gs.lt_half += mv < 0.5f ? 1 : 0;
            // hx * mask + (1 - hx) * hard, two roundings as the reference's tensor expression
            if (!P.soft_only) G[i] = __fadd_rn(__fmul_rn(P.hx, mv), top ? P.one_minus_hx : 0.0f);
        }
        if (wm != nullptr) store_product_run<E>(wm + e, W + e, G);
    }
    nm_reduce_stats(gs, stats);
}

// hard 0/1 view of a soft mask (generic row strides, fp32 or bf16; NaN counts as the largest value, as
// in a stable descending sort of the group)
template <typename TI, typename TO, int M>
__global__ void __launch_bounds__(kNmThreads)
project_nm_kernel(const TI* __restrict__ soft, int64_t ld_soft, TO* __restrict__ hard, int64_t ld_hard, int64_t rows,
                  int64_t groups_per_row, int n) {
    const int64_t groups = rows * groups_per_row;
    for (int64_t g = (int64_t)blockIdx.x * kNmThreads + threadIdx.x; g < groups; g += (int64_t)gridDim.x * kNmThreads) {
        const int64_t r = g / groups_per_row, c = (g - r * groups_per_row) * M;
        float m[M];
        const TI* src = soft + r * ld_soft + c;
#pragma unroll
        for (int i = 0; i < M; ++i) m[i] = (float)src[i];
        const uint32_t k = topn_keep<M>(m, n);
        TO* dst = hard + r * ld_hard + c;
#pragma unroll
        for (int i = 0; i < M; ++i) dst[i] = (TO)(((k >> i) & 1u) ? 1.0f : 0.0f);
    }
}

// wm = W * cast(hx m + (1 - hx) topN(m)) of a contiguous layer (the soft mask holds no NaN)
template <typename TW, int M, int GPT>
__global__ void __launch_bounds__(kNmThreads)
effective_weight_nm_kernel(const float* __restrict__ mask, const TW* __restrict__ W, TW* __restrict__ wm, int64_t chunks,
                           int n, float hx, float one_minus_hx, int soft_only, int hard_threshold) {
    constexpr int E = GPT * M;
    for (int64_t c = (int64_t)blockIdx.x * kNmThreads + threadIdx.x; c < chunks; c += (int64_t)gridDim.x * kNmThreads) {
        const int64_t e = c * E;
        float m[E];
        load_run<E>(mask + e, m);
        if (!soft_only) {
            uint32_t keep = 0;
#pragma unroll
            for (int g = 0; g < GPT; ++g)
                keep |= (hard_threshold ? above_half<M>(m + g * M) : keep_fast<M>(m + g * M, n)) << ((g * M) & 31);
#pragma unroll
            for (int i = 0; i < E; ++i) m[i] = __fadd_rn(__fmul_rn(hx, m[i]), ((keep >> i) & 1u) ? one_minus_hx : 0.0f);
        }
        store_product_run<E>(wm + e, W + e, m);
    }
}

static int nm_grid(int64_t groups) {
    int64_t g = (groups + kNmThreads - 1) / kNmThreads;
    const int64_t cap = (int64_t)sm_count() * 8;
    return (int)(g < cap ? (g < 1 ? 1 : g) : cap);
}

template <typename TW, int M, int GPT>
static int launch_update(const float* score, const float* norm, float* mask, const void* W, void* wm, double* stats,
                         int64_t groups, const NmUpdateParams& P, cudaStream_t st) {
    const int64_t chunks = groups / GPT;
    mask_update_nm_kernel<TW, M, GPT><<<nm_grid(chunks), kNmThreads, 0, st>>>(score, norm, mask, (const TW*)W, (TW*)wm,
                                                                            stats, chunks, P);
    SF_CHECK_CUDA(cudaGetLastError());
    return SF_OK;
}

template <typename TW>
static int dispatch_update(int m, const float* score, const float* norm, float* mask, const void* W, void* wm,
                           double* stats, int64_t groups, const NmUpdateParams& P, cudaStream_t st) {
    switch (m) {
        case 2:
            if (groups % 4 == 0) return launch_update<TW, 2, 4>(score, norm, mask, W, wm, stats, groups, P, st);
            return launch_update<TW, 2, 1>(score, norm, mask, W, wm, stats, groups, P, st);
        case 4:
            if (groups % 2 == 0) return launch_update<TW, 4, 2>(score, norm, mask, W, wm, stats, groups, P, st);
            return launch_update<TW, 4, 1>(score, norm, mask, W, wm, stats, groups, P, st);
        case 8: return launch_update<TW, 8, 1>(score, norm, mask, W, wm, stats, groups, P, st);
        case 16: return launch_update<TW, 16, 1>(score, norm, mask, W, wm, stats, groups, P, st);
        case 32: return launch_update<TW, 32, 1>(score, norm, mask, W, wm, stats, groups, P, st);
    }
    return fail(SF_ERR_UNSUPPORTED, "N:M mask update: M=%d is not one of 2, 4, 8, 16, 32", m);
}

template <typename TI, typename TO>
static int dispatch_project(int m, const void* soft, int64_t ld_soft, void* hard, int64_t ld_hard, int64_t rows, int64_t cols,
                            int n, cudaStream_t st) {
    const int64_t gpr = cols / m;
    const int grid = nm_grid(rows * gpr);
#define SF_NM_PROJECT(MM)                                                                                               \
    case MM:                                                                                                            \
        project_nm_kernel<TI, TO, MM><<<grid, kNmThreads, 0, st>>>((const TI*)soft, ld_soft, (TO*)hard, ld_hard, rows,   \
                                                                  gpr, n);                                              \
        break;
    switch (m) {
        SF_NM_PROJECT(2)
        SF_NM_PROJECT(4)
        SF_NM_PROJECT(8)
        SF_NM_PROJECT(16)
        SF_NM_PROJECT(32)
        default: return fail(SF_ERR_UNSUPPORTED, "N:M projection: M=%d is not one of 2, 4, 8, 16, 32", m);
    }
#undef SF_NM_PROJECT
    SF_CHECK_CUDA(cudaGetLastError());
    return SF_OK;
}

static int check_group(const char* who, int n_keep, int m_group, int64_t rows, int64_t cols) {
    if (m_group < 2 || n_keep < 1 || n_keep >= m_group) return fail(SF_ERR_BAD_ARG, "%s: need 1 <= N < M (got %d:%d)", who, n_keep, m_group);
    if (m_group != 2 && m_group != 4 && m_group != 8 && m_group != 16 && m_group != 32)
        return fail(SF_ERR_UNSUPPORTED, "%s: M=%d is not one of 2, 4, 8, 16, 32", who, m_group);
    if (rows <= 0 || cols <= 0 || cols % m_group != 0)
        return fail(SF_ERR_BAD_ARG, "%s: cols=%lld must be a multiple of M=%d", who, (long long)cols, m_group);
    return SF_OK;
}

template <typename TW, int M, int GPT>
static int launch_effective(const float* mask, const void* W, void* wm, int64_t groups, int n, double hx, int soft_only,
                            int hard_threshold, cudaStream_t st) {
    const int64_t chunks = groups / GPT;
    effective_weight_nm_kernel<TW, M, GPT><<<nm_grid(chunks), kNmThreads, 0, st>>>(mask, (const TW*)W, (TW*)wm, chunks, n,
                                                                                 (float)hx, (float)(1.0 - hx), soft_only,
                                                                                 hard_threshold);
    SF_CHECK_CUDA(cudaGetLastError());
    return SF_OK;
}

template <typename TW>
static int dispatch_effective(int m, const float* mask, const void* W, void* wm, int64_t groups, int n, double hx,
                              int soft_only, int hard_threshold, cudaStream_t st) {
    switch (m) {
        case 2:
            if (groups % 4 == 0) return launch_effective<TW, 2, 4>(mask, W, wm, groups, n, hx, soft_only, hard_threshold, st);
            return launch_effective<TW, 2, 1>(mask, W, wm, groups, n, hx, soft_only, hard_threshold, st);
        case 4:
            if (groups % 2 == 0) return launch_effective<TW, 4, 2>(mask, W, wm, groups, n, hx, soft_only, hard_threshold, st);
            return launch_effective<TW, 4, 1>(mask, W, wm, groups, n, hx, soft_only, hard_threshold, st);
        case 8: return launch_effective<TW, 8, 1>(mask, W, wm, groups, n, hx, soft_only, hard_threshold, st);
        case 16: return launch_effective<TW, 16, 1>(mask, W, wm, groups, n, hx, soft_only, hard_threshold, st);
        case 32: return launch_effective<TW, 32, 1>(mask, W, wm, groups, n, hx, soft_only, hard_threshold, st);
    }
    return fail(SF_ERR_UNSUPPORTED, "N:M masked weight: M=%d is not one of 2, 4, 8, 16, 32", m);
}

}  // namespace sf

using namespace sf;

extern "C" {

int sf_mask_update_nm(const float* score, const float* norm, const float* tau, const float* pen_mask, float* mask, const void* W,
                      int w_dtype,
                      void* wm, double* stats, int64_t rows, int64_t cols, int n_keep, int m_group, double temperature,
                      double mask_lr, double pen, int penalty_mode, double beta_s, double binarize_decay, double hx,
                      int structured_exact, int score_bf16, int hard_view, void* stream) {
    SF_CHECK_ARG(score && norm && mask && stats, "sf_mask_update_nm: score, norm, mask, stats must be non-null");
    if (int rc = check_group("sf_mask_update_nm", n_keep, m_group, rows, cols)) return rc;
    SF_CHECK_ARG(penalty_mode >= 0 && penalty_mode <= 2, "sf_mask_update_nm: penalty_mode must be 0, 1 or 2");
    SF_CHECK_ARG(hard_view == SF_HARD_TOPN || hard_view == SF_HARD_THRESHOLD, "sf_mask_update_nm: hard_view must be 0 or 1");
    SF_CHECK_ARG((wm == nullptr) || (W != nullptr), "sf_mask_update_nm: wm requested without W");
    SF_CHECK_ARG(w_dtype == SF_F32 || w_dtype == SF_BF16, "sf_mask_update_nm: w_dtype must be SF_F32 or SF_BF16");
    if (!(aligned16(score) && aligned16(mask) && aligned16(W) && aligned16(wm) && aligned16(pen_mask)))
        return fail(SF_ERR_ALIGNMENT, "sf_mask_update_nm: tensors must be 16-byte aligned");
    cudaStream_t st = (cudaStream_t)stream;
    NmUpdateParams P;
    P.n_keep = n_keep;
    P.neg_log2e_over_t = (float)(-1.4426950408889634 / (double)((float)temperature + 1e-8f));
    P.a = (float)mask_lr;
    P.one_minus_a = (float)(1.0 - mask_lr);
    P.pen = penalty_mode == 0 ? 0.0f : (float)pen;
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
    P.tau = tau;
    P.pen_mask = pen_mask;
    P.hard_threshold = hard_view == SF_HARD_THRESHOLD;
    SF_CHECK_CUDA(cudaMemsetAsync(stats, 0, SF_MSTAT_COUNT * sizeof(double), st));
    const int64_t groups = rows * (cols / m_group);
    if (w_dtype == SF_BF16) return dispatch_update<__nv_bfloat16>(m_group, score, norm, mask, W, wm, stats, groups, P, st);
    return dispatch_update<float>(m_group, score, norm, mask, W, wm, stats, groups, P, st);
}

int sf_project_nm(const void* soft, int in_dtype, int64_t ld_soft, void* hard, int out_dtype, int64_t ld_hard, int64_t rows,
                  int64_t cols, int n_keep, int m_group, void* stream) {
    SF_CHECK_ARG(soft && hard, "sf_project_nm: soft and hard must be non-null");
    if (int rc = check_group("sf_project_nm", n_keep, m_group, rows, cols)) return rc;
    SF_CHECK_ARG(ld_soft >= cols && ld_hard >= cols, "sf_project_nm: row strides must be at least cols");
    SF_CHECK_ARG((in_dtype == SF_F32 || in_dtype == SF_BF16) && (out_dtype == SF_F32 || out_dtype == SF_BF16),
                 "sf_project_nm: dtypes must be SF_F32 or SF_BF16");
    cudaStream_t st = (cudaStream_t)stream;
    if (in_dtype == SF_F32 && out_dtype == SF_F32)
        return dispatch_project<float, float>(m_group, soft, ld_soft, hard, ld_hard, rows, cols, n_keep, st);
    if (in_dtype == SF_F32)
        return dispatch_project<float, __nv_bfloat16>(m_group, soft, ld_soft, hard, ld_hard, rows, cols, n_keep, st);
    if (out_dtype == SF_F32)
        return dispatch_project<__nv_bfloat16, float>(m_group, soft, ld_soft, hard, ld_hard, rows, cols, n_keep, st);
    return dispatch_project<__nv_bfloat16, __nv_bfloat16>(m_group, soft, ld_soft, hard, ld_hard, rows, cols, n_keep, st);
}

int sf_effective_weight_nm(const void* W, int w_dtype, const float* mask, void* wm, int64_t rows, int64_t cols, int n_keep,
                           int m_group, double hx, int finalized, int hard_view, void* stream) {
    SF_CHECK_ARG(W && mask && wm, "sf_effective_weight_nm: W, mask, wm must be non-null");
    if (int rc = check_group("sf_effective_weight_nm", n_keep, m_group, rows, cols)) return rc;
    SF_CHECK_ARG(w_dtype == SF_F32 || w_dtype == SF_BF16, "sf_effective_weight_nm: w_dtype must be SF_F32 or SF_BF16");
    if (!(aligned16(W) && aligned16(mask) && aligned16(wm)))
        return fail(SF_ERR_ALIGNMENT, "sf_effective_weight_nm: tensors must be 16-byte aligned");
    cudaStream_t st = (cudaStream_t)stream;
    SF_CHECK_ARG(hard_view == SF_HARD_TOPN || hard_view == SF_HARD_THRESHOLD, "sf_effective_weight_nm: hard_view must be 0 or 1");
    const int soft_only = (finalized != 0) || hx >= 1.0 - 1e-6;
    const int hard_threshold = hard_view == SF_HARD_THRESHOLD;
    const int64_t groups = rows * (cols / m_group);
    if (w_dtype == SF_BF16) return dispatch_effective<__nv_bfloat16>(m_group, mask, W, wm, groups, n_keep, hx, soft_only, hard_threshold, st);
    return dispatch_effective<float>(m_group, mask, W, wm, groups, n_keep, hx, soft_only, hard_threshold, st);
}

}  // extern "C"
