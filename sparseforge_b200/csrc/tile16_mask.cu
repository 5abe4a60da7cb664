// hard_mask_type 'block16' of the reference: inside every 16 x 16 tile of the layer the keep_k
// entries with the largest soft-mask value are kept (legacy/sparse_modeling.py:537-574), and the
// 'block16' penalty pulls the gate towards the same per-tile top-k of the gate (:1298-1348).
//
// One warp owns one tile: lane l holds the eight consecutive entries [8 l, 8 l + 8) of the tile in
// row-major order (row l / 2, columns 8 (l % 2) ...), i.e. one 32-byte run of a mask row. The k-th
// largest of the 256 values is found by a radix select over an order-preserving 32-bit key, eight
// bits per round with a 256-bin histogram in shared memory; ties at the threshold are resolved
// towards the lower row-major position with a warp prefix count, so the result equals a stable
// descending sort of the tile.
#include "common.cuh"

namespace sf {

constexpr int kTileThreads = 256;  // eight warps, eight tiles per CTA at a time

__device__ __forceinline__ uint32_t order_key(float x) {
    const uint32_t u = __float_as_uint(x);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__device__ __forceinline__ int warp_excl_scan(int v, int lane) {
    int s = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, s, o);
        if (lane >= o) s += t;
    }
    return s - v;
}

// keep bits (bit j = entry j of this lane) of the k largest of the warp's 256 values, ties to the
// lower row-major position. hist: 256 ints of shared memory owned by this warp. 0 < k < 256.
__device__ __forceinline__ uint32_t tile_topk(const float (&x)[8], int k, int* hist, int lane) {
    uint32_t key[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) key[j] = order_key(x[j]);
    uint32_t prefix = 0, prefix_mask = 0;
    int need = k;  // how many of the entries matching `prefix` are still to be kept
#pragma unroll 1
    for (int shift = 24; shift >= 0; shift -= 8) {
#pragma unroll
        for (int j = 0; j < 8; ++j) hist[lane * 8 + j] = 0;
        __syncwarp();
#pragma unroll
        for (int j = 0; j < 8; ++j)
            if ((key[j] & prefix_mask) == prefix) atomicAdd(&hist[(key[j] >> shift) & 0xffu], 1);
        __syncwarp();
        // lane l owns digits 255 - 8 l ... 248 - 8 l (descending): count of entries with a larger digit
        int local[8], lsum = 0;
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            local[j] = hist[255 - (lane * 8 + j)];
            lsum += local[j];
        }
        const int above = warp_excl_scan(lsum, lane);  // entries with digits above this lane's range
        // the digit d with count(> d) < need <= count(>= d) lies in exactly one lane's range
        const bool mine = above < need && need <= above + lsum;
        int d = 0, gt = 0;
        if (mine) {
            int run = above;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                if (run < need && need <= run + local[j]) { d = 255 - (lane * 8 + j); gt = run; }
                run += local[j];
            }
        }
        const int src = __ffs(__ballot_sync(0xffffffffu, mine)) - 1;
        d = __shfl_sync(0xffffffffu, d, src);
        gt = __shfl_sync(0xffffffffu, gt, src);
        need -= gt;
        prefix |= (uint32_t)d << shift;
        prefix_mask |= 0xffu << shift;
        __syncwarp();
    }
    // prefix is the key of the k-th largest value; `need` of the entries equal to it are kept
    int eq = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) eq += key[j] == prefix ? 1 : 0;
    int rank = warp_excl_scan(eq, lane);
    uint32_t keep = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
        if (key[j] > prefix) keep |= 1u << j;
        else if (key[j] == prefix) {
            if (rank < need) keep |= 1u << j;
            ++rank;
        }
    }
    return keep;
}

__device__ __forceinline__ uint32_t tile_keep(const float (&x)[8], int k, int* hist, int lane) {
    if (k <= 0) return 0u;
    if (k >= 256) return 0xffu;
    return tile_topk(x, k, hist, lane);
}

struct GroupStatsLite {
    float sum_m = 0.f, sum_m1m = 0.f, sum_kept = 0.f;
    int flips = 0, lt_half = 0;
};

// stats[SF_MSTAT_*] += this block's sums (kept / not kept sums go to the TOP2 / BOT2 slots)
__device__ __forceinline__ void tile_reduce_stats(const GroupStatsLite& g, double* __restrict__ stats) {
    __shared__ double red[6][kTileThreads / 32];
    double v[6] = {(double)g.flips, (double)g.sum_m, (double)g.sum_m1m, (double)g.sum_kept,
                   (double)g.sum_m - (double)g.sum_kept, (double)g.lt_half};
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
        for (int i = 0; i < kTileThreads / 32; ++i) a += red[threadIdx.x][i];
        atomicAdd(&stats[threadIdx.x], a);
    }
}

struct TileUpdateParams {
    float neg_log2e_over_t;
    float a, one_minus_a;
    float pen;
    int penalty_mode;  // 0 none, 1 per-tile top-k of the gate, 2 mid
    float bin_lo, bin_hi;
    int binarize;
    float hx, one_minus_hx;
    int soft_only;
    int keep_k;
};

// Fused mask update for the 'block16' mode: unstructured gate (global threshold tau in
// normalised-score units), per-tile top-k / mid penalty, binarise push, EMA, per-tile hard view,
// effective masked weight, flip count and mask sums. rows, cols multiples of 16.
template <typename TW>
__global__ void __launch_bounds__(kTileThreads)
mask_update_tile16_kernel(const float* __restrict__ score, const float* __restrict__ norm, const float* __restrict__ tau_p,
                          float* __restrict__ mask, const TW* __restrict__ W, TW* __restrict__ wm,
                          double* __restrict__ stats, int64_t cols, int tiles_r, int tiles_c, TileUpdateParams P) {
    __shared__ int hist_all[kTileThreads / 32][256];
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    int* hist = hist_all[wid];
    const float mu = norm[0], inv_sigma = __fdiv_rn(1.0f, norm[1]), tau = *tau_p;
    GroupStatsLite gs;
    const int64_t tiles = (int64_t)tiles_r * tiles_c;
    for (int64_t t = (int64_t)blockIdx.x * (kTileThreads / 32) + wid; t < tiles; t += (int64_t)gridDim.x * (kTileThreads / 32)) {
        const int64_t tr = t / tiles_c, tc = t - tr * tiles_c;
        const int64_t e = (tr * 16 + (lane >> 1)) * cols + tc * 16 + (lane & 1) * 8;
        float sc[8], mp[8], G[8], mn[8];
        Vec8<float>::load(score + e, sc);
        Vec8<float>::load(mask + e, mp);
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float s = __fmul_rn(__fsub_rn(sc[j], mu), inv_sigma);
            G[j] = fast_rcp(1.0f + fast_ex2(__fmul_rn(__fsub_rn(s, tau), P.neg_log2e_over_t)));
        }
        if (P.pen != 0.0f) {
            if (P.penalty_mode == 1) {
                const uint32_t kg = tile_keep(G, P.keep_k, hist, lane);
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    G[j] = __fsub_rn(G[j], __fmul_rn(P.pen, __fsub_rn(mp[j], ((kg >> j) & 1u) ? 1.0f : 0.0f)));
            } else if (P.penalty_mode == 2) {
#pragma unroll
                for (int j = 0; j < 8; ++j)
                    G[j] = __fsub_rn(G[j], __fmul_rn(P.pen, __fsub_rn(1.0f, __fmul_rn(2.0f, mp[j]))));
            }
#pragma unroll
            for (int j = 0; j < 8; ++j) G[j] = fminf(fmaxf(G[j], 0.0f), 1.0f);
        }
        if (P.binarize) {
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                if (G[j] < 0.5f) G[j] = __fmul_rn(G[j], P.bin_lo);
                else if (G[j] > 0.5f) G[j] = __fmul_rn(G[j], P.bin_hi);
            }
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) mn[j] = __saturatef(__fmaf_rn(P.a, G[j], __fmul_rn(mp[j], P.one_minus_a)));
        const uint32_t kp = tile_keep(mp, P.keep_k, hist, lane);
        const uint32_t kn = tile_keep(mn, P.keep_k, hist, lane);
        gs.flips += __popc(kp ^ kn);
        float eff[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const float mv = mn[j];
            const bool top = (kn >> j) & 1u;
            gs.sum_m += mv;
            gs.sum_m1m += __fmaf_rn(-mv, mv, mv);
            gs.sum_kept += top ? mv : 0.0f;
            gs.lt_half += mv < 0.5f ? 1 : 0;
            eff[j] = P.soft_only ? mv : __fadd_rn(__fmul_rn(P.hx, mv), top ? P.one_minus_hx : 0.0f);
        }
        Vec8<float>::store(mask + e, mn);
        if (wm != nullptr) {
            const typename Vec8<TW>::Raw wraw = Vec8<TW>::load_raw(W + e);
            Vec8<TW>::store_product(wm + e, wraw, eff);
        }
    }
    tile_reduce_stats(gs, stats);
}

// Per-tile hard view of a soft mask, and / or the masked weight W * (hx m + (1 - hx) hard).
template <typename TW>
__global__ void __launch_bounds__(kTileThreads)
project_tile16_kernel(const float* __restrict__ soft, float* __restrict__ hard, const TW* __restrict__ W,
                      TW* __restrict__ wm, int64_t cols, int tiles_r, int tiles_c, int keep_k, float hx) {
    __shared__ int hist_all[kTileThreads / 32][256];
    const int lane = threadIdx.x & 31, wid = threadIdx.x >> 5;
    int* hist = hist_all[wid];
    const int64_t tiles = (int64_t)tiles_r * tiles_c;
    for (int64_t t = (int64_t)blockIdx.x * (kTileThreads / 32) + wid; t < tiles; t += (int64_t)gridDim.x * (kTileThreads / 32)) {
        const int64_t tr = t / tiles_c, tc = t - tr * tiles_c;
        const int64_t e = (tr * 16 + (lane >> 1)) * cols + tc * 16 + (lane & 1) * 8;
        float m[8], o[8];
        Vec8<float>::load(soft + e, m);
        const uint32_t k = tile_keep(m, keep_k, hist, lane);
        if (hard != nullptr) {
#pragma unroll
            for (int j = 0; j < 8; ++j) o[j] = ((k >> j) & 1u) ? 1.0f : 0.0f;
            Vec8<float>::store(hard + e, o);
        }
        if (wm != nullptr) {
#pragma unroll
            for (int j = 0; j < 8; ++j)
                o[j] = hx >= 1.0f - 1e-6f ? m[j] : __fadd_rn(__fmul_rn(hx, m[j]), ((k >> j) & 1u) ? 1.0f - hx : 0.0f);
            const typename Vec8<TW>::Raw wraw = Vec8<TW>::load_raw(W + e);
            Vec8<TW>::store_product(wm + e, wraw, o);
        }
    }
}

static int tile_grid(int64_t tiles) {
    int64_t g = (tiles + kTileThreads / 32 - 1) / (kTileThreads / 32);
    const int64_t cap = 148 * 8;
    return (int)(g < cap ? (g < 1 ? 1 : g) : cap);
}

}  // namespace sf

using namespace sf;

extern "C" {

int sf_mask_update_tile16(const float* score, const float* norm, const float* tau, float* mask, const void* W, int w_dtype,
                          void* wm, double* stats, int64_t rows, int64_t cols, int keep_k, double temperature,
                          double mask_lr, double pen, int penalty_mode, double binarize_decay, double hx, void* stream) {
    SF_CHECK_ARG(score && norm && tau && mask && stats, "sf_mask_update_tile16: score, norm, tau, mask, stats must be non-null");
    SF_CHECK_ARG(rows > 0 && cols > 0 && rows % 16 == 0 && cols % 16 == 0,
                 "sf_mask_update_tile16: rows=%lld and cols=%lld must be multiples of 16", (long long)rows, (long long)cols);
    SF_CHECK_ARG(keep_k >= 0 && keep_k <= 256, "sf_mask_update_tile16: keep_k must be in [0, 256]");
    SF_CHECK_ARG(penalty_mode >= 0 && penalty_mode <= 2, "sf_mask_update_tile16: penalty_mode must be 0, 1 or 2");
    SF_CHECK_ARG((wm == nullptr) || (W != nullptr), "sf_mask_update_tile16: wm requested without W");
    SF_CHECK_ARG(w_dtype == SF_F32 || w_dtype == SF_BF16, "sf_mask_update_tile16: w_dtype must be SF_F32 or SF_BF16");
    if (!(aligned16(score) && aligned16(mask) && aligned16(W) && aligned16(wm)))
        return fail(SF_ERR_ALIGNMENT, "sf_mask_update_tile16: buffers must be 16-byte aligned");
    TileUpdateParams P;
    P.neg_log2e_over_t = (float)(-1.4426950408889634 / (double)((float)temperature + 1e-8f));
    P.a = (float)mask_lr;
    P.one_minus_a = (float)(1.0 - mask_lr);
    P.pen = (float)pen;
    P.penalty_mode = pen != 0.0 ? penalty_mode : 0;
    P.bin_lo = (float)(1.0 - binarize_decay);
    P.bin_hi = (float)(1.0 + binarize_decay);
    P.binarize = binarize_decay != 0.0;
    P.hx = (float)hx;
    P.one_minus_hx = (float)(1.0 - hx);
    P.soft_only = hx >= 1.0 - 1e-6;
    P.keep_k = keep_k;
    cudaStream_t st = (cudaStream_t)stream;
    SF_CHECK_CUDA(cudaMemsetAsync(stats, 0, SF_MSTAT_COUNT * sizeof(double), st));
    const int tr = (int)(rows / 16), tc = (int)(cols / 16);
    const int grid = tile_grid((int64_t)tr * tc);
    if (w_dtype == SF_F32)
        mask_update_tile16_kernel<float><<<grid, kTileThreads, 0, st>>>(score, norm, tau, mask, (const float*)W, (float*)wm, stats, cols, tr, tc, P);
    else
        mask_update_tile16_kernel<__nv_bfloat16><<<grid, kTileThreads, 0, st>>>(score, norm, tau, mask, (const __nv_bfloat16*)W,
                                                                               (__nv_bfloat16*)wm, stats, cols, tr, tc, P);
    SF_CHECK_CUDA(cudaGetLastError());
    return SF_OK;
}

int sf_project_tile16(const float* soft, float* hard, const void* W, int w_dtype, void* wm, int64_t rows, int64_t cols,
                      int keep_k, double hx, void* stream) {
    SF_CHECK_ARG(soft != nullptr && (hard != nullptr || wm != nullptr), "sf_project_tile16: soft and one of hard / wm must be non-null");
    SF_CHECK_ARG(rows > 0 && cols > 0 && rows % 16 == 0 && cols % 16 == 0,
                 "sf_project_tile16: rows=%lld and cols=%lld must be multiples of 16", (long long)rows, (long long)cols);
    SF_CHECK_ARG(keep_k >= 0 && keep_k <= 256, "sf_project_tile16: keep_k must be in [0, 256]");
    SF_CHECK_ARG((wm == nullptr) || (W != nullptr), "sf_project_tile16: wm requested without W");
    SF_CHECK_ARG(w_dtype == SF_F32 || w_dtype == SF_BF16, "sf_project_tile16: w_dtype must be SF_F32 or SF_BF16");
    if (!(aligned16(soft) && aligned16(hard) && aligned16(W) && aligned16(wm)))
        return fail(SF_ERR_ALIGNMENT, "sf_project_tile16: buffers must be 16-byte aligned");
    cudaStream_t st = (cudaStream_t)stream;
    const int tr = (int)(rows / 16), tc = (int)(cols / 16);
    const int grid = tile_grid((int64_t)tr * tc);
    if (w_dtype == SF_F32)
        project_tile16_kernel<float><<<grid, kTileThreads, 0, st>>>(soft, hard, (const float*)W, (float*)wm, cols, tr, tc, keep_k, (float)hx);
    else
        project_tile16_kernel<__nv_bfloat16><<<grid, kTileThreads, 0, st>>>(soft, hard, (const __nv_bfloat16*)W, (__nv_bfloat16*)wm,
                                                                           cols, tr, tc, keep_k, (float)hx);
    SF_CHECK_CUDA(cudaGetLastError());
    return SF_OK;
}

}  // extern "C"
