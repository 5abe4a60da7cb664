// Block-granular soft masks (hard_mask_type block_sparse16 / block_sparse32 of the reference).
//
// In these modes the reference pools scores and masks over bs x bs blocks and keeps the soft mask
// block-constant (legacy/sparse_modeling.py:461-508 _blockify_tensor, :1122-1157 gate, :1395-1530
// penalty, :1600 mask blockify, :607-718 hard projection). Everything that depends on the whole
// layer (quantile of the block scores, top-k blocks) works on [out/bs, in/bs] arrays, 256 or 1024
// times smaller than the layer; the passes over the layer itself are the three kernels here:
//   block_sums:        per-block sum and sum of squares of an fp32 tensor (scores, or a mask)
//   block_mask_update: the EMA update of every element from its block's gate / target values,
//                      returning only the per-block sums of the result (the mask is re-written
//                      block-constant by the next kernel); the ragged tail beyond whole blocks is
//                      updated in place
//   block_mask_apply:  mask <- block value, masked weight <- W * (hx * mask + (1 - hx) * keep)
// A CTA owns one band of bs rows; a thread owns four consecutive columns of every row of the band,
// so loads are contiguous 16-byte accesses and the bs / 4 lanes that share a block are neighbours.
#include "common.cuh"

namespace sf {

constexpr int kBlkThreads = 256;

__device__ __forceinline__ float load_scalar_w(const float* p) { return *p; }
__device__ __forceinline__ float load_scalar_w(const __nv_bfloat16* p) { return __bfloat162float(*p); }
__device__ __forceinline__ void store_scalar_w(float* p, float v) { *p = v; }
__device__ __forceinline__ void store_scalar_w(__nv_bfloat16* p, float v) { *p = __float2bfloat16_rn(v); }

template <int BS>
__device__ __forceinline__ float group_sum(float v) {
    // lanes of one block: BS / 4 consecutive lanes (4 for 16, 8 for 32)
#pragma unroll
    for (int o = BS / 8; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

template <int BS>
__global__ void __launch_bounds__(kBlkThreads)
block_sums_kernel(const float* __restrict__ x, int64_t ld, int ob, int ib, const float* __restrict__ norm,
                  float* __restrict__ sum, float* __restrict__ sumsq) {
    // norm != null: the sums are taken over (x - norm[0]) / norm[1], the normalised score
    const float mu = norm != nullptr ? norm[0] : 0.0f;
    const float inv_sigma = norm != nullptr ? __fdiv_rn(1.0f, norm[1]) : 1.0f;
    const int band = blockIdx.x;  // block row
    const int cols_full = ib * BS;
    // every thread of a warp takes part in the shuffles: the loop bound is the same for all
    for (int base = 0; base < cols_full; base += kBlkThreads * 4) {
        const int c0 = base + threadIdx.x * 4;
        const bool valid = c0 < cols_full;
        float s = 0.f, s2 = 0.f;
        if (valid) {
#pragma unroll 4
            for (int r = 0; r < BS; ++r) {
                float4 v = __ldcs(reinterpret_cast<const float4*>(x + ((int64_t)band * BS + r) * ld + c0));
                if (norm != nullptr) {
                    v.x = __fmul_rn(__fsub_rn(v.x, mu), inv_sigma); v.y = __fmul_rn(__fsub_rn(v.y, mu), inv_sigma);
                    v.z = __fmul_rn(__fsub_rn(v.z, mu), inv_sigma); v.w = __fmul_rn(__fsub_rn(v.w, mu), inv_sigma);
                }
                s += (v.x + v.y) + (v.z + v.w);
                s2 = fmaf(v.x, v.x, fmaf(v.y, v.y, fmaf(v.z, v.z, fmaf(v.w, v.w, s2))));
            }
        }
        s = group_sum<BS>(s);
        s2 = group_sum<BS>(s2);
        if (valid && (c0 / 4) % (BS / 4) == 0) {
            sum[(int64_t)band * ib + c0 / BS] = s;
            if (sumsq != nullptr) sumsq[(int64_t)band * ib + c0 / BS] = s2;
        }
    }
}

struct BlockUpdateParams {
    float a, one_minus_a;  // mask_lr
    float pen;             // penalty_lr * lambda_mid (0: no pull)
    float bin_lo, bin_hi;  // binarise push factors (1 - d, 1 + d)
    int binarize;
};

__device__ __forceinline__ float block_ema(float m, float g, float tgt, const BlockUpdateParams& P) {
    float G = g;
    if (P.pen != 0.0f) G = fminf(fmaxf(__fsub_rn(G, __fmul_rn(P.pen, __fsub_rn(m, tgt))), 0.0f), 1.0f);
    if (P.binarize) {
        if (G < 0.5f) G = __fmul_rn(G, P.bin_lo);
        else if (G > 0.5f) G = __fmul_rn(G, P.bin_hi);
    }
    return __saturatef(__fmaf_rn(P.a, G, __fmul_rn(m, P.one_minus_a)));
}

// new_sum[block] = sum over the block of clamp((1-a) m + a G'), G' the block's gate after the penalty
// pull towards the block's target and the binarise push. Elements beyond the whole blocks (tail
// rows / columns) have gate 1 and target 1 and are updated in place.
template <int BS>
__global__ void __launch_bounds__(kBlkThreads)
block_mask_update_kernel(float* __restrict__ mask, int64_t rows, int64_t cols, int ob, int ib,
                         const float* __restrict__ gate, const float* __restrict__ target, BlockUpdateParams P,
                         float* __restrict__ new_sum) {
    const int band = blockIdx.x;
    const int cols_full = ib * BS;
    if (band < ob) {
        for (int base = 0; base < cols_full; base += kBlkThreads * 4) {
            const int c0 = base + threadIdx.x * 4;
            const bool valid = c0 < cols_full;
            const int64_t b = (int64_t)band * ib + (valid ? c0 / BS : 0);
            float s = 0.f;
            if (valid) {
                const float g = gate[b];
                const float tgt = target != nullptr ? target[b] : 0.0f;
#pragma unroll 4
                for (int r = 0; r < BS; ++r) {
                    const float4 v = __ldcs(reinterpret_cast<const float4*>(mask + ((int64_t)band * BS + r) * cols + c0));
                    s += (block_ema(v.x, g, tgt, P) + block_ema(v.y, g, tgt, P)) +
                         (block_ema(v.z, g, tgt, P) + block_ema(v.w, g, tgt, P));
                }
            }
            s = group_sum<BS>(s);
            if (valid && (c0 / 4) % (BS / 4) == 0) new_sum[b] = s;
        }
        // tail columns of this band
        for (int64_t i = threadIdx.x; i < (int64_t)BS * (cols - cols_full); i += kBlkThreads) {
            const int64_t r = (int64_t)band * BS + i / (cols - cols_full), c = cols_full + i % (cols - cols_full);
            mask[r * cols + c] = block_ema(mask[r * cols + c], 1.0f, 1.0f, P);
        }
    } else {
        // tail rows (all columns): one extra CTA
        const int64_t r0 = (int64_t)ob * BS;
        for (int64_t i = threadIdx.x; i < (rows - r0) * cols; i += kBlkThreads)
            mask[r0 * cols + i] = block_ema(mask[r0 * cols + i], 1.0f, 1.0f, P);
    }
}

// mask <- block value inside the whole blocks; wm <- W * cast(hx * mask + (1 - hx) * hard), hard =
// keep[block] inside the whole blocks and 1 in the tail.
template <typename TW, int BS>
__global__ void __launch_bounds__(kBlkThreads)
block_mask_apply_kernel(float* __restrict__ mask, const TW* __restrict__ W, TW* __restrict__ wm, int64_t rows,
                        int64_t cols, int ob, int ib, const float* __restrict__ value,
                        const uint8_t* __restrict__ keep, float hx, int write_mask) {
    const int64_t total = rows * cols;
    // cols % 4 == 0 and bs % 4 == 0: four consecutive elements share row, block and tail status
    for (int64_t i = ((int64_t)blockIdx.x * kBlkThreads + threadIdx.x) * 4; i < total;
         i += (int64_t)gridDim.x * kBlkThreads * 4) {
        const int64_t r = i / cols, c = i - r * cols;
        const bool inside = r < (int64_t)ob * BS && c < (int64_t)ib * BS;
        float4 m4;
        float hard = 1.0f;
        if (inside) {
            const int64_t b = (r / BS) * ib + c / BS;
            hard = keep[b] ? 1.0f : 0.0f;
            if (value != nullptr) {
                const float v = value[b];
                m4 = make_float4(v, v, v, v);
                if (write_mask) *reinterpret_cast<float4*>(mask + i) = m4;
            } else {
                m4 = *reinterpret_cast<const float4*>(mask + i);
            }
        } else {
            m4 = *reinterpret_cast<const float4*>(mask + i);
        }
        if (wm != nullptr) {
            const float m[4] = {m4.x, m4.y, m4.z, m4.w};
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float eff = hx >= 1.0f - 1e-6f ? m[e] : __fadd_rn(__fmul_rn(hx, m[e]), __fmul_rn(1.0f - hx, hard));
                store_scalar_w(wm + i + e, __fmul_rn(load_scalar_w(W + i + e), Vec8<TW>::round(eff)));
            }
        }
    }
}

}  // namespace sf

using namespace sf;

extern "C" {

int sf_block_sums(const float* x, int64_t rows, int64_t cols, int bs, const float* norm, float* sum, float* sumsq,
                  void* stream) {
    SF_CHECK_ARG(x && sum, "sf_block_sums: x and sum must be non-null");
    SF_CHECK_ARG(bs == 16 || bs == 32, "sf_block_sums: bs must be 16 or 32");
    SF_CHECK_ARG(rows >= bs && cols >= bs && cols % 4 == 0, "sf_block_sums: need at least one whole block and cols %% 4 == 0");
    if (!aligned16(x)) return fail(SF_ERR_ALIGNMENT, "sf_block_sums: x must be 16-byte aligned");
    const int ob = (int)(rows / bs), ib = (int)(cols / bs);
    cudaStream_t st = (cudaStream_t)stream;
    if (bs == 16) block_sums_kernel<16><<<ob, kBlkThreads, 0, st>>>(x, cols, ob, ib, norm, sum, sumsq);
    else block_sums_kernel<32><<<ob, kBlkThreads, 0, st>>>(x, cols, ob, ib, norm, sum, sumsq);
    SF_CHECK_CUDA(cudaGetLastError());
    return SF_OK;
}

int sf_block_mask_update(float* mask, int64_t rows, int64_t cols, int bs, const float* gate, const float* target,
                         double mask_lr, double pen, double binarize_decay, float* new_sum, void* stream) {
    SF_CHECK_ARG(mask && gate && new_sum, "sf_block_mask_update: mask, gate, new_sum must be non-null");
    SF_CHECK_ARG(bs == 16 || bs == 32, "sf_block_mask_update: bs must be 16 or 32");
    SF_CHECK_ARG(rows >= bs && cols >= bs && cols % 4 == 0, "sf_block_mask_update: need at least one whole block and cols %% 4 == 0");
    SF_CHECK_ARG(pen == 0.0 || target != nullptr, "sf_block_mask_update: a penalty needs the block targets");
    if (!aligned16(mask)) return fail(SF_ERR_ALIGNMENT, "sf_block_mask_update: mask must be 16-byte aligned");
    const int ob = (int)(rows / bs), ib = (int)(cols / bs);
    BlockUpdateParams P;
    P.a = (float)mask_lr;
    P.one_minus_a = (float)(1.0 - mask_lr);
    P.pen = (float)pen;
    P.bin_lo = (float)(1.0 - binarize_decay);
    P.bin_hi = (float)(1.0 + binarize_decay);
    P.binarize = binarize_decay != 0.0;
    cudaStream_t st = (cudaStream_t)stream;
    const int grid = ob + ((int64_t)ob * bs < rows ? 1 : 0);
    if (bs == 16) block_mask_update_kernel<16><<<grid, kBlkThreads, 0, st>>>(mask, rows, cols, ob, ib, gate, target, P, new_sum);
    else block_mask_update_kernel<32><<<grid, kBlkThreads, 0, st>>>(mask, rows, cols, ob, ib, gate, target, P, new_sum);
    SF_CHECK_CUDA(cudaGetLastError());
    return SF_OK;
}

int sf_block_mask_apply(float* mask, const void* W, int w_dtype, void* wm, int64_t rows, int64_t cols, int bs,
                        const float* value, const uint8_t* keep, double hx, void* stream) {
    SF_CHECK_ARG(mask && keep, "sf_block_mask_apply: mask and keep must be non-null");
    SF_CHECK_ARG(bs == 16 || bs == 32, "sf_block_mask_apply: bs must be 16 or 32");
    SF_CHECK_ARG(rows >= bs && cols >= bs && cols % 4 == 0, "sf_block_mask_apply: need at least one whole block and cols %% 4 == 0");
    if (!aligned16(mask)) return fail(SF_ERR_ALIGNMENT, "sf_block_mask_apply: mask must be 16-byte aligned");
    SF_CHECK_ARG((wm == nullptr) || (W != nullptr), "sf_block_mask_apply: wm requested without W");
    SF_CHECK_ARG(w_dtype == SF_F32 || w_dtype == SF_BF16, "sf_block_mask_apply: w_dtype must be SF_F32 or SF_BF16");
    const int ob = (int)(rows / bs), ib = (int)(cols / bs);
    cudaStream_t st = (cudaStream_t)stream;
    int64_t blocks = (rows * cols / 4 + kBlkThreads - 1) / kBlkThreads;
    if (blocks > 148 * 8) blocks = 148 * 8;
    if (blocks < 1) blocks = 1;
#define SF_BA(TW, BS)                                                                                          \
    block_mask_apply_kernel<TW, BS><<<(int)blocks, kBlkThreads, 0, st>>>(mask, (const TW*)W, (TW*)wm, rows, cols, ob, ib, \
                                                                        value, keep, (float)hx, 1)
    if (w_dtype == SF_F32) { if (bs == 16) SF_BA(float, 16); else SF_BA(float, 32); }
    else { if (bs == 16) SF_BA(__nv_bfloat16, 16); else SF_BA(__nv_bfloat16, 32); }
#undef SF_BA
    SF_CHECK_CUDA(cudaGetLastError());
    return SF_OK;
}

}  // extern "C"
