// Block-sparse-16 weights (block-CSR: blocks[nnz,16,16], row_ptr[out/16+1], col_idx[nnz]).
//
// The block-CSR is built on the device (the reference builds it with a Python double loop).
// The three products run on the tcgen05 GEMM kernels through a dense workspace: kept blocks are
// scattered into a zeroed [out,in] matrix (forward, dgrad) or gathered out of the dense weight
// gradient (wgrad). A 16x16 block is one 128x16x16 MMA whose cost is dominated by fetching the
// 128x16 activation operand, so skipping blocks inside the MMA loop does not beat the dense
// tile at 50 % density; the workspace route keeps the tensor cores on full 128x256 tiles.
#include "common.cuh"

namespace sf {

constexpr int BS = 16;

template <typename T>
__device__ __forceinline__ float ldf(const T* p);
template <>
__device__ __forceinline__ float ldf<float>(const float* p) { return *p; }
template <>
__device__ __forceinline__ float ldf<__nv_bfloat16>(const __nv_bfloat16* p) { return __bfloat162float(*p); }
template <typename T>
__device__ __forceinline__ T from_f(float v);
template <>
__device__ __forceinline__ float from_f<float>(float v) { return v; }
template <>
__device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// One CTA per block row; warp w looks at block columns w, w+8, ...; a block is kept iff
// sum |w * mask| > 0 (legacy/triton_block_sparse.py:79, 87).
template <typename TW, typename TM>
__device__ __forceinline__ bool block_nonzero(const TW* W, const TM* mask, int64_t in, int64_t brow, int64_t bcol, int lane) {
    float acc = 0.0f;
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int e = lane * 8 + i;  // 256 elements per block, 8 per lane
        const int64_t idx = (brow * BS + (e >> 4)) * in + bcol * BS + (e & 15);
        acc += fabsf(ldf<TW>(W + idx) * (mask ? ldf<TM>(mask + idx) : 1.0f));
    }
    acc = warp_sum(acc);
    return acc > 0.0f;
}

template <typename TW, typename TM>
__global__ void __launch_bounds__(256)
bsr16_count_kernel(const TW* __restrict__ W, const TM* __restrict__ mask, int32_t* __restrict__ row_ptr, int64_t in, int64_t ib) {
    __shared__ int cnt;
    if (threadIdx.x == 0) cnt = 0;
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    int local = 0;
    for (int64_t c = warp; c < ib; c += 8) local += block_nonzero<TW, TM>(W, mask, in, blockIdx.x, c, lane) ? 1 : 0;
    if (lane == 0 && local) atomicAdd(&cnt, local);
    __syncthreads();
    if (threadIdx.x == 0) row_ptr[blockIdx.x + 1] = cnt;
}

// Exclusive scan of the per-row counts, in place (one CTA; out/16 is a few hundred to a few thousand).
__global__ void __launch_bounds__(1024)
bsr16_scan_kernel(int32_t* __restrict__ row_ptr, int64_t ob, int32_t* __restrict__ nnz_out) {
    __shared__ int32_t part[1024];
    const int64_t per = (ob + 1023) / 1024;
    const int64_t b = (int64_t)threadIdx.x * per;
    int32_t s = 0;
    for (int64_t i = b; i < b + per && i < ob; ++i) s += row_ptr[i + 1];
    part[threadIdx.x] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
        int32_t run = 0;
        for (int i = 0; i < 1024; ++i) { int32_t v = part[i]; part[i] = run; run += v; }
        row_ptr[0] = 0;
        if (nnz_out) *nnz_out = run;
    }
    __syncthreads();
    int32_t run = part[threadIdx.x];
    for (int64_t i = b; i < b + per && i < ob; ++i) { run += row_ptr[i + 1]; row_ptr[i + 1] = run; }
}

// One CTA per block row: keeps block columns in ascending order, copies W*mask into blocks.
template <typename TW, typename TM>
__global__ void __launch_bounds__(256)
bsr16_fill_kernel(const TW* __restrict__ W, const TM* __restrict__ mask, const int32_t* __restrict__ row_ptr,
                  int32_t* __restrict__ col_idx, TW* __restrict__ blocks, int64_t in, int64_t ib) {
    __shared__ int flags[8];
    __shared__ int base;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) base = row_ptr[blockIdx.x];
    __syncthreads();
    for (int64_t c0 = 0; c0 < ib; c0 += 8) {
        const int64_t c = c0 + warp;
        const bool keep = c < ib && block_nonzero<TW, TM>(W, mask, in, blockIdx.x, c, lane);
        if (lane == 0) flags[warp] = keep ? 1 : 0;
        __syncthreads();
        int before = 0, total = 0;
#pragma unroll
        for (int w = 0; w < 8; ++w) { if (w < warp) before += flags[w]; total += flags[w]; }
        if (keep) {
            const int64_t slot = base + before;
            if (lane == 0) col_idx[slot] = (int32_t)c;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const int e = lane * 8 + i;
                const int64_t idx = ((int64_t)blockIdx.x * BS + (e >> 4)) * in + c * BS + (e & 15);
                blocks[slot * 256 + e] = from_f<TW>(ldf<TW>(W + idx) * (mask ? ldf<TM>(mask + idx) : 1.0f));
            }
        }
        __syncthreads();
        if (threadIdx.x == 0) base += total;
        __syncthreads();
    }
}

// blocks -> dense [out,in] (dense must be zeroed first): one warp per kept block.
template <typename TW>
__global__ void __launch_bounds__(256)
bsr16_scatter_kernel(const TW* __restrict__ blocks, const int32_t* __restrict__ row_ptr, const int32_t* __restrict__ col_idx,
                     TW* __restrict__ dense, int64_t in) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int b0 = row_ptr[blockIdx.x], b1 = row_ptr[blockIdx.x + 1];
    for (int b = b0 + warp; b < b1; b += 8) {
        const int64_t c = col_idx[b];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int e = lane * 8 + i;
            dense[((int64_t)blockIdx.x * BS + (e >> 4)) * in + c * BS + (e & 15)] = blocks[(int64_t)b * 256 + e];
        }
    }
}

// dense [out,in] -> blocks at the kept positions.
template <typename TW>
__global__ void __launch_bounds__(256)
bsr16_gather_kernel(const TW* __restrict__ dense, const int32_t* __restrict__ row_ptr, const int32_t* __restrict__ col_idx,
                    TW* __restrict__ blocks, int64_t in) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int b0 = row_ptr[blockIdx.x], b1 = row_ptr[blockIdx.x + 1];
    for (int b = b0 + warp; b < b1; b += 8) {
        const int64_t c = col_idx[b];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int e = lane * 8 + i;
            blocks[(int64_t)b * 256 + e] = dense[((int64_t)blockIdx.x * BS + (e >> 4)) * in + c * BS + (e & 15)];
        }
    }
}

static int check_bsr(const char* who, int64_t out, int64_t in, int dtype) {
    if (out <= 0 || in <= 0 || out % BS || in % BS)
        return fail(SF_ERR_BAD_ARG, "%s: out=%lld and in=%lld must be positive multiples of 16", who, (long long)out, (long long)in);
    if (dtype != SF_F32 && dtype != SF_BF16) return fail(SF_ERR_BAD_ARG, "%s: dtype must be SF_F32 or SF_BF16", who);
    if (out / BS > 0x7fffffff) return fail(SF_ERR_UNSUPPORTED, "%s: too many block rows", who);
    return SF_OK;
}

static size_t esize(int dtype) { return dtype == SF_F32 ? 4 : 2; }

static int scatter(const void* blocks, const int32_t* row_ptr, const int32_t* col_idx, void* dense, int64_t in, int64_t out,
                   int dtype, cudaStream_t st) {
    SF_CHECK_CUDA(cudaMemsetAsync(dense, 0, (size_t)out * in * esize(dtype), st));
    if (dtype == SF_F32)
        bsr16_scatter_kernel<float><<<(unsigned)(out / BS), 256, 0, st>>>((const float*)blocks, row_ptr, col_idx, (float*)dense, in);
    else
        bsr16_scatter_kernel<__nv_bfloat16><<<(unsigned)(out / BS), 256, 0, st>>>((const __nv_bfloat16*)blocks, row_ptr, col_idx,
                                                                                 (__nv_bfloat16*)dense, in);
    SF_CHECK_CUDA(cudaGetLastError());
    return SF_OK;
}

}  // namespace sf

using namespace sf;

extern "C" {

int sf_bsr16_build(const void* W, const void* mask, int dtype, int mask_dtype, void* blocks, int32_t* row_ptr,
                   int32_t* col_idx, int32_t* nnz_out, int64_t out, int64_t in, void* stream) {
    int rc = check_bsr("sf_bsr16_build", out, in, dtype);
    if (rc) return rc;
    SF_CHECK_ARG(W && row_ptr, "sf_bsr16_build: W and row_ptr must be non-null");
    SF_CHECK_ARG(mask == nullptr || mask_dtype == SF_F32 || mask_dtype == SF_BF16, "sf_bsr16_build: mask_dtype must be SF_F32 or SF_BF16");
    SF_CHECK_ARG((blocks == nullptr) == (col_idx == nullptr), "sf_bsr16_build: blocks and col_idx must be given together");
    cudaStream_t st = (cudaStream_t)stream;
    const int64_t ob = out / BS, ib = in / BS;
#define SF_BSR_DISPATCH(KERNEL, ...)                                                                              \
    do {                                                                                                          \
        if (dtype == SF_F32 && (mask == nullptr || mask_dtype == SF_F32))                                         \
            KERNEL<float, float><<<(unsigned)ob, 256, 0, st>>>((const float*)W, (const float*)mask, __VA_ARGS__); \
        else if (dtype == SF_F32)                                                                                 \
            KERNEL<float, __nv_bfloat16><<<(unsigned)ob, 256, 0, st>>>((const float*)W, (const __nv_bfloat16*)mask, __VA_ARGS__); \
        else if (mask == nullptr || mask_dtype == SF_BF16)                                                        \
            KERNEL<__nv_bfloat16, __nv_bfloat16><<<(unsigned)ob, 256, 0, st>>>((const __nv_bfloat16*)W, (const __nv_bfloat16*)mask, __VA_ARGS__); \
        else                                                                                                      \
            KERNEL<__nv_bfloat16, float><<<(unsigned)ob, 256, 0, st>>>((const __nv_bfloat16*)W, (const float*)mask, __VA_ARGS__); \
    } while (0)
    if (blocks == nullptr) {
        SF_BSR_DISPATCH(bsr16_count_kernel, row_ptr, in, ib);
        SF_CHECK_CUDA(cudaGetLastError());
        bsr16_scan_kernel<<<1, 1024, 0, st>>>(row_ptr, ob, nnz_out);
        SF_CHECK_CUDA(cudaGetLastError());
        return SF_OK;
    }
    if (dtype == SF_F32 && (mask == nullptr || mask_dtype == SF_F32))
        bsr16_fill_kernel<float, float><<<(unsigned)ob, 256, 0, st>>>((const float*)W, (const float*)mask, row_ptr, col_idx, (float*)blocks, in, ib);
    else if (dtype == SF_F32)
        bsr16_fill_kernel<float, __nv_bfloat16><<<(unsigned)ob, 256, 0, st>>>((const float*)W, (const __nv_bfloat16*)mask, row_ptr, col_idx, (float*)blocks, in, ib);
    else if (mask == nullptr || mask_dtype == SF_BF16)
        bsr16_fill_kernel<__nv_bfloat16, __nv_bfloat16><<<(unsigned)ob, 256, 0, st>>>((const __nv_bfloat16*)W, (const __nv_bfloat16*)mask, row_ptr, col_idx, (__nv_bfloat16*)blocks, in, ib);
    else
        bsr16_fill_kernel<__nv_bfloat16, float><<<(unsigned)ob, 256, 0, st>>>((const __nv_bfloat16*)W, (const float*)mask, row_ptr, col_idx, (__nv_bfloat16*)blocks, in, ib);
#undef SF_BSR_DISPATCH
    SF_CHECK_CUDA(cudaGetLastError());
    return SF_OK;
}

int sf_bsr16_to_dense(const void* blocks, const int32_t* row_ptr, const int32_t* col_idx, void* dense, int64_t in,
                      int64_t out, int dtype, void* stream) {
    int rc = check_bsr("sf_bsr16_to_dense", out, in, dtype);
    if (rc) return rc;
    SF_CHECK_ARG(blocks && row_ptr && col_idx && dense, "sf_bsr16_to_dense: pointers must be non-null");
    return scatter(blocks, row_ptr, col_idx, dense, in, out, dtype, (cudaStream_t)stream);
}

int sf_bsr16_fwd(const void* x, const void* blocks, const int32_t* row_ptr, const int32_t* col_idx, const void* bias,
                 void* y, void* workspace, int64_t T, int64_t in, int64_t out, int dtype, int32_t* status, void* stream) {
    int rc = check_bsr("sf_bsr16_fwd", out, in, dtype);
    if (rc) return rc;
    SF_CHECK_ARG(x && blocks && row_ptr && col_idx && y && workspace, "sf_bsr16_fwd: pointers must be non-null");
    rc = scatter(blocks, row_ptr, col_idx, workspace, in, out, dtype, (cudaStream_t)stream);
    if (rc) return rc;
    return sf_masked_gemm_fwd(x, workspace, bias, y, T, in, out, 1.0f, dtype, status, stream);
}

int sf_bsr16_dgrad(const void* dy, const void* blocks, const int32_t* row_ptr, const int32_t* col_idx, void* dx,
                   void* workspace, int64_t T, int64_t in, int64_t out, int dtype, int32_t* status, void* stream) {
    int rc = check_bsr("sf_bsr16_dgrad", out, in, dtype);
    if (rc) return rc;
    SF_CHECK_ARG(dy && blocks && row_ptr && col_idx && dx && workspace, "sf_bsr16_dgrad: pointers must be non-null");
    rc = scatter(blocks, row_ptr, col_idx, workspace, in, out, dtype, (cudaStream_t)stream);
    if (rc) return rc;
    return sf_masked_gemm_dgrad(dy, workspace, dx, T, in, out, dtype, status, stream);
}

int sf_bsr16_wgrad(const void* dy, const void* x, const int32_t* row_ptr, const int32_t* col_idx, void* dblocks,
                   void* workspace, int64_t T, int64_t in, int64_t out, int dtype, int32_t* status, void* stream) {
    int rc = check_bsr("sf_bsr16_wgrad", out, in, dtype);
    if (rc) return rc;
    SF_CHECK_ARG(dy && x && row_ptr && col_idx && dblocks && workspace, "sf_bsr16_wgrad: pointers must be non-null");
    rc = sf_masked_gemm_wgrad(dy, x, workspace, T, in, out, dtype, status, stream);
    if (rc) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == SF_F32)
        bsr16_gather_kernel<float><<<(unsigned)(out / BS), 256, 0, st>>>((const float*)workspace, row_ptr, col_idx, (float*)dblocks, in);
    else
        bsr16_gather_kernel<__nv_bfloat16><<<(unsigned)(out / BS), 256, 0, st>>>((const __nv_bfloat16*)workspace, row_ptr, col_idx,
                                                                                (__nv_bfloat16*)dblocks, in);
    SF_CHECK_CUDA(cudaGetLastError());
    return SF_OK;
}

}  // extern "C"
