// Peer-memory plumbing for row-sharded layers: exporting a device buffer to the other ranks of
// one node through CUDA IPC, and the owner-side sum of the partial input gradients that the
// sharded dgrad epilogue scattered into per-rank slots.
#include <cuda.h>
#include <cuda_runtime.h>

#include <cstdint>
#include <cstring>

#include "common.cuh"

namespace sf {

constexpr int kThreads = 256;

// out[i] = sum_g slots[g][i], accumulated in fp32 in rank order (deterministic), 8 elements per thread.
// GT > 0: the slot count is a compile-time constant, so all GT loads of a chunk are in flight together.
template <typename T, int GT>
__global__ void __launch_bounds__(kThreads)
reduce_slots_kernel(const T* __restrict__ slots, T* __restrict__ out, int64_t chunks, int64_t slot_stride, int G) {
    for (int64_t c = (int64_t)blockIdx.x * kThreads + threadIdx.x; c < chunks; c += (int64_t)gridDim.x * kThreads) {
        float acc[8];
        if (GT > 0) {
            float x[GT > 0 ? GT : 1][8];
#pragma unroll
            for (int g = 0; g < GT; ++g) Vec8<T>::load(slots + g * slot_stride + c * 8, x[g]);
#pragma unroll
            for (int i = 0; i < 8; ++i) acc[i] = x[0][i];
#pragma unroll
            for (int g = 1; g < GT; ++g)
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[i] += x[g][i];
        } else {
            float x[8];
            Vec8<T>::load(slots + c * 8, acc);
            for (int g = 1; g < G; ++g) {
                Vec8<T>::load(slots + g * slot_stride + c * 8, x);
#pragma unroll
                for (int i = 0; i < 8; ++i) acc[i] += x[i];
            }
        }
        Vec8<T>::store(out + c * 8, acc);
    }
}

// out[i] = sum over the GPUs bound to a multicast object of their copy of src[i]: one
// multimem.ld_reduce per 16 bytes (eight bf16) makes the NVSwitch read every GPU's copy and add them
// in fp32, so an owner receives only the sum of its rows (1/N of what a store-based scatter lands on
// it) while every GPU's copy leaves it once. A read takes about 4 us to come back, so the rate is set by
// the bytes in flight: eight reads per thread; the thread blocks need no shared memory and fit beside
// the blocks of a tensor-core product.
__global__ void __launch_bounds__(kThreads)
multimem_reduce_bf16_kernel(const uint4* __restrict__ mc_src, uint4* __restrict__ out, int64_t chunks) {
    const int64_t stride = (int64_t)gridDim.x * kThreads;
    for (int64_t c0 = (int64_t)blockIdx.x * kThreads + threadIdx.x; c0 < chunks; c0 += 8 * stride) {
        uint4 v[8];
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int64_t c = c0 + j * stride;
            if (c < chunks)
                asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                             : "=r"(v[j].x), "=r"(v[j].y), "=r"(v[j].z), "=r"(v[j].w)
                             : "l"(mc_src + c)
                             : "memory");
        }
#pragma unroll
        for (int j = 0; j < 8; ++j) {
            const int64_t c = c0 + j * stride;
            if (c < chunks) out[c] = v[j];
        }
    }
}

}  // namespace sf

using namespace sf;

extern "C" {

int sf_multimem_reduce(const void* mc_src, void* out, int64_t n, int dtype, int max_ctas, void* stream) {
    SF_CHECK_ARG(mc_src && out, "sf_multimem_reduce: mc_src and out must be non-null");
    SF_CHECK_ARG(n > 0 && n % 8 == 0, "sf_multimem_reduce: n=%lld must be a positive multiple of 8", (long long)n);
    if (dtype != SF_BF16) return fail(SF_ERR_UNSUPPORTED, "sf_multimem_reduce: bf16 only");
    SF_CHECK_ARG(max_ctas >= 0, "sf_multimem_reduce: max_ctas must be >= 0 (0 = default)");
    if (!aligned16(mc_src) || !aligned16(out)) return fail(SF_ERR_ALIGNMENT, "sf_multimem_reduce: buffers must be 16-byte aligned");
    const int64_t chunks = n / 8;
    int64_t blocks = (chunks + 8 * kThreads - 1) / (8 * kThreads);
    const int64_t cap = max_ctas > 0 ? max_ctas : 64;
    if (blocks > cap) blocks = cap;
    multimem_reduce_bf16_kernel<<<(int)blocks, kThreads, 0, (cudaStream_t)stream>>>((const uint4*)mc_src, (uint4*)out, chunks);
    SF_CHECK_CUDA(cudaGetLastError());
    return SF_OK;
}

int sf_reduce_slots(const void* slots, void* out, int64_t n_slots, int64_t n, int dtype, void* stream) {
    SF_CHECK_ARG(slots && out, "sf_reduce_slots: slots and out must be non-null");
    SF_CHECK_ARG(n_slots >= 1 && n_slots <= 64, "sf_reduce_slots: 1..64 slots expected");
    SF_CHECK_ARG(n > 0 && n % 8 == 0, "sf_reduce_slots: n=%lld must be a positive multiple of 8", (long long)n);
    SF_CHECK_ARG(dtype == SF_F32 || dtype == SF_BF16, "sf_reduce_slots: dtype must be SF_F32 or SF_BF16");
    if (!aligned16(slots) || !aligned16(out)) return fail(SF_ERR_ALIGNMENT, "sf_reduce_slots: buffers must be 16-byte aligned");
    const int64_t chunks = n / 8;
    int64_t blocks = (chunks + kThreads - 1) / kThreads;
    if (blocks > 148 * 8) blocks = 148 * 8;
    cudaStream_t st = (cudaStream_t)stream;
#define SF_REDUCE(TT, GT) reduce_slots_kernel<TT, GT><<<(int)blocks, kThreads, 0, st>>>((const TT*)slots, (TT*)out, chunks, n, (int)n_slots)
    if (dtype == SF_F32) {
        SF_REDUCE(float, 0);
    } else {
        switch (n_slots) {
            case 2: SF_REDUCE(__nv_bfloat16, 2); break;
            case 4: SF_REDUCE(__nv_bfloat16, 4); break;
            case 8: SF_REDUCE(__nv_bfloat16, 8); break;
            default: SF_REDUCE(__nv_bfloat16, 0);
        }
    }
#undef SF_REDUCE
    SF_CHECK_CUDA(cudaGetLastError());
    return SF_OK;
}

int sf_peer_handle_bytes(void) { return (int)sizeof(cudaIpcMemHandle_t); }

int sf_peer_export(const void* ptr, void* handle, int64_t* offset) {
    SF_CHECK_ARG(ptr && handle && offset, "sf_peer_export: ptr, handle and offset must be non-null");
    cudaIpcMemHandle_t h;
    SF_CHECK_CUDA(cudaIpcGetMemHandle(&h, const_cast<void*>(ptr)));
    // the handle names the whole allocation the pointer lies in; its base is what a peer maps
    typedef CUresult (*AddressRangeFn)(CUdeviceptr*, size_t*, CUdeviceptr);
    void* fp = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &fp, cudaEnableDefault, &qres) != cudaSuccess ||
        qres != cudaDriverEntryPointSuccess || fp == nullptr)
        return fail(SF_ERR_CUDA, "sf_peer_export: cuMemGetAddressRange is not available from the driver");
    CUdeviceptr base = 0;
    size_t size = 0;
    const CUresult r = reinterpret_cast<AddressRangeFn>(fp)(&base, &size, (CUdeviceptr)(uintptr_t)ptr);
    if (r != CUDA_SUCCESS) return fail(SF_ERR_CUDA, "sf_peer_export: cuMemGetAddressRange failed (CUresult %d)", (int)r);
    std::memcpy(handle, &h, sizeof(h));
    *offset = (int64_t)((uintptr_t)ptr - (uintptr_t)base);
    return SF_OK;
}

int sf_peer_open(const void* handle, int64_t offset, void** base, void** ptr) {
    SF_CHECK_ARG(handle && base && ptr && offset >= 0, "sf_peer_open: handle, base, ptr must be non-null");
    cudaIpcMemHandle_t h;
    std::memcpy(&h, handle, sizeof(h));
    void* b = nullptr;
    SF_CHECK_CUDA(cudaIpcOpenMemHandle(&b, h, cudaIpcMemLazyEnablePeerAccess));
    *base = b;
    *ptr = (char*)b + offset;
    return SF_OK;
}

int sf_peer_close(void* base) {
    SF_CHECK_ARG(base != nullptr, "sf_peer_close: base must be non-null");
    SF_CHECK_CUDA(cudaIpcCloseMemHandle(base));
    return SF_OK;
}

}  // extern "C"
