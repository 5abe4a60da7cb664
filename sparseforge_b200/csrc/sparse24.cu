// Hard-2:4 compressed weights and their GEMM on the sparse tensor cores.
//
// Storage: values[out, in/2] (the two kept bf16 of every group of four, in column order) and
// logical metadata (one nibble per group, i0 | i1 << 2; see sparseforge_b200.h). For the GEMM the
// metadata is reordered once into "tensor-core order": tiles of 128 rows x 128 logical columns,
// 2048 contiguous bytes each, laid out so that one tcgen05.cp.128x128b moves a tile from shared
// memory into 4 TMEM columns in exactly the lane / bit positions tcgen05.mma.sp reads:
//   row m = m0 + 8 m1 + 16 m2 (m0 < 8, m1 < 2, m2 < 8), logical column k = k0 + 16 k1 + 32 k2
//   byte offset in the tile = 256 m2 + 128 k1 + 16 m0 + 4 k2 + 2 m1 + (k0 >> 3)
// i.e. TMEM lane 16 m2 + 8 k1 + m0, column k2, bits [16 m1, 16 m1 + 16) hold the four nibbles of
// row m, columns [32 k2 + 16 k1, +16).
//
// GEMM: y[T,out] = x[T,in] . Wc^T computed as D[out-tile 128, token-tile BN] so that the sparse
// operand is the MMA's A operand. One CTA = TMA producer warp, MMA warp (tcgen05.cp of the
// metadata + four tcgen05.mma.sp 128 x BN x 32 per 128-deep stage), four epilogue warps that
// write the transposed accumulator to y. Token tile BN is picked from T (16 ... 128).
#include <cuda.h>

#include "common.cuh"
#include "ptx_sm100.cuh"

namespace sf {

int make_bf16_tensor_map(CUtensorMap* map, const void* ptr, int64_t inner, int64_t outer, int64_t ld, int box_outer);

constexpr int kThreadsE = 256;

static inline int grid_for_e(int64_t items) {
    int64_t need = (items + kThreadsE - 1) / kThreadsE;
    int64_t cap = (int64_t)sm_count() * 8;
    if (need < 1) need = 1;
    return (int)(need < cap ? need : cap);
}

// ------------------------------------------------------------------------------------------
// compress / decompress / metadata reorder
// ------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(kThreadsE)
sparse24_compress_kernel(const __nv_bfloat16* __restrict__ W, const float* __restrict__ soft,
                         __nv_bfloat16* __restrict__ values, uint8_t* __restrict__ meta, int64_t chunks) {
    for (int64_t c = (int64_t)blockIdx.x * kThreadsE + threadIdx.x; c < chunks; c += (int64_t)gridDim.x * kThreadsE) {
        const uint4 wraw = ld_stream16(W + c * 8);
        const uint16_t* wh = reinterpret_cast<const uint16_t*>(&wraw);
        float s[8];
        Vec8<float>::load(soft + c * 8, s);
        uint16_t out[4];
        uint32_t mb = 0;
#pragma unroll
        for (int g = 0; g < 2; ++g) {
            float x[4] = {s[4 * g], s[4 * g + 1], s[4 * g + 2], s[4 * g + 3]};
            const uint32_t k = top2_keep(x);
            const uint32_t i0 = __ffs(k) - 1, i1 = 31 - __clz(k);
            out[2 * g] = wh[4 * g + i0];
            out[2 * g + 1] = wh[4 * g + i1];
            mb |= (i0 | (i1 << 2)) << (4 * g);
        }
        st_stream8(values + c * 4, make_uint2(out[0] | ((uint32_t)out[1] << 16), out[2] | ((uint32_t)out[3] << 16)));
        meta[c] = (uint8_t)mb;
    }
}

__global__ void __launch_bounds__(kThreadsE)
sparse24_decompress_kernel(const __nv_bfloat16* __restrict__ values, const uint8_t* __restrict__ meta,
                           __nv_bfloat16* __restrict__ dense, int64_t chunks) {
    for (int64_t c = (int64_t)blockIdx.x * kThreadsE + threadIdx.x; c < chunks; c += (int64_t)gridDim.x * kThreadsE) {
        const uint2 v = ld_stream8(values + c * 4);
        const uint16_t vals[4] = {(uint16_t)(v.x & 0xffff), (uint16_t)(v.x >> 16), (uint16_t)(v.y & 0xffff), (uint16_t)(v.y >> 16)};
        const uint32_t mb = meta[c];
        uint16_t o[8] = {0, 0, 0, 0, 0, 0, 0, 0};
#pragma unroll
        for (int g = 0; g < 2; ++g) {
            const uint32_t nib = (mb >> (4 * g)) & 0xF;
            o[4 * g + (nib & 3)] = vals[2 * g];
            o[4 * g + (nib >> 2)] = vals[2 * g + 1];
        }
        st_stream16(dense + c * 8, make_uint4(o[0] | ((uint32_t)o[1] << 16), o[2] | ((uint32_t)o[3] << 16),
                                              o[4] | ((uint32_t)o[5] << 16), o[6] | ((uint32_t)o[7] << 16)));
    }
}

// One thread per 16-bit unit of the tensor-core ordered buffer.
__global__ void __launch_bounds__(kThreadsE)
sparse24_pack_meta_kernel(const uint8_t* __restrict__ meta, uint16_t* __restrict__ meta_tc, int64_t out, int64_t in,
                          int64_t k_tiles, int64_t units) {
    const int64_t row_bytes = in / 8;
    for (int64_t u = (int64_t)blockIdx.x * kThreadsE + threadIdx.x; u < units; u += (int64_t)gridDim.x * kThreadsE) {
        const int64_t tile = u >> 10;           // 1024 units of 2 bytes per tile
        const int w = (int)(u & 1023);          // unit index inside the tile = byte offset / 2
        const int m2 = w >> 7, k1 = (w >> 6) & 1, m0 = (w >> 3) & 7, k2 = (w >> 1) & 3, m1 = w & 1;
        const int64_t mt = tile / k_tiles, kt = tile - mt * k_tiles;
        const int64_t row = mt * 128 + m0 + 8 * m1 + 16 * m2;
        const int64_t byte = kt * 16 + k2 * 4 + k1 * 2;  // logical metadata byte of column 128 kt + 32 k2 + 16 k1
        uint16_t v = 0;
        if (row < out && byte + 1 < row_bytes + 1) {
            const uint8_t b0 = byte < row_bytes ? meta[row * row_bytes + byte] : 0;
            const uint8_t b1 = byte + 1 < row_bytes ? meta[row * row_bytes + byte + 1] : 0;
            v = (uint16_t)b0 | ((uint16_t)b1 << 8);
        }
        meta_tc[u] = v;
    }
}

// ------------------------------------------------------------------------------------------
// sparse tensor-core GEMM
// ------------------------------------------------------------------------------------------
constexpr int SP_BM = 128, SP_BK = 128 /* logical */, SP_THREADS = 192;
constexpr int SP_A_BYTES = SP_BM * (SP_BK / 2) * 2;  // 16 KiB of compressed values
constexpr int SP_META_BYTES = 2048;

template <int BN> struct SpCfg {
    static constexpr int STAGES = BN >= 128 ? 4 : (BN == 64 ? 6 : 8);
    static constexpr int B_BOX_BYTES = BN * 128;              // 64 logical columns of BN token rows
    static constexpr int STAGE_BYTES = SP_A_BYTES + 2 * B_BOX_BYTES + SP_META_BYTES;
    static constexpr int META_COL0 = 2 * BN;                  // TMEM columns after the two accumulators
    static constexpr int TMEM_NEED = 2 * BN + 4 * STAGES;
    static constexpr int TMEM_COLS = TMEM_NEED <= 64 ? 64 : (TMEM_NEED <= 128 ? 128 : (TMEM_NEED <= 256 ? 256 : 512));
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
};

template <int STAGES>
struct SpSmemTail {
    uint64_t full[STAGES];
    uint64_t empty[STAGES];
    uint64_t tmem_full[2];
    uint64_t tmem_empty[2];
    uint32_t tmem_base;
    int abort_flag;
};

__device__ __forceinline__ void bulk_load_1d(uint32_t smem_dst, const void* gsrc, uint32_t bytes, uint32_t bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_dst), "l"(gsrc), "r"(bytes), "r"(bar)
                 : "memory");
}

__device__ __forceinline__ void tmem_ld_32x32b_x16(uint32_t taddr, uint32_t (&r)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"
        : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]),
          "=r"(r[8]), "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
        : "r"(taddr)
        : "memory");
}

// Same near-square patch order as the dense GEMM: groups of 16 weight-row tiles.
__device__ __forceinline__ void sp_tile_coords(int tile, int tiles_m, int tiles_n, int& tm, int& tn) {
    constexpr int G = 16;
    const int per_group = G * tiles_n;
    const int g = tile / per_group;
    const int first_m = g * G;
    const int gm = min(G, tiles_m - first_m);
    const int r = tile - g * per_group;
    tm = first_m + r % gm;
    tn = r / gm;
}

// Work of one CTA of the 1-CTA kernel. Whole-tile mode (range_kb = 0): tiles round robin, each with its
// whole K loop. Ranged mode (few tiles, short activations): the K blocks of all tiles, numbered tile by
// tile, are dealt out in equal runs of range_kb blocks, one run per CTA, so that every SM streams the same
// share of the weight whatever the tile count; a run that crosses a tile boundary yields two items. A
// tile covered by several runs is summed through the workspace: part p of the tile is the p-th run that
// touches it, nparts their number.
struct SpItem {
    int mn, kb0, kb1, part, nparts;
};
struct SpIter {
    int range_kb, num_kb, mn_tiles, g, g_end, tile;
    __device__ __forceinline__ void init(int range_kb_, int num_kb_, int mn_tiles_) {
        range_kb = range_kb_; num_kb = num_kb_; mn_tiles = mn_tiles_;
        g = (int)blockIdx.x * range_kb;
        g_end = min(g + range_kb, mn_tiles * num_kb);
        tile = (int)blockIdx.x;
    }
    __device__ __forceinline__ bool next(SpItem& it) {
        if (range_kb > 0) {
            if (g >= g_end) return false;
            const int t = g / num_kb;
            it.mn = t;
            it.kb0 = g - t * num_kb;
            it.kb1 = min(num_kb, it.kb0 + (g_end - g));
            const int first = (t * num_kb) / range_kb, last = ((t + 1) * num_kb - 1) / range_kb;
            it.part = (int)blockIdx.x - first;
            it.nparts = last - first + 1;
            g += it.kb1 - it.kb0;
            return true;
        }
        if (tile >= mn_tiles) return false;
        it.mn = tile; it.kb0 = 0; it.kb1 = num_kb; it.part = 0; it.nparts = 1;
        tile += (int)gridDim.x;
        return true;
    }
};

template <int BN>
__global__ void __launch_bounds__(SP_THREADS, 1)
sparse24_gemm_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                     const uint8_t* __restrict__ meta_tc, __nv_bfloat16* __restrict__ Y,
                     const __nv_bfloat16* __restrict__ bias, int out, int T, int in, int32_t* status,
                     int range_kb, float* __restrict__ ws, int* __restrict__ counters) {
    // An item that is one of several parts of a tile stores its fp32 partial sums into ws[part][out][BN];
    // the part that draws the last ticket of the tile adds the partial sums in the order part = 0, 1, ...
    // (a fixed order, whoever arrives last), writes Y and resets the ticket.
    using C = SpCfg<BN>;
    constexpr int STAGES = C::STAGES;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = ptx::smem_u32(smem_raw);
    const uint32_t base = (raw_addr + 1023u) & ~1023u;
    uint8_t* base_ptr = smem_raw + (base - raw_addr);
    auto* tail = reinterpret_cast<SpSmemTail<STAGES>*>(base_ptr + STAGES * C::STAGE_BYTES);
    volatile int* abort_flag = &tail->abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_m = (out + SP_BM - 1) / SP_BM, tiles_n = (T + BN - 1) / BN;
    const int mn_tiles = tiles_m * tiles_n;
    const int num_kb = (in + SP_BK - 1) / SP_BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            ptx::mbar_init(ptx::smem_u32(&tail->full[s]), 1);
            ptx::mbar_init(ptx::smem_u32(&tail->empty[s]), 1);
        }
        for (int a = 0; a < 2; ++a) {
            ptx::mbar_init(ptx::smem_u32(&tail->tmem_full[a]), 1);
            ptx::mbar_init(ptx::smem_u32(&tail->tmem_empty[a]), 4);
        }
        tail->abort_flag = 0;
        ptx::fence_barrier_init();
    }
    if (warp == 1) {
        ptx::tmem_alloc(ptx::smem_u32(&tail->tmem_base), C::TMEM_COLS);
        ptx::tmem_relinquish();
    }
    if (warp == 0 && lane == 0) {
        ptx::prefetch_tensormap(&tmA);
        ptx::prefetch_tensormap(&tmB);
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem_base = tail->tmem_base;

    if (warp == 0) {
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        SpIter iter;
        iter.init(range_kb, num_kb, mn_tiles);
        SpItem it;
        while (ok && iter.next(it)) {
            int mt, nt;
            sp_tile_coords(it.mn, tiles_m, tiles_n, mt, nt);
            for (int kb = it.kb0; kb < it.kb1; ++kb) {
                ok = ptx::mbar_wait(ptx::smem_u32(&tail->empty[stage]), phase ^ 1u, abort_flag, status, 11);
                if (!ok) break;
                if (lane == 0) {
                    const uint32_t bar = ptx::smem_u32(&tail->full[stage]);
                    const uint32_t sa = base + stage * C::STAGE_BYTES, sb = sa + SP_A_BYTES;
                    const uint32_t sm = sb + 2 * C::B_BOX_BYTES;
                    ptx::mbar_arrive_expect_tx(bar, C::STAGE_BYTES);
                    ptx::tma_load_2d(sa, &tmA, bar, kb * (SP_BK / 2), mt * SP_BM);
                    ptx::tma_load_2d(sb, &tmB, bar, kb * SP_BK, nt * BN);
                    ptx::tma_load_2d(sb + C::B_BOX_BYTES, &tmB, bar, kb * SP_BK + 64, nt * BN);
                    bulk_load_1d(sm, meta_tc + ((int64_t)mt * num_kb + kb) * SP_META_BYTES, SP_META_BYTES, bar);
                }
                __syncwarp();
                if (++stage == STAGES) { stage = 0; phase ^= 1u; }
            }
        }
        if (!ok) for (int i = 0; i < 1000; ++i) __nanosleep(1000);
    } else if (warp == 1) {
        constexpr uint32_t idesc = ptx::make_idesc_bf16(SP_BM, BN, 0, 0, 1);
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        int t = 0;
        SpIter iter;
        iter.init(range_kb, num_kb, mn_tiles);
        SpItem it;
        for (; ok && iter.next(it); ++t) {
            const int acc = t & 1;
            const uint32_t acc_phase = (uint32_t)(t >> 1) & 1u;
            ok = ptx::mbar_wait(ptx::smem_u32(&tail->tmem_empty[acc]), acc_phase ^ 1u, abort_flag, status, 13);
            if (!ok) break;
            ptx::tc_fence_after();
            const uint32_t tmem_d = tmem_base + (uint32_t)(acc * BN);
            const int kb0 = it.kb0, kb1 = it.kb1;
            for (int kb = kb0; kb < kb1; ++kb) {
                ok = ptx::mbar_wait(ptx::smem_u32(&tail->full[stage]), phase, abort_flag, status, 12);
                if (!ok) break;
                ptx::tc_fence_after();
                if (lane == 0) {
                    const uint32_t sa = base + stage * C::STAGE_BYTES, sb = sa + SP_A_BYTES;
                    const uint32_t sm = sb + 2 * C::B_BOX_BYTES;
                    const uint32_t tmem_e = tmem_base + (uint32_t)(C::META_COL0 + 4 * stage);
                    // metadata tile: 128 rows of 16 bytes, 8-row groups 128 bytes apart, no swizzle
                    ptx::tmem_cp_128x128b(tmem_e, ptx::make_smem_desc(sm, 16, 128, 0));
#pragma unroll
                    for (int k = 0; k < 4; ++k) {
                        const uint64_t adesc = ptx::make_smem_desc(sa + k * 32, 16, 1024, 2);
                        const uint64_t bdesc = ptx::make_smem_desc(sb + (k >> 1) * C::B_BOX_BYTES + (k & 1) * 64, 16, 1024, 2);
                        ptx::mma_f16_ss_sp(tmem_d, adesc, bdesc, tmem_e + (uint32_t)(k & ~1), idesc | (uint32_t)(k & 1),
                                           (kb != kb0 || k != 0) ? 1u : 0u);
                    }
                    ptx::mma_commit(ptx::smem_u32(&tail->empty[stage]));
                }
                __syncwarp();
                if (++stage == STAGES) { stage = 0; phase ^= 1u; }
            }
            if (!ok) break;
            if (lane == 0) ptx::mma_commit(ptx::smem_u32(&tail->tmem_full[acc]));
            __syncwarp();
        }
    } else {
        const int q = warp & 3;
        bool ok = true;
        int t = 0;
        SpIter iter;
        iter.init(range_kb, num_kb, mn_tiles);
        SpItem it;
        for (; ok && iter.next(it); ++t) {
            int mt, nt;
            const int mn = it.mn;
            const int splits = it.nparts;
            sp_tile_coords(mn, tiles_m, tiles_n, mt, nt);
            const int acc = t & 1;
            const uint32_t acc_phase = (uint32_t)(t >> 1) & 1u;
            ok = ptx::mbar_wait(ptx::smem_u32(&tail->tmem_full[acc]), acc_phase, abort_flag, status, 14);
            if (!ok) break;
            ptx::tc_fence_after();
            const int o = mt * SP_BM + q * 32 + lane;  // output feature of this thread
            const float b = (bias != nullptr && o < out) ? __bfloat162float(bias[o]) : 0.0f;
            const uint32_t taddr = tmem_base + (uint32_t)(acc * BN) + ((uint32_t)(q * 32) << 16);
            constexpr int CH = BN >= 32 ? 32 : 16;
#pragma unroll 1
            for (int c = 0; c < BN / CH; ++c) {
                uint32_t r[32];
                if (CH == 32) ptx::tmem_ld_32x32b_x32(taddr + (uint32_t)(c * CH), r);
                else tmem_ld_32x32b_x16(taddr + (uint32_t)(c * CH), r);
                ptx::tmem_ld_wait();
                if (o < out) {
                    if (splits > 1) {
                        // partial sums of part p: ws[p][o][0..BN), a contiguous run per thread
                        float4* dst = reinterpret_cast<float4*>(&ws[((int64_t)it.part * out + o) * BN + c * CH]);
#pragma unroll
                        for (int j = 0; j < CH / 4; ++j)
                            __stcg(dst + j, make_float4(__uint_as_float(r[4 * j]), __uint_as_float(r[4 * j + 1]),
                                                        __uint_as_float(r[4 * j + 2]), __uint_as_float(r[4 * j + 3])));
                    } else {
#pragma unroll
                        for (int j = 0; j < CH; ++j) {
                            const int tok = nt * BN + c * CH + j;
                            if (tok < T) Y[(int64_t)tok * out + o] = __float2bfloat16_rn(__uint_as_float(r[j]) + b);
                        }
                    }
                }
            }
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&tail->tmem_empty[acc]));
            if (splits > 1) {
                // Each warp owns 32 output features of the tile in every unit, so the ticket is per
                // warp quarter: no barrier between warps. The warp that draws the last ticket sees
                // the sums of all units (fence before the ticket, fence after it).
                __threadfence();
                __syncwarp();
                int ticket = 0;
                if (lane == 0) ticket = atomicAdd(&counters[mn * 4 + q], 1);
                ticket = __shfl_sync(0xffffffffu, ticket, 0);
                if (ticket == splits - 1) {
                    __threadfence();
                    if (o < out) {
                        // sixteen tokens at a time, four 16-byte loads per unit in flight
                        for (int tok0 = 0; tok0 < BN && tok0 < T; tok0 += 16) {
                            float4 sum[4];
#pragma unroll
                            for (int i = 0; i < 4; ++i) sum[i] = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll 4
                            for (int sidx = 0; sidx < splits; ++sidx) {
                                const float4* src = reinterpret_cast<const float4*>(&ws[((int64_t)sidx * out + o) * BN + tok0]);
                                float4 part[4];
#pragma unroll
                                for (int i = 0; i < 4; ++i) part[i] = __ldcg(src + i);
#pragma unroll
                                for (int i = 0; i < 4; ++i) {
                                    sum[i].x += part[i].x; sum[i].y += part[i].y; sum[i].z += part[i].z; sum[i].w += part[i].w;
                                }
                            }
#pragma unroll
                            for (int i = 0; i < 4; ++i) {
                                const float v[4] = {sum[i].x, sum[i].y, sum[i].z, sum[i].w};
#pragma unroll
                                for (int e = 0; e < 4; ++e) {
                                    const int tok = tok0 + 4 * i + e;
                                    if (tok < T) Y[(int64_t)tok * out + o] = __float2bfloat16_rn(v[e] + b);
                                }
                            }
                        }
                    }
                    __syncwarp();
                    if (lane == 0) counters[mn * 4 + q] = 0;
                }
            }
        }
    }

    ptx::tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc(tmem_base, C::TMEM_COLS);
    }
}

// ------------------------------------------------------------------------------------------
// CTA-pair variant for large token counts
// ------------------------------------------------------------------------------------------
// At 2x the MMA rate the 1-CTA kernel is bound by the L2 -> SM operand traffic (the activation
// tile is 2/3 of each stage). Here a cluster of two CTAs computes a 256 (weight rows) x 224
// (tokens) tile with tcgen05 .cta_group::2: each CTA loads its own 128 weight rows (values +
// metadata) but only half of the activation rows, and the leader's MMAs read both halves. Per
// dense-equivalent FLOP that halves the operand bytes. Barriers: each CTA has its own `empty`
// ring (released by a multicast commit of the leader), the leader's `full` ring counts the
// bytes of both CTAs, accumulator hand-over uses the leader's `tmem_empty` (8 epilogue warps)
// and a multicast `tmem_full`.
constexpr int P2_BN = 224, P2_BNH = P2_BN / 2, P2_STAGES = 4;
constexpr int P2_B_BOX_BYTES = P2_BNH * 128;  // 112 token rows x 64 logical columns
constexpr int P2_STAGE_BYTES = SP_A_BYTES + 2 * P2_B_BOX_BYTES + SP_META_BYTES;  // 47104
constexpr int P2_META_COL0 = 2 * P2_BN;       // 448
constexpr int P2_TMEM_COLS = 512;
constexpr int P2_SMEM_BYTES = P2_STAGES * P2_STAGE_BYTES + 1024 + 256;

// Token-tile width and accumulator count of the one-tile pair kernel. 224 tokens with two
// accumulators (epilogue hidden behind the next tile) is the general case; 256 tokens with a single
// accumulator serves products whose tiles all fit in one wave of pairs, where there is no next tile
// to overlap with and the wider tile means fewer, fuller work units (T = 1024 on a 4096-row
// matrix: 16 x 4 = 64 units for 74 pairs instead of 16 x 5 = 80).
template <int BN, int NACC>
struct PairCfg {
    static constexpr int BNH = BN / 2;
    static constexpr int B_BOX_BYTES = BNH * 128;
    static constexpr int STAGE_BYTES = SP_A_BYTES + 2 * B_BOX_BYTES + SP_META_BYTES;
    static constexpr int STAGES = 4;
    static constexpr int META_COL0 = NACC * BN;
    static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 1024 + 256;
    static_assert(NACC * BN + 4 * STAGES <= 512, "accumulators and metadata must fit the tensor memory");
    static_assert(SMEM_BYTES <= 232448, "stages must fit the shared memory of one CTA");
    static_assert(STAGE_BYTES % 1024 == 0 && B_BOX_BYTES % 1024 == 0, "swizzled operand tiles need 1024-byte alignment");
};

template <int BN, int NACC>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(SP_THREADS, 1)
sparse24_gemm_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                          const __grid_constant__ CUtensorMap tmE, __nv_bfloat16* __restrict__ Y,
                          const __nv_bfloat16* __restrict__ bias, int out, int T, int in, int32_t* status) {
    using C = PairCfg<BN, NACC>;
    constexpr int STAGES = C::STAGES;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = ptx::smem_u32(smem_raw);
    const uint32_t base = (raw_addr + 1023u) & ~1023u;
    uint8_t* base_ptr = smem_raw + (base - raw_addr);
    auto* tail = reinterpret_cast<SpSmemTail<STAGES>*>(base_ptr + STAGES * C::STAGE_BYTES);
    volatile int* abort_flag = &tail->abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t cta = ptx::cluster_ctarank();  // 0 = leader
    const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
    const int tiles_m = (out + 255) / 256, tiles_n = (T + BN - 1) / BN;
    const int total_tiles = tiles_m * tiles_n;
    const int num_kb = (in + SP_BK - 1) / SP_BK;
    const int meta_tiles_m = (out + 127) / 128;  // 128-row metadata tiles per K tile column

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            ptx::mbar_init(ptx::smem_u32(&tail->full[s]), 1);
            ptx::mbar_init(ptx::smem_u32(&tail->empty[s]), 1);
        }
        for (int a = 0; a < 2; ++a) {
            ptx::mbar_init(ptx::smem_u32(&tail->tmem_full[a]), 1);
            ptx::mbar_init(ptx::smem_u32(&tail->tmem_empty[a]), 8);  // 4 epilogue warps of each CTA
        }
        tail->abort_flag = 0;
        ptx::fence_barrier_init();
    }
    if (warp == 1) {
        ptx::tmem_alloc_pair(ptx::smem_u32(&tail->tmem_base), P2_TMEM_COLS);
        ptx::tmem_relinquish_pair();
    }
    if (warp == 0 && lane == 0) {
        ptx::prefetch_tensormap(&tmA);
        ptx::prefetch_tensormap(&tmB);
        ptx::prefetch_tensormap(&tmE);
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::cluster_sync_all();  // barriers of both CTAs are initialised before anything remote happens
    ptx::tc_fence_after();
    const uint32_t tmem_base = tail->tmem_base;

    if (warp == 0) {
        // ---------------- TMA producer (both CTAs) ----------------
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        for (int tile = pair; tile < total_tiles && ok; tile += num_pairs) {
            int mt, nt;
            sp_tile_coords(tile, tiles_m, tiles_n, mt, nt);
            const int m0 = mt * 256 + (int)cta * 128;    // this CTA's weight rows
            const int n0 = nt * BN + (int)cta * C::BNH;  // this CTA's half of the token rows
            for (int kb = 0; kb < num_kb; ++kb) {
                ok = ptx::mbar_wait(ptx::smem_u32(&tail->empty[stage]), phase ^ 1u, abort_flag, status, 21);
                if (!ok) break;
                if (lane == 0) {
                    const uint32_t local_bar = ptx::smem_u32(&tail->full[stage]);
                    const uint32_t leader_bar = ptx::map_to_cta(local_bar, 0);
                    const uint32_t sa = base + stage * C::STAGE_BYTES, sb = sa + SP_A_BYTES;
                    const uint32_t sm = sb + 2 * C::B_BOX_BYTES;
                    if (cta == 0) ptx::mbar_arrive_expect_tx(local_bar, 2 * C::STAGE_BYTES);
                    ptx::tma_load_2d_pair(sa, &tmA, leader_bar, kb * (SP_BK / 2), m0);
                    ptx::tma_load_2d_pair(sb, &tmB, leader_bar, kb * SP_BK, n0);
                    ptx::tma_load_2d_pair(sb + C::B_BOX_BYTES, &tmB, leader_bar, kb * SP_BK + 64, n0);
                    // metadata tile (m0 / 128, kb): 128 rows of 16 bytes
                    ptx::tma_load_2d_pair(sm, &tmE, leader_bar, 0, ((m0 >> 7) * num_kb + kb) * 128);
                }
                __syncwarp();
                if (++stage == STAGES) { stage = 0; phase ^= 1u; }
            }
        }
        if (!ok) for (int i = 0; i < 1000; ++i) __nanosleep(1000);
        (void)meta_tiles_m;
    } else if (warp == 1) {
        // ---------------- MMA issuer (leader CTA only) ----------------
        if (cta == 0) {
            constexpr uint32_t idesc = ptx::make_idesc_bf16(256, BN, 0, 0, 1);
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            int t = 0;
            for (int tile = pair; tile < total_tiles && ok; tile += num_pairs, ++t) {
                // two accumulators alternate; with one, every tile waits for the previous one to be drained
                const int acc = NACC == 2 ? (t & 1) : 0;
                const uint32_t acc_phase = NACC == 2 ? ((uint32_t)(t >> 1) & 1u) : ((uint32_t)t & 1u);
                ok = ptx::mbar_wait(ptx::smem_u32(&tail->tmem_empty[acc]), acc_phase ^ 1u, abort_flag, status, 23);
                if (!ok) break;
                ptx::tc_fence_after();
                const uint32_t tmem_d = tmem_base + (uint32_t)(acc * BN);
                for (int kb = 0; kb < num_kb; ++kb) {
                    ok = ptx::mbar_wait(ptx::smem_u32(&tail->full[stage]), phase, abort_flag, status, 22);
                    if (!ok) break;
                    ptx::tc_fence_after();
                    if (lane == 0) {
                        const uint32_t sa = base + stage * C::STAGE_BYTES, sb = sa + SP_A_BYTES;
                        const uint32_t sm = sb + 2 * C::B_BOX_BYTES;
                        const uint32_t tmem_e = tmem_base + (uint32_t)(C::META_COL0 + 4 * stage);
                        ptx::tmem_cp_128x128b_pair(tmem_e, ptx::make_smem_desc(sm, 16, 128, 0));
#pragma unroll
                        for (int k = 0; k < 4; ++k) {
                            const uint64_t adesc = ptx::make_smem_desc(sa + k * 32, 16, 1024, 2);
                            const uint64_t bdesc = ptx::make_smem_desc(sb + (k >> 1) * C::B_BOX_BYTES + (k & 1) * 64, 16, 1024, 2);
                            ptx::mma_f16_ss_sp_pair(tmem_d, adesc, bdesc, tmem_e + (uint32_t)(k & ~1), idesc | (uint32_t)(k & 1),
                                                    (kb | k) != 0 ? 1u : 0u);
                        }
                        ptx::mma_commit_pair(ptx::smem_u32(&tail->empty[stage]), (uint16_t)3);
                    }
                    __syncwarp();
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
                if (!ok) break;
                if (lane == 0) ptx::mma_commit_pair(ptx::smem_u32(&tail->tmem_full[acc]), (uint16_t)3);
                __syncwarp();
            }
        }
    } else {
        // ---------------- epilogue (both CTAs): 128 weight rows x 224 tokens each ----------------
        const int q = warp & 3;
        const uint32_t leader_empty0 = ptx::map_to_cta(ptx::smem_u32(&tail->tmem_empty[0]), 0);
        const uint32_t leader_empty1 = ptx::map_to_cta(ptx::smem_u32(&tail->tmem_empty[1]), 0);
        bool ok = true;
        int t = 0;
        for (int tile = pair; tile < total_tiles && ok; tile += num_pairs, ++t) {
            int mt, nt;
            sp_tile_coords(tile, tiles_m, tiles_n, mt, nt);
            const int acc = NACC == 2 ? (t & 1) : 0;
            const uint32_t acc_phase = NACC == 2 ? ((uint32_t)(t >> 1) & 1u) : ((uint32_t)t & 1u);
            ok = ptx::mbar_wait(ptx::smem_u32(&tail->tmem_full[acc]), acc_phase, abort_flag, status, 24);
            if (!ok) break;
            ptx::tc_fence_after();
            const int o = mt * 256 + (int)cta * 128 + q * 32 + lane;
            const float b = (bias != nullptr && o < out) ? __bfloat162float(bias[o]) : 0.0f;
            const uint32_t taddr = tmem_base + (uint32_t)(acc * BN) + ((uint32_t)(q * 32) << 16);
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                uint32_t r[32];
                ptx::tmem_ld_32x32b_x32(taddr + (uint32_t)(c * 32), r);
                ptx::tmem_ld_wait();
                if (o < out) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const int tok = nt * BN + c * 32 + j;
                        if (tok < T) Y[(int64_t)tok * out + o] = __float2bfloat16_rn(__uint_as_float(r[j]) + b);
                    }
                }
            }
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive_cluster(acc ? leader_empty1 : leader_empty0);
        }
    }

    // ---------------- teardown: nobody leaves while the peer may still touch this CTA ----------------
    ptx::tc_fence_before();
    __syncthreads();
    ptx::cluster_sync_all();
    if (warp == 1) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc_pair(tmem_base, P2_TMEM_COLS);
    }
}

// ------------------------------------------------------------------------------------------
// CTA pair, two weight tiles per CTA: a pair computes 512 weight rows x 224 tokens. Both sparse MMAs
// of a K step (rows [0,256) and [256,512) of the pair tile, 128 of each in every CTA) read the SAME
// staged activation tile, so the bytes a CTA pulls from L2 per FLOP drop from 46 KiB to 32 KiB per
// 7.3 MFLOP: the one-tile pair kernel stalls on operand delivery (about 100 B per clock and SM
// wanted at the sparse rate, 70-75 delivered), this one asks for about 70. Price: the two
// accumulators fill the tensor memory (2 x 224 + metadata columns), so they are not double
// buffered and the epilogue of a tile is not hidden behind the next tile's MMAs; eight epilogue
// warps per CTA (two per TMEM lane quarter, one per weight tile) keep it short.
// ------------------------------------------------------------------------------------------
constexpr int Q_STAGES = 3;
constexpr int Q_THREADS = 320;  // TMA warp, MMA warp, eight epilogue warps
constexpr int Q_STAGE_BYTES = 2 * SP_A_BYTES + 2 * P2_B_BOX_BYTES + 2 * SP_META_BYTES;  // 65536
constexpr int Q_META_COL0 = 2 * P2_BN;  // 448: after the two accumulators
constexpr int Q_EPI_ROW_BYTES = 64 + 16;                      // 32 bf16 features of one token, padded against bank conflicts
constexpr int Q_EPI_WARP_BYTES = 32 * Q_EPI_ROW_BYTES;        // one turn buffer per epilogue warp
constexpr int Q_SMEM_BYTES = Q_STAGES * Q_STAGE_BYTES + 1024 + 256 + 8 * Q_EPI_WARP_BYTES;

__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(Q_THREADS, 1)
sparse24_gemm_pair2_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                           const __grid_constant__ CUtensorMap tmE, __nv_bfloat16* __restrict__ Y,
                           const __nv_bfloat16* __restrict__ bias, int out, int T, int in, int32_t* status) {
    constexpr int STAGES = Q_STAGES;
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = ptx::smem_u32(smem_raw);
    const uint32_t base = (raw_addr + 1023u) & ~1023u;
    uint8_t* base_ptr = smem_raw + (base - raw_addr);
    auto* tail = reinterpret_cast<SpSmemTail<STAGES>*>(base_ptr + STAGES * Q_STAGE_BYTES);
    volatile int* abort_flag = &tail->abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t cta = ptx::cluster_ctarank();
    const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
    const int tiles_m = (out + 511) / 512, tiles_n = (T + P2_BN - 1) / P2_BN;
    const int total_tiles = tiles_m * tiles_n;
    const int num_kb = (in + SP_BK - 1) / SP_BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            ptx::mbar_init(ptx::smem_u32(&tail->full[s]), 1);
            ptx::mbar_init(ptx::smem_u32(&tail->empty[s]), 1);
        }
        ptx::mbar_init(ptx::smem_u32(&tail->tmem_full[0]), 1);
        ptx::mbar_init(ptx::smem_u32(&tail->tmem_empty[0]), 16);  // 8 epilogue warps of each CTA
        tail->abort_flag = 0;
        ptx::fence_barrier_init();
    }
    if (warp == 1) {
        ptx::tmem_alloc_pair(ptx::smem_u32(&tail->tmem_base), P2_TMEM_COLS);
        ptx::tmem_relinquish_pair();
    }
    if (warp == 0 && lane == 0) {
        ptx::prefetch_tensormap(&tmA);
        ptx::prefetch_tensormap(&tmB);
        ptx::prefetch_tensormap(&tmE);
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::cluster_sync_all();
    ptx::tc_fence_after();
    const uint32_t tmem_base = tail->tmem_base;

    if (warp == 0) {
        // ---------------- TMA producer (both CTAs) ----------------
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        for (int tile = pair; tile < total_tiles && ok; tile += num_pairs) {
            int mt, nt;
            sp_tile_coords(tile, tiles_m, tiles_n, mt, nt);
            const int n0 = nt * P2_BN + (int)cta * P2_BNH;
            for (int kb = 0; kb < num_kb; ++kb) {
                ok = ptx::mbar_wait(ptx::smem_u32(&tail->empty[stage]), phase ^ 1u, abort_flag, status, 41);
                if (!ok) break;
                if (lane == 0) {
                    const uint32_t local_bar = ptx::smem_u32(&tail->full[stage]);
                    const uint32_t leader_bar = ptx::map_to_cta(local_bar, 0);
                    const uint32_t sa = base + stage * Q_STAGE_BYTES, sb = sa + 2 * SP_A_BYTES;
                    const uint32_t sm = sb + 2 * P2_B_BOX_BYTES;
                    if (cta == 0) ptx::mbar_arrive_expect_tx(local_bar, 2 * Q_STAGE_BYTES);
#pragma unroll
                    for (int u = 0; u < 2; ++u) {
                        const int m0 = mt * 512 + u * 256 + (int)cta * 128;  // this CTA's rows of weight tile u
                        ptx::tma_load_2d_pair(sa + u * SP_A_BYTES, &tmA, leader_bar, kb * (SP_BK / 2), m0);
                        ptx::tma_load_2d_pair(sm + u * SP_META_BYTES, &tmE, leader_bar, 0, ((m0 >> 7) * num_kb + kb) * 128);
                    }
                    ptx::tma_load_2d_pair(sb, &tmB, leader_bar, kb * SP_BK, n0);
                    ptx::tma_load_2d_pair(sb + P2_B_BOX_BYTES, &tmB, leader_bar, kb * SP_BK + 64, n0);
                }
                __syncwarp();
                if (++stage == STAGES) { stage = 0; phase ^= 1u; }
            }
        }
        if (!ok) for (int i = 0; i < 1000; ++i) __nanosleep(1000);
    } else if (warp == 1) {
        // ---------------- MMA issuer (leader CTA only) ----------------
        if (cta == 0) {
            constexpr uint32_t idesc = ptx::make_idesc_bf16(256, P2_BN, 0, 0, 1);
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            int t = 0;
            for (int tile = pair; tile < total_tiles && ok; tile += num_pairs, ++t) {
                // both accumulators are free once the sixteen epilogue warps have drained the last tile
                ok = ptx::mbar_wait(ptx::smem_u32(&tail->tmem_empty[0]), ((uint32_t)t & 1u) ^ 1u, abort_flag, status, 43);
                if (!ok) break;
                ptx::tc_fence_after();
                for (int kb = 0; kb < num_kb; ++kb) {
                    ok = ptx::mbar_wait(ptx::smem_u32(&tail->full[stage]), phase, abort_flag, status, 42);
                    if (!ok) break;
                    ptx::tc_fence_after();
                    if (lane == 0) {
                        const uint32_t sa = base + stage * Q_STAGE_BYTES, sb = sa + 2 * SP_A_BYTES;
                        const uint32_t sm = sb + 2 * P2_B_BOX_BYTES;
#pragma unroll
                        for (int u = 0; u < 2; ++u) {
                            const uint32_t tmem_e = tmem_base + (uint32_t)(Q_META_COL0 + 4 * (stage * 2 + u));
                            ptx::tmem_cp_128x128b_pair(tmem_e, ptx::make_smem_desc(sm + u * SP_META_BYTES, 16, 128, 0));
                        }
#pragma unroll
                        for (int u = 0; u < 2; ++u) {
                            const uint32_t tmem_d = tmem_base + (uint32_t)(u * P2_BN);
                            const uint32_t tmem_e = tmem_base + (uint32_t)(Q_META_COL0 + 4 * (stage * 2 + u));
#pragma unroll
                            for (int k = 0; k < 4; ++k) {
                                const uint64_t adesc = ptx::make_smem_desc(sa + u * SP_A_BYTES + k * 32, 16, 1024, 2);
                                const uint64_t bdesc = ptx::make_smem_desc(sb + (k >> 1) * P2_B_BOX_BYTES + (k & 1) * 64, 16, 1024, 2);
                                ptx::mma_f16_ss_sp_pair(tmem_d, adesc, bdesc, tmem_e + (uint32_t)(k & ~1), idesc | (uint32_t)(k & 1),
                                                        (kb | k) != 0 ? 1u : 0u);
                            }
                        }
                        ptx::mma_commit_pair(ptx::smem_u32(&tail->empty[stage]), (uint16_t)3);
                    }
                    __syncwarp();
                    if (++stage == STAGES) { stage = 0; phase ^= 1u; }
                }
                if (!ok) break;
                if (lane == 0) ptx::mma_commit_pair(ptx::smem_u32(&tail->tmem_full[0]), (uint16_t)3);
                __syncwarp();
            }
        }
    } else {
        // ---------------- epilogue (both CTAs): warp (u, q) drains 32 rows x 224 tokens of weight tile u ----------------
        // The two accumulators fill the tensor memory, so the next tile's MMAs cannot start before
        // both are read. The read is therefore all that stays exposed: every warp pulls its 32 x 224
        // block into registers (rounded to bf16 with the bias added, two tokens per register: 112
        // registers), hands the accumulators back, and only then turns 32 x 32 chunks through a
        // private shared-memory buffer into token-major 16-byte stores, while the MMAs of the next
        // tile already run.
        const int q = warp & 3, u = (warp - 2) >> 2;
        const uint32_t leader_empty = ptx::map_to_cta(ptx::smem_u32(&tail->tmem_empty[0]), 0);
        uint8_t* ebuf = base_ptr + STAGES * Q_STAGE_BYTES + 256 + (warp - 2) * Q_EPI_WARP_BYTES;
        const bool vec_ok = (out & 7) == 0;
        bool ok = true;
        int t = 0;
        for (int tile = pair; tile < total_tiles && ok; tile += num_pairs, ++t) {
            int mt, nt;
            sp_tile_coords(tile, tiles_m, tiles_n, mt, nt);
            ok = ptx::mbar_wait(ptx::smem_u32(&tail->tmem_full[0]), (uint32_t)t & 1u, abort_flag, status, 44);
            if (!ok) break;
            ptx::tc_fence_after();
            const int o_base = mt * 512 + u * 256 + (int)cta * 128 + q * 32;
            const int o = o_base + lane;
            const float b = (bias != nullptr && o < out) ? __bfloat162float(bias[o]) : 0.0f;
            const uint32_t taddr = tmem_base + (uint32_t)(u * P2_BN) + ((uint32_t)(q * 32) << 16);
            constexpr int CHUNKS = P2_BN / 32;
            uint32_t pk[CHUNKS * 16];
#pragma unroll
            for (int c = 0; c < CHUNKS; ++c) {
                uint32_t r[32];
                ptx::tmem_ld_32x32b_x32(taddr + (uint32_t)(c * 32), r);
                ptx::tmem_ld_wait();
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const __nv_bfloat162 v = __floats2bfloat162_rn(__uint_as_float(r[2 * j]) + b,
                                                                   __uint_as_float(r[2 * j + 1]) + b);
                    pk[c * 16 + j] = *reinterpret_cast<const uint32_t*>(&v);
                }
            }
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive_cluster(leader_empty);
#pragma unroll
            for (int c = 0; c < CHUNKS; ++c) {
                // feature-major registers -> token-major rows of 32 features (64 bytes, padded to 80)
#pragma unroll
                for (int j = 0; j < 16; ++j) {
                    const uint32_t v = pk[c * 16 + j];
                    *reinterpret_cast<uint16_t*>(ebuf + (2 * j) * Q_EPI_ROW_BYTES + lane * 2) = (uint16_t)(v & 0xffffu);
                    *reinterpret_cast<uint16_t*>(ebuf + (2 * j + 1) * Q_EPI_ROW_BYTES + lane * 2) = (uint16_t)(v >> 16);
                }
                __syncwarp();
                const int tok = nt * P2_BN + c * 32 + lane;
                if (tok < T) {
                    __nv_bfloat16* yrow = Y + (int64_t)tok * out + o_base;
                    if (vec_ok) {
#pragma unroll
                        for (int i = 0; i < 4; ++i)
                            if (o_base + 8 * i < out)
                                *reinterpret_cast<uint4*>(yrow + 8 * i) =
                                    *reinterpret_cast<const uint4*>(ebuf + lane * Q_EPI_ROW_BYTES + i * 16);
                    } else {
                        for (int i = 0; i < 32 && o_base + i < out; ++i)
                            yrow[i] = *reinterpret_cast<const __nv_bfloat16*>(ebuf + lane * Q_EPI_ROW_BYTES + i * 2);
                    }
                }
                __syncwarp();  // the buffer is rewritten by the next chunk
            }
        }
    }

    ptx::tc_fence_before();
    __syncthreads();
    ptx::cluster_sync_all();
    if (warp == 1) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc_pair(tmem_base, P2_TMEM_COLS);
    }
}

int make_meta_tensor_map(CUtensorMap* map, const void* ptr, int64_t rows, int box_rows);

static int launch_sparse_pair(const void* x, const void* values, const uint8_t* meta_tc, const void* bias, void* y,
                              int64_t T, int64_t in, int64_t out, int32_t* status, cudaStream_t st) {
    CUtensorMap tmA, tmB, tmE;
    int rc = make_bf16_tensor_map(&tmA, values, in / 2, out, in / 2, SP_BM);
    if (rc) return rc;
    const int64_t max_pairs = sm_count() / 2;
    // one wave of pairs covers the product with 256-token tiles: single accumulator, wider tile
    const int64_t tiles_wide = ((out + 255) / 256) * ((T + 255) / 256);
    const int64_t tiles_std = ((out + 255) / 256) * ((T + P2_BN - 1) / P2_BN);
    const bool wide = tiles_wide <= max_pairs && tiles_std > tiles_wide;
    rc = make_bf16_tensor_map(&tmB, x, in, T, in, wide ? 128 : P2_BNH);
    if (rc) return rc;
    const int64_t meta_rows = sf_sparse24_meta_tc_bytes(out, in) / 16;
    rc = make_meta_tensor_map(&tmE, meta_tc, meta_rows, 128);
    if (rc) return rc;
    static thread_local int configured_dev = -1;
    int dev = 0;
    SF_CHECK_CUDA(cudaGetDevice(&dev));
    if (configured_dev != dev) {
        SF_CHECK_CUDA(cudaFuncSetAttribute(sparse24_gemm_pair_kernel<P2_BN, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           PairCfg<P2_BN, 2>::SMEM_BYTES));
        SF_CHECK_CUDA(cudaFuncSetAttribute(sparse24_gemm_pair_kernel<256, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                           PairCfg<256, 1>::SMEM_BYTES));
        SF_CHECK_CUDA(cudaFuncSetAttribute(sparse24_gemm_pair2_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, Q_SMEM_BYTES));
        configured_dev = dev;
    }
    if (wide) {
        sparse24_gemm_pair_kernel<256, 1><<<2 * (int)tiles_wide, SP_THREADS, PairCfg<256, 1>::SMEM_BYTES, st>>>(
            tmA, tmB, tmE, (__nv_bfloat16*)y, (const __nv_bfloat16*)bias, (int)out, (int)T, (int)in, status);
        SF_CHECK_CUDA(cudaGetLastError());
        return SF_OK;
    }
    // Two weight tiles per CTA when the matrix has at least two 256-row tiles and there are enough
    // work units for the pairs (measured at T = 8192, interleaved runs: K = 11008 301 us against
    // 335 us for the one-tile kernel, K = 4096 123 against 127 us, the 11008-row matrix 341 against
    // 342 us). SF_SPARSE24_ONE_TILE=1 forces the one-tile kernel for A/B runs.
    const char* e1 = getenv("SF_SPARSE24_ONE_TILE");
    const bool one_tile_only = e1 && e1[0] == '1';
    const int64_t tiles2 = ((out + 511) / 512) * ((T + P2_BN - 1) / P2_BN);
    // waves of pairs each variant needs; a two-tile unit costs about 1.9 one-tile units
    const int64_t tiles1 = ((out + 255) / 256) * ((T + P2_BN - 1) / P2_BN);
    const double cost1 = (double)((tiles1 + max_pairs - 1) / max_pairs);
    const double cost2 = 1.9 * (double)((tiles2 + max_pairs - 1) / max_pairs);
    if (!one_tile_only && out >= 512 && tiles2 >= max_pairs && cost2 <= cost1) {
        const int pairs2 = (int)(tiles2 < max_pairs ? tiles2 : max_pairs);
        sparse24_gemm_pair2_kernel<<<2 * pairs2, Q_THREADS, Q_SMEM_BYTES, st>>>(tmA, tmB, tmE, (__nv_bfloat16*)y,
                                                                                (const __nv_bfloat16*)bias, (int)out, (int)T,
                                                                                (int)in, status);
        SF_CHECK_CUDA(cudaGetLastError());
        return SF_OK;
    }
    const int64_t tiles = ((out + 255) / 256) * ((T + P2_BN - 1) / P2_BN);
    const int pairs = (int)(tiles < max_pairs ? tiles : max_pairs);
    sparse24_gemm_pair_kernel<P2_BN, 2><<<2 * pairs, SP_THREADS, P2_SMEM_BYTES, st>>>(tmA, tmB, tmE, (__nv_bfloat16*)y,
                                                                            (const __nv_bfloat16*)bias, (int)out, (int)T,
                                                                            (int)in, status);
    SF_CHECK_CUDA(cudaGetLastError());
    return SF_OK;
}

constexpr int SP_MAX_SPLITS = 8;
// The arrival tickets sit at the head of the workspace in a region of fixed size, so that a
// workspace reused for another matrix never has partial sums where tickets are expected.
constexpr int64_t SP_TICKET_BYTES = 64 * 1024;
static int64_t sp_ticket_bytes(int64_t) { return SP_TICKET_BYTES; }

// K blocks per CTA for a product with fewer tiles than SMs and at most 128 activation rows: the K blocks of
// all tiles are dealt out in equal runs, one per SM, at least four blocks each (a run shorter than that
// does not cover the latency of its first loads), and long enough that no tile is cut into more than
// SP_MAX_SPLITS parts. 0 = whole tiles. Measured on 4096-row matrices with uniform K ranges per tile: 12.7 ->
// 8.6 us at 16 rows, K = 4096; 38 -> 13 us at 16 rows and 44 -> 35 us at 128 rows, K = 11008; beyond 32 rows
// with a short K the final sum over the partial results costs more than it saves (17.5 -> 31 us at 128 rows).
static int choose_range_kb(int64_t tiles, int64_t num_kb, int64_t T) {
    if (T > 32 && num_kb < 64) return 0;
    const int64_t sms = sm_count();
    // a matrix whose tiles already fill more than half of the SMs streams its weights at over 3 TB/s as it is;
    // measured at 16 rows on the 11008-row matrix (86 tiles): 15.3 us whole tiles, 16.2 us in balanced runs
    // (the round trip of the partial sums costs more than the idle SMs), against 18.7 -> 15.9 us on the
    // 4096 x 11008 matrix (32 tiles)
    if (2 * tiles > sms) return 0;
    const int64_t total = tiles * num_kb;
    int64_t ctas = total / 4 < sms ? total / 4 : sms;
    if (ctas <= tiles) return 0;
    int64_t L = (total + ctas - 1) / ctas;
    if (T > 32) {
        // the partial sums grow with the rows: equal K ranges per tile, as few as fill the SMs once (measured at
        // 128 rows on the 4096 x 11008 matrix: 47 us with four ranges per tile, 64 us in balanced runs of 19 blocks)
        int64_t per_tile = sms / tiles;
        if (per_tile > SP_MAX_SPLITS) per_tile = SP_MAX_SPLITS;
        if (per_tile > num_kb / 4) per_tile = num_kb / 4;
        if (per_tile < 2) return 0;
        L = (num_kb + per_tile - 1) / per_tile;
    }
    const int64_t min_l = (num_kb + SP_MAX_SPLITS - 2) / (SP_MAX_SPLITS - 1);  // at most SP_MAX_SPLITS parts per tile
    if (L < min_l) L = min_l;
    return L >= num_kb ? 0 : (int)L;
}

template <int BN>
static int launch_sparse(const void* x, const void* values, const uint8_t* meta_tc, const void* bias, void* y,
                         int64_t T, int64_t in, int64_t out, int32_t* status, cudaStream_t st, int range_kb = 0,
                         float* ws = nullptr, int* counters = nullptr) {
    using C = SpCfg<BN>;
    CUtensorMap tmA, tmB;
    int rc = make_bf16_tensor_map(&tmA, values, in / 2, out, in / 2, SP_BM);
    if (rc) return rc;
    rc = make_bf16_tensor_map(&tmB, x, in, T, in, BN);
    if (rc) return rc;
    auto kern = sparse24_gemm_kernel<BN>;
    static thread_local int configured_dev = -1;
    int dev = 0;
    SF_CHECK_CUDA(cudaGetDevice(&dev));
    if (configured_dev != dev) {
        SF_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES));
        configured_dev = dev;
    }
    const int64_t tiles = ((out + SP_BM - 1) / SP_BM) * ((T + BN - 1) / BN);
    int grid = (int)(tiles < sm_count() ? tiles : sm_count());
    if (range_kb > 0) {
        const int64_t total_kb = tiles * ((in + SP_BK - 1) / SP_BK);
        grid = (int)((total_kb + range_kb - 1) / range_kb);  // one run of range_kb K blocks per CTA
    }
    kern<<<grid, SP_THREADS, C::SMEM_BYTES, st>>>(tmA, tmB, meta_tc, (__nv_bfloat16*)y, (const __nv_bfloat16*)bias,
                                                  (int)out, (int)T, (int)in, status, range_kb, ws, counters);
    SF_CHECK_CUDA(cudaGetLastError());
    return SF_OK;
}

}  // namespace sf

using namespace sf;

extern "C" {

int sf_sparse24_compress(const void* W, const float* soft, void* values, uint8_t* meta, int64_t out, int64_t in,
                         void* stream) {
    SF_CHECK_ARG(W && soft && values && meta, "sf_sparse24_compress: W, soft, values, meta must be non-null");
    SF_CHECK_ARG(out > 0 && in > 0 && in % 8 == 0, "sf_sparse24_compress: in=%lld must be a positive multiple of 8", (long long)in);
    if (!(aligned16(W) && aligned16(soft)) || (reinterpret_cast<uintptr_t>(values) & 7u))
        return fail(SF_ERR_ALIGNMENT, "sf_sparse24_compress: W, soft must be 16-byte and values 8-byte aligned");
    const int64_t chunks = out * in / 8;
    sparse24_compress_kernel<<<grid_for_e(chunks), kThreadsE, 0, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)W, soft, (__nv_bfloat16*)values, meta, chunks);
    SF_CHECK_CUDA(cudaGetLastError());
    return SF_OK;
}

int sf_sparse24_decompress(const void* values, const uint8_t* meta, void* dense, int64_t out, int64_t in, void* stream) {
    SF_CHECK_ARG(values && meta && dense, "sf_sparse24_decompress: values, meta, dense must be non-null");
    SF_CHECK_ARG(out > 0 && in > 0 && in % 8 == 0, "sf_sparse24_decompress: in=%lld must be a positive multiple of 8", (long long)in);
    if (!aligned16(dense) || (reinterpret_cast<uintptr_t>(values) & 7u))
        return fail(SF_ERR_ALIGNMENT, "sf_sparse24_decompress: dense must be 16-byte and values 8-byte aligned");
    const int64_t chunks = out * in / 8;
    sparse24_decompress_kernel<<<grid_for_e(chunks), kThreadsE, 0, (cudaStream_t)stream>>>(
        (const __nv_bfloat16*)values, meta, (__nv_bfloat16*)dense, chunks);
    SF_CHECK_CUDA(cudaGetLastError());
    return SF_OK;
}

int64_t sf_sparse24_meta_tc_bytes(int64_t out, int64_t in) {
    if (out <= 0 || in <= 0) return 0;
    return ((out + 127) / 128) * ((in + 127) / 128) * (int64_t)SP_META_BYTES;
}

int sf_sparse24_pack_meta(const uint8_t* meta, uint8_t* meta_tc, int64_t out, int64_t in, void* stream) {
    SF_CHECK_ARG(meta && meta_tc, "sf_sparse24_pack_meta: meta and meta_tc must be non-null");
    SF_CHECK_ARG(out > 0 && in > 0 && in % 8 == 0, "sf_sparse24_pack_meta: in=%lld must be a positive multiple of 8", (long long)in);
    if (!aligned16(meta_tc)) return fail(SF_ERR_ALIGNMENT, "sf_sparse24_pack_meta: meta_tc must be 16-byte aligned");
    const int64_t k_tiles = (in + 127) / 128;
    const int64_t units = sf_sparse24_meta_tc_bytes(out, in) / 2;
    sparse24_pack_meta_kernel<<<grid_for_e(units), kThreadsE, 0, (cudaStream_t)stream>>>(
        meta, (uint16_t*)meta_tc, out, in, k_tiles, units);
    SF_CHECK_CUDA(cudaGetLastError());
    return SF_OK;
}

int64_t sf_sparse24_splitk_workspace_bytes(int64_t T, int64_t out) {
    if (T <= 0 || out <= 0 || T > 128) return 0;
    // the tickets, then fp32 partial sums [splits][out][token tile of up to 128]
    return sp_ticket_bytes(out) + (int64_t)SP_MAX_SPLITS * out * 128 * (int64_t)sizeof(float);
}

static int sparse24_gemm_impl(const void* x, const void* values, const uint8_t* meta_tc, const void* bias, void* y,
                              int64_t T, int64_t in, int64_t out, void* workspace, int64_t workspace_bytes, int splits,
                              int32_t* status, void* stream);

int sf_sparse24_gemm(const void* x, const void* values, const uint8_t* meta_tc, const void* bias, void* y, int64_t T,
                     int64_t in, int64_t out, int32_t* status, void* stream) {
    return sparse24_gemm_impl(x, values, meta_tc, bias, y, T, in, out, nullptr, 0, 1, status, stream);
}

int sf_sparse24_gemm_splitk(const void* x, const void* values, const uint8_t* meta_tc, const void* bias, void* y,
                            int64_t T, int64_t in, int64_t out, void* workspace, int64_t workspace_bytes, int splits,
                            int32_t* status, void* stream) {
    SF_CHECK_ARG(splits >= 0 && splits <= SP_MAX_SPLITS, "sf_sparse24_gemm_splitk: splits must be 0 (choose) .. %d", SP_MAX_SPLITS);
    if (T <= 128) {
        SF_CHECK_ARG(((out + SP_BM - 1) / SP_BM) * 16 <= SP_TICKET_BYTES, "sf_sparse24_gemm_splitk: out=%lld has more tiles than tickets", (long long)out);
        SF_CHECK_ARG(workspace != nullptr && aligned16(workspace), "sf_sparse24_gemm_splitk: workspace must be non-null and 16-byte aligned");
        SF_CHECK_ARG(workspace_bytes >= sf_sparse24_splitk_workspace_bytes(T, out),
                     "sf_sparse24_gemm_splitk: workspace of %lld bytes, %lld needed", (long long)workspace_bytes,
                     (long long)sf_sparse24_splitk_workspace_bytes(T, out));
    }
    return sparse24_gemm_impl(x, values, meta_tc, bias, y, T, in, out, workspace, workspace_bytes, splits, status, stream);
}

static int sparse24_gemm_impl(const void* x, const void* values, const uint8_t* meta_tc, const void* bias, void* y,
                              int64_t T, int64_t in, int64_t out, void* workspace, int64_t workspace_bytes, int splits,
                              int32_t* status, void* stream) {
    (void)workspace_bytes;
    SF_CHECK_ARG(x && values && meta_tc && y, "sf_sparse24_gemm: x, values, meta_tc, y must be non-null");
    SF_CHECK_ARG(T > 0 && in > 0 && out > 0, "sf_sparse24_gemm: T, in, out must be positive");
    if (in % 16 != 0)
        return fail(SF_ERR_UNSUPPORTED, "sf_sparse24_gemm: in=%lld must be a multiple of 16 (16-byte rows of compressed values)", (long long)in);
    if (T > 0x7fffffff || in > 0x7fffffff || out > 0x7fffffff)
        return fail(SF_ERR_UNSUPPORTED, "sf_sparse24_gemm: dimension beyond 2^31-1");
    if (!(aligned16(x) && aligned16(values) && aligned16(meta_tc)))
        return fail(SF_ERR_ALIGNMENT, "sf_sparse24_gemm: x, values, meta_tc must be 16-byte aligned");
    cudaStream_t st = (cudaStream_t)stream;
    if (T <= 128) {
        const int64_t tiles_m = (out + SP_BM - 1) / SP_BM, num_kb = (in + SP_BK - 1) / SP_BK;
        // splits = 0: runs of K blocks balanced over the SMs; splits = N > 1: N equal K ranges per tile (the same
        // machinery with a run length of ceil(num_kb / N)); splits = 1 or no workspace: whole tiles
        int L = 0;
        if (workspace != nullptr) {
            if (splits == 0) L = choose_range_kb(tiles_m, num_kb, T);
            else if (splits > 1) {
                int64_t S = splits < num_kb ? splits : num_kb;
                const int64_t min_l = (num_kb + SP_MAX_SPLITS - 2) / (SP_MAX_SPLITS - 1);
                L = (int)((num_kb + S - 1) / S);
                if (L < min_l) L = (int)min_l;
                if (L >= num_kb) L = 0;
            }
        }
        int* cnt = L > 0 ? (int*)workspace : nullptr;
        float* ws = L > 0 ? (float*)((char*)workspace + sp_ticket_bytes(out)) : nullptr;
        if (T <= 16) return launch_sparse<16>(x, values, meta_tc, bias, y, T, in, out, status, st, L, ws, cnt);
        if (T <= 32) return launch_sparse<32>(x, values, meta_tc, bias, y, T, in, out, status, st, L, ws, cnt);
        if (T <= 64) return launch_sparse<64>(x, values, meta_tc, bias, y, T, in, out, status, st, L, ws, cnt);
        return launch_sparse<128>(x, values, meta_tc, bias, y, T, in, out, status, st, L, ws, cnt);
    }
    // Pick the tiling that wastes fewer tile slots in its last wave; a CTA-pair tile does the same
    // work with about 1.3x less operand traffic, so it wins unless its wave fill is much worse.
    const int64_t sms = sm_count();
    // a product that 256-row x 256-token pair tiles cover in one wave goes to the single-accumulator
    // pair kernel (launch_sparse_pair picks it)
    if (out >= 256 && ((out + 255) / 256) * ((T + 255) / 256) <= sms / 2 &&
        ((out + 255) / 256) * ((T + P2_BN - 1) / P2_BN) > ((out + 255) / 256) * ((T + 255) / 256))
        return launch_sparse_pair(x, values, meta_tc, bias, y, T, in, out, status, st);
    const int64_t t1 = ((out + SP_BM - 1) / SP_BM) * ((T + 127) / 128), s1 = sms;
    const int64_t t2 = ((out + 255) / 256) * ((T + P2_BN - 1) / P2_BN), s2 = sms / 2;
    const double fill1 = (double)t1 / (double)(((t1 + s1 - 1) / s1) * s1);
    const double fill2 = (double)t2 / (double)(((t2 + s2 - 1) / s2) * s2);
    if (fill1 > 1.3 * fill2) return launch_sparse<128>(x, values, meta_tc, bias, y, T, in, out, status, st);
    return launch_sparse_pair(x, values, meta_tc, bias, y, T, in, out, status, st);
}

}  // extern "C"
