// Masked dense GEMMs of SparseLinear on the 5th-generation tensor cores.
//
// One persistent, warp-specialised kernel computes D[M,N] = A[M,K] . B[N,K]^T in bf16 with
// fp32 accumulation in tensor memory (TMEM). Each operand is either K-major (K contiguous
// in memory) or MN-major (the M / N index contiguous), selected by template parameters, so
// the three products of the layer run without any transposed copy:
//   forward : y  = x  . wm^T   A = x  [T,in]   K-major,   B = wm [out,in]  K-major
//   dgrad   : dx = dy . wm     A = dy [T,out]  K-major,   B = wm [out,in]  MN-major (N = in)
//   wgrad   : dw = dy^T . x    A = dy [T,out]  MN-major,  B = x  [T,in]    MN-major
//
// CTA = 6 warps: warp 0 issues TMA loads (128-byte swizzled tiles into a 4-stage ring),
// warp 1 issues tcgen05.mma (128 x 256 x 16 per instruction, four per 64-deep stage) and
// owns the TMEM allocation (2 accumulators x 256 columns), warps 2-5 drain an accumulator
// with tcgen05.ld, convert to bf16 and store, while the MMA warp already fills the other
// accumulator. Tiles are handed out round-robin to min(#tiles, #SMs) CTAs.
//
// Every mbarrier wait is bounded; a wait that runs out sets status[0] and the CTA leaves
// through the common teardown (TMEM is always released).
#include <cuda.h>

#include <cstdlib>
#include <mutex>
#include <unordered_map>

#include "common.cuh"
#include "ptx_sm100.cuh"

namespace sf {

constexpr int BM = 128, BN = 256, BK = 64, STAGES = 4, UMMA_K = 16;
constexpr int A_STAGE_BYTES = BM * BK * 2;  // 16 KiB
constexpr int B_STAGE_BYTES = BN * BK * 2;  // 32 KiB
constexpr int STAGE_BYTES = A_STAGE_BYTES + B_STAGE_BYTES;
constexpr int MN_BOX_BYTES = 64 * BK * 2;  // one 64(MN) x 64(K) box of an MN-major operand
constexpr int GEMM_THREADS = 192;
constexpr int TMEM_COLS = 512;
constexpr int GEMM_SMEM_BYTES = STAGES * STAGE_BYTES + 1024 /* alignment slack */ + 256 /* barriers */;

enum { WAIT_PRODUCER = 1, WAIT_MMA_FULL = 2, WAIT_MMA_TMEM = 3, WAIT_EPILOGUE = 4 };

// Tile order: groups of RASTER_GROUP_M tile rows, walked column by column inside a group, so the
// ~148 tiles in flight cover a near-square patch of the output and share operand panels in L2.
constexpr int RASTER_GROUP_M = 16;
__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int& tm, int& tn) {
    const int per_group = RASTER_GROUP_M * tiles_n;
    const int g = tile / per_group;
    const int first_m = g * RASTER_GROUP_M;
    const int gm = min(RASTER_GROUP_M, tiles_m - first_m);
    const int r = tile - g * per_group;
    tm = first_m + r % gm;
    tn = r / gm;
}

// 32 consecutive fp32 accumulators of one output row -> bf16, scaled, biased, stored as four
// 16-byte vectors (columns beyond N are dropped; N is a multiple of 8).
__device__ __forceinline__ void store_row_chunk(const uint32_t (&r)[32], __nv_bfloat16* dst, int col0, int N, float alpha,
                                                const __nv_bfloat16* __restrict__ bias) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int col = col0 + j * 8;
        if (col < N) {
            uint32_t pk[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                float v0 = __uint_as_float(r[j * 8 + 2 * i]) * alpha;
                float v1 = __uint_as_float(r[j * 8 + 2 * i + 1]) * alpha;
                if (bias != nullptr) {
                    v0 += __bfloat162float(bias[col + 2 * i]);
                    v1 += __bfloat162float(bias[col + 2 * i + 1]);
                }
                __nv_bfloat162 h = __floats2bfloat162_rn(v0, v1);
                pk[i] = *reinterpret_cast<uint32_t*>(&h);
            }
            *reinterpret_cast<uint4*>(dst + j * 8) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
        }
    }
}

// The same conversion kept in registers, so that one accumulator chunk can be stored to several
// destinations (its own memory and peers' memory over NVLink).
__device__ __forceinline__ void pack_row_chunk(const uint32_t (&r)[32], int col0, float alpha,
                                               const __nv_bfloat16* __restrict__ bias, int N, uint4 (&pk)[4]) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        uint32_t w[4] = {0u, 0u, 0u, 0u};
        const int col = col0 + j * 8;
        if (col < N) {
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                float v0 = __uint_as_float(r[j * 8 + 2 * i]) * alpha;
                float v1 = __uint_as_float(r[j * 8 + 2 * i + 1]) * alpha;
                if (bias != nullptr) {
                    v0 += __bfloat162float(bias[col + 2 * i]);
                    v1 += __bfloat162float(bias[col + 2 * i + 1]);
                }
                __nv_bfloat162 h = __floats2bfloat162_rn(v0, v1);
                w[i] = *reinterpret_cast<uint32_t*>(&h);
            }
        }
        pk[j] = make_uint4(w[0], w[1], w[2], w[3]);
    }
}
__device__ __forceinline__ void store_packed_chunk(__nv_bfloat16* dst, int col0, int N, const uint4 (&pk)[4]) {
#pragma unroll
    for (int j = 0; j < 4; ++j)
        if (col0 + j * 8 < N) *reinterpret_cast<uint4*>(dst + j * 8) = pk[j];
}

// Where the epilogue of a row-sharded product writes. DIST_LOCAL: the one output matrix D.
// DIST_BROADCAST (output all-gather): every tile goes to all `count` destinations, each the full
// [M, ld] output of one GPU, at column offset col_off (this shard's columns).
// DIST_SCATTER (input-gradient reduce-scatter): rows [c*rows_per, (c+1)*rows_per) go to ptr[c], the
// slot GPU c keeps for this GPU's partial sums ([rows_per, ld]); the owner adds the slots up.
// Peer pointers are plain global addresses mapped through CUDA IPC; the stores cross NVLink.
// With `multicast` set, DIST_BROADCAST has ONE destination, the multicast address of the output
// (the same buffer on every GPU, bound to one NVSwitch multicast object): each 16-byte piece is
// stored once with multimem.st and replicated by the switch instead of once per destination.
constexpr int DIST_LOCAL = 0, DIST_BROADCAST = 1, DIST_SCATTER = 2;
constexpr int DIST_EPI_ROW_BYTES = 128 + 16;                   // 64 bf16 columns + padding against bank conflicts
constexpr int DIST_EPI_WARP_BYTES = 32 * DIST_EPI_ROW_BYTES;   // one turn buffer per epilogue warp
constexpr int DIST_EPI_BYTES = 4 * DIST_EPI_WARP_BYTES;
constexpr int MAX_PEERS = 8;
struct PeerOut {
    __nv_bfloat16* ptr[MAX_PEERS];
    int64_t ld;
    int64_t col_off;
    int count;
    int rows_per;
    int interleave;  // DIST_SCATTER: > 1 walks the tile rows owner by owner in turn (see interleave_rows)
    int rot;         // ... starting with the owner after this rank
    int multicast;   // DIST_BROADCAST: ptr[0] is a multicast address
};

// A second operand pair whose product lands in the same accumulator: D = A.B^T + A2.B2^T. The K loop
// simply runs on over the second pair's K blocks (a low-rank bypass next to the main product).
struct SecondOperands {
    CUtensorMap a, b;
    int k;
};

// Tile rows in raster order all belong to one owner for a long stretch, which would send the
// kernel's whole NVLink traffic in one burst (and every rank to the same GPU at once). Walking
// them owner by owner in turn, each rank starting at another owner, spreads the stores evenly
// over the kernel's duration and over the destinations. A bijection when tiles_m % G == 0.
__device__ __forceinline__ int interleave_rows(int tm, int tiles_m, int G, int rot) {
    const int owner = (tm % G + rot) % G;
    return owner * (tiles_m / G) + tm / G;
}

struct GemmSmemTail {
    uint64_t full[STAGES];
    uint64_t empty[STAGES];
    uint64_t tmem_full[2];
    uint64_t tmem_empty[2];
    uint32_t tmem_base;
    int abort_flag;
};

template <int A_MN, int B_MN>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_tcgen05_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                         __nv_bfloat16* __restrict__ D, int64_t ldD, const __nv_bfloat16* __restrict__ bias,
                         float alpha, int M, int N, int K, int32_t* status) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = ptx::smem_u32(smem_raw);
    const uint32_t base = (raw_addr + 1023u) & ~1023u;
    uint8_t* base_ptr = smem_raw + (base - raw_addr);
    GemmSmemTail* tail = reinterpret_cast<GemmSmemTail*>(base_ptr + STAGES * STAGE_BYTES);
    volatile int* abort_flag = &tail->abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tiles_m = (M + BM - 1) / BM, tiles_n = (N + BN - 1) / BN;
    const int total_tiles = tiles_m * tiles_n;
    const int num_kb = (K + BK - 1) / BK;

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
        ptx::tmem_alloc(ptx::smem_u32(&tail->tmem_base), TMEM_COLS);
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
        // ------------------------------ TMA producer ------------------------------
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x) {
            int tm, tn;
            tile_coords(tile, tiles_m, tiles_n, tm, tn);
            const int m0 = tm * BM, n0 = tn * BN;
            for (int kb = 0; kb < num_kb; ++kb) {
                ok = ptx::mbar_wait(ptx::smem_u32(&tail->empty[stage]), phase ^ 1u, abort_flag, status, WAIT_PRODUCER);
                if (!ok) break;
                if (lane == 0) {
                    const uint32_t bar = ptx::smem_u32(&tail->full[stage]);
                    const uint32_t sa = base + stage * STAGE_BYTES, sb = sa + A_STAGE_BYTES;
                    const int k0 = kb * BK;
                    ptx::mbar_arrive_expect_tx(bar, STAGE_BYTES);
                    if (A_MN) {
#pragma unroll
                        for (int j = 0; j < BM / 64; ++j) ptx::tma_load_2d(sa + j * MN_BOX_BYTES, &tmA, bar, m0 + 64 * j, k0);
                    } else {
                        ptx::tma_load_2d(sa, &tmA, bar, k0, m0);
                    }
                    if (B_MN) {
#pragma unroll
                        for (int j = 0; j < BN / 64; ++j) ptx::tma_load_2d(sb + j * MN_BOX_BYTES, &tmB, bar, n0 + 64 * j, k0);
                    } else {
                        ptx::tma_load_2d(sb, &tmB, bar, k0, n0);
                    }
                }
                __syncwarp();
                if (++stage == STAGES) { stage = 0; phase ^= 1u; }
            }
        }
        if (!ok) {
            // Give copies that are still in flight time to land before shared memory is released.
            for (int i = 0; i < 1000; ++i) __nanosleep(1000);
        }
    } else if (warp == 1) {
        // ------------------------------ MMA issuer ------------------------------
        constexpr uint32_t idesc = ptx::make_idesc_bf16(BM, BN, A_MN, B_MN, 0);
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        int t = 0;
        for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++t) {
            const int acc = t & 1;
            const uint32_t acc_phase = (uint32_t)(t >> 1) & 1u;
            ok = ptx::mbar_wait(ptx::smem_u32(&tail->tmem_empty[acc]), acc_phase ^ 1u, abort_flag, status, WAIT_MMA_TMEM);
            if (!ok) break;
            ptx::tc_fence_after();
            const uint32_t tmem_d = tmem_base + (uint32_t)(acc * BN);
            for (int kb = 0; kb < num_kb; ++kb) {
                ok = ptx::mbar_wait(ptx::smem_u32(&tail->full[stage]), phase, abort_flag, status, WAIT_MMA_FULL);
                if (!ok) break;
                ptx::tc_fence_after();
                if (lane == 0) {
                    const uint32_t sa = base + stage * STAGE_BYTES, sb = sa + A_STAGE_BYTES;
#pragma unroll
                    for (int k = 0; k < BK / UMMA_K; ++k) {
                        // K-major: 16 elements = 32 bytes inside the 128-byte swizzled row.
                        // MN-major: 16 K-rows of 128 bytes.
                        const uint64_t adesc = A_MN ? ptx::make_smem_desc(sa + k * (UMMA_K * 128), MN_BOX_BYTES, 1024, 2)
                                                    : ptx::make_smem_desc(sa + k * (UMMA_K * 2), 16, 1024, 2);
                        const uint64_t bdesc = B_MN ? ptx::make_smem_desc(sb + k * (UMMA_K * 128), MN_BOX_BYTES, 1024, 2)
                                                    : ptx::make_smem_desc(sb + k * (UMMA_K * 2), 16, 1024, 2);
                        ptx::mma_f16_ss(tmem_d, adesc, bdesc, idesc, (kb | k) != 0 ? 1u : 0u);
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
        // ------------------------------ epilogue ------------------------------
        const int q = warp & 3;  // TMEM lanes [32q, 32q+32) belong to warps with warp % 4 == q
        bool ok = true;
        int t = 0;
        for (int tile = blockIdx.x; tile < total_tiles && ok; tile += gridDim.x, ++t) {
            int tm, tn;
            tile_coords(tile, tiles_m, tiles_n, tm, tn);
            const int m0 = tm * BM, n0 = tn * BN;
            const int acc = t & 1;
            const uint32_t acc_phase = (uint32_t)(t >> 1) & 1u;
            ok = ptx::mbar_wait(ptx::smem_u32(&tail->tmem_full[acc]), acc_phase, abort_flag, status, WAIT_EPILOGUE);
            if (!ok) break;
            ptx::tc_fence_after();
            const int row = m0 + q * 32 + lane;
            __nv_bfloat16* drow = D + (int64_t)row * ldD + n0;
            const uint32_t taddr = tmem_base + (uint32_t)(acc * BN) + ((uint32_t)(q * 32) << 16);
#pragma unroll 1
            for (int c = 0; c < BN / 32; ++c) {
                uint32_t r[32];
                ptx::tmem_ld_32x32b_x32(taddr + (uint32_t)(c * 32), r);
                ptx::tmem_ld_wait();
                if (row < M) store_row_chunk(r, drow + c * 32, n0 + c * 32, N, alpha, bias);
            }
            ptx::tc_fence_before();
            __syncwarp();
            if (lane == 0) ptx::mbar_arrive(ptx::smem_u32(&tail->tmem_empty[acc]));
        }
    }

    // ------------------------------ teardown ------------------------------
    ptx::tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// ---------------------------------------------------------------------------------------
// CTA-pair variant (tcgen05 .cta_group::2): a cluster of two CTAs computes a 256 x 256 tile.
// Each CTA loads its own 128 rows of A but only 128 of the 256 rows of B; the leader's MMAs
// read both halves. A stage shrinks from 48 KiB to 32 KiB for the same FLOPs, so the ring
// holds 6 stages and the L2 -> SM operand traffic per FLOP drops by a third. Barrier protocol:
// `full` lives in the leader and counts the bytes of both CTAs, `empty` and `tmem_full` are
// released in both CTAs by multicast commits, `tmem_empty` of the leader collects the eight
// epilogue warps of the pair.
// ---------------------------------------------------------------------------------------
// 64 columns of 32 rows (a thread holds one row, ra / rb its two 32-column halves) are packed to bf16
// and turned in the warp's shared buffer: afterwards lane (rsub = lane / 8, piece = lane % 8) holds in
// v[rg] the 16-byte piece `piece` of row rg * 4 + rsub, so that a warp store covers four rows x 128
// contiguous bytes.
__device__ __forceinline__ void dist_turn_chunk(uint8_t* ebuf, int lane, const uint32_t (&ra)[32], const uint32_t (&rb)[32],
                                                int col0, float alpha, const __nv_bfloat16* __restrict__ bias, int N,
                                                uint4 (&v)[8]) {
    const int piece = lane & 7, rsub = lane >> 3;
    uint4 pk[4];
    pack_row_chunk(ra, col0, alpha, bias, N, pk);
#pragma unroll
    for (int j = 0; j < 4; ++j) *reinterpret_cast<uint4*>(ebuf + lane * DIST_EPI_ROW_BYTES + j * 16) = pk[j];
    pack_row_chunk(rb, col0 + 32, alpha, bias, N, pk);
#pragma unroll
    for (int j = 0; j < 4; ++j) *reinterpret_cast<uint4*>(ebuf + lane * DIST_EPI_ROW_BYTES + (4 + j) * 16) = pk[j];
    __syncwarp();
#pragma unroll
    for (int rg = 0; rg < 8; ++rg)
        v[rg] = *reinterpret_cast<const uint4*>(ebuf + (rg * 4 + rsub) * DIST_EPI_ROW_BYTES + piece * 16);
    __syncwarp();  // ebuf may be overwritten by the next chunk
}

// Stores the turned chunk (rows row0 ... row0 + 31, columns col0 ... col0 + 63 of the product) to where
// the sharded epilogue sends it.
template <int DIST>
__device__ __forceinline__ void dist_store_chunk(const PeerOut& po, const uint4 (&v)[8], int lane, int row0, int col0, int M,
                                                 int N) {
    const int piece = lane & 7, rsub = lane >> 3;
    const int col = col0 + piece * 8;
#pragma unroll
    for (int rg = 0; rg < 8; ++rg) {
        const int orow = row0 + rg * 4 + rsub;
        if (orow < M && col < N) {
            if (DIST == DIST_SCATTER) {
                const int owner = min(orow / po.rows_per, po.count - 1);
                *reinterpret_cast<uint4*>(po.ptr[owner] + (int64_t)(orow - owner * po.rows_per) * po.ld + col) = v[rg];
            } else {
                const int64_t off = (int64_t)orow * po.ld + po.col_off + col;
                if (po.multicast) ptx::multimem_st_v4(po.ptr[0] + off, v[rg]);
                else
                    for (int d = 0; d < po.count; ++d) *reinterpret_cast<uint4*>(po.ptr[d] + off) = v[rg];
            }
        }
    }
}

constexpr int PAIR_STAGES = 6;
constexpr int PAIR_BNH = BN / 2;                       // B rows loaded by each CTA for a whole tile
constexpr int PAIR_B_BYTES = PAIR_BNH * BK * 2;        // 16 KiB
constexpr int PAIR_STAGE_BYTES = A_STAGE_BYTES + PAIR_B_BYTES;
constexpr int PAIR_SMEM_BYTES = PAIR_STAGES * PAIR_STAGE_BYTES + 1024 + 256;

struct PairSmemTail {
    uint64_t full[PAIR_STAGES];
    uint64_t empty[PAIR_STAGES];
    uint64_t tmem_full[2];
    uint64_t tmem_empty[2];
    uint32_t tmem_base;
    int abort_flag;
};

template <int A_MN, int B_MN, int DIST = DIST_LOCAL, int DUAL = 0>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                      __nv_bfloat16* __restrict__ D, int64_t ldD, const __nv_bfloat16* __restrict__ bias,
                      float alpha, int M, int N, int K, int32_t* status, const __grid_constant__ PeerOut po,
                      const __grid_constant__ SecondOperands second) {
    static_assert(!DUAL || (A_MN == 0 && B_MN == 0 && DIST == DIST_LOCAL), "second operand pair: K-contiguous, local output");

    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw_addr = ptx::smem_u32(smem_raw);
    const uint32_t base = (raw_addr + 1023u) & ~1023u;
    uint8_t* base_ptr = smem_raw + (base - raw_addr);
    PairSmemTail* tail = reinterpret_cast<PairSmemTail*>(base_ptr + PAIR_STAGES * PAIR_STAGE_BYTES);
    volatile int* abort_flag = &tail->abort_flag;

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t cta = ptx::cluster_ctarank();
    const int pair = blockIdx.x >> 1, num_pairs = gridDim.x >> 1;
    const int tiles_m = (M + 2 * BM - 1) / (2 * BM), tiles_n = (N + BN - 1) / BN;
    const int total_tiles = tiles_m * tiles_n;
    const int num_kb1 = (K + BK - 1) / BK;
    const int num_kb = num_kb1 + (DUAL ? (second.k + BK - 1) / BK : 0);

    if (threadIdx.x == 0) {
        for (int s = 0; s < PAIR_STAGES; ++s) {
            ptx::mbar_init(ptx::smem_u32(&tail->full[s]), 1);
            ptx::mbar_init(ptx::smem_u32(&tail->empty[s]), 1);
        }
        for (int a = 0; a < 2; ++a) {
            ptx::mbar_init(ptx::smem_u32(&tail->tmem_full[a]), 1);
            ptx::mbar_init(ptx::smem_u32(&tail->tmem_empty[a]), 8);
        }
        tail->abort_flag = 0;
        ptx::fence_barrier_init();
    }
    if (warp == 1) {
        ptx::tmem_alloc_pair(ptx::smem_u32(&tail->tmem_base), TMEM_COLS);
        ptx::tmem_relinquish_pair();
    }
    if (warp == 0 && lane == 0) {
        ptx::prefetch_tensormap(&tmA);
        ptx::prefetch_tensormap(&tmB);
        if (DUAL) {
            ptx::prefetch_tensormap(&second.a);
            ptx::prefetch_tensormap(&second.b);
        }
    }
    ptx::tc_fence_before();
    __syncthreads();
    ptx::cluster_sync_all();
    ptx::tc_fence_after();
    const uint32_t tmem_base = tail->tmem_base;

    if (warp == 0) {
        int stage = 0;
        uint32_t phase = 0;
        bool ok = true;
        for (int tile = pair; tile < total_tiles && ok; tile += num_pairs) {
            int tm, tn;
            tile_coords(tile, tiles_m, tiles_n, tm, tn);
            if (DIST == DIST_SCATTER && po.interleave > 1) tm = interleave_rows(tm, tiles_m, po.interleave, po.rot);
            const int m0 = tm * 2 * BM + (int)cta * BM;       // this CTA's rows of A / D
            const int n0 = tn * BN + (int)cta * PAIR_BNH;     // this CTA's half of the B rows
            for (int kb = 0; kb < num_kb; ++kb) {
                ok = ptx::mbar_wait(ptx::smem_u32(&tail->empty[stage]), phase ^ 1u, abort_flag, status, 31);
                if (!ok) break;
                if (lane == 0) {
                    const uint32_t local_bar = ptx::smem_u32(&tail->full[stage]);
                    const uint32_t bar = ptx::map_to_cta(local_bar, 0);
                    const uint32_t sa = base + stage * PAIR_STAGE_BYTES, sb = sa + A_STAGE_BYTES;
                    const bool two = DUAL && kb >= num_kb1;  // the second pair's K blocks (zero-filled past its K)
                    const int k0 = (two ? kb - num_kb1 : kb) * BK;
                    if (cta == 0) ptx::mbar_arrive_expect_tx(local_bar, 2 * PAIR_STAGE_BYTES);
                    if (A_MN) {
#pragma unroll
                        for (int j = 0; j < BM / 64; ++j) ptx::tma_load_2d_pair(sa + j * MN_BOX_BYTES, &tmA, bar, m0 + 64 * j, k0);
                    } else {
                        ptx::tma_load_2d_pair(sa, two ? &second.a : &tmA, bar, k0, m0);
                    }
                    if (B_MN) {
#pragma unroll
                        for (int j = 0; j < PAIR_BNH / 64; ++j) ptx::tma_load_2d_pair(sb + j * MN_BOX_BYTES, &tmB, bar, n0 + 64 * j, k0);
                    } else {
                        ptx::tma_load_2d_pair(sb, two ? &second.b : &tmB, bar, k0, n0);
                    }
                }
                __syncwarp();
                if (++stage == PAIR_STAGES) { stage = 0; phase ^= 1u; }
            }
        }
        if (!ok) for (int i = 0; i < 1000; ++i) __nanosleep(1000);
    } else if (warp == 1) {
        if (cta == 0) {
            constexpr uint32_t idesc = ptx::make_idesc_bf16(2 * BM, BN, A_MN, B_MN, 0);
            int stage = 0;
            uint32_t phase = 0;
            bool ok = true;
            int t = 0;
            for (int tile = pair; tile < total_tiles && ok; tile += num_pairs, ++t) {
                const int acc = t & 1;
                const uint32_t acc_phase = (uint32_t)(t >> 1) & 1u;
                ok = ptx::mbar_wait(ptx::smem_u32(&tail->tmem_empty[acc]), acc_phase ^ 1u, abort_flag, status, 33);
                if (!ok) break;
                ptx::tc_fence_after();
                const uint32_t tmem_d = tmem_base + (uint32_t)(acc * BN);
                for (int kb = 0; kb < num_kb; ++kb) {
                    ok = ptx::mbar_wait(ptx::smem_u32(&tail->full[stage]), phase, abort_flag, status, 32);
                    if (!ok) break;
                    ptx::tc_fence_after();
                    if (lane == 0) {
                        const uint32_t sa = base + stage * PAIR_STAGE_BYTES, sb = sa + A_STAGE_BYTES;
#pragma unroll
                        for (int k = 0; k < BK / UMMA_K; ++k) {
                            const uint64_t adesc = A_MN ? ptx::make_smem_desc(sa + k * (UMMA_K * 128), MN_BOX_BYTES, 1024, 2)
                                                        : ptx::make_smem_desc(sa + k * (UMMA_K * 2), 16, 1024, 2);
                            const uint64_t bdesc = B_MN ? ptx::make_smem_desc(sb + k * (UMMA_K * 128), MN_BOX_BYTES, 1024, 2)
                                                        : ptx::make_smem_desc(sb + k * (UMMA_K * 2), 16, 1024, 2);
                            ptx::mma_f16_ss_pair(tmem_d, adesc, bdesc, idesc, (kb | k) != 0 ? 1u : 0u);
                        }
                        ptx::mma_commit_pair(ptx::smem_u32(&tail->empty[stage]), (uint16_t)3);
                    }
                    __syncwarp();
                    if (++stage == PAIR_STAGES) { stage = 0; phase ^= 1u; }
                }
                if (!ok) break;
                if (lane == 0) ptx::mma_commit_pair(ptx::smem_u32(&tail->tmem_full[acc]), (uint16_t)3);
                __syncwarp();
            }
        }
    } else {
        const int q = warp & 3;
        const uint32_t leader_empty0 = ptx::map_to_cta(ptx::smem_u32(&tail->tmem_empty[0]), 0);
        const uint32_t leader_empty1 = ptx::map_to_cta(ptx::smem_u32(&tail->tmem_empty[1]), 0);
        bool ok = true;
        int t = 0;
        for (int tile = pair; tile < total_tiles && ok; tile += num_pairs, ++t) {
            int tm, tn;
            tile_coords(tile, tiles_m, tiles_n, tm, tn);
            if (DIST == DIST_SCATTER && po.interleave > 1) tm = interleave_rows(tm, tiles_m, po.interleave, po.rot);
            const int m0 = tm * 2 * BM + (int)cta * BM, n0 = tn * BN;
            const int acc = t & 1;
            const uint32_t acc_phase = (uint32_t)(t >> 1) & 1u;
            ok = ptx::mbar_wait(ptx::smem_u32(&tail->tmem_full[acc]), acc_phase, abort_flag, status, 34);
            if (!ok) break;
            ptx::tc_fence_after();
            const int row = m0 + q * 32 + lane;
            const uint32_t taddr = tmem_base + (uint32_t)(acc * BN) + ((uint32_t)(q * 32) << 16);
            if (DIST == DIST_LOCAL) {
                __nv_bfloat16* drow = D + (int64_t)row * ldD + n0;
#pragma unroll 1
                for (int c = 0; c < BN / 32; ++c) {
                    uint32_t r[32];
                    ptx::tmem_ld_32x32b_x32(taddr + (uint32_t)(c * 32), r);
                    ptx::tmem_ld_wait();
                    if (row < M) store_row_chunk(r, drow + c * 32, n0 + c * 32, N, alpha, bias);
                }
            } else {
                // Stores that cross NVLink are not merged by the local L2, so the tile is turned in
                // shared memory first: a thread holds one row, a warp store then covers four rows
                // x 128 contiguous bytes (8 lanes x 16 B per row) in every destination.
                uint8_t* ebuf = base_ptr + PAIR_STAGES * PAIR_STAGE_BYTES + 256 + (warp - 2) * DIST_EPI_WARP_BYTES;
                // The accumulator reads of the next 64 columns are in flight while the stores of
                // this chunk are issued; the accumulator is handed back to the MMA warp as soon as
                // its last column has been read, before the last stores go out.
                uint32_t ra[32], rb[32];
                ptx::tmem_ld_32x32b_x32(taddr, ra);
                ptx::tmem_ld_32x32b_x32(taddr + 32u, rb);
                ptx::tmem_ld_wait();
                constexpr int chunks = BN / 64;
#pragma unroll 1
                for (int c = 0; c < chunks; ++c) {
                    uint4 v[8];
                    dist_turn_chunk(ebuf, lane, ra, rb, n0 + c * 64, alpha, bias, N, v);
                    if (c + 1 < chunks) {
                        ptx::tmem_ld_32x32b_x32(taddr + (uint32_t)((c + 1) * 64), ra);
                        ptx::tmem_ld_32x32b_x32(taddr + (uint32_t)((c + 1) * 64 + 32), rb);
                    } else {
                        ptx::tc_fence_before();
                        __syncwarp();
                        if (lane == 0) ptx::mbar_arrive_cluster(acc ? leader_empty1 : leader_empty0);
                    }
                    dist_store_chunk<DIST>(po, v, lane, m0 + q * 32, n0 + c * 64, M, N);
                    if (c + 1 < chunks) ptx::tmem_ld_wait();
                }
            }
            if (DIST == DIST_LOCAL) {
                ptx::tc_fence_before();
                __syncwarp();
                if (lane == 0) ptx::mbar_arrive_cluster(acc ? leader_empty1 : leader_empty0);
            }
        }
        // stores to other GPUs' memory are made visible system-wide before the kernel ends
        if (DIST != DIST_LOCAL) __threadfence_system();
    }

    ptx::tc_fence_before();
    __syncthreads();
    ptx::cluster_sync_all();
    if (warp == 1) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc_pair(tmem_base, TMEM_COLS);
    }
}

// ---------------------------------------------------------------------------------------
// fp32 FMA GEMM for the fp32 parity cases: C[m,n] = alpha * sum_k A(m,k) B(n,k) (+ bias[n]).
// Operands are addressed through element strides, so one kernel covers the three products.
// ---------------------------------------------------------------------------------------
constexpr int FT = 64, FK = 16;

__global__ void __launch_bounds__(256)
gemm_f32_fma_kernel(const float* __restrict__ A, int64_t sAm, int64_t sAk, const float* __restrict__ B,
                    int64_t sBn, int64_t sBk, float* __restrict__ C, int64_t ldC, const float* __restrict__ bias,
                    float alpha, int M, int N, int K) {
    __shared__ float As[FK][FT + 1];
    __shared__ float Bs[FK][FT + 1];
    const int tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const int m0 = blockIdx.y * FT, n0 = blockIdx.x * FT;
    float acc[4][4] = {};
    for (int k0 = 0; k0 < K; k0 += FK) {
        for (int i = threadIdx.x; i < FT * FK; i += 256) {
            // Pick the index order that walks the contiguous dimension of each operand.
            int ma, ka, nb, kb;
            if (sAk == 1) { ka = i % FK; ma = i / FK; } else { ma = i % FT; ka = i / FT; }
            if (sBk == 1) { kb = i % FK; nb = i / FK; } else { nb = i % FT; kb = i / FT; }
            As[ka][ma] = (m0 + ma < M && k0 + ka < K) ? A[(int64_t)(m0 + ma) * sAm + (int64_t)(k0 + ka) * sAk] : 0.0f;
            Bs[kb][nb] = (n0 + nb < N && k0 + kb < K) ? B[(int64_t)(n0 + nb) * sBn + (int64_t)(k0 + kb) * sBk] : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int k = 0; k < FK; ++k) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) { a[i] = As[k][ty * 4 + i]; b[i] = Bs[k][tx * 4 + i]; }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int n = n0 + tx * 4 + j;
            if (n < N) C[(int64_t)m * ldC + n] = acc[i][j] * alpha + (bias ? bias[n] : 0.0f);
        }
    }
}

// ---------------------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                  CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

typedef CUresult (*CtxGetCurrentFn)(CUcontext*);

// Driver calls need a context current on the calling thread. A thread that has made no runtime
// call yet (an autograd worker on device 0) has none; a no-op runtime call binds the primary
// context of the current device. Checked through the driver so that nothing but the two queries
// runs on threads that are already set up (cudaFree is not allowed during stream capture).
static int ensure_context() {
    static CtxGetCurrentFn get_current = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuCtxGetCurrent", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            get_current = reinterpret_cast<CtxGetCurrentFn>(p);
    });
    CUcontext ctx = nullptr;
    if (get_current && get_current(&ctx) == CUDA_SUCCESS && ctx != nullptr) return SF_OK;
    SF_CHECK_CUDA(cudaFree(nullptr));
    return SF_OK;
}

static EncodeTiledFn encode_tiled_fn() {
    static EncodeTiledFn fn = nullptr;
    static std::once_flag once;
    std::call_once(once, [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) == cudaSuccess &&
            qres == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
    });
    return fn;
}

// Encoded tensor maps are kept in a small process-wide table keyed by what they were encoded from
// (address, extents, leading dimension, box, kind): a training step launches the same products on the
// same buffers over and over, and a lookup is cheaper than the driver call. The table owns nothing: an
// entry is only a function of its key, so a buffer that was freed and reallocated at the same address
// with the same shape gets an identical map. It is emptied when it reaches kMapCacheMax entries.
struct MapKey {
    const void* ptr;
    int64_t inner, outer, ld;
    int box, kind;
    bool operator==(const MapKey& o) const {
        return ptr == o.ptr && inner == o.inner && outer == o.outer && ld == o.ld && box == o.box && kind == o.kind;
    }
};
struct MapKeyHash {
    size_t operator()(const MapKey& k) const {
        uint64_t h = reinterpret_cast<uintptr_t>(k.ptr) * 0x9E3779B97F4A7C15ull;
        h ^= (uint64_t)k.inner * 0xC2B2AE3D27D4EB4Full + (uint64_t)k.outer * 0x165667B19E3779F9ull;
        h ^= ((uint64_t)k.ld << 20) ^ ((uint64_t)k.box << 8) ^ (uint64_t)k.kind;
        return (size_t)(h ^ (h >> 29));
    }
};
constexpr size_t kMapCacheMax = 2048;
static std::mutex g_map_mu;
static std::unordered_map<MapKey, CUtensorMap, MapKeyHash> g_map_cache;

static bool map_cache_get(const MapKey& k, CUtensorMap* out) {
    std::lock_guard<std::mutex> lock(g_map_mu);
    auto it = g_map_cache.find(k);
    if (it == g_map_cache.end()) return false;
    *out = it->second;
    return true;
}
static void map_cache_put(const MapKey& k, const CUtensorMap& m) {
    std::lock_guard<std::mutex> lock(g_map_mu);
    if (g_map_cache.size() >= kMapCacheMax) g_map_cache.clear();
    g_map_cache[k] = m;
}

// Tensor map over a row-major bf16 matrix [outer, inner] with a 128-byte-swizzled box of
// 64 inner elements x box_outer rows.
int make_bf16_tensor_map(CUtensorMap* map, const void* ptr, int64_t inner, int64_t outer, int64_t ld,
                         int box_outer) {
    const MapKey key{ptr, inner, outer, ld, box_outer, 0};
    if (map_cache_get(key, map)) return SF_OK;
    if (int rc = ensure_context()) return rc;
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return fail(SF_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    cuuint64_t dims[2] = {(cuuint64_t)inner, (cuuint64_t)outer};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {64, (cuuint32_t)box_outer};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(SF_ERR_CUDA, "cuTensorMapEncodeTiled failed with CUresult %d", (int)r);
    map_cache_put(key, *map);
    return SF_OK;
}

// Tensor map over a byte matrix [rows, 16] (rows of 16 bytes, no swizzle) with a box of box_rows rows:
// the tensor-core ordered 2:4 metadata, one 2048-byte tile = 128 such rows.
int make_meta_tensor_map(CUtensorMap* map, const void* ptr, int64_t rows, int box_rows) {
    const MapKey key{ptr, 16, rows, 16, box_rows, 1};
    if (map_cache_get(key, map)) return SF_OK;
    if (int rc = ensure_context()) return rc;
    EncodeTiledFn fn = encode_tiled_fn();
    if (!fn) return fail(SF_ERR_CUDA, "cuTensorMapEncodeTiled is not available from the driver");
    cuuint64_t dims[2] = {16, (cuuint64_t)rows};
    cuuint64_t strides[1] = {16};
    cuuint32_t box[2] = {16, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, const_cast<void*>(ptr), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(SF_ERR_CUDA, "cuTensorMapEncodeTiled (metadata) failed with CUresult %d", (int)r);
    map_cache_put(key, *map);
    return SF_OK;
}

// D[M,N] = alpha * A . B^T (+bias). a_mn / b_mn: operand stored with its M / N index contiguous
// (as [K, M] / [K, N] row-major with leading dimension lda / ldb), else as [M, K] / [N, K].
// The CTA-pair kernel serves every problem with more than one 128-row tile; setting
// SF_GEMM_SINGLE_CTA=1 in the environment keeps the 1-CTA kernel (for A/B measurements).
static bool use_pair_kernel() {
    static const bool v = [] {
        const char* e = getenv("SF_GEMM_SINGLE_CTA");
        return !(e && e[0] == '1');
    }();
    return v;
}

// Per-stream setting of the tensor-core products, registered by the caller with
// sf_masked_gemm_configure_stream: a limit on the CTAs a launch may occupy, so that two products on two
// streams can share the chip.
static std::mutex g_cfg_mu;
static std::unordered_map<void*, int> g_stream_max_ctas;

static int stream_max_ctas(cudaStream_t st) {
    std::lock_guard<std::mutex> lock(g_cfg_mu);
    auto it = g_stream_max_ctas.find((void*)st);
    return it == g_stream_max_ctas.end() ? 0 : it->second;
}

template <int A_MN, int B_MN>
static int launch_bf16(const void* A, int64_t lda, const void* B, int64_t ldb, void* D, int64_t ldD,
                       const void* bias, float alpha, int64_t M, int64_t N, int64_t K, int32_t* status,
                       cudaStream_t st, int dist = DIST_LOCAL, const PeerOut* peers = nullptr) {
    CUtensorMap tmA, tmB;
    int rc;
    if (A_MN) rc = make_bf16_tensor_map(&tmA, A, M, K, lda, 64);
    else rc = make_bf16_tensor_map(&tmA, A, K, M, lda, BM);
    if (rc) return rc;
    const bool pair = M > BM && use_pair_kernel();
    if (B_MN) rc = make_bf16_tensor_map(&tmB, B, N, K, ldb, 64);
    int64_t max_pairs = sm_count() / 2;
    const int limit = stream_max_ctas(st);
    if (limit >= 2 && limit / 2 < max_pairs) max_pairs = limit / 2;
    const int64_t ptiles = ((M + 2 * BM - 1) / (2 * BM)) * ((N + BN - 1) / BN);
    if (!B_MN) rc = make_bf16_tensor_map(&tmB, B, K, N, ldb, pair ? PAIR_BNH : BN);
    if (rc) return rc;
    int dev = 0;
    SF_CHECK_CUDA(cudaGetDevice(&dev));
    if (dist != DIST_LOCAL && !pair)
        return fail(SF_ERR_UNSUPPORTED, "the sharded epilogue needs more than %d rows and the CTA-pair kernel", BM);
    if (pair) {
        const int pairs = (int)(ptiles < max_pairs ? ptiles : max_pairs);
        const PeerOut none = {};
        const SecondOperands no_second = {};
#define SF_LAUNCH_PAIR(DISTV, SLOT)                                                                              \
    do {                                                                                                         \
        auto pk = gemm_bf16_pair_kernel<A_MN, B_MN, DISTV>;                                                      \
        static thread_local int pair_dev[3] = {-1, -1, -1};                                                      \
        const int smem_bytes = PAIR_SMEM_BYTES + (DISTV == DIST_LOCAL ? 0 : DIST_EPI_BYTES);                     \
        if (pair_dev[SLOT] != dev) {                                                                             \
            SF_CHECK_CUDA(cudaFuncSetAttribute(pk, cudaFuncAttributeMaxDynamicSharedMemorySize, smem_bytes));    \
            pair_dev[SLOT] = dev;                                                                                \
        }                                                                                                        \
        pk<<<2 * pairs, GEMM_THREADS, smem_bytes, st>>>(tmA, tmB, (__nv_bfloat16*)D, ldD,                        \
                                                             (const __nv_bfloat16*)bias, alpha, (int)M, (int)N,  \
                                                             (int)K, status, peers ? *peers : none, no_second);  \
    } while (0)
        if (dist == DIST_BROADCAST) SF_LAUNCH_PAIR(DIST_BROADCAST, 1);
        else if (dist == DIST_SCATTER) SF_LAUNCH_PAIR(DIST_SCATTER, 2);
        else SF_LAUNCH_PAIR(DIST_LOCAL, 0);
#undef SF_LAUNCH_PAIR
        SF_CHECK_CUDA(cudaGetLastError());
        return SF_OK;
    }
    auto kern = gemm_bf16_tcgen05_kernel<A_MN, B_MN>;
    static thread_local int configured_dev = -1;
    if (configured_dev != dev) {
        SF_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, GEMM_SMEM_BYTES));
        configured_dev = dev;
    }
    const int64_t tiles = ((M + BM - 1) / BM) * ((N + BN - 1) / BN);
    const int grid = (int)(tiles < sm_count() ? tiles : sm_count());
    kern<<<grid, GEMM_THREADS, GEMM_SMEM_BYTES, st>>>(tmA, tmB, (__nv_bfloat16*)D, ldD, (const __nv_bfloat16*)bias,
                                                      alpha, (int)M, (int)N, (int)K, status);
    SF_CHECK_CUDA(cudaGetLastError());
    return SF_OK;
}

// y[T, out] = x[T, in] . wm[out, in]^T + z[T, rank] . sw[out, rank]^T (+ bias): one launch of the pair kernel
// whose K loop runs over both operand pairs.
static int launch_bf16_dual(const void* x, const void* wm, const void* z, const void* sw, const void* bias, void* y,
                            int64_t T, int64_t in, int64_t out, int64_t rank, int32_t* status, cudaStream_t st) {
    if (T <= BM || !use_pair_kernel())
        return fail(SF_ERR_UNSUPPORTED, "the two-pair product needs more than %d rows and the CTA-pair kernel", BM);
    CUtensorMap tmA, tmB;
    SecondOperands second;
    int rc = make_bf16_tensor_map(&tmA, x, in, T, in, BM);
    if (!rc) rc = make_bf16_tensor_map(&tmB, wm, in, out, in, PAIR_BNH);
    if (!rc) rc = make_bf16_tensor_map(&second.a, z, rank, T, rank, BM);
    if (!rc) rc = make_bf16_tensor_map(&second.b, sw, rank, out, rank, PAIR_BNH);
    if (rc) return rc;
    second.k = (int)rank;
    int64_t max_pairs = sm_count() / 2;
    const int limit = stream_max_ctas(st);
    if (limit >= 2 && limit / 2 < max_pairs) max_pairs = limit / 2;
    const int64_t ptiles = ((T + 2 * BM - 1) / (2 * BM)) * ((out + BN - 1) / BN);
    const int pairs = (int)(ptiles < max_pairs ? ptiles : max_pairs);
    int dev = 0;
    SF_CHECK_CUDA(cudaGetDevice(&dev));
    auto pk = gemm_bf16_pair_kernel<0, 0, DIST_LOCAL, 1>;
    static thread_local int dual_dev = -1;
    if (dual_dev != dev) {
        SF_CHECK_CUDA(cudaFuncSetAttribute(pk, cudaFuncAttributeMaxDynamicSharedMemorySize, PAIR_SMEM_BYTES));
        dual_dev = dev;
    }
    const PeerOut none = {};
    pk<<<2 * pairs, GEMM_THREADS, PAIR_SMEM_BYTES, st>>>(tmA, tmB, (__nv_bfloat16*)y, out, (const __nv_bfloat16*)bias, 1.0f,
                                                         (int)T, (int)out, (int)in, status, none, second);
    SF_CHECK_CUDA(cudaGetLastError());
    return SF_OK;
}

static int launch_f32(const float* A, int64_t sAm, int64_t sAk, const float* B, int64_t sBn, int64_t sBk, float* C,
                      int64_t ldC, const float* bias, float alpha, int64_t M, int64_t N, int64_t K,
                      cudaStream_t st) {
    dim3 grid((unsigned)((N + FT - 1) / FT), (unsigned)((M + FT - 1) / FT));
    gemm_f32_fma_kernel<<<grid, 256, 0, st>>>(A, sAm, sAk, B, sBn, sBk, C, ldC, bias, alpha, (int)M, (int)N, (int)K);
    SF_CHECK_CUDA(cudaGetLastError());
    return SF_OK;
}

static int check_gemm_args(const char* who, const void* a, const void* b, const void* d, int64_t T, int64_t in,
                           int64_t out, int dtype) {
    if (!a || !b || !d) return fail(SF_ERR_BAD_ARG, "%s: operand pointers must be non-null", who);
    if (T <= 0 || in <= 0 || out <= 0) return fail(SF_ERR_BAD_ARG, "%s: T, in, out must be positive", who);
    if (dtype != SF_F32 && dtype != SF_BF16) return fail(SF_ERR_BAD_ARG, "%s: dtype must be SF_F32 or SF_BF16", who);
    if (T > 0x7fffffff || in > 0x7fffffff || out > 0x7fffffff)
        return fail(SF_ERR_UNSUPPORTED, "%s: dimension beyond 2^31-1", who);
    if (dtype == SF_BF16) {
        if ((T % 8) || (in % 8) || (out % 8))
            return fail(SF_ERR_UNSUPPORTED, "%s: bf16 path needs T, in, out multiples of 8 (16-byte rows), got %lld %lld %lld",
                        who, (long long)T, (long long)in, (long long)out);
        if (!aligned16(a) || !aligned16(b) || !aligned16(d))
            return fail(SF_ERR_ALIGNMENT, "%s: operands must be 16-byte aligned", who);
    }
    return SF_OK;
}

}  // namespace sf

using namespace sf;

extern "C" {

int sf_masked_gemm_fwd(const void* x, const void* wm, const void* bias, void* y, int64_t T, int64_t in, int64_t out,
                       float alpha, int dtype, int32_t* status, void* stream) {
    int rc = check_gemm_args("sf_masked_gemm_fwd", x, wm, y, T, in, out, dtype);
    if (rc) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    if (dtype == SF_F32)
        return launch_f32((const float*)x, in, 1, (const float*)wm, in, 1, (float*)y, out, (const float*)bias, alpha, T, out, in, st);
    return launch_bf16<0, 0>(x, in, wm, in, y, out, bias, alpha, T, out, in, status, st);
}

int sf_masked_gemm_fwd_lowrank(const void* x, const void* wm, const void* z, const void* sw, const void* bias, void* y,
                               int64_t T, int64_t in, int64_t out, int64_t rank, int dtype, int32_t* status, void* stream) {
    int rc = check_gemm_args("sf_masked_gemm_fwd_lowrank", x, wm, y, T, in, out, dtype);
    if (rc) return rc;
    if (!z || !sw) return fail(SF_ERR_BAD_ARG, "sf_masked_gemm_fwd_lowrank: z and sw must be non-null");
    if (dtype != SF_BF16) return fail(SF_ERR_UNSUPPORTED, "sf_masked_gemm_fwd_lowrank: bf16 only");
    if (rank <= 0 || (rank % 8) || rank > 0x7fffffff)
        return fail(SF_ERR_UNSUPPORTED, "sf_masked_gemm_fwd_lowrank: rank=%lld must be a positive multiple of 8", (long long)rank);
    if (!aligned16(z) || !aligned16(sw)) return fail(SF_ERR_ALIGNMENT, "sf_masked_gemm_fwd_lowrank: operands must be 16-byte aligned");
    return launch_bf16_dual(x, wm, z, sw, bias, y, T, in, out, rank, status, (cudaStream_t)stream);
}

int sf_masked_gemm_dgrad(const void* dy, const void* wm, void* dx, int64_t T, int64_t in, int64_t out, int dtype,
                         int32_t* status, void* stream) {
    int rc = check_gemm_args("sf_masked_gemm_dgrad", dy, wm, dx, T, in, out, dtype);
    if (rc) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    // dx[t, i] = sum_o dy[t, o] wm[o, i]: B(n = i, k = o) = wm[o*in + i]
    if (dtype == SF_F32)
        return launch_f32((const float*)dy, out, 1, (const float*)wm, 1, in, (float*)dx, in, nullptr, 1.0f, T, in, out, st);
    return launch_bf16<0, 1>(dy, out, wm, in, dx, in, nullptr, 1.0f, T, in, out, status, st);
}

int sf_masked_gemm_wgrad(const void* dy, const void* x, void* dw, int64_t T, int64_t in, int64_t out, int dtype,
                         int32_t* status, void* stream) {
    int rc = check_gemm_args("sf_masked_gemm_wgrad", dy, x, dw, T, in, out, dtype);
    if (rc) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    // dw[o, i] = sum_t dy[t, o] x[t, i]: A(m = o, k = t) = dy[t*out + o], B(n = i, k = t) = x[t*in + i]
    if (dtype == SF_F32)
        return launch_f32((const float*)dy, 1, out, (const float*)x, 1, in, (float*)dw, in, nullptr, 1.0f, out, in, T, st);
    return launch_bf16<1, 1>(dy, out, x, in, dw, in, nullptr, 1.0f, out, in, T, status, st);
}

int sf_masked_gemm_configure_stream(void* stream, int max_ctas) {
    SF_CHECK_ARG(max_ctas >= 0, "sf_masked_gemm_configure_stream: max_ctas must be >= 0 (0 = no limit)");
    std::lock_guard<std::mutex> lock(g_cfg_mu);
    if (max_ctas == 0) g_stream_max_ctas.erase(stream);
    else g_stream_max_ctas[stream] = max_ctas;
    return SF_OK;
}

// The bounded wait every pipeline role of the GEMM kernels uses, exercised on a barrier that nobody
// arrives at: the wait gives up after `limit_cycles`, records `code` in *status, and the kernel
// returns normally.
__global__ void bounded_wait_selftest_kernel(long long limit_cycles, int32_t* status, int code) {
    __shared__ uint64_t bar;
    __shared__ int abort_flag;
    if (threadIdx.x == 0) {
        ptx::mbar_init(ptx::smem_u32(&bar), 1);
        abort_flag = 0;
        ptx::fence_barrier_init();
    }
    __syncthreads();
    volatile int* af = &abort_flag;
    // two waiters: the first to run out sets the abort flag, the other leaves through it
    if (threadIdx.x == 0 || threadIdx.x == 32) ptx::mbar_wait_limit(ptx::smem_u32(&bar), 0, af, status, code, limit_cycles);
    __syncthreads();
}

// Issue-rate probe of the tensor cores: one CTA per SM issues `iters` MMAs of shape 128 x N x 16 (bf16,
// fp32 accumulation) back to back from one thread, with precomputed descriptors and four accumulators in
// turn, the A operand read from shared memory or from tensor memory, then commits once and waits (bounded).
// The slowest CTA's cycle count goes to cycles[0]. Operand contents do not matter for the rate.
__global__ void __launch_bounds__(128, 1)
mma_issue_rate_kernel(int n, int a_from_tmem, int iters, long long* cycles, int32_t* status) {
    extern __shared__ uint8_t smem_raw[];
    const uint32_t raw = ptx::smem_u32(smem_raw);
    const uint32_t base = (raw + 1023u) & ~1023u;
    uint8_t* bp = smem_raw + (base - raw);
    constexpr int OPERAND_BYTES = 16384 + 32768;  // A tile 128 x 64, B tile 256 x 64
    uint64_t* bar = reinterpret_cast<uint64_t*>(bp + OPERAND_BYTES);
    uint32_t* tbase = reinterpret_cast<uint32_t*>(bp + OPERAND_BYTES + 64);
    volatile int* abort_flag = reinterpret_cast<int*>(bp + OPERAND_BYTES + 128);
    for (int i = threadIdx.x; i < OPERAND_BYTES / 4; i += blockDim.x) reinterpret_cast<uint32_t*>(bp)[i] = 0x3c003c00u;
    if (threadIdx.x == 0) {
        ptx::mbar_init(ptx::smem_u32(bar), 1);
        *abort_flag = 0;
        ptx::fence_barrier_init();
    }
    const int warp = threadIdx.x >> 5;
    if (warp == 0) {
        ptx::tmem_alloc(ptx::smem_u32(tbase), 512);
        ptx::tmem_relinquish();
    }
    ptx::fence_proxy_async();
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tm = *tbase;
    if (threadIdx.x == 32) {
        const uint32_t idesc = ptx::make_idesc_bf16(128, n, 0, 0, 0);
        uint64_t ad[4], bd[4];
        for (int k = 0; k < 4; ++k) {
            ad[k] = ptx::make_smem_desc(base + k * 32, 16, 1024, 2);
            bd[k] = ptx::make_smem_desc(base + 16384 + k * 32, 16, 1024, 2);
        }
        const uint32_t step = n <= 64 ? (uint32_t)n : 0u;  // four accumulators where they fit in 256 columns
        const uint32_t ta = tm + 384u;
        long long best = 1LL << 62;
        for (int rep = 0; rep < 3; ++rep) {
            const long long t0 = clock64();
            // sixteen MMAs per trip, so that the loop itself does not bound the rate
            if (a_from_tmem) {
                for (int i = 0; i < iters; i += 16) {
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const uint32_t acc = (i | u) ? 1u : 0u;
                        ptx::mma_f16_ts(tm, ta, bd[0], idesc, acc);
                        ptx::mma_f16_ts(tm + step, ta + 8u, bd[1], idesc, acc);
                        ptx::mma_f16_ts(tm + 2 * step, ta + 16u, bd[2], idesc, acc);
                        ptx::mma_f16_ts(tm + 3 * step, ta + 24u, bd[3], idesc, acc);
                    }
                }
            } else {
                for (int i = 0; i < iters; i += 16) {
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        const uint32_t acc = (i | u) ? 1u : 0u;
                        ptx::mma_f16_ss(tm, ad[0], bd[0], idesc, acc);
                        ptx::mma_f16_ss(tm + step, ad[1], bd[1], idesc, acc);
                        ptx::mma_f16_ss(tm + 2 * step, ad[2], bd[2], idesc, acc);
                        ptx::mma_f16_ss(tm + 3 * step, ad[3], bd[3], idesc, acc);
                    }
                }
            }
            ptx::mma_commit(ptx::smem_u32(bar));
            if (!ptx::mbar_wait(ptx::smem_u32(bar), (uint32_t)(rep & 1), abort_flag, status, 98)) break;
            const long long t1 = clock64();
            if (t1 - t0 < best) best = t1 - t0;
        }
        atomicMax(reinterpret_cast<unsigned long long*>(cycles), (unsigned long long)best);
    }
    ptx::tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        ptx::tc_fence_after();
        ptx::tmem_dealloc(tm, 512);
    }
}

int sf_selftest_mma_issue_rate(int n, int a_from_tmem, int iters, int ctas, long long* cycles, int32_t* status, void* stream) {
    SF_CHECK_ARG(cycles != nullptr && status != nullptr, "sf_selftest_mma_issue_rate: cycles and status must be non-null");
    SF_CHECK_ARG(n >= 16 && n <= 256 && n % 16 == 0, "sf_selftest_mma_issue_rate: n must be a multiple of 16 in [16, 256]");
    SF_CHECK_ARG(iters >= 16 && iters <= (1 << 20) && iters % 16 == 0, "sf_selftest_mma_issue_rate: iters must be a multiple of 16 in [16, 2^20]");
    SF_CHECK_ARG(ctas >= 1 && ctas <= 1024, "sf_selftest_mma_issue_rate: ctas must be in [1, 1024]");
    constexpr int SMEM = 16384 + 32768 + 1024 + 256;
    static thread_local int configured_dev = -1;
    int dev = 0;
    SF_CHECK_CUDA(cudaGetDevice(&dev));
    if (configured_dev != dev) {
        SF_CHECK_CUDA(cudaFuncSetAttribute(mma_issue_rate_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM));
        configured_dev = dev;
    }
    cudaStream_t st = (cudaStream_t)stream;
    SF_CHECK_CUDA(cudaMemsetAsync(cycles, 0, sizeof(long long), st));
    mma_issue_rate_kernel<<<ctas, 128, SMEM, st>>>(n, a_from_tmem, iters, cycles, status);
    SF_CHECK_CUDA(cudaGetLastError());
    return SF_OK;
}

static int fill_peers(const char* who, void* const* ptrs, int n_peers, PeerOut* po) {
    if (!ptrs || n_peers < 1 || n_peers > MAX_PEERS)
        return fail(SF_ERR_BAD_ARG, "%s: 1..%d destination pointers expected, got %d", who, MAX_PEERS, n_peers);
    *po = PeerOut{};
    for (int i = 0; i < n_peers; ++i) {
        if (!ptrs[i] || !aligned16(ptrs[i])) return fail(SF_ERR_ALIGNMENT, "%s: destination %d is null or not 16-byte aligned", who, i);
        po->ptr[i] = (__nv_bfloat16*)ptrs[i];
    }
    po->count = n_peers;
    return SF_OK;
}

int sf_selftest_bounded_wait(double limit_ms, int32_t* status, void* stream) {
    SF_CHECK_ARG(status != nullptr, "sf_selftest_bounded_wait: status must be non-null");
    SF_CHECK_ARG(limit_ms > 0.0 && limit_ms <= 100.0, "sf_selftest_bounded_wait: limit_ms must be in (0, 100]");
    int dev = 0, khz = 0;
    SF_CHECK_CUDA(cudaGetDevice(&dev));
    SF_CHECK_CUDA(cudaDeviceGetAttribute(&khz, cudaDevAttrClockRate, dev));
    const long long cycles = (long long)(limit_ms * (double)khz);
    bounded_wait_selftest_kernel<<<1, 64, 0, (cudaStream_t)stream>>>(cycles, status, 99);
    SF_CHECK_CUDA(cudaGetLastError());
    return SF_OK;
}

static int fwd_exchange(const char* who, const void* x, const void* wm, const void* bias, void* const* dests, int n_dest,
                        int multicast, int64_t T, int64_t in, int64_t out_local, int64_t out_total, int64_t col_offset,
                        float alpha, int dtype, int32_t* status, void* stream) {
    if (dtype != SF_BF16) return fail(SF_ERR_UNSUPPORTED, "%s: bf16 only", who);
    PeerOut po;
    int rc = fill_peers(who, dests, n_dest, &po);
    if (rc) return rc;
    rc = check_gemm_args(who, x, wm, dests[0], T, in, out_local, dtype);
    if (rc) return rc;
    if (col_offset < 0 || col_offset % 8 || out_total % 8 || col_offset + out_local > out_total)
        return fail(SF_ERR_BAD_ARG, "%s: columns [%lld, %lld) do not fit %lld (multiples of 8)", who,
                    (long long)col_offset, (long long)(col_offset + out_local), (long long)out_total);
    po.ld = out_total;
    po.col_off = col_offset;
    po.multicast = multicast;
    return launch_bf16<0, 0>(x, in, wm, in, nullptr, 0, bias, alpha, T, out_local, in, status, (cudaStream_t)stream,
                             DIST_BROADCAST, &po);
}

int sf_masked_gemm_fwd_allgather(const void* x, const void* wm, const void* bias, void* const* y_all, int n_dest,
                                 int64_t T, int64_t in, int64_t out_local, int64_t out_total, int64_t col_offset,
                                 float alpha, int dtype, int32_t* status, void* stream) {
    return fwd_exchange("sf_masked_gemm_fwd_allgather", x, wm, bias, y_all, n_dest, 0, T, in, out_local, out_total,
                        col_offset, alpha, dtype, status, stream);
}

int sf_masked_gemm_fwd_multicast(const void* x, const void* wm, const void* bias, void* y_mc, int64_t T, int64_t in,
                                 int64_t out_local, int64_t out_total, int64_t col_offset, float alpha, int dtype,
                                 int32_t* status, void* stream) {
    void* one[1] = {y_mc};
    return fwd_exchange("sf_masked_gemm_fwd_multicast", x, wm, bias, one, 1, 1, T, in, out_local, out_total, col_offset,
                        alpha, dtype, status, stream);
}

int sf_masked_gemm_dgrad_reducescatter(const void* dy, const void* wm, void* const* slots, int n_ranks, int rank,
                                       int64_t T, int64_t in, int64_t out_local, int dtype, int32_t* status,
                                       void* stream) {
    if (dtype != SF_BF16) return fail(SF_ERR_UNSUPPORTED, "sf_masked_gemm_dgrad_reducescatter: bf16 only");
    PeerOut po;
    int rc = fill_peers("sf_masked_gemm_dgrad_reducescatter", slots, n_ranks, &po);
    if (rc) return rc;
    rc = check_gemm_args("sf_masked_gemm_dgrad_reducescatter", dy, wm, slots[0], T, in, out_local, dtype);
    if (rc) return rc;
    if (T % n_ranks) return fail(SF_ERR_BAD_ARG, "sf_masked_gemm_dgrad_reducescatter: T=%lld is not a multiple of %d ranks",
                                 (long long)T, n_ranks);
    if (rank < 0 || rank >= n_ranks) return fail(SF_ERR_BAD_ARG, "sf_masked_gemm_dgrad_reducescatter: rank %d of %d", rank, n_ranks);
    po.ld = in;
    po.rows_per = (int)(T / n_ranks);
    // whole 256-row tiles per owner: walk the owners in turn, starting after this rank
    po.interleave = (T % ((int64_t)2 * BM * n_ranks) == 0) ? n_ranks : 1;
    po.rot = (rank + 1) % n_ranks;
    return launch_bf16<0, 1>(dy, out_local, wm, in, nullptr, 0, nullptr, 1.0f, T, in, out_local, status,
                             (cudaStream_t)stream, DIST_SCATTER, &po);
}

}  // extern "C"
