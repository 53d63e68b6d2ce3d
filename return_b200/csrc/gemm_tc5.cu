// out[M, N] = x[M, K] * W[N, K]^T in bfloat16 on the fifth-generation tensor cores (tcgen05), float32
// accumulation in tensor memory, operands brought in by TMA.
//
//   rb_tc5_gemm          the product path for many rows: one CTA per 128 x BN output tile; a producer
//                        thread streams 64-wide K blocks of both operands through a ring of
//                        shared-memory stages with cp.async.bulk.tensor (128-byte swizzle), an MMA
//                        thread issues tcgen05.mma (M = 128, N = BN, K = 16) into TMEM and frees each
//                        stage with tcgen05.commit, four epilogue warps read the accumulator with
//                        tcgen05.ld and store it.  Optional epilogue: SwiGLU over gate/up columns
//                        woven in blocks of 8 (see SwiGLUSpec).
//   rb_tc5_gemm_simple   the same tile computed with plain loads and one stage: the small twin that
//                        pins the descriptor encodings down in tests.
//
// Every mbarrier wait is bounded; a wait that gives up raises *status and the kernel still frees its
// TMEM and returns.
#include <cuda.h>

#include "tc5.cuh"
#include "tma.cuh"

namespace {

using namespace tc5;

constexpr int BM = 128;
constexpr int BK = 64;                    // bf16 elements: one 128-byte swizzle row

__device__ __forceinline__ void store_row_chunk(float* dst, const unsigned (&r)[32], int n_valid) {
#pragma unroll
    for (int j = 0; j < 32; ++j)
        if (j < n_valid) dst[j] = __uint_as_float(r[j]);
}
__device__ __forceinline__ void store_row_chunk(bf16* dst, const unsigned (&r)[32], int n_valid) {
    if (n_valid == 32 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
        for (int j = 0; j < 32; j += 8) {
            uint4 v;
            __nv_bfloat162 p0 = __floats2bfloat162_rn(__uint_as_float(r[j]), __uint_as_float(r[j + 1]));
            __nv_bfloat162 p1 = __floats2bfloat162_rn(__uint_as_float(r[j + 2]), __uint_as_float(r[j + 3]));
            __nv_bfloat162 p2 = __floats2bfloat162_rn(__uint_as_float(r[j + 4]), __uint_as_float(r[j + 5]));
            __nv_bfloat162 p3 = __floats2bfloat162_rn(__uint_as_float(r[j + 6]), __uint_as_float(r[j + 7]));
            v.x = *reinterpret_cast<unsigned*>(&p0); v.y = *reinterpret_cast<unsigned*>(&p1);
            v.z = *reinterpret_cast<unsigned*>(&p2); v.w = *reinterpret_cast<unsigned*>(&p3);
            *reinterpret_cast<uint4*>(dst + j) = v;
        }
        return;
    }
#pragma unroll
    for (int j = 0; j < 32; ++j)
        if (j < n_valid) dst[j] = __float2bfloat16_rn(__uint_as_float(r[j]));
}

// ------------------------------------------------------------------------------------ the small twin
template <int BN, typename TOut>
__global__ void __launch_bounds__(128)
tc5_gemm_simple_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w, TOut* __restrict__ out,
                       int M, int N, int K, int ldx, int ldw, int ldo, int* __restrict__ status) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char* sA = base;                             // 128 rows x 128 B
    unsigned char* sB = base + BM * 128;                  // BN rows x 128 B
    __shared__ __align__(8) unsigned long long bar_storage;
    __shared__ unsigned tmem_slot;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n0 = blockIdx.x * BN, m0 = blockIdx.y * BM;
    const unsigned bar = smem_u32(&bar_storage);
    constexpr unsigned TMEM_COLS = BN < 32 ? 32 : BN;

    if (warp == 0) tmem_alloc(smem_u32(&tmem_slot), TMEM_COLS);
    if (tid == 0) { mbar_init(bar, 1); mbar_init_fence(); }
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const unsigned tacc = tmem_slot;
    const unsigned idesc = instr_desc_bf16(BM, BN);
    unsigned phase = 0;
    bool ok = true;

    const int nkb = (K + BK - 1) / BK;
    for (int kb = 0; kb < nkb; ++kb) {
        for (int c = tid; c < BM * 8; c += 128) {
            const int r = c >> 3, ch = c & 7, m = m0 + r, k = kb * BK + ch * 8;
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (m < M && k < K) v = *reinterpret_cast<const uint4*>(x + (size_t)m * ldx + k);
            *reinterpret_cast<uint4*>(sA + sw128_offset(r, ch)) = v;
        }
        for (int c = tid; c < BN * 8; c += 128) {
            const int r = c >> 3, ch = c & 7, n = n0 + r, k = kb * BK + ch * 8;
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (n < N && k < K) v = *reinterpret_cast<const uint4*>(w + (size_t)n * ldw + k);
            *reinterpret_cast<uint4*>(sB + sw128_offset(r, ch)) = v;
        }
        fence_proxy_async();
        __syncthreads();
        if (tid == 0) {
            fence_after_sync();
#pragma unroll
            for (int k16 = 0; k16 < BK / 16; ++k16)
                mma_ss(tacc, smem_desc_sw128(smem_u32(sA), k16 * 32), smem_desc_sw128(smem_u32(sB), k16 * 32), idesc,
                       kb > 0 || k16 > 0);
            mma_commit(bar);
        }
        ok = mbar_wait(bar, phase) && ok;                   // the MMAs have read this stage: it may be refilled
        phase ^= 1;
        __syncthreads();
    }
    if (!ok && lane == 0) atomicExch(status, 1);
    fence_after_sync();
    const int m = m0 + warp * 32 + lane;
#pragma unroll 1
    for (int c0 = 0; c0 < BN; c0 += 32) {
        unsigned r[32];
        tmem_ld32(tacc + ((unsigned)(warp * 32) << 16) + c0, r);
        tmem_ld_wait();
        if (m < M && n0 + c0 < N) store_row_chunk(out + (size_t)m * ldo + n0 + c0, r, min(32, N - n0 - c0));
    }
    fence_before_sync();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tacc, TMEM_COLS);
}

// The twin with B given as [K, N] row-major (N contiguous): an MN-major B operand, as the values of
// an attention tile are.  One 128 x BN tile per CTA, K a multiple of 64.  The descriptor's leading
// offset (8192 B) steps over blocks of 64 columns of N, its stride offset (1024 B) over groups of 8 k-rows.
template <int BN>
__global__ void __launch_bounds__(128)
tc5_gemm_bmn_kernel(const bf16* __restrict__ x, const bf16* __restrict__ bmat, float* __restrict__ out,
                    int M, int N, int K, int ldx, int ldb, int ldo, int* __restrict__ status) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char* sA = base;                             // 128 rows x 128 B
    unsigned char* sB = base + BM * 128;                  // BN / 64 slabs of 64 k-rows x 128 B
    __shared__ __align__(8) unsigned long long bar_storage;
    __shared__ unsigned tmem_slot;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n0 = blockIdx.x * BN, m0 = blockIdx.y * BM;
    const unsigned bar = smem_u32(&bar_storage);
    constexpr unsigned TMEM_COLS = BN < 32 ? 32 : BN;
    if (warp == 0) tmem_alloc(smem_u32(&tmem_slot), TMEM_COLS);
    if (tid == 0) { mbar_init(bar, 1); mbar_init_fence(); }
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const unsigned tacc = tmem_slot;
    const unsigned idesc = instr_desc_bf16(BM, BN, true);
    unsigned phase = 0;
    bool ok = true;
    for (int kb = 0; kb < K / BK; ++kb) {
        for (int c = tid; c < BM * 8; c += 128) {
            const int r = c >> 3, ch = c & 7, m = m0 + r, k = kb * BK + ch * 8;
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (m < M) v = *reinterpret_cast<const uint4*>(x + (size_t)m * ldx + k);
            *reinterpret_cast<uint4*>(sA + sw128_offset(r, ch)) = v;
        }
        for (int c = tid; c < BK * (BN / 8); c += 128) {      // 64 k-rows, BN / 8 chunks of 8 n
            const int kr = c / (BN / 8), nc = c % (BN / 8), n = n0 + nc * 8;
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (n < N) v = *reinterpret_cast<const uint4*>(bmat + (size_t)(kb * BK + kr) * ldb + n);
            *reinterpret_cast<uint4*>(sB + (nc >> 3) * 8192 + sw128_offset(kr, nc & 7)) = v;
        }
        fence_proxy_async();
        __syncthreads();
        if (tid == 0) {
            fence_after_sync();
#pragma unroll
            for (int k16 = 0; k16 < BK / 16; ++k16) {
                mma_ss(tacc, smem_desc_sw128(smem_u32(sA), k16 * 32),
                       smem_desc_sw128_mn(smem_u32(sB) + k16 * 2048, 8192u, 1024u), idesc, kb > 0 || k16 > 0);
            }
            mma_commit(bar);
        }
        ok = mbar_wait(bar, phase) && ok;
        phase ^= 1;
        __syncthreads();
    }
    if (!ok && lane == 0) atomicExch(status, 1);
    fence_after_sync();
    const int m = m0 + warp * 32 + lane;
#pragma unroll 1
    for (int c0 = 0; c0 < BN; c0 += 32) {
        unsigned r[32];
        tmem_ld32(tacc + ((unsigned)(warp * 32) << 16) + c0, r);
        tmem_ld_wait();
        if (m < M && n0 + c0 < N) store_row_chunk(out + (size_t)m * ldo + n0 + c0, r, min(32, N - n0 - c0));
    }
    fence_before_sync();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tacc, TMEM_COLS);
}

// ------------------------------------------------------------------------------------ the product kernel
constexpr int TC5_STAGES = 4;             // the ring: stages x k blocks a stage x 48 KB <= 192 KB
constexpr int TC5_KPS = 1;
constexpr int TC5_THREADS = 192;          // warp 0: TMA, warp 1: MMA, warps 2..5: epilogue

// Persistent: a CTA walks output tiles tile = blockIdx.x, + gridDim.x, ...; tiles that share a block
// of W are neighbours (the M tile index runs fastest), so W is read from HBM once and X stays in L2.
// The accumulator is double-buffered in TMEM (2 x BN columns): the epilogue warps drain tile i while
// the MMA thread fills tile i + 1.  The ring of operand stages runs on across tiles.
// KPS k blocks of 64 make one stage, with one wait and one commit of the issuing thread: a wait costs that
// thread some 230 cycles even when it succeeds at once and a commit 90, beside 512 cycles for the four MMAs
// of a k block, and they add up.
template <int BN, int STAGES, int KPS, typename TOut, bool GATED>
__global__ void __launch_bounds__(TC5_THREADS)
tc5_gemm_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                TOut* __restrict__ out, int M, int N, int K, int ldo, int* __restrict__ status) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    constexpr unsigned A_BYTES = BM * BK * 2, B_BYTES = BN * BK * 2, BLOCK_BYTES = A_BYTES + B_BYTES, STAGE_BYTES = KPS * BLOCK_BYTES;
    __shared__ __align__(8) unsigned long long full_bar[STAGES], empty_bar[STAGES], acc_full[2], acc_empty[2];
    __shared__ unsigned tmem_slot;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    constexpr unsigned TMEM_COLS = 2 * BN < 32 ? 32 : 2 * BN;
    static_assert(2 * BN <= 512, "two accumulators must fit the 512 columns of tensor memory");
    const int nkb = (K + BK * KPS - 1) / (BK * KPS);        // stages a tile; k blocks past K are zero-filled by the copy
    const int m_tiles = (M + BM - 1) / BM, n_tiles = (N + BN - 1) / BN, tiles = m_tiles * n_tiles;

    if (warp == 1) tmem_alloc(smem_u32(&tmem_slot), TMEM_COLS);
    if (tid == 0) {
        tma::prefetch_desc(&map_x);
        tma::prefetch_desc(&map_w);
#pragma unroll
        for (int s = 0; s < STAGES; ++s) { mbar_init(smem_u32(&full_bar[s]), 1); mbar_init(smem_u32(&empty_bar[s]), 1); }
#pragma unroll
        for (int b = 0; b < 2; ++b) { mbar_init(smem_u32(&acc_full[b]), 1); mbar_init(smem_u32(&acc_empty[b]), 4); }
        mbar_init_fence();
    }
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    pdl_wait();                                             // the tokens come from the kernel before
    const unsigned tacc = tmem_slot;
    bool ok = true;

    if (warp == 0) {
        if (lane == 0) {                                    // ---- producer
            int it = 0;                                     // k blocks issued so far, over all tiles
            for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x) {
                const int m0 = (tile % m_tiles) * BM, n0 = (tile / m_tiles) * BN;
                for (int kb = 0; kb < nkb; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (it >= STAGES) ok = mbar_wait(smem_u32(&empty_bar[s]), ((it / STAGES) - 1) & 1) && ok;
                    const unsigned full = smem_u32(&full_bar[s]);
                    mbar_arrive_expect_tx(full, STAGE_BYTES);
                    const unsigned dst = smem_u32(base + (size_t)s * STAGE_BYTES);
#pragma unroll
                    for (int j = 0; j < KPS; ++j) {
                        tma::load_2d(dst + j * BLOCK_BYTES, &map_x, (kb * KPS + j) * BK, m0, full);
                        tma::load_2d(dst + j * BLOCK_BYTES + A_BYTES, &map_w, (kb * KPS + j) * BK, n0, full);
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {                                    // ---- MMA issuer
            const unsigned idesc = instr_desc_bf16(BM, BN);
            int it = 0, local = 0;
            for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x, ++local) {
                const int buf = local & 1;
                if (local >= 2) ok = mbar_wait(smem_u32(&acc_empty[buf]), ((local >> 1) - 1) & 1) && ok;
                fence_after_sync();
                const unsigned d = tacc + buf * BN;
                for (int kb = 0; kb < nkb; ++kb, ++it) {
                    const int s = it % STAGES;
                    ok = mbar_wait(smem_u32(&full_bar[s]), (it / STAGES) & 1) && ok;
                    fence_after_sync();
                    const unsigned a0 = smem_u32(base + (size_t)s * STAGE_BYTES);
#pragma unroll
                    for (int j = 0; j < KPS; ++j) {
                        const unsigned a = a0 + j * BLOCK_BYTES, b = a + A_BYTES;
#pragma unroll
                        for (int k16 = 0; k16 < BK / 16; ++k16)
                            mma_ss(d, smem_desc_sw128(a, k16 * 32), smem_desc_sw128(b, k16 * 32), idesc, kb > 0 || j > 0 || k16 > 0);
                    }
                    mma_commit(smem_u32(&empty_bar[s]));    // the stage is free once these MMAs have read it
                }
                mma_commit(smem_u32(&acc_full[buf]));       // this tile's accumulator is complete
            }
        }
    } else {                                                // ---- epilogue: TMEM lanes by warp % 4
        const int q = warp & 3;
        int local = 0;
        for (int tile = blockIdx.x; tile < tiles; tile += gridDim.x, ++local) {
            const int m0 = (tile % m_tiles) * BM, n0 = (tile / m_tiles) * BN;
            const int buf = local & 1;
            ok = mbar_wait(smem_u32(&acc_full[buf]), (local >> 1) & 1) && ok;
            if (tile + (int)gridDim.x >= tiles) pdl_trigger_late();        // the last tile of this CTA
            fence_after_sync();
            const int m = m0 + q * 32 + lane;
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 32) {
                unsigned r[32];
                tmem_ld32(tacc + ((unsigned)(q * 32) << 16) + buf * BN + c0, r);
                tmem_ld_wait();
                if (m >= M || n0 + c0 >= N) continue;
                if (GATED) {
                    // columns come in blocks of 8 gate values and their 8 up values: 32 columns give 16 outputs
                    TOut* dst = out + (size_t)m * ldo + ((n0 + c0) >> 1);
                    const int valid = min(16, (N - n0 - c0) >> 1);
                    float g[16];
#pragma unroll
                    for (int b = 0; b < 2; ++b)
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            const float gate = __uint_as_float(r[b * 16 + j]), up = __uint_as_float(r[b * 16 + 8 + j]);
                            g[b * 8 + j] = gate / (1.0f + __expf(-gate)) * up;
                        }
                    if (valid == 16 && sizeof(TOut) == 2 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
                        for (int j = 0; j < 16; j += 8) {
                            uint4 v;
                            __nv_bfloat162 p0 = __floats2bfloat162_rn(g[j], g[j + 1]), p1 = __floats2bfloat162_rn(g[j + 2], g[j + 3]);
                            __nv_bfloat162 p2 = __floats2bfloat162_rn(g[j + 4], g[j + 5]), p3 = __floats2bfloat162_rn(g[j + 6], g[j + 7]);
                            v.x = *reinterpret_cast<unsigned*>(&p0); v.y = *reinterpret_cast<unsigned*>(&p1);
                            v.z = *reinterpret_cast<unsigned*>(&p2); v.w = *reinterpret_cast<unsigned*>(&p3);
                            *reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(dst) + j) = v;
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (j < valid) dst[j] = from_f32<TOut>(g[j]);
                    }
                } else {
                    store_row_chunk(out + (size_t)m * ldo + n0 + c0, r, min(32, N - n0 - c0));
                }
            }
            fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(smem_u32(&acc_empty[buf]));         // this warp has drained its quarter
        }
    }
    if (!ok) atomicExch(status, 1);
    fence_before_sync();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tacc, TMEM_COLS);
}

// ------------------------------------------------------------------------------------ the pair kernel
// Two CTAs of a cluster, on neighbouring SMs, compute one 256 x 256 tile with the two-SM form of the MMA
// (cta_group::2, M = 256): CTA r of the pair holds rows r*128.. of the tile's tokens and rows r*128.. of its
// weights, so a k block costs each SM 32 KB of operands from L2 instead of the 48 KB a 128 x 256 tile of its
// own would, and the tensor core of each SM reads the other half of the weights from its peer's shared memory.
// The pair's even CTA (the leader) issues the MMAs; each CTA's accumulator half (its 128 rows x 256 columns,
// two buffers) is in its own tensor memory and is drained by its own epilogue warps.
//   producer thread (both CTAs): waits for its own "stage empty" barrier and asks for its two boxes with TMA;
//       the bytes of both CTAs are counted on the leader's "stage full" barrier (cp.async.bulk.tensor with
//       .cta_group::2 may signal a barrier of the peer), which the leader arms with the sum;
//   MMA thread (leader): waits for "stage full", issues four MMAs, and commits with a multicast to the "stage
//       empty" barriers of both CTAs; after the last k block it commits to "accumulator full" of both;
//   epilogue warps (both CTAs): wait for "accumulator full", drain, and arrive on the leader's "accumulator
//       empty" barrier (eight arrivals: four warps of each CTA).
// Nothing is multicast by TMA.  Every mbarrier wait is bounded; the two cluster barriers (after set-up, before
// the tensor memory is given back) are reached by every thread whatever the waits did.
// The order of the tiles.  Tiles that run at the same time should share operands in L2: row tiles of one block of
// weights run back to back (the row index fastest), but only PR_GROUP_ROWS row tiles of them; then the next block of
// weights for the same rows, and the next group of rows only after the last block.  What is live at a time is then
// a group's rows (16 x 256 tokens) and a few blocks of weights, whatever the number of tokens; with the row index
// fastest over all rows, 32,768 tokens (268 MB) would be read again from HBM for every block of weights.
constexpr int PR_GROUP_ROWS = 16;
__device__ __forceinline__ void pair_tile_coords(int tile, int m_tiles, int n_tiles, int& mt, int& nt) {
    const int per_group = PR_GROUP_ROWS * n_tiles;
    const int g = tile / per_group, r = tile - g * per_group;
    const int rows = min(PR_GROUP_ROWS, m_tiles - g * PR_GROUP_ROWS);     // the last group may be short
    nt = r / rows;
    mt = g * PR_GROUP_ROWS + (r - nt * rows);
}

constexpr int PR_BN = 256;                // columns of the pair's tile
constexpr int PR_HALF = PR_BN / 2;        // weight rows a CTA holds
constexpr int PR_KPS = 2;                 // k blocks of 64 a stage: one wait and one commit of the issuing thread for both
constexpr int PR_STAGES = 3;              // x 64 KB (measured at 2,048 x 24,576 x 4,096: 1.41 / 1.45 / 1.32 PFLOP/s with 1 / 2 / 3 k blocks a stage)
constexpr unsigned PR_A_BYTES = BM * BK * 2, PR_B_BYTES = PR_HALF * BK * 2, PR_BLOCK_BYTES = PR_A_BYTES + PR_B_BYTES;
constexpr unsigned PR_STAGE_BYTES = PR_KPS * PR_BLOCK_BYTES;

__device__ __forceinline__ unsigned cluster_ctarank() {
    unsigned r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void cluster_sync_all() {
    asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
// the address, in the cluster's shared window, of the same variable in CTA `rank`
__device__ __forceinline__ unsigned map_to_cta(unsigned smem_addr, unsigned rank) {
    unsigned r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_arrive_in_cluster(unsigned cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(cluster_addr) : "memory");
}
__device__ __forceinline__ void tma_load_2d_pair(unsigned smem_dst, const CUtensorMap* map, int x, int y, unsigned bar_in_cluster) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
        ::"r"(smem_dst), "l"(map), "r"(x), "r"(y), "r"(bar_in_cluster) : "memory");
}
__device__ __forceinline__ void mma_ss_pair(unsigned d_tmem, unsigned long long a_desc, unsigned long long b_desc,
                                            unsigned idesc, bool accumulate) {
    asm volatile(
        "{\n.reg .pred p;\n"
        "setp.ne.b32 p, %4, 0;\n"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"((unsigned)accumulate) : "memory");
}
// one arrival on the barrier at this address in both CTAs of the pair, when the MMAs issued so far are done
__device__ __forceinline__ void mma_commit_pair(unsigned bar) {
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(bar), "h"((unsigned short)3) : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(unsigned slot_smem, unsigned cols) {
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(slot_smem), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(unsigned taddr, unsigned cols) {
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}

template <typename TOut, bool GATED>
__global__ void __launch_bounds__(TC5_THREADS)
tc5_gemm_pair_kernel(const __grid_constant__ CUtensorMap map_x, const __grid_constant__ CUtensorMap map_w,
                     TOut* __restrict__ out, int M, int N, int K, int ldo, int* __restrict__ status) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    __shared__ __align__(8) unsigned long long full_bar[PR_STAGES], empty_bar[PR_STAGES], acc_full[2], acc_empty[2];
    __shared__ unsigned tmem_slot;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const unsigned rank = cluster_ctarank();                // 0: the leader
    const int pair = (int)blockIdx.x >> 1, pairs = (int)gridDim.x >> 1;
    constexpr unsigned TMEM_COLS = 2 * PR_BN;
    const int nkb = (K + BK * PR_KPS - 1) / (BK * PR_KPS);  // stages a tile; k blocks past K are zero-filled by the copy
    const int m_tiles = (M + 2 * BM - 1) / (2 * BM), n_tiles = (N + PR_BN - 1) / PR_BN, tiles = m_tiles * n_tiles;

    if (warp == 1) tmem_alloc_pair(smem_u32(&tmem_slot), TMEM_COLS);
    if (tid == 0) {
        tma::prefetch_desc(&map_x);
        tma::prefetch_desc(&map_w);
#pragma unroll
        for (int s = 0; s < PR_STAGES; ++s) { mbar_init(smem_u32(&full_bar[s]), 1); mbar_init(smem_u32(&empty_bar[s]), 1); }
#pragma unroll
        for (int b = 0; b < 2; ++b) { mbar_init(smem_u32(&acc_full[b]), 1); mbar_init(smem_u32(&acc_empty[b]), 8); }
        mbar_init_fence();
    }
    fence_before_sync();
    cluster_sync_all();                                     // both CTAs' barriers exist before either is signalled
    fence_after_sync();
    pdl_wait();                                             // the tokens come from the kernel before
    const unsigned tacc = tmem_slot;
    bool ok = true;

    if (warp == 0) {
        if (lane == 0) {                                    // ---- producer (both CTAs)
            int it = 0;
            for (int tile = pair; tile < tiles; tile += pairs) {
                int mt, nt;
                pair_tile_coords(tile, m_tiles, n_tiles, mt, nt);
                const int m0 = mt * 2 * BM + (int)rank * BM, n0 = nt * PR_BN + (int)rank * PR_HALF;
                for (int kb = 0; kb < nkb; ++kb, ++it) {
                    const int s = it % PR_STAGES;
                    if (it >= PR_STAGES) ok = mbar_wait(smem_u32(&empty_bar[s]), ((it / PR_STAGES) - 1) & 1) && ok;
                    const unsigned full_local = smem_u32(&full_bar[s]);
                    if (rank == 0) mbar_arrive_expect_tx(full_local, 2 * PR_STAGE_BYTES);
                    const unsigned full = map_to_cta(full_local, 0);
                    const unsigned dst = smem_u32(base + (size_t)s * PR_STAGE_BYTES);
#pragma unroll
                    for (int j = 0; j < PR_KPS; ++j) {
                        tma_load_2d_pair(dst + j * PR_BLOCK_BYTES, &map_x, (kb * PR_KPS + j) * BK, m0, full);
                        tma_load_2d_pair(dst + j * PR_BLOCK_BYTES + PR_A_BYTES, &map_w, (kb * PR_KPS + j) * BK, n0, full);
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && rank == 0) {                       // ---- MMA issuer (the leader)
            const unsigned idesc = instr_desc_bf16(2 * BM, PR_BN);
            int it = 0, local = 0;
            for (int tile = pair; tile < tiles; tile += pairs, ++local) {
                const int buf = local & 1;
                if (local >= 2) ok = mbar_wait(smem_u32(&acc_empty[buf]), ((local >> 1) - 1) & 1) && ok;
                fence_after_sync();
                const unsigned d = tacc + buf * PR_BN;
                for (int kb = 0; kb < nkb; ++kb, ++it) {
                    const int s = it % PR_STAGES;
                    ok = mbar_wait(smem_u32(&full_bar[s]), (it / PR_STAGES) & 1) && ok;
                    fence_after_sync();
                    const unsigned a0 = smem_u32(base + (size_t)s * PR_STAGE_BYTES);
#pragma unroll
                    for (int j = 0; j < PR_KPS; ++j) {
                        const unsigned a = a0 + j * PR_BLOCK_BYTES, b = a + PR_A_BYTES;
#pragma unroll
                        for (int k16 = 0; k16 < BK / 16; ++k16)
                            mma_ss_pair(d, smem_desc_sw128(a, k16 * 32), smem_desc_sw128(b, k16 * 32), idesc, kb > 0 || j > 0 || k16 > 0);
                    }
                    mma_commit_pair(smem_u32(&empty_bar[s]));   // the stage is free in both CTAs once these MMAs have read it
                }
                mma_commit_pair(smem_u32(&acc_full[buf]));      // both halves of this tile's accumulator are complete
            }
        }
    } else {                                                // ---- epilogue (both CTAs): TMEM lanes by warp % 4
        const int q = warp & 3;
        const unsigned acc_empty_leader0 = map_to_cta(smem_u32(&acc_empty[0]), 0);
        const unsigned acc_empty_leader1 = map_to_cta(smem_u32(&acc_empty[1]), 0);
        int local = 0;
        for (int tile = pair; tile < tiles; tile += pairs, ++local) {
            int mt, nt;
            pair_tile_coords(tile, m_tiles, n_tiles, mt, nt);
            const int m0 = mt * 2 * BM + (int)rank * BM, n0 = nt * PR_BN;
            const int buf = local & 1;
            ok = mbar_wait(smem_u32(&acc_full[buf]), (local >> 1) & 1) && ok;
            if (tile + pairs >= tiles) pdl_trigger_late();                 // the last tile of this CTA
            fence_after_sync();
            const int m = m0 + q * 32 + lane;
#pragma unroll 1
            for (int c0 = 0; c0 < PR_BN; c0 += 32) {
                unsigned r[32];
                tmem_ld32(tacc + ((unsigned)(q * 32) << 16) + buf * PR_BN + c0, r);
                tmem_ld_wait();
                if (m >= M || n0 + c0 >= N) continue;
                if (GATED) {
                    // columns come in blocks of 8 gate values and their 8 up values: 32 columns give 16 outputs
                    TOut* dst = out + (size_t)m * ldo + ((n0 + c0) >> 1);
                    const int valid = min(16, (N - n0 - c0) >> 1);
                    float g[16];
#pragma unroll
                    for (int b = 0; b < 2; ++b)
#pragma unroll
                        for (int j = 0; j < 8; ++j) {
                            const float gate = __uint_as_float(r[b * 16 + j]), up = __uint_as_float(r[b * 16 + 8 + j]);
                            g[b * 8 + j] = __fdividef(gate, 1.0f + __expf(-gate)) * up;
                        }
                    if (valid == 16 && sizeof(TOut) == 2 && (reinterpret_cast<uintptr_t>(dst) & 15) == 0) {
#pragma unroll
                        for (int j = 0; j < 16; j += 8) {
                            uint4 v;
                            __nv_bfloat162 p0 = __floats2bfloat162_rn(g[j], g[j + 1]), p1 = __floats2bfloat162_rn(g[j + 2], g[j + 3]);
                            __nv_bfloat162 p2 = __floats2bfloat162_rn(g[j + 4], g[j + 5]), p3 = __floats2bfloat162_rn(g[j + 6], g[j + 7]);
                            v.x = *reinterpret_cast<unsigned*>(&p0); v.y = *reinterpret_cast<unsigned*>(&p1);
                            v.z = *reinterpret_cast<unsigned*>(&p2); v.w = *reinterpret_cast<unsigned*>(&p3);
                            *reinterpret_cast<uint4*>(reinterpret_cast<bf16*>(dst) + j) = v;
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 16; ++j)
                            if (j < valid) dst[j] = from_f32<TOut>(g[j]);
                    }
                } else {
                    store_row_chunk(out + (size_t)m * ldo + n0 + c0, r, min(32, N - n0 - c0));
                }
            }
            fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive_in_cluster(buf ? acc_empty_leader1 : acc_empty_leader0);   // this warp has drained its quarter
        }
    }
    if (!ok) atomicExch(status, 1);
    __syncwarp();
    fence_before_sync();
    cluster_sync_all();                                     // neither CTA leaves, or gives its tensor memory back, while the other works
    if (warp == 1) tmem_dealloc_pair(tacc, TMEM_COLS);
}

// ------------------------------------------------------------------------------------ host side
template <int BN, int STAGES, int KPS, typename TOut, bool GATED>
int launch_tc5(const void* x, const void* w, void* out, int M, int N, int K, int ldx, int ldw, int ldo, int* status,
               cudaStream_t st) {
    CUtensorMap mx, mw;
    if (!tma::make_map_bf16(&mx, x, M, K, ldx, BM) || !tma::make_map_bf16(&mw, w, N, K, ldw, BN)) return (int)cudaErrorInvalidValue;
    const size_t smem = (size_t)STAGES * KPS * (BM + BN) * BK * 2 + 1024;
    static PerDevice configured;
    const int rc = configured.once([&](int) {
        return cudaFuncSetAttribute(tc5_gemm_kernel<BN, STAGES, KPS, TOut, GATED>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    });
    if (rc != 0) return rc;
    const int tiles = ((N + BN - 1) / BN) * ((M + BM - 1) / BM);
    const int num_sms = rb_num_sms();
    if (num_sms <= 0) return (int)cudaErrorInvalidDevice;
    dim3 grid(tiles < num_sms ? tiles : num_sms);
    return rb_launch_pdl(tc5_gemm_kernel<BN, STAGES, KPS, TOut, GATED>, grid, dim3(TC5_THREADS), smem, st, mx, mw,
                         (TOut*)out, M, N, K, ldo, status);
}

template <typename TOut, bool GATED>
int launch_pair(const void* x, const void* w, void* out, int M, int N, int K, int ldx, int ldw, int ldo, int* status,
                cudaStream_t st) {
    CUtensorMap mx, mw;
    if (!tma::make_map_bf16(&mx, x, M, K, ldx, BM) || !tma::make_map_bf16(&mw, w, N, K, ldw, PR_HALF)) return (int)cudaErrorInvalidValue;
    const size_t smem = (size_t)PR_STAGES * PR_STAGE_BYTES + 1024;
    // pairs that the device holds at once (an SM whose neighbour is switched off takes none)
    static PerDevice configured;
    static int pairs_of_device[PerDevice::MAX_DEVICES] = {0};
    const int rc = configured.once([&](int dev) {
        cudaError_t e = cudaFuncSetAttribute(tc5_gemm_pair_kernel<TOut, GATED>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return e;
        cudaLaunchConfig_t probe = {};
        probe.gridDim = dim3(2);
        probe.blockDim = dim3(TC5_THREADS);
        probe.dynamicSmemBytes = smem;
        cudaLaunchAttribute pa[1];
        pa[0].id = cudaLaunchAttributeClusterDimension;
        pa[0].val.clusterDim.x = 2;
        pa[0].val.clusterDim.y = 1;
        pa[0].val.clusterDim.z = 1;
        probe.attrs = pa;
        probe.numAttrs = 1;
        int clusters = 0;
        e = cudaOccupancyMaxActiveClusters(&clusters, tc5_gemm_pair_kernel<TOut, GATED>, &probe);
        if (e != cudaSuccess) return e;
        if (clusters < 1) return cudaErrorInvalidConfiguration;
        pairs_of_device[dev] = clusters;
        return cudaSuccess;
    });
    if (rc != 0) return rc;
    int dev = 0;
    cudaGetDevice(&dev);
    const int resident = pairs_of_device[dev];
    const int tiles = ((N + PR_BN - 1) / PR_BN) * ((M + 2 * BM - 1) / (2 * BM));
    const int pairs = tiles < resident ? tiles : resident;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(2 * pairs);
    cfg.blockDim = dim3(TC5_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = RB_PDL_MODE == 3 ? 1 : 2;
    return (int)cudaLaunchKernelEx(&cfg, tc5_gemm_pair_kernel<TOut, GATED>, mx, mw, (TOut*)out, M, N, K, ldo, status);
}

}  // namespace

// out dtype: 0 bfloat16, 1 float32.  gated: SwiGLU epilogue over woven gate/up columns (out is [M, N/2]).
// status: one int in device memory, set to 1 if a wait inside the kernel gave up (zero it beforehand).
RB_EXPORT int rb_tc5_gemm(const void* x, const void* w, void* out, int out_f32, int gated, int M, int N, int K,
                          int ldx, int ldw, int ldo, int* status, cudaStream_t st) {
    if (M <= 0 || N <= 0) return 0;
    if (K % 8 || ldx % 8 || ldw % 8 || ((uintptr_t)x % 16) || ((uintptr_t)w % 16)) return (int)cudaErrorInvalidValue;
    if (gated) {
        if (out_f32 || N % 16) return (int)cudaErrorInvalidValue;
        return launch_tc5<256, TC5_STAGES, TC5_KPS, bf16, true>(x, w, out, M, N, K, ldx, ldw, ldo, status, st);
    }
    if (out_f32) return launch_tc5<256, TC5_STAGES, TC5_KPS, float, false>(x, w, out, M, N, K, ldx, ldw, ldo, status, st);
    return launch_tc5<256, TC5_STAGES, TC5_KPS, bf16, false>(x, w, out, M, N, K, ldx, ldw, ldo, status, st);
}

RB_EXPORT int rb_tc5_gemm_simple(const void* x, const void* w, void* out, int out_f32, int bn, int M, int N, int K,
                                 int ldx, int ldw, int ldo, int* status, cudaStream_t st) {
    if (M <= 0 || N <= 0) return 0;
    if (K % 8 || ldx % 8 || ldw % 8) return (int)cudaErrorInvalidValue;
    dim3 grid((N + bn - 1) / bn, (M + BM - 1) / BM);
    const size_t smem = (size_t)(BM + bn) * 128 + 1024;
#define RB_SIMPLE(BN_, T_)                                                                                           \
    {                                                                                                                \
        cudaFuncSetAttribute(tc5_gemm_simple_kernel<BN_, T_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        tc5_gemm_simple_kernel<BN_, T_><<<grid, 128, smem, st>>>((const bf16*)x, (const bf16*)w, (T_*)out, M, N, K,  \
                                                                 ldx, ldw, ldo, status);                             \
        return rb_launch_status();                                                                                   \
    }
    if (bn == 64 && out_f32) RB_SIMPLE(64, float)
    if (bn == 64) RB_SIMPLE(64, bf16)
    if (bn == 128 && out_f32) RB_SIMPLE(128, float)
    if (bn == 128) RB_SIMPLE(128, bf16)
    if (bn == 256 && out_f32) RB_SIMPLE(256, float)
    if (bn == 256) RB_SIMPLE(256, bf16)
#undef RB_SIMPLE
    return (int)cudaErrorInvalidValue;
}

// out[M, N] (float32) = x[M, K] * b[K, N] with b row-major: the MN-major-B twin.  bn in {64, 128, 256}, K % 64 == 0, N % 8 == 0.
RB_EXPORT int rb_tc5_gemm_bmn(const void* x, const void* b, float* out, int bn, int M, int N, int K, int ldx, int ldb,
                              int ldo, int* status, cudaStream_t st) {
    if (M <= 0 || N <= 0) return 0;
    if (K % 64 || N % 8 || ldx % 8 || ldb % 8) return (int)cudaErrorInvalidValue;
    dim3 grid((N + bn - 1) / bn, (M + BM - 1) / BM);
    const size_t smem = (size_t)BM * 128 + (size_t)bn * 128 + 1024;
#define RB_BMN(BN_)                                                                                                   \
    {                                                                                                                 \
        cudaFuncSetAttribute(tc5_gemm_bmn_kernel<BN_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);       \
        tc5_gemm_bmn_kernel<BN_><<<grid, 128, smem, st>>>((const bf16*)x, (const bf16*)b, out, M, N, K, ldx, ldb, ldo, \
                                                          status);                                              \
        return rb_launch_status();                                                                                    \
    }
    if (bn == 64) RB_BMN(64)
    if (bn == 128) RB_BMN(128)
    if (bn == 256) RB_BMN(256)
#undef RB_BMN
    return (int)cudaErrorInvalidValue;
}

// The same product by pairs of CTAs on 256 x 256 tiles (two-SM MMAs); same arguments as rb_tc5_gemm.
RB_EXPORT int rb_tc5_gemm_pair(const void* x, const void* w, void* out, int out_f32, int gated, int M, int N, int K,
                               int ldx, int ldw, int ldo, int* status, cudaStream_t st) {
    if (M <= 0 || N <= 0) return 0;
    if (K % 8 || ldx % 8 || ldw % 8 || ((uintptr_t)x % 16) || ((uintptr_t)w % 16)) return (int)cudaErrorInvalidValue;
    if (gated) {
        if (out_f32 || N % 16) return (int)cudaErrorInvalidValue;
        return launch_pair<bf16, true>(x, w, out, M, N, K, ldx, ldw, ldo, status, st);
    }
    if (out_f32) return launch_pair<float, false>(x, w, out, M, N, K, ldx, ldw, ldo, status, st);
    return launch_pair<bf16, false>(x, w, out, M, N, K, ldx, ldw, ldo, status, st);
}
