// Paged causal attention for prompt portions on the fifth-generation tensor cores (tcgen05), compiled
// for one head size: -DHEAD_DIM=64 or 128.
//
// One CTA owns 128 query rows of one segment and one query head.  Per tile of 64 keys:
//   S = Q K^T     tcgen05.mma, M = 128, N = 64, both operands K-major in shared memory, S in TMEM;
//   softmax       128 threads, one query row each (its TMEM lane): tcgen05.ld of the row, scale, mask,
//                 running maximum and sum in float32 with no shuffles, P rounded to bfloat16 into
//                 shared memory as the next MMA's A operand; the O accumulator is rescaled in TMEM
//                 (tcgen05.ld / st) only when a row's maximum moved;
//   O += P V      tcgen05.mma, M = 128, N = head dim, V as it lies in the cache (rows = keys): an
//                 MN-major B operand.
// One thread issues the MMAs; completion comes back through mbarriers (tcgen05.commit).  K and V
// tiles are gathered page by page with cp.async into the 128-byte-swizzled layout the MMA reads
// (keys outside the visible range, or on a page that was given back, are zero-filled, never read).
// 100 KB of shared memory and 256 TMEM columns a CTA: two CTAs share an SM, so one's softmax
// overlaps the other's MMAs.  Same contract as the reference's prefill kernel
// (rollout/attention.py:45-142) and as attention_mma.cu; keys arrive rotated, tiles are aligned to
// absolute positions, a sliding window bounds the keys from below.
// Every wait is bounded (tc5.cuh); *status is raised if one gave up.
#include "tc5.cuh"

#ifndef HEAD_DIM
#error "compile with -DHEAD_DIM=64 or -DHEAD_DIM=128"
#endif
static_assert(HEAD_DIM == 64 || HEAD_DIM == 128, "the tcgen05 attention kernel takes head sizes 64 and 128");

namespace {

using namespace tc5;

constexpr int D = HEAD_DIM;
constexpr int DS = D / 64;                    // 64-wide slabs of the head dim
constexpr int QM = 128;                       // query rows per CTA
constexpr int KN = 64;                        // keys per tile
constexpr int BT_CAP = 1024;                  // block-table entries staged in shared memory
constexpr int THREADS = 160;                  // warps 0..3: one query row per thread; warp 4: MMA issuer
constexpr unsigned Q_BYTES = DS * QM * 128, K_BYTES = DS * KN * 128, P_BYTES = QM * 128;
constexpr unsigned SMEM_BYTES = Q_BYTES + K_BYTES + 2 * K_BYTES + P_BYTES + BT_CAP * 4 + 1024;
constexpr unsigned TMEM_COLS = 256;           // S: 64 columns, O: HEAD_DIM columns
constexpr unsigned S_COL = 0, O_COL = 64;
constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ void cp_async16(unsigned smem_addr, const void* gmem, bool pred) {
    const int bytes = pred ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_addr), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

struct Paging {
    int page_size, shift;
    __device__ __forceinline__ explicit Paging(int p) : page_size(p), shift(-1) {
        if ((p & (p - 1)) == 0) {
            shift = 0;
            while ((1 << shift) < p) ++shift;
        }
    }
    __device__ __forceinline__ int block(int j) const { return shift >= 0 ? j >> shift : j / page_size; }
    __device__ __forceinline__ int row(int j) const { return shift >= 0 ? j & (page_size - 1) : j % page_size; }
};

__global__ void __launch_bounds__(THREADS)
attn_prefill_tc5_kernel(const bf16* __restrict__ q, int ld, const bf16* __restrict__ kpool,
                        const bf16* __restrict__ vpool, const int* __restrict__ tiles,
                        const int* __restrict__ cu_q, const int* __restrict__ seg_pos0,
                        const int* __restrict__ block_table, int bt_stride, int page_size,
                        bf16* __restrict__ out, int Hq, int Hkv, float scale_log2, int window,
                        int* __restrict__ status) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    unsigned char* sQ = base;
    unsigned char* sK = sQ + Q_BYTES;
    unsigned char* sV = sK + K_BYTES;                     // two buffers
    unsigned char* sP = sV + 2 * K_BYTES;
    int* sBT = reinterpret_cast<int*>(sP + P_BYTES);
    __shared__ __align__(8) unsigned long long bar_s_full, bar_p_ready, bar_pv_done;
    __shared__ unsigned tmem_slot;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int h = blockIdx.y, kvh = h / (Hq / Hkv);
    const int seg = tiles[2 * blockIdx.x], row0 = tiles[2 * blockIdx.x + 1];
    const int q_begin = cu_q[seg];
    const int m_rows = min(QM, cu_q[seg + 1] - q_begin - row0);
    const int p0 = seg_pos0[seg] + row0;                  // position of the tile's first query
    const int p_last = p0 + m_rows - 1;
    const int lo_min = window > 0 ? max(0, p0 - window + 1) : 0;
    const int jt_begin = lo_min / KN, n_tiles = p_last / KN - jt_begin + 1;
    const int* bt_row = block_table + (size_t)seg * bt_stride;
    const Paging pg(page_size);
    const unsigned s_full = smem_u32(&bar_s_full), p_ready = smem_u32(&bar_p_ready), pv_done = smem_u32(&bar_pv_done);

    if (warp == 4) tmem_alloc(smem_u32(&tmem_slot), TMEM_COLS);
    if (tid == 0) {
        mbar_init(s_full, 1);
        mbar_init(p_ready, 128);
        mbar_init(pv_done, 1);
        mbar_init_fence();
    }
    const int bt_first = pg.block(lo_min), bt_count = min(BT_CAP, pg.block(p_last) - bt_first + 1);
    for (int i = tid; i < bt_count; i += THREADS) sBT[i] = bt_row[bt_first + i];
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const unsigned tmem = tmem_slot;
    bool ok = true;

    if (warp < 4) {
        // ================================================================== one query row per thread
        const int r = tid;
        const int pos_r = p0 + r;
        const bool row_valid = r < m_rows;
        // K/V gather: two threads a key row, each half of the row's 16-byte chunks
        constexpr int CPT = D / 16;                       // chunks per thread
        const int krow = tid >> 1, c_first = (tid & 1) * CPT;
        auto issue_kv = [&](unsigned tile_smem, const bf16* pool, int jt) {
            const int j = jt * KN + krow;
            bool pred = j >= lo_min && j <= p_last;
            const bf16* src = pool;
            if (pred) {
                const int blk = pg.block(j), i = blk - bt_first;
                const int page = i < bt_count ? sBT[i] : bt_row[blk];
                pred = page >= 0;
                if (pred) src = pool + (((size_t)page * Hkv + kvh) * pg.page_size + pg.row(j)) * D;
            }
#pragma unroll
            for (int c = 0; c < CPT; ++c) {
                const int cc = c_first + c;
                cp_async16(tile_smem + (cc >> 3) * (KN * 128) + sw128_offset(krow, cc & 7), pred ? src + cc * 8 : pool, pred);
            }
        };
        // ---- prologue: this row of Q, the first K and V tiles
        {
            const bf16* qrow = q + (size_t)(q_begin + row0 + r) * ld + (size_t)h * D;
#pragma unroll
            for (int c = 0; c < D / 8; ++c) {
                uint4 v = make_uint4(0u, 0u, 0u, 0u);
                if (row_valid) v = *reinterpret_cast<const uint4*>(qrow + c * 8);
                *reinterpret_cast<uint4*>(sQ + (c >> 3) * (QM * 128) + sw128_offset(r, c & 7)) = v;
            }
        }
        issue_kv(smem_u32(sK), kpool, jt_begin);
        cp_async_commit();
        issue_kv(smem_u32(sV), vpool, jt_begin);
        cp_async_commit();
        cp_async_wait<0>();
        fence_proxy_async();
        mbar_arrive(p_ready);                             // phase 0: the operands of the first tile are in place

        float m_run = -INFINITY, l_run = 0.f;
        for (int t = 0; t < n_tiles; ++t) {
            const int jt = jt_begin + t;
            ok = mbar_wait(s_full, t & 1) && ok;          // S(t) is complete, so the K buffer is free
            fence_after_sync();
            if (t + 1 < n_tiles) issue_kv(smem_u32(sK), kpool, jt + 1);
            cp_async_commit();

            unsigned sr[64];
            {
                unsigned a[32], b[32];
                tmem_ld32(tmem + ((unsigned)(warp * 32) << 16) + S_COL, a);
                tmem_ld32(tmem + ((unsigned)(warp * 32) << 16) + S_COL + 32, b);
                tmem_ld_wait();
#pragma unroll
                for (int i = 0; i < 32; ++i) { sr[i] = a[i]; sr[32 + i] = b[i]; }
            }
            const int j_base = jt * KN;
            float mx = -INFINITY;
            const bool all_visible = j_base + KN - 1 <= p0 && (window <= 0 || j_base > p_last - window) && m_rows == QM;
            if (all_visible) {
#pragma unroll
                for (int i = 0; i < 64; ++i) {
                    const float v = __uint_as_float(sr[i]) * scale_log2;
                    sr[i] = __float_as_uint(v);
                    mx = fmaxf(mx, v);
                }
            } else {
#pragma unroll
                for (int i = 0; i < 64; ++i) {
                    const int j = j_base + i;
                    const bool vis = row_valid && j <= pos_r && (window <= 0 || j > pos_r - window);
                    const float v = vis ? __uint_as_float(sr[i]) * scale_log2 : -INFINITY;
                    sr[i] = __float_as_uint(v);
                    mx = fmaxf(mx, v);
                }
            }
            const float m_new = fmaxf(m_run, mx);
            const float mu = m_new == -INFINITY ? 0.f : m_new;
            const float alpha = fast_exp2(m_run - mu);
            float sum = 0.f;
#pragma unroll
            for (int i = 0; i < 64; ++i) {
                const float p = fast_exp2(__uint_as_float(sr[i]) - mu);
                sr[i] = __float_as_uint(p);
                sum += p;
            }
            l_run = l_run * alpha + sum;
            const bool moved = m_new != m_run;
            m_run = m_new;

            if (t > 0) ok = mbar_wait(pv_done, (t - 1) & 1) && ok;    // O, P and the other V buffer are free
            fence_after_sync();
            if (t + 1 < n_tiles) issue_kv(smem_u32(sV) + ((t + 1) & 1) * K_BYTES, vpool, jt + 1);
            cp_async_commit();

            if (t > 0 && __any_sync(0xffffffffu, moved)) {            // rescale this row of O in tensor memory
#pragma unroll 1
                for (int c0 = 0; c0 < D; c0 += 32) {
                    unsigned o[32];
                    const unsigned addr = tmem + ((unsigned)(warp * 32) << 16) + O_COL + c0;
                    tmem_ld32(addr, o);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                    tmem_st32(addr, o);
                }
                tmem_st_wait();
            }
            // P, rounded to bfloat16, as the A operand of the next MMA: this thread's row, 8 chunks of 8 keys
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                uint4 v;
                __nv_bfloat162 p0 = __floats2bfloat162_rn(__uint_as_float(sr[8 * c]), __uint_as_float(sr[8 * c + 1]));
                __nv_bfloat162 p1 = __floats2bfloat162_rn(__uint_as_float(sr[8 * c + 2]), __uint_as_float(sr[8 * c + 3]));
                __nv_bfloat162 p2 = __floats2bfloat162_rn(__uint_as_float(sr[8 * c + 4]), __uint_as_float(sr[8 * c + 5]));
                __nv_bfloat162 p3 = __floats2bfloat162_rn(__uint_as_float(sr[8 * c + 6]), __uint_as_float(sr[8 * c + 7]));
                v.x = *reinterpret_cast<unsigned*>(&p0); v.y = *reinterpret_cast<unsigned*>(&p1);
                v.z = *reinterpret_cast<unsigned*>(&p2); v.w = *reinterpret_cast<unsigned*>(&p3);
                *reinterpret_cast<uint4*>(sP + sw128_offset(r, c)) = v;
            }
            cp_async_wait<1>();                            // K(t+1) and V(t) have landed; V(t+1) may still fly
            fence_proxy_async();
            fence_before_sync();
            mbar_arrive(p_ready);                          // phase t+1
        }
        ok = mbar_wait(pv_done, (n_tiles - 1) & 1) && ok;
        fence_after_sync();
        cp_async_wait<0>();
        const float inv = 1.f / l_run;
        bf16* orow = out + (size_t)(q_begin + row0 + r) * ((size_t)Hq * D) + (size_t)h * D;
#pragma unroll 1
        for (int c0 = 0; c0 < D; c0 += 32) {
            unsigned o[32];
            tmem_ld32(tmem + ((unsigned)(warp * 32) << 16) + O_COL + c0, o);
            tmem_ld_wait();
            if (row_valid) {
#pragma unroll
                for (int i = 0; i < 32; i += 8) {
                    uint4 v;
                    __nv_bfloat162 a0 = __floats2bfloat162_rn(__uint_as_float(o[i]) * inv, __uint_as_float(o[i + 1]) * inv);
                    __nv_bfloat162 a1 = __floats2bfloat162_rn(__uint_as_float(o[i + 2]) * inv, __uint_as_float(o[i + 3]) * inv);
                    __nv_bfloat162 a2 = __floats2bfloat162_rn(__uint_as_float(o[i + 4]) * inv, __uint_as_float(o[i + 5]) * inv);
                    __nv_bfloat162 a3 = __floats2bfloat162_rn(__uint_as_float(o[i + 6]) * inv, __uint_as_float(o[i + 7]) * inv);
                    v.x = *reinterpret_cast<unsigned*>(&a0); v.y = *reinterpret_cast<unsigned*>(&a1);
                    v.z = *reinterpret_cast<unsigned*>(&a2); v.w = *reinterpret_cast<unsigned*>(&a3);
                    *reinterpret_cast<uint4*>(orow + c0 + i) = v;
                }
            }
        }
    } else if (lane == 0) {
        // ================================================================== the MMA issuer
        const unsigned idesc_s = instr_desc_bf16(QM, KN, false);
        const unsigned idesc_o = instr_desc_bf16(QM, D, true);
        const unsigned aQ = smem_u32(sQ), aK = smem_u32(sK), aV = smem_u32(sV), aP = smem_u32(sP);
        auto issue_s = [&]() {
#pragma unroll
            for (int d16 = 0; d16 < D / 16; ++d16)
                mma_ss(tmem + S_COL, smem_desc_sw128(aQ + (d16 >> 2) * (QM * 128), (d16 & 3) * 32),
                       smem_desc_sw128(aK + (d16 >> 2) * (KN * 128), (d16 & 3) * 32), idesc_s, d16 > 0);
            mma_commit(s_full);
        };
        ok = mbar_wait(p_ready, 0) && ok;                  // Q, K(0), V(0) are in shared memory
        fence_after_sync();
        issue_s();
        for (int t = 0; t < n_tiles; ++t) {
            ok = mbar_wait(p_ready, (t + 1) & 1) && ok;    // P(t) written, O rescaled, V(t) and K(t+1) landed
            fence_after_sync();
            const unsigned v_tile = aV + (t & 1) * K_BYTES;
#pragma unroll
            for (int k16 = 0; k16 < KN / 16; ++k16)
                mma_ss(tmem + O_COL, smem_desc_sw128(aP, k16 * 32),
                       smem_desc_sw128_mn(v_tile + k16 * 2048, KN * 128, 1024u), idesc_o, t > 0 || k16 > 0);
            mma_commit(pv_done);
            if (t + 1 < n_tiles) issue_s();
        }
    }
    if (!ok) atomicExch(status, 1);
    fence_before_sync();
    __syncthreads();
    if (warp == 4) tmem_dealloc(tmem, TMEM_COLS);
}

}  // namespace

RB_EXPORT int rb_attn_tc5_head_dim() { return D; }

// tiles: [n_tiles, 2] = (segment, first row of a block of up to 128 query rows).
RB_EXPORT int rb_attn_prefill_tc5(const void* q, int ld, const void* kpool, const void* vpool, const int* tiles,
                                  int n_tiles, const int* cu_q, const int* seg_pos0, const int* block_table,
                                  int bt_stride, int page_size, void* out, int Hq, int Hkv, float scale, int window,
                                  int* status, cudaStream_t st) {
    if (n_tiles <= 0) return 0;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attn_prefill_tc5_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES);
        if (e != cudaSuccess) return (int)e;
        configured = true;
    }
    dim3 grid(n_tiles, Hq);
    attn_prefill_tc5_kernel<<<grid, THREADS, SMEM_BYTES, st>>>(
        (const bf16*)q, ld, (const bf16*)kpool, (const bf16*)vpool, tiles, cu_q, seg_pos0, block_table, bt_stride,
        page_size, (bf16*)out, Hq, Hkv, scale * LOG2E, window, status);
    return rb_launch_status();
}
