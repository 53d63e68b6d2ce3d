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
// Seven warps with fixed roles, tied together by mbarriers (every wait bounded, tc5.cuh):
//   warps 0-3  the softmax rows;
//   warp 4     one thread issues every MMA; S is double-buffered in TMEM, so S(t+1) is computed
//              while the rows work on S(t);
//   warp 5     gathers K tiles, warp 6 V tiles, page by page with cp.async into the
//              128-byte-swizzled layout the MMA reads (two buffers each; keys outside the visible
//              range, or on a page that was given back, are zero-filled, never read).
// 112 KB of shared memory and 256 TMEM columns a CTA: two CTAs share an SM.  Same contract as the
// reference's prefill kernel (rollout/attention.py:45-142) and as attention_mma.cu; keys arrive
// rotated, tiles are aligned to absolute positions, a sliding window bounds the keys from below.
// *status is raised if a wait gave up.
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
constexpr int THREADS = 224;                  // warps 0..3: one query row per thread; 4: MMA; 5: K loader; 6: V loader
constexpr unsigned Q_BYTES = DS * QM * 128, K_BYTES = DS * KN * 128, P_BYTES = QM * 128;
constexpr unsigned SMEM_BYTES = Q_BYTES + 2 * K_BYTES + 2 * K_BYTES + P_BYTES + 256;   // two CTAs must fit 228 KB
constexpr unsigned TMEM_COLS = 256;           // S: 2 x 64 columns, O: HEAD_DIM columns
constexpr unsigned S_COL = 0, O_COL = 128;
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

__global__ void __launch_bounds__(THREADS, 2)
attn_prefill_tc5_kernel(const bf16* __restrict__ q, int ld, const bf16* __restrict__ kpool,
                        const bf16* __restrict__ vpool, const int* __restrict__ tiles,
                        const int* __restrict__ cu_q, const int* __restrict__ seg_pos0,
                        const int* __restrict__ block_table, int bt_stride, int page_size,
                        bf16* __restrict__ out, int Hq, int Hkv, float scale_log2, int window,
                        int* __restrict__ status) {
    // The swizzled tiles need 1024-byte alignment.  The kernel has no static shared memory, so the
    // dynamic window starts at the CTA's shared base; should it ever not be aligned, the kernel
    // reports it and does nothing.
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    if ((smem_u32(smem_raw) & 1023u) != 0u) {
        if (threadIdx.x == 0) atomicExch(status, 2);
        return;
    }
    unsigned char* sQ = smem_raw;
    unsigned char* sK = sQ + Q_BYTES;                     // two buffers
    unsigned char* sV = sK + 2 * K_BYTES;                 // two buffers
    unsigned char* sP = sV + 2 * K_BYTES;
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(sP + P_BYTES);
    unsigned* tmem_slot = reinterpret_cast<unsigned*>(bars + 16);

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
    // barriers: [0,1] S buffer full, [2,3] K buffer loaded, [4,5] V buffer loaded, 6 P ready, 7 PV done, 8 Q ready,
    // [9,10] V buffer free.  Each barrier's next phase needs its waiter to have passed the current one, so a
    // parity wait can never fall two phases behind (the V loader has its own barrier for that reason: PV_DONE
    // moves on without it).
    const unsigned bar0 = smem_u32(bars);
    auto bar = [&](int i) { return bar0 + 8u * i; };
    constexpr int S_FULL = 0, K_READY = 2, V_READY = 4, P_READY = 6, PV_DONE = 7, Q_READY = 8, V_FREE = 9;

    if (warp == 4) tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
    if (tid == 0) {
        for (int i = 0; i < 6; ++i) mbar_init(bar(i), 1);
        mbar_init(bar(P_READY), 128);
        mbar_init(bar(PV_DONE), 1);
        mbar_init(bar(Q_READY), 128);
        mbar_init(bar(V_FREE), 1);
        mbar_init(bar(V_FREE + 1), 1);
        mbar_init_fence();
    }
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const unsigned tmem = *tmem_slot;
    bool ok = true;

    if (warp < 4) {
        // ================================================================== one query row per thread
        const int r = tid;
        const int pos_r = p0 + r;
        const bool row_valid = r < m_rows;
        {
            const bf16* qrow = q + (size_t)(q_begin + row0 + r) * ld + (size_t)h * D;
#pragma unroll
            for (int c = 0; c < D / 8; ++c) {
                uint4 v = make_uint4(0u, 0u, 0u, 0u);
                if (row_valid) v = *reinterpret_cast<const uint4*>(qrow + c * 8);
                *reinterpret_cast<uint4*>(sQ + (c >> 3) * (QM * 128) + sw128_offset(r, c & 7)) = v;
            }
        }
        fence_proxy_async();
        mbar_arrive(bar(Q_READY));

        float m_run = -INFINITY, l_run = 0.f;
        const unsigned lane_addr = tmem + ((unsigned)(warp * 32) << 16);
        for (int t = 0; t < n_tiles; ++t) {
            const int j_base = (jt_begin + t) * KN;
            const unsigned s_addr = lane_addr + S_COL + (t & 1) * KN;
            ok = mbar_wait(bar(S_FULL + (t & 1)), (t >> 1) & 1) && ok;
            fence_after_sync();
            const bool all_visible = j_base + KN - 1 <= p0 && (window <= 0 || j_base > p_last - window) && m_rows == QM;
            // pass 1: the row's maximum over the tile (two halves of 32 keys)
            float mx = -INFINITY;
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                unsigned a[32];
                tmem_ld32(s_addr + half * 32, a);
                tmem_ld_wait();
                if (all_visible) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) mx = fmaxf(mx, __uint_as_float(a[i]));
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const int j = j_base + half * 32 + i;
                        const bool vis = row_valid && j <= pos_r && (window <= 0 || j > pos_r - window);
                        if (vis) mx = fmaxf(mx, __uint_as_float(a[i]));
                    }
                }
            }
            mx *= scale_log2;                              // the scale is positive: max(scale * s) = scale * max(s)
            const float m_new = fmaxf(m_run, mx);
            const float mu = m_new == -INFINITY ? 0.f : m_new;
            const float alpha = fast_exp2(m_run - mu);
            const bool moved = m_new != m_run;
            m_run = m_new;

            if (t > 0) ok = mbar_wait(bar(PV_DONE), (t - 1) & 1) && ok;     // O and the P buffer are free
            fence_after_sync();
            if (t > 0 && __any_sync(0xffffffffu, moved)) {                  // rescale this row of O in tensor memory
#pragma unroll 1
                for (int c0 = 0; c0 < D; c0 += 32) {
                    unsigned o[32];
                    tmem_ld32(lane_addr + O_COL + c0, o);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                    tmem_st32(lane_addr + O_COL + c0, o);
                }
                tmem_st_wait();
            }
            // pass 2: p = 2^(scale * s - m), summed in float32, rounded to bfloat16 into the A operand of P V
            float sum = 0.f;
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                unsigned a[32];
                tmem_ld32(s_addr + half * 32, a);
                tmem_ld_wait();
                if (all_visible) {
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const float p = fast_exp2(fmaf(__uint_as_float(a[i]), scale_log2, -mu));
                        sum += p;
                        a[i] = __float_as_uint(p);
                    }
                } else {
#pragma unroll
                    for (int i = 0; i < 32; ++i) {
                        const int j = j_base + half * 32 + i;
                        const bool vis = row_valid && j <= pos_r && (window <= 0 || j > pos_r - window);
                        const float p = vis ? fast_exp2(fmaf(__uint_as_float(a[i]), scale_log2, -mu)) : 0.f;
                        sum += p;
                        a[i] = __float_as_uint(p);
                    }
                }
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    uint4 v;
                    __nv_bfloat162 q0 = __floats2bfloat162_rn(__uint_as_float(a[8 * c]), __uint_as_float(a[8 * c + 1]));
                    __nv_bfloat162 q1 = __floats2bfloat162_rn(__uint_as_float(a[8 * c + 2]), __uint_as_float(a[8 * c + 3]));
                    __nv_bfloat162 q2 = __floats2bfloat162_rn(__uint_as_float(a[8 * c + 4]), __uint_as_float(a[8 * c + 5]));
                    __nv_bfloat162 q3 = __floats2bfloat162_rn(__uint_as_float(a[8 * c + 6]), __uint_as_float(a[8 * c + 7]));
                    v.x = *reinterpret_cast<unsigned*>(&q0); v.y = *reinterpret_cast<unsigned*>(&q1);
                    v.z = *reinterpret_cast<unsigned*>(&q2); v.w = *reinterpret_cast<unsigned*>(&q3);
                    *reinterpret_cast<uint4*>(sP + sw128_offset(r, half * 4 + c)) = v;
                }
            }
            l_run = l_run * alpha + sum;
            fence_proxy_async();
            fence_before_sync();
            mbar_arrive(bar(P_READY));                     // S(t) is read, O is rescaled, P(t) is written
        }
        ok = mbar_wait(bar(PV_DONE), (n_tiles - 1) & 1) && ok;
        fence_after_sync();
        const float inv = 1.f / l_run;
        bf16* orow = out + (size_t)(q_begin + row0 + r) * ((size_t)Hq * D) + (size_t)h * D;
#pragma unroll 1
        for (int c0 = 0; c0 < D; c0 += 32) {
            unsigned o[32];
            tmem_ld32(lane_addr + O_COL + c0, o);
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
    } else if (warp == 4) {
        if (lane == 0) {
            // ============================================================== the MMA issuer
            const unsigned idesc_s = instr_desc_bf16(QM, KN, false);
            const unsigned idesc_o = instr_desc_bf16(QM, D, true);
            const unsigned aQ = smem_u32(sQ), aK = smem_u32(sK), aV = smem_u32(sV), aP = smem_u32(sP);
            auto issue_s = [&](int t) {                    // S(t) = Q K(t)^T into S buffer t & 1
                ok = mbar_wait(bar(K_READY + (t & 1)), (t >> 1) & 1) && ok;
                fence_after_sync();
                const unsigned k_tile = aK + (t & 1) * K_BYTES;
#pragma unroll
                for (int d16 = 0; d16 < D / 16; ++d16)
                    mma_ss(tmem + S_COL + (t & 1) * KN, smem_desc_sw128(aQ + (d16 >> 2) * (QM * 128), (d16 & 3) * 32),
                           smem_desc_sw128(k_tile + (d16 >> 2) * (KN * 128), (d16 & 3) * 32), idesc_s, d16 > 0);
                mma_commit(bar(S_FULL + (t & 1)));
            };
            ok = mbar_wait(bar(Q_READY), 0) && ok;
            fence_after_sync();
            issue_s(0);
            if (n_tiles > 1) issue_s(1);
            for (int t = 0; t < n_tiles; ++t) {
                ok = mbar_wait(bar(P_READY), t & 1) && ok;
                ok = mbar_wait(bar(V_READY + (t & 1)), (t >> 1) & 1) && ok;
                fence_after_sync();
                const unsigned v_tile = aV + (t & 1) * K_BYTES;
#pragma unroll
                for (int k16 = 0; k16 < KN / 16; ++k16)
                    mma_ss(tmem + O_COL, smem_desc_sw128(aP, k16 * 32),
                           smem_desc_sw128_mn(v_tile + k16 * 2048, KN * 128, 1024u), idesc_o, t > 0 || k16 > 0);
                mma_commit(bar(PV_DONE));
                mma_commit(bar(V_FREE + (t & 1)));
                if (t + 2 < n_tiles) issue_s(t + 2);       // its S buffer was read by the rows before P_READY(t)
            }
        }
    } else {
        // ================================================================== the loaders: warp 5 K, warp 6 V
        const bool is_k = warp == 5;
        const bf16* pool = is_k ? kpool : vpool;
        unsigned char* bufs = is_k ? sK : sV;
        for (int t = 0; t < n_tiles; ++t) {
            if (t >= 2) {
                // buffer t & 1 is free once S(t-2) (for K) or the P V product of tile t-2 (for V) is complete
                if (is_k) ok = mbar_wait(bar(S_FULL + (t & 1)), ((t - 2) >> 1) & 1) && ok;
                else ok = mbar_wait(bar(V_FREE + (t & 1)), ((t - 2) >> 1) & 1) && ok;
            }
            const unsigned tile_smem = smem_u32(bufs) + (t & 1) * K_BYTES;
            const int jt = jt_begin + t;
#pragma unroll 1
            for (int rr = 0; rr < KN; rr += 32) {          // a lane gathers the whole row of two keys
                const int krow = rr + lane;
                const int j = jt * KN + krow;
                bool pred = j >= lo_min && j <= p_last;
                const bf16* src = pool;
                if (pred) {
                    const int page = bt_row[pg.block(j)];
                    pred = page >= 0;
                    if (pred) src = pool + (((size_t)page * Hkv + kvh) * pg.page_size + pg.row(j)) * D;
                }
#pragma unroll
                for (int cc = 0; cc < D / 8; ++cc)
                    cp_async16(tile_smem + (cc >> 3) * (KN * 128) + sw128_offset(krow, cc & 7), pred ? src + cc * 8 : pool, pred);
            }
            cp_async_commit();
            cp_async_wait<0>();
            fence_proxy_async();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar((is_k ? K_READY : V_READY) + (t & 1)));
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
