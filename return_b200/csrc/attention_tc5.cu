// Paged causal attention for prompt portions on the fifth-generation tensor cores (tcgen05), compiled
// for one head size: -DHEAD_DIM=64 or 128.
//
// One CTA (one a SM) owns 256 query rows of one segment and one query head, as two tiles of 128 rows,
// A and B, that share every key tile the CTA loads.  Per tile of 64 keys and per query tile:
//   S = Q K^T     tcgen05.mma, M = 128, N = 64, both operands K-major in shared memory, S in TMEM
//                 (two buffers a query tile);
//   softmax       128 threads a query tile, one query row each (its TMEM lane): tcgen05.ld of the row
//                 once, scale, mask, maximum and sum in float32 with no shuffles, P rounded to bfloat16
//                 into shared memory as the next MMA's A operand.  The reference maximum of a row moves
//                 only when the true one has outrun it by 2^8, so the O accumulator is rescaled in
//                 TMEM (tcgen05.ld / st) a few times at most;
//   O += P V      tcgen05.mma, M = 128, N = head dim, V as it lies in the cache (rows = keys): an
//                 MN-major B operand.
// While the rows of A work on their scores, the tensor core computes B's, and so on in turn.
// Twelve warps with fixed roles, tied together by mbarriers (every wait bounded, tc5.cuh):
//   warps 0-3  the rows of query tile A, warps 4-7 those of B;
//   warp 8     one thread issues A's MMAs, warp 11 one thread B's, with descriptors that are a base plus a
//              constant.  An issuing thread is stopped while its MMAs wait for the tensor pipe, and pays some
//              230 cycles for every barrier wait, even one that succeeds at once, and 90 for every commit
//              (measured with a loop of MMAs alone), all of which adds up in one thread; so a key tile costs each of
//              the two threads two waits and two commits and no more: K(u) and V(u - 1) arrive on one barrier,
//              and the commits that tell the rows that S is there and that P V is done free the K and V
//              stages for the loaders as well;
//   warp 9     gathers K tiles, warp 10 V tiles, page by page with cp.async into the
//              128-byte-swizzled layout the MMA reads, through rings of three tiles each so that a
//              tile is asked for two tiles before it is needed (keys outside the visible range, or on
//              a page that was given back, are zero-filled, never read).
// P has two buffers a query tile, so the exponentials of tile t run while P V(t - 1) does; the rows wait for
// P V(t - 1) itself only when they have to rescale O.
// Every barrier's next phase needs all its waiters to have passed the current one: no parity wait can fall two
// phases behind.  That is why the barriers that a query tile's P and P V use come in pairs (tile & 1), and why
// a loader announces tile t - 1 only after it has waited for the stage of tile t.
// 224 KB of shared memory and all 512 TMEM columns a CTA (head size 128).  Same contract as the
// reference's prefill kernel (rollout/attention.py:45-142) and as attention_mma.cu; keys arrive
// rotated, tiles are aligned to absolute positions, a sliding window bounds the keys from below.
// A step with too few such CTAs to fill the GPU (a short portion of a long prompt) splits the keys of every
// block over gridDim.z CTAs; each leaves its unnormalised O with its reference maximum and sum in float32,
// and a second kernel merges them (the same arithmetic as the decode kernel's merge).
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
constexpr int QM = 128;                       // rows of a query tile
constexpr int NQ = 2;                         // query tiles per CTA
constexpr int KN = 64;                        // keys per tile
constexpr int STAGES = 3;                     // K tiles, and V tiles, in flight
constexpr int THREADS = 384;                  // warps 0..3: tile A's rows; 4..7: tile B's; 8: A's MMAs; 9: K loader; 10: V loader; 11: B's MMAs
constexpr int W_MMA = 8, W_K = 9, W_V = 10, W_MMA_B = 11;
constexpr float RESCALE_STEP = 8.0f;          // log2 units the true maximum may run ahead of the reference
constexpr unsigned Q_BYTES = DS * QM * 128, K_BYTES = DS * KN * 128, P_BYTES = QM * 128;
constexpr unsigned SMEM_USED = NQ * Q_BYTES + 2 * STAGES * K_BYTES + 2 * NQ * P_BYTES + 512;
// a CTA takes all of an SM's tensor memory, so it asks for more than half of its shared memory too
constexpr unsigned SMEM_BYTES = SMEM_USED > 120 * 1024 ? SMEM_USED : 120 * 1024;
constexpr unsigned TMEM_COLS = 512;           // S: 2 query tiles x 2 buffers x 64 columns; O: 2 x HEAD_DIM columns from 256
constexpr unsigned O_COL = 256;
constexpr float LOG2E = 1.4426950408889634f;

// barriers.  A thread that issues MMAs pays some 200 cycles for every wait, even one that succeeds at once, 90
// for every commit and 55 to 90 for every MMA, so each query tile has an issuing thread of its own, with two
// waits and two commits a key tile.
constexpr int B_KV_FULL = 0;                  // [stage]: K of tile u and V of tile u - 1 have landed, u % STAGES == stage (the two loaders)
constexpr int B_S_FULL = 3;                   // [query tile][S buffer]: S is computed (its issuer's commit); also frees the K stage
constexpr int B_P_READY = 7;                  // [query tile][tile & 1 = P buffer]: P is written (the tile's four warps of rows)
constexpr int B_PV_DONE = 11;                 // [query tile][tile & 1]: P V is done (its issuer's commit); also frees the V stage
constexpr int B_Q_READY = 15;
constexpr int N_BARS = 16;
static_assert(STAGES == 3, "the barrier numbering above is for rings of three");

__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}
// Two float32 operations an instruction (fma.rn.f32x2, add.rn.f32x2) and the three-input maximum: the rows are
// bound by the instructions they issue, and these halve the count of the arithmetic around the exponentials.
__device__ __forceinline__ unsigned long long pack2(float lo, float hi) {
    unsigned long long v;
    asm("mov.b64 %0, {%1, %2};" : "=l"(v) : "f"(lo), "f"(hi));
    return v;
}
__device__ __forceinline__ void unpack2(unsigned long long v, float& lo, float& hi) {
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ unsigned long long fma2(unsigned long long a, unsigned long long b, unsigned long long c) {
    unsigned long long d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ unsigned long long add2(unsigned long long a, unsigned long long b) {
    unsigned long long d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ float max3(float a, float b, float c) {
    float d;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
    return d;
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

__global__ void __launch_bounds__(THREADS, 1)
attn_prefill_tc5_kernel(const bf16* __restrict__ q, int ld, const bf16* __restrict__ kpool,
                        const bf16* __restrict__ vpool, const int* __restrict__ tiles,
                        const int* __restrict__ cu_q, const int* __restrict__ seg_pos0,
                        const int* __restrict__ block_table, int bt_stride, int page_size,
                        bf16* __restrict__ out, int Hq, int Hkv, float scale_log2, int window,
                        float* __restrict__ part_o, float* __restrict__ part_ml, int total_rows,
                        int* __restrict__ status) {
    // The swizzled tiles need 1024-byte alignment.  The kernel has no static shared memory, so the
    // dynamic window starts at the CTA's shared base; should it ever not be aligned, the kernel
    // reports it and does nothing.
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    if ((smem_u32(smem_raw) & 1023u) != 0u) {
        if (threadIdx.x == 0) atomicExch(status, 2);
        return;
    }
    unsigned char* sQ = smem_raw;                         // [query tile]
    unsigned char* sK = sQ + NQ * Q_BYTES;                // [stage]
    unsigned char* sV = sK + STAGES * K_BYTES;            // [stage]
    unsigned char* sP = sV + STAGES * K_BYTES;            // [query tile][P buffer]
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(sP + 2 * NQ * P_BYTES);
    unsigned* tmem_slot = reinterpret_cast<unsigned*>(bars + 32);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int h = blockIdx.x, kvh = h / (Hq / Hkv);       // heads run fastest: the heaviest tiles of all heads start first
    const int seg = tiles[2 * blockIdx.y], row0 = tiles[2 * blockIdx.y + 1];
    const int q_begin = cu_q[seg];
    const int m_rows = min(NQ * QM, cu_q[seg + 1] - q_begin - row0);
    const int p0 = seg_pos0[seg] + row0;                  // position of the CTA's first query
    const int p_last = p0 + m_rows - 1;
    const int lo_min = window > 0 ? max(0, p0 - window + 1) : 0;
    int jt_first = lo_min / KN;
    // key tiles of each query tile, counted from the first: B (if it has rows) needs all of the block's, A stops earlier
    int na = min(p_last, p0 + QM - 1) / KN - jt_first + 1;
    int nb = m_rows > QM ? p_last / KN - jt_first + 1 : 0;
    int nt = max(na, nb);
    const int n_split = gridDim.z, split = blockIdx.z;
    if (n_split > 1) {                                    // this CTA's share of the block's key tiles; it may be empty
        const int per = (nt + n_split - 1) / n_split;
        const int t0 = split * per;
        const int len = max(0, min(nt, t0 + per) - t0);
        jt_first += t0;
        na = min(max(na - t0, 0), len);
        nb = min(max(nb - t0, 0), len);
        nt = len;
    }
    const int jt_begin = jt_first, n_a = na, n_b = nb, n_tiles = nt;
    const int* bt_row = block_table + (size_t)seg * bt_stride;
    const Paging pg(page_size);
    const unsigned bar0 = smem_u32(bars);
    auto bar = [&](int i) { return bar0 + 8u * i; };

    if (warp == W_MMA) tmem_alloc(smem_u32(tmem_slot), TMEM_COLS);
    if (tid == 0) {
        for (int i = 0; i < N_BARS; ++i)
            mbar_init(bar(i), i < B_KV_FULL + STAGES ? 2 : i >= B_P_READY && i < B_P_READY + 2 * NQ ? 4 : i == B_Q_READY ? NQ * 4 : 1);
        mbar_init_fence();
    }
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const unsigned tmem = *tmem_slot;
    bool ok = true;

    if (warp < 2 * 4) {
        // ================================================================== one query row per thread
        const int qt = warp >> 2;                            // query tile A or B
        const int r = (warp & 3) * 32 + lane;                // row in the tile = TMEM lane
        const int grow = qt * QM + r;                        // row in the CTA
        const int pos_r = p0 + grow;
        const bool row_valid = grow < m_rows;
        const int n_mine = qt == 0 ? n_a : n_b;
        const int p0_t = p0 + qt * QM, p_last_t = min(p_last, p0_t + QM - 1);      // the tile's first and last position
        const bool full_tile = m_rows >= (qt + 1) * QM;
        unsigned char* myQ = sQ + qt * Q_BYTES;
        unsigned char* myPs = sP + qt * 2 * P_BYTES;           // this query tile's two P buffers
        {
            const bf16* qrow = q + (size_t)(q_begin + row0 + grow) * ld + (size_t)h * D;
#pragma unroll
            for (int c = 0; c < D / 8; ++c) {
                uint4 v = make_uint4(0u, 0u, 0u, 0u);
                if (row_valid) v = *reinterpret_cast<const uint4*>(qrow + c * 8);
                *reinterpret_cast<uint4*>(myQ + (c >> 3) * (QM * 128) + sw128_offset(r, c & 7)) = v;
            }
        }
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) mbar_arrive(bar(B_Q_READY));

        float m_ref = -INFINITY, l_run = 0.f;                // the reference maximum and the sum relative to it
        const unsigned lane_addr = tmem + ((unsigned)((warp & 3) * 32) << 16);
        const unsigned o_addr = lane_addr + O_COL + qt * D;
        for (int t = 0; t < n_mine; ++t) {
            const int j_base = (jt_begin + t) * KN;
            ok = mbar_wait(bar(B_S_FULL + qt * 2 + (t & 1)), (t >> 1) & 1) && ok;
            fence_after_sync();
            const bool all_visible = full_tile && j_base + KN - 1 <= p0_t && (window <= 0 || j_base > p_last_t - window);
            unsigned a[64];
            tmem_ld32(lane_addr + (qt * 2 + (t & 1)) * KN, reinterpret_cast<unsigned(&)[32]>(a[0]));
            tmem_ld32(lane_addr + (qt * 2 + (t & 1)) * KN + 32, reinterpret_cast<unsigned(&)[32]>(a[32]));
            tmem_ld_wait();
            float mx = -INFINITY;
            if (all_visible) {
#pragma unroll
                for (int i = 0; i < 64; i += 2) mx = max3(mx, __uint_as_float(a[i]), __uint_as_float(a[i + 1]));
            } else {
#pragma unroll
                for (int i = 0; i < 64; ++i) {
                    const int j = j_base + i;
                    const bool vis = row_valid && j <= pos_r && (window <= 0 || j > pos_r - window);
                    if (!vis) a[i] = 0xff800000u;            // -inf: 2^(-inf) = 0 below
                    mx = fmaxf(mx, __uint_as_float(a[i]));
                }
            }
            mx *= scale_log2;                                // the scale is positive: max(scale * s) = scale * max(s)
            // the reference moves only when the maximum has outrun it by RESCALE_STEP (or was -inf)
            float alpha = 1.f;
            bool moved = false;
            if (mx > m_ref + RESCALE_STEP || (m_ref == -INFINITY && mx != -INFINITY)) {
                alpha = fast_exp2(m_ref - mx);               // 0 on the first move
                m_ref = mx;
                moved = true;
            }
            const float mu = m_ref == -INFINITY ? 0.f : m_ref;

            // P(t) goes into the buffer that P V(t - 2) read, so the exponentials of this tile run while P V(t - 1)
            // does.  P V(t - 2) is done: the commit that announced S(t) came from the same thread after it, and
            // a commit stands for everything that thread issued before.  O may only be touched when P V(t - 1)
            // is done too, which the rows wait for only when they have to rescale it.  Tile t's P V commits
            // to barrier [t & 1], phase t >> 1.
            if (t > 0 && __any_sync(0xffffffffu, moved)) {                  // rescale this row of O in tensor memory
                ok = mbar_wait(bar(B_PV_DONE + qt * 2 + ((t - 1) & 1)), ((t - 1) >> 1) & 1) && ok;
                fence_after_sync();
#pragma unroll 1
                for (int c0 = 0; c0 < D; c0 += 32) {
                    unsigned o[32];
                    tmem_ld32(o_addr + c0, o);
                    tmem_ld_wait();
#pragma unroll
                    for (int i = 0; i < 32; ++i) o[i] = __float_as_uint(__uint_as_float(o[i]) * alpha);
                    tmem_st32(o_addr + c0, o);
                }
                tmem_st_wait();
            }
            unsigned char* myP = myPs + (t & 1) * P_BYTES;
            // p = 2^(scale * s - m), summed in float32, rounded to bfloat16 into the A operand of P V
            const unsigned long long scale2 = pack2(scale_log2, scale_log2), shift2 = pack2(-mu, -mu);
            unsigned long long sum2 = pack2(0.f, 0.f);
#pragma unroll
            for (int i = 0; i < 64; i += 2) {
                float x0, x1;
                unpack2(fma2(pack2(__uint_as_float(a[i]), __uint_as_float(a[i + 1])), scale2, shift2), x0, x1);
                const float p0 = fast_exp2(x0), p1 = fast_exp2(x1);
                sum2 = add2(sum2, pack2(p0, p1));
                a[i] = __float_as_uint(p0);
                a[i + 1] = __float_as_uint(p1);
            }
            float sum_lo, sum_hi;
            unpack2(sum2, sum_lo, sum_hi);
            const float sum = sum_lo + sum_hi;
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                uint4 v;
                __nv_bfloat162 q0 = __floats2bfloat162_rn(__uint_as_float(a[8 * c]), __uint_as_float(a[8 * c + 1]));
                __nv_bfloat162 q1 = __floats2bfloat162_rn(__uint_as_float(a[8 * c + 2]), __uint_as_float(a[8 * c + 3]));
                __nv_bfloat162 q2 = __floats2bfloat162_rn(__uint_as_float(a[8 * c + 4]), __uint_as_float(a[8 * c + 5]));
                __nv_bfloat162 q3 = __floats2bfloat162_rn(__uint_as_float(a[8 * c + 6]), __uint_as_float(a[8 * c + 7]));
                v.x = *reinterpret_cast<unsigned*>(&q0); v.y = *reinterpret_cast<unsigned*>(&q1);
                v.z = *reinterpret_cast<unsigned*>(&q2); v.w = *reinterpret_cast<unsigned*>(&q3);
                *reinterpret_cast<uint4*>(myP + sw128_offset(r, c)) = v;
            }
            l_run = l_run * alpha + sum;
            fence_proxy_async();
            fence_before_sync();
            __syncwarp();
            if (lane == 0) mbar_arrive(bar(B_P_READY + qt * 2 + (t & 1)));      // S(t) is read, O is rescaled, P(t) is written
        }
        if (n_mine > 0) {
            ok = mbar_wait(bar(B_PV_DONE + qt * 2 + ((n_mine - 1) & 1)), ((n_mine - 1) >> 1) & 1) && ok;
            fence_after_sync();
        }
        const size_t token = (size_t)(q_begin + row0 + grow);
        if (n_split > 1) {
            // one of several CTAs over this row's keys: O as it stands, with the reference maximum and the sum
            const size_t slot = ((size_t)split * total_rows + token) * Hq + h;
            if (row_valid) {
                part_ml[2 * slot] = n_mine > 0 ? m_ref : -INFINITY;
                part_ml[2 * slot + 1] = n_mine > 0 ? l_run : 0.f;
            }
            if (n_mine > 0) {
                float* prow = part_o + slot * D;
#pragma unroll 1
                for (int c0 = 0; c0 < D; c0 += 32) {
                    unsigned o[32];
                    tmem_ld32(o_addr + c0, o);
                    tmem_ld_wait();
                    if (row_valid) {
#pragma unroll
                        for (int i = 0; i < 32; i += 4)
                            *reinterpret_cast<uint4*>(prow + c0 + i) = make_uint4(o[i], o[i + 1], o[i + 2], o[i + 3]);
                    }
                }
            }
        } else if (n_mine > 0) {
            const float inv = 1.f / l_run;
            bf16* orow = out + token * ((size_t)Hq * D) + (size_t)h * D;
#pragma unroll 1
            for (int c0 = 0; c0 < D; c0 += 32) {
                unsigned o[32];
                tmem_ld32(o_addr + c0, o);
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
        }
    } else if (warp == W_MMA || warp == W_MMA_B) {
        const int qt = warp == W_MMA ? 0 : 1;
        const int n_q = qt == 0 ? n_a : n_b;                 // key tiles of this query tile: the first n_q of the CTA's
        if (lane == 0 && n_q > 0) {
            // ============================================================== the MMA issuer of one query tile
            // One thread's instruction latency is its pace, so every descriptor is a base worked out once plus a
            // constant, and stage, buffer and parity of the tile being issued are kept as running values.
            const unsigned idesc_s = instr_desc_bf16(QM, KN, false);
            const unsigned idesc_o = instr_desc_bf16(QM, D, true);
            const unsigned long long q_tile = smem_desc_sw128(smem_u32(sQ) + qt * Q_BYTES, 0), dK = smem_desc_sw128(smem_u32(sK), 0);
            const unsigned long long dP = smem_desc_sw128(smem_u32(sP) + qt * 2 * P_BYTES, 0);
            const unsigned long long dV = smem_desc_sw128_mn(smem_u32(sV), KN * 128, 1024u);
            const unsigned d_o = tmem + O_COL + qt * D;
            unsigned long long k_tile = dK, v_tile = dV;   // descriptors of the K stage of S's tile and the V stage of P V's tile
            unsigned kv_full = bar(B_KV_FULL), kv_par = 0;
            int kv_st = 0, v_st = 0;
            unsigned s_buf = 0;                            // S buffer of the tile being issued: u & 1
            // S(u) = Q K(u)^T once K(u) has landed; V(u - 1) has landed then too.  For u = n_q only the wait is left.
            auto issue_s = [&](int u) {
                ok = mbar_wait(kv_full, kv_par) && ok;
                fence_after_sync();
                if (u < n_q) {
                    const unsigned d_s = tmem + (qt * 2 + s_buf) * KN;
#pragma unroll
                    for (int d16 = 0; d16 < D / 16; ++d16)     // 64-wide slabs of the head dim, four steps of 16 (32 bytes) in each
                        mma_ss(d_s, q_tile + (unsigned long long)(((d16 >> 2) * (QM * 128) + (d16 & 3) * 32) >> 4),
                               k_tile + (unsigned long long)(((d16 >> 2) * (KN * 128) + (d16 & 3) * 32) >> 4), idesc_s, d16 > 0);
                    mma_commit(bar(B_S_FULL + qt * 2) + 8u * s_buf);    // the rows may read S; the K loader may reuse the stage
                    s_buf ^= 1u;
                }
                if (++kv_st == STAGES) {
                    kv_st = 0; kv_par ^= 1u;
                    k_tile = dK; kv_full = bar(B_KV_FULL);
                } else {
                    k_tile += (unsigned long long)(K_BYTES >> 4); kv_full += 8u;
                }
            };
            ok = mbar_wait(bar(B_Q_READY), 0) && ok;
            fence_after_sync();
            issue_s(0);
            unsigned p_par = 0;
            for (int t = 0; t < n_q; ++t) {
                // S(t+1) goes into the buffer that S(t-1) used: its rows were read before P(t-1) was ready
                issue_s(t + 1);
                ok = mbar_wait(bar(B_P_READY + qt * 2) + 8u * (unsigned)(t & 1), p_par) && ok;
                fence_after_sync();
                const unsigned long long p_tile = dP + (unsigned long long)((t & 1) * (P_BYTES >> 4));
                if (t == 0) mma_ss(d_o, p_tile, v_tile, idesc_o, false);
                else mma_ss(d_o, p_tile, v_tile, idesc_o, true);
#pragma unroll
                for (int k16 = 1; k16 < KN / 16; ++k16)    // 16 keys: 32 bytes along P's rows, 2048 bytes down V's
                    mma_ss(d_o, p_tile + (unsigned long long)(k16 * 2), v_tile + (unsigned long long)(k16 * 128), idesc_o, true);
                mma_commit(bar(B_PV_DONE + qt * 2) + 8u * (unsigned)(t & 1));      // the rows may touch O and P; the V loader may reuse the stage
                p_par ^= (unsigned)(t & 1);                 // each of the two barriers has a phase every other tile
                if (++v_st == STAGES) { v_st = 0; v_tile = dV; }
                else v_tile += (unsigned long long)(K_BYTES >> 4);
            }
        }
    } else {
        // ================================================================== the loaders: warp 9 K, warp 10 V
        const bool is_k = warp == W_K;
        const bf16* pool = is_k ? kpool : vpool;
        const unsigned bufs = smem_u32(is_k ? sK : sV);
        if (n_tiles > 0) {
        // K(u) and V(u - 1) arrive on the same barrier, stage u % STAGES; "V(-1)" and "K(n_tiles)" stand in at the ends.
        if (!is_k && lane == 0) mbar_arrive(bar(B_KV_FULL));
        int st = 0;
        // The pages of rows `lane` and `lane + 32` of a key tile are asked for one tile ahead and not looked at
        // until that tile's turn, so the look-up's latency passes while the loader copies and waits.
        auto ask_pages = [&](int jt, int (&page)[2]) {
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const int j = jt * KN + u * 32 + lane;
                page[u] = bt_row[j >= lo_min && j <= p_last ? pg.block(j) : 0];      // entry 0 exists; the range is checked again at use
            }
        };
        int next_page[2];
        ask_pages(jt_begin, next_page);
        for (int t = 0; t < n_tiles; ++t) {
            if (t >= STAGES) {
                // the stage held tile t - 3: its keys are free when S(t - 3) is computed, its values when P V(t - 3) is done
                const int f = t - STAGES;
                const int b_free = is_k ? B_S_FULL : B_PV_DONE;
                if (f < n_a) ok = mbar_wait(bar(b_free + (f & 1)), (f >> 1) & 1) && ok;
                if (f < n_b) ok = mbar_wait(bar(b_free + 2 + (f & 1)), (f >> 1) & 1) && ok;
            }
            const unsigned tile_smem = bufs + st * K_BYTES;
            const int jt = jt_begin + t;
            // Lane L looks up where rows L and L + 32 of the tile lie (a null pointer: not to be read).  The copies
            // then go row by row, D / 8 neighbouring lanes taking the 16-byte pieces of one row, so that a
            // warp's instruction reads whole 128-byte lines; each row's address comes from the lane that
            // looked it up.  (One lane a row, piece by piece, asked for 32 lines an instruction and took
            // 1,800 cycles a tile.)
            unsigned long long where[2];
#pragma unroll
            for (int u = 0; u < 2; ++u) {
                const int j = jt * KN + u * 32 + lane;
                where[u] = 0ull;
                if (j >= lo_min && j <= p_last && next_page[u] >= 0)
                    where[u] = reinterpret_cast<unsigned long long>(pool + (((size_t)next_page[u] * Hkv + kvh) * pg.page_size + pg.row(j)) * D);
            }
            constexpr int LPR = D / 8, RPI = 32 / LPR;              // lanes a row, rows an instruction
            const int sub = lane % LPR, rsel = lane / LPR;
            const unsigned piece = (unsigned)(sub >> 3) * (KN * 128), c7 = (unsigned)(sub & 7);
#pragma unroll
            for (int u = 0; u < 2; ++u) {
#pragma unroll
                for (int i = 0; i < 32 / RPI; ++i) {
                    const int owner = i * RPI + rsel;                 // the lane that looked this row up
                    const int krow = u * 32 + owner;
                    const unsigned long long w = __shfl_sync(0xffffffffu, where[u], owner);
                    const bf16* src = w ? reinterpret_cast<const bf16*>(w) + sub * 8 : pool;
                    cp_async16(tile_smem + (krow >> 3) * 1024 + (krow & 7) * 128 + piece + ((c7 ^ (unsigned)(krow & 7)) << 4), src, w != 0ull);
                }
            }
            cp_async_commit();
            if (t + 1 < n_tiles) ask_pages(jt + 1, next_page);
            // tile t is on its way; tile t - 1 has to have landed.  It is announced only now, after the wait for
            // the stage above: the product that completes the next phase of that wait's barrier needs this
            // announcement, so the wait cannot fall a phase behind.
            const int st_prev = st == 0 ? STAGES - 1 : st - 1;      // stage of tile t - 1
            if (t > 0) {
                cp_async_wait<1>();
                fence_proxy_async();
                __syncwarp();
                if (lane == 0) mbar_arrive(bar(B_KV_FULL + (is_k ? st_prev : st)));      // K(t-1): its own stage; V(t-1): the stage of K(t)
            }
            st = st + 1 == STAGES ? 0 : st + 1;
        }
        cp_async_wait<0>();
        fence_proxy_async();
        __syncwarp();
        if (lane == 0) {
            const int st_last = st == 0 ? STAGES - 1 : st - 1;      // stage of the last tile; st is that of "tile n_tiles"
            mbar_arrive(bar(B_KV_FULL + (is_k ? st_last : st)));
            if (is_k) mbar_arrive(bar(B_KV_FULL + st));
        }
        }
    }
    if (!ok) atomicExch(status, 1);
    fence_before_sync();
    __syncthreads();
    if (warp == W_MMA) tmem_dealloc(tmem, TMEM_COLS);
}

// out[row, h] = sum_s O_s 2^(m_s - M) / sum_s l_s 2^(m_s - M) over the splits of the keys: one warp a (row, head).
__global__ void __launch_bounds__(256)
merge_key_splits_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                        const int* __restrict__ tiles, const int* __restrict__ cu_q, int n_split, int total_rows,
                        int Hq, bf16* __restrict__ out) {
    const int seg = tiles[2 * blockIdx.y], row0 = tiles[2 * blockIdx.y + 1];
    const int q_begin = cu_q[seg];
    const int m_rows = min(NQ * QM, cu_q[seg + 1] - q_begin - row0);
    const int r = blockIdx.z * 8 + (threadIdx.x >> 5), lane = threadIdx.x & 31, h = blockIdx.x;
    if (r >= m_rows) return;
    const size_t token = (size_t)(q_begin + row0 + r);
    constexpr int PER = D / 32;                            // floats of a row a lane holds: 2 or 4
    float m_all = -INFINITY;
    for (int s = 0; s < n_split; ++s) m_all = fmaxf(m_all, part_ml[2 * (((size_t)s * total_rows + token) * Hq + h)]);
    float acc[PER] = {}, l_all = 0.f;
    for (int s = 0; s < n_split; ++s) {
        const size_t slot = ((size_t)s * total_rows + token) * Hq + h;
        const float l = part_ml[2 * slot + 1];
        if (l == 0.f) continue;                            // a share without keys for this row left no O
        const float wgt = fast_exp2(part_ml[2 * slot] - m_all);
        l_all += l * wgt;
        const float* prow = part_o + slot * D + lane * PER;
#pragma unroll
        for (int i = 0; i < PER; ++i) acc[i] += prow[i] * wgt;
    }
    const float inv = 1.f / l_all;
    bf16* orow = out + token * ((size_t)Hq * D) + (size_t)h * D + lane * PER;
#pragma unroll
    for (int i = 0; i < PER; i += 2)
        *reinterpret_cast<__nv_bfloat162*>(orow + i) = __floats2bfloat162_rn(acc[i] * inv, acc[i + 1] * inv);
}

}  // namespace

RB_EXPORT int rb_attn_tc5_head_dim() { return D; }
RB_EXPORT int rb_attn_tc5_tile_rows() { return NQ * QM; }

// float32 values of the two buffers that n_split > 1 needs: [n_split, total_rows, Hq, D] and [n_split, total_rows, Hq, 2]
RB_EXPORT long long rb_attn_tc5_split_floats(int n_split, int total_rows, int Hq) {
    return n_split > 1 ? (long long)n_split * total_rows * Hq * (D + 2) : 0;
}

// tiles: [n_tiles, 2] = (segment, first row of a block of up to 256 query rows), the blocks with the
// longest contexts first.  n_split > 1 splits the keys of every block over that many CTAs; ``scratch`` then
// holds rb_attn_tc5_split_floats(...) floats and total_rows is the number of rows of q.
RB_EXPORT int rb_attn_prefill_tc5(const void* q, int ld, const void* kpool, const void* vpool, const int* tiles,
                                  int n_tiles, const int* cu_q, const int* seg_pos0, const int* block_table,
                                  int bt_stride, int page_size, void* out, int Hq, int Hkv, float scale, int window,
                                  int n_split, void* scratch, int total_rows, int* status, cudaStream_t st) {
    if (n_tiles <= 0) return 0;
    if (n_tiles > 65535 || n_split < 1 || n_split > 64 || (n_split > 1 && scratch == nullptr)) return (int)cudaErrorInvalidValue;
    static PerDevice configured;
    const int rc = configured.once([](int) {
        return cudaFuncSetAttribute(attn_prefill_tc5_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES);
    });
    if (rc != 0) return rc;
    float* part_o = (float*)scratch;
    float* part_ml = part_o ? part_o + (size_t)n_split * total_rows * Hq * D : nullptr;
    dim3 grid(Hq, n_tiles, n_split);
    attn_prefill_tc5_kernel<<<grid, THREADS, SMEM_BYTES, st>>>(
        (const bf16*)q, ld, (const bf16*)kpool, (const bf16*)vpool, tiles, cu_q, seg_pos0, block_table, bt_stride,
        page_size, (bf16*)out, Hq, Hkv, scale * LOG2E, window, part_o, part_ml, total_rows, status);
    if (n_split > 1) {
        dim3 mgrid(Hq, n_tiles, NQ * QM / 8);
        merge_key_splits_kernel<<<mgrid, 256, 0, st>>>(part_o, part_ml, tiles, cu_q, n_split, total_rows, Hq, (bf16*)out);
    }
    return rb_launch_status();
}
