// Paged causal attention in bfloat16 on the tensor cores (mma.sync m16n8k16, float32 accumulate),
// compiled for one head size: -DHEAD_DIM=<multiple of 16, 16..256>.
//
//   rb_attn_prefill   prompt portions: one CTA per (tile of 64 query rows of one segment, q head).
//   rb_attn_decode    single decoded tokens: one CTA per (segment, kv head, split of the keys); the
//                     G query heads of the kv head share every K/V tile (rows of one MMA tile).
//   rb_attn_combine   merges the splits of rb_attn_decode.
//
// Same contract as the reference's kernels (rollout/attention.py:45-142 prefill, :430-514 split
// decode, :517-540 combine): online softmax with float32 running maximum and sum, probabilities
// rounded to bfloat16 for the P.V product, empty splits neutral (m = -inf, l = 0).  Different:
// keys arrive rotated, pages are found through a per-segment block table, K/V tiles are aligned
// to absolute positions (so a row's arithmetic in the prefill kernel does not depend on how the
// prompt was cut), and a sliding window bounds the keys from below.
//
// K and V of one layer: [num_pages, Hkv, P, D] bfloat16.  Shared-memory tiles are [rows][D] with
// the 16-byte chunks of a row XOR-swizzled by the row index, which keeps ldmatrix conflict-free.
#include "common.cuh"

#include <mutex>

#ifndef HEAD_DIM
#error "compile with -DHEAD_DIM=<head size>"
#endif
static_assert(HEAD_DIM % 16 == 0 && HEAD_DIM >= 16 && HEAD_DIM <= 256, "head size: multiple of 16 in 16..256");

namespace {

constexpr int D = HEAD_DIM;
constexpr int CHUNKS = D / 8;                 // 16-byte chunks in a row
constexpr int SWZ = (CHUNKS % 8 == 0) ? 7 : (CHUNKS % 4 == 0) ? 3 : 1;
constexpr int KSTEPS = D / 16;                // k16 steps over the head dim
constexpr int DTILES = D / 8;                 // n8 tiles over the head dim
constexpr float LOG2E = 1.4426950408889634f;

__device__ __forceinline__ int soff(int row, int chunk) { return row * D + ((chunk ^ (row & SWZ)) << 3); }

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem, bool pred) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    const int bytes = pred ? 16 : 0;          // 0: nothing is read, the 16 bytes are zero-filled
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

__device__ __forceinline__ void ldsm_x4(unsigned (&r)[4], const void* p) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void ldsm_x4_trans(unsigned (&r)[4], const void* p) {
    const unsigned s = (unsigned)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ unsigned smem_u32(const void* p) { return (unsigned)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void cp_async16_u(unsigned smem_addr, const void* gmem, bool pred) {
    const int bytes = pred ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(smem_addr), "l"(gmem), "r"(bytes));
}
__device__ __forceinline__ void ldsm_x4_u(unsigned (&r)[4], unsigned smem_addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr));
}
__device__ __forceinline__ void ldsm_x4_trans_u(unsigned (&r)[4], unsigned smem_addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr));
}
// 2^x for x <= 0 (and -inf -> 0): the hardware approximation, two units in the last place
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;\n" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ unsigned pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<unsigned*>(&v);
}

// Position -> (block, row in page).  Page sizes are powers of two in practice; any size works.
struct Paging {
    int page_size, shift;                       // shift < 0: not a power of two
    __device__ __forceinline__ explicit Paging(int p) : page_size(p), shift(-1) {
        if ((p & (p - 1)) == 0) {
            shift = 0;
            while ((1 << shift) < p) ++shift;
        }
    }
    __device__ __forceinline__ int block(int j) const { return shift >= 0 ? j >> shift : j / page_size; }
    __device__ __forceinline__ int row(int j) const { return shift >= 0 ? j & (page_size - 1) : j % page_size; }
};

// The part of a request's block table that a CTA walks, copied to shared memory once: a lookup on
// the way to every tile would put a trip to L2 into the loop.  Entries past the capacity are read
// from global memory.
constexpr int BT_CAP = 2048;
struct StagedTable {
    const int* global_row;
    const int* staged;
    int first, count;
    __device__ __forceinline__ int page(int block) const {
        const int i = block - first;
        return (i >= 0 && i < count) ? staged[i] : global_row[block];
    }
};
__device__ __forceinline__ StagedTable stage_table(int* smem_bt, const int* bt_row, int first_block, int last_block,
                                                   int tid, int nthreads) {
    StagedTable t;
    t.global_row = bt_row;
    t.staged = smem_bt;
    t.first = first_block;
    t.count = max(0, min(BT_CAP, last_block - first_block + 1));
    for (int i = tid; i < t.count; i += nthreads) smem_bt[i] = bt_row[first_block + i];
    return t;                                    // the caller synchronises before the first lookup
}

// Copies ROWS keys starting at absolute position j0 (rows of D elements) of one kv head into a
// swizzled tile, with NTHREADS threads: a group of NTHREADS / ROWS threads owns a row, looks its
// page up once, and its threads take neighbouring 16-byte chunks so that each 32-byte sector is
// asked for once.  A key outside [lo, hi] (or on a page that was given back) is zero-filled and
// never read.
template <int ROWS, int NTHREADS>
__device__ __forceinline__ void load_kv_rows(bf16* tile, const bf16* pool, const StagedTable& bt, const Paging& pg,
                                             int Hkv, int kvh, int j0, int lo, int hi, int tid) {
    constexpr int TPR = NTHREADS / ROWS;          // threads per row
    constexpr int CPT = CHUNKS / TPR;             // chunks per thread
    static_assert(NTHREADS % ROWS == 0 && CHUNKS % TPR == 0, "rows and chunks must divide evenly");
    const int r = tid / TPR, sub = tid - r * TPR;
    const int j = j0 + r;
    bool pred = j >= lo && j <= hi;
    const bf16* src = pool;
    if (pred) {
        const int page = bt.page(pg.block(j));
        pred = page >= 0;
        if (pred) src = pool + (((size_t)page * Hkv + kvh) * pg.page_size + pg.row(j)) * D;
    }
#pragma unroll
    for (int c = 0; c < CPT; ++c) {
        const int ch = c * TPR + sub;
        cp_async16(tile + soff(r, ch), pred ? src + ch * 8 : pool, pred);
    }
}

// ---------------------------------------------------------------------------------------- prefill
constexpr int PF_M = 64;      // query rows per CTA (4 warps x 16)
constexpr int PF_N = 64;      // keys per tile

__global__ void __launch_bounds__(128)
attn_prefill_kernel(const bf16* __restrict__ q, int ld, const bf16* __restrict__ kpool,
                    const bf16* __restrict__ vpool, const int* __restrict__ tiles,
                    const int* __restrict__ cu_q, const int* __restrict__ seg_pos0,
                    const int* __restrict__ block_table, int bt_stride, int page_size,
                    bf16* __restrict__ out, int Hq, int Hkv, float scale_log2, int window) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    bf16* sQ = reinterpret_cast<bf16*>(smem_raw);
    bf16* sK = sQ + PF_M * D;                 // two stages
    bf16* sV = sK + 2 * PF_N * D;             // two stages
    int* sBT = reinterpret_cast<int*>(sV + 2 * PF_N * D);
    pdl_launch_dependents();
    pdl_wait();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t4 = lane & 3;
    const int h = blockIdx.y, kvh = h / (Hq / Hkv);
    const int seg = tiles[2 * blockIdx.x], row0 = tiles[2 * blockIdx.x + 1];
    const int q_begin = cu_q[seg];
    const int m_rows = min(PF_M, cu_q[seg + 1] - q_begin - row0);
    const int p0 = seg_pos0[seg] + row0;      // position of the tile's first query
    const int p_last = p0 + m_rows - 1;
    const int lo_min = window > 0 ? max(0, p0 - window + 1) : 0;
    const int jt_begin = lo_min / PF_N, jt_end = p_last / PF_N;
    const Paging pg(page_size);
    const StagedTable bt = stage_table(sBT, block_table + (size_t)seg * bt_stride, pg.block(lo_min), pg.block(p_last), tid, 128);
    __syncthreads();

    for (int c = tid; c < PF_M * CHUNKS; c += 128) {
        const int r = c / CHUNKS, ch = c - r * CHUNKS;
        const bool pred = r < m_rows;
        const bf16* src = pred ? q + (size_t)(q_begin + row0 + r) * ld + (size_t)h * D + ch * 8 : q;
        cp_async16(sQ + soff(r, ch), src, pred);
    }
    load_kv_rows<PF_N, 128>(sK, kpool, bt, pg, Hkv, kvh, jt_begin * PF_N, lo_min, p_last, tid);
    load_kv_rows<PF_N, 128>(sV, vpool, bt, pg, Hkv, kvh, jt_begin * PF_N, lo_min, p_last, tid);
    cp_async_commit();

    unsigned qf[KSTEPS][4];
    float o[DTILES][4];
#pragma unroll
    for (int i = 0; i < DTILES; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
    const int wrow = warp * 16;
    const bool warp_active = wrow < m_rows;
    const int pos_r0 = p0 + wrow + g, pos_r1 = pos_r0 + 8;          // positions of this thread's two rows

    for (int jt = jt_begin; jt <= jt_end; ++jt) {
        const int stage = (jt - jt_begin) & 1;
        if (jt < jt_end) {
            load_kv_rows<PF_N, 128>(sK + (stage ^ 1) * PF_N * D, kpool, bt, pg, Hkv, kvh, (jt + 1) * PF_N, lo_min, p_last, tid);
            load_kv_rows<PF_N, 128>(sV + (stage ^ 1) * PF_N * D, vpool, bt, pg, Hkv, kvh, (jt + 1) * PF_N, lo_min, p_last, tid);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        if (jt == jt_begin) {
#pragma unroll
            for (int kk = 0; kk < KSTEPS; ++kk)
                ldsm_x4(qf[kk], sQ + soff(wrow + (lane & 7) + ((lane >> 3) & 1) * 8, 2 * kk + (lane >> 4)));
        }
        const int j_base = jt * PF_N;
        // a tile that starts above the warp's last row, or ends below its first row's window, adds nothing
        const bool skip = !warp_active || j_base > p0 + wrow + 15 ||
                          (window > 0 && j_base + PF_N - 1 <= p0 + wrow - window);
        if (!skip) {
            const bf16* tK = sK + stage * PF_N * D;
            const bf16* tV = sV + stage * PF_N * D;
            float s[PF_N / 8][4];
#pragma unroll
            for (int nt = 0; nt < PF_N / 8; ++nt) { s[nt][0] = s[nt][1] = s[nt][2] = s[nt][3] = 0.f; }
#pragma unroll
            for (int kk = 0; kk < KSTEPS; ++kk) {
#pragma unroll
                for (int np = 0; np < PF_N / 16; ++np) {
                    unsigned kf[4];
                    ldsm_x4(kf, tK + soff(np * 16 + ((lane >> 4) << 3) + (lane & 7), 2 * kk + ((lane >> 3) & 1)));
                    mma_bf16(s[2 * np], qf[kk], kf[0], kf[1]);
                    mma_bf16(s[2 * np + 1], qf[kk], kf[2], kf[3]);
                }
            }
            // scale, mask, running maximum
            float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
            for (int nt = 0; nt < PF_N / 8; ++nt) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int j = j_base + nt * 8 + 2 * t4 + (e & 1);
                    const int pr = (e & 2) ? pos_r1 : pos_r0;
                    const bool vis = j <= pr && (window <= 0 || j > pr - window);
                    const float v = vis ? s[nt][e] * scale_log2 : -INFINITY;
                    s[nt][e] = v;
                    if (e & 2) mx1 = fmaxf(mx1, v); else mx0 = fmaxf(mx0, v);
                }
            }
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
            mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
            mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
            const float mn0 = fmaxf(m_run[0], mx0), mn1 = fmaxf(m_run[1], mx1);
            const float mu0 = mn0 == -INFINITY ? 0.f : mn0, mu1 = mn1 == -INFINITY ? 0.f : mn1;
            const float a0 = exp2f(m_run[0] - mu0), a1 = exp2f(m_run[1] - mu1);
            m_run[0] = mn0; m_run[1] = mn1;
            float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
            for (int nt = 0; nt < PF_N / 8; ++nt) {
                s[nt][0] = exp2f(s[nt][0] - mu0); s[nt][1] = exp2f(s[nt][1] - mu0);
                s[nt][2] = exp2f(s[nt][2] - mu1); s[nt][3] = exp2f(s[nt][3] - mu1);
                sum0 += s[nt][0] + s[nt][1];
                sum1 += s[nt][2] + s[nt][3];
            }
            l_run[0] = l_run[0] * a0 + sum0;      // per-thread partial sums; quads are added at the end
            l_run[1] = l_run[1] * a1 + sum1;
#pragma unroll
            for (int i = 0; i < DTILES; ++i) { o[i][0] *= a0; o[i][1] *= a0; o[i][2] *= a1; o[i][3] *= a1; }
            // O += P V
#pragma unroll
            for (int ks = 0; ks < PF_N / 16; ++ks) {
                unsigned pf[4];
                pf[0] = pack_bf16(s[2 * ks][0], s[2 * ks][1]);
                pf[1] = pack_bf16(s[2 * ks][2], s[2 * ks][3]);
                pf[2] = pack_bf16(s[2 * ks + 1][0], s[2 * ks + 1][1]);
                pf[3] = pack_bf16(s[2 * ks + 1][2], s[2 * ks + 1][3]);
#pragma unroll
                for (int dp = 0; dp < DTILES / 2; ++dp) {
                    unsigned vf[4];
                    ldsm_x4_trans(vf, tV + soff(ks * 16 + (((lane >> 3) & 1) << 3) + (lane & 7), 2 * dp + (lane >> 4)));
                    mma_bf16(o[2 * dp], pf, vf[0], vf[1]);
                    mma_bf16(o[2 * dp + 1], pf, vf[2], vf[3]);
                }
            }
        }
        __syncthreads();      // everyone is done with this stage before the next load overwrites it
    }

    if (!warp_active) return;
    float l0 = l_run[0], l1 = l_run[1];
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    const float inv0 = 1.f / l0, inv1 = 1.f / l1;
    const int r0 = wrow + g, r1 = r0 + 8;
    const size_t ostride = (size_t)Hq * D;
    bf16* orow0 = out + (size_t)(q_begin + row0 + r0) * ostride + (size_t)h * D;
    bf16* orow1 = out + (size_t)(q_begin + row0 + r1) * ostride + (size_t)h * D;
#pragma unroll
    for (int i = 0; i < DTILES; ++i) {
        const int d = i * 8 + 2 * t4;
        if (r0 < m_rows) *reinterpret_cast<unsigned*>(orow0 + d) = pack_bf16(o[i][0] * inv0, o[i][1] * inv0);
        if (r1 < m_rows) *reinterpret_cast<unsigned*>(orow1 + d) = pack_bf16(o[i][2] * inv1, o[i][3] * inv1);
    }
}

// ---------------------------------------------------------------------------------------- decode
constexpr int DC_WARPS = 4;        // two CTAs share an SM for D <= 128, so one CTA's tail overlaps another's body
constexpr int DC_STAGES = (D <= 128) ? 3 : 2;   // pipeline depth per warp, bounded by shared memory
constexpr int DC_N = 16;      // keys per warp tile

// The decode kernel can do the work of the q/k norm + rotation + cache-write kernel for its own
// token: its query heads go normed and rotated straight into shared memory, and the CTA whose key
// range ends at the new token writes that token's key (normed, rotated) and value into the cache
// before it reads them back with everything else.  The arithmetic is that of rope_cache.cu.
struct FusedRope {
    const void* qw;            // per-head norm weights of q and k, or null: no norm
    const void* kw;
    int w_dtype;
    float eps, offset;
    const float* cos_t;        // [positions, rot_dim / 2] each
    const float* sin_t;
    int rot_dim;
    bf16* kpool;               // the pools again, to write to
    bf16* vpool;
    int write_kv;
};

__device__ __forceinline__ float2 ld_pair(const bf16* p) { return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p)); }
__device__ __forceinline__ void st_pair(bf16* p, float2 v) { *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(v.x, v.y); }

// One warp norms and rotates one head x[0..D) at position p; dst(i) is where elements i, i + 1 go.
template <typename DstFn>
__device__ __forceinline__ void warp_norm_rope(const bf16* __restrict__ x, const void* __restrict__ w, int w_dtype,
                                               float eps, float offset, const float* __restrict__ cos_t,
                                               const float* __restrict__ sin_t, int rot_dim, int p, int lane, DstFn dst) {
    const int half = rot_dim >> 1;
    const float* cs = cos_t + (size_t)p * half;
    const float* sn = sin_t + (size_t)p * half;
    // every load is issued before the first use: the head, its norm weights and its angles arrive together
    float2 a[2], b[2], wa[2], wb[2], c[2], sv[2];
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        const int i = 2 * lane + 64 * j;
        if (i < half) {
            a[j] = ld_pair(x + i);
            b[j] = ld_pair(x + i + half);
            c[j] = *reinterpret_cast<const float2*>(cs + i);
            sv[j] = *reinterpret_cast<const float2*>(sn + i);
            wa[j] = wb[j] = make_float2(1.f, 1.f);
            if (w) {
                wa[j] = make_float2(offset + load_as_f32(w, w_dtype, i), offset + load_as_f32(w, w_dtype, i + 1));
                wb[j] = make_float2(offset + load_as_f32(w, w_dtype, i + half), offset + load_as_f32(w, w_dtype, i + half + 1));
            }
        }
    }
#pragma unroll
    for (int j = 0; j < 2; ++j)
        if (2 * lane + 64 * j < half)
            ss += a[j].x * a[j].x + a[j].y * a[j].y + b[j].x * b[j].x + b[j].y * b[j].y;
    for (int i = rot_dim + 2 * lane; i < D; i += 64) {
        const float2 v = ld_pair(x + i);
        ss += v.x * v.x + v.y * v.y;
    }
    float rstd = 1.f;
    if (w) {
        ss = warp_sum(ss);
        rstd = 1.0f / sqrtf(ss / (float)D + eps);
    }
#pragma unroll
    for (int j = 0; j < 2; ++j) {
        const int i = 2 * lane + 64 * j;
        if (i < half) {
            float2 x1 = make_float2(a[j].x * rstd, a[j].y * rstd), x2 = make_float2(b[j].x * rstd, b[j].y * rstd);
            if (w) {
                x1.x *= wa[j].x; x1.y *= wa[j].y;
                x2.x *= wb[j].x; x2.y *= wb[j].y;
            }
            st_pair(dst(i), make_float2(x1.x * c[j].x - x2.x * sv[j].x, x1.y * c[j].y - x2.y * sv[j].y));
            st_pair(dst(i + half), make_float2(x2.x * c[j].x + x1.x * sv[j].x, x2.y * c[j].y + x1.y * sv[j].y));
        }
    }
    for (int i = rot_dim + 2 * lane; i < D; i += 64) {
        float2 v = ld_pair(x + i);
        v.x *= rstd; v.y *= rstd;
        if (w) { v.x *= offset + load_as_f32(w, w_dtype, i); v.y *= offset + load_as_f32(w, w_dtype, i + 1); }
        st_pair(dst(i), v);
    }
}

template <bool FUSED>
__global__ void __launch_bounds__(DC_WARPS * 32)
attn_decode_kernel(const bf16* __restrict__ q, int ld, const bf16* __restrict__ kpool,
                   const bf16* __restrict__ vpool, const int* __restrict__ dec_segs,
                   const int* __restrict__ cu_q, const int* __restrict__ seg_kv_len,
                   const int* __restrict__ block_table, int bt_stride, int page_size,
                   float* __restrict__ part_o, float* __restrict__ part_ml, bf16* __restrict__ out,
                   int Hq, int Hkv, int m_tiles, float scale_log2, int window, int num_splits, FusedRope fr) {
    extern __shared__ __align__(128) unsigned char smem_raw[];
    bf16* sQ = reinterpret_cast<bf16*>(smem_raw);                    // 16 x D
    int* sBT = reinterpret_cast<int*>(sQ + 16 * D);                  // the block-table entries this CTA walks
    bf16* sKV = reinterpret_cast<bf16*>(sBT + BT_CAP);               // [warp][stage][K 16xD | V 16xD]
    pdl_launch_dependents();
    // When this kernel itself puts the new token into the cache, every key it asks for before that was written
    // by an earlier step, and the step's tables were uploaded before its first kernel: the first tiles can be on
    // their way while the kernel before this one (the projections) still runs.  Otherwise the kernel before it
    // wrote the new token's key and value, and everything waits for it.
    const bool wait_first = !(FUSED && fr.write_kv);
    if (wait_first) pdl_wait();
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t4 = lane & 3;
    const int G = Hq / Hkv;
    const int seg = dec_segs[blockIdx.x];
    const int kvh = blockIdx.y / m_tiles, mt = blockIdx.y - kvh * m_tiles;
    const int split = blockIdx.z;
    const int h0 = kvh * G + mt * 16;
    const int rows_valid = min(16, G - mt * 16);
    const int tok_row = cu_q[seg];
    const int kv_len = seg_kv_len[seg];
    const int lo = window > 0 ? max(0, kv_len - window) : 0;        // first visible key
    const int hi = kv_len - 1;                                       // the query's own position
    const int first = lo / DC_N, n_tiles = hi / DC_N - first + 1;
    const int per_split = (n_tiles + num_splits - 1) / num_splits;
    const int t_begin = first + split * per_split;
    const int t_end = min(first + n_tiles, t_begin + per_split);     // exclusive
    const Paging pg(page_size);
    const StagedTable bt = stage_table(sBT, block_table + (size_t)seg * bt_stride, pg.block(max(lo, t_begin * DC_N)),
                                       pg.block(min(hi, t_end * DC_N - 1)), tid, DC_WARPS * 32);

    __syncthreads();                                              // the staged block table

    // Everything that depends on the lane only is worked out once: byte offsets of the ldmatrix
    // rows inside a stage, and of the 16-byte chunks this lane copies.
    constexpr unsigned TILE_BYTES = DC_N * D * 2;               // one K or V tile
    constexpr unsigned STAGE_BYTES = 2 * TILE_BYTES;
    const unsigned my_u = smem_u32(sKV) + warp * DC_STAGES * STAGE_BYTES;
    unsigned koff[KSTEPS], voff[DTILES / 2];
    {
        const int row = ((lane >> 4) << 3) + (lane & 7), c0 = (lane >> 3) & 1;
#pragma unroll
        for (int kk = 0; kk < KSTEPS; ++kk) koff[kk] = (unsigned)(row * D + (((2 * kk + c0) ^ (row & SWZ)) << 3)) * 2u;
    }
    {
        const int row = (((lane >> 3) & 1) << 3) + (lane & 7), c0 = lane >> 4;
#pragma unroll
        for (int dp = 0; dp < DTILES / 2; ++dp)
            voff[dp] = TILE_BYTES + (unsigned)(row * D + (((2 * dp + c0) ^ (row & SWZ)) << 3)) * 2u;
    }
    constexpr int CPT = CHUNKS / 2;                               // two lanes a row
    const int lr = lane >> 1, lsub = lane & 1;
    unsigned doff[CPT];
#pragma unroll
    for (int c = 0; c < CPT; ++c) doff[c] = (unsigned)(lr * D + (((2 * c + lsub) ^ (lr & SWZ)) << 3)) * 2u;

    const int n_my = t_begin + warp < t_end ? (t_end - t_begin - warp + DC_WARPS - 1) / DC_WARPS : 0;
    auto issue = [&](int i, int stage) {
        const unsigned st = my_u + stage * STAGE_BYTES;
        const int j = (t_begin + warp + i * DC_WARPS) * DC_N + lr;
        bool pred = j >= lo && j <= hi;
        size_t eoff = 0;
        if (pred) {
            const int page = bt.page(pg.block(j));
            pred = page >= 0;
            if (pred) eoff = (((size_t)page * Hkv + kvh) * pg.page_size + pg.row(j)) * D + lsub * 8;
        }
        const bf16* ks = kpool + eoff;
        const bf16* vs = vpool + eoff;
#pragma unroll
        for (int c = 0; c < CPT; ++c) cp_async16_u(st + doff[c], ks + c * 16, pred);
#pragma unroll
        for (int c = 0; c < CPT; ++c) cp_async16_u(st + TILE_BYTES + doff[c], vs + c * 16, pred);
    };
    // The first tiles are requested before anything else is done; only when this CTA is about to write
    // the new token into the cache and that token's tile is among the first, the requests wait for
    // the write.
    const bool writes_new = FUSED && fr.write_kv && hi / DC_N >= t_begin && hi / DC_N < t_end;
    const bool early = !writes_new || hi / DC_N - t_begin >= DC_WARPS * (DC_STAGES - 1);
    if (early) {
#pragma unroll
        for (int s = 0; s < DC_STAGES - 1; ++s) {
            if (s < n_my) issue(s, s);
            cp_async_commit();
        }
    }

    if (!wait_first) pdl_wait();                                     // the projections come from the kernel before
    if (FUSED) {
        const bf16* tok = q + (size_t)tok_row * ld;                  // the raw projections of this token
        // the CTA whose keys end at the new token puts that token into the cache; the barrier below
        // orders these stores before the asynchronous copies that read them back
        if (writes_new && warp < 2) {
            const int page = block_table[(size_t)seg * bt_stride + pg.block(hi)];
            if (page >= 0) {
                const size_t slot = (((size_t)page * Hkv + kvh) * pg.page_size + pg.row(hi)) * D;
                if (warp == 0) {
                    bf16* kd = fr.kpool + slot;
                    warp_norm_rope(tok + (size_t)(Hq + kvh) * D, fr.kw, fr.w_dtype, fr.eps, fr.offset, fr.cos_t, fr.sin_t,
                                   fr.rot_dim, hi, lane, [&](int i) { return kd + i; });
                } else {
                    const bf16* vs = tok + (size_t)(Hq + Hkv + kvh) * D;
                    for (int ch = lane; ch < CHUNKS; ch += 32)
                        *reinterpret_cast<uint4*>(fr.vpool + slot + ch * 8) = *reinterpret_cast<const uint4*>(vs + ch * 8);
                }
            }
        }
        // the query heads, starting with the warps that had no key or value to write
        for (int r = (warp + 2) % DC_WARPS; r < 16; r += DC_WARPS) {
            if (r < rows_valid) {
                warp_norm_rope(tok + (size_t)(h0 + r) * D, fr.qw, fr.w_dtype, fr.eps, fr.offset, fr.cos_t, fr.sin_t,
                               fr.rot_dim, hi, lane, [&](int i) { return sQ + soff(r, i >> 3) + (i & 7); });
            } else {
                for (int ch = lane; ch < CHUNKS; ch += 32) *reinterpret_cast<uint4*>(sQ + soff(r, ch)) = make_uint4(0u, 0u, 0u, 0u);
            }
        }
    } else {
        for (int c = tid; c < 16 * CHUNKS; c += DC_WARPS * 32) {
            const int r = c / CHUNKS, ch = c - r * CHUNKS;
            uint4 v = make_uint4(0u, 0u, 0u, 0u);
            if (r < rows_valid) v = *reinterpret_cast<const uint4*>(q + (size_t)tok_row * ld + (size_t)(h0 + r) * D + ch * 8);
            *reinterpret_cast<uint4*>(sQ + soff(r, ch)) = v;
        }
    }
    __syncthreads();
    if (!early) {
#pragma unroll
        for (int s = 0; s < DC_STAGES - 1; ++s) {
            if (s < n_my) issue(s, s);
            cp_async_commit();
        }
    }
    unsigned qf[KSTEPS][4];
#pragma unroll
    for (int kk = 0; kk < KSTEPS; ++kk)
        ldsm_x4(qf[kk], sQ + soff((lane & 7) + ((lane >> 3) & 1) * 8, 2 * kk + (lane >> 4)));

    float o[DTILES][4];
#pragma unroll
    for (int i = 0; i < DTILES; ++i) { o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.f; }
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};

    int stage = 0, fill_stage = DC_STAGES - 1;
    for (int i = 0; i < n_my; ++i) {
        if (i + DC_STAGES - 1 < n_my) issue(i + DC_STAGES - 1, fill_stage);
        cp_async_commit();
        cp_async_wait<DC_STAGES - 1>();
        __syncwarp();
        const unsigned tile = my_u + stage * STAGE_BYTES;
        const int j_base = (t_begin + warp + i * DC_WARPS) * DC_N;
        float s[2][4], s2[2][4];                  // two chains over the head dim, added at the end
#pragma unroll
        for (int e = 0; e < 4; ++e) { s[0][e] = s[1][e] = s2[0][e] = s2[1][e] = 0.f; }
#pragma unroll
        for (int kk = 0; kk < KSTEPS; ++kk) {
            unsigned kf[4];
            ldsm_x4_u(kf, tile + koff[kk]);
            if (kk & 1) {
                mma_bf16(s2[0], qf[kk], kf[0], kf[1]);
                mma_bf16(s2[1], qf[kk], kf[2], kf[3]);
            } else {
                mma_bf16(s[0], qf[kk], kf[0], kf[1]);
                mma_bf16(s[1], qf[kk], kf[2], kf[3]);
            }
        }
        float mx0 = -INFINITY, mx1 = -INFINITY;
        if (j_base >= lo && j_base + DC_N - 1 <= hi) {            // every key of the tile is visible
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float v = (s[nt][e] + s2[nt][e]) * scale_log2;
                    s[nt][e] = v;
                    if (e & 2) mx1 = fmaxf(mx1, v); else mx0 = fmaxf(mx0, v);
                }
            }
        } else {
#pragma unroll
            for (int nt = 0; nt < 2; ++nt) {
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int j = j_base + nt * 8 + 2 * t4 + (e & 1);
                    const float v = (j >= lo && j <= hi) ? (s[nt][e] + s2[nt][e]) * scale_log2 : -INFINITY;
                    s[nt][e] = v;
                    if (e & 2) mx1 = fmaxf(mx1, v); else mx0 = fmaxf(mx0, v);
                }
            }
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float mn0 = fmaxf(m_run[0], mx0), mn1 = fmaxf(m_run[1], mx1);
        const float mu0 = mn0 == -INFINITY ? 0.f : mn0, mu1 = mn1 == -INFINITY ? 0.f : mn1;
        // the accumulators are rescaled only when a running maximum moved (it rarely does after the first tiles)
        if (__any_sync(0xffffffffu, mn0 != m_run[0] || mn1 != m_run[1])) {
            const float a0 = fast_exp2(m_run[0] - mu0), a1 = fast_exp2(m_run[1] - mu1);
            l_run[0] *= a0;
            l_run[1] *= a1;
#pragma unroll
            for (int d = 0; d < DTILES; ++d) { o[d][0] *= a0; o[d][1] *= a0; o[d][2] *= a1; o[d][3] *= a1; }
            m_run[0] = mn0; m_run[1] = mn1;
        }
        float sum0 = 0.f, sum1 = 0.f;
#pragma unroll
        for (int nt = 0; nt < 2; ++nt) {
            s[nt][0] = fast_exp2(s[nt][0] - mu0); s[nt][1] = fast_exp2(s[nt][1] - mu0);
            s[nt][2] = fast_exp2(s[nt][2] - mu1); s[nt][3] = fast_exp2(s[nt][3] - mu1);
            sum0 += s[nt][0] + s[nt][1];
            sum1 += s[nt][2] + s[nt][3];
        }
        l_run[0] += sum0;
        l_run[1] += sum1;
        unsigned pf[4];
        pf[0] = pack_bf16(s[0][0], s[0][1]);
        pf[1] = pack_bf16(s[0][2], s[0][3]);
        pf[2] = pack_bf16(s[1][0], s[1][1]);
        pf[3] = pack_bf16(s[1][2], s[1][3]);
#pragma unroll
        for (int dp = 0; dp < DTILES / 2; ++dp) {
            unsigned vf[4];
            ldsm_x4_trans_u(vf, tile + voff[dp]);
            mma_bf16(o[2 * dp], pf, vf[0], vf[1]);
            mma_bf16(o[2 * dp + 1], pf, vf[2], vf[3]);
        }
        __syncwarp();
        stage = stage + 1 == DC_STAGES ? 0 : stage + 1;
        fill_stage = fill_stage + 1 == DC_STAGES ? 0 : fill_stage + 1;
    }
    pdl_trigger_late();
    cp_async_wait<0>();
    __syncthreads();                                              // the pipeline buffers become merge buffers

    float* mbuf = reinterpret_cast<float*>(sKV);                  // [warp][16] maxima, then [warp][16] sums
    float* lbuf = mbuf + DC_WARPS * 16;
    float* obuf = lbuf + DC_WARPS * 16;                           // [warp][16][D]
    float l0 = l_run[0], l1 = l_run[1];
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    if (t4 == 0) {
        mbuf[warp * 16 + g] = m_run[0]; mbuf[warp * 16 + g + 8] = m_run[1];
        lbuf[warp * 16 + g] = l0;       lbuf[warp * 16 + g + 8] = l1;
    }
#pragma unroll
    for (int i = 0; i < DTILES; ++i) {
        const int d = i * 8 + 2 * t4;
        if (g < rows_valid) { obuf[(warp * 16 + g) * D + d] = o[i][0]; obuf[(warp * 16 + g) * D + d + 1] = o[i][1]; }
        if (g + 8 < rows_valid) { obuf[(warp * 16 + g + 8) * D + d] = o[i][2]; obuf[(warp * 16 + g + 8) * D + d + 1] = o[i][3]; }
    }
    __syncthreads();
    for (int idx = tid; idx < rows_valid * D; idx += DC_WARPS * 32) {
        const int r = idx / D, d = idx - r * D;
        float mg = -INFINITY;
#pragma unroll
        for (int w = 0; w < DC_WARPS; ++w) mg = fmaxf(mg, mbuf[w * 16 + r]);
        float lg = 0.f, og = 0.f;
#pragma unroll
        for (int w = 0; w < DC_WARPS; ++w) {
            const float mw = mbuf[w * 16 + r];
            const float sc = mw == -INFINITY ? 0.f : exp2f(mw - mg);
            lg += lbuf[w * 16 + r] * sc;
            og += obuf[(w * 16 + r) * D + d] * sc;
        }
        const int h = h0 + r;
        if (num_splits == 1) {
            out[(size_t)tok_row * Hq * D + (size_t)h * D + d] = __float2bfloat16_rn(og / lg);
        } else {
            const size_t pidx = ((size_t)blockIdx.x * Hq + h) * num_splits + split;
            part_o[pidx * D + d] = og;
            if (d == 0) { part_ml[pidx * 2] = mg; part_ml[pidx * 2 + 1] = lg; }
        }
    }
}

// One CTA per (token, query head).  Every load is asked for before anything waits for one: the splits' (maximum,
// sum) pairs by one thread each, the splits' outputs eight at a time by the thread of their column, so the kernel
// takes about two trips to memory however many splits there are (a loop that loads, uses and loads again takes
// one trip per few splits, three times over).
constexpr int COMBINE_MAX_SPLITS = 64;
constexpr int COMBINE_THREADS = 128;
__global__ void __launch_bounds__(COMBINE_THREADS)
attn_combine_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                    const int* __restrict__ dec_segs, const int* __restrict__ cu_q,
                    bf16* __restrict__ out, int Hq, int num_splits) {
    __shared__ float s_w[COMBINE_MAX_SPLITS];
    __shared__ float s_red[2][COMBINE_THREADS / 32];
    pdl_launch_dependents();
    const int i = blockIdx.x, h = blockIdx.y, tid = threadIdx.x;
    const int tok_row = cu_q[dec_segs[i]];             // the step's tables: written before its first kernel
    const size_t base = ((size_t)i * Hq + h) * num_splits;
    pdl_wait();
    constexpr int COLS = (D + COMBINE_THREADS - 1) / COMBINE_THREADS;       // columns of a thread
    constexpr int UNROLL = 8;
    float po[COLS][UNROLL];
    auto load_o = [&](int s0) {
#pragma unroll
        for (int c = 0; c < COLS; ++c) {
            const int d = tid + c * COMBINE_THREADS;
#pragma unroll
            for (int u = 0; u < UNROLL; ++u)
                po[c][u] = (s0 + u < num_splits && d < D) ? part_o[(base + s0 + u) * D + d] : 0.f;
        }
    };
    float2 ml = make_float2(-INFINITY, 0.f);
    if (tid < num_splits) ml = *reinterpret_cast<const float2*>(part_ml + (base + tid) * 2);
    load_o(0);
    // the common maximum, every split's weight and the common sum
    float mg = ml.x;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) mg = fmaxf(mg, __shfl_xor_sync(0xffffffffu, mg, o));
    if ((tid & 31) == 0) s_red[0][tid >> 5] = mg;
    __syncthreads();
    mg = s_red[0][0];
#pragma unroll
    for (int w = 1; w < COMBINE_THREADS / 32; ++w) mg = fmaxf(mg, s_red[0][w]);
    const float wgt = ml.x == -INFINITY ? 0.f : exp2f(ml.x - mg);
    if (tid < COMBINE_MAX_SPLITS) s_w[tid] = wgt;
    float lg = ml.y * wgt;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) lg += __shfl_xor_sync(0xffffffffu, lg, o);
    if ((tid & 31) == 0) s_red[1][tid >> 5] = lg;
    __syncthreads();
    lg = 0.f;
#pragma unroll
    for (int w = 0; w < COMBINE_THREADS / 32; ++w) lg += s_red[1][w];       // in the order of the splits
    float acc[COLS];
#pragma unroll
    for (int c = 0; c < COLS; ++c) acc[c] = 0.f;
    for (int s0 = 0; s0 < num_splits; s0 += UNROLL) {
        if (s0 > 0) load_o(s0);
#pragma unroll
        for (int c = 0; c < COLS; ++c)
#pragma unroll
            for (int u = 0; u < UNROLL; ++u)
                if (s0 + u < num_splits) acc[c] += po[c][u] * s_w[s0 + u];
    }
    const float inv = 1.0f / lg;
#pragma unroll
    for (int c = 0; c < COLS; ++c) {
        const int d = tid + c * COMBINE_THREADS;
        if (d < D) out[(size_t)tok_row * Hq * D + (size_t)h * D + d] = __float2bfloat16_rn(acc[c] * inv);
    }
}

}  // namespace

RB_EXPORT int rb_attn_head_dim() { return D; }

RB_EXPORT int rb_attn_prefill(const void* q, int ld, const void* kpool, const void* vpool, const int* tiles,
                              int n_tiles, const int* cu_q, const int* seg_pos0, const int* block_table,
                              int bt_stride, int page_size, void* out, int Hq, int Hkv, float scale,
                              int window, cudaStream_t st) {
    if (n_tiles <= 0) return 0;
    const size_t smem = (size_t)(PF_M + 4 * PF_N) * D * sizeof(bf16) + BT_CAP * sizeof(int);
    static PerDevice configured;
    const int cfg = configured.once([&](int) {
        return cudaFuncSetAttribute(attn_prefill_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    });
    if (cfg != 0) return cfg;
    dim3 grid(n_tiles, Hq);
    return rb_launch_pdl(attn_prefill_kernel, grid, dim3(128), smem, st, (const bf16*)q, ld, (const bf16*)kpool,
                         (const bf16*)vpool, tiles, cu_q, seg_pos0, block_table, bt_stride, page_size, (bf16*)out,
                         Hq, Hkv, scale * LOG2E, window);
}

// Floats of scratch that rb_attn_decode needs: part_o [n_dec, Hq, splits, D], part_ml [n_dec, Hq, splits, 2].
RB_EXPORT long long rb_attn_decode_scratch_floats(int n_dec, int Hq, int num_splits) {
    return num_splits <= 1 ? 0 : (long long)n_dec * Hq * num_splits * (D + 2);
}

namespace {
int launch_decode(const void* q, int ld, const void* kpool, const void* vpool, const int* dec_segs,
                  int n_dec, const int* cu_q, const int* seg_kv_len, const int* block_table,
                  int bt_stride, int page_size, float* scratch, void* out, int Hq, int Hkv,
                  float scale, int window, int num_splits, const FusedRope* fused, cudaStream_t st) {
    if (n_dec <= 0) return 0;
    if (num_splits < 1 || num_splits > COMBINE_MAX_SPLITS || (num_splits > 1 && scratch == nullptr)) return (int)cudaErrorInvalidValue;
    const int G = Hq / Hkv, m_tiles = (G + 15) / 16;
    const size_t pipe = (size_t)DC_WARPS * DC_STAGES * 2 * DC_N * D * sizeof(bf16);
    const size_t merge = (size_t)DC_WARPS * 16 * (D + 2) * sizeof(float);
    const size_t smem = (size_t)16 * D * sizeof(bf16) + BT_CAP * sizeof(int) + (pipe > merge ? pipe : merge);
    // the kernels' shared-memory limit is a setting per device: made once for each device that calls
    static PerDevice configured;
    const int cfg = configured.once([&](int) {
        cudaError_t e = cudaFuncSetAttribute(attn_decode_kernel<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(attn_decode_kernel<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        return e;
    });
    if (cfg != 0) return cfg;
    float* part_o = scratch;
    float* part_ml = scratch ? scratch + (size_t)n_dec * Hq * num_splits * D : nullptr;
    dim3 grid(n_dec, Hkv * m_tiles, num_splits);
    FusedRope none = {};
    int rc;
    if (fused != nullptr)
        rc = rb_launch_pdl(attn_decode_kernel<true>, grid, dim3(DC_WARPS * 32), smem, st,
            (const bf16*)q, ld, (const bf16*)kpool, (const bf16*)vpool, dec_segs, cu_q, seg_kv_len, block_table,
            bt_stride, page_size, part_o, part_ml, (bf16*)out, Hq, Hkv, m_tiles, scale * LOG2E, window, num_splits, *fused);
    else
        rc = rb_launch_pdl(attn_decode_kernel<false>, grid, dim3(DC_WARPS * 32), smem, st,
            (const bf16*)q, ld, (const bf16*)kpool, (const bf16*)vpool, dec_segs, cu_q, seg_kv_len, block_table,
            bt_stride, page_size, part_o, part_ml, (bf16*)out, Hq, Hkv, m_tiles, scale * LOG2E, window, num_splits, none);
    if (rc != 0 || num_splits == 1) return rc;
    dim3 cgrid(n_dec, Hq);
    return rb_launch_pdl(attn_combine_kernel, cgrid, dim3(128), 0, st, (const float*)part_o, (const float*)part_ml,
                         dec_segs, cu_q, (bf16*)out, Hq, num_splits);
}
}  // namespace

RB_EXPORT int rb_attn_decode(const void* q, int ld, const void* kpool, const void* vpool, const int* dec_segs,
                             int n_dec, const int* cu_q, const int* seg_kv_len, const int* block_table,
                             int bt_stride, int page_size, float* scratch, void* out, int Hq, int Hkv,
                             float scale, int window, int num_splits, cudaStream_t st) {
    return launch_decode(q, ld, kpool, vpool, dec_segs, n_dec, cu_q, seg_kv_len, block_table, bt_stride, page_size,
                         scratch, out, Hq, Hkv, scale, window, num_splits, nullptr, st);
}

// The same for a step of single tokens only, with the q/k norm, the rotation and the cache write of
// those tokens done inside (qkv holds the raw projections; nothing else has touched them).
RB_EXPORT int rb_attn_decode_fused(const void* qkv, int ld, void* kpool, void* vpool, const int* dec_segs,
                                   int n_dec, const int* cu_q, const int* seg_kv_len, const int* block_table,
                                   int bt_stride, int page_size, float* scratch, void* out, int Hq, int Hkv,
                                   float scale, int window, int num_splits, const void* qw, const void* kw,
                                   int w_dtype, float eps, float offset, const float* cos_t, const float* sin_t,
                                   int rot_dim, int write_kv, cudaStream_t st) {
    if (rot_dim > D || (rot_dim & 3) || rot_dim > 256) return (int)cudaErrorInvalidValue;
    FusedRope fr;
    fr.qw = qw; fr.kw = kw; fr.w_dtype = w_dtype; fr.eps = eps; fr.offset = offset;
    fr.cos_t = cos_t; fr.sin_t = sin_t; fr.rot_dim = rot_dim;
    fr.kpool = (bf16*)kpool; fr.vpool = (bf16*)vpool; fr.write_kv = write_kv;
    return launch_decode(qkv, ld, kpool, vpool, dec_segs, n_dec, cu_q, seg_kv_len, block_table, bt_stride, page_size,
                         scratch, out, Hq, Hkv, scale, window, num_splits, &fr, st);
}

// ------------------------------------------------------------------ decode attention without allocation
// See attention_static.h.  The scratch of the split kernel is this array; host code must not pass
// its name to a kernel (in host code the name is a host-side stand-in, not a device address), so
// the address is looked up once per device with cudaGetSymbolAddress.
#include "attention_static.h"

static __device__ __align__(256) float g_decode_scratch[RB_ATTN_STATIC_SCRATCH_FLOATS];

RB_EXPORT long long rb_attn_decode_static_capacity() { return RB_ATTN_STATIC_SCRATCH_FLOATS; }

RB_EXPORT int rb_attn_decode_static(const void* q, int ld, const void* kpool, const void* vpool, const int* dec_segs,
                                    int n_dec, const int* cu_q, const int* seg_kv_len, const int* block_table,
                                    int bt_stride, int page_size, void* out, int Hq, int Hkv, float scale,
                                    int window, int num_splits, cudaStream_t st) {
    if (n_dec <= 0) return 0;
    if (num_splits < 1) return (int)cudaErrorInvalidValue;
    if (rb_attn_decode_scratch_floats(n_dec, Hq, num_splits) > (long long)RB_ATTN_STATIC_SCRATCH_FLOATS)
        return RB_ERR_SCRATCH_TOO_LARGE;
    constexpr int MAX_DEVICES = 64;
    static std::mutex mu;
    static float* scratch_of_device[MAX_DEVICES] = {nullptr};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= MAX_DEVICES) return RB_ERR_SCRATCH_LOOKUP;
    {
        std::lock_guard<std::mutex> lock(mu);
        if (scratch_of_device[dev] == nullptr) {         // set-up, once per device, that device current
            float* p = nullptr;
            if (cudaGetSymbolAddress((void**)&p, g_decode_scratch) != cudaSuccess || p == nullptr) return RB_ERR_SCRATCH_LOOKUP;
            scratch_of_device[dev] = p;
        }
    }
    return rb_attn_decode(q, ld, kpool, vpool, dec_segs, n_dec, cu_q, seg_kv_len, block_table, bt_stride, page_size,
                          scratch_of_device[dev], out, Hq, Hkv, scale, window, num_splits, st);
}
