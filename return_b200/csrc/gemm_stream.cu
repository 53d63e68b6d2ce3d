// out[M, N] = x[M, K] * W[N, K]^T for few rows of x (a decode step's tokens, M <= 128) in bfloat16:
// the weight-streaming product on the fifth-generation tensor cores.
//
// Such a product is bound by reading W once, so the work is cut so that every SM reads the same
// number of bytes: the N weight rows are dealt out to one persistent CTA per SM in contiguous
// ranges whose lengths differ by at most one granule (one row; 16 rows for the gated form), and a
// CTA walks the whole of K for its rows.  No row is shared between CTAs, so nothing is summed
// across CTAs and the result does not depend on timing.
//
// The roles of the operands are exchanged: weight rows are the MMA's M side (the 128 lanes of
// tensor memory), the tokens are its N side (16 to 128 columns).  A CTA's range is cut into
// chunks of at most 128 rows of nearly equal height h; for a chunk the TMA box is h rows by 64
// elements of K (128 bytes, 128-byte swizzle), and the MMA (always M = 128) reads 128 rows of
// shared memory of which the first h are the box: the lanes past h hold garbage nobody reads.
// An MMA takes the issuing thread some 50 cycles whatever its shape, so a CTA with few rows (a product
// with N of a few thousand) could not keep up if most lanes idled: there K is cut into 2 or 4 parts
// that lie side by side on the lanes (lane = part * slot + row) with their x boxes side by side in
// the columns, every MMA carries 128 lanes of weights, and the epilogue adds the parts' diagonal
// blocks in the order of the parts.
//   warp 0, one thread   TMA producer: for each K block the weight box and the x box (tokens x 64)
//                        into a ring of stages.  Weights do not depend on the kernel before, so the
//                        first ring of weight boxes is requested before the programmatic-dependent-
//                        launch wait and only x waits for the predecessor.
//   warp 1, one thread   tcgen05.mma (M = 128, N = tokens, K = 16) into one of two accumulators in
//                        tensor memory; tcgen05.commit frees the stage / publishes the accumulator.
//   warps 2..5           epilogue: one weight row per thread, tcgen05.ld of its tokens, optional
//                        SwiGLU over gate/up rows woven in blocks of 8 (partner row = lane ^ 8), store.
// The CTA uses under half of an SM's shared memory and tensor memory, so that the next product's
// CTAs can move in and prefetch their weights while this one drains.
//
// Measured on B200 (8 tokens): 4.4 TB/s for N = 24576, K = 4096 and 5.8 to 6.4 TB/s for N = 151936,
// where the mma.sync kernel of gemm_skinny.cu reaches 5.7 and 6.6; 11 us against 8 us for N = K = 4096.
// What holds it back is the TMA path itself: with 128-byte rows an SM keeps about 44 KB of tiled
// loads in flight however deep the ring is (one 128-byte row per ~5.5 cycles, x boxes included),
// which is the copy bandwidth and no more, and every K step pays for its x box again.  So the
// engine's product path keeps the mma.sync kernel for up to 32 rows and the library above; this
// kernel is built, tested and timed (kernel-bench gemm, impl=3) as the tcgen05 form of the same product.
//
// Every mbarrier wait is bounded; a wait that gives up raises *status and the kernel still frees its
// tensor memory and returns.
#include <cuda.h>

#include "tc5.cuh"
#include "tma.cuh"

namespace {

using namespace tc5;

constexpr int LANES = 128;                // rows of an MMA tile
constexpr int BK = 64;                    // bf16 elements of K per box: one 128-byte swizzle row
constexpr int THREADS = 192;
constexpr int MAX_STAGES = 32;
constexpr int RING_BYTES = 96 * 1024;     // shared memory given to the ring of stages

struct Plan {
    int granule;      // rows that stay together: 1, or 16 for the gated form
    int base, extra;  // CTA c owns base + (c < extra) granules, from granule c * base + min(c, extra)
    int nchunk;       // chunks per CTA (the same for all)
    int qmax;         // granules of the tallest chunk; a chunk has qmax, qmax - 1 or qmax - 2
    int kq;           // parts of K side by side on the lanes (1, 2 or 4); more than 1 only with one chunk
    int slot;         // lanes per part: 128 / kq
    int nks;          // K steps of a sweep: ceil(ceil(K / 64) / kq)
    int stages;
    unsigned w_bytes; // shared memory of a stage's weights (all parts), a multiple of 1024
};

struct Chunk {
    int row0, h;      // first weight row and number of rows
};

__device__ __forceinline__ int cta_granules(const Plan& p) { return p.base + ((int)blockIdx.x < p.extra ? 1 : 0); }

__device__ __forceinline__ Chunk chunk_of(const Plan& p, int i) {
    const int c = blockIdx.x;
    const int g0 = c * p.base + (c < p.extra ? c : p.extra);
    const int u = cta_granules(p);
    const int q = u / p.nchunk, r = u % p.nchunk;
    Chunk ch;
    ch.row0 = (g0 + i * q + (i < r ? i : r)) * p.granule;
    ch.h = (q + (i < r ? 1 : 0)) * p.granule;
    return ch;
}

__device__ __forceinline__ void epi_barrier() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

template <typename TOut> __device__ __forceinline__ TOut cvt_out(float v);
template <> __device__ __forceinline__ float cvt_out<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 cvt_out<bf16>(float v) { return __float2bfloat16_rn(v); }

// Stores the value of weight row n for token m.  All 32 lanes of the warp call it together (the
// gated form exchanges values between lanes: rows come as 8 gate rows, then their 8 up rows).
template <typename TOut, bool GATED>
__device__ __forceinline__ void store_one(TOut* __restrict__ out, int ldo, float v, int m, int n, bool valid, int lane) {
    if (GATED) {
        const float other = __shfl_xor_sync(0xffffffffu, v, 8);
        if ((lane & 8) == 0 && valid)
            out[(size_t)m * ldo + (n >> 4) * 8 + (n & 7)] = cvt_out<TOut>(v / (1.0f + __expf(-v)) * other);
    } else {
        if (valid) out[(size_t)m * ldo + n] = cvt_out<TOut>(v);
    }
}

template <int MPAD, typename TOut, bool GATED>
__global__ void __launch_bounds__(THREADS)
gemm_stream_kernel(const __grid_constant__ CUtensorMap map_w0, const __grid_constant__ CUtensorMap map_w1,
                   const __grid_constant__ CUtensorMap map_w2, const __grid_constant__ CUtensorMap map_x,
                   TOut* __restrict__ out, int M, int ldo, Plan plan, int* __restrict__ status) {
    extern __shared__ unsigned char smem_raw[];
    unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
    constexpr unsigned X_BYTES = MPAD * BK * 2;           // one part's x box
    constexpr int C = MPAD < 32 ? MPAD : 32;              // tokens read from tensor memory at a time
    __shared__ __align__(8) unsigned long long full_bar[MAX_STAGES], empty_bar[MAX_STAGES], acc_full[2], acc_empty[2];
    __shared__ unsigned tmem_slot;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int S = plan.stages, KQ = plan.kq;
    const int ncols = KQ * MPAD;                          // accumulator columns: every part's tokens
    const unsigned tmem_cols = 2 * ncols < 32 ? 32 : 2 * ncols;       // a power of two: kq and MPAD are
    const unsigned slot_bytes = (unsigned)plan.slot * BK * 2;
    const unsigned stage_bytes = plan.w_bytes + X_BYTES * KQ;
    const int nchunk = cta_granules(plan) > 0 ? plan.nchunk : 0;
    const int total = nchunk * plan.nks;                  // stages this CTA walks, over all its chunks
    float* red = reinterpret_cast<float*>(base + (size_t)S * stage_bytes + LANES * BK * 2);    // [kq][token][slot]

    if (warp == 1) tmem_alloc(smem_u32(&tmem_slot), tmem_cols);
    if (tid == 0) {
        tma::prefetch_desc(&map_w0);
        tma::prefetch_desc(&map_w1);
        tma::prefetch_desc(&map_w2);
        tma::prefetch_desc(&map_x);
        for (int s = 0; s < S; ++s) { mbar_init(smem_u32(&full_bar[s]), 1); mbar_init(smem_u32(&empty_bar[s]), 1); }
#pragma unroll
        for (int b = 0; b < 2; ++b) { mbar_init(smem_u32(&acc_full[b]), 1); mbar_init(smem_u32(&acc_empty[b]), 4); }
        mbar_init_fence();
    }
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const unsigned tacc = tmem_slot;
    bool ok = true;

    if (warp == 0) {
        if (lane == 0) {                                    // ---- producer
            const unsigned long long stream_once = tma::policy_evict_first();
            // No division inside the K loops: one thread runs them, and its instruction latency is the
            // pipeline's clock.  Part p of K starts at block p * nks.
            // the first ring of weight boxes: no predecessor writes weights
            const int pre = total < S ? total : S;
            {
                int it = 0;
                for (int i = 0; i < nchunk && it < pre; ++i) {
                    const Chunk ch = chunk_of(plan, i);
                    const int which = plan.qmax - ch.h / plan.granule;
                    const CUtensorMap* map = which == 0 ? &map_w0 : which == 1 ? &map_w1 : &map_w2;
                    const unsigned bytes = ((unsigned)ch.h * BK * 2 + X_BYTES) * KQ;
                    for (int ks = 0; ks < plan.nks && it < pre; ++ks, ++it) {
                        const unsigned full = smem_u32(&full_bar[it]);
                        unsigned dst = smem_u32(base) + (unsigned)it * stage_bytes;
                        mbar_arrive_expect_tx(full, bytes);
                        for (int p = 0, kb = ks; p < KQ; ++p, kb += plan.nks, dst += slot_bytes)
                            tma::load_2d_hint(dst, map, kb * BK, ch.row0, full, stream_once);
                    }
                }
            }
            pdl_wait();                                     // x comes from the kernel before
            int s = 0, round = 0, it = 0;
            unsigned stage = smem_u32(base);
            for (int i = 0; i < nchunk; ++i) {
                const Chunk ch = chunk_of(plan, i);
                const int which = plan.qmax - ch.h / plan.granule;
                const CUtensorMap* map = which == 0 ? &map_w0 : which == 1 ? &map_w1 : &map_w2;
                const unsigned bytes = ((unsigned)ch.h * BK * 2 + X_BYTES) * KQ;
                for (int ks = 0; ks < plan.nks; ++ks, ++it) {
                    const unsigned full = smem_u32(&full_bar[s]);
                    if (it >= S) {
                        ok = mbar_wait(smem_u32(&empty_bar[s]), (round - 1) & 1) && ok;
                        mbar_arrive_expect_tx(full, bytes);
                        unsigned dst = stage;
                        for (int p = 0, kb = ks; p < KQ; ++p, kb += plan.nks, dst += slot_bytes)
                            tma::load_2d_hint(dst, map, kb * BK, ch.row0, full, stream_once);
                    }
                    unsigned dst = stage + plan.w_bytes;
                    for (int p = 0, kb = ks; p < KQ; ++p, kb += plan.nks, dst += X_BYTES)
                        tma::load_2d(dst, &map_x, kb * BK, 0, full);
                    stage += stage_bytes;
                    if (++s == S) { s = 0; ++round; stage = smem_u32(base); }
                }
            }
            pdl_trigger_late();                             // everything this CTA reads is on its way
        }
    } else if (warp == 1) {
        if (lane == 0) {                                    // ---- MMA issuer
            // With kq parts the lanes are (part, row) and the columns (part, token): the MMA also
            // multiplies a part's weights with the other parts' tokens, which nobody reads; what it
            // buys is that all 128 lanes of every MMA carry weights that were streamed in.
            const unsigned idesc = instr_desc_bf16(LANES, ncols);
            // descriptors advance by additions: 16 bytes are one unit of the address field
            const unsigned long long desc0 = smem_desc_sw128(smem_u32(base), 0);
            const unsigned x_off = plan.w_bytes >> 4, stage_step = stage_bytes >> 4;
            int s = 0, round = 0;
            unsigned long long a = desc0;
            for (int i = 0; i < nchunk; ++i) {
                const int buf = i & 1;
                if (i >= 2) ok = mbar_wait(smem_u32(&acc_empty[buf]), ((i >> 1) - 1) & 1) && ok;
                fence_after_sync();
                const unsigned d = tacc + buf * ncols;
                for (int ks = 0; ks < plan.nks; ++ks) {
                    ok = mbar_wait(smem_u32(&full_bar[s]), round & 1) && ok;
                    fence_after_sync();
                    const unsigned long long b = a + x_off;
                    mma_ss(d, a, b, idesc, ks > 0);             // four steps of 16 along K: 32 bytes = 2 address units
                    mma_ss(d, a + 2, b + 2, idesc, true);
                    mma_ss(d, a + 4, b + 4, idesc, true);
                    mma_ss(d, a + 6, b + 6, idesc, true);
                    mma_commit(smem_u32(&empty_bar[s]));
                    a += stage_step;
                    if (++s == S) { s = 0; ++round; a = desc0; }
                }
                mma_commit(smem_u32(&acc_full[buf]));
            }
        }
    } else {                                                // ---- epilogue: TMEM lanes by warp % 4
        const int q = warp & 3, L = q * 32 + lane;          // this thread's lane of tensor memory
        const int part = L / plan.slot, row = L - part * plan.slot;
        const int etid = (warp - 2) * 32 + lane;
        for (int i = 0; i < nchunk; ++i) {
            const Chunk ch = chunk_of(plan, i);          // never empty: a range holds at least as many granules as chunks
            const int buf = i & 1;
            ok = mbar_wait(smem_u32(&acc_full[buf]), (i >> 1) & 1) && ok;
            fence_after_sync();
            const unsigned src = tacc + ((unsigned)(q * 32) << 16) + buf * ncols + part * MPAD;
            if (KQ == 1) {
                if (q * 32 < ch.h) {                        // this warp's lanes hold rows of the chunk
#pragma unroll 1
                    for (int m0 = 0; m0 < MPAD && m0 < M; m0 += C) {
                        unsigned r[C];
                        if (C == 16) tmem_ld16(src + m0, reinterpret_cast<unsigned(&)[16]>(r));
                        else tmem_ld32(src + m0, reinterpret_cast<unsigned(&)[32]>(r));
                        tmem_ld_wait();
#pragma unroll
                        for (int j = 0; j < C; ++j) {
                            if (m0 + j >= M) break;         // uniform over the warp
                            store_one<TOut, GATED>(out, ldo, __uint_as_float(r[j]), m0 + j, ch.row0 + row, row < ch.h, lane);
                        }
                    }
                }
                fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&acc_empty[buf]));
            } else {
                // the parts of K are summed through shared memory, in the order of the parts
#pragma unroll 1
                for (int m0 = 0; m0 < MPAD && m0 < M; m0 += C) {
                    unsigned r[C];
                    if (C == 16) tmem_ld16(src + m0, reinterpret_cast<unsigned(&)[16]>(r));
                    else tmem_ld32(src + m0, reinterpret_cast<unsigned(&)[32]>(r));
                    tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < C; ++j)
                        if (m0 + j < M) red[(part * MPAD + m0 + j) * plan.slot + row] = __uint_as_float(r[j]);
                }
                fence_before_sync();
                __syncwarp();
                if (lane == 0) mbar_arrive(smem_u32(&acc_empty[buf]));
                epi_barrier();
                // thread (g, r): row r, tokens g, g + kq, ...; a warp holds 32 consecutive rows of one token
                const int g = etid / plan.slot, r = etid - g * plan.slot;
                for (int mb = 0; mb < M; mb += KQ) {         // the same number of turns for every lane of a warp
                    const int m = mb + g;
                    float v = 0.f;
                    if (m < M)
                        for (int p = 0; p < KQ; ++p) v += red[(p * MPAD + m) * plan.slot + r];
                    store_one<TOut, GATED>(out, ldo, v, m, ch.row0 + r, m < M && r < ch.h, lane);
                }
                epi_barrier();                               // red is free for the next chunk
            }
        }
    }
    if (!ok) atomicExch(status, 1);
    fence_before_sync();
    __syncthreads();
    if (warp == 1) tmem_dealloc(tacc, tmem_cols);
}

Plan make_plan(int N, int K, int grid, int mpad, bool gated) {
    Plan p;
    p.granule = gated ? 16 : 1;
    const int units = (N + p.granule - 1) / p.granule;
    p.base = units / grid;
    p.extra = units % grid;
    const int most = p.base + (p.extra ? 1 : 0);          // granules of the largest range
    const int rows = most * p.granule;
    const int nkb = (K + BK - 1) / BK;
    // few rows a CTA: parts of K side by side on the lanes, as many as fit (columns: kq * mpad <= 256); at most
    // 4, so that a warp's 32 lanes belong to one part and read one block of columns
    p.kq = 1;
    while (p.kq < 4 && rows * (p.kq * 2) <= LANES && mpad * (p.kq * 2) <= 256 && nkb >= p.kq * 2) p.kq *= 2;
    p.slot = LANES / p.kq;
    const int per_chunk = LANES / p.granule;
    p.nchunk = p.kq > 1 ? 1 : (most + per_chunk - 1) / per_chunk;
    p.qmax = (most + p.nchunk - 1) / p.nchunk;
    p.nks = (nkb + p.kq - 1) / p.kq;
    p.w_bytes = p.kq > 1 ? (unsigned)(LANES * BK * 2) : (((unsigned)(p.qmax * p.granule * BK * 2) + 1023u) & ~1023u);
    const int stage_bytes = (int)p.w_bytes + p.kq * mpad * BK * 2;
    p.stages = RING_BYTES / stage_bytes;
    if (p.stages > MAX_STAGES) p.stages = MAX_STAGES;
    if (p.stages < 2) p.stages = 2;
    return p;
}

template <int MPAD, typename TOut, bool GATED>
int launch_stream(const void* x, const void* w, void* out, int M, int N, int K, int ldx, int ldw, int ldo,
                  int* status, cudaStream_t st) {
    const int sms = rb_num_sms();
    if (sms <= 0) return (int)cudaErrorInvalidDevice;
    const Plan plan = make_plan(N, K, sms, MPAD, GATED);
    CUtensorMap mw[3], mx;
    for (int i = 0; i < 3; ++i) {
        int rows = (plan.qmax - i) * plan.granule;
        if (rows < 1) rows = 1;                            // never used: a range has no chunk that small
        if (!tma::make_map_bf16(&mw[i], w, N, K, ldw, rows)) return (int)cudaErrorInvalidValue;
    }
    if (!tma::make_map_bf16(&mx, x, M, K, ldx, MPAD)) return (int)cudaErrorInvalidValue;
    // the MMA reads 128 rows from a stage's base: room for that behind the last stage; then the sums of the parts
    const size_t red_bytes = plan.kq > 1 ? (size_t)LANES * MPAD * 4 : 0;
    const size_t smem = (size_t)plan.stages * (plan.w_bytes + plan.kq * MPAD * BK * 2) + LANES * BK * 2 + red_bytes + 1024;
    static PerDevice configured;                           // the largest shared-memory size asked for so far, per device
    const int rc = configured.once([&](int) {
        return cudaFuncSetAttribute(gemm_stream_kernel<MPAD, TOut, GATED>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    }, (long long)smem);
    if (rc != 0) return rc;
    const int units = (N + plan.granule - 1) / plan.granule;
    dim3 grid(units < sms ? units : sms);
    return rb_launch_pdl(gemm_stream_kernel<MPAD, TOut, GATED>, grid, dim3(THREADS), smem, st, mw[0], mw[1], mw[2], mx,
                         (TOut*)out, M, ldo, plan, status);
}

}  // namespace

// out dtype: 0 bfloat16, 1 float32.  gated: SwiGLU epilogue over woven gate/up rows (out is [M, N/2]).
// status: raised if a bounded wait gave up.
RB_EXPORT int rb_gemm_stream(const void* x, const void* w, void* out, int out_f32, int gated, int M, int N, int K,
                             int ldx, int ldw, int ldo, int* status, cudaStream_t st) {
    if (M <= 0 || N <= 0) return 0;
    if (M > 128 || K % 8 || ldx % 8 || ldw % 8 || ((uintptr_t)x % 16) || ((uintptr_t)w % 16)) return (int)cudaErrorInvalidValue;
    if (gated && (out_f32 || N % 16)) return (int)cudaErrorInvalidValue;
#define RB_STREAM(MP)                                                                                                  \
    {                                                                                                                  \
        if (gated) return launch_stream<MP, bf16, true>(x, w, out, M, N, K, ldx, ldw, ldo, status, st);                \
        if (out_f32) return launch_stream<MP, float, false>(x, w, out, M, N, K, ldx, ldw, ldo, status, st);            \
        return launch_stream<MP, bf16, false>(x, w, out, M, N, K, ldx, ldw, ldo, status, st);                          \
    }
    if (M <= 16) RB_STREAM(16)
    if (M <= 32) RB_STREAM(32)
    if (M <= 64) RB_STREAM(64)
    RB_STREAM(128)
#undef RB_STREAM
}

// The plan a call would use on this device: {rows of the largest range, chunks per CTA, rows of the
// tallest chunk, parts of K side by side}.
RB_EXPORT void rb_gemm_stream_plan(int M, int N, int K, int gated, int* out4) {
    const int mpad = M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : 128;
    const Plan p = make_plan(N, K, rb_num_sms(), mpad, gated != 0);
    out4[0] = (p.base + (p.extra ? 1 : 0)) * p.granule; out4[1] = p.nchunk; out4[2] = p.qmax * p.granule; out4[3] = p.kq;
}
