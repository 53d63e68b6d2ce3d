// out[M, N] = x[M, K] * W[N, K]^T in bfloat16 for a handful of rows (M <= 64): the matrix products
// of a decode step, which stream every weight once and are bound by HBM bandwidth.
//
// The weight matrix is the A operand of mma.sync.m16n8k16 (16 weight rows per warp), the tokens are
// the B operand (8 tokens per instruction), so a product with few tokens wastes no tensor-core rows.
// A group is 16 weight rows; the 8 warps of a CTA split K and add their partial sums through shared memory.
// Every lane reads 16 contiguous bytes of a weight row and of a token row straight into registers:
// within a block of 32 k the four 16-byte pieces of a row are handed to the MMA in a permuted
// order, the same for both operands, which leaves the dot product unchanged and makes all loads
// full 16-byte vectors without shared-memory staging.  Accumulation is float32.
//
// The RMSNorm and the residual add around a product cost no kernel of their own (rb_gemm_skinny_fused, up to 8
// rows).  With v = stream + x W^T the norm's output is v * rstd * w, where rstd is one number per token.  The
// product before the norm ("residual" form) stores v into the float32 stream, v * (offset + w) in bfloat16 for the
// next product, and each CTA's share of sum(v^2); the product after it multiplies its accumulators by
// rstd = 1 / sqrt(sum(v^2) / H + eps) in its epilogue, which gives the same number:
// (v * rstd * w) W^T = rstd * ((v * w) W^T).  The shares are added in the order of the CTAs, so the result does not
// depend on timing.
//
// Needs K % 8 == 0 and 16-byte aligned rows (ldx, ldw multiples of 8 elements).
#include "common.cuh"

namespace {

constexpr int SK_WARPS = 8;
constexpr int SK_ROWS = 16;       // weight rows per group
constexpr int SK_CTAS_PER_SM = 2;

__device__ __forceinline__ uint4 ld_stream16(const void* p) {       // read once: do not keep in L1
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}

__device__ __forceinline__ void mma_bf16(float (&c)[4], unsigned a0, unsigned a1, unsigned a2, unsigned a3,
                                         unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

template <typename T> __device__ __forceinline__ void store_out(T* p, float v);
template <> __device__ __forceinline__ void store_out<float>(float* p, float v) { *p = v; }
template <> __device__ __forceinline__ void store_out<bf16>(bf16* p, float v) { *p = __float2bfloat16_rn(v); }

// What the fused forms need beside the product itself.
struct SkinnyFused {
    const float* ssq_in;      // [8, ssq_ld] shares of sum(v^2) of each token, or null: no scaling
    int ssq_in_count;         // shares per token
    int norm_dim;             // length of the normed row
    float eps;
    float* stream;            // residual form: [M, N] float32, contiguous
    const void* norm_w;       // residual form: weight [N] of the norm that follows, or null: no normed rows wanted
    int norm_w_dtype;
    float offset;
    float* ssq_out;           // residual form: [8, ssq_ld], this CTA writes column blockIdx.x; or null
    int ssq_ld;
};

template <int MT, int U>
struct Regs {                         // one buffer: U blocks of 32 k of the weight rows and of the tokens
    uint4 a0[U], a1[U], b[U][MT];
};

// GATED: the 16 weight rows of a group are 8 gate rows followed by their 8 up rows (the feed-forward's
// interleaved layout); the epilogue writes silu(gate) * up, 8 values per token, into out[M, N / 2].
//
// Persistent: a CTA walks groups of 16 weight rows (group = blockIdx.x, + gridDim.x, ...).  Each
// warp owns one slice of K, cut into buffers of U blocks of 32; the buffers of all its groups form
// one sequence, and the loads of buffer i + 1 are in flight while buffer i is multiplied, also
// across the boundary between two groups, so the weight stream never drains while a group's
// partial sums are added up and stored.
// FUSED 0: plain.  1: the accumulators are scaled by each token's rstd (F.ssq_in).  2: the same and the residual
// form: out gets the normed rows for the next product (if F.norm_w), the stream gets v.  MT == 1 for FUSED != 0.
template <int MT, typename TOut, bool GATED, int FUSED>
__global__ void __launch_bounds__(SK_WARPS * 32)
gemm_skinny_kernel(const bf16* __restrict__ x, const bf16* __restrict__ w, TOut* __restrict__ out,
                   int M, int N, int K, int ldx, int ldw, int ldo, const SkinnyFused F) {
    constexpr int U = MT == 1 ? 4 : 2;                    // k32 blocks per buffer; two buffers in flight
    __shared__ float red[SK_WARPS][SK_ROWS][8 * MT + 1];
    __shared__ float s_scale[8];
    float ssq_acc = 0.f;                                  // residual form: this thread's part of sum(v^2) of its token
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int g = lane >> 2, t4 = lane & 3;
    const bf16* xr[MT];
    bool xok[MT];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) {
        const int m = mt * 8 + g;
        xok[mt] = m < M;
        xr[mt] = x + (size_t)(xok[mt] ? m : 0) * ldx + 8 * t4;
    }
    const int nkb = (K + 31) >> 5;
    const int per = (nkb + SK_WARPS - 1) / SK_WARPS;
    const int kb_begin = warp * per, kb_end = min(nkb, kb_begin + per);
    const int nbuf = max(1, (per + U - 1) / U);          // buffers per group (the same for every warp)
    const int n_groups = (N + SK_ROWS - 1) / SK_ROWS;
    const int my_groups = (int)blockIdx.x < n_groups ? (n_groups - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
    const int total = my_groups * nbuf;                  // buffers this warp walks
    float acc[MT][4];
#pragma unroll
    for (int mt = 0; mt < MT; ++mt) { acc[mt][0] = acc[mt][1] = acc[mt][2] = acc[mt][3] = 0.f; }
    const uint4 zero = make_uint4(0u, 0u, 0u, 0u);

    // buffer i of this warp: group (i / nbuf) of this CTA, blocks kb_begin + (i % nbuf) * U ...
    auto load_w = [&](Regs<MT, U>& r, int i) {           // blocks past the slice, or past the last group, load zeros
        const int gi = i / nbuf, kb = kb_begin + (i - gi * nbuf) * U;
        const int n0 = ((int)blockIdx.x + gi * (int)gridDim.x) * SK_ROWS;
        const int r0 = n0 + g, r1 = r0 + 8;
        const bool ok0 = i < total && r0 < N, ok1 = i < total && r1 < N;
        const bf16* w0 = w + (size_t)(ok0 ? r0 : 0) * ldw + 8 * t4;
        const bf16* w1 = w + (size_t)(ok1 ? r1 : 0) * ldw + 8 * t4;
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int k = (kb + u) << 5;
            const bool kin = kb + u < kb_end && k + 8 * t4 < K;
            r.a0[u] = (kin && ok0) ? ld_stream16(w0 + k) : zero;
            r.a1[u] = (kin && ok1) ? ld_stream16(w1 + k) : zero;
        }
    };
    auto load_x = [&](Regs<MT, U>& r, int i) {
        const int kb = kb_begin + (i % nbuf) * U;
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int k = (kb + u) << 5;
            const bool kin = i < total && kb + u < kb_end && k + 8 * t4 < K;
#pragma unroll
            for (int mt = 0; mt < MT; ++mt)
                r.b[u][mt] = (kin && xok[mt]) ? __ldg(reinterpret_cast<const uint4*>(xr[mt] + k)) : zero;
        }
    };
    auto compute = [&](const Regs<MT, U>& r) {
#pragma unroll
        for (int u = 0; u < U; ++u) {
#pragma unroll
            for (int mt = 0; mt < MT; ++mt) {
                mma_bf16(acc[mt], r.a0[u].x, r.a1[u].x, r.a0[u].y, r.a1[u].y, r.b[u][mt].x, r.b[u][mt].y);
                mma_bf16(acc[mt], r.a0[u].z, r.a1[u].z, r.a0[u].w, r.a1[u].w, r.b[u][mt].z, r.b[u][mt].w);
            }
        }
    };
    // after the last buffer of a group: the warps' partial sums meet in shared memory and are stored
    auto finish_group = [&](int i) {
        const int n0 = ((int)blockIdx.x + (i / nbuf) * (int)gridDim.x) * SK_ROWS;
        if (i + 1 >= total) pdl_trigger_late();
#pragma unroll
        for (int mt = 0; mt < MT; ++mt) {
            red[warp][g][mt * 8 + 2 * t4] = acc[mt][0];
            red[warp][g][mt * 8 + 2 * t4 + 1] = acc[mt][1];
            red[warp][g + 8][mt * 8 + 2 * t4] = acc[mt][2];
            red[warp][g + 8][mt * 8 + 2 * t4 + 1] = acc[mt][3];
            acc[mt][0] = acc[mt][1] = acc[mt][2] = acc[mt][3] = 0.f;
        }
        __syncthreads();
        if constexpr (GATED) {
            for (int idx = tid; idx < 8 * 8 * MT; idx += SK_WARPS * 32) {
                const int j = idx & 7, m = idx >> 3;
                if (m < M && n0 + 8 + j < N) {
                    float gate = 0.f, up = 0.f;
#pragma unroll
                    for (int wi = 0; wi < SK_WARPS; ++wi) { gate += red[wi][j][m]; up += red[wi][8 + j][m]; }
                    if constexpr (FUSED != 0) { gate *= s_scale[m]; up *= s_scale[m]; }
                    store_out<TOut>(out + (size_t)m * ldo + (n0 >> 1) + j, gate / (1.0f + expf(-gate)) * up);
                }
            }
        } else {
            for (int idx = tid; idx < SK_ROWS * 8 * MT; idx += SK_WARPS * 32) {
                const int n = idx & (SK_ROWS - 1), m = idx >> 4;
                if (m < M && n0 + n < N) {
                    float s = 0.f;
#pragma unroll
                    for (int wi = 0; wi < SK_WARPS; ++wi) s += red[wi][n][m];
                    if constexpr (FUSED == 2) {
                        float* sp = F.stream + (size_t)m * N + n0 + n;
                        const float v = *sp + s * s_scale[m];
                        *sp = v;
                        ssq_acc += v * v;
                        if (F.norm_w != nullptr)
                            store_out<TOut>(out + (size_t)m * ldo + n0 + n,
                                            v * (F.offset + load_as_f32(F.norm_w, F.norm_w_dtype, (size_t)(n0 + n))));
                    } else {
                        if constexpr (FUSED == 1) s *= s_scale[m];
                        store_out<TOut>(out + (size_t)m * ldo + n0 + n, s);
                    }
                }
            }
        }
        __syncthreads();                                 // red is free for the next group
    };

    Regs<MT, U> ra, rb;
    pdl_launch_dependents();
    load_w(ra, 0);                                       // weights are nobody's output: stream them at once
    pdl_wait();                                          // the tokens come from the kernel before
    if constexpr (FUSED != 0) {
        // warp m adds up the shares of token m, in the order of the CTAs that wrote them; the barrier inside the first
        // finish_group stands between this and the first use
        float scale = 1.0f;
        if (F.ssq_in != nullptr) {
            float part = 0.f;
            if (warp < M)
                for (int c = lane; c < F.ssq_in_count; c += 32) part += F.ssq_in[(size_t)warp * F.ssq_ld + c];
            part = warp_sum(part);
            scale = 1.0f / sqrtf(part / (float)F.norm_dim + F.eps);
        }
        if (lane == 0) s_scale[warp] = scale;
    }
    load_x(ra, 0);
    for (int i = 0; i < total; i += 2) {                 // buffer i + 1 is in flight while buffer i is used
        load_w(rb, i + 1);
        load_x(rb, i + 1);
        compute(ra);
        if ((i + 1) % nbuf == 0) finish_group(i);
        load_w(ra, i + 2);
        load_x(ra, i + 2);
        if (i + 1 < total) {
            compute(rb);
            if ((i + 2) % nbuf == 0) finish_group(i + 1);
        }
    }
    if constexpr (FUSED == 2) {
        if (F.ssq_out != nullptr) {
            // threads 0..127 hold the part of one token each (m = tid / 16) over the columns they stored
            float s = ssq_acc;
            s += __shfl_xor_sync(0xffffffffu, s, 8);
            s += __shfl_xor_sync(0xffffffffu, s, 4);
            s += __shfl_xor_sync(0xffffffffu, s, 2);
            s += __shfl_xor_sync(0xffffffffu, s, 1);
            if (tid < SK_ROWS * 8 && (tid & 15) == 0) F.ssq_out[(size_t)(tid >> 4) * F.ssq_ld + blockIdx.x] = s;
        }
    }
}

int resident_ctas() { return rb_num_sms() * SK_CTAS_PER_SM; }      // CTAs that fit the current GPU at once

int grid_for(int N) {
    const int groups = (N + SK_ROWS - 1) / SK_ROWS, resident = resident_ctas();
    return groups < resident ? groups : resident;
}

template <int MT>
int launch(const bf16* x, const bf16* w, void* out, int out_f32, int gated, int M, int N, int K, int ldx, int ldw,
           int ldo, cudaStream_t st) {
    const int grid = grid_for(N);
    if (grid <= 0) return (int)cudaErrorInvalidDevice;
    const SkinnyFused none = {};
    if (gated)
        return rb_launch_pdl(gemm_skinny_kernel<MT, bf16, true, 0>, dim3(grid), dim3(SK_WARPS * 32), 0, st, x, w, (bf16*)out, M, N, K, ldx, ldw, ldo, none);
    if (out_f32)
        return rb_launch_pdl(gemm_skinny_kernel<MT, float, false, 0>, dim3(grid), dim3(SK_WARPS * 32), 0, st, x, w, (float*)out, M, N, K, ldx, ldw, ldo, none);
    return rb_launch_pdl(gemm_skinny_kernel<MT, bf16, false, 0>, dim3(grid), dim3(SK_WARPS * 32), 0, st, x, w, (bf16*)out, M, N, K, ldx, ldw, ldo, none);
}

}  // namespace

RB_EXPORT int rb_gemm_skinny_max_rows() { return 32; }

// CTAs that a product with N weight rows is launched with on the current device: the number of shares of sum(v^2)
// that its residual form writes per token.
RB_EXPORT int rb_gemm_skinny_ctas(int N) { return grid_for(N); }

// The fused forms, for up to 8 rows, bfloat16 out.  form 0: out[M, N] = rstd * acc (or silu(rstd gate) * (rstd up) into
// out[M, N / 2] with gated = 1), rstd from ssq_in (null: 1).  form 1 (residual): v = stream[M, N] + rstd * acc goes to the
// stream; out[M, N] = v * (offset + norm_w) if norm_w is given; ssq_out[m][cta] = this CTA's share of sum_n v^2.
RB_EXPORT int rb_gemm_skinny_fused(const void* x, const void* w, void* out, int form, int gated, int M, int N, int K,
                                   int ldx, int ldw, int ldo, const float* ssq_in, int ssq_in_count, int norm_dim, float eps,
                                   float* stream, const void* norm_w, int norm_w_dtype, float offset, float* ssq_out,
                                   int ssq_ld, cudaStream_t st) {
    if (M <= 0 || N <= 0) return 0;
    if (M > 8 || K % 8 || ldx % 8 || ldw % 8 || ((uintptr_t)x % 16) || ((uintptr_t)w % 16)) return (int)cudaErrorInvalidValue;
    if (gated && (N % 16 || form != 0)) return (int)cudaErrorInvalidValue;
    if (form == 1 && (stream == nullptr || (norm_w != nullptr && out == nullptr))) return (int)cudaErrorInvalidValue;
    if (form == 0 && out == nullptr) return (int)cudaErrorInvalidValue;
    const int grid = grid_for(N);
    if (grid <= 0) return (int)cudaErrorInvalidDevice;
    if ((ssq_in != nullptr && (ssq_in_count < 1 || ssq_in_count > ssq_ld || norm_dim < 1)) || (ssq_out != nullptr && ssq_ld < grid))
        return (int)cudaErrorInvalidValue;
    SkinnyFused F;
    F.ssq_in = ssq_in; F.ssq_in_count = ssq_in_count; F.norm_dim = norm_dim; F.eps = eps; F.stream = stream;
    F.norm_w = norm_w; F.norm_w_dtype = norm_w_dtype; F.offset = offset; F.ssq_out = ssq_out; F.ssq_ld = ssq_ld;
    const bf16* xp = (const bf16*)x;
    const bf16* wp = (const bf16*)w;
    if (form == 1)
        return rb_launch_pdl(gemm_skinny_kernel<1, bf16, false, 2>, dim3(grid), dim3(SK_WARPS * 32), 0, st, xp, wp, (bf16*)out, M, N, K, ldx, ldw, ldo, F);
    if (gated)
        return rb_launch_pdl(gemm_skinny_kernel<1, bf16, true, 1>, dim3(grid), dim3(SK_WARPS * 32), 0, st, xp, wp, (bf16*)out, M, N, K, ldx, ldw, ldo, F);
    return rb_launch_pdl(gemm_skinny_kernel<1, bf16, false, 1>, dim3(grid), dim3(SK_WARPS * 32), 0, st, xp, wp, (bf16*)out, M, N, K, ldx, ldw, ldo, F);
}

// gated = 1: w holds gate and up rows interleaved in blocks of 8 (N % 16 == 0) and out is
// bfloat16 [M, N / 2] = silu(gate) * up.
RB_EXPORT int rb_gemm_skinny(const void* x, const void* w, void* out, int out_f32, int gated, int M, int N, int K,
                             int ldx, int ldw, int ldo, cudaStream_t st) {
    if (M <= 0 || N <= 0) return 0;
    if (M > 32 || K % 8 || ldx % 8 || ldw % 8 || ((uintptr_t)x % 16) || ((uintptr_t)w % 16))
        return (int)cudaErrorInvalidValue;
    if (gated && (N % 16 || out_f32)) return (int)cudaErrorInvalidValue;
    const bf16* xp = (const bf16*)x;
    const bf16* wp = (const bf16*)w;
    if (M <= 8) return launch<1>(xp, wp, out, out_f32, gated, M, N, K, ldx, ldw, ldo, st);
    if (M <= 16) return launch<2>(xp, wp, out, out_f32, gated, M, N, K, ldx, ldw, ldo, st);
    return launch<4>(xp, wp, out, out_f32, gated, M, N, K, ldx, ldw, ldo, st);
}
