// A chain of matrix products for a handful of token rows (M <= 8) in ONE persistent kernel: the products of
// a decode step that follow one another (output projection -> residual add + norm -> gated feed-forward ->
// down projection) stream their weights through one ring of shared-memory stages that never drains, not
// even while the CTAs of the grid wait for one another between two products.
//
//   out_0 = f_0(x_0) W_0^T ;  grid barrier ;  out_1 = f_1(...) W_1^T ;  grid barrier ; ...
//
// A decode step is bound by the time it takes to read every weight once.  Launched one product a kernel,
// each product pays its ramp-up and its tail (a few microseconds in which HBM idles), and the short kernels
// between them (residual add + RMSNorm, SwiGLU) pay a launch each.  Here one CTA per SM owns a contiguous
// range of weight rows of every product; a producer warp copies those rows into a ring of stages with
// cp.async.bulk (completion counted on mbarriers), as far ahead as the ring has room, across the boundaries
// between products: weights are nobody's output, so the next product's first rows are already in shared
// memory when the grid barrier before it opens.  Eight consumer warps take stages in turn: ldmatrix of a
// [16 weight rows x 16 k] tile as the A operand of mma.sync.m16n8k16, the (up to 8) tokens as the B
// operand; their partial sums meet in shared memory after each 16-row unit.
//
// What an op may do before its product (x_kind) and after it (epilogue):
//   x_kind 0  x [M, K] bfloat16 in global memory (written by the kernel before);
//   x_kind 1  x = rmsnorm(stream_in + delta) * (offset + norm_w), float32 arithmetic, one rounding; the
//             sum goes to stream_out (another buffer than stream_in: every CTA reads stream_in while
//             CTA 0 writes stream_out), so the residual add and the norm need no kernel of their own;
//   x_kind 2  x written by the op before it in this chain, in the permuted order described below;
//   epilogue 0  out[M, N] bfloat16;   epilogue 1  the weight holds gate and up rows woven in blocks of 8
//             (N % 16 == 0) and out[M, N / 2] = silu(gate) * up.
//
// Order of k inside x.  A lane of the MMA needs, of every 8 consecutive k of its token, one pair (2 t4,
// 2 t4 + 1).  So that a lane gets the pairs of four such groups with ONE 16-byte load, x is kept with the
// k of each block of 32 permuted: element 8 c + 2 q + e (c the group, q the pair) sits at 8 q + 2 c + e.
// The kernel writes this order itself (staging x into shared memory, or storing an epilogue's output for
// the op after it), so nothing outside ever sees it.
//
// Needs K % 16 == 0, 16-byte aligned weight rows, M <= 8.  The grid must be resident at once (one CTA per
// SM, at most as many CTAs as SMs): CTAs wait for one another.  Every wait is bounded; one that gives up
// raises *status and lets the kernel end.
#include "tc5.cuh"

namespace {

using tc5::mbar_arrive;
using tc5::mbar_arrive_expect_tx;
using tc5::mbar_init;
using tc5::mbar_init_fence;
using tc5::mbar_wait;
using tc5::smem_u32;

constexpr int CH_CONSUMER_WARPS = 8;
constexpr int CH_CONSUMERS = CH_CONSUMER_WARPS * 32;
constexpr int CH_THREADS = CH_CONSUMERS + 32;            // + the producer warp
constexpr int CH_ROWS = 16;                              // weight rows of a unit (one MMA A tile)
constexpr int CH_KC = 256;                               // k of a stage
constexpr int CH_ROW_BYTES = CH_KC * 2 + 16;             // a row of a stage, padded: ldmatrix rows fall on different banks
constexpr int CH_STAGE_BYTES = CH_ROWS * CH_ROW_BYTES;
constexpr int CH_MAX_OPS = 4;
constexpr int CH_MAX_STAGES = 24;
constexpr int CH_TOKENS = 8;
constexpr int CH_RED_STRIDE = CH_TOKENS + 1;

struct ChainOp {
    const bf16* w;            // [N, K], row stride ldw
    const bf16* x;            // x_kind 0: [M, K] natural order, row stride ldx; x_kind 2: permuted, row stride ldx
    const float* stream_in;   // x_kind 1: [M, K] float32
    float* stream_out;        // x_kind 1: stream_in + delta, written by CTA 0 (null: not wanted)
    const bf16* delta;        // x_kind 1: [M, K] row stride ld_delta, or null
    const void* norm_w;       // x_kind 1: [K]
    bf16* out;                // [M, N] (epilogue 0) or [M, N / 2] (epilogue 1), row stride ldo
    int N, K, ldw, ldx, ldo, ld_delta;
    int x_kind, epilogue, out_permuted, norm_w_dtype;
    float eps, offset;
};

struct ChainParams {
    ChainOp op[CH_MAX_OPS];
    int n_ops, M, n_stages, xs_k;     // xs_k: k capacity of the shared-memory copy of x (a multiple of 32)
    unsigned* barrier;                // [2]: arrivals, generation
    int* status;
};

__device__ __forceinline__ int perm32(int k) {            // position of element k in the permuted order
    return (k & ~31) | (((k >> 1) & 3) << 3) | (((k >> 3) & 3) << 1) | (k & 1);
}

__device__ __forceinline__ void bulk_copy(unsigned dst_smem, const void* src, unsigned bytes, unsigned bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(dst_smem), "l"(src), "r"(bytes), "r"(bar) : "memory");
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(CH_CONSUMERS) : "memory"); }
__device__ __forceinline__ unsigned ld_acquire(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release(unsigned* p, unsigned v) {
    asm volatile("st.release.gpu.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ void ldsm_x4(unsigned (&r)[4], unsigned addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma16816(float (&c)[4], const unsigned (&a)[4], unsigned b0, unsigned b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// One thread of the grid's CTAs: all CTAs have arrived when this returns (false: gave up).
__device__ __forceinline__ bool grid_arrive_and_wait(unsigned* bar, unsigned n_ctas) {
    __threadfence();
    const unsigned gen = ld_acquire(bar + 1);
    const unsigned prev = atomicAdd(bar, 1u);
    bool ok = true;
    if (prev == n_ctas - 1) {
        atomicExch(bar, 0u);                              // the count is ready for the next barrier before anyone can arrive at it
        st_release(bar + 1, gen + 1);
    } else {
        ok = false;
        for (unsigned spin = 0; spin < (1u << 22); ++spin) {
            if (ld_acquire(bar + 1) != gen) { ok = true; break; }
            __nanosleep(20);
        }
    }
    __threadfence();
    return ok;
}

// The units (blocks of 16 weight rows) of an op that CTA `cta` of `n_ctas` owns: [u0, u1).
__device__ __forceinline__ void my_units(int N, int cta, int n_ctas, int& u0, int& u1) {
    const int units = (N + CH_ROWS - 1) / CH_ROWS;
    u0 = (int)((long long)units * cta / n_ctas);
    u1 = (int)((long long)units * (cta + 1) / n_ctas);
}

__global__ void __launch_bounds__(CH_THREADS, 1)
gemm_chain_kernel(const __grid_constant__ ChainParams P) {
    extern __shared__ __align__(128) unsigned char smem[];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int NS = P.n_stages;
    const int xs_stride = P.xs_k * 2 + 64;                // bytes of a token row in shared memory (== 64 mod 128)
    unsigned char* ring = smem;
    unsigned char* xs = ring + (size_t)NS * CH_STAGE_BYTES;
    float* red = reinterpret_cast<float*>(xs + (size_t)CH_TOKENS * xs_stride);          // [2][warps][16][9]
    unsigned long long* bars = reinterpret_cast<unsigned long long*>(red + 2 * CH_CONSUMER_WARPS * CH_ROWS * CH_RED_STRIDE);
    const unsigned full0 = smem_u32(bars), empty0 = smem_u32(bars + NS);
    const unsigned ring_u = smem_u32(ring);
    if (tid == 0) {
        for (int s = 0; s < NS; ++s) {
            mbar_init(full0 + 8 * s, 1);
            mbar_init(empty0 + 8 * s, 1);
        }
        mbar_init_fence();
    }
    __syncthreads();
    const int cta = blockIdx.x, n_ctas = gridDim.x;
    const int M = P.M;

    if (warp == CH_CONSUMER_WARPS) {
        // ------------------------------------------------------------ producer: weights into the ring, as far ahead as it has room
        unsigned q = 0;
        bool ok = true;
        for (int o = 0; o < P.n_ops && ok; ++o) {
            const ChainOp& op = P.op[o];
            int u0, u1;
            my_units(op.N, cta, n_ctas, u0, u1);
            const int spu = (op.K + CH_KC - 1) / CH_KC;
            for (int u = u0; u < u1 && ok; ++u) {
                const int n0 = u * CH_ROWS, rows = min(CH_ROWS, op.N - n0);
                for (int s = 0; s < spu; ++s, ++q) {
                    const unsigned slot = q % NS, round = q / NS;
                    if (round > 0 && !mbar_wait(empty0 + 8 * slot, (round - 1) & 1)) { ok = false; break; }
                    const int k0 = s * CH_KC;
                    const unsigned bytes = (unsigned)min(CH_KC, op.K - k0) * 2u;
                    if (lane == 0) mbar_arrive_expect_tx(full0 + 8 * slot, bytes * (unsigned)rows);
                    __syncwarp();
                    if (lane < rows)
                        bulk_copy(ring_u + slot * CH_STAGE_BYTES + lane * CH_ROW_BYTES,
                                  op.w + (size_t)(n0 + lane) * op.ldw + k0, bytes, full0 + 8 * slot);
                }
            }
        }
        // (no launch_dependents here: the kernel after this one must not take SMs before every CTA of this grid
        // is resident, which only the consumers know, after their last grid barrier)
        if (!ok && lane == 0) atomicExch(P.status, 11);
        return;
    }

    // ---------------------------------------------------------------- consumers
    pdl_wait();                                          // x, the stream and delta come from the kernels before
    const int g = lane >> 2, t4 = lane & 3;
    const unsigned a_lane = (unsigned)(((lane & 7) + ((lane >> 3) & 1) * 8) * CH_ROW_BYTES + (lane >> 4) * 16);
    unsigned q = 0;
    int unit_count = 0;
    bool ok = true;
    for (int o = 0; o < P.n_ops; ++o) {
        const ChainOp& op = P.op[o];
        const int K = op.K;
        // ---- x into shared memory, in the permuted order (x_kind 2 is read from global memory as it is)
        if (op.x_kind == 0) {
            const int nblk = (K + 31) >> 5;
            for (int i = tid; i < CH_TOKENS * nblk; i += CH_CONSUMERS) {
                const int m = i / nblk, b = i - m * nblk;
                uint4 v[4];
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const int k = 32 * b + 8 * c;
                    v[c] = (m < M && k < K) ? __ldcg(reinterpret_cast<const uint4*>(op.x + (size_t)m * op.ldx + k))
                                            : make_uint4(0u, 0u, 0u, 0u);
                }
                // pair q of group c (word q of v[c]) goes to word c of chunk q
                uint4* dst = reinterpret_cast<uint4*>(xs + (size_t)m * xs_stride + (size_t)b * 64);
                dst[0] = make_uint4(v[0].x, v[1].x, v[2].x, v[3].x);
                dst[1] = make_uint4(v[0].y, v[1].y, v[2].y, v[3].y);
                dst[2] = make_uint4(v[0].z, v[1].z, v[2].z, v[3].z);
                dst[3] = make_uint4(v[0].w, v[1].w, v[2].w, v[3].w);
            }
        } else if (op.x_kind == 1) {
            // warp m norms token row m: two passes over the row (the second finds it in L2), the same
            // arithmetic as the stand-alone kernel: (stream + delta) * rstd * (offset + w), one rounding
            const int m = warp;
            const int nblk = (K + 31) >> 5;
            unsigned char* xrow = xs + (size_t)m * xs_stride;
            if (m < M) {
                const float* s_in = op.stream_in + (size_t)m * K;
                const bf16* dl = op.delta ? op.delta + (size_t)m * op.ld_delta : nullptr;
                float* s_out = (cta == 0 && op.stream_out) ? op.stream_out + (size_t)m * K : nullptr;
                float ss = 0.f;
                for (int b = lane; b < nblk; b += 32) {
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const int k = 32 * b + 8 * c;
                        if (k >= K) break;
                        float4 lo = __ldcg(reinterpret_cast<const float4*>(s_in + k));
                        float4 hi = __ldcg(reinterpret_cast<const float4*>(s_in + k + 4));
                        if (dl) {
                            const uint4 dv = __ldcg(reinterpret_cast<const uint4*>(dl + k));
                            const float2 d0 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&dv.x));
                            const float2 d1 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&dv.y));
                            const float2 d2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&dv.z));
                            const float2 d3 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&dv.w));
                            lo.x += d0.x; lo.y += d0.y; lo.z += d1.x; lo.w += d1.y;
                            hi.x += d2.x; hi.y += d2.y; hi.z += d3.x; hi.w += d3.y;
                        }
                        ss += lo.x * lo.x + lo.y * lo.y + lo.z * lo.z + lo.w * lo.w
                            + hi.x * hi.x + hi.y * hi.y + hi.z * hi.z + hi.w * hi.w;
                        if (s_out) {
                            *reinterpret_cast<float4*>(s_out + k) = lo;
                            *reinterpret_cast<float4*>(s_out + k + 4) = hi;
                        }
                    }
                }
                ss = warp_sum(ss);
                const float rstd = 1.0f / sqrtf(ss / (float)K + op.eps);
                for (int b = lane; b < nblk; b += 32) {
                    unsigned wd[4][4];                    // [group c][pair q]
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        const int k = 32 * b + 8 * c;
                        float v[8];
                        if (k < K) {
                            const float4 lo = __ldcg(reinterpret_cast<const float4*>(s_in + k));
                            const float4 hi = __ldcg(reinterpret_cast<const float4*>(s_in + k + 4));
                            v[0] = lo.x; v[1] = lo.y; v[2] = lo.z; v[3] = lo.w; v[4] = hi.x; v[5] = hi.y; v[6] = hi.z; v[7] = hi.w;
                            if (dl) {
                                const uint4 dv = __ldcg(reinterpret_cast<const uint4*>(dl + k));
                                const unsigned dw[4] = {dv.x, dv.y, dv.z, dv.w};
#pragma unroll
                                for (int p2 = 0; p2 < 4; ++p2) {
                                    const float2 d = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&dw[p2]));
                                    v[2 * p2] += d.x; v[2 * p2 + 1] += d.y;
                                }
                            }
#pragma unroll
                            for (int e = 0; e < 8; ++e)
                                v[e] = v[e] * rstd * (op.offset + load_as_f32(op.norm_w, op.norm_w_dtype, (size_t)(k + e)));
                        } else {
#pragma unroll
                            for (int e = 0; e < 8; ++e) v[e] = 0.f;
                        }
#pragma unroll
                        for (int p2 = 0; p2 < 4; ++p2) {
                            __nv_bfloat162 h = __floats2bfloat162_rn(v[2 * p2], v[2 * p2 + 1]);
                            wd[c][p2] = *reinterpret_cast<unsigned*>(&h);
                        }
                    }
                    uint4* dst = reinterpret_cast<uint4*>(xrow + (size_t)b * 64);
#pragma unroll
                    for (int p2 = 0; p2 < 4; ++p2) dst[p2] = make_uint4(wd[0][p2], wd[1][p2], wd[2][p2], wd[3][p2]);
                }
            } else {
                for (int b = lane; b < nblk; b += 32) {
                    uint4* dst = reinterpret_cast<uint4*>(xrow + (size_t)b * 64);
                    dst[0] = dst[1] = dst[2] = dst[3] = make_uint4(0u, 0u, 0u, 0u);
                }
            }
        }
        consumer_sync();

        // ---- the units of this CTA
        int u0, u1;
        my_units(op.N, cta, n_ctas, u0, u1);
        const int spu = (K + CH_KC - 1) / CH_KC;
        const bool x_global = op.x_kind == 2;
        const unsigned char* xg = reinterpret_cast<const unsigned char*>(op.x) + (size_t)g * op.ldx * 2 + t4 * 16;
        const unsigned char* xl = xs + (size_t)g * xs_stride + t4 * 16;
        for (int u = u0; u < u1; ++u, ++unit_count) {
            float acc0[4] = {0.f, 0.f, 0.f, 0.f}, acc1[4] = {0.f, 0.f, 0.f, 0.f};
            for (int s = 0; s < spu; ++s, ++q) {
                if ((int)(q % CH_CONSUMER_WARPS) != warp) continue;
                const unsigned slot = q % NS, round = q / NS;
                if (ok && !mbar_wait(full0 + 8 * slot, round & 1)) ok = false;
                const int k0 = s * CH_KC;
                const int ksteps = min(CH_KC, K - k0) >> 4;
                const unsigned a_base = ring_u + slot * CH_STAGE_BYTES + a_lane;
                const size_t xoff = (size_t)k0 * 2;
#pragma unroll 4
                for (int j = 0; j < ksteps; j += 2) {
                    uint4 b;
                    if (x_global) b = g < M ? __ldcg(reinterpret_cast<const uint4*>(xg + xoff + (size_t)j * 32)) : make_uint4(0u, 0u, 0u, 0u);
                    else b = *reinterpret_cast<const uint4*>(xl + xoff + (size_t)j * 32);
                    unsigned a[4];
                    ldsm_x4(a, a_base + j * 32);
                    mma16816(acc0, a, b.x, b.y);
                    if (j + 1 < ksteps) {
                        ldsm_x4(a, a_base + (j + 1) * 32);
                        mma16816(acc1, a, b.z, b.w);
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(empty0 + 8 * slot);
            }
            // the warps' partial sums of this unit meet in shared memory
            float* r = red + ((size_t)(unit_count & 1) * CH_CONSUMER_WARPS + warp) * CH_ROWS * CH_RED_STRIDE;
            r[g * CH_RED_STRIDE + 2 * t4] = acc0[0] + acc1[0];
            r[g * CH_RED_STRIDE + 2 * t4 + 1] = acc0[1] + acc1[1];
            r[(g + 8) * CH_RED_STRIDE + 2 * t4] = acc0[2] + acc1[2];
            r[(g + 8) * CH_RED_STRIDE + 2 * t4 + 1] = acc0[3] + acc1[3];
            consumer_sync();
            const float* rb = red + (size_t)(unit_count & 1) * CH_CONSUMER_WARPS * CH_ROWS * CH_RED_STRIDE;
            const int n0 = u * CH_ROWS;
            if (op.epilogue == 1) {
                if (tid < 8 * CH_TOKENS) {
                    const int jj = tid & 7, m = tid >> 3;
                    if (m < M && n0 + 8 + jj < op.N) {
                        float gate = 0.f, up = 0.f;
#pragma unroll
                        for (int wi = 0; wi < CH_CONSUMER_WARPS; ++wi) {
                            gate += rb[(wi * CH_ROWS + jj) * CH_RED_STRIDE + m];
                            up += rb[(wi * CH_ROWS + 8 + jj) * CH_RED_STRIDE + m];
                        }
                        const int col = (n0 >> 1) + jj;
                        op.out[(size_t)m * op.ldo + (op.out_permuted ? perm32(col) : col)] =
                            __float2bfloat16_rn(gate / (1.0f + expf(-gate)) * up);
                    }
                }
            } else {
                if (tid < CH_ROWS * CH_TOKENS) {
                    const int n = tid & (CH_ROWS - 1), m = tid >> 4;
                    if (m < M && n0 + n < op.N) {
                        float sum = 0.f;
#pragma unroll
                        for (int wi = 0; wi < CH_CONSUMER_WARPS; ++wi) sum += rb[(wi * CH_ROWS + n) * CH_RED_STRIDE + m];
                        const int col = n0 + n;
                        op.out[(size_t)m * op.ldo + (op.out_permuted ? perm32(col) : col)] = __float2bfloat16_rn(sum);
                    }
                }
            }
        }
        // ---- every CTA has stored its part of this op's output before anyone reads it
        if (o + 1 < P.n_ops) {
            consumer_sync();
            if (tid == 0 && !grid_arrive_and_wait(P.barrier, (unsigned)n_ctas)) atomicExch(P.status, 12);
            consumer_sync();
        }
    }
    if (!ok && lane == 0) atomicExch(P.status, 13);
    pdl_trigger_late();
}

}  // namespace

// The layout of ChainParams for callers that build it outside C++ (ctypes): sizes to check against.
RB_EXPORT int rb_gemm_chain_param_bytes() { return (int)sizeof(ChainParams); }
RB_EXPORT int rb_gemm_chain_op_bytes() { return (int)sizeof(ChainOp); }
RB_EXPORT int rb_gemm_chain_stage_bytes() { return CH_STAGE_BYTES; }

// Shared memory of a launch with a ring of n_stages stages and room for xs_k elements of x per token.
static size_t chain_smem_bytes(int n_stages, int xs_k) {
    return (size_t)n_stages * CH_STAGE_BYTES + (size_t)CH_TOKENS * (xs_k * 2 + 64) +
           (size_t)2 * CH_CONSUMER_WARPS * CH_ROWS * CH_RED_STRIDE * sizeof(float) + (size_t)2 * n_stages * 8 + 128;
}

// Plans a launch on the current device: the k capacity of the shared-memory copy of x that the chain needs
// (xs_k_needed, a multiple of 32) -> the number of ring stages that fit beside it, or 0 if too few do.
RB_EXPORT int rb_gemm_chain_plan(int xs_k_needed) {
    int dev = 0, max_smem = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    cudaDeviceGetAttribute(&max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
    int stages = CH_MAX_STAGES;
    while (stages >= 6 && chain_smem_bytes(stages, xs_k_needed) > (size_t)max_smem) --stages;
    return stages >= 6 ? stages : 0;
}

// params: a ChainParams (host memory); n_stages and xs_k as planned.  barrier: two zeroed unsigned ints that
// belong to launches of this kernel on this stream; status: an int that is raised when a wait gave up.
RB_EXPORT int rb_gemm_chain(const void* params, cudaStream_t st) {
    ChainParams P = *reinterpret_cast<const ChainParams*>(params);
    if (P.n_ops < 1 || P.n_ops > CH_MAX_OPS || P.M < 1 || P.M > CH_TOKENS) return (int)cudaErrorInvalidValue;
    if (P.n_stages < 2 || P.n_stages > CH_MAX_STAGES || P.xs_k % 32) return (int)cudaErrorInvalidValue;
    for (int o = 0; o < P.n_ops; ++o) {
        const ChainOp& op = P.op[o];
        if (op.N <= 0 || op.K <= 0 || op.K % 16 || op.ldw % 8 || ((uintptr_t)op.w % 16)) return (int)cudaErrorInvalidValue;
        if (op.epilogue == 1 && op.N % 16) return (int)cudaErrorInvalidValue;
        if (op.x_kind != 2 && op.K > P.xs_k) return (int)cudaErrorInvalidValue;
        if (op.x_kind == 0 && (op.ldx % 8 || ((uintptr_t)op.x % 16))) return (int)cudaErrorInvalidValue;
        if (op.x_kind == 2 && (o == 0 || op.ldx % 32 || ((uintptr_t)op.x % 16))) return (int)cudaErrorInvalidValue;
        if (op.x_kind == 1 && (((uintptr_t)op.stream_in % 16) || ((uintptr_t)op.stream_out % 16) || op.stream_in == op.stream_out ||
                               ((uintptr_t)op.delta % 16) || op.ld_delta % 8))
            return (int)cudaErrorInvalidValue;
    }
    static int sms_of_device[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return (int)cudaErrorInvalidDevice;
    const size_t smem = chain_smem_bytes(P.n_stages, P.xs_k);
    if (sms_of_device[dev] == 0) {
        int sms = 0, max_smem = 0;
        cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
        cudaDeviceGetAttribute(&max_smem, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
        cudaError_t e = cudaFuncSetAttribute(gemm_chain_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, max_smem);
        if (e != cudaSuccess) return (int)e;
        sms_of_device[dev] = sms;
    }
    // one CTA per SM and never more CTAs than SMs: the CTAs wait for one another, so all must be resident
    int most_units = 0;
    for (int o = 0; o < P.n_ops; ++o) most_units = max(most_units, (P.op[o].N + CH_ROWS - 1) / CH_ROWS);
    const int grid = min(sms_of_device[dev], most_units);
    return rb_launch_pdl(gemm_chain_kernel, dim3(grid), dim3(CH_THREADS), smem, st, P);
}
