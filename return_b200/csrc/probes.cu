// Measurement probes (not on the engine's path): the issue rate and latency of mma.sync.m16n8k16
// on this part, which is the ceiling of the kernels that use it.
#include "common.cuh"
#include "tc5.cuh"

namespace {

__device__ __forceinline__ void mma(float (&c)[4], unsigned a, unsigned b) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a), "r"(a), "r"(a), "r"(a), "r"(b), "r"(b));
}

template <int CHAINS>
__global__ void mma_rate_kernel(float* sink, int iters, long long* cycles) {
    float c[CHAINS][4];
#pragma unroll
    for (int i = 0; i < CHAINS; ++i) c[i][0] = c[i][1] = c[i][2] = c[i][3] = 0.f;
    const unsigned a = 0x3c003c00u, b = 0x3c003c00u;
    const long long t0 = clock64();
    for (int it = 0; it < iters; ++it) {
#pragma unroll
        for (int i = 0; i < CHAINS; ++i) mma(c[i], a, b);
    }
    const long long t1 = clock64();
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < CHAINS; ++i) s += c[i][0] + c[i][1] + c[i][2] + c[i][3];
    if (s == 12345.f) sink[0] = s;
    if (threadIdx.x == 0 && blockIdx.x == 0) *cycles = t1 - t0;
}

}  // namespace

// Runs `iters` rounds of `chains` (1 or 8) independent MMAs per warp with `warps` warps on each of
// `ctas` CTAs; writes the cycles the first CTA took to *cycles (device memory, 8 bytes).
RB_EXPORT int rb_probe_mma_rate(int ctas, int warps, int chains, int iters, float* sink, long long* cycles,
                                cudaStream_t st) {
    if (chains == 1) mma_rate_kernel<1><<<ctas, warps * 32, 0, st>>>(sink, iters, cycles);
    else if (chains == 8) mma_rate_kernel<8><<<ctas, warps * 32, 0, st>>>(sink, iters, cycles);
    else return (int)cudaErrorInvalidValue;
    return rb_launch_status();
}


// ------------------------------------------------------------------------------------ tcgen05.mma rate
// `threads` issuing threads (lane 0 of warps 0..threads-1) of one CTA per SM issue `iters` MMAs of
// M x N x 16 each (bf16, both operands in shared memory, the same tiles every time, eight MMAs per
// loop turn with constant descriptor offsets) into accumulators of their own, then commit and wait.
// cycles[2 * w] = clocks until warp w had issued everything, cycles[2 * w + 1] = until all had completed.
//
// mode bit 0: B is an MN-major operand (its 128-byte rows run along N, as the attention kernel reads V from the
// cache); bit 1: the three other warps write 16-byte pieces to another part of shared memory all the while (what
// softmax rows and loaders do beside the MMAs); bit 2: the mix of one key tile of the attention kernel instead of
// one shape: 2 x 8 MMAs of 128 x 64 x 16 (K-major) and 2 x 4 of 128 x 128 x 16 (B MN-major), `iters` tiles,
// cycles counted per tile; bit 3 (with bit 2): a tcgen05.commit to a barrier nobody waits on after each of the
// tile's four groups of MMAs and two more, as the attention kernel has them.  cycles[8] = 16-byte stores the
// other warps made.  bit 4: the CTA has eleven warps and the ten that issue nothing
// wait on a barrier that completes only when the MMAs are done, every thread polling as the kernels' waits do.
// mode 32: no MMAs; one thread does `iters` rounds of tcgen05.commit to a barrier and a wait for it: cycles a
// round = what a commit takes to reach its barrier with nothing in flight.  mode 33: the same with one
// 128 x 64 x 16 MMA before every commit.  mode 64: no MMAs; lane 0 of warps 0 and 1 hand a token back and
// forth through two barriers (arrive, wait): cycles a round trip = two arrive-to-wake latencies.
namespace {
__global__ void __launch_bounds__(352) tc5_rate_kernel(int M, int N, int iters, int threads, int mode, long long* cycles) {
    using namespace tc5;
    extern __shared__ unsigned char probe_smem[];
    unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(probe_smem) + 1023) & ~uintptr_t(1023));
    __shared__ __align__(8) unsigned long long bar[4];
    __shared__ unsigned tmem_slot;
    __shared__ volatile int done;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    for (int i = tid; i < 48 * 1024 / 4; i += blockDim.x) reinterpret_cast<unsigned*>(base)[i] = 0x3c003c00u;     // bf16 1.0
    if (warp == 0) tmem_alloc(smem_u32(&tmem_slot), 512);
    if (tid == 0) {
        done = 0;
        for (int i = 0; i < 4; ++i) mbar_init(smem_u32(&bar[i]), 1);
        mbar_init_fence();
    }
    fence_proxy_async();
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const unsigned tacc = tmem_slot;
    const bool b_mn = mode & 1, hammer = mode & 2, mix = mode & 4, commits = mode & 8, pollers = mode & 16;
    if (mode == 32 || mode == 33) {
        if (tid == 0) {
            const unsigned idesc = instr_desc_bf16(128, 64);
            const unsigned long long a = smem_desc_sw128(smem_u32(base), 0), b = smem_desc_sw128(smem_u32(base) + 16384, 0);
            bool ok = true;
            const long long t0 = clock64();
            for (int i = 0; i < iters; ++i) {
                if (mode == 33) mma_ss(tacc, a, b, idesc, true);
                mma_commit(smem_u32(&bar[0]));
                ok = mbar_wait(smem_u32(&bar[0]), i & 1) && ok;
            }
            const long long t1 = clock64();
            if (blockIdx.x == 0) { cycles[0] = t1 - t0; cycles[1] = ok ? t1 - t0 : -1; }
        }
    } else if (mode >= 65 && mode <= 69) {
        // what one operation costs the thread that issues it, back to back: 65 a commit (to a barrier nobody
        // waits on), 66 a wait that succeeds at once, 67 tcgen05.fence::after_thread_sync, 68 one mbarrier.test_wait,
        // 69 one mbarrier.try_wait.relaxed.cta
        if (tid == 0) {
            mbar_arrive(smem_u32(&bar[1]));                   // phase 0 of bar[1] is complete from here on
            bool ok = true;
            const long long t0 = clock64();
            for (int i = 0; i < iters; ++i) {
                if (mode == 65) mma_commit(smem_u32(&bar[0]));
                else if (mode == 66) ok = mbar_wait(smem_u32(&bar[1]), 0) && ok;
                else if (mode == 67) fence_after_sync();
                else {
                    unsigned done;
                    if (mode == 68)
                        asm volatile("{\n.reg .pred p;\nmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
                                     : "=r"(done) : "r"(smem_u32(&bar[1])), "r"(0u) : "memory");
                    else
                        asm volatile("{\n.reg .pred p;\nmbarrier.try_wait.parity.relaxed.cta.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}"
                                     : "=r"(done) : "r"(smem_u32(&bar[1])), "r"(0u) : "memory");
                    ok = ok && done;
                }
            }
            const long long t1 = clock64();
            if (blockIdx.x == 0) { cycles[0] = t1 - t0; cycles[1] = ok ? t1 - t0 : -1; }
        }
    } else if (mode >= 100 && mode <= 102) {
        // the key tile's mix again, with the four waits (each on a phase that is complete already) and fences that
        // the kernel has between its groups of MMAs: 100 in the issuing thread, 101 waits without the fences,
        // 102 none in the issuing thread, but lane 0 of the next warp waits and fences in a loop meanwhile
        if (tid == 0) mbar_arrive(smem_u32(&bar[1]));           // phase 0 of bar[1] is complete from here on
        __syncthreads();
        if (tid == 0) {
            const unsigned idesc_s = instr_desc_bf16(128, 64, false), idesc_o = instr_desc_bf16(128, 128, true);
            const unsigned long long a = smem_desc_sw128(smem_u32(base), 0);
            const unsigned long long bk = smem_desc_sw128(smem_u32(base) + 16384, 0);
            const unsigned long long bv = smem_desc_sw128_mn(smem_u32(base) + 32768, 64 * 128, 1024u);
            bool ok = true;
            const long long t0 = clock64();
            for (int i = 0; i < iters; ++i) {
                if (mode != 102) { ok = mbar_wait(smem_u32(&bar[1]), 0) && ok; if (mode == 100) fence_after_sync(); }
#pragma unroll
                for (int qt = 0; qt < 2; ++qt) {
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        mma_ss(tacc + qt * 64, a + (unsigned long long)(((j >> 2) * (128 * 128) + (j & 3) * 32) >> 4),
                               bk + (unsigned long long)(((j >> 2) * (64 * 128) + (j & 3) * 32) >> 4), idesc_s, j > 0);
                }
                if (mode != 102) { ok = mbar_wait(smem_u32(&bar[1]), 0) && ok; if (mode == 100) fence_after_sync(); }
#pragma unroll
                for (int qt = 0; qt < 2; ++qt) {
                    if (mode != 102) { ok = mbar_wait(smem_u32(&bar[1]), 0) && ok; if (mode == 100) fence_after_sync(); }
#pragma unroll
                    for (int j = 0; j < 4; ++j) mma_ss(tacc + 256 + qt * 128, a + 2 * j, bv + 128 * j, idesc_o, true);
                }
            }
            const long long t1 = clock64();
            mma_commit(smem_u32(&bar[0]));
            ok = mbar_wait(smem_u32(&bar[0]), 0) && ok;
            const long long t2 = clock64();
            if (blockIdx.x == 0) { cycles[0] = t1 - t0; cycles[1] = ok ? t2 - t0 : -1; }
            done = 1;
        } else if (mode == 102 && tid == 32) {
            long long n = 0;
            while (!done && n < (1ll << 22)) {
                mbar_wait(smem_u32(&bar[1]), 0);
                fence_after_sync();
                ++n;
            }
            if (blockIdx.x == 0) cycles[8] = n;
        }
    } else if (mode == 64) {
        if (lane == 0 && warp < 2) {
            bool ok = true;
            const long long t0 = clock64();
            for (int i = 0; i < iters; ++i) {
                if (warp == 0) {
                    mbar_arrive(smem_u32(&bar[0]));
                    ok = mbar_wait(smem_u32(&bar[1]), i & 1) && ok;
                } else {
                    ok = mbar_wait(smem_u32(&bar[0]), i & 1) && ok;
                    mbar_arrive(smem_u32(&bar[1]));
                }
            }
            const long long t1 = clock64();
            if (blockIdx.x == 0 && warp == 0) { cycles[0] = t1 - t0; cycles[1] = ok ? t1 - t0 : -1; }
        }
    } else if (lane == 0 && warp < threads) {
        const unsigned idesc = instr_desc_bf16(M, N, b_mn);
        const unsigned long long a = smem_desc_sw128(smem_u32(base), 0);
        const unsigned long long b = b_mn ? smem_desc_sw128_mn(smem_u32(base) + 16384, 64 * 128, 1024u)
                                          : smem_desc_sw128(smem_u32(base) + 16384, 0);
        const unsigned b_step = b_mn ? 128u : 2u;               // 16 k: 16 rows of 128 bytes, or 32 bytes along a row
        const unsigned d = tacc + (unsigned)(warp * N);
        const long long t0 = clock64();
        if (mix) {
            const unsigned idesc_s = instr_desc_bf16(128, 64, false), idesc_o = instr_desc_bf16(128, 128, true);
            const unsigned long long bk = smem_desc_sw128(smem_u32(base) + 16384, 0);
            const unsigned long long bv = smem_desc_sw128_mn(smem_u32(base) + 32768, 64 * 128, 1024u);
            for (int i = 0; i < iters; ++i) {
#pragma unroll
                for (int qt = 0; qt < 2; ++qt) {
#pragma unroll
                    for (int j = 0; j < 8; ++j)
                        mma_ss(tacc + qt * 64, a + (unsigned long long)(((j >> 2) * (128 * 128) + (j & 3) * 32) >> 4),
                               bk + (unsigned long long)(((j >> 2) * (64 * 128) + (j & 3) * 32) >> 4), idesc_s, j > 0);
                    if (commits) mma_commit(smem_u32(&bar[1]));
                }
                if (commits) mma_commit(smem_u32(&bar[2]));
#pragma unroll
                for (int qt = 0; qt < 2; ++qt) {
#pragma unroll
                    for (int j = 0; j < 4; ++j) mma_ss(tacc + 256 + qt * 128, a + 2 * j, bv + 128 * j, idesc_o, true);
                    if (commits) mma_commit(smem_u32(&bar[1]));
                }
                if (commits) mma_commit(smem_u32(&bar[3]));
            }
        } else {
            for (int i = 0; i < iters; i += 8) {
#pragma unroll
                for (int j = 0; j < 8; ++j) mma_ss(d, a + 2 * (j & 3), b + b_step * (j & 3), idesc, true);
            }
        }
        const long long t1 = clock64();
        mma_commit(smem_u32(&bar[warp]));
        mbar_wait(smem_u32(&bar[warp]), 0);
        const long long t2 = clock64();
        if (blockIdx.x == 0) { cycles[warp * 2] = t1 - t0; cycles[warp * 2 + 1] = t2 - t0; }
        if (warp == 0) {
            done = 1;
            mbar_arrive(smem_u32(&bar[3]));
        }
    } else if (pollers && warp >= threads) {
        mbar_wait(smem_u32(&bar[3]), 0);
    } else if (hammer && warp >= threads) {
        // 16-byte stores, each warp over 8 KB of its own beyond the operand tiles, until the MMAs are done
        unsigned addr = smem_u32(base) + 49152 + (unsigned)(warp * 2048) + (unsigned)(lane * 16);
        long long n = 0;
        while (!done && n < (1ll << 24)) {
#pragma unroll
            for (int k = 0; k < 4; ++k)
                asm volatile("st.shared.v4.u32 [%0], {%1, %1, %1, %1};\n" ::"r"(addr + (unsigned)(k * 512)), "r"((unsigned)n));
            n += 4;
        }
        if (blockIdx.x == 0 && lane == 0 && warp == threads) cycles[8] = n * 32;
    }
    fence_before_sync();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tacc, 512);
}
}  // namespace

RB_EXPORT int rb_probe_tc5_rate(int ctas, int M, int N, int iters, int threads, int mode, long long* cycles, cudaStream_t st) {
    if ((M != 64 && M != 128) || N < 16 || N > 256 || N % 16 || threads < 1 || threads > 3 || threads * N > 512 || iters % 8)
        return (int)cudaErrorInvalidValue;
    if (mode < 32 && (mode & 1) && N != 128) return (int)cudaErrorInvalidValue;       // the MN-major tile here is 64 keys x 128
    if (mode < 32 && (mode & 4) && threads != 1) return (int)cudaErrorInvalidValue;
    if (mode >= 32 && mode != 32 && mode != 33 && (mode < 64 || mode > 69) && (mode < 100 || mode > 102)) return (int)cudaErrorInvalidValue;
    if (mode < 32 && (mode & 16) && (mode & 8)) return (int)cudaErrorInvalidValue;      // bar[3] is the pollers' barrier then
    cudaError_t e = cudaFuncSetAttribute(tc5_rate_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
    if (e != cudaSuccess) return (int)e;
    tc5_rate_kernel<<<ctas, (mode < 32 && (mode & 16)) ? 352 : 128, 64 * 1024, st>>>(M, N, iters, threads, mode, cycles);
    return rb_launch_status();
}
