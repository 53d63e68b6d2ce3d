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
namespace {
__global__ void __launch_bounds__(128) tc5_rate_kernel(int M, int N, int iters, int threads, long long* cycles) {
    using namespace tc5;
    extern __shared__ unsigned char probe_smem[];
    unsigned char* base = reinterpret_cast<unsigned char*>((reinterpret_cast<uintptr_t>(probe_smem) + 1023) & ~uintptr_t(1023));
    __shared__ __align__(8) unsigned long long bar[4];
    __shared__ unsigned tmem_slot;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    for (int i = tid; i < 48 * 1024 / 4; i += 128) reinterpret_cast<unsigned*>(base)[i] = 0x3c003c00u;     // bf16 1.0
    if (warp == 0) tmem_alloc(smem_u32(&tmem_slot), 512);
    if (tid == 0) {
        for (int i = 0; i < 4; ++i) mbar_init(smem_u32(&bar[i]), 1);
        mbar_init_fence();
    }
    fence_proxy_async();
    fence_before_sync();
    __syncthreads();
    fence_after_sync();
    const unsigned tacc = tmem_slot;
    if (lane == 0 && warp < threads) {
        const unsigned idesc = instr_desc_bf16(M, N);
        const unsigned long long a = smem_desc_sw128(smem_u32(base), 0), b = smem_desc_sw128(smem_u32(base) + 16384, 0);
        const unsigned d = tacc + (unsigned)(warp * N);
        const long long t0 = clock64();
        for (int i = 0; i < iters; i += 8) {
#pragma unroll
            for (int j = 0; j < 8; ++j) mma_ss(d, a + 2 * (j & 3), b + 2 * (j & 3), idesc, true);
        }
        const long long t1 = clock64();
        mma_commit(smem_u32(&bar[warp]));
        mbar_wait(smem_u32(&bar[warp]), 0);
        const long long t2 = clock64();
        if (blockIdx.x == 0) { cycles[warp * 2] = t1 - t0; cycles[warp * 2 + 1] = t2 - t0; }
    }
    fence_before_sync();
    __syncthreads();
    if (warp == 0) tmem_dealloc(tacc, 512);
}
}  // namespace

RB_EXPORT int rb_probe_tc5_rate(int ctas, int M, int N, int iters, int threads, long long* cycles, cudaStream_t st) {
    if ((M != 64 && M != 128) || N < 16 || N > 256 || N % 16 || threads < 1 || threads > 4 || threads * N > 512 || iters % 8)
        return (int)cudaErrorInvalidValue;
    cudaError_t e = cudaFuncSetAttribute(tc5_rate_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024);
    if (e != cudaSuccess) return (int)e;
    tc5_rate_kernel<<<ctas, 128, 64 * 1024, st>>>(M, N, iters, threads, cycles);
    return rb_launch_status();
}
