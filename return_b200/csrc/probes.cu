// Measurement probes (not on the engine's path): the issue rate and latency of mma.sync.m16n8k16
// on this part, which is the ceiling of the kernels that use it.
#include "common.cuh"

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
