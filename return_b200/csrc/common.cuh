// Shared helpers of the sm_100a kernels: element types, warp and block reductions.
//
// Every exported launcher is `extern "C"`, takes raw device pointers, plain integers and a
// cudaStream_t, launches on that stream and returns the cudaError_t of the launch as an int
// (0 = success).  Nothing here allocates device memory.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <mutex>

#define RB_EXPORT extern "C" __attribute__((visibility("default")))

// dtype codes shared with return_b200/ext/ops.py
#define RB_F32 0
#define RB_BF16 1

typedef __nv_bfloat16 bf16;

// Host-side set-up that CUDA keeps per device (cudaFuncSetAttribute, a device's properties): a launcher holds one of
// these as a static and runs its set-up the first time it is called with each device current, under a lock.
// `amount` lets a set-up be run again when more is asked for than before (a larger shared-memory limit).
struct PerDevice {
    static constexpr int MAX_DEVICES = 64;
    std::mutex mu;
    long long have[MAX_DEVICES] = {0};
    template <typename F>
    int once(F set_up, long long amount = 1) {             // set_up(device) -> cudaError_t; returns 0 or the CUDA error
        int dev = 0;
        cudaError_t e = cudaGetDevice(&dev);
        if (e != cudaSuccess) return (int)e;
        if (dev < 0 || dev >= MAX_DEVICES) return (int)cudaErrorInvalidDevice;
        std::lock_guard<std::mutex> lock(mu);
        if (have[dev] >= amount) return 0;
        e = set_up(dev);
        if (e == cudaSuccess) have[dev] = amount;
        return (int)e;
    }
};

// Streaming multiprocessors of the current device (0 if it cannot be asked).
static inline int rb_num_sms() {
    static std::mutex mu;
    static int sms[PerDevice::MAX_DEVICES] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= PerDevice::MAX_DEVICES) return 0;
    std::lock_guard<std::mutex> lock(mu);
    if (sms[dev] == 0) cudaDeviceGetAttribute(&sms[dev], cudaDevAttrMultiProcessorCount, dev);
    return sms[dev];
}

__device__ __forceinline__ float to_f32(float x) { return x; }
__device__ __forceinline__ float to_f32(bf16 x) { return __bfloat162float(x); }

template <typename T> __device__ __forceinline__ T from_f32(float x);
template <> __device__ __forceinline__ float from_f32<float>(float x) { return x; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float x) { return __float2bfloat16_rn(x); }

// Loads a weight element whose storage dtype is only known at run time.
__device__ __forceinline__ float load_as_f32(const void* p, int dtype, size_t i) {
    return dtype == RB_F32 ? ((const float*)p)[i] : __bfloat162float(((const bf16*)p)[i]);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.  `scratch` holds 33 floats.
// The order of the additions is fixed, so the result does not depend on timing.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarps ? scratch[lane] : 0.f;
        t = warp_sum(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

__device__ __forceinline__ float block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < nwarps ? scratch[lane] : -INFINITY;
        t = warp_max(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

static inline int rb_launch_status() { return (int)cudaGetLastError(); }

// Programmatic dependent launch.  A kernel launched with rb_launch_pdl may begin while the kernel
// before it in the stream is still draining: its CTAs are placed as soon as every CTA of the
// predecessor has called pdl_launch_dependents() (or exited), and run up to pdl_wait(), which
// returns once the predecessor has finished and its writes are visible.  The rule every such
// kernel keeps: before pdl_wait() it touches nothing a predecessor could have written (it may read
// weights, which no kernel writes) and writes nothing at all.  This hides launch and ramp-up
// latency between the many short kernels of a decode step; it is captured into CUDA graphs as
// programmatic dependency edges.
//
// RB_PDL_MODE: 0 launch attribute only (the successor starts when this kernel ends); 1 trigger at
// the start of every kernel; 2 trigger when a kernel's main loop is done, so that only its
// epilogue and tail overlap the successor's prologue; 3 plain launches.
#ifndef RB_PDL_MODE
#define RB_PDL_MODE 2
#endif
__device__ __forceinline__ void pdl_wait() {
#if RB_PDL_MODE != 3
    asm volatile("griddepcontrol.wait;" ::: "memory");
#endif
}
__device__ __forceinline__ void pdl_launch_dependents() {       // at the start of a kernel
#if RB_PDL_MODE == 1
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
#endif
}
__device__ __forceinline__ void pdl_trigger_late() {            // after a kernel's main loop
#if RB_PDL_MODE == 2
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
#endif
}

template <typename... KArgs, typename... Args>
static inline int rb_launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st,
                                Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = RB_PDL_MODE == 3 ? 0 : 1;
    return (int)cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}
