// Embedding gather, fused residual-add + RMSNorm, SwiGLU, row gather.
//
// The residual stream is float32 in both precisions; the "delta" a block adds to it and the
// normalised activations are in the activation dtype (float32 or bfloat16).  All arithmetic
// is float32 with one rounding at the store, as in the reference's Triton kernels
// (rollout/fused.py:6-17 for the norm, rollout/fused.py:103-127 for SwiGLU).
#include "common.cuh"

// ---------------------------------------------------------------- embedding
// stream[t, :] = float(table[tokens[t], :]).  A token id outside [0, V) writes NaN so that the
// fault shows in the logits instead of reading foreign memory.
template <typename TW>
__global__ void embedding_kernel(const TW* __restrict__ table, const int* __restrict__ tokens,
                                 float* __restrict__ stream, int H, int V) {
    const int t = blockIdx.x;
    const int id = tokens[t];
    float* dst = stream + (size_t)t * H;
    if (id < 0 || id >= V) {
        for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = __int_as_float(0x7fc00000);
        return;
    }
    const TW* src = table + (size_t)id * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = to_f32(src[i]);
}

// Sixteen bytes of the table per thread and iteration, for rows whose length allows it.
template <typename TW>
__global__ void embedding_vec_kernel(const TW* __restrict__ table, const int* __restrict__ tokens,
                                     float* __restrict__ stream, int H, int V) {
    constexpr int E = 16 / sizeof(TW);
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int id = tokens[t];
    float* dst = stream + (size_t)t * H;
    const bool bad = id < 0 || id >= V;
    const TW* src = table + (size_t)(bad ? 0 : id) * H;
    for (int i = threadIdx.x * E; i < H; i += blockDim.x * E) {
        const uint4 raw = *reinterpret_cast<const uint4*>(src + i);
        const TW* e = reinterpret_cast<const TW*>(&raw);
        float out[E];
#pragma unroll
        for (int k = 0; k < E; ++k) out[k] = bad ? __int_as_float(0x7fc00000) : to_f32(e[k]);
#pragma unroll
        for (int k = 0; k < E; k += 4)
            *reinterpret_cast<float4*>(dst + i + k) = make_float4(out[k], out[k + 1], out[k + 2], out[k + 3]);
    }
}

RB_EXPORT int rb_embedding(const void* table, int table_dtype, const int* tokens, float* stream,
                           int T, int H, int V, cudaStream_t st) {
    if (T <= 0) return 0;
    const int threads = H >= 1024 ? 256 : 128;
    const bool aligned = ((uintptr_t)table % 16) == 0 && ((uintptr_t)stream % 16) == 0;
    if (table_dtype == RB_F32) {
        if (aligned && H % 4 == 0)
            return rb_launch_pdl(embedding_vec_kernel<float>, dim3(T), dim3(threads), 0, st, (const float*)table, tokens, stream, H, V);
        else
            embedding_kernel<float><<<T, threads, 0, st>>>((const float*)table, tokens, stream, H, V);
    } else {
        if (aligned && H % 8 == 0)
            return rb_launch_pdl(embedding_vec_kernel<bf16>, dim3(T), dim3(threads), 0, st, (const bf16*)table, tokens, stream, H, V);
        else
            embedding_kernel<bf16><<<T, threads, 0, st>>>((const bf16*)table, tokens, stream, H, V);
    }
    return rb_launch_status();
}

// ---------------------------------------------------------------- residual add + RMSNorm
// x = stream[row] (+ delta[row]);  if rows == nullptr the sum is written back to the stream;
// out[blockIdx.x] = x * rsqrt(mean(x^2) + eps) * (offset + w).
// With `rows` the kernel normalises only the listed rows (the rows whose logits are wanted)
// and leaves the stream untouched, so a row may be listed twice.
template <typename TA>
__global__ void add_rmsnorm_kernel(float* __restrict__ stream, const TA* __restrict__ delta,
                                   const int* __restrict__ rows, const void* __restrict__ w,
                                   int w_dtype, float eps, float offset, TA* __restrict__ out, int H) {
    extern __shared__ float smem[];
    float* xrow = smem;          // H floats
    float* scratch = smem + H;   // 33 floats
    const int orow = blockIdx.x;
    const int irow = rows ? rows[orow] : orow;
    float* s = stream + (size_t)irow * H;
    const TA* d = delta ? delta + (size_t)irow * H : nullptr;
    float ss = 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float x = s[i];
        if (d) x += to_f32(d[i]);
        xrow[i] = x;
        if (d && !rows) s[i] = x;
        ss += x * x;
    }
    ss = block_sum(ss, scratch);
    const float rstd = 1.0f / sqrtf(ss / (float)H + eps);
    TA* o = out + (size_t)orow * H;
    for (int i = threadIdx.x; i < H; i += blockDim.x)
        o[i] = from_f32<TA>(xrow[i] * rstd * (offset + load_as_f32(w, w_dtype, i)));
}

// The same, four elements per vector and up to VPT vectors per thread held in registers: every
// load of a row is in flight at once, which is what a step of a few rows needs (it is bound by
// the latency of one trip to memory, not by bandwidth).  Needs H % 4 == 0 and H <= 4 * VPT * threads.
template <typename TA> struct Vec4;
template <> struct Vec4<float> {
    static __device__ __forceinline__ float4 load(const float* p) { return *reinterpret_cast<const float4*>(p); }
    static __device__ __forceinline__ void store(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
};
template <> struct Vec4<bf16> {
    static __device__ __forceinline__ float4 load(const bf16* p) {
        const uint2 raw = *reinterpret_cast<const uint2*>(p);
        const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(&raw.x);
        const __nv_bfloat162 b = *reinterpret_cast<const __nv_bfloat162*>(&raw.y);
        return make_float4(__low2float(a), __high2float(a), __low2float(b), __high2float(b));
    }
    static __device__ __forceinline__ void store(bf16* p, float4 v) {
        __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
        uint2 raw;
        raw.x = *reinterpret_cast<unsigned*>(&a);
        raw.y = *reinterpret_cast<unsigned*>(&b);
        *reinterpret_cast<uint2*>(p) = raw;
    }
};

template <typename TA, typename TW, int VPT>
__global__ void add_rmsnorm_vec_kernel(float* __restrict__ stream, const TA* __restrict__ delta,
                                       const int* __restrict__ rows, const TW* __restrict__ w,
                                       float eps, float offset, TA* __restrict__ out, int H) {
    __shared__ float scratch[33];
    pdl_launch_dependents();
    const int orow = blockIdx.x;
    const int nvec = H >> 2;
    float4 x[VPT], wv[VPT];
#pragma unroll
    for (int v = 0; v < VPT; ++v) {                      // the norm weight is nobody's output: read it early
        const int i = threadIdx.x + v * blockDim.x;
        wv[v] = i < nvec ? Vec4<TW>::load(w + 4 * i) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    pdl_wait();
    const int irow = rows ? rows[orow] : orow;
    float* s = stream + (size_t)irow * H;
    const TA* d = delta ? delta + (size_t)irow * H : nullptr;
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
        const int i = threadIdx.x + v * blockDim.x;
        x[v] = i < nvec ? Vec4<float>::load(s + 4 * i) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
    if (d) {
#pragma unroll
        for (int v = 0; v < VPT; ++v) {
            const int i = threadIdx.x + v * blockDim.x;
            if (i < nvec) {
                const float4 dv = Vec4<TA>::load(d + 4 * i);
                x[v].x += dv.x; x[v].y += dv.y; x[v].z += dv.z; x[v].w += dv.w;
            }
        }
    }
    float ss = 0.f;
#pragma unroll
    for (int v = 0; v < VPT; ++v) ss += x[v].x * x[v].x + x[v].y * x[v].y + x[v].z * x[v].z + x[v].w * x[v].w;
    if (d && !rows) {
#pragma unroll
        for (int v = 0; v < VPT; ++v) {
            const int i = threadIdx.x + v * blockDim.x;
            if (i < nvec) Vec4<float>::store(s + 4 * i, x[v]);
        }
    }
    pdl_trigger_late();
    ss = block_sum(ss, scratch);
    const float rstd = 1.0f / sqrtf(ss / (float)H + eps);
    TA* o = out + (size_t)orow * H;
#pragma unroll
    for (int v = 0; v < VPT; ++v) {
        const int i = threadIdx.x + v * blockDim.x;
        if (i < nvec)
            Vec4<TA>::store(o + 4 * i, make_float4(x[v].x * rstd * (offset + wv[v].x), x[v].y * rstd * (offset + wv[v].y),
                                                   x[v].z * rstd * (offset + wv[v].z), x[v].w * rstd * (offset + wv[v].w)));
    }
}

template <typename TA, typename TW>
static int launch_add_rmsnorm_vec(float* stream, const void* delta, const int* rows, const void* w, float eps,
                                  float offset, void* out, int n_rows, int H, cudaStream_t st) {
    const int nvec = H >> 2;
    int threads = 128;
    while (threads < 1024 && threads * 4 < nvec) threads <<= 1;
    if (threads >= nvec)
        return rb_launch_pdl(add_rmsnorm_vec_kernel<TA, TW, 1>, dim3(n_rows), dim3(threads), 0, st, stream, (const TA*)delta, rows, (const TW*)w, eps, offset, (TA*)out, H);
    else if (threads * 2 >= nvec)
        return rb_launch_pdl(add_rmsnorm_vec_kernel<TA, TW, 2>, dim3(n_rows), dim3(threads), 0, st, stream, (const TA*)delta, rows, (const TW*)w, eps, offset, (TA*)out, H);
    else
        return rb_launch_pdl(add_rmsnorm_vec_kernel<TA, TW, 4>, dim3(n_rows), dim3(threads), 0, st, stream, (const TA*)delta, rows, (const TW*)w, eps, offset, (TA*)out, H);
    return rb_launch_status();
}

RB_EXPORT int rb_add_rmsnorm(float* stream, const void* delta, const int* rows, const void* w,
                             int w_dtype, float eps, float offset, void* out, int act_dtype,
                             int n_rows, int H, cudaStream_t st) {
    if (n_rows <= 0) return 0;
    const bool aligned = ((uintptr_t)stream % 16) == 0 && ((uintptr_t)delta % 16) == 0 &&
                         ((uintptr_t)w % 16) == 0 && ((uintptr_t)out % 16) == 0;
    if (aligned && H % 4 == 0 && H <= 4 * 4 * 1024) {
        if (act_dtype == RB_F32 && w_dtype == RB_F32) return launch_add_rmsnorm_vec<float, float>(stream, delta, rows, w, eps, offset, out, n_rows, H, st);
        if (act_dtype == RB_F32) return launch_add_rmsnorm_vec<float, bf16>(stream, delta, rows, w, eps, offset, out, n_rows, H, st);
        if (w_dtype == RB_F32) return launch_add_rmsnorm_vec<bf16, float>(stream, delta, rows, w, eps, offset, out, n_rows, H, st);
        return launch_add_rmsnorm_vec<bf16, bf16>(stream, delta, rows, w, eps, offset, out, n_rows, H, st);
    }
    const size_t smem = (size_t)(H + 33) * sizeof(float);
    if (smem > 200 * 1024) return (int)cudaErrorInvalidValue;
    int threads = 128;
    while (threads < 1024 && threads * 8 < H) threads <<= 1;
    if (act_dtype == RB_F32) {
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(add_rmsnorm_kernel<float>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        add_rmsnorm_kernel<float><<<n_rows, threads, smem, st>>>(stream, (const float*)delta, rows, w, w_dtype,
                                                                eps, offset, (float*)out, H);
    } else {
        if (smem > 48 * 1024)
            cudaFuncSetAttribute(add_rmsnorm_kernel<bf16>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        add_rmsnorm_kernel<bf16><<<n_rows, threads, smem, st>>>(stream, (const bf16*)delta, rows, w, w_dtype,
                                                               eps, offset, (bf16*)out, H);
    }
    return rb_launch_status();
}

// ---------------------------------------------------------------- plain RMSNorm over the last dim
// y[r, :] = x[r, :] * rsqrt(mean(x^2) + eps) * (offset + w), rows of length N (any N), one warp a row.
// The stand-alone form of the norm, used for kernel tests and by parts that need no residual.
template <typename TA>
__global__ void rmsnorm_rows_kernel(const TA* __restrict__ x, const void* __restrict__ w, int w_dtype,
                                    float eps, float offset, TA* __restrict__ y, int rows, int N) {
    const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (warp >= rows) return;
    const TA* xr = x + (size_t)warp * N;
    float ss = 0.f;
    for (int i = lane; i < N; i += 32) { float v = to_f32(xr[i]); ss += v * v; }
    ss = warp_sum(ss);
    const float rstd = 1.0f / sqrtf(ss / (float)N + eps);
    TA* yr = y + (size_t)warp * N;
    for (int i = lane; i < N; i += 32)
        yr[i] = from_f32<TA>(to_f32(xr[i]) * rstd * (offset + load_as_f32(w, w_dtype, i)));
}

RB_EXPORT int rb_rmsnorm_rows(const void* x, const void* w, int w_dtype, float eps, float offset, void* y,
                              int act_dtype, int rows, int N, cudaStream_t st) {
    if (rows <= 0) return 0;
    const int threads = 128, per_block = threads / 32;
    const int blocks = (rows + per_block - 1) / per_block;
    if (act_dtype == RB_F32)
        rmsnorm_rows_kernel<float><<<blocks, threads, 0, st>>>((const float*)x, w, w_dtype, eps, offset, (float*)y, rows, N);
    else
        rmsnorm_rows_kernel<bf16><<<blocks, threads, 0, st>>>((const bf16*)x, w, w_dtype, eps, offset, (bf16*)y, rows, N);
    return rb_launch_status();
}

// ---------------------------------------------------------------- SwiGLU
// out[t, i] = silu(gate) * up.  gu is [T, 2I].  block == 0: gate columns [0, I), up columns [I, 2I)
// (the reference's concatenation, rollout/monkey_patch/qwen3.py:99-105).  block == 8: columns come in
// blocks of 8 gate then 8 up (the layout that lets a matrix product's epilogue do this step).
template <typename TA>
__global__ void swiglu_kernel(const TA* __restrict__ gu, TA* __restrict__ out, int T, int I, int block) {
    const size_t total = (size_t)T * I;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * blockDim.x) {
        const size_t t = idx / I, i = idx - t * I;
        const size_t gi = block ? (i / block) * 2 * block + i % block : i;
        const size_t ui = block ? gi + block : I + i;
        const float g = to_f32(gu[t * 2 * I + gi]);
        const float u = to_f32(gu[t * 2 * I + ui]);
        out[idx] = from_f32<TA>(g / (1.0f + expf(-g)) * u);
    }
}

// bfloat16 with I a multiple of 8: eight elements (16 bytes) per thread, two such pieces in flight.
// The exponential and the division are the fast float32 forms (a few units in the last place, far
// below the rounding to bfloat16 that follows): with the accurate ones the kernel is bound by
// instruction issue, not by memory.
__device__ __forceinline__ uint4 swiglu8(const uint4 gv, const uint4 uv) {
    const bf16* g = (const bf16*)&gv;
    const bf16* u = (const bf16*)&uv;
    uint4 ov;
    bf16* o = (bf16*)&ov;
#pragma unroll
    for (int k = 0; k < 8; ++k) {
        const float gf = __bfloat162float(g[k]);
        o[k] = __float2bfloat16_rn(__fdividef(gf, 1.0f + __expf(-gf)) * __bfloat162float(u[k]));
    }
    return ov;
}

__global__ void swiglu_bf16x8_kernel(const bf16* __restrict__ gu, bf16* __restrict__ out, int T, int I, int block) {
    pdl_launch_dependents();
    pdl_wait();
    const int I8 = I >> 3;
    const size_t total = (size_t)T * I8;
    const size_t stride = (size_t)gridDim.x * blockDim.x;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += 2 * stride) {
        const size_t idx2 = idx + stride;
        const bool two = idx2 < total;
        const size_t t = idx / I8, i = (idx - t * I8) << 3;
        const size_t t2 = two ? idx2 / I8 : t, i2 = two ? (idx2 - t2 * I8) << 3 : i;
        const uint4 gv = *(const uint4*)(gu + t * 2 * I + (block ? 2 * i : i));
        const uint4 uv = *(const uint4*)(gu + t * 2 * I + (block ? 2 * i + 8 : I + i));
        const uint4 gv2 = *(const uint4*)(gu + t2 * 2 * I + (block ? 2 * i2 : i2));
        const uint4 uv2 = *(const uint4*)(gu + t2 * 2 * I + (block ? 2 * i2 + 8 : I + i2));
        *(uint4*)(out + t * I + i) = swiglu8(gv, uv);
        if (two) *(uint4*)(out + t2 * I + i2) = swiglu8(gv2, uv2);
    }
}

RB_EXPORT int rb_swiglu(const void* gu, void* out, int act_dtype, int T, int I, int block, cudaStream_t st) {
    if (T <= 0) return 0;
    if (block != 0 && (block != 8 || I % 8)) return (int)cudaErrorInvalidValue;
    const int threads = 256;
    if (act_dtype == RB_BF16 && (I % 8) == 0 && ((uintptr_t)gu % 16) == 0 && ((uintptr_t)out % 16) == 0) {
        const size_t total = (size_t)T * (I >> 3);
        int blocks = (int)((total + threads - 1) / threads);
        if (blocks > 148 * 16) blocks = 148 * 16;
        return rb_launch_pdl(swiglu_bf16x8_kernel, dim3(blocks), dim3(threads), 0, st, (const bf16*)gu, (bf16*)out, T, I, block);
    }
    const size_t total = (size_t)T * I;
    int blocks = (int)((total + threads - 1) / threads);
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (act_dtype == RB_F32)
        swiglu_kernel<float><<<blocks, threads, 0, st>>>((const float*)gu, (float*)out, T, I, block);
    else
        swiglu_kernel<bf16><<<blocks, threads, 0, st>>>((const bf16*)gu, (bf16*)out, T, I, block);
    return rb_launch_status();
}

