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

RB_EXPORT int rb_embedding(const void* table, int table_dtype, const int* tokens, float* stream,
                           int T, int H, int V, cudaStream_t st) {
    if (T <= 0) return 0;
    const int threads = H >= 1024 ? 256 : 128;
    if (table_dtype == RB_F32)
        embedding_kernel<float><<<T, threads, 0, st>>>((const float*)table, tokens, stream, H, V);
    else
        embedding_kernel<bf16><<<T, threads, 0, st>>>((const bf16*)table, tokens, stream, H, V);
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

RB_EXPORT int rb_add_rmsnorm(float* stream, const void* delta, const int* rows, const void* w,
                             int w_dtype, float eps, float offset, void* out, int act_dtype,
                             int n_rows, int H, cudaStream_t st) {
    if (n_rows <= 0) return 0;
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
// out[t, i] = silu(gu[t, i]) * gu[t, I + i];  gu is [T, 2I] with gate columns first.
template <typename TA>
__global__ void swiglu_kernel(const TA* __restrict__ gu, TA* __restrict__ out, int T, int I) {
    const size_t total = (size_t)T * I;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * blockDim.x) {
        const size_t t = idx / I, i = idx - t * I;
        const float g = to_f32(gu[t * 2 * I + i]);
        const float u = to_f32(gu[t * 2 * I + I + i]);
        out[idx] = from_f32<TA>(g / (1.0f + expf(-g)) * u);
    }
}

// bfloat16 with I a multiple of 8: eight elements (16 bytes) per thread and iteration.
__global__ void swiglu_bf16x8_kernel(const bf16* __restrict__ gu, bf16* __restrict__ out, int T, int I) {
    const int I8 = I >> 3;
    const size_t total = (size_t)T * I8;
    for (size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
         idx += (size_t)gridDim.x * blockDim.x) {
        const size_t t = idx / I8, i = (idx - t * I8) << 3;
        const uint4 gv = *(const uint4*)(gu + t * 2 * I + i);
        const uint4 uv = *(const uint4*)(gu + t * 2 * I + I + i);
        const bf16* g = (const bf16*)&gv;
        const bf16* u = (const bf16*)&uv;
        uint4 ov;
        bf16* o = (bf16*)&ov;
#pragma unroll
        for (int k = 0; k < 8; ++k) {
            const float gf = __bfloat162float(g[k]);
            o[k] = __float2bfloat16_rn(gf / (1.0f + expf(-gf)) * __bfloat162float(u[k]));
        }
        *(uint4*)(out + t * I + i) = ov;
    }
}

RB_EXPORT int rb_swiglu(const void* gu, void* out, int act_dtype, int T, int I, cudaStream_t st) {
    if (T <= 0) return 0;
    const int threads = 256;
    if (act_dtype == RB_BF16 && (I % 8) == 0 && ((uintptr_t)gu % 16) == 0 && ((uintptr_t)out % 16) == 0) {
        const size_t total = (size_t)T * (I >> 3);
        int blocks = (int)((total + threads - 1) / threads);
        if (blocks > 148 * 16) blocks = 148 * 16;
        swiglu_bf16x8_kernel<<<blocks, threads, 0, st>>>((const bf16*)gu, (bf16*)out, T, I);
        return rb_launch_status();
    }
    const size_t total = (size_t)T * I;
    int blocks = (int)((total + threads - 1) / threads);
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (act_dtype == RB_F32)
        swiglu_kernel<float><<<blocks, threads, 0, st>>>((const float*)gu, (float*)out, T, I);
    else
        swiglu_kernel<bf16><<<blocks, threads, 0, st>>>((const bf16*)gu, (bf16*)out, T, I);
    return rb_launch_status();
}
