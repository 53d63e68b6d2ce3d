// Per-head q/k RMSNorm, rotary position encoding and the write into the paged KV cache, fused.
//
// Input is the row-major output of the fused QKV projection, [T, ld] with q heads first, then
// k heads, then v heads.  For every token:
//   q head: (optional) RMSNorm over head_dim, rotation, stored back in place;
//   k head: (optional) RMSNorm, rotation, stored to the K page of the token's position
//           (write_kv = 0: stored back in place, nothing is written to the cache);
//   v head: copied to the V page.
// The reference norms before it rotates (rollout/monkey_patch/qwen3.py:29-30) and rotates inside
// its attention kernels (rollout/attention.py:10-25, half-split pairs (i, i + R/2)); it caches
// un-rotated keys because cached tokens can change position there.  Here a cached token keeps
// its position, so the key is rotated once, before the write.  Norm and rotation are float32,
// with one rounding at the store.
//
// Cache layout of one layer: [num_pages, Hkv, P, D]; the page of a token is
// block_table[segment][pos / P], its row in the page pos % P.
#include "common.cuh"

// Two neighbouring elements at a time.
template <typename TA> struct Pair;
template <> struct Pair<float> {
    static __device__ __forceinline__ float2 load(const float* p) { return *reinterpret_cast<const float2*>(p); }
    static __device__ __forceinline__ void store(float* p, float2 v) { *reinterpret_cast<float2*>(p) = v; }
};
template <> struct Pair<bf16> {
    static __device__ __forceinline__ float2 load(const bf16* p) {
        return __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(p));
    }
    static __device__ __forceinline__ void store(bf16* p, float2 v) {
        *reinterpret_cast<__nv_bfloat162*>(p) = __floats2bfloat162_rn(v.x, v.y);
    }
};

// One warp per (token, head).  A lane holds the element pairs (i, i+1) of the first rotary half and
// their partners (i + R/2, i + R/2 + 1) in registers, so a head is read once; head sizes up to 256.
constexpr int ROPE_MAX_J = 2;                     // pairs of pairs per lane: R/2 <= 128

template <typename TA>
__global__ void qk_norm_rope_write_kernel(
        TA* __restrict__ qkv, int ld,
        const void* __restrict__ qw, const void* __restrict__ kw, int w_dtype, float eps, float offset,
        const float* __restrict__ cos_t, const float* __restrict__ sin_t, int rot_dim,
        const int* __restrict__ pos, const int* __restrict__ tok_seg,
        const int* __restrict__ block_table, int bt_stride, int page_size,
        TA* __restrict__ kpool, TA* __restrict__ vpool,
        int Hq, int Hkv, int D, int write_kv) {
    pdl_launch_dependents();
    pdl_wait();
    const int t = blockIdx.x;
    const int lane = threadIdx.x & 31;
    const int hh = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5);      // one warp per head
    const int n_heads = write_kv ? Hq + 2 * Hkv : Hq + Hkv;   // without a write, k is normed and rotated in place
    if (hh >= n_heads) return;
    const int p = pos[t];
    const int half = rot_dim >> 1;
    long long slot_base = -1;     // element offset of (page, kv head 0, row) in a pool
    if (write_kv && hh >= Hq) {
        const int page = block_table[(size_t)tok_seg[t] * bt_stride + p / page_size];
        if (page >= 0) slot_base = ((long long)page * Hkv * page_size + (p % page_size)) * D;
    }
    TA* x = qkv + (size_t)t * ld + (size_t)hh * D;
    if (hh >= Hq + Hkv) {                           // v head: copy
        if (slot_base < 0) return;
        TA* dst = vpool + slot_base + (long long)(hh - Hq - Hkv) * page_size * D;
        for (int i = 2 * lane; i < D; i += 64) Pair<TA>::store(dst + i, Pair<TA>::load(x + i));
        return;
    }
    const bool is_k = hh >= Hq;
    const void* w = is_k ? kw : qw;
    TA* dst = x;
    if (is_k && write_kv) {
        if (slot_base < 0) return;
        dst = kpool + slot_base + (long long)(hh - Hq) * page_size * D;
    }
    float2 a[ROPE_MAX_J], b[ROPE_MAX_J];            // first-half pairs and their second-half partners
    float ss = 0.f;
#pragma unroll
    for (int j = 0; j < ROPE_MAX_J; ++j) {
        const int i = 2 * lane + 64 * j;
        if (i < half) {
            a[j] = Pair<TA>::load(x + i);
            b[j] = Pair<TA>::load(x + i + half);
            ss += a[j].x * a[j].x + a[j].y * a[j].y + b[j].x * b[j].x + b[j].y * b[j].y;
        }
    }
    for (int i = rot_dim + 2 * lane; i < D; i += 64) {        // dims beyond the rotary width
        const float2 v = Pair<TA>::load(x + i);
        ss += v.x * v.x + v.y * v.y;
    }
    float rstd = 1.f;
    if (w) {
        ss = warp_sum(ss);
        rstd = 1.0f / sqrtf(ss / (float)D + eps);
    }
    const float* cs = cos_t + (size_t)p * half;
    const float* sn = sin_t + (size_t)p * half;
#pragma unroll
    for (int j = 0; j < ROPE_MAX_J; ++j) {
        const int i = 2 * lane + 64 * j;
        if (i < half) {
            float2 x1 = make_float2(a[j].x * rstd, a[j].y * rstd), x2 = make_float2(b[j].x * rstd, b[j].y * rstd);
            if (w) {
                x1.x *= offset + load_as_f32(w, w_dtype, i);        x1.y *= offset + load_as_f32(w, w_dtype, i + 1);
                x2.x *= offset + load_as_f32(w, w_dtype, i + half); x2.y *= offset + load_as_f32(w, w_dtype, i + half + 1);
            }
            const float2 c = *reinterpret_cast<const float2*>(cs + i), s = *reinterpret_cast<const float2*>(sn + i);
            Pair<TA>::store(dst + i, make_float2(x1.x * c.x - x2.x * s.x, x1.y * c.y - x2.y * s.y));
            Pair<TA>::store(dst + i + half, make_float2(x2.x * c.x + x1.x * s.x, x2.y * c.y + x1.y * s.y));
        }
    }
    for (int i = rot_dim + 2 * lane; i < D; i += 64) {
        float2 v = Pair<TA>::load(x + i);
        v.x *= rstd; v.y *= rstd;
        if (w) { v.x *= offset + load_as_f32(w, w_dtype, i); v.y *= offset + load_as_f32(w, w_dtype, i + 1); }
        Pair<TA>::store(dst + i, v);
    }
}

RB_EXPORT int rb_qk_norm_rope_write(
        void* qkv, int ld, const void* qw, const void* kw, int w_dtype, float eps, float offset,
        const float* cos_t, const float* sin_t, int rot_dim,
        const int* pos, const int* tok_seg, const int* block_table, int bt_stride, int page_size,
        void* kpool, void* vpool, int act_dtype, int T, int Hq, int Hkv, int D, int write_kv,
        cudaStream_t st) {
    if (T <= 0) return 0;
    // pairs of neighbours: the rotary half must be even, and a lane holds at most ROPE_MAX_J pairs of pairs
    if (rot_dim > D || (rot_dim & 3) || (D & 1) || rot_dim > 128 * ROPE_MAX_J) return (int)cudaErrorInvalidValue;
    const int threads = 128;
    const int heads = write_kv ? Hq + 2 * Hkv : Hq + Hkv;
    const dim3 grid(T, (heads + 3) / 4);
    if (act_dtype == RB_F32)
        return rb_launch_pdl(qk_norm_rope_write_kernel<float>, grid, dim3(threads), 0, st,
            (float*)qkv, ld, qw, kw, w_dtype, eps, offset, cos_t, sin_t, rot_dim, pos, tok_seg,
            block_table, bt_stride, page_size, (float*)kpool, (float*)vpool, Hq, Hkv, D, write_kv);
    return rb_launch_pdl(qk_norm_rope_write_kernel<bf16>, grid, dim3(threads), 0, st,
            (bf16*)qkv, ld, qw, kw, w_dtype, eps, offset, cos_t, sin_t, rot_dim, pos, tok_seg,
            block_table, bt_stride, page_size, (bf16*)kpool, (bf16*)vpool, Hq, Hkv, D, write_kv);
}
