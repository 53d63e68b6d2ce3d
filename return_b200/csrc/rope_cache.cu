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
    const int warp = blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5);      // one warp per head
    const int nwarps = gridDim.y * (blockDim.x >> 5);
    const int p = pos[t];
    const int half = rot_dim >> 1;
    const float* cs = cos_t + (size_t)p * half;
    const float* sn = sin_t + (size_t)p * half;
    long long slot_base = -1;     // element offset of (page, kv head 0, row) in a pool
    if (write_kv) {
        const int page = block_table[(size_t)tok_seg[t] * bt_stride + p / page_size];
        if (page >= 0) slot_base = ((long long)page * Hkv * page_size + (p % page_size)) * D;
    }
    const int n_heads = write_kv ? Hq + 2 * Hkv : Hq + Hkv;   // without a write, k is normed and rotated in place
    for (int hh = warp; hh < n_heads; hh += nwarps) {
        TA* x = qkv + (size_t)t * ld + (size_t)hh * D;
        if (hh >= Hq + Hkv) {                       // v head: copy
            if (slot_base < 0) continue;
            TA* dst = vpool + slot_base + (long long)(hh - Hq - Hkv) * page_size * D;
            for (int i = lane; i < D; i += 32) dst[i] = x[i];
            continue;
        }
        const bool is_k = hh >= Hq;
        const void* w = is_k ? kw : qw;
        float rstd = 1.f;
        if (w) {
            float ss = 0.f;
            for (int i = lane; i < D; i += 32) { const float v = to_f32(x[i]); ss += v * v; }
            ss = warp_sum(ss);
            rstd = 1.0f / sqrtf(ss / (float)D + eps);
        }
        TA* dst = x;
        if (is_k && write_kv) {
            if (slot_base < 0) continue;
            dst = kpool + slot_base + (long long)(hh - Hq) * page_size * D;
        }
        for (int i = lane; i < half; i += 32) {
            float x1 = to_f32(x[i]) * rstd, x2 = to_f32(x[i + half]) * rstd;
            if (w) {
                x1 *= offset + load_as_f32(w, w_dtype, i);
                x2 *= offset + load_as_f32(w, w_dtype, i + half);
            }
            const float c = cs[i], s = sn[i];
            dst[i] = from_f32<TA>(x1 * c - x2 * s);
            dst[i + half] = from_f32<TA>(x2 * c + x1 * s);
        }
        for (int i = rot_dim + lane; i < D; i += 32) {       // dims beyond the rotary width pass through
            float v = to_f32(x[i]) * rstd;
            if (w) v *= offset + load_as_f32(w, w_dtype, i);
            dst[i] = from_f32<TA>(v);
        }
    }
}

RB_EXPORT int rb_qk_norm_rope_write(
        void* qkv, int ld, const void* qw, const void* kw, int w_dtype, float eps, float offset,
        const float* cos_t, const float* sin_t, int rot_dim,
        const int* pos, const int* tok_seg, const int* block_table, int bt_stride, int page_size,
        void* kpool, void* vpool, int act_dtype, int T, int Hq, int Hkv, int D, int write_kv,
        cudaStream_t st) {
    if (T <= 0) return 0;
    if (rot_dim > D || (rot_dim & 1)) return (int)cudaErrorInvalidValue;
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
