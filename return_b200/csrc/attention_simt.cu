// Paged causal attention on the CUDA cores, for any element type, head size, page size and
// segment shape: the kernel of the 32-bit path, and the plain twin of the tensor-core kernels.
//
// One warp owns one (token, query head).  Keys are taken in tiles of 32 that are aligned to
// absolute positions (0-31, 32-63, ...), lane j of a tile scores key j, and the online softmax
// (running maximum m, running sum l, float32 accumulators) advances tile by tile as in the
// reference's kernels (rollout/attention.py:125-139).  Because the tiles are fixed by position
// and a row never looks at another row, the result for a token does not depend on how the
// prompt was cut into steps or on what else is in the batch: it is bit-identical.
//
// q: rotated queries inside the QKV buffer, row stride ld.  K and V: one layer's pools
// [num_pages, Hkv, P, D].  A key at position j is visible to the query at position p iff
// lo <= j <= p with lo = max(0, p - window + 1) when window > 0, else 0.
#include "common.cuh"

#define SIMT_MAX_D 256

template <typename TA>
__global__ void __launch_bounds__(128)
attention_simt_kernel(const TA* __restrict__ q, int ld, const TA* __restrict__ kpool,
                      const TA* __restrict__ vpool, const int* __restrict__ pos,
                      const int* __restrict__ tok_seg, const int* __restrict__ block_table,
                      int bt_stride, int page_size, TA* __restrict__ out, int Hq, int Hkv, int D,
                      float scale, int window) {
    extern __shared__ float qs_all[];                    // 4 warps x D floats
    const int t = blockIdx.x;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int h = blockIdx.y * 4 + warp;
    if (h >= Hq) return;                                  // no block-wide barrier below
    const int G = Hq / Hkv, kvh = h / G;
    const int p = pos[t];
    const int* bt = block_table + (size_t)tok_seg[t] * bt_stride;
    const int lo = window > 0 ? max(0, p - window + 1) : 0;
    float* qs = qs_all + warp * D;
    const TA* qrow = q + (size_t)t * ld + (size_t)h * D;
    for (int d = lane; d < D; d += 32) qs[d] = to_f32(qrow[d]);
    __syncwarp();

    float m = -INFINITY, l = 0.f;
    float acc[SIMT_MAX_D / 32];
#pragma unroll
    for (int i = 0; i < SIMT_MAX_D / 32; ++i) acc[i] = 0.f;
    const size_t head_stride = (size_t)page_size * D;    // one kv head of one page

    for (int j0 = (lo / 32) * 32; j0 <= p; j0 += 32) {
        const int j = j0 + lane;
        const bool valid = j >= lo && j <= p;
        float s = -INFINITY;
        if (valid) {
            const int page = bt[j / page_size];
            if (page < 0) {
                s = __int_as_float(0x7fc00000);       // a page that was given back: show it as NaN
            } else {
                const TA* kr = kpool + ((size_t)page * Hkv + kvh) * head_stride + (size_t)(j % page_size) * D;
                float dot = 0.f;
                for (int d = 0; d < D; ++d) dot = fmaf(qs[d], to_f32(kr[d]), dot);
                s = dot * scale;
            }
        }
        const float m_new = fmaxf(m, warp_max(s));
        const float pj = valid ? expf(s - m_new) : 0.f;
        const float alpha = expf(m - m_new);              // m = -inf on the first tile gives 0
        l = l * alpha + warp_sum(pj);
#pragma unroll
        for (int i = 0; i < SIMT_MAX_D / 32; ++i) acc[i] *= alpha;
        const int jend = min(32, p - j0 + 1);
        for (int jj = max(0, lo - j0); jj < jend; ++jj) {
            const float pjj = __shfl_sync(0xffffffffu, pj, jj);
            const int jk = j0 + jj;
            const int page = bt[jk / page_size];
            if (page < 0) continue;
            const TA* vr = vpool + ((size_t)page * Hkv + kvh) * head_stride + (size_t)(jk % page_size) * D;
#pragma unroll
            for (int i = 0; i < SIMT_MAX_D / 32; ++i) {
                const int d = lane + 32 * i;
                if (d < D) acc[i] = fmaf(pjj, to_f32(vr[d]), acc[i]);
            }
        }
        m = m_new;
    }
    TA* orow = out + ((size_t)t * Hq + h) * D;
    const float inv = 1.0f / l;
#pragma unroll
    for (int i = 0; i < SIMT_MAX_D / 32; ++i) {
        const int d = lane + 32 * i;
        if (d < D) orow[d] = from_f32<TA>(acc[i] * inv);
    }
}

RB_EXPORT int rb_attention_simt(const void* q, int ld, const void* kpool, const void* vpool,
                                const int* pos, const int* tok_seg, const int* block_table,
                                int bt_stride, int page_size, void* out, int act_dtype, int T,
                                int Hq, int Hkv, int D, float scale, int window, cudaStream_t st) {
    if (T <= 0) return 0;
    if (D > SIMT_MAX_D || D <= 0 || Hkv <= 0 || Hq % Hkv) return (int)cudaErrorInvalidValue;
    dim3 grid(T, (Hq + 3) / 4);
    const size_t smem = (size_t)4 * D * sizeof(float);
    if (act_dtype == RB_F32)
        attention_simt_kernel<float><<<grid, 128, smem, st>>>(
            (const float*)q, ld, (const float*)kpool, (const float*)vpool, pos, tok_seg, block_table,
            bt_stride, page_size, (float*)out, Hq, Hkv, D, scale, window);
    else
        attention_simt_kernel<bf16><<<grid, 128, smem, st>>>(
            (const bf16*)q, ld, (const bf16*)kpool, (const bf16*)vpool, pos, tok_seg, block_table,
            bt_stride, page_size, (bf16*)out, Hq, Hkv, D, scale, window);
    return rb_launch_status();
}
