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

// One warp per token and HPW neighbouring heads; a lane holds the element pairs (i, i+1) of the first
// rotary half and their partners (i + R/2, i + R/2 + 1) in registers, so a head is read once; head sizes
// up to 256.  The loads of all of a warp's heads go out before the first is used: a head is only 256
// to 512 bytes, and with one head a warp the kernel sat on memory latency at a quarter of the bandwidth.
constexpr int ROPE_MAX_J = 2;                     // pairs of pairs per lane: R/2 <= 128

template <typename TA, int HPW>
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
    const int hh0 = (blockIdx.y * (blockDim.x >> 5) + (threadIdx.x >> 5)) * HPW;      // this warp's first head
    const int n_heads = write_kv ? Hq + 2 * Hkv : Hq + Hkv;   // without a write, k is normed and rotated in place
    if (hh0 >= n_heads) return;
    const int p = pos[t];
    const int half = rot_dim >> 1;
    long long slot_base = -1;     // element offset of (page, kv head 0, row) in a pool
    if (write_kv && hh0 + HPW > Hq) {
        const int page = block_table[(size_t)tok_seg[t] * bt_stride + p / page_size];
        if (page >= 0) slot_base = ((long long)page * Hkv * page_size + (p % page_size)) * D;
    }
    TA* row = qkv + (size_t)t * ld;
    // ---- every load first
    float2 a[HPW][ROPE_MAX_J], b[HPW][ROPE_MAX_J];            // first-half pairs and their second-half partners
    float2 c[ROPE_MAX_J], sn[ROPE_MAX_J];
    const float* cs = cos_t + (size_t)p * half;
    const float* ss_t = sin_t + (size_t)p * half;
#pragma unroll
    for (int j = 0; j < ROPE_MAX_J; ++j) {
        const int i = 2 * lane + 64 * j;
        if (i < half) {
            c[j] = *reinterpret_cast<const float2*>(cs + i);
            sn[j] = *reinterpret_cast<const float2*>(ss_t + i);
        }
    }
#pragma unroll
    for (int u = 0; u < HPW; ++u) {
        const int hh = hh0 + u;
        if (hh >= n_heads) break;
        const TA* x = row + (size_t)hh * D;
        if (hh >= Hq + Hkv) {                       // v head: its two pairs ride in a[u][*]
#pragma unroll
            for (int j = 0; j < ROPE_MAX_J; ++j) {
                const int i = 2 * lane + 64 * j;
                if (i < D) a[u][j] = Pair<TA>::load(x + i);
                if (i + 128 < D) b[u][j] = Pair<TA>::load(x + i + 128);
            }
            continue;
        }
#pragma unroll
        for (int j = 0; j < ROPE_MAX_J; ++j) {
            const int i = 2 * lane + 64 * j;
            if (i < half) {
                a[u][j] = Pair<TA>::load(x + i);
                b[u][j] = Pair<TA>::load(x + i + half);
            }
        }
    }
    // ---- then head by head
#pragma unroll
    for (int u = 0; u < HPW; ++u) {
        const int hh = hh0 + u;
        if (hh >= n_heads) break;
        TA* x = row + (size_t)hh * D;
        if (hh >= Hq + Hkv) {                       // v head: copy
            if (slot_base < 0) continue;
            TA* dst = vpool + slot_base + (long long)(hh - Hq - Hkv) * page_size * D;
#pragma unroll
            for (int j = 0; j < ROPE_MAX_J; ++j) {
                const int i = 2 * lane + 64 * j;
                if (i < D) Pair<TA>::store(dst + i, a[u][j]);
                if (i + 128 < D) Pair<TA>::store(dst + i + 128, b[u][j]);
            }
            continue;
        }
        const bool is_k = hh >= Hq;
        const void* w = is_k ? kw : qw;
        TA* dst = x;
        if (is_k && write_kv) {
            if (slot_base < 0) continue;
            dst = kpool + slot_base + (long long)(hh - Hq) * page_size * D;
        }
        float ss = 0.f;
#pragma unroll
        for (int j = 0; j < ROPE_MAX_J; ++j) {
            const int i = 2 * lane + 64 * j;
            if (i < half) ss += a[u][j].x * a[u][j].x + a[u][j].y * a[u][j].y + b[u][j].x * b[u][j].x + b[u][j].y * b[u][j].y;
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
#pragma unroll
        for (int j = 0; j < ROPE_MAX_J; ++j) {
            const int i = 2 * lane + 64 * j;
            if (i < half) {
                float2 x1 = make_float2(a[u][j].x * rstd, a[u][j].y * rstd), x2 = make_float2(b[u][j].x * rstd, b[u][j].y * rstd);
                if (w) {
                    x1.x *= offset + load_as_f32(w, w_dtype, i);        x1.y *= offset + load_as_f32(w, w_dtype, i + 1);
                    x2.x *= offset + load_as_f32(w, w_dtype, i + half); x2.y *= offset + load_as_f32(w, w_dtype, i + half + 1);
                }
                Pair<TA>::store(dst + i, make_float2(x1.x * c[j].x - x2.x * sn[j].x, x1.y * c[j].y - x2.y * sn[j].y));
                Pair<TA>::store(dst + i + half, make_float2(x2.x * c[j].x + x1.x * sn[j].x, x2.y * c[j].y + x1.y * sn[j].y));
            }
        }
        for (int i = rot_dim + 2 * lane; i < D; i += 64) {
            float2 v = Pair<TA>::load(x + i);
            v.x *= rstd; v.y *= rstd;
            if (w) { v.x *= offset + load_as_f32(w, w_dtype, i); v.y *= offset + load_as_f32(w, w_dtype, i + 1); }
            Pair<TA>::store(dst + i, v);
        }
    }
}

// The same for many tokens of bfloat16 with head sizes 64, 128 or 256 rotated over their whole width, in
// 16-byte pieces: LPH = D / 16 lanes share a head, each holding 8 neighbouring elements of the first half and
// their partners in the second, so a warp works on 32 / LPH heads at once, twice over (ROUNDS), and a head is
// two 16-byte loads and two 16-byte stores a lane.  A warp takes one (token, group of heads) item.
constexpr int ROPE_VEC_ROUNDS = 2;

__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
    const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 p = __bfloat1622float2(h[i]);
        f[2 * i] = p.x;
        f[2 * i + 1] = p.y;
    }
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
    uint4 v;
    __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
    return v;
}

template <int LPH>
__global__ void __launch_bounds__(128)
qk_norm_rope_write_vec_kernel(
        bf16* __restrict__ qkv, int ld,
        const void* __restrict__ qw, const void* __restrict__ kw, int w_dtype, float eps, float offset,
        const float* __restrict__ cos_t, const float* __restrict__ sin_t,
        const int* __restrict__ pos, const int* __restrict__ tok_seg,
        const int* __restrict__ block_table, int bt_stride, int page_size,
        bf16* __restrict__ kpool, bf16* __restrict__ vpool,
        int T, int Hq, int Hkv, int write_kv, int groups_per_token) {
    constexpr int D = LPH * 16, HALF = D / 2, HEADS_AT_ONCE = 32 / LPH, HEADS_PER_WARP = HEADS_AT_ONCE * ROPE_VEC_ROUNDS;
    pdl_launch_dependents();
    pdl_wait();
    const int lane = threadIdx.x & 31;
    const long long item = (long long)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int t = (int)(item / groups_per_token), hg = (int)(item % groups_per_token);
    if (t >= T) return;
    const int sub = lane % LPH, hsel = lane / LPH;
    const int n_heads = write_kv ? Hq + 2 * Hkv : Hq + Hkv;
    const int p = pos[t];
    long long slot_base = -1;     // element offset of (page, kv head 0, row) in a pool
    if (write_kv && (hg + 1) * HEADS_PER_WARP > Hq) {
        const int page = block_table[(size_t)tok_seg[t] * bt_stride + p / page_size];
        if (page >= 0) slot_base = ((long long)page * Hkv * page_size + (p % page_size)) * D;
    }
    bf16* row = qkv + (size_t)t * ld;
    uint4 a[ROPE_VEC_ROUNDS], b[ROPE_VEC_ROUNDS];
#pragma unroll
    for (int r = 0; r < ROPE_VEC_ROUNDS; ++r) {
        const int hh = hg * HEADS_PER_WARP + r * HEADS_AT_ONCE + hsel;
        if (hh < n_heads) {
            const bf16* x = row + (size_t)hh * D + 8 * sub;
            a[r] = *reinterpret_cast<const uint4*>(x);
            b[r] = *reinterpret_cast<const uint4*>(x + HALF);
        }
    }
    float c[8], sn[8];
    {
        const float4* cp = reinterpret_cast<const float4*>(cos_t + (size_t)p * HALF + 8 * sub);
        const float4* sp = reinterpret_cast<const float4*>(sin_t + (size_t)p * HALF + 8 * sub);
        const float4 c0 = cp[0], c1 = cp[1], s0 = sp[0], s1 = sp[1];
        c[0] = c0.x; c[1] = c0.y; c[2] = c0.z; c[3] = c0.w; c[4] = c1.x; c[5] = c1.y; c[6] = c1.z; c[7] = c1.w;
        sn[0] = s0.x; sn[1] = s0.y; sn[2] = s0.z; sn[3] = s0.w; sn[4] = s1.x; sn[5] = s1.y; sn[6] = s1.z; sn[7] = s1.w;
    }
#pragma unroll
    for (int r = 0; r < ROPE_VEC_ROUNDS; ++r) {
        const int hh = hg * HEADS_PER_WARP + r * HEADS_AT_ONCE + hsel;
        const bool live = hh < n_heads;
        const bool is_v = hh >= Hq + Hkv, is_k = hh >= Hq && !is_v;
        float x1[8], x2[8];
        if (live) { unpack8(a[r], x1); unpack8(b[r], x2); }
        else {
#pragma unroll
            for (int i = 0; i < 8; ++i) x1[i] = x2[i] = 0.f;
        }
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < 8; ++i) ss += x1[i] * x1[i] + x2[i] * x2[i];
#pragma unroll
        for (int o = LPH / 2; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);     // over the lanes of this head
        if (!live) continue;
        if (is_v) {
            if (slot_base < 0) continue;
            bf16* dst = vpool + slot_base + (long long)(hh - Hq - Hkv) * page_size * D + 8 * sub;
            *reinterpret_cast<uint4*>(dst) = a[r];
            *reinterpret_cast<uint4*>(dst + HALF) = b[r];
            continue;
        }
        const void* w = is_k ? kw : qw;
        bf16* dst = row + (size_t)hh * D;
        if (is_k && write_kv) {
            if (slot_base < 0) continue;
            dst = kpool + slot_base + (long long)(hh - Hq) * page_size * D;
        }
        if (w) {
            const float rstd = 1.0f / sqrtf(ss / (float)D + eps);
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                x1[i] = x1[i] * rstd * (offset + load_as_f32(w, w_dtype, 8 * sub + i));        // (x * rstd) * w, as the other form
                x2[i] = x2[i] * rstd * (offset + load_as_f32(w, w_dtype, HALF + 8 * sub + i));
            }
        }
        float o1[8], o2[8];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            o1[i] = x1[i] * c[i] - x2[i] * sn[i];
            o2[i] = x2[i] * c[i] + x1[i] * sn[i];
        }
        *reinterpret_cast<uint4*>(dst + 8 * sub) = pack8(o1);
        *reinterpret_cast<uint4*>(dst + HALF + 8 * sub) = pack8(o2);
    }
}

template <int LPH>
static int launch_rope_vec(void* qkv, int ld, const void* qw, const void* kw, int w_dtype, float eps, float offset,
                           const float* cos_t, const float* sin_t, const int* pos, const int* tok_seg,
                           const int* block_table, int bt_stride, int page_size, void* kpool, void* vpool,
                           int T, int Hq, int Hkv, int write_kv, cudaStream_t st) {
    const int heads = write_kv ? Hq + 2 * Hkv : Hq + Hkv;
    const int per_warp = (32 / LPH) * ROPE_VEC_ROUNDS;
    const int groups = (heads + per_warp - 1) / per_warp;
    const long long items = (long long)T * groups;
    const dim3 grid((unsigned)((items + 3) / 4));
    return rb_launch_pdl(qk_norm_rope_write_vec_kernel<LPH>, grid, dim3(128), 0, st,
        (bf16*)qkv, ld, qw, kw, w_dtype, eps, offset, cos_t, sin_t, pos, tok_seg, block_table, bt_stride, page_size,
        (bf16*)kpool, (bf16*)vpool, T, Hq, Hkv, write_kv, groups);
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
    // many tokens: four heads a warp, so that enough bytes are in flight; few tokens: one head a warp, so that
    // the few warps there are spread over the SMs
    const bool aligned = ld % 8 == 0 && ((uintptr_t)qkv % 16) == 0 && ((uintptr_t)kpool % 16) == 0 && ((uintptr_t)vpool % 16) == 0;
    if ((long long)T * heads >= 8192 && act_dtype != RB_F32 && rot_dim == D && aligned && (D == 64 || D == 128 || D == 256)) {
        // many tokens of bfloat16 with a whole-head rotation: 16-byte pieces
        if (D == 64) return launch_rope_vec<4>(qkv, ld, qw, kw, w_dtype, eps, offset, cos_t, sin_t, pos, tok_seg, block_table,
                                               bt_stride, page_size, kpool, vpool, T, Hq, Hkv, write_kv, st);
        if (D == 128) return launch_rope_vec<8>(qkv, ld, qw, kw, w_dtype, eps, offset, cos_t, sin_t, pos, tok_seg, block_table,
                                                bt_stride, page_size, kpool, vpool, T, Hq, Hkv, write_kv, st);
        return launch_rope_vec<16>(qkv, ld, qw, kw, w_dtype, eps, offset, cos_t, sin_t, pos, tok_seg, block_table,
                                   bt_stride, page_size, kpool, vpool, T, Hq, Hkv, write_kv, st);
    }
    if ((long long)T * heads >= 8192) {
        constexpr int HPW = 4;
        const dim3 grid(T, (heads + 4 * HPW - 1) / (4 * HPW));
        if (act_dtype == RB_F32)
            return rb_launch_pdl(qk_norm_rope_write_kernel<float, HPW>, grid, dim3(threads), 0, st,
                (float*)qkv, ld, qw, kw, w_dtype, eps, offset, cos_t, sin_t, rot_dim, pos, tok_seg,
                block_table, bt_stride, page_size, (float*)kpool, (float*)vpool, Hq, Hkv, D, write_kv);
        return rb_launch_pdl(qk_norm_rope_write_kernel<bf16, HPW>, grid, dim3(threads), 0, st,
                (bf16*)qkv, ld, qw, kw, w_dtype, eps, offset, cos_t, sin_t, rot_dim, pos, tok_seg,
                block_table, bt_stride, page_size, (bf16*)kpool, (bf16*)vpool, Hq, Hkv, D, write_kv);
    }
    const dim3 grid(T, (heads + 3) / 4);
    if (act_dtype == RB_F32)
        return rb_launch_pdl(qk_norm_rope_write_kernel<float, 1>, grid, dim3(threads), 0, st,
            (float*)qkv, ld, qw, kw, w_dtype, eps, offset, cos_t, sin_t, rot_dim, pos, tok_seg,
            block_table, bt_stride, page_size, (float*)kpool, (float*)vpool, Hq, Hkv, D, write_kv);
    return rb_launch_pdl(qk_norm_rope_write_kernel<bf16, 1>, grid, dim3(threads), 0, st,
            (bf16*)qkv, ld, qw, kw, w_dtype, eps, offset, cos_t, sin_t, rot_dim, pos, tok_seg,
            block_table, bt_stride, page_size, (bf16*)kpool, (bf16*)vpool, Hq, Hkv, D, write_kv);
}
