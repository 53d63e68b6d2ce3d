// Sampling from float32 logits: greedy, temperature, top-k and top-p, with the log-probability
// of the chosen token.  One thread block per row; rows carry their own parameters.
//
// Meaning of the options follows the reference's sampler (rollout/model.py:15-67):
//   temperature <= 0        argmax of the raw logits;
//   otherwise               x = logits / temperature;
//   top_k > 0               only the k largest x stay;
//   top_p < 1               sorted by falling x, a token stays iff the mass of the tokens before it
//                           is <= top_p (the token that crosses top_p stays, the first always stays);
//   the log-probability     log_softmax(raw logits)[token], temperature not applied.
// Instead of sorting, the kernel finds the two cut-off values by bisection on the bit pattern of
// x (32 passes each, with deterministic block reductions).  Tokens that tie with the cut-off
// value all stay, where the reference keeps as many of them as its sort puts first.
// The random draw is one uniform number per row, made by the host from (seed, request, token
// index), so a request's samples do not depend on what else is in the batch.  The chosen token
// is the first one, in vocabulary order, at which the running mass of the kept tokens reaches
// u * (kept mass).
#include "common.cuh"

#define SAMPLE_THREADS 1024

__device__ __forceinline__ unsigned ordered_key(float f) {
    const unsigned u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);
}

__device__ __forceinline__ int block_sum_int(int v, int* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nwarps = blockDim.x >> 5;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        int t = lane < nwarps ? scratch[lane] : 0;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

__global__ void __launch_bounds__(SAMPLE_THREADS)
sample_kernel(const float* __restrict__ logits, int ld, int V,
              const float* __restrict__ temperature, const int* __restrict__ top_k,
              const float* __restrict__ top_p, const float* __restrict__ uniform,
              int* __restrict__ token_out, float* __restrict__ logprob_out) {
    __shared__ float fscratch[33];
    __shared__ int iscratch[33];
    __shared__ float warp_tot[32];
    __shared__ int s_choice;
    const int row = blockIdx.x, tid = threadIdx.x;
    const float* x = logits + (size_t)row * ld;
    const float temp = temperature[row];

    // ---- maximum of the raw logits and the lowest index that holds it
    float best = -INFINITY;
    int best_i = 0x7fffffff;
    for (int i = tid; i < V; i += blockDim.x) {
        const float v = x[i];
        if (v > best) { best = v; best_i = i; }
    }
    const float mx = block_max(best, fscratch);
    {
        int cand = (best == mx) ? best_i : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) cand = min(cand, __shfl_xor_sync(0xffffffffu, cand, o));
        __syncthreads();
        if ((tid & 31) == 0) iscratch[tid >> 5] = cand;
        __syncthreads();
        if (tid < 32) {
            int c = tid < (blockDim.x >> 5) ? iscratch[tid] : 0x7fffffff;
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) c = min(c, __shfl_xor_sync(0xffffffffu, c, o));
            if (tid == 0) iscratch[32] = c;
        }
        __syncthreads();
    }
    const int argmax = iscratch[32] == 0x7fffffff ? 0 : iscratch[32];   // all -inf or NaN: token 0
    __syncthreads();

    // ---- sum of exp over the raw logits, for the log-probability
    float se = 0.f;
    for (int i = tid; i < V; i += blockDim.x) se += expf(x[i] - mx);
    const float lse = mx + logf(block_sum(se, fscratch));

    if (!(temp > 0.f)) {
        if (tid == 0) {
            token_out[row] = argmax;
            if (logprob_out) logprob_out[row] = x[argmax] - lse;
        }
        return;
    }

    const float mxs = mx / temp;
    const int k = top_k[row];
    const float p_keep = top_p[row];
    unsigned cut = 0u;                       // tokens with key >= cut stay

    if (k > 0 && k < V) {
        // smallest c with count{key > c} <= k - 1
        unsigned c = 0u;
        for (int b = 31; b >= 0; --b) {
            const unsigned cand = c | ((1u << b) - 1u);
            int cnt = 0;
            for (int i = tid; i < V; i += blockDim.x) cnt += ordered_key(x[i] / temp) > cand;
            cnt = block_sum_int(cnt, iscratch);
            if (cnt > k - 1) c |= 1u << b;
        }
        cut = c;
    }
    if (p_keep < 1.f) {
        float z = 0.f;
        for (int i = tid; i < V; i += blockDim.x) {
            const float xs = x[i] / temp;
            if (ordered_key(xs) >= cut) z += expf(xs - mxs);
        }
        z = block_sum(z, fscratch);
        const float budget = p_keep * z;
        // smallest c with mass{key > c, key >= cut} <= budget
        unsigned c = 0u;
        for (int b = 31; b >= 0; --b) {
            const unsigned cand = c | ((1u << b) - 1u);
            float mass = 0.f;
            for (int i = tid; i < V; i += blockDim.x) {
                const float xs = x[i] / temp;
                const unsigned key = ordered_key(xs);
                if (key > cand && key >= cut) mass += expf(xs - mxs);
            }
            mass = block_sum(mass, fscratch);
            if (mass > budget) c |= 1u << b;
        }
        cut = max(cut, c);
    }

    // ---- inverse CDF over the kept tokens in vocabulary order; thread `tid` owns a contiguous chunk
    const int chunk = (V + blockDim.x - 1) / blockDim.x;
    const int i0 = min(V, tid * chunk), i1 = min(V, i0 + chunk);
    float own = 0.f;
    int last_kept = -1;
    for (int i = i0; i < i1; ++i) {
        const float xs = x[i] / temp;
        if (ordered_key(xs) >= cut) { own += expf(xs - mxs); last_kept = i; }
    }
    // inclusive scan of `own` over the block
    const int lane = tid & 31, warp = tid >> 5;
    float incl = own;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const float n = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += n;
    }
    if (lane == 31) warp_tot[warp] = incl;
    if (tid == 0) s_choice = 0x7fffffff;
    __syncthreads();
    float base = 0.f;
    for (int w = 0; w < warp; ++w) base += warp_tot[w];
    incl += base;
    float total = 0.f;
    for (int w = 0; w < (int)(blockDim.x >> 5); ++w) total += warp_tot[w];
    const float target = uniform[row] * total;
    // the first thread whose inclusive sum reaches the target and that keeps a token
    if (last_kept >= 0 && incl >= target) atomicMin(&s_choice, tid);
    __syncthreads();
    int chooser = s_choice;
    if (chooser == 0x7fffffff) {
        // rounding left the target above every partial sum: the last thread that keeps a token
        __syncthreads();
        if (tid == 0) s_choice = -1;
        __syncthreads();
        if (last_kept >= 0) atomicMax(&s_choice, tid);
        __syncthreads();
        chooser = s_choice;
        if (tid == chooser) {
            token_out[row] = last_kept;
            if (logprob_out) logprob_out[row] = x[last_kept] - lse;
        }
        return;
    }
    if (tid == chooser) {
        float run = incl - own;
        int tok = last_kept;
        for (int i = i0; i < i1; ++i) {
            const float xs = x[i] / temp;
            if (ordered_key(xs) >= cut) {
                run += expf(xs - mxs);
                if (run >= target) { tok = i; break; }
            }
        }
        token_out[row] = tok;
        if (logprob_out) logprob_out[row] = x[tok] - lse;
    }
}

RB_EXPORT int rb_sample(const float* logits, int ld, int n_rows, int V, const float* temperature,
                        const int* top_k, const float* top_p, const float* uniform, int* token_out,
                        float* logprob_out, cudaStream_t st) {
    if (n_rows <= 0) return 0;
    sample_kernel<<<n_rows, SAMPLE_THREADS, 0, st>>>(logits, ld, V, temperature, top_k, top_p, uniform,
                                                    token_out, logprob_out);
    return rb_launch_status();
}

// ---------------------------------------------------------------- greedy only
// argmax (lowest index on ties) of every row; the fast path when no row of a batch samples.
__global__ void __launch_bounds__(SAMPLE_THREADS)
argmax_kernel(const float* __restrict__ logits, int ld, int V, int* __restrict__ token_out) {
    __shared__ float fscratch[33];
    __shared__ int iscratch[33];
    const int row = blockIdx.x, tid = threadIdx.x;
    const float* x = logits + (size_t)row * ld;
    float best = -INFINITY;
    int best_i = 0x7fffffff;
    for (int i = tid; i < V; i += blockDim.x) {
        const float v = x[i];
        if (v > best) { best = v; best_i = i; }
    }
    const float mx = block_max(best, fscratch);
    int cand = (best == mx) ? best_i : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) cand = min(cand, __shfl_xor_sync(0xffffffffu, cand, o));
    __syncthreads();
    if ((tid & 31) == 0) iscratch[tid >> 5] = cand;
    __syncthreads();
    if (tid < 32) {
        int c = tid < (blockDim.x >> 5) ? iscratch[tid] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) c = min(c, __shfl_xor_sync(0xffffffffu, c, o));
        if (tid == 0) token_out[row] = c == 0x7fffffff ? 0 : c;
    }
}

RB_EXPORT int rb_argmax(const float* logits, int ld, int n_rows, int V, int* token_out, cudaStream_t st) {
    if (n_rows <= 0) return 0;
    argmax_kernel<<<n_rows, SAMPLE_THREADS, 0, st>>>(logits, ld, V, token_out);
    return rb_launch_status();
}
