// Sampling from float32 logits: greedy, temperature, top-k and top-p, with the log-probability
// of the chosen token.  Rows carry their own parameters.  Two kernels with the same meanings: one CTA a row
// (sample_kernel, any row length: the twin that tests compare with, and the fallback for very long rows) and a
// cluster of eight CTAs a row (sample_cluster_kernel, further down: what the engine runs).
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

// ---------------------------------------------------------------- a row by a cluster of eight CTAs
// The kernel above reads a row (600 KB at a vocabulary of 151,936) some seventy times with one CTA: 60 us a greedy
// row, 2.5 ms with top-k and top-p.  Here a cluster of eight CTAs takes a row: each CTA reads an eighth of it once
// into its shared memory, and every later pass runs there.  What the CTAs have to tell one another (maxima, sums,
// histograms) each writes into all eight shared memories (st.shared::cluster) and a cluster barrier follows; the
// values are then added in the order of the CTAs.
// The cut-off values are found digit by digit, sixteen bins a pass (eight passes of four bits instead of thirty-two
// of one), counts as integers and masses as fixed point (exp(x - max) * 2^32, added in 64 bits), so every sum is
// exact and the result does not depend on the order of the additions.  Same meanings as above; the chosen token is the first,
// in vocabulary order, at which the running mass of the kept tokens reaches u * (kept mass).
constexpr int SC_CTAS = 8;
constexpr int SC_THREADS = 512;                        // two CTAs share an SM
constexpr int SC_WARPS = SC_THREADS / 32;
constexpr float SC_MASS_ONE = 4294967296.0f;              // 2^32
typedef unsigned long long u64;

__device__ __forceinline__ unsigned sc_rank() {
    unsigned r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
__device__ __forceinline__ void sc_sync() {
    asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ void sc_store(const void* local, unsigned rank, u64 v) {      // the same variable in CTA `rank`
    unsigned a = (unsigned)__cvta_generic_to_shared(local), r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(a), "r"(rank));
    asm volatile("st.shared::cluster.u64 [%0], %1;" ::"r"(r), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned sc_mass(float xs, float mxs) {
    return __float2uint_rz(fminf(expf(xs - mxs) * SC_MASS_ONE, 4294967040.0f));
}
// v[d] += m with v in registers: one case runs (the lanes of a warp mostly agree on the digit), not sixteen compares
__device__ __forceinline__ void sc_bin_add(u64 (&v)[16], unsigned d, u64 m) {
    switch (d) {
        case 0: v[0] += m; break;   case 1: v[1] += m; break;   case 2: v[2] += m; break;   case 3: v[3] += m; break;
        case 4: v[4] += m; break;   case 5: v[5] += m; break;   case 6: v[6] += m; break;   case 7: v[7] += m; break;
        case 8: v[8] += m; break;   case 9: v[9] += m; break;   case 10: v[10] += m; break; case 11: v[11] += m; break;
        case 12: v[12] += m; break; case 13: v[13] += m; break; case 14: v[14] += m; break; default: v[15] += m; break;
    }
}

struct ScShared {
    u64 cta_tot[2][16];                // this CTA's sums of a step (two steps in flight; zero before a step adds to them)
    u64 gath[2][SC_CTAS][16];          // what every CTA of the cluster said in this step
    u64 warp_incl[SC_WARPS];
    unsigned digit, pad;
    u64 above;
    int choice;
};

// Every thread brings 16 numbers; afterwards sh.gath[step & 1][r][b] holds CTA r's sums, for every r, in every CTA.
// Most bins are empty in most warps (the values of a row share their leading digits, and late passes match few
// values), so a warp adds up only the bins in which one of its lanes has something, and its first lane adds the
// sum to the CTA's with an atomic in shared memory; integer sums, so the order does not matter.
__device__ __forceinline__ void sc_all_gather16(u64 (&v)[16], ScShared& sh, int step, unsigned rank, int n_used) {
    const int tid = threadIdx.x, lane = tid & 31, par = step & 1;
    if (tid < 16) sh.cta_tot[par ^ 1][tid] = 0;            // for the step after this one: nobody reads or adds to it now
#pragma unroll
    for (int b = 0; b < 16; ++b) {
        if (b < n_used && __any_sync(0xffffffffu, v[b] != 0)) {
            u64 t = v[b];
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) t += __shfl_xor_sync(0xffffffffu, t, o);
            if (lane == 0) atomicAdd(&sh.cta_tot[par][b], t);
        }
    }
    __syncthreads();
    if (tid < n_used * SC_CTAS) {
        const int r = tid / n_used, b = tid - r * n_used;
        sc_store(&sh.gath[par][rank][b], (unsigned)r, sh.cta_tot[par][b]);
    }
    sc_sync();
}

// After a gather of 16 bins, in warp 0: lane l holds the row's sum of bin 15 - l (the bins from the top down), `incl`
// the sum of the bins from the top down to its own.
__device__ __forceinline__ void sc_bins_from_the_top(const ScShared& sh, int step, u64& own, u64& incl) {
    const int lane = threadIdx.x & 31;
    own = 0;
    if (lane < 16)
        for (int r = 0; r < SC_CTAS; ++r) own += sh.gath[step & 1][r][15 - lane];
    incl = own;
#pragma unroll
    for (int o = 1; o < 16; o <<= 1) {
        const u64 t = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += t;
    }
}

__global__ void __launch_bounds__(SC_THREADS)
sample_cluster_kernel(const float* __restrict__ logits, int ld, int V, int per,
                      const float* __restrict__ temperature, const int* __restrict__ top_k,
                      const float* __restrict__ top_p, const float* __restrict__ uniform,
                      int* __restrict__ token_out, float* __restrict__ logprob_out) {
    extern __shared__ float sx[];                         // this CTA's part of the row
    __shared__ ScShared sh;
    __shared__ float fscratch[33];
    __shared__ int iscratch[33];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const unsigned rank = sc_rank();
    const int row = blockIdx.x / SC_CTAS;
    const float* x = logits + (size_t)row * ld;
    const int i0 = min(V, (int)rank * per), n = min(V, i0 + per) - i0;
    const float temp = temperature ? temperature[row] : 0.f;
    int step = 0;
    u64 v16[16];
    if (tid < 32) sh.cta_tot[tid >> 4][tid & 15] = 0;
    sc_sync();                                             // no CTA writes into another's shared memory before all have started

    // ---- the part of the row, its maximum and the lowest index that holds it
    float best = -INFINITY;
    int best_i = 0x7fffffff;
    for (int j = tid; j < n; j += SC_THREADS) {
        const float v = x[i0 + j];
        sx[j] = v;
        if (v > best) { best = v; best_i = i0 + j; }
    }
    const float mx_cta = block_max(best, fscratch);
    int cand = (best == mx_cta) ? best_i : 0x7fffffff;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) cand = min(cand, __shfl_xor_sync(0xffffffffu, cand, o));
    __syncthreads();
    if (lane == 0) iscratch[warp] = cand;
    __syncthreads();
    if (tid < 32) {
        int c = tid < SC_WARPS ? iscratch[tid] : 0x7fffffff;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) c = min(c, __shfl_xor_sync(0xffffffffu, c, o));
        if (tid == 0) iscratch[32] = c;
    }
    __syncthreads();
    if (tid < SC_CTAS) sc_store(&sh.gath[step & 1][rank][0], (unsigned)tid, ((u64)__float_as_uint(mx_cta) << 32) | (unsigned)iscratch[32]);
    sc_sync();
    float mx = -INFINITY;
    int argmax = 0x7fffffff;
    for (int r = 0; r < SC_CTAS; ++r) {
        const u64 g = sh.gath[step & 1][r][0];
        const float m = __uint_as_float((unsigned)(g >> 32));
        const int a = (int)(unsigned)g;
        if (m > mx || (m == mx && a < argmax)) { mx = m; argmax = a; }
    }
    if (argmax == 0x7fffffff) argmax = 0;                  // all -inf or NaN: token 0
    ++step;
    const bool greedy = !(temp > 0.f);
    if (greedy && logprob_out == nullptr) {
        if (rank == 0 && tid == 0) token_out[row] = argmax;
        return;
    }

    // ---- sum of exp over the raw logits, for the log-probability
    float se = 0.f;
    for (int j = tid; j < n; j += SC_THREADS) se += expf(sx[j] - mx);
    se = block_sum(se, fscratch);
    if (tid < SC_CTAS) sc_store(&sh.gath[step & 1][rank][0], (unsigned)tid, (u64)__float_as_uint(se));
    sc_sync();
    float se_all = 0.f;
    for (int r = 0; r < SC_CTAS; ++r) se_all += __uint_as_float((unsigned)sh.gath[step & 1][r][0]);
    const float lse = mx + logf(se_all);
    ++step;
    if (greedy) {
        if (rank == 0 && tid == 0) {
            token_out[row] = argmax;
            logprob_out[row] = x[argmax] - lse;
        }
        return;
    }

    const float mxs = mx / temp;
    for (int j = tid; j < n; j += SC_THREADS) sx[j] = sx[j] / temp;
    __syncthreads();
    auto mass_at = [&](int j) -> u64 { return (u64)sc_mass(sx[j], mxs); };
    const int k = top_k[row];
    const float p_keep = top_p[row];
    unsigned cut = 0u;                                     // tokens with key >= cut stay

    if (k > 0 && k < V) {
        // the k-th largest key, four bits a pass: among the keys that share the digits found so far, the bin in
        // which the count from the top reaches k
        unsigned prefix = 0u;
        u64 above = 0;                                     // keys above every key that shares the prefix
        for (int shift = 28; shift >= 0; shift -= 4) {
            const unsigned hi_mask = shift == 28 ? 0u : (0xffffffffu << (shift + 4));
#pragma unroll
            for (int b = 0; b < 16; ++b) v16[b] = 0;
            for (int j = tid; j < n; j += SC_THREADS) {
                const unsigned key = ordered_key(sx[j]);
                if ((key & hi_mask) == prefix) sc_bin_add(v16, (key >> shift) & 15u, 1ull);
            }
            sc_all_gather16(v16, sh, step, rank, 16);
            if (warp == 0) {
                // from the top: the first bin at which the count reaches k (the lowest bin if none does)
                u64 own, incl;
                sc_bins_from_the_top(sh, step, own, incl);
                const unsigned reached = __ballot_sync(0xffffffffu, lane < 16 && above + incl >= (u64)k) & 0xffffu;
                const int l = reached ? __ffs(reached) - 1 : 15;
                const u64 before = __shfl_sync(0xffffffffu, incl - own, l);
                if (lane == 0) { sh.digit = (unsigned)(15 - l); sh.above = above + before; }
            }
            __syncthreads();                               // (the next write to these comes after the next gather's barrier)
            prefix |= sh.digit << shift;
            above = sh.above;
            ++step;
        }
        cut = prefix;
    }
    if (p_keep < 1.f) {
        // kept mass so far, then the smallest c with mass{key > c, key >= cut} <= top_p * (that mass), four bits a pass
#pragma unroll
        for (int b = 0; b < 16; ++b) v16[b] = 0;
        for (int j = tid; j < n; j += SC_THREADS)
            if (ordered_key(sx[j]) >= cut) v16[0] += mass_at(j);
        sc_all_gather16(v16, sh, step, rank, 1);
        u64 z = 0;
        for (int r = 0; r < SC_CTAS; ++r) z += sh.gath[step & 1][r][0];
        ++step;
        const u64 budget = (u64)((double)p_keep * (double)z);
        unsigned prefix = 0u;
        u64 above = 0;                                     // mass above every key that shares the prefix: never more than the budget
        for (int shift = 28; shift >= 0; shift -= 4) {
            const unsigned hi_mask = shift == 28 ? 0u : (0xffffffffu << (shift + 4));
#pragma unroll
            for (int b = 0; b < 16; ++b) v16[b] = 0;
            for (int j = tid; j < n; j += SC_THREADS) {
                const unsigned key = ordered_key(sx[j]);
                if (key >= cut && (key & hi_mask) == prefix) sc_bin_add(v16, (key >> shift) & 15u, mass_at(j));
            }
            sc_all_gather16(v16, sh, step, rank, 16);
            if (warp == 0) {
                // the lowest bin for which the mass above it stays within the budget (for the top bin it does)
                u64 own, incl;
                sc_bins_from_the_top(sh, step, own, incl);
                const unsigned within = __ballot_sync(0xffffffffu, lane < 16 && above + (incl - own) <= budget) & 0xffffu;
                const int l = within ? 31 - __clz(within) : 0;
                const u64 before = __shfl_sync(0xffffffffu, incl - own, l);
                if (lane == 0) { sh.digit = (unsigned)(15 - l); sh.above = above + before; }
            }
            __syncthreads();
            prefix |= sh.digit << shift;
            above = sh.above;
            ++step;
        }
        cut = max(cut, prefix);
    }

    // ---- inverse CDF over the kept tokens in vocabulary order; a thread owns a run of its CTA's part
    const int chunk = (n + SC_THREADS - 1) / SC_THREADS;
    const int j0 = min(n, tid * chunk), j1 = min(n, j0 + chunk);
    u64 own = 0;
    int last_kept = -1;
    for (int j = j0; j < j1; ++j)
        if (ordered_key(sx[j]) >= cut) { own += mass_at(j); last_kept = j; }
    u64 incl = own;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const u64 t = __shfl_up_sync(0xffffffffu, incl, o);
        if (lane >= o) incl += t;
    }
    if (lane == 31) sh.warp_incl[warp] = incl;
    if (tid == 0) sh.choice = 0x7fffffff;
    __syncthreads();
    u64 before = 0, cta_total = 0;
    for (int w = 0; w < SC_WARPS; ++w) {
        if (w < warp) before += sh.warp_incl[w];
        cta_total += sh.warp_incl[w];
    }
    incl += before;
    if (tid < SC_CTAS) sc_store(&sh.gath[step & 1][rank][0], (unsigned)tid, cta_total);
    sc_sync();
    u64 total = 0, base = 0;
    for (int r = 0; r < SC_CTAS; ++r) {
        const u64 t = sh.gath[step & 1][r][0];
        if (r < (int)rank) base += t;
        total += t;
    }
    // u has 24 bits: u * total without leaving 64 bits; a target of zero would be met before the first token
    const u64 u24 = (u64)(fminf(fmaxf(uniform[row], 0.f), 0.99999994f) * 16777216.0f);
    u64 target = (total >> 24) * u24 + (((total & 0xffffffull) * u24) >> 24);
    if (target == 0) target = 1;
    // the CTA in whose part the running mass reaches the target does the rest
    if (!(base < target && base + cta_total >= target)) return;
    if (last_kept >= 0 && base + incl >= target) atomicMin(&sh.choice, tid);
    __syncthreads();
    if (tid == sh.choice) {
        u64 run = base + incl - own;
        int tok = last_kept;
        for (int j = j0; j < j1; ++j) {
            if (ordered_key(sx[j]) >= cut) {
                run += mass_at(j);
                if (run >= target) { tok = j; break; }
            }
        }
        token_out[row] = i0 + tok;
        if (logprob_out) logprob_out[row] = x[i0 + tok] - lse;
    }
}

// Rows of up to this many values go to the cluster kernel (an eighth of a row has to fit a CTA's shared memory).
constexpr int SC_MAX_PART_BYTES = 200 * 1024;

static int sample_cluster_part(int V) { return ((V + SC_CTAS - 1) / SC_CTAS + 3) & ~3; }     // values of a row a CTA holds
static bool sample_cluster_fits(int V) { return (size_t)sample_cluster_part(V) * sizeof(float) <= (size_t)SC_MAX_PART_BYTES; }

static int launch_sample_cluster(const float* logits, int ld, int n_rows, int V, const float* temperature,
                                 const int* top_k, const float* top_p, const float* uniform, int* token_out,
                                 float* logprob_out, cudaStream_t st) {
    const int per = sample_cluster_part(V);
    const size_t smem = (size_t)per * sizeof(float);
    static PerDevice configured;                           // the largest shared-memory size asked for so far, per device
    const int rc = configured.once([&](int) {
        return cudaFuncSetAttribute(sample_cluster_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    }, (long long)smem + 1);
    if (rc != 0) return rc;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(n_rows * SC_CTAS);
    cfg.blockDim = dim3(SC_THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = SC_CTAS;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    return (int)cudaLaunchKernelEx(&cfg, sample_cluster_kernel, logits, ld, V, per, temperature, top_k, top_p, uniform,
                                   token_out, logprob_out);
}

// one_cta != 0: the kernel with one CTA a row (any row length; the twin that the tests compare with).
RB_EXPORT int rb_sample(const float* logits, int ld, int n_rows, int V, const float* temperature,
                        const int* top_k, const float* top_p, const float* uniform, int* token_out,
                        float* logprob_out, int one_cta, cudaStream_t st) {
    if (n_rows <= 0) return 0;
    if (!one_cta && sample_cluster_fits(V))
        return launch_sample_cluster(logits, ld, n_rows, V, temperature, top_k, top_p, uniform, token_out, logprob_out, st);
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
    if (sample_cluster_fits(V))
        return launch_sample_cluster(logits, ld, n_rows, V, nullptr, nullptr, nullptr, nullptr, token_out, nullptr, st);
    argmax_kernel<<<n_rows, SAMPLE_THREADS, 0, st>>>(logits, ld, V, token_out);
    return rb_launch_status();
}
