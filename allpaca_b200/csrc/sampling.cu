// Next-token choice on the GPU: greedy arg-max, and temperature sampling with
// optional top-k and top-p, one thread block per row of logits.
//
// Meaning of the options follows the reference (crates/allpaca-core/src/sampling.rs):
// temperature <= 1e-5 picks the first maximum (:36-38, :215-225); otherwise logits are
// divided by the temperature (:227-234), non-finite ones are dropped (:236-244), the
// top_k largest are kept with ties going to the lower token id (:246-271, 0 = off), then
// the smallest prefix (by descending logit, ties by id) whose probability reaches top_p
// is kept when 0 <= top_p < 1 (:276-309), the survivors are soft-maxed (:311-331) and
// one is drawn by walking them with a uniform number (:55-67).  The walk here goes in
// token-id order; the uniform number comes from the host so that a draw does not depend
// on what else is in the batch.
//
// Selection of "the k largest" and "the prefix that reaches a probability" is done with
// a 4-pass radix search over the order-preserving integer image of the logits, counting
// either candidates or probability mass, so no sort of the vocabulary is needed.
#include "common.cuh"
#include <float.h>

#define SAMP_THREADS 1024

__device__ __forceinline__ unsigned ordered_key(float f) {
    unsigned u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);   // ascending floats -> ascending keys
}
__device__ __forceinline__ bool finite_f(float f) { return fabsf(f) <= FLT_MAX; }

// ---------------------------------------------------------------------------
// arg-max: first maximum wins; rows with no finite value give token 0.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(SAMP_THREADS)
argmax_kernel(const float* __restrict__ logits, long long row_stride, int V, int* __restrict__ out) {
    __shared__ float best_v[32];
    __shared__ int best_i[32];
    const float* row = logits + (size_t)blockIdx.x * row_stride;
    ap_pdl_trigger();
    ap_pdl_wait();
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < V; i += SAMP_THREADS) {
        const float v = row[i];
        if (v > bv) { bv = v; bi = i; }          // ascending i per thread: first maximum kept
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
    }
    if ((threadIdx.x & 31) == 0) { best_v[threadIdx.x >> 5] = bv; best_i[threadIdx.x >> 5] = bi; }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < SAMP_THREADS / 32; ++w)
            if (best_v[w] > bv || (best_v[w] == bv && best_i[w] < bi)) { bv = best_v[w]; bi = best_i[w]; }
        out[blockIdx.x] = (bi == 0x7fffffff) ? 0 : bi;
    }
}

AP_EXPORT int ap_argmax(const float* logits, long long row_stride, int R, int V, int* out,
                        cudaStream_t stream) {
    AP_REQUIRE(R >= 0 && V > 0 && row_stride >= V, "argmax: bad sizes R=%d V=%d", R, V);
    if (R == 0) return AP_OK;
    AP_CHECK_PDL_LAUNCH("argmax", ap_launch_pdl(argmax_kernel, dim3(R), dim3(SAMP_THREADS), 0, stream, logits,
                                                row_stride, V, out));
    return AP_OK;
}

// ---------------------------------------------------------------------------
// temperature / top-k / top-p sampling
// ---------------------------------------------------------------------------
struct Cut {            // keep key > key, or key == key with id <= tie_id
    unsigned key;
    int tie_id;
    int active;         // 0: keeps everything
};

__device__ __forceinline__ bool passes(const Cut& c, unsigned key, int id) {
    return !c.active || key > c.key || (key == c.key && id <= c.tie_id);
}

struct SampShared {
    float hist[256];
    float warp_tot[32];
    float f0, f1;
    int i0, i1;
    unsigned u0;
};

// inclusive block scan of v; returns the inclusive prefix, total through *total
__device__ __forceinline__ float block_scan(float v, SampShared& sh, float* total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float x = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const float y = __shfl_up_sync(0xffffffffu, x, o);
        if (lane >= o) x += y;
    }
    __syncthreads();
    if (lane == 31) sh.warp_tot[warp] = x;
    __syncthreads();
    float before = 0.f, tot = 0.f;
    for (int w = 0; w < SAMP_THREADS / 32; ++w) {
        const float wt = sh.warp_tot[w];
        if (w < warp) before += wt;
        tot += wt;
    }
    *total = tot;
    return x + before;
}

// Radix search.  Among candidates (finite, passing c0 and c1), ordered by descending key,
// find the key at which the running weight first reaches `target`.  weighted == false
// counts candidates; true sums exp(l/T - m).  Returns through shared memory:
//   sel_key, weight of strictly greater keys (gt), and found (0 if the total stays below
//   the target, possible only through rounding of a weighted sum).
__device__ void radix_search(const float* row, int V, float tdiv, float m, const Cut& c0, const Cut& c1,
                             bool weighted, float target, SampShared& sh, unsigned* sel_key, float* gt,
                             int* found) {
    unsigned prefix = 0, mask = 0;
    float greater = 0.f;
    int ok = 1;
    for (int pass = 0; pass < 4 && ok; ++pass) {
        const int shift = 24 - 8 * pass;
        __syncthreads();
        for (int b = threadIdx.x; b < 256; b += SAMP_THREADS) sh.hist[b] = 0.f;
        __syncthreads();
        for (int i = threadIdx.x; i < V; i += SAMP_THREADS) {
            const float l = row[i] / tdiv;
            if (!finite_f(row[i])) continue;
            const unsigned key = ordered_key(l);
            if ((key & mask) != prefix || !passes(c0, key, i) || !passes(c1, key, i)) continue;
            atomicAdd(&sh.hist[(key >> shift) & 255u], weighted ? expf(l - m) : 1.0f);
        }
        __syncthreads();
        if (threadIdx.x == 0) {
            float cum = greater;
            int sel = -1;
            for (int b = 255; b >= 0; --b) {
                const float hb = sh.hist[b];
                if (hb > 0.f && cum + hb >= target) { sel = b; break; }
                cum += hb;
            }
            sh.i0 = sel;
            sh.f0 = cum;
        }
        __syncthreads();
        if (sh.i0 < 0) { ok = 0; break; }
        greater = sh.f0;
        prefix |= ((unsigned)sh.i0) << shift;
        mask |= 0xffu << shift;
    }
    *sel_key = prefix;
    *gt = greater;
    *found = ok;
}

// id of the n-th (1-based) candidate whose key equals `key`, in ascending id order;
// the last such id if there are fewer.
__device__ int nth_equal(const float* row, int V, float tdiv, const Cut& c0, const Cut& c1, unsigned key,
                         int n, SampShared& sh) {
    float running = 0.f;
    __syncthreads();
    if (threadIdx.x == 0) { sh.i1 = -1; }
    int last = -1;
    for (int base = 0; base < V; base += SAMP_THREADS) {
        const int i = base + threadIdx.x;
        bool eq = false;
        if (i < V && finite_f(row[i])) {
            const unsigned k = ordered_key(row[i] / tdiv);
            eq = (k == key) && passes(c0, k, i) && passes(c1, k, i);
        }
        float tot;
        const float inc = block_scan(eq ? 1.f : 0.f, sh, &tot);
        if (eq && running + inc == (float)n) sh.i1 = i;
        if (eq) last = i;
        __syncthreads();
        if (sh.i1 >= 0) break;
        running += tot;
    }
    const int hit = sh.i1;
    if (hit >= 0) return hit;
    // fewer than n equal candidates: take the highest id among them
    __syncthreads();
    if (threadIdx.x == 0) sh.i1 = -1;
    __syncthreads();
    if (last >= 0) atomicMax(&sh.i1, last);
    __syncthreads();
    return sh.i1;
}

__global__ void __launch_bounds__(SAMP_THREADS)
sample_kernel(const float* __restrict__ logits, long long row_stride, int V,
              const float* __restrict__ temperature, const int* __restrict__ top_k,
              const float* __restrict__ top_p, const float* __restrict__ uniform, int* __restrict__ out) {
    __shared__ SampShared sh;
    __shared__ float red[32];
    const int r = blockIdx.x;
    const float* row = logits + (size_t)r * row_stride;
    const float temp = temperature[r];

    // maximum (first index) over finite logits; also the greedy answer
    float bv = -INFINITY;
    int bi = 0x7fffffff;
    int n_finite = 0;
    for (int i = threadIdx.x; i < V; i += SAMP_THREADS) {
        const float v = row[i];
        if (!finite_f(v)) continue;
        ++n_finite;
        if (v > bv) { bv = v; bi = i; }
    }
    const float vmax = ap_block_max(bv, red);
    const float cnt = ap_block_sum((float)n_finite, red);
    __syncthreads();
    if (threadIdx.x == 0) sh.i0 = 0x7fffffff;
    __syncthreads();
    if (bv == vmax && bi != 0x7fffffff) atomicMin(&sh.i0, bi);
    __syncthreads();
    const int arg = sh.i0 == 0x7fffffff ? 0 : sh.i0;
    __syncthreads();
    if (cnt == 0.f || temp <= 1e-5f) {           // nothing finite -> token 0; greedy -> first maximum
        if (threadIdx.x == 0) out[r] = arg;
        return;
    }
    const float tdiv = fmaxf(temp, 1e-5f);
    const float m = vmax / tdiv;
    const int n_cand = (int)cnt;

    Cut ck = {0u, 0, 0}, cp = {0u, 0, 0};
    const int k = top_k[r];
    int kept = n_cand;
    if (k > 0 && k < n_cand) {
        unsigned key; float gt; int found;
        radix_search(row, V, tdiv, m, ck, cp, false, (float)k, sh, &key, &gt, &found);
        const int need = k - (int)gt;            // how many of the equal keys are kept
        const int tie = nth_equal(row, V, tdiv, ck, cp, key, need, sh);
        ck.key = key; ck.tie_id = tie; ck.active = 1;
        kept = k;
    }
    const float pth = top_p[r];
    if (pth >= 0.f && pth < 1.f && kept > 1) {
        float z = 0.f;
        for (int i = threadIdx.x; i < V; i += SAMP_THREADS) {
            if (!finite_f(row[i])) continue;
            const float l = row[i] / tdiv;
            if (passes(ck, ordered_key(l), i)) z += expf(l - m);
        }
        z = ap_block_sum(z, red);
        unsigned key; float gt; int found;
        radix_search(row, V, tdiv, m, ck, cp, true, pth * z, sh, &key, &gt, &found);
        if (found) {
            // weight of one candidate with this key, recovered from the key itself
            const unsigned u = (key & 0x80000000u) ? (key & 0x7fffffffu) : ~key;
            const float e = expf(__uint_as_float(u) - m);
            int need = 1;
            if (e > 0.f) {
                const float lack = pth * z - gt;
                need = (int)ceilf(lack / e);
                if (need < 1) need = 1;
            }
            const int tie = nth_equal(row, V, tdiv, ck, cp, key, need, sh);
            cp.key = key; cp.tie_id = tie; cp.active = 1;
        }
    }

    // soft-max of the survivors and the walk in id order
    float z = 0.f;
    for (int i = threadIdx.x; i < V; i += SAMP_THREADS) {
        if (!finite_f(row[i])) continue;
        const float l = row[i] / tdiv;
        const unsigned key = ordered_key(l);
        if (passes(ck, key, i) && passes(cp, key, i)) z += expf(l - m);
    }
    z = ap_block_sum(z, red);
    const float target = uniform[r] * z;
    float running = 0.f;
    __syncthreads();
    if (threadIdx.x == 0) { sh.i0 = 0x7fffffff; sh.i1 = -1; }
    __syncthreads();
    int last = -1;
    for (int base = 0; base < V; base += SAMP_THREADS) {
        const int i = base + threadIdx.x;
        float w = 0.f;
        bool c = false;
        if (i < V && finite_f(row[i])) {
            const float l = row[i] / tdiv;
            const unsigned key = ordered_key(l);
            if (passes(ck, key, i) && passes(cp, key, i)) { w = expf(l - m); c = true; }
        }
        float tot;
        const float inc = block_scan(w, sh, &tot);
        if (c) last = i;
        if (c && running + inc >= target) atomicMin(&sh.i0, i);
        __syncthreads();
        if (sh.i0 != 0x7fffffff) break;
        running += tot;
    }
    if (sh.i0 == 0x7fffffff) {       // rounding left the walk short: the last survivor
        if (last >= 0) atomicMax(&sh.i1, last);
        __syncthreads();
        if (threadIdx.x == 0) out[r] = sh.i1 < 0 ? arg : sh.i1;
    } else if (threadIdx.x == 0) {
        out[r] = sh.i0;
    }
}

// The kernel above: one CTA per row, any vocabulary.
AP_EXPORT int ap_sample_rows(const float* logits, long long row_stride, int R, int V, const float* temperature,
                             const int* top_k, const float* top_p, const float* uniform, int* out,
                             cudaStream_t stream) {
    AP_REQUIRE(R >= 0 && V > 0 && row_stride >= V, "sample: bad sizes R=%d V=%d", R, V);
    if (R == 0) return AP_OK;
    sample_kernel<<<R, SAMP_THREADS, 0, stream>>>(logits, row_stride, V, temperature, top_k, top_p, uniform, out);
    AP_CHECK_LAUNCH("sample");
    return AP_OK;
}

// sampling_cluster.cu: a cluster of CTAs per row, the row in registers
extern "C" int ap_sample_cluster_max_vocab(void);
extern "C" int ap_sample_cluster(const float* logits, long long row_stride, int R, int V, const float* temperature,
                                 const int* top_k, const float* top_p, const float* uniform, int* out,
                                 cudaStream_t stream);

// One token per row: the cluster kernel where the vocabulary fits its registers (up to 262144
// entries), else one CTA per row.
AP_EXPORT int ap_sample(const float* logits, long long row_stride, int R, int V, const float* temperature,
                        const int* top_k, const float* top_p, const float* uniform, int* out,
                        cudaStream_t stream) {
    if (V > 0 && V <= ap_sample_cluster_max_vocab() && R <= 65535)
        return ap_sample_cluster(logits, row_stride, R, V, temperature, top_k, top_p, uniform, out, stream);
    return ap_sample_rows(logits, row_stride, R, V, temperature, top_k, top_p, uniform, out, stream);
}
