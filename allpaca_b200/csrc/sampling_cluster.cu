// Temperature / top-k / top-p sampling with a thread-block cluster per row of logits.
//
// The meaning of the options is that of sampling.cu (the reference's
// crates/allpaca-core/src/sampling.rs: temperature :227-234, non-finite logits dropped
// :236-244, top_k with ties to the lower token id :246-271, top_p as the smallest prefix by
// descending logit whose probability reaches it :276-309, soft-max :311-331, one draw by a
// walk with a uniform number :55-67, here in token-id order).  What differs is how the work
// is laid out: one CTA per row has to pass a vocabulary of 128 k entries a dozen times on one
// SM, and a histogram in shared memory serialises where most logits share their leading
// bits.  Here eight CTAs (4096 threads) hold a row in registers, each thread a run of
// consecutive token ids, and no pass writes a histogram:
//
//   * the cut of top_k or top_p lies at some logit between the row's minimum and maximum.
//     A pass counts (or sums the weights exp(l - max) of) the logits above each of fifteen
//     thresholds that divide the current interval evenly, the cluster adds the partial
//     results through distributed shared memory, and the interval shrinks to the sixteenth
//     that holds the cut.  Two or three passes leave at most 2048 candidates;
//   * the candidates go to the first CTA, which sorts them (by logit descending, token id
//     ascending) and reads the cut off the sorted list;
//   * with a top_k of up to 2048 the list holds every survivor: top_p and the draw are then
//     finished on the list by the first CTA alone.  Otherwise the survivors stay where they
//     are, and the draw is a prefix sum of their weights in token-id order over the cluster.
//
// Every decision that steers a CTA is taken from values that all CTAs of the cluster read in
// the same order, so they all take the same way to every cluster barrier.
#include "common.cuh"
#include <cooperative_groups.h>
#include <float.h>

namespace cg = cooperative_groups;

#define SC_THREADS 512
#define SC_WARPS (SC_THREADS / 32)
#define SC_CLUSTER 8
#define SC_PROBES 15
#define SC_CAP 2048            // candidates the first CTA sorts
#define SC_WORDS 24            // 32-bit words a CTA publishes per exchange
#define SC_MAX_PASSES 64
#define SC_REACH 120.0f        // exp(-120) is zero in 32-bit: logits further below the maximum weigh nothing

__device__ __forceinline__ unsigned sc_key(float f) {
    unsigned u = __float_as_uint(f);
    return (u & 0x80000000u) ? ~u : (u | 0x80000000u);   // ascending floats -> ascending keys
}
__device__ __forceinline__ float sc_unkey(unsigned k) {
    return __uint_as_float((k & 0x80000000u) ? (k & 0x7fffffffu) : ~k);
}

struct ScCut {          // keep key > key, or key == key with id <= tie_id
    unsigned key;
    int tie_id;
    int active;         // 0: keeps everything
};
__device__ __forceinline__ bool sc_passes(const ScCut& c, unsigned key, int id) {
    return !c.active || key > c.key || (key == c.key && id <= c.tie_id);
}

struct ScShared {
    unsigned pub[2][SC_WORDS];              // what this CTA shows the others (two in turn)
    unsigned all[SC_CLUSTER][SC_WORDS];     // every CTA's words of the last exchange
    unsigned wred[SC_WARPS][SC_WORDS];      // per-warp partial results
    float sum[SC_WORDS];                    // the cluster's results of a pass
    float scan_f[SC_WARPS];
    int scan_i[SC_WARPS];
    int pick;
    unsigned long long list[SC_CAP];        // candidates, gathered in the first CTA
    float weight[SC_CAP];
};

// Every CTA has written pub[parity]; afterwards all[r] holds CTA r's words in every CTA.
// pub[parity] is written again two exchanges later: by then every CTA has passed the barrier
// of the exchange between, which it reaches only after it has read this one.
__device__ __forceinline__ void sc_exchange(cg::cluster_group& cl, ScShared& sh, int& parity) {
    cl.sync();
    const int t = threadIdx.x;
    if (t < SC_CLUSTER * SC_WORDS) {
        const int r = t / SC_WORDS, i = t % SC_WORDS;
        const unsigned* remote = cl.map_shared_rank(&sh.pub[parity][0], r);
        sh.all[r][i] = remote[i];
    }
    __syncthreads();
    parity ^= 1;
}

// exclusive prefix of v over the block's threads, the block's total through *total
__device__ __forceinline__ int sc_scan_int(int v, ScShared& sh, int* total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int x = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const int y = __shfl_up_sync(0xffffffffu, x, o);
        if (lane >= o) x += y;
    }
    __syncthreads();
    if (lane == 31) sh.scan_i[warp] = x;
    __syncthreads();
    int before = 0, tot = 0;
#pragma unroll
    for (int w = 0; w < SC_WARPS; ++w) {
        const int wt = sh.scan_i[w];
        if (w < warp) before += wt;
        tot += wt;
    }
    *total = tot;
    return before + x - v;
}
// inclusive prefix of v over the block's threads; *total is the last thread's prefix itself
__device__ __forceinline__ float sc_scan_float(float v, ScShared& sh, float* total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float x = v;
#pragma unroll
    for (int o = 1; o < 32; o <<= 1) {
        const float y = __shfl_up_sync(0xffffffffu, x, o);
        if (lane >= o) x += y;
    }
    __syncthreads();
    if (lane == 31) sh.scan_f[warp] = x;
    __syncthreads();
    float before = 0.f, tot = 0.f;
#pragma unroll
    for (int w = 0; w < SC_WARPS; ++w) {
        const float wt = sh.scan_f[w];
        if (w < warp) before += wt;
        tot += wt;
    }
    // (before + x) of the last thread must be what *total says: the same additions in the same order
    *total = tot;
    return before + x;
}

// list[0..n) sorted in place; n2 = n rounded up to a power of two, the rest filled with `pad`
template <bool DESCENDING>
__device__ void sc_sort(unsigned long long* list, int n, unsigned long long pad) {
    int n2 = 1;
    while (n2 < n) n2 <<= 1;
    for (int i = n + threadIdx.x; i < n2; i += SC_THREADS) list[i] = pad;
    __syncthreads();
    for (int k = 2; k <= n2; k <<= 1) {
        for (int j = k >> 1; j > 0; j >>= 1) {
            for (int i = threadIdx.x; i < n2; i += SC_THREADS) {
                const int o = i ^ j;
                if (o > i) {
                    const unsigned long long a = list[i], b = list[o];
                    const bool up = ((i & k) == 0) != DESCENDING;      // this pair in ascending order?
                    if ((a > b) == up) { list[i] = b; list[o] = a; }
                }
            }
            __syncthreads();
        }
    }
}

// inclusive prefix sums of weight[0..n) in place (n <= SC_CAP: four consecutive entries a thread)
__device__ float sc_prefix_weights(ScShared& sh, int n) {
    constexpr int PER = SC_CAP / SC_THREADS;
    float w[PER], s = 0.f;
    const int base = threadIdx.x * PER;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        w[i] = base + i < n ? sh.weight[base + i] : 0.f;
        s += w[i];
    }
    float total;
    const float incl = sc_scan_float(s, sh, &total);
    float run = incl - s;
#pragma unroll
    for (int i = 0; i < PER; ++i) {
        run += w[i];
        if (base + i < n) sh.weight[base + i] = run;
    }
    __syncthreads();
    return total;
}
// first index i < n with weight[i] >= target (prefix sums), or n
__device__ int sc_first_reaching(ScShared& sh, int n, float target) {
    if (threadIdx.x == 0) sh.pick = n;
    __syncthreads();
    for (int i = threadIdx.x; i < n; i += SC_THREADS)
        if (sh.weight[i] >= target && (i == 0 || sh.weight[i - 1] < target)) atomicMin(&sh.pick, i);
    __syncthreads();
    const int got = sh.pick;
    __syncthreads();
    return got;
}

template <int E>
struct ScRow {
    float l[E];         // logit / temperature, -inf for what is dropped or beyond the vocabulary
    int id0;            // token id of l[0]
};

// Where the cut lies.  Among the row's candidates (finite, passing c0) in descending order
// (ties by ascending token id) the cut is the first whose running weight reaches the target:
// weight 1 and target `count` for top_k, weight exp(l - m) and target frac * total for top_p.
//   gather_above == false: returns the cut (inactive when rounding leaves the total short);
//   gather_above == true:  stops as soon as everything above the interval's lower end fits the
//                          list, and leaves all of it sorted in the first CTA's list (*listed
//                          entries; the cut is entry number `count`).
template <int E>
__device__ ScCut sc_search(cg::cluster_group& cl, ScShared& sh, int& parity, const ScRow<E>& row, float m, float gmin,
                           const ScCut& c0, bool weighted, float count, float frac, bool gather_above, int* listed) {
    const int rank = (int)cl.block_rank();
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const float floor_lo = gmin - 1e-3f * fmaxf(1.f, fabsf(gmin));       // below every candidate
    float lo = fmaxf(floor_lo, m - SC_REACH), hi = m;
    float greater = 0.f;                 // weight of the candidates above hi
    float target = count;
    ScCut cut = {0u, 0, 0};
    int n_list = 0;
    bool degenerate = false, found = true;
    float n_cand = 0.f, equal_value = 0.f;
    for (int pass = 0; pass < SC_MAX_PASSES; ++pass) {
        const float step = (hi - lo) * (1.f / (SC_PROBES + 1));
        float acc[SC_PROBES];
#pragma unroll
        for (int j = 0; j < SC_PROBES; ++j) acc[j] = 0.f;
        float tot = 0.f, nc = 0.f, cmin = INFINITY, cmax = -INFINITY;
#pragma unroll
        for (int e = 0; e < E; ++e) {
            const float x = row.l[e];
            if (x > lo && x <= hi && sc_passes(c0, sc_key(x), row.id0 + e)) {
                const float w = weighted ? expf(x - m) : 1.f;
                tot += w;
                nc += 1.f;
                cmin = fminf(cmin, x);
                cmax = fmaxf(cmax, x);
#pragma unroll
                for (int j = 0; j < SC_PROBES; ++j) acc[j] += (x > hi - step * (float)(j + 1)) ? w : 0.f;
            }
        }
        // block: 15 sums, total, count (sums), minimum, maximum
#pragma unroll
        for (int j = 0; j < SC_PROBES; ++j) acc[j] = ap_warp_sum(acc[j]);
        tot = ap_warp_sum(tot);
        nc = ap_warp_sum(nc);
        cmin = -ap_warp_max(-cmin);
        cmax = ap_warp_max(cmax);
        __syncthreads();
        if (lane == 0) {
#pragma unroll
            for (int j = 0; j < SC_PROBES; ++j) sh.wred[warp][j] = __float_as_uint(acc[j]);
            sh.wred[warp][15] = __float_as_uint(tot);
            sh.wred[warp][16] = __float_as_uint(nc);
            sh.wred[warp][17] = __float_as_uint(cmin);
            sh.wred[warp][18] = __float_as_uint(cmax);
        }
        __syncthreads();
        if (threadIdx.x < 19) {
            float v = __uint_as_float(sh.wred[0][threadIdx.x]);
            for (int w = 1; w < SC_WARPS; ++w) {
                const float o = __uint_as_float(sh.wred[w][threadIdx.x]);
                v = threadIdx.x == 17 ? fminf(v, o) : threadIdx.x == 18 ? fmaxf(v, o) : v + o;
            }
            sh.pub[parity][threadIdx.x] = __float_as_uint(v);
        }
        sc_exchange(cl, sh, parity);
        // the cluster's results, added in the order of the ranks by one thread per word
        if (threadIdx.x < 19) {
            float v = __uint_as_float(sh.all[0][threadIdx.x]);
            for (int r = 1; r < SC_CLUSTER; ++r) {
                const float o = __uint_as_float(sh.all[r][threadIdx.x]);
                v = threadIdx.x == 17 ? fminf(v, o) : threadIdx.x == 18 ? fmaxf(v, o) : v + o;
            }
            sh.sum[threadIdx.x] = v;
        }
        __syncthreads();
        const float TOT = sh.sum[15], NC = sh.sum[16], CMIN = sh.sum[17], CMAX = sh.sum[18];
        if (pass == 0 && weighted) target = fmaxf(frac * TOT, FLT_MIN);
        if (greater + TOT < target) {
            // the cut lies below this interval
            if (lo <= floor_lo) {            // nothing is left below: rounding left the sum short
                found = false;
                break;
            }
            greater += TOT;
            hi = lo;
            lo = floor_lo;
            continue;
        }
        n_cand = NC;
        const float above = gather_above ? greater : 0.f;       // (a count, when everything above is gathered)
        if (above + NC <= (float)SC_CAP) break;
        if (CMIN == CMAX) {
            degenerate = true;
            equal_value = CMIN;
            break;
        }
        // the sixteenth that holds the cut
        int j = 0;
        while (j < SC_PROBES && greater + sh.sum[j] < target) ++j;
        const float new_hi = j == 0 ? hi : hi - step * (float)j;
        const float new_lo = j == SC_PROBES ? lo : hi - step * (float)(j + 1);
        if (j > 0) greater += sh.sum[j - 1];
        if (!(new_hi > new_lo) || (new_hi == hi && new_lo == lo)) {
            // the interval no longer divides: its candidates count as equal (cannot happen
            // while minimum and maximum differ by more than the spacing of floats)
            degenerate = true;
            equal_value = CMAX;
            hi = new_hi;
            lo = new_lo;
            break;
        }
        hi = new_hi;
        lo = new_lo;
    }
    if (!found) {
        if (listed) *listed = 0;
        return cut;
    }
    if (degenerate) {
        // more equal candidates than the list holds: the cut is the need-th of them by token id
        float need_f = weighted ? (expf(equal_value - m) > 0.f ? ceilf((target - greater) / expf(equal_value - m)) : n_cand)
                                : target - greater;
        need_f = fminf(fmaxf(need_f, 1.f), n_cand);
        const int need = (int)need_f;
        int mine = 0;
#pragma unroll
        for (int e = 0; e < E; ++e) {
            const float x = row.l[e];
            mine += (x > lo && x <= hi && sc_passes(c0, sc_key(x), row.id0 + e)) ? 1 : 0;
        }
        int block_total;
        int before = sc_scan_int(mine, sh, &block_total);
        if (threadIdx.x == 0) {
            sh.pub[parity][0] = (unsigned)block_total;
            sh.pub[parity][1] = 0u;
        }
        sc_exchange(cl, sh, parity);
        for (int r = 0; r < rank; ++r) before += (int)sh.all[r][0];
        if (threadIdx.x == 0) sh.pub[parity][1] = 0u;
        __syncthreads();
        if (before < need && need <= before + mine) {
            int seen = before;
#pragma unroll
            for (int e = 0; e < E; ++e) {
                const float x = row.l[e];
                if (x > lo && x <= hi && sc_passes(c0, sc_key(x), row.id0 + e) && ++seen == need) {
                    sh.pub[parity][0] = (unsigned)(row.id0 + e);
                    sh.pub[parity][1] = 1u;
                }
            }
        }
        sc_exchange(cl, sh, parity);
        cut.key = sc_key(equal_value);
        cut.active = 1;
        cut.tie_id = 0x7fffffff;
        for (int r = 0; r < SC_CLUSTER; ++r)
            if (sh.all[r][1]) cut.tie_id = (int)sh.all[r][0];
        if (listed) *listed = -1;            // no list: the caller goes on over the whole row
        return cut;
    }
    // the candidates (with gather_above: everything above lo) into the first CTA's list
    int mine = 0;
#pragma unroll
    for (int e = 0; e < E; ++e) {
        const float x = row.l[e];
        mine += (x > lo && (gather_above || x <= hi) && sc_passes(c0, sc_key(x), row.id0 + e)) ? 1 : 0;
    }
    int block_total;
    int at = sc_scan_int(mine, sh, &block_total);
    if (threadIdx.x == 0) sh.pub[parity][0] = (unsigned)block_total;
    sc_exchange(cl, sh, parity);
    for (int r = 0; r < SC_CLUSTER; ++r) {
        if (r < rank) at += (int)sh.all[r][0];
        n_list += (int)sh.all[r][0];
    }
    unsigned long long* first_list = cl.map_shared_rank(&sh.list[0], 0);
#pragma unroll
    for (int e = 0; e < E; ++e) {
        const float x = row.l[e];
        if (x > lo && (gather_above || x <= hi) && sc_passes(c0, sc_key(x), row.id0 + e)) {
            if (at < SC_CAP)
                first_list[at] = ((unsigned long long)sc_key(x) << 32) | (unsigned)(0xffffffffu - (unsigned)(row.id0 + e));
            ++at;
        }
    }
    cl.sync();
    if (n_list > SC_CAP) n_list = SC_CAP;        // (cannot happen: the pass counted them)
    if (rank == 0) {
        sc_sort<true>(sh.list, n_list, 0ull);
        if (!gather_above) {
            int at_cut = -1;
            if (!weighted) {
                at_cut = (int)(target - greater) - 1;
            } else {
                for (int i = threadIdx.x; i < n_list; i += SC_THREADS)
                    sh.weight[i] = expf(sc_unkey((unsigned)(sh.list[i] >> 32)) - m);
                __syncthreads();
                sc_prefix_weights(sh, n_list);
                const int i = sc_first_reaching(sh, n_list, target - greater);
                at_cut = i < n_list ? i : n_list - 1;      // rounding left the sum short: the interval's last
            }
            if (threadIdx.x == 0) {
                if (at_cut >= n_list) at_cut = n_list - 1;
                sh.pub[parity][2] = at_cut >= 0 ? 1u : 0u;
                if (at_cut >= 0) {
                    sh.pub[parity][0] = (unsigned)(sh.list[at_cut] >> 32);
                    sh.pub[parity][1] = 0xffffffffu - (unsigned)(sh.list[at_cut] & 0xffffffffu);
                }
            }
        }
    }
    if (gather_above) {
        if (listed) *listed = n_list;
        return cut;
    }
    sc_exchange(cl, sh, parity);
    cut.active = (int)sh.all[0][2];
    cut.key = sh.all[0][0];
    cut.tie_id = (int)sh.all[0][1];
    if (listed) *listed = -1;
    return cut;
}

template <int E>
__global__ void __launch_bounds__(SC_THREADS, 1)
sample_cluster_kernel(const float* __restrict__ logits, long long row_stride, int V,
                      const float* __restrict__ temperature, const int* __restrict__ top_k,
                      const float* __restrict__ top_p, const float* __restrict__ uniform, int* __restrict__ out) {
    cg::cluster_group cl = cg::this_cluster();
    __shared__ ScShared sh;
    const int rank = (int)cl.block_rank();
    const int r = blockIdx.y;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const float* src = logits + (size_t)r * row_stride;
    const float temp = temperature[r];
    const float tdiv = fmaxf(temp, 1e-5f);
    int parity = 0;

    ScRow<E> row;
    row.id0 = (rank * SC_THREADS + (int)threadIdx.x) * E;
    const bool vec = (((uintptr_t)src) & 15) == 0;
#pragma unroll
    for (int q = 0; q < E; q += 4) {
        const int id = row.id0 + q;
        float v[4];
        if (vec && id + 3 < V) {
            const float4 f = *reinterpret_cast<const float4*>(src + id);
            v[0] = f.x; v[1] = f.y; v[2] = f.z; v[3] = f.w;
        } else {
#pragma unroll
            for (int i = 0; i < 4; ++i) v[i] = id + i < V ? src[id + i] : INFINITY;
        }
#pragma unroll
        for (int i = 0; i < 4; ++i) row.l[q + i] = fabsf(v[i]) <= FLT_MAX ? v[i] / tdiv : -INFINITY;
    }

    // maximum (first index), minimum and number of the finite logits
    float bv = -INFINITY, mn = INFINITY;
    int bi = 0x7fffffff, cnt = 0;
#pragma unroll
    for (int e = 0; e < E; ++e) {
        const float x = row.l[e];
        if (x > -INFINITY) {
            ++cnt;
            mn = fminf(mn, x);
            if (x > bv) { bv = x; bi = row.id0 + e; }
        }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, bv, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
        mn = fminf(mn, __shfl_xor_sync(0xffffffffu, mn, o));
        cnt += __shfl_xor_sync(0xffffffffu, cnt, o);
    }
    if (lane == 0) {
        sh.wred[warp][0] = __float_as_uint(bv);
        sh.wred[warp][1] = (unsigned)bi;
        sh.wred[warp][2] = __float_as_uint(mn);
        sh.wred[warp][3] = (unsigned)cnt;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < SC_WARPS; ++w) {
            const float ov = __uint_as_float(sh.wred[w][0]);
            const int oi = (int)sh.wred[w][1];
            if (ov > bv || (ov == bv && oi < bi)) { bv = ov; bi = oi; }
            mn = fminf(mn, __uint_as_float(sh.wred[w][2]));
            cnt += (int)sh.wred[w][3];
        }
        sh.pub[parity][0] = __float_as_uint(bv);
        sh.pub[parity][1] = (unsigned)bi;
        sh.pub[parity][2] = __float_as_uint(mn);
        sh.pub[parity][3] = (unsigned)cnt;
    }
    sc_exchange(cl, sh, parity);
    float m = -INFINITY, gmin = INFINITY;
    int arg = 0x7fffffff, n_cand = 0;
    for (int c = 0; c < SC_CLUSTER; ++c) {
        const float ov = __uint_as_float(sh.all[c][0]);
        const int oi = (int)sh.all[c][1];
        if (ov > m || (ov == m && oi < arg)) { m = ov; arg = oi; }
        gmin = fminf(gmin, __uint_as_float(sh.all[c][2]));
        n_cand += (int)sh.all[c][3];
    }
    if (n_cand == 0 || temp <= 1e-5f) {          // nothing finite -> token 0; greedy -> first maximum
        if (rank == 0 && threadIdx.x == 0) out[r] = n_cand == 0 ? 0 : arg;
        cl.sync();
        return;
    }

    const int k = top_k[r];
    const float pth = top_p[r];
    const float u = uniform[r];
    const bool use_k = k > 0 && k < n_cand;
    const bool use_p = pth >= 0.f && pth < 1.f;
    const ScCut none = {0u, 0, 0};
    ScCut ck = none, cp = none;

    if (use_k && k <= SC_CAP) {
        // everything from the k-th logit up fits the list: the first CTA finishes alone
        int n_list = 0;
        ScCut tie = sc_search<E>(cl, sh, parity, row, m, gmin, none, false, (float)k, 0.f, true, &n_list);
        if (n_list >= 0) {
            if (rank == 0) {
                int kept = n_list < k ? n_list : k;
                if (use_p && kept > 1) {
                    for (int i = threadIdx.x; i < kept; i += SC_THREADS)
                        sh.weight[i] = expf(sc_unkey((unsigned)(sh.list[i] >> 32)) - m);
                    __syncthreads();
                    const float z = sc_prefix_weights(sh, kept);
                    const int i = sc_first_reaching(sh, kept, fmaxf(pth * z, FLT_MIN));
                    if (i < kept) kept = i + 1;
                }
                // in token-id order: (id, key), ascending
                for (int i = threadIdx.x; i < kept; i += SC_THREADS) {
                    const unsigned long long e = sh.list[i];
                    sh.list[i] = ((unsigned long long)(0xffffffffu - (unsigned)(e & 0xffffffffu)) << 32) | (e >> 32);
                }
                __syncthreads();
                sc_sort<false>(sh.list, kept, ~0ull);
                for (int i = threadIdx.x; i < kept; i += SC_THREADS)
                    sh.weight[i] = expf(sc_unkey((unsigned)(sh.list[i] & 0xffffffffu)) - m);
                __syncthreads();
                const float z = sc_prefix_weights(sh, kept);
                int i = sc_first_reaching(sh, kept, u * z);
                if (i >= kept) i = kept - 1;             // rounding left the walk short: the last survivor
                if (threadIdx.x == 0) out[r] = (int)(sh.list[i] >> 32);
            }
            cl.sync();
            return;
        }
        ck = tie;                   // more equal logits at the cut than the list holds: go on over the row
    } else if (use_k) {
        ck = sc_search<E>(cl, sh, parity, row, m, gmin, none, false, (float)k, 0.f, false, nullptr);
    }
    if (use_p && (!use_k || k > 1)) cp = sc_search<E>(cl, sh, parity, row, m, gmin, ck, true, 0.f, pth, false, nullptr);

    // the draw: prefix sums of the survivors' weights in token-id order
    float mine = 0.f;
    int alive = 0;
#pragma unroll
    for (int e = 0; e < E; ++e) {
        const float x = row.l[e];
        const unsigned key = sc_key(x);
        if (x > -INFINITY && sc_passes(ck, key, row.id0 + e) && sc_passes(cp, key, row.id0 + e)) {
            mine += expf(x - m);
            ++alive;
        }
    }
    float block_total;
    const float incl = sc_scan_float(mine, sh, &block_total);
    int alive_total;
    sc_scan_int(alive, sh, &alive_total);
    if (threadIdx.x == 0) {
        sh.pub[parity][0] = __float_as_uint(block_total);
        sh.pub[parity][1] = (unsigned)alive_total;
        sh.pick = 0x7fffffff;
    }
    sc_exchange(cl, sh, parity);
    float z = 0.f, before = 0.f;
    for (int c = 0; c < SC_CLUSTER; ++c) {
        if (c == rank) before = z;
        z += __uint_as_float(sh.all[c][0]);
    }
    const float target = u * z;
    // the CTA of the draw: the first with survivors whose prefix reaches the target, else the
    // last with survivors
    int chosen = -1, last_alive = -1;
    {
        float run = 0.f;
        for (int c = 0; c < SC_CLUSTER; ++c) {
            run += __uint_as_float(sh.all[c][0]);
            if (sh.all[c][1] > 0u) {
                last_alive = c;
                if (chosen < 0 && run >= target) chosen = c;
            }
        }
        if (chosen < 0) chosen = last_alive;
    }
    if (rank == chosen) {
        if (alive > 0 && before + incl >= target) atomicMin(&sh.pick, (int)threadIdx.x);
        __syncthreads();
        if (sh.pick == 0x7fffffff) {
            // rounding: nobody's prefix reaches the target; the last thread with survivors draws its last one
            __syncthreads();
            if (threadIdx.x == 0) sh.scan_i[0] = -1;
            __syncthreads();
            if (alive > 0) atomicMax(&sh.scan_i[0], (int)threadIdx.x);
            __syncthreads();
            if (threadIdx.x == 0) sh.pick = sh.scan_i[0];
            __syncthreads();
        }
        if ((int)threadIdx.x == sh.pick) {
            float run = before + incl - mine;
            int token = -1, last = -1;
#pragma unroll
            for (int e = 0; e < E; ++e) {
                const float x = row.l[e];
                const unsigned key = sc_key(x);
                if (x > -INFINITY && sc_passes(ck, key, row.id0 + e) && sc_passes(cp, key, row.id0 + e)) {
                    run += expf(x - m);
                    last = row.id0 + e;
                    if (token < 0 && run >= target) token = last;
                }
            }
            out[r] = token >= 0 ? token : last;
        }
    }
    cl.sync();
}

template <int E>
static int sc_launch(const float* logits, long long row_stride, int R, int V, const float* temperature,
                     const int* top_k, const float* top_p, const float* uniform, int* out, cudaStream_t stream) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(SC_CLUSTER, R);
    cfg.blockDim = dim3(SC_THREADS);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = SC_CLUSTER;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    cudaError_t e = cudaLaunchKernelEx(&cfg, sample_cluster_kernel<E>, logits, row_stride, V, temperature, top_k,
                                       top_p, uniform, out);
    AP_REQUIRE(e == cudaSuccess, "sample (cluster): launch failed: %s", cudaGetErrorString(e));
    return AP_OK;
}

// Largest vocabulary the cluster kernel takes (64 logits a thread)
AP_EXPORT int ap_sample_cluster_max_vocab(void) { return SC_CLUSTER * SC_THREADS * 64; }

AP_EXPORT int ap_sample_cluster(const float* logits, long long row_stride, int R, int V, const float* temperature,
                                const int* top_k, const float* top_p, const float* uniform, int* out,
                                cudaStream_t stream) {
    AP_REQUIRE(R >= 0 && V > 0 && row_stride >= V, "sample: bad sizes R=%d V=%d", R, V);
    AP_REQUIRE(V <= ap_sample_cluster_max_vocab(), "sample (cluster): a vocabulary of %d exceeds %d", V,
               ap_sample_cluster_max_vocab());
    AP_REQUIRE(R <= 65535, "sample (cluster): %d rows exceed the grid", R);
    if (R == 0) return AP_OK;
    const int per = (V + SC_CLUSTER * SC_THREADS - 1) / (SC_CLUSTER * SC_THREADS);
    if (per <= 4) return sc_launch<4>(logits, row_stride, R, V, temperature, top_k, top_p, uniform, out, stream);
    if (per <= 16) return sc_launch<16>(logits, row_stride, R, V, temperature, top_k, top_p, uniform, out, stream);
    if (per <= 32) return sc_launch<32>(logits, row_stride, R, V, temperature, top_k, top_p, uniform, out, stream);
    return sc_launch<64>(logits, row_stride, R, V, temperature, top_k, top_p, uniform, out, stream);
}
