// Causal grouped-query attention for long prompt portions on the 5th-generation tensor cores:
// the kernel of attention_tcgen05.cu with two query tiles to a CTA, for head sizes 64 and 128.
//
// That kernel is bound by bringing K and V to the SM: every tile of 128 keys (64 KB) serves 128
// query rows.  Here a CTA owns 256 rows = two tiles "a" and "b" of (128 / group) tokens x the
// `group` query heads of one KV head, and every K and V tile that reaches shared memory
// serves both: half the traffic for the same arithmetic.  Tensor memory holds S_a, S_b, O_a,
// O_b (4 x 128 columns); the two tiles take turns, so the tensor cores work on one while the
// softmax warps work on the other:
//
//   tensor cores   ... P_a V -> O_a | Q_a K'^T -> S_a | P_b V -> O_b | Q_b K'^T -> S_b ...
//   softmax a      ... (waits)      |                 | softmax of S_a -> P_a            ...
//   softmax b      ... softmax of S_b -> P_b          | (waits)        |                 ...
//
// A softmax group is four warps, one row per thread, the row's 128 scores of the tile in
// registers (one pass over tensor memory: maximum, then probabilities packed over the scores).
// For that the block is three groups of four warps: `setmaxnreg` takes registers from the
// last (the loading warp, the issuing warp, two idle ones: 56 each) and gives them to the two
// softmax groups (224 each), which adds up to what the launch holds.  P goes back
// into tensor memory over the S it came from (two bfloat16 to a column) and is the second
// product's A operand there; O is accumulated in tensor memory over all key tiles and scaled
// down only when a row's maximum has grown by more than 2^8 over its reference.  Loads,
// masks, pages and the bounded waits are those of attention_tcgen05.cu.
//
// Reference counterpart: attention_qtile_kernel (cuda/src/kernels.cu:1801), causal rule
// :1583-1585.
#include "common.cuh"
#include "tcgen05.cuh"
#include <math.h>

#ifndef AP_HEAD_DIM
#error "compile with -DAP_HEAD_DIM=<head size>"
#endif

#if (AP_HEAD_DIM == 64 || AP_HEAD_DIM == 128)

#define HD AP_HEAD_DIM
#define NHALF (HD / 64)
#define BQ 128
#define BKV 128
#define SUB_BYTES (128 * 128)              // a [128 rows x 64 bf16] sub-tile
#define Q_BYTES (NHALF * SUB_BYTES)        // one query tile
#define KV_BYTES (NHALF * SUB_BYTES)       // K (or V) of one tile
#define W5_THREADS 384                     // 2 x 4 softmax warps, then producer warp, MMA warp and two idle ones
#define W5_PRODUCER_WARP 8
#define W5_MMA_WARP 9
#define W5_TMEM_COLS 512                   // S_a, S_b: 2 x 128 columns; O_a, O_b: 2 x HD
#define W5_O_COL 256
#define W5_STAGES 2
#define LOG2E_F 1.4426950408889634f
#define W5_ERR_WAIT 7

static __device__ int g_w5_status;

__device__ __forceinline__ float w5_max3(float a, float b, float c) {
    float r;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}
// 2^x by the special-function unit; exactly 0 for x = -inf
__device__ __forceinline__ float w5_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

struct AttnW5Params {
    bf16* out;
    const int* block_table;
    const int* seq_start;
    const int* positions;
    int max_blocks, nseq, nh, nkv, P, window, group, tokens_per_tile;   // tokens_per_tile: of one query tile
    float scale_log2;
};

struct W5Smem {
    static constexpr int kQ = 0;                                  // tile a, tile b
    static constexpr int kK = kQ + 2 * Q_BYTES;
    static constexpr int kV = kK + W5_STAGES * KV_BYTES;
    static constexpr int kBars = kV + W5_STAGES * KV_BYTES;
    static constexpr int kTotal = kBars + 256 + 1024;             // + alignment slack
};

__global__ void __launch_bounds__(W5_THREADS, 1)
attention_tcgen05_wide_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_kv,
                              const __grid_constant__ CUtensorMap tmap_run, const AttnW5Params p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = (uint64_t*)(smem + W5Smem::kBars);
    uint64_t* q_full = bars + 0;
    uint64_t* k_full = bars + 1;                          // [stage]
    uint64_t* v_full = k_full + W5_STAGES;                // [stage]
    uint64_t* kv_free = v_full + W5_STAGES;               // [key tile & 1]: V of that tile and K of the next are read
    uint64_t* s_full = kv_free + 2;                       // [query tile]
    uint64_t* p_ready = s_full + 2;                       // [query tile]
    uint64_t* o_full = p_ready + 2;                       // [query tile]: the last product into O is done
    uint32_t* tmem_slot = (uint32_t*)(o_full + 2);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
    volatile int* s_seq = (volatile int*)(tmem_slot + 2);
    volatile int* s_tile = (volatile int*)(tmem_slot + 3);

    if (*(volatile int*)&g_w5_status != 0) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int per_cta = 2 * p.tokens_per_tile;            // tokens of one CTA

    if (threadIdx.x == 0) {
        // late portions of a sequence have the most keys to walk: hand them out first
        // (the KV head is the fast index of the grid: all heads of the longest portions start first)
        int t = (int)((gridDim.x - 1 - blockIdx.x) / (unsigned)p.nkv), found = -1;
        for (int s = 0; s < p.nseq; ++s) {
            const int n = p.seq_start[s + 1] - p.seq_start[s];
            const int nt = (n + per_cta - 1) / per_cta;
            if (t < nt) { found = s; break; }
            t -= nt;
        }
        *s_seq = found;
        *s_tile = t;
        tc::mbar_init(q_full, 1);
        for (int s = 0; s < W5_STAGES; ++s) {
            tc::mbar_init(&k_full[s], 1);
            tc::mbar_init(&v_full[s], 1);
        }
        for (int x = 0; x < 2; ++x) {
            tc::mbar_init(&kv_free[x], 1);
            tc::mbar_init(&s_full[x], 1);
            tc::mbar_init(&p_ready[x], 4);                // one arrival per warp of the tile's group
            tc::mbar_init(&o_full[x], 1);
        }
        *abort_flag = 0;
        tc::fence_barrier_init();
        tc::prefetch_tensormap(&tmap_q);
        tc::prefetch_tensormap(&tmap_kv);
        tc::prefetch_tensormap(&tmap_run);
    }
    // V stages and the second query tile start as zeros: what a skipped page (or a tile b that
    // does not exist) leaves there must be finite, because zero times a NaN would poison a row
    for (int i = threadIdx.x; i < W5_STAGES * KV_BYTES / 16; i += W5_THREADS)
        reinterpret_cast<uint4*>(smem + W5Smem::kV)[i] = make_uint4(0, 0, 0, 0);
    for (int i = threadIdx.x; i < Q_BYTES / 16; i += W5_THREADS)
        reinterpret_cast<uint4*>(smem + W5Smem::kQ + Q_BYTES)[i] = make_uint4(0, 0, 0, 0);
    tc::fence_proxy_async();
    if (warp == W5_MMA_WARP) tc::tmem_alloc(tmem_slot, W5_TMEM_COLS);
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const int seq = *s_seq;
    const uint32_t tmem_base = *tmem_slot;
    const bool active = seq >= 0;

    // geometry of this CTA (identical in every thread)
    const int G = p.group;
    int row0 = 0, ntok = 0, kmax = -1, kmin = 0, kvh = 0, head0 = 0;
    if (active) {
        row0 = p.seq_start[seq] + *s_tile * per_cta;
        ntok = min(per_cta, p.seq_start[seq + 1] - row0);
        kvh = (int)(blockIdx.x % (unsigned)p.nkv);
        head0 = kvh * G;
    }
    const bool has_b = ntok > p.tokens_per_tile;          // the second query tile holds rows
    ap_pdl_wait();
    if (active) {
        kmax = p.positions[row0 + ntok - 1];
        const int first = p.positions[row0];
        kmin = (p.window > 0 && first - p.window + 1 > 0) ? first - p.window + 1 : 0;
    }
    const int t_lo = kmin / BKV, t_hi = active ? kmax / BKV : -1;
    const int ntiles = t_hi - t_lo + 1;
    const int* table = p.block_table + (size_t)(active ? seq : 0) * p.max_blocks;

    // Registers move from the warps that only issue copies and products to the softmax warps,
    // which hold a row of 128 scores each (the unit of such a move is four warps)
    if (warp >= 8) {
    asm volatile("setmaxnreg.dec.sync.aligned.u32 56;");
    if (warp == W5_PRODUCER_WARP) {
        if (active) {
            if (lane == 0) {
                tc::mbar_expect_tx(q_full, (uint32_t)((has_b ? 2 : 1) * Q_BYTES));
                for (int x = 0; x < (has_b ? 2 : 1); ++x)
                    for (int h = 0; h < NHALF; ++h)
                        tc::tma_load_3d(smem + W5Smem::kQ + x * Q_BYTES + h * SUB_BYTES, &tmap_q, h * 64, head0,
                                        row0 + x * p.tokens_per_tile, q_full);
            }
            const int pages_per_tile = BKV / p.P;
            const int page_bytes = p.P * 128;                       // one page, one half: P rows of 128 bytes
            auto page_of = [&](int it) {
                const int lp = (t_lo + it) * (BKV / p.P) + lane;
                if (it >= ntiles || lane >= pages_per_tile || lp >= p.max_blocks || lp * p.P > kmax ||
                    lp * p.P + p.P - 1 < kmin)
                    return -1;
                return table[lp];
            };
            // `after`: the key tile whose turn in the MMA warp frees the stage (kv_free is given one
            // arrival before the first turn, "tile -1", and one at the end of every turn)
            auto load = [&](int it, int page, int which, uint64_t* full, int after, int base) -> int {
                const int s = it % W5_STAGES;
                const int valid = __popc(__ballot_sync(0xffffffffu, page >= 0));
                int fine = 1;
                if (lane == 0) {
                    if (*abort_flag) fine = 0;
                    if (fine && it >= W5_STAGES &&
                        !tc::mbar_wait(&kv_free[after & 1], (uint32_t)(((after + (after & 1)) >> 1) & 1))) {
                        *abort_flag = 1;
                        atomicExch(&g_w5_status, W5_ERR_WAIT);
                        fine = 0;
                    }
                    if (fine) tc::mbar_expect_tx(&full[s], (uint32_t)(valid * page_bytes * NHALF));
                }
                fine = __shfl_sync(0xffffffffu, fine, 0);
                // pages that follow one another in memory come with one box per half
                const int page0 = __shfl_sync(0xffffffffu, page, 0);
                const bool run = page0 >= 0 &&
                                 __all_sync(0xffffffffu, lane >= pages_per_tile || page == page0 + lane);
                if (fine && run) {
                    if (lane == 0) {
                        for (int h = 0; h < NHALF; ++h)
                            tc::tma_load_3d(smem + base + s * KV_BYTES + h * SUB_BYTES, &tmap_run, h * 64,
                                            (which * p.nkv + kvh) * p.P, page0, &full[s]);
                    }
                } else if (fine && page >= 0) {
                    const int row = ((page * 2 + which) * p.nkv + kvh) * p.P;
                    for (int h = 0; h < NHALF; ++h)
                        tc::tma_load_2d(smem + base + s * KV_BYTES + h * SUB_BYTES + lane * page_bytes, &tmap_kv,
                                        h * 64, row, &full[s]);
                }
                return fine;
            };
            // K runs one tile ahead of V; the block table is read four tiles ahead of its use
            int page_v = page_of(0);
            int q0 = page_of(1), q1 = page_of(2), q2 = page_of(3), q3 = page_of(4);
            int fine = load(0, page_v, 0, k_full, 0, W5Smem::kK);
            for (int it = 0; it < ntiles && fine; ++it) {
                const int page_k = q0;
                q0 = q1; q1 = q2; q2 = q3;
                q3 = page_of(it + 5);
                // K of tile j was read by the scores of turn j - 1; V of tile j by the products of turn j
                if (it + 1 < ntiles) fine = load(it + 1, page_k, 0, k_full, it - 2, W5Smem::kK);
                if (fine) fine = load(it, page_v, 1, v_full, it - 2, W5Smem::kV);
                page_v = page_k;
            }
        }
    } else if (warp == W5_MMA_WARP) {
        if (lane == 0 && active) {
            constexpr uint32_t idesc_s = tc::instr_desc_bf16_f32(BQ, BKV);
            constexpr uint32_t idesc_o = tc::instr_desc_bf16_f32_b_mn(BQ, HD);
            const int nx = has_b ? 2 : 1;
            // S_x = Q_x K^T of key tile `it`
            auto scores = [&](int it, int x) {
                const int s = it % W5_STAGES;
#pragma unroll
                for (int h = 0; h < NHALF; ++h) {
                    const uint64_t qd = tc::smem_desc_k_major_sw128(smem + W5Smem::kQ + x * Q_BYTES + h * SUB_BYTES);
                    const uint64_t kd = tc::smem_desc_k_major_sw128(smem + W5Smem::kK + s * KV_BYTES + h * SUB_BYTES);
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        tc::mma_bf16(tmem_base + (uint32_t)(x * BKV), qd + 2 * k, kd + 2 * k, idesc_s,
                                     (h > 0 || k > 0) ? 1u : 0u);
                }
                tc::mma_commit(&s_full[x]);
            };
            bool ok = tc::mbar_wait(q_full, 0);
            if (ok) ok = tc::mbar_wait(&k_full[0], 0);
            if (ok) {
                tc::fence_after_sync();
                for (int x = 0; x < nx; ++x) scores(0, x);
                tc::mma_commit(&kv_free[1]);              // "tile -1": K of tile 0 is read
            }
            for (int it = 0; it < ntiles && ok; ++it) {
                const int sv = it % W5_STAGES;
                const bool more = it + 1 < ntiles;
                // V of this tile and K of the next have been on their way for a whole turn; what this
                // thread then waits for is the softmax group's P
                ok = tc::mbar_wait(&v_full[sv], (uint32_t)((it / W5_STAGES) & 1)) &&
                     (!more || tc::mbar_wait(&k_full[(it + 1) % W5_STAGES], (uint32_t)(((it + 1) / W5_STAGES) & 1)));
                if (!ok || *abort_flag) break;
                const uint64_t vd = tc::smem_desc_mn_major_sw128(smem + W5Smem::kV + sv * KV_BYTES, SUB_BYTES);
                for (int x = 0; x < nx && ok; ++x) {
                    // O_x += P_x V as soon as the tile's group has written P_x (and scaled O_x down
                    // where a row's reference maximum moved); then S_x of the next key tile, which
                    // the group turns to while the other tile's products run
                    ok = tc::mbar_wait(&p_ready[x], (uint32_t)(it & 1));
                    if (!ok) break;
                    tc::fence_after_sync();
                    const uint32_t pt = tmem_base + (uint32_t)(x * BKV);      // P_x lies over S_x
#pragma unroll
                    for (int ks = 0; ks < 8; ++ks)
                        tc::mma_bf16_a_tmem(tmem_base + (uint32_t)(W5_O_COL + x * HD), pt + (uint32_t)(ks * 8),
                                            vd + (uint64_t)(ks * (16 * 128 / 16)), idesc_o, (it > 0 || ks > 0) ? 1u : 0u);
                    if (!more) tc::mma_commit(&o_full[x]);
                    if (more) scores(it + 1, x);
                }
                if (!ok) break;
                tc::mma_commit(&kv_free[it & 1]);
            }
            if (!ok && !*abort_flag) {
                *abort_flag = 1;
                atomicExch(&g_w5_status, W5_ERR_WAIT);
            }
        }
    }
    } else {
    asm volatile("setmaxnreg.inc.sync.aligned.u32 224;");
    if (active && (warp < 4 || has_b)) {
        // ---- softmax: warps 0..3 own query tile a, warps 4..7 tile b; one row per thread ----
        const int x = warp >> 2;
        const int qtr = warp & 3;
        const int r = qtr * 32 + lane;                 // row of the tile = (token r / G, head r % G)
        const int tok = x * p.tokens_per_tile + r / G, hq = r % G;
        const bool rvalid = tok < ntok;
        const uint32_t lane_base = tmem_base + ((uint32_t)(qtr * 32) << 16);
        const uint32_t s_cols = lane_base + (uint32_t)(x * BKV);
        const uint32_t o_cols = lane_base + (uint32_t)(W5_O_COL + x * HD);
        const int qpos = p.positions[row0 + (rvalid ? tok : 0)];
        float mref = -INFINITY, l = 0.f;               // the row's reference maximum (log2 units) and sum
        bool ok = true;                                // the same in all lanes of a warp
        for (int it = 0; it < ntiles; ++it) {
            const int k0 = (t_lo + it) * BKV;
            // tcgen05.ld and .st are warp-wide instructions: whatever decides whether one runs is a vote
            if (!__all_sync(0xffffffffu, tc::mbar_wait(&s_full[x], (uint32_t)(it & 1)))) { ok = false; break; }
            tc::fence_after_sync();
            const bool row_all = rvalid && k0 + BKV - 1 <= qpos && (p.window <= 0 || qpos - k0 < p.window);
            const bool row_none = !rvalid || k0 > qpos || (p.window > 0 && qpos - (k0 + BKV - 1) >= p.window);
            const bool all_visible = __all_sync(0xffffffffu, row_all);
            const bool none_visible = __all_sync(0xffffffffu, row_none);
            float lsum = 0.f;
            if (none_visible) {
                // nothing of this tile is for this warp's rows: P = 0
                uint32_t zero[32];
#pragma unroll
                for (int j = 0; j < 32; ++j) zero[j] = 0u;
                tc::tmem_st_x32(s_cols, zero);
                tc::tmem_st_x32(s_cols + 32u, zero);
            } else {
                // the row's 128 scores, masked ones as -inf (their probability below is exactly zero)
                uint32_t v[128];
#pragma unroll
                for (int c = 0; c < 128; c += 32) tc::tmem_ld_x32(s_cols + (uint32_t)c, v + c);
                tc::tmem_ld_wait();
                if (!all_visible) {
#pragma unroll
                    for (int j = 0; j < 128; ++j) {
                        const int kpos = k0 + j;
                        const bool vis = rvalid && kpos <= qpos && (p.window <= 0 || qpos - kpos < p.window);
                        v[j] = vis ? v[j] : 0xff800000u;
                    }
                }
                float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
                for (int j = 0; j < 128; j += 2)
                    mx4[(j >> 1) & 3] = w5_max3(mx4[(j >> 1) & 3], __uint_as_float(v[j]), __uint_as_float(v[j + 1]));
                // the scale is positive: the maximum of the scaled scores is the scaled maximum
                const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * p.scale_log2;
                const bool grow = mx > mref + 8.0f;            // also the row's first visible key
                float alpha = 1.f;
                if (grow) {
                    alpha = w5_exp2(mref - mx);                // 0 when the row had no key yet
                    mref = mx;
                    l *= alpha;
                }
                if (it > 0 && __any_sync(0xffffffffu, grow)) {
                    // scale this warp's rows of O_x down.  The product of the tile before into O_x is in:
                    // it was issued before the scores whose arrival (s_full) this warp has seen, and an
                    // arrival stands for everything issued before it
#pragma unroll 1
                    for (int c = 0; c < HD; c += 32) {
                        uint32_t w[32];
                        tc::tmem_ld_x32(o_cols + (uint32_t)c, w);
                        tc::tmem_ld_wait();
#pragma unroll
                        for (int j = 0; j < 32; ++j) w[j] = __float_as_uint(__uint_as_float(w[j]) * alpha);
                        tc::tmem_st_x32(o_cols + (uint32_t)c, w);
                    }
                    tc::tmem_st_wait();
                }
                // probabilities, two bfloat16 to a column, over the first half of S
                const float muse = mref == -INFINITY ? 0.f : mref;
                const float2 scale2 = make_float2(p.scale_log2, p.scale_log2), shift2 = make_float2(-muse, -muse);
                float2 l2[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
#pragma unroll
                for (int j = 0; j < 128; j += 2) {
                    const float2 a = __ffma2_rn(make_float2(__uint_as_float(v[j]), __uint_as_float(v[j + 1])), scale2, shift2);
                    const float2 e = make_float2(w5_exp2(a.x), w5_exp2(a.y));
                    l2[(j >> 1) & 1] = __fadd2_rn(l2[(j >> 1) & 1], e);
                    __nv_bfloat162 b2 = __floats2bfloat162_rn(e.x, e.y);
                    v[j >> 1] = *reinterpret_cast<uint32_t*>(&b2);
                }
                lsum = (l2[0].x + l2[0].y) + (l2[1].x + l2[1].y);
                tc::tmem_st_x32(s_cols, v);
                tc::tmem_st_x32(s_cols + 32u, v + 32);
            }
            l += lsum;
            tc::tmem_st_wait();
            tc::fence_before_sync();
            __syncwarp();                       // every lane's part of P is written: one arrival for the warp
            if (lane == 0) tc::mbar_arrive(&p_ready[x]);
        }
        // the last product into O_x, then the row goes out
        if (ok && !__all_sync(0xffffffffu, tc::mbar_wait(&o_full[x], 0))) ok = false;
        tc::fence_after_sync();
        if (!ok) {
            if (!*abort_flag) {
                *abort_flag = 1;
                atomicExch(&g_w5_status, W5_ERR_WAIT);
            }
        } else {
            const float inv = l > 0.f ? 1.0f / l : 0.f;
            bf16* dst = p.out + ((size_t)(row0 + (rvalid ? tok : 0)) * p.nh + head0 + hq) * HD;
#pragma unroll 1
            for (int c = 0; c < HD; c += 32) {
                uint32_t w[32];
                tc::tmem_ld_x32(o_cols + (uint32_t)c, w);
                tc::tmem_ld_wait();
                if (rvalid) {
#pragma unroll
                    for (int d = 0; d < 32; d += 8) {
                        uint4 o8;
                        __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o8);
#pragma unroll
                        for (int e = 0; e < 4; ++e)
                            o2[e] = __floats2bfloat162_rn(__uint_as_float(w[d + 2 * e]) * inv,
                                                          __uint_as_float(w[d + 2 * e + 1]) * inv);
                        *reinterpret_cast<uint4*>(dst + c + d) = o8;
                    }
                }
            }
        }
    }
    }
    tc::fence_before_sync();
    __syncthreads();
    ap_pdl_trigger();
    if (warp == W5_MMA_WARP) {
        __syncwarp();
        tc::tmem_dealloc(tmem_base, W5_TMEM_COLS);
    }
}

// ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFnW5)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFnW5 encode_fn_w5() {
    static EncodeTiledFnW5 fn = nullptr;
    if (!fn) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFnW5)ptr;
    }
    return fn;
}

// 1 when ap_attention_tcgen05_wide takes this shape, else 0
AP_EXPORT int ap_attention_tcgen05_wide_supports(int nh, int nkv, int hd, int P) {
    if (hd != HD || nkv <= 0 || nh % nkv) return 0;
    const int g = nh / nkv;
    if (g > 128 || 128 % g) return 0;
    if (P <= 0 || P % 8 || BKV % P) return 0;
    return encode_fn_w5() != nullptr;
}

// tokens of one sequence that one CTA takes (two query tiles)
AP_EXPORT int ap_attention_tcgen05_wide_tokens_per_cta(int nh, int nkv) { return 2 * (128 / (nh / nkv)); }

// As ap_attention_tcgen05; `total_ctas`: the sum over the sequences of ceil(rows / tokens per CTA).
AP_EXPORT int ap_attention_tcgen05_wide(const void* q, void* out, const void* cache, long long num_pages,
                                        const int* block_table, int max_blocks, const int* seq_start,
                                        const int* positions, int nseq, int T, int nh, int nkv, int hd, int P,
                                        long long page_stride, float scale, int window, int total_ctas,
                                        cudaStream_t stream) {
    AP_REQUIRE(ap_attention_tcgen05_wide_supports(nh, nkv, hd, P), "attention (tcgen05, two query tiles): shape not "
               "supported: heads=%d kv_heads=%d head_dim=%d page=%d", nh, nkv, hd, P);
    AP_REQUIRE(page_stride == 2LL * nkv * P * HD, "attention (tcgen05): pages must be contiguous");
    AP_REQUIRE(T > 0 && nseq > 0 && total_ctas > 0 && max_blocks > 0 && num_pages > 0, "attention (tcgen05): bad sizes");
    AP_REQUIRE(((uintptr_t)q & 15) == 0 && ((uintptr_t)cache & 15) == 0, "attention (tcgen05): operands must be 16-byte aligned");
    const int G = nh / nkv;
    EncodeTiledFnW5 enc = encode_fn_w5();
    CUtensorMap mq, mkv, mrun;
    {
        cuuint64_t dims[3] = {(cuuint64_t)HD, (cuuint64_t)nh, (cuuint64_t)T};
        cuuint64_t strides[2] = {(cuuint64_t)HD * 2, (cuuint64_t)nh * HD * 2};
        cuuint32_t box[3] = {64, (cuuint32_t)G, (cuuint32_t)(128 / G)};
        cuuint32_t es[3] = {1, 1, 1};
        AP_REQUIRE(enc(&mq, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(q), dims, strides, box, es,
                       CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                       CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS,
                   "attention (tcgen05): cannot encode the query tensor map");
    }
    {
        cuuint64_t dims[2] = {(cuuint64_t)HD, (cuuint64_t)(num_pages * 2 * nkv * P)};
        cuuint64_t strides[1] = {(cuuint64_t)HD * 2};
        cuuint32_t box[2] = {64, (cuuint32_t)P};
        cuuint32_t es[2] = {1, 1};
        AP_REQUIRE(enc(&mkv, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(cache), dims, strides, box, es,
                       CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                       CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS,
                   "attention (tcgen05): cannot encode the cache tensor map");
    }
    {
        // the same cache as [page][row within the page][column]: a box spans the pages of a key tile
        cuuint64_t dims[3] = {(cuuint64_t)HD, (cuuint64_t)(2 * nkv * P), (cuuint64_t)num_pages};
        cuuint64_t strides[2] = {(cuuint64_t)HD * 2, (cuuint64_t)page_stride * 2};
        cuuint32_t box[3] = {64, (cuuint32_t)P, (cuuint32_t)(BKV / P)};
        cuuint32_t es[3] = {1, 1, 1};
        AP_REQUIRE(enc(&mrun, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(cache), dims, strides, box, es,
                       CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                       CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS,
                   "attention (tcgen05): cannot encode the tensor map of page runs");
    }
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(attention_tcgen05_wide_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             W5Smem::kTotal);
        AP_REQUIRE(e == cudaSuccess, "attention (tcgen05): cannot reserve %d bytes of shared memory: %s",
                   W5Smem::kTotal, cudaGetErrorString(e));
        configured = true;
    }
    AttnW5Params p;
    p.out = (bf16*)out; p.block_table = block_table; p.seq_start = seq_start; p.positions = positions;
    p.max_blocks = max_blocks; p.nseq = nseq; p.nh = nh; p.nkv = nkv; p.P = P; p.window = window; p.group = G;
    p.tokens_per_tile = 128 / G;
    p.scale_log2 = scale * LOG2E_F;
    AP_REQUIRE((long long)total_ctas * nkv < (1LL << 31), "attention (tcgen05): too many CTAs for the grid");
    dim3 grid((unsigned)(total_ctas * nkv));
    AP_CHECK_PDL_LAUNCH("attention_tcgen05_wide", ap_launch_pdl(attention_tcgen05_wide_kernel, grid, dim3(W5_THREADS),
                                                                (size_t)W5Smem::kTotal, stream, mq, mkv, mrun, p));
    return AP_OK;
}

AP_EXPORT int ap_attention_tcgen05_wide_status(void) {
    int v = -1;
    if (cudaMemcpyFromSymbol(&v, g_w5_status, sizeof(int)) != cudaSuccess) return -1;
    return v;
}

#else   // head sizes the tcgen05 kernels are not built for

AP_EXPORT int ap_attention_tcgen05_wide_supports(int, int, int, int) { return 0; }

#endif
