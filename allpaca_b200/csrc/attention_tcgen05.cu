// Causal grouped-query attention for prompt portions on the 5th-generation tensor cores,
// over paged keys and values, for head sizes 64 and 128 (-DAP_HEAD_DIM).
//
// A CTA owns 128 rows = (128 / group) tokens x the `group` query heads of one KV head of
// one sequence, and walks the sequence's keys in tiles of 128:
//
//   TMA      Q once (a 3-D box tokens x heads x 64 columns per half of the head), then per
//            tile the pages of K and V named by the block table (one 2-D box per page and
//            half), into two stages of shared memory, 128-byte swizzle.
//   MMA 1    S[128 x 128] = Q K^T        tcgen05.mma, accumulator in tensor memory
//   softmax  two groups of four warps, one row per thread and 64 of the tile's 128 keys per
//            group: read S from tensor memory, scale, mask, running maximum and sum in
//            32-bit, write P in bfloat16 back into tensor memory (two to a column, over the
//            part of S just read), where the second product takes its A operand.  The two
//            groups keep separate running maxima, like two key slices, and are combined at
//            the end; eight warps give every scheduler two streams of this latency-bound work.
//   MMA 2    O_g[128 x HD] += P_g V_g for each group's 64 keys, accumulated in tensor memory
//            over all tiles.  V is stored [key][dim], i.e. the B operand is "MN-major": no
//            transposition of V anywhere.
//
// A row's probabilities are taken against a reference maximum that is moved only when the
// true maximum has grown by more than 2^8 over it; only then is the row of O_g in tensor
// memory scaled down (read, multiplied, written back by the row's thread).  The row sum uses
// the same reference, so the quotient is the same up to rounding, and the scaling, which would
// otherwise cost a pass over O per tile, happens a few times per row.
//
// One thread issues the MMAs, one warp the TMA loads.  S and P are double-buffered and K and V
// have barriers of their own, so the tensor cores compute S of tile i+1 and P V of tile i-1
// while the softmax warps work on tile i.  Every barrier wait is bounded (status word as in
// the matrix product).  Rows of other sequences that fall into a tile, keys past a row's
// position or outside its window, and pages that were given back are masked or skipped.
//
// Shapes this kernel takes: head size 64 or 128, page size a multiple of 8 that divides
// 128, a group size that divides 128.  Everything else runs on attention_tile_kernel.
//
// Reference counterpart: attention_qtile_kernel (cuda/src/kernels.cu:1801), causal rule
// :1583-1585; the reference first packs pages into a contiguous buffer
// (crates/allpaca-core/src/kv_tier.rs:1317-1417).
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
#define Q_BYTES (NHALF * SUB_BYTES)
#define KV_BYTES (NHALF * SUB_BYTES)       // K (or V) of one tile
#define T5_THREADS 320                     // producer warp, MMA warp, 2 x 4 softmax warps
#define T5_TMEM_COLS 512                   // S twice: 2 x 128 columns, then two O_tiles of HD columns
#define T5_O_COL 256
#define LOG2E_F 1.4426950408889634f

#define T5_ERR_WAIT 4
#define T5_KV_STAGES 2                     // K and V tiles in flight: a load takes longer than a tile's products

static __device__ int g_t5_status;

__device__ __forceinline__ float t5_max3(float a, float b, float c) {
    float r;
    asm("max.f32 %0, %1, %2, %3;" : "=f"(r) : "f"(a), "f"(b), "f"(c));
    return r;
}

// 2^x by the special-function unit; exactly 0 for x = -inf
__device__ __forceinline__ float t5_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

struct AttnT5Params {
    bf16* out;
    const int* block_table;
    const int* seq_start;
    const int* positions;
    int max_blocks, nseq, nh, nkv, P, window, group, tokens_per_tile;
    float scale_log2;
};

struct T5Smem {
    static constexpr int kQ = 0;
    static constexpr int kK = kQ + Q_BYTES;                 // two stages
    static constexpr int kV = kK + T5_KV_STAGES * KV_BYTES;
    static constexpr int kBars = kV + T5_KV_STAGES * KV_BYTES;
    static constexpr int kTotal = kBars + 256 + 1024;       // + alignment slack
};

__global__ void __launch_bounds__(T5_THREADS)
attention_tcgen05_kernel(const __grid_constant__ CUtensorMap tmap_q, const __grid_constant__ CUtensorMap tmap_kv,
                         const __grid_constant__ CUtensorMap tmap_run,
                         const AttnT5Params p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = (uint64_t*)(smem + T5Smem::kBars);
    uint64_t* q_full = bars + 0;
    uint64_t* k_full = bars + 1;                          // [stage]
    uint64_t* k_empty = k_full + T5_KV_STAGES;            // [stage]
    uint64_t* v_full = k_empty + T5_KV_STAGES;            // [stage]
    uint64_t* v_empty = v_full + T5_KV_STAGES;            // [stage]
    uint64_t* s_full = v_empty + T5_KV_STAGES;            // [S buffer]
    uint64_t* p_ready = s_full + 2;                       // [softmax group][P buffer]
    uint64_t* o_full = p_ready + 4;                       // [softmax group]
    uint32_t* tmem_slot = (uint32_t*)(o_full + 2);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
    volatile int* s_seq = (volatile int*)(tmem_slot + 2);
    volatile int* s_tile = (volatile int*)(tmem_slot + 3);

    if (*(volatile int*)&g_t5_status != 0) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    if (threadIdx.x == 0) {
        // late tiles of a sequence have the most keys to walk: hand them out first
        // (the KV head is the fast index of the grid: all heads of the longest portions start first)
        int t = (int)((gridDim.x - 1 - blockIdx.x) / (unsigned)p.nkv), found = -1;
        for (int s = 0; s < p.nseq; ++s) {
            const int n = p.seq_start[s + 1] - p.seq_start[s];
            const int nt = (n + p.tokens_per_tile - 1) / p.tokens_per_tile;
            if (t < nt) { found = s; break; }
            t -= nt;
        }
        *s_seq = found;
        *s_tile = t;
        tc::mbar_init(q_full, 1);
        for (int s = 0; s < T5_KV_STAGES; ++s) {
            tc::mbar_init(&k_full[s], 1);
            tc::mbar_init(&k_empty[s], 1);
            tc::mbar_init(&v_full[s], 1);
            tc::mbar_init(&v_empty[s], 1);
        }
        for (int s = 0; s < 2; ++s) {
            tc::mbar_init(&s_full[s], 1);
            tc::mbar_init(&p_ready[s], 4);          // one arrival per warp of the group
            tc::mbar_init(&p_ready[2 + s], 4);
            tc::mbar_init(&o_full[s], 1);
        }
        *abort_flag = 0;
        tc::fence_barrier_init();
        tc::prefetch_tensormap(&tmap_q);
        tc::prefetch_tensormap(&tmap_kv);
        tc::prefetch_tensormap(&tmap_run);
    }
    // V stages start as zeros: what a skipped page leaves in them must be finite, because a
    // probability of zero times a NaN would poison the row
    for (int i = threadIdx.x; i < T5_KV_STAGES * KV_BYTES / 16; i += T5_THREADS)
        reinterpret_cast<uint4*>(smem + T5Smem::kV)[i] = make_uint4(0, 0, 0, 0);
    tc::fence_proxy_async();
    if (warp == 1) tc::tmem_alloc(tmem_slot, T5_TMEM_COLS);
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const int seq = *s_seq;
    const uint32_t tmem_base = *tmem_slot;
    const bool active = seq >= 0;

    // geometry of this CTA's tile (identical in every thread)
    const int G = p.group;
    int row0 = 0, ntok = 0, kmax = -1, kmin = 0, kvh = 0, head0 = 0;
    if (active) {
        row0 = p.seq_start[seq] + *s_tile * p.tokens_per_tile;
        ntok = min(p.tokens_per_tile, p.seq_start[seq + 1] - row0);
        kvh = (int)(blockIdx.x % (unsigned)p.nkv);
        head0 = kvh * G;
        // positions are read after the kernels before this one have finished
    }
    ap_pdl_wait();
    if (active) {
        kmax = p.positions[row0 + ntok - 1];
        const int first = p.positions[row0];
        kmin = (p.window > 0 && first - p.window + 1 > 0) ? first - p.window + 1 : 0;
    }
    const int t_lo = kmin / BKV, t_hi = active ? kmax / BKV : -1;
    const int ntiles = t_hi - t_lo + 1;
    const int* table = p.block_table + (size_t)(active ? seq : 0) * p.max_blocks;

    if (warp == 0) {
        if (active) {
            // The whole warp produces: lane j looks up page j of the tile in the block table and
            // issues that page's loads, so the table reads of a tile cost one round trip to L2.
            if (lane == 0) {
                tc::mbar_expect_tx(q_full, Q_BYTES);
                for (int h = 0; h < NHALF; ++h)
                    tc::tma_load_3d(smem + T5Smem::kQ + h * SUB_BYTES, &tmap_q, h * 64, head0, row0, q_full);
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
            // K runs one tile ahead of V: K of tile i+1 feeds S of tile i+1, which the tensor cores
            // compute while the softmax warps are still on tile i; V of tile i is wanted last.
            auto load = [&](int it, int page, int which, uint64_t* full, uint64_t* empty, int base) -> int {
                const int s = it % T5_KV_STAGES;
                const uint32_t ph = (uint32_t)((it / T5_KV_STAGES) & 1);
                const int valid = __popc(__ballot_sync(0xffffffffu, page >= 0));
                int fine = 1;
                if (lane == 0) {
                    if (*abort_flag) fine = 0;
                    if (fine && !tc::mbar_wait(&empty[s], ph ^ 1)) {
                        *abort_flag = 1;
                        atomicExch(&g_t5_status, T5_ERR_WAIT);
                        fine = 0;
                    }
                    if (fine) tc::mbar_expect_tx(&full[s], (uint32_t)(valid * page_bytes * NHALF));
                }
                fine = __shfl_sync(0xffffffffu, fine, 0);
                // The pages of a tile often follow one another in memory (a sequence's pages are
                // handed out in rising order): then one box per half fetches them all.  Loads are
                // issued at a limited rate, so few large ones keep the tensor cores fed where
                // many small ones do not.
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
            // The block table is read four tiles ahead of its use: a lookup is a round trip to L2,
            // and one per tile on the loads' critical path would be most of a tile's time.
            int page_v = page_of(0);
            int q0 = page_of(1), q1 = page_of(2), q2 = page_of(3), q3 = page_of(4);
            int fine = load(0, page_v, 0, k_full, k_empty, T5Smem::kK);
            for (int it = 0; it < ntiles && fine; ++it) {
                const int page_k = q0;                              // pages of tile it + 1
                q0 = q1; q1 = q2; q2 = q3;
                q3 = page_of(it + 5);
                if (it + 1 < ntiles) fine = load(it + 1, page_k, 0, k_full, k_empty, T5Smem::kK);
                if (fine) fine = load(it, page_v, 1, v_full, v_empty, T5Smem::kV);
                page_v = page_k;
            }
        }
    } else if (warp == 1) {
        if (lane == 0 && active) {
            constexpr uint32_t idesc_s = tc::instr_desc_bf16_f32(BQ, BKV);
            constexpr uint32_t idesc_o = tc::instr_desc_bf16_f32_b_mn(BQ, HD);
            const uint32_t tmem_o = tmem_base + T5_O_COL;
            // S[buffer it & 1] = Q K^T of tile `it`; K's stage is free as soon as this product is done
            auto scores = [&](int it) -> bool {
                const int s = it % T5_KV_STAGES, sb = it & 1;          // K stage, S buffer
                if (!tc::mbar_wait(&k_full[s], (uint32_t)((it / T5_KV_STAGES) & 1))) return false;
                tc::fence_after_sync();
#pragma unroll
                for (int h = 0; h < NHALF; ++h) {
                    const uint64_t qd = tc::smem_desc_k_major_sw128(smem + T5Smem::kQ + h * SUB_BYTES);
                    const uint64_t kd = tc::smem_desc_k_major_sw128(smem + T5Smem::kK + s * KV_BYTES + h * SUB_BYTES);
#pragma unroll
                    for (int k = 0; k < 4; ++k)
                        tc::mma_bf16(tmem_base + (uint32_t)(sb * BKV), qd + 2 * k, kd + 2 * k, idesc_s,
                                     (h > 0 || k > 0) ? 1u : 0u);
                }
                tc::mma_commit(&k_empty[s]);
                tc::mma_commit(&s_full[sb]);
                return true;
            };
            bool ok = tc::mbar_wait(q_full, 0);
            if (ok) ok = scores(0);
            for (int it = 0; it < ntiles && ok && !*abort_flag; ++it) {
                const int s = it & 1, sv = it % T5_KV_STAGES;          // S/P buffer, V stage
                // S of tile it+1 goes into the buffer that tile it-1 used; the softmax groups have
                // handed over P of tile it-1 (waited for below, one iteration ago), so they have read it
                if (it + 1 < ntiles) ok = scores(it + 1);
                if (ok) ok = tc::mbar_wait(&v_full[sv], (uint32_t)((it / T5_KV_STAGES) & 1));
                // O_g += P_g V_g, one product per softmax group as soon as its P is written (by then
                // the group has also scaled O_g down where a row's reference maximum moved)
                const uint64_t vd = tc::smem_desc_mn_major_sw128(smem + T5Smem::kV + sv * KV_BYTES, SUB_BYTES);
                for (int g = 0; g < 2 && ok; ++g) {
                    ok = tc::mbar_wait(&p_ready[g * 2 + s], (it >> 1) & 1);
                    if (!ok) break;
                    tc::fence_after_sync();
                    // P_g lies in tensor memory, over the first columns of the half of S it came from
                    const uint32_t pt = tmem_base + (uint32_t)(s * BKV + g * 64);
#pragma unroll
                    for (int ks = 0; ks < 4; ++ks)
                        tc::mma_bf16_a_tmem(tmem_o + g * HD, pt + (uint32_t)(ks * 8),
                                            vd + (uint64_t)((g * 4 + ks) * (16 * 128 / 16)), idesc_o,
                                            (it > 0 || ks > 0) ? 1u : 0u);
                    tc::mma_commit(&o_full[g]);
                }
                if (!ok) break;
                tc::mma_commit(&v_empty[sv]);
            }
            if (!ok && !*abort_flag) {
                *abort_flag = 1;
                atomicExch(&g_t5_status, T5_ERR_WAIT);
            }
        }
    }
    // ---- softmax groups: warps 2..5 take keys 0..63 of every tile, warps 6..9 keys 64..127 ----
    const int grp = warp >= 6 ? 1 : 0;
    const int qtr = warp & 3;
    const int r = qtr * 32 + lane;                 // row of the tile = (token r / G, head r % G)
    const int tok = r / G, hq = r - tok * G;
    const bool rvalid = active && warp >= 2 && tok < ntok;
    const uint32_t lane_base = tmem_base + ((uint32_t)(qtr * 32) << 16);
    const uint32_t o_cols = lane_base + (uint32_t)(T5_O_COL + grp * HD);
    float mref = -INFINITY, l = 0.f;               // the row's reference maximum (log2 units) and sum
    bool ok = true;                                // the same in all lanes of a warp
    if (warp >= 2 && active) {
        const int qpos = p.positions[row0 + (rvalid ? tok : 0)];
        for (int it = 0; it < ntiles; ++it) {
            const int k0 = (t_lo + it) * BKV + grp * 64;       // first key of this group's half tile
            const int buf = it & 1;
            const uint32_t s_cols = lane_base + (uint32_t)(buf * BKV + grp * 64);
            // tcgen05.ld and .st are warp-wide instructions: whatever decides whether one runs is a vote
            if (!__all_sync(0xffffffffu, tc::mbar_wait(&s_full[buf], (it >> 1) & 1))) { ok = false; break; }
            tc::fence_after_sync();
            const bool row_all = rvalid && k0 + 63 <= qpos && (p.window <= 0 || qpos - k0 < p.window);
            const bool row_none = !rvalid || k0 > qpos || (p.window > 0 && qpos - (k0 + 63) >= p.window);
            const bool all_visible = __all_sync(0xffffffffu, row_all);
            const bool none_visible = __all_sync(0xffffffffu, row_none);
            uint32_t packed[32];
            float lsum = 0.f;
            if (none_visible) {
#pragma unroll
                for (int j = 0; j < 32; ++j) packed[j] = 0u;
            } else {
                uint32_t v[64];
                tc::tmem_ld_x32(s_cols, v);
                tc::tmem_ld_x32(s_cols + 32u, v + 32);
                tc::tmem_ld_wait();
                if (!all_visible) {
                    // a masked score becomes -inf, whose probability below is exactly zero
#pragma unroll
                    for (int j = 0; j < 64; ++j) {
                        const int kpos = k0 + j;
                        const bool vis = rvalid && kpos <= qpos && (p.window <= 0 || qpos - kpos < p.window);
                        v[j] = vis ? v[j] : 0xff800000u;
                    }
                }
                // (three-input maximum and two-wide multiply-add and add: half the instructions)
                float mx4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
                for (int j = 0; j < 64; j += 2)
                    mx4[(j >> 1) & 3] = t5_max3(mx4[(j >> 1) & 3], __uint_as_float(v[j]), __uint_as_float(v[j + 1]));
                // the scale is positive: the maximum of the scaled scores is the scaled maximum
                const float mx = fmaxf(fmaxf(mx4[0], mx4[1]), fmaxf(mx4[2], mx4[3])) * p.scale_log2;
                const bool grow = mx > mref + 8.0f;            // also the row's first visible key
                float alpha = 1.f;
                if (grow) {
                    alpha = t5_exp2(mref - mx);                // 0 when the row had no key yet
                    mref = mx;
                    l *= alpha;
                }
                if (it > 0 && __any_sync(0xffffffffu, grow)) {
                    // scale this warp's rows of O_g down, once the product of the tile before is in
                    if (!__all_sync(0xffffffffu, tc::mbar_wait(&o_full[grp], (it - 1) & 1))) { ok = false; break; }
                    tc::fence_after_sync();
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
                const float muse = mref == -INFINITY ? 0.f : mref;
                float2 l2[2] = {make_float2(0.f, 0.f), make_float2(0.f, 0.f)};
                const float2 scale2 = make_float2(p.scale_log2, p.scale_log2), shift2 = make_float2(-muse, -muse);
#pragma unroll
                for (int j = 0; j < 64; j += 2) {
                    const float2 a = __ffma2_rn(make_float2(__uint_as_float(v[j]), __uint_as_float(v[j + 1])), scale2, shift2);
                    const float2 x = make_float2(t5_exp2(a.x), t5_exp2(a.y));
                    l2[(j >> 1) & 1] = __fadd2_rn(l2[(j >> 1) & 1], x);
                    __nv_bfloat162 b2 = __floats2bfloat162_rn(x.x, x.y);
                    packed[j >> 1] = *reinterpret_cast<uint32_t*>(&b2);
                }
                lsum = (l2[0].x + l2[0].y) + (l2[1].x + l2[1].y);
            }
            l += lsum;
            // P goes back into tensor memory, two bfloat16 to a column, over the part of S this
            // thread has just read: the second product takes it from there
            tc::tmem_st_x32(s_cols, packed);
            tc::tmem_st_wait();
            tc::fence_before_sync();
            __syncwarp();                       // every lane's part of P is written: one arrival for the warp
            if (lane == 0) tc::mbar_arrive(&p_ready[grp * 2 + buf]);
        }
        // the last product into O_g
        if (ok && !__all_sync(0xffffffffu, tc::mbar_wait(&o_full[grp], (ntiles - 1) & 1))) ok = false;
        tc::fence_after_sync();
        if (!ok && !*abort_flag) {
            *abort_flag = 1;
            atomicExch(&g_t5_status, T5_ERR_WAIT);
        }
    }
    // ---- combine the two groups (like two key slices) and write the rows ----
    __syncthreads();                       // every load has landed and every product is done
    const bool fine = active && !*abort_flag;
    constexpr int XS = HD + 3;             // row stride in floats: odd, so rows fall into different banks
    float* xch = reinterpret_cast<float*>(smem + T5Smem::kK);      // [128 rows][XS], over the K/V stages
    if (warp >= 6 && fine) {
        float* dst = xch + (size_t)r * XS;
#pragma unroll 1
        for (int c = 0; c < HD; c += 32) {
            uint32_t w[32];
            tc::tmem_ld_x32(o_cols + (uint32_t)c, w);
            tc::tmem_ld_wait();
#pragma unroll
            for (int j = 0; j < 32; ++j) dst[c + j] = __uint_as_float(w[j]);
        }
        dst[HD] = mref;
        dst[HD + 1] = l;
    }
    __syncthreads();
    if (warp >= 2 && warp < 6 && fine) {
        const float* src = xch + (size_t)r * XS;
        const float m1 = src[HD], l1 = src[HD + 1];
        const float M = fmaxf(mref, m1);
        const float f0 = mref == -INFINITY ? 0.f : t5_exp2(mref - M), f1 = m1 == -INFINITY ? 0.f : t5_exp2(m1 - M);
        const float L = l * f0 + l1 * f1;
        const float inv = L > 0.f ? 1.0f / L : 0.f;
        const float g0 = f0 * inv, g1 = f1 * inv;
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
                    for (int e = 0; e < 4; ++e) {
                        // a group that saw no key of this row holds zeros (0 x finite V) or, where
                        // its factor is zero, is not counted at all
                        const float a0 = f0 > 0.f ? __uint_as_float(w[d + 2 * e]) * g0 : 0.f;
                        const float a1 = f0 > 0.f ? __uint_as_float(w[d + 2 * e + 1]) * g0 : 0.f;
                        const float b0 = f1 > 0.f ? src[c + d + 2 * e] * g1 : 0.f;
                        const float b1 = f1 > 0.f ? src[c + d + 2 * e + 1] * g1 : 0.f;
                        o2[e] = __floats2bfloat162_rn(a0 + b0, a1 + b1);
                    }
                    *reinterpret_cast<uint4*>(dst + c + d) = o8;
                }
            }
        }
    }
    tc::fence_before_sync();
    __syncthreads();
    ap_pdl_trigger();
    if (warp == 1) {
        __syncwarp();
        tc::tmem_dealloc(tmem_base, T5_TMEM_COLS);
    }
}

// ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn5)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                   const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                   CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn5 encode_fn5() {
    static EncodeTiledFn5 fn = nullptr;
    if (!fn) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn5)ptr;
    }
    return fn;
}

// 1 when ap_attention_tcgen05 takes this shape, else 0 (the caller then uses the tile kernel)
AP_EXPORT int ap_attention_tcgen05_supports(int nh, int nkv, int hd, int P) {
    if (hd != HD || nkv <= 0 || nh % nkv) return 0;
    const int g = nh / nkv;
    if (g > 128 || 128 % g) return 0;
    if (P <= 0 || P % 8 || BKV % P) return 0;
    return encode_fn5() != nullptr;
}

AP_EXPORT int ap_attention_tcgen05_tokens_per_tile(int nh, int nkv) { return 128 / (nh / nkv); }

AP_EXPORT int ap_attention_tcgen05(const void* q, void* out, const void* cache, long long num_pages,
                                   const int* block_table, int max_blocks, const int* seq_start,
                                   const int* positions, int nseq, int T, int nh, int nkv, int hd, int P,
                                   long long page_stride, float scale, int window, int total_tiles,
                                   cudaStream_t stream) {
    AP_REQUIRE(ap_attention_tcgen05_supports(nh, nkv, hd, P), "attention (tcgen05): shape not supported: heads=%d "
               "kv_heads=%d head_dim=%d page=%d", nh, nkv, hd, P);
    AP_REQUIRE(page_stride == 2LL * nkv * P * HD, "attention (tcgen05): pages must be contiguous");
    AP_REQUIRE(T > 0 && nseq > 0 && total_tiles > 0 && max_blocks > 0 && num_pages > 0, "attention (tcgen05): bad sizes");
    AP_REQUIRE(((uintptr_t)q & 15) == 0 && ((uintptr_t)cache & 15) == 0, "attention (tcgen05): operands must be 16-byte aligned");
    const int G = nh / nkv;
    EncodeTiledFn5 enc = encode_fn5();
    CUtensorMap mq, mkv;
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
    CUtensorMap mrun;
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
        cudaError_t e = cudaFuncSetAttribute(attention_tcgen05_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             T5Smem::kTotal);
        AP_REQUIRE(e == cudaSuccess, "attention (tcgen05): cannot reserve %d bytes of shared memory: %s",
                   T5Smem::kTotal, cudaGetErrorString(e));
        configured = true;
    }
    AttnT5Params p;
    p.out = (bf16*)out; p.block_table = block_table; p.seq_start = seq_start; p.positions = positions;
    p.max_blocks = max_blocks; p.nseq = nseq; p.nh = nh; p.nkv = nkv; p.P = P; p.window = window; p.group = G;
    p.tokens_per_tile = 128 / G;
    p.scale_log2 = scale * LOG2E_F;
    AP_REQUIRE((long long)total_tiles * nkv < (1LL << 31), "attention (tcgen05): too many CTAs for the grid");
    dim3 grid((unsigned)(total_tiles * nkv));
    AP_CHECK_PDL_LAUNCH("attention_tcgen05", ap_launch_pdl(attention_tcgen05_kernel, grid, dim3(T5_THREADS),
                                                           (size_t)T5Smem::kTotal, stream, mq, mkv, mrun, p));
    return AP_OK;
}

AP_EXPORT int ap_attention_tcgen05_status(void) {
    int v = -1;
    if (cudaMemcpyFromSymbol(&v, g_t5_status, sizeof(int)) != cudaSuccess) return -1;
    return v;
}

#else   // head sizes the tcgen05 kernel is not built for

AP_EXPORT int ap_attention_tcgen05_supports(int, int, int, int) { return 0; }

#endif
