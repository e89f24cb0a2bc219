// bfloat16 matrix product for many rows (prompt portions) on pairs of SMs:
//     out[M, N] = A[M, K] * W[N, K]^T
//
// Two CTAs of a thread-block cluster (two SMs) share one output tile of 256 weight rows x up
// to 256 tokens.  Each CTA brings 128 weight rows and HALF of the token rows into its shared
// memory by TMA; one thread of the pair's first CTA issues tcgen05.mma.cta_group::2, with
// which each SM's tensor cores multiply their own 128 weight rows with all the token rows,
// reading the other half from the partner's shared memory.  A block of 64 along K thus costs an
// SM 32 KB of loads for the products that cost 48 KB with one CTA to a tile, and what an SM can
// take in from L2 is what bounds these products.  Each CTA holds its 128 rows of the accumulator
// in its own tensor memory (twice: the epilogue warps write tile j while tile j+1 is computed).
//
// The kernel is persistent: one pair per two SMs walks the tiles round robin, token tile first,
// so that pairs running side by side share weight tiles in L2.
//
// Roles in each CTA: warp 0 = TMA producer for this CTA's halves; warp 1 = in the first CTA
// the MMA issuer (idle in the second); warps 2..5 = epilogue.  The loads of both CTAs are
// counted on the first CTA's barrier of the stage: the second CTA issues its loads with
// .cta_group::2 and that barrier's address (the data itself goes to the issuing CTA
// only), and the first CTA expects the bytes of both.  (A relay thread in the second CTA,
// forwarding "my stage has landed" by a remote arrival, cost 5 to 12 % of the product's time.)
// A stage is freed, and an accumulator handed to the epilogue, in both CTAs at once by
// tcgen05.commit with a multicast arrival.
//
// Every barrier wait has a time limit; on expiry the CTA raises a status word, lets its loads
// land and walks on to the cluster barrier at the end (its partner would wait there otherwise).
//
// Reference counterpart: gemm_nt_kernel (cuda/src/kernels.cu:431-459), one thread per output.
#include "common.cuh"
#include "tcgen05.cuh"

#define PAIR_TILE_W 128         // weight rows per CTA (256 per pair)
#define PAIR_TILE_K 64
#define PAIR_MAX_BN 256         // tokens per tile (both halves)
#define PAIR_STAGES 6
#define PAIR_W_BYTES (PAIR_TILE_W * PAIR_TILE_K * 2)
#define PAIR_A_BYTES ((PAIR_MAX_BN / 2) * PAIR_TILE_K * 2)
#define PAIR_STAGE_BYTES (PAIR_W_BYTES + PAIR_A_BYTES)
#define PAIR_SMEM_BYTES (PAIR_STAGES * PAIR_STAGE_BYTES + 1024 + 512)
#define PAIR_TMEM_COLS 512

#define PAIR_ERR_EMPTY 1
#define PAIR_ERR_FULL 2
#define PAIR_ERR_ACCUM 3
#define PAIR_ERR_TMEM 4

#define PAIR_ERR_PEER 5
#define PAIR_MAX_CTAS 256                                   // flags at the head of the scratch buffer
#define PAIR_PARTIAL_FLOATS ((long long)PAIR_TILE_W * PAIR_MAX_BN)   // per CTA: [token][weight row]
#define PAIR_MAX_SPLIT 4

static __device__ int g_pair_status;

// A pair's next piece of work: blocks [kb0, kb1) of K of one tile.  The first tiles_total - shared
// tiles go round robin to the pairs, whole (tile pair, pair + pairs, ...).  The last `shared`
// tiles are each cut along K into `split` ranges: pair g < shared * split takes range g / shared
// of tile (tiles_total - shared) + g % shared as its last piece of work, and the pair of range 0
// finishes the tile with what the others hand over in global memory.
struct PairWork { int tile, kb0, kb1, range; };
__device__ __forceinline__ bool pair_next(int& it, int pair, int pairs_in_grid, int tiles_total, int nkb, int split,
                                          int shared, PairWork& w) {
    if (it < 0) return false;
    const int whole = tiles_total - shared;
    const int tile = pair + it * pairs_in_grid;
    if (tile < whole) {
        ++it;
        w.tile = tile;
        w.kb0 = 0;
        w.kb1 = nkb;
        w.range = 0;
        return true;
    }
    it = -1;
    if (shared <= 0 || pair >= shared * split) return false;
    w.range = pair / shared;
    w.tile = whole + pair - w.range * shared;
    w.kb0 = (int)((long long)nkb * w.range / split);
    w.kb1 = (int)((long long)nkb * (w.range + 1) / split);
    return true;
}
__device__ __forceinline__ int pair_ld_acquire(const int* p) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void pair_st_release(int* p, int v) {
    asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ void pair_epilogue_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

template <typename TO, bool PAIRS>
__global__ void __launch_bounds__(192)
gemm_tc_pair_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_a,
                    TO* __restrict__ out, int M, int N, int K, long long ldc, int tiles_m, int tiles_total, int bn,
                    int split, int shared, int* __restrict__ flags, float* __restrict__ partials) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* w_tiles = smem;
    uint8_t* a_tiles = smem + PAIR_STAGES * PAIR_W_BYTES;
    uint64_t* full = (uint64_t*)(smem + PAIR_STAGES * PAIR_STAGE_BYTES);
    uint64_t* empty = full + PAIR_STAGES;
    uint64_t* acc_full = empty + PAIR_STAGES;        // [2]
    uint64_t* acc_empty = acc_full + 2;              // [2], first CTA: both CTAs' epilogues are done with it
    uint32_t* tmem_slot = (uint32_t*)(acc_empty + 2);
    uint32_t* peer_tmem = tmem_slot + 1;             // first CTA: where the second CTA's tensor memory starts
    volatile int* abort_flag = (volatile int*)(tmem_slot + 2);
    volatile int* peer_ok = (volatile int*)(tmem_slot + 3);
    uint64_t* xfer = acc_empty + 4;                  // [2]: other pairs' partial sums arriving in the idle ring

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t rank = tc::cluster_ctarank();            // 0: issues the MMAs
    const int pairs_in_grid = gridDim.x / 2, pair = blockIdx.x / 2;
    const int nkb = (K + PAIR_TILE_K - 1) / PAIR_TILE_K;
    const int half_bn = bn / 2;
    const uint32_t stage_bytes = (uint32_t)(PAIR_W_BYTES + half_bn * PAIR_TILE_K * 2);
    // once a wait has expired anywhere, later launches do no work (but walk to their barriers)
    const bool skip = *(volatile int*)&g_pair_status != 0;

    if (threadIdx.x == 0) {
        for (int s = 0; s < PAIR_STAGES; ++s) {
            tc::mbar_init(&full[s], 1);
            tc::mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            tc::mbar_init(&acc_full[b], 1);
            tc::mbar_init(&acc_empty[b], 2);              // one arrival from each CTA's epilogue
            tc::mbar_init(&xfer[b], 1);
        }
        *abort_flag = skip ? 1 : 0;
        tc::fence_barrier_init();
        tc::prefetch_tensormap(&tmap_w);
        tc::prefetch_tensormap(&tmap_a);
    }
    // All of this SM's tensor memory: the allocation then starts at the same place (column 0) in
    // both CTAs, which the pair's instructions require; it is granted once every other CTA on
    // this SM has given its tensor memory back.
    if (warp == 1) tc::tmem_alloc(tmem_slot, PAIR_TMEM_COLS);
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    if (threadIdx.x == 0 && rank == 1) {
        // tell the first CTA where this CTA's tensor memory starts
        const uint32_t remote = tc::map_to_rank(tc::smem_addr(peer_tmem), 0u);
        asm volatile("st.shared::cluster.u32 [%0], %1;" ::"r"(remote), "r"(tmem_base) : "memory");
    }
    tc::cluster_sync();          // both CTAs' barriers are initialised, the second CTA's address is here
    if (rank == 0 && threadIdx.x == 0 && *peer_tmem != tmem_base && !skip) {
        *abort_flag = 1;
        atomicCAS(&g_pair_status, 0, PAIR_ERR_TMEM);
    }
    __syncthreads();

    const int n_rank = rank * PAIR_TILE_W;            // this CTA's weight rows inside the tile
    const int m_rank = rank * half_bn;                // this CTA's token rows inside the tile

    if (warp == 0) {
        if (lane == 0) {
            long long idx = 0, issued = 0;
            bool first = true;
            int it = 0;
            PairWork wk;
            while (!*abort_flag && pair_next(it, pair, pairs_in_grid, tiles_total, nkb, split, shared, wk)) {
                const int tile = wk.tile;
                const int n0 = (tile / tiles_m) * 2 * PAIR_TILE_W + n_rank, m0 = (tile % tiles_m) * bn + m_rank;
                int kb = wk.kb0;
                if (first) {
                    // the weight does not depend on earlier kernels: fill the ring with weight blocks,
                    // then wait for the kernels that produce the activations
                    first = false;
                    const int pre = min(PAIR_STAGES, wk.kb1 - wk.kb0);
                    for (int i = 0; i < pre; ++i) {
                        if (rank == 0) {
                            tc::mbar_expect_tx(&full[i], 2 * stage_bytes);       // both CTAs' halves
                            tc::tma_load_2d(w_tiles + i * PAIR_W_BYTES, &tmap_w, (kb + i) * PAIR_TILE_K, n0, &full[i]);
                        } else {
                            tc::tma_load_2d_signal_peer(w_tiles + i * PAIR_W_BYTES, &tmap_w, (kb + i) * PAIR_TILE_K, n0,
                                                        tc::map_to_rank(tc::smem_addr(&full[i]), 0u));
                        }
                    }
                    ap_pdl_wait();
                    for (int i = 0; i < pre; ++i) {
                        if (rank == 0)
                            tc::tma_load_2d(a_tiles + i * PAIR_A_BYTES, &tmap_a, (kb + i) * PAIR_TILE_K, m0, &full[i]);
                        else
                            tc::tma_load_2d_signal_peer(a_tiles + i * PAIR_A_BYTES, &tmap_a, (kb + i) * PAIR_TILE_K, m0,
                                                        tc::map_to_rank(tc::smem_addr(&full[i]), 0u));
                    }
                    kb += pre;
                    idx = issued = pre;
                }
                for (; kb < wk.kb1; ++kb, ++idx) {
                    const int s = (int)(idx % PAIR_STAGES);
                    const uint32_t ph = (uint32_t)((idx / PAIR_STAGES) & 1);
                    if (*abort_flag) break;
                    if (!tc::mbar_wait(&empty[s], ph ^ 1)) {
                        *abort_flag = 1;
                        atomicCAS(&g_pair_status, 0, PAIR_ERR_EMPTY);
                        break;
                    }
                    if (rank == 0) {
                        tc::mbar_expect_tx(&full[s], 2 * stage_bytes);
                        tc::tma_load_2d(w_tiles + s * PAIR_W_BYTES, &tmap_w, kb * PAIR_TILE_K, n0, &full[s]);
                        tc::tma_load_2d(a_tiles + s * PAIR_A_BYTES, &tmap_a, kb * PAIR_TILE_K, m0, &full[s]);
                    } else {
                        const uint32_t leader = tc::map_to_rank(tc::smem_addr(&full[s]), 0u);
                        tc::tma_load_2d_signal_peer(w_tiles + s * PAIR_W_BYTES, &tmap_w, kb * PAIR_TILE_K, n0, leader);
                        tc::tma_load_2d_signal_peer(a_tiles + s * PAIR_A_BYTES, &tmap_a, kb * PAIR_TILE_K, m0, leader);
                    }
                    issued = idx + 1;
                }
            }
            if (first) ap_pdl_wait();
            // The arrivals that free the stages reach both CTAs of the pair from the tensor cores of
            // the first, and those of the last blocks are waited for by nobody: wait for them here,
            // so that none is still on its way when this CTA's shared memory passes to the next CTA
            // on this SM (where it would count as an arrival on that CTA's barrier).
            if (!*abort_flag) {
                for (long long i = max(0LL, idx - PAIR_STAGES); i < idx; ++i) {
                    if (!tc::mbar_wait(&empty[i % PAIR_STAGES], (uint32_t)((i / PAIR_STAGES) & 1))) {
                        *abort_flag = 1;
                        atomicCAS(&g_pair_status, 0, PAIR_ERR_EMPTY);
                        break;
                    }
                }
            }
            if (*abort_flag && rank == 0) {
                // let the loads that are still in flight (of both CTAs: all are counted here) land before
                // the CTAs' memory goes away; the second CTA leaves after the cluster barrier at the end
                for (long long i = max(0LL, issued - PAIR_STAGES); i < issued; ++i)
                    tc::mbar_wait(&full[i % PAIR_STAGES], (uint32_t)((i / PAIR_STAGES) & 1), 200000000LL);
            }
        }
    } else if (warp == 1) {
        if (rank == 1) {
            // (the second CTA's tensor cores are driven from the first)
        } else if (lane == 0) {
            const uint32_t idesc = tc::instr_desc_bf16_f32(2 * PAIR_TILE_W, bn);
            bool ok = true;
            long long idx = 0;
            int j = 0;
            int it = 0;
            PairWork wk;
            for (; ok && pair_next(it, pair, pairs_in_grid, tiles_total, nkb, split, shared, wk); ++j) {
                const int b = j & 1;
                // both CTAs' epilogue warps have read this buffer's tile of two rounds ago
                if (*abort_flag || !tc::mbar_wait(&acc_empty[b], (uint32_t)(((j >> 1) & 1) ^ 1))) {
                    if (!*abort_flag) {
                        *abort_flag = 1;
                        atomicCAS(&g_pair_status, 0, PAIR_ERR_ACCUM);
                    }
                    ok = false;
                    break;
                }
                tc::fence_after_sync();
                const uint32_t acc = tmem_base + (uint32_t)(b * PAIR_MAX_BN);
                for (int kb = wk.kb0; kb < wk.kb1; ++kb, ++idx) {
                    const int s = (int)(idx % PAIR_STAGES);
                    const uint32_t ph = (uint32_t)((idx / PAIR_STAGES) & 1);
                    if (*abort_flag) { ok = false; break; }
                    if (!tc::mbar_wait(&full[s], ph)) {             // both CTAs' halves of the stage have landed
                        *abort_flag = 1;
                        atomicCAS(&g_pair_status, 0, PAIR_ERR_FULL);
                        ok = false;
                        break;
                    }
                    tc::fence_after_sync();
                    const uint64_t wd = tc::smem_desc_k_major_sw128(w_tiles + s * PAIR_W_BYTES);
                    const uint64_t ad = tc::smem_desc_k_major_sw128(a_tiles + s * PAIR_A_BYTES);
#pragma unroll
                    for (int k = 0; k < PAIR_TILE_K / 16; ++k)
                        tc::mma_bf16_pair(acc, wd + 2 * k, ad + 2 * k, idesc, (kb > wk.kb0 || k > 0) ? 1u : 0u);
                    tc::mma_commit_pair(&empty[s]);              // the stage is free in both CTAs
                }
                if (ok) tc::mma_commit_pair(&acc_full[b]);       // both epilogues may read their halves
            }
        }
    } else {
        // epilogue: warp q reads lanes 32q..32q+31 = weight rows n0 + 32q + lane of this CTA's half
        const int q = warp & 3;
        const int row = q * 32 + lane;
        const int et = threadIdx.x - 64;
        ap_pdl_wait();          // `out` may still be read by an earlier kernel
        bool ok = true;
        int j = 0;
        const uint32_t remote_empty0 = tc::map_to_rank(tc::smem_addr(&acc_empty[0]), 0u);
        int it = 0;
        PairWork wk;
        for (; ok && pair_next(it, pair, pairs_in_grid, tiles_total, nkb, split, shared, wk); ++j) {
            const int tile = wk.tile;
            const int n0 = (tile / tiles_m) * 2 * PAIR_TILE_W + n_rank, m0 = (tile % tiles_m) * bn;
            const int b = j & 1;
            // tcgen05.ld is warp-wide: the whole warp goes on, or none of it
            if (!__all_sync(0xffffffffu, !*abort_flag && tc::mbar_wait(&acc_full[b], (uint32_t)((j >> 1) & 1)))) {
                if (!*abort_flag) {
                    *abort_flag = 1;
                    atomicCAS(&g_pair_status, 0, PAIR_ERR_ACCUM);
                }
                ok = false;
                break;
            }
            tc::fence_after_sync();
            const uint32_t acc = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(b * PAIR_MAX_BN);
            const int n = n0 + row;
            const int cols = min(bn, M - m0);           // token rows of this tile that exist
            if (wk.range > 0) {
                // a later range of a shared tile: this CTA's 128 rows of the partial sums go to global
                // memory, [token][weight row], for the CTA of the same rank in the pair of range 0
                float* mine = partials + (size_t)blockIdx.x * PAIR_PARTIAL_FLOATS;
#pragma unroll 1
                for (int c = 0; c < cols; c += 32) {
                    uint32_t v[32];
                    tc::tmem_ld_x32(acc + (uint32_t)c, v);
                    tc::tmem_ld_wait();
#pragma unroll
                    for (int jj = 0; jj < 32; ++jj) mine[(size_t)(c + jj) * PAIR_TILE_W + row] = __uint_as_float(v[jj]);
                }
                __threadfence();
                tc::fence_before_sync();
                pair_epilogue_sync();
                if (et == 0) {
                    pair_st_release(&flags[blockIdx.x], 1);
                    if (rank == 0) tc::mbar_arrive(&acc_empty[b]);
                    else tc::mbar_arrive_remote(remote_empty0 + (uint32_t)b * 8u);
                }
                continue;
            }
            // Range 0 of a shared tile: the CTAs of the same rank in the pairs pair + shared, pair + 2 shared,
            // ... hold the rest of K.  Their sums come through the operand ring, which is idle (this is
            // the pair's last piece of work and its products are done): blocks of 32 tokens (16 KB a peer)
            // arrive by bulk copy, two blocks in turn, and are added in the order of the ranges.
            const int peers = (wk.kb1 - wk.kb0 < nkb) ? split - 1 : 0;
            constexpr uint32_t XFER_BYTES = 32 * PAIR_TILE_W * 4;
            static_assert(2 * (PAIR_MAX_SPLIT - 1) * XFER_BYTES <= PAIR_STAGES * PAIR_STAGE_BYTES, "the ring holds the blocks");
            float* xbuf = reinterpret_cast<float*>(smem);
            auto peer_cta = [&](int pi) { return (int)blockIdx.x + 2 * (1 + pi) * shared; };
            auto fetch = [&](int block, int buf) {
                tc::mbar_expect_tx(&xfer[buf], (uint32_t)peers * XFER_BYTES);
                for (int pi = 0; pi < peers; ++pi)
                    tc::bulk_load(xbuf + (size_t)(buf * (PAIR_MAX_SPLIT - 1) + pi) * 32 * PAIR_TILE_W,
                                  partials + (size_t)peer_cta(pi) * PAIR_PARTIAL_FLOATS + (size_t)block * 32 * PAIR_TILE_W,
                                  XFER_BYTES, &xfer[buf]);
            };
            if (peers > 0) {
                if (et == 0) {
                    int fine = 1;
                    const long long t0 = clock64();
                    for (int pi = 0; pi < peers && fine; ++pi) {
                        while (pair_ld_acquire(&flags[peer_cta(pi)]) == 0) {
                            if (clock64() - t0 > 2000000000LL || *abort_flag) { fine = 0; break; }
                        }
                        if (fine) flags[peer_cta(pi)] = 0;            // ready for the next product
                    }
                    *peer_ok = fine;
                    if (fine) {
                        tc::fence_proxy_async();
                        fetch(0, 0);
                        if (cols > 32) fetch(1, 1);
                    }
                }
                pair_epilogue_sync();
                if (!*peer_ok) {
                    if (et == 0 && !*abort_flag) {
                        *abort_flag = 1;
                        atomicCAS(&g_pair_status, 0, PAIR_ERR_PEER);
                    }
                    ok = false;
                    break;
                }
            }
#pragma unroll 1
            for (int c = 0; c < cols; c += 32) {
                uint32_t v[32];
                tc::tmem_ld_x32(acc + (uint32_t)c, v);
                tc::tmem_ld_wait();
                if (peers > 0) {
                    const int block = c >> 5, buf = block & 1;
                    if (!__all_sync(0xffffffffu, tc::mbar_wait(&xfer[buf], (uint32_t)((block >> 1) & 1)))) {
                        if (!*abort_flag) {
                            *abort_flag = 1;
                            atomicCAS(&g_pair_status, 0, PAIR_ERR_PEER);
                        }
                        ok = false;
                        break;
                    }
                    for (int pi = 0; pi < peers; ++pi) {
                        const float* theirs = xbuf + (size_t)(buf * (PAIR_MAX_SPLIT - 1) + pi) * 32 * PAIR_TILE_W + row;
#pragma unroll
                        for (int jj = 0; jj < 32; ++jj)
                            v[jj] = __float_as_uint(__uint_as_float(v[jj]) + theirs[jj * PAIR_TILE_W]);
                    }
                    pair_epilogue_sync();                             // everybody has read this block
                    if (et == 0 && c + 64 < cols) fetch(block + 2, buf);
                }
                if (PAIRS) {
                    // even lane: gate of column n/2, odd lane: up.  The even lane finishes rows
                    // c..c+15, the odd lane rows c+16..c+31, each with the other's half.
                    const bool odd = lane & 1;
                    TO* dst = out + (size_t)(m0 + c + (odd ? 16 : 0)) * ldc + (n >> 1);
#pragma unroll
                    for (int jj = 0; jj < 16; ++jj) {
                        const uint32_t other = __shfl_xor_sync(0xffffffffu, odd ? v[jj] : v[16 + jj], 1);
                        // the gate and the up value pass through the storage type, as when the
                        // activation is a kernel of its own
                        const float gt = ap_to_float(ap_from_float<TO>(__uint_as_float(odd ? other : v[jj])));
                        const float up = ap_to_float(ap_from_float<TO>(__uint_as_float(odd ? v[16 + jj] : other)));
                        const int col = c + (odd ? 16 : 0) + jj;
                        if (col < cols && n < N)
                            dst[(size_t)jj * ldc] = ap_from_float<TO>(__fdividef(gt, 1.0f + __expf(-gt)) * up);
                    }
                } else if (n < N) {
#pragma unroll
                    for (int jj = 0; jj < 32; ++jj) {
                        if (c + jj < cols) out[(size_t)(m0 + c + jj) * ldc + n] = ap_from_float<TO>(__uint_as_float(v[jj]));
                    }
                }
            }
            // this CTA's half of the buffer has been read: one arrival on the first CTA's barrier
            tc::fence_before_sync();
            pair_epilogue_sync();
            if (et == 0) {
                if (rank == 0) tc::mbar_arrive(&acc_empty[b]);
                else tc::mbar_arrive_remote(remote_empty0 + (uint32_t)b * 8u);
            }
        }
    }
    tc::fence_before_sync();
    __syncthreads();
    ap_pdl_trigger();
    // neither CTA leaves while the other may still read its shared memory or signal its barriers
    tc::cluster_sync();
    if (warp == 1) {
        __syncwarp();
        tc::tmem_dealloc(tmem_base, PAIR_TMEM_COLS);
    }
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
typedef CUresult (*PairEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                 const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                 CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static PairEncodeFn pair_encode_fn() {
    static PairEncodeFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (PairEncodeFn)p;
    }
    return fn;
}

// rows x K bf16 matrix with leading dimension ld (elements); box = box_rows x 64.
static bool pair_make_map(CUtensorMap* map, const void* base, long long rows, long long K, long long ld, int box_rows) {
    PairEncodeFn fn = pair_encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {PAIR_TILE_K, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

template <typename TO, bool PAIRS>
static int launch_pair(const CUtensorMap& mw, const CUtensorMap& ma, void* out, int M, int N, int K, long long ldc,
                       int bn, int tiles_m, void* scratch, long long scratch_bytes, cudaStream_t stream) {
    auto kern = gemm_tc_pair_kernel<TO, PAIRS>;
    static bool configured = false;
    static int sms = 0;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, PAIR_SMEM_BYTES);
        AP_REQUIRE(e == cudaSuccess, "gemm_tc_pair: cannot reserve %d bytes of shared memory: %s", PAIR_SMEM_BYTES,
                   cudaGetErrorString(e));
        int dev = 0;
        AP_REQUIRE(cudaGetDevice(&dev) == cudaSuccess &&
                       cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && sms > 1,
                   "gemm_tc_pair: cannot read the number of SMs");
        configured = true;
    }
    const long long tiles = (long long)tiles_m * ((N + 2 * PAIR_TILE_W - 1) / (2 * PAIR_TILE_W));
    AP_REQUIRE(tiles < (1LL << 30), "gemm_tc_pair: too many output tiles");
    cudaLaunchConfig_t cfg = {};
    cfg.blockDim = dim3(192);
    cfg.dynamicSmemBytes = PAIR_SMEM_BYTES;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 2;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = 1;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    // The tiles are dealt out statically, so every pair of the grid must run at once: as many
    // pairs as the GPU holds side by side (a pair lies inside one GPC; a GPC with an odd number
    // of SMs leaves one without a partner).
    static int resident_pairs = 0;
    if (resident_pairs == 0) {
        cfg.gridDim = dim3((unsigned)(sms / 2 * 2), 1, 1);
        cfg.numAttrs = 1;
        int n = 0;
        cudaError_t e = cudaOccupancyMaxActiveClusters(&n, kern, &cfg);
        AP_REQUIRE(e == cudaSuccess && n > 0, "gemm_tc_pair: cannot find out how many pairs of CTAs run at once: %s",
                   cudaGetErrorString(e));
        resident_pairs = n < sms / 2 ? n : sms / 2;
    }
    int pairs = (int)((long long)resident_pairs < tiles ? resident_pairs : tiles);
    // Fewer tiles than half the pairs, a scratch buffer at hand and a K of 6144 and more: every tile is
    // shared by up to four pairs that take equal ranges of K (at least 24 blocks of it).  (Sharing out
    // the tiles left over after whole rounds in the same way was measured too: the 8B gate+up
    // product at 1024 to 4096 rows gains nothing from it, so whole rounds stay as they are.)
    const int nkb = (K + PAIR_TILE_K - 1) / PAIR_TILE_K;
    const int rounds = (int)(tiles / resident_pairs), left = (int)(tiles - (long long)rounds * resident_pairs);
    int split = 1, shared = 0;
    int* flags = nullptr;
    float* partials = nullptr;
    if (scratch && rounds == 0 && left * 2 <= resident_pairs && nkb >= 96) {
        split = min(PAIR_MAX_SPLIT, resident_pairs / left);
        split = min(split, nkb / 24);
        const long long need = (long long)PAIR_MAX_CTAS * 4 + 2LL * resident_pairs * PAIR_PARTIAL_FLOATS * 4;
        if (split < 2 || scratch_bytes < need || 2 * resident_pairs > PAIR_MAX_CTAS) split = 1;
    }
    if (split > 1) {
        AP_REQUIRE(((uintptr_t)scratch & 15) == 0, "gemm_tc_pair: the scratch buffer must be 16-byte aligned");
        flags = (int*)scratch;
        partials = (float*)((char*)scratch + PAIR_MAX_CTAS * 4);
        shared = left;
        if (rounds == 0) pairs = left * split;
    }
    cfg.gridDim = dim3((unsigned)(2 * pairs), 1, 1);
    cfg.numAttrs = ap_pdl_enabled() ? 2 : 1;
    AP_CHECK_PDL_LAUNCH("gemm_tc_pair", cudaLaunchKernelEx(&cfg, kern, mw, ma, (TO*)out, M, N, K, ldc, tiles_m,
                                                           (int)tiles, bn, split, shared, flags, partials));
    return AP_OK;
}

// The product on pairs of SMs (see gemm_tc_pair_kernel), for products with many rows.
//   pairs == 0: out[M, N] = a * w^T for w [N, K].
//   pairs != 0: w [N, K] has gate and up rows alternating; out[M, N/2] = silu(gate) * up.
//   scratch: null, or a zeroed buffer of ap_gemm_tc_pair_scratch_bytes() bytes that belongs to one
//   stream (few tiles of a long K are then shared among several pairs; the kernel leaves the flags
//   at its head zero again).  The persistent kernel's scratch buffer serves both.
AP_EXPORT long long ap_gemm_tc_pair_scratch_bytes(void) {
    return (long long)PAIR_MAX_CTAS * 4 + (long long)PAIR_MAX_CTAS * PAIR_PARTIAL_FLOATS * 4;
}
AP_EXPORT int ap_gemm_tc_pair(const void* a, const void* w, void* out, int out_dtype, int M, int N, int K,
                              long long lda, long long ldw, long long ldc, int pairs, void* scratch,
                              long long scratch_bytes, cudaStream_t stream) {
    AP_REQUIRE(M >= 0 && N > 0 && K > 0, "gemm_tc_pair: bad sizes M=%d N=%d K=%d", M, N, K);
    if (M == 0) return AP_OK;
    AP_REQUIRE(K % 8 == 0 && lda % 8 == 0 && ldw % 8 == 0,
               "gemm_tc_pair: K=%d and the leading dimensions must be multiples of 8 (16-byte rows for TMA)", K);
    AP_REQUIRE(((uintptr_t)a & 15) == 0 && ((uintptr_t)w & 15) == 0, "gemm_tc_pair: operands must be 16-byte aligned");
    AP_REQUIRE(!pairs || N % 2 == 0, "gemm_tc_pair: gate and up rows alternate, so the weight has an even number of rows");
    AP_REQUIRE(lda >= K && ldw >= K && ldc >= (pairs ? N / 2 : N), "gemm_tc_pair: a leading dimension is below its row length");
    AP_REQUIRE(out_dtype == AP_F32 || out_dtype == AP_BF16, "gemm_tc_pair: unknown output dtype %d", out_dtype);
    // token tiles of at most 256 rows, evenly filled; a tile's width is a multiple of 32 (each CTA
    // of the pair brings half of it, in whole groups of 16 rows)
    const int tiles_m = (M + PAIR_MAX_BN - 1) / PAIR_MAX_BN;
    const int bn = ((M + tiles_m - 1) / tiles_m + 31) / 32 * 32;
    CUtensorMap mw, ma;
    AP_REQUIRE(pair_make_map(&mw, w, N, K, ldw, PAIR_TILE_W), "gemm_tc_pair: cannot encode the weight's tensor map");
    AP_REQUIRE(pair_make_map(&ma, a, M, K, lda, bn / 2), "gemm_tc_pair: cannot encode the activations' tensor map");
    if (pairs) {
        return out_dtype == AP_F32
                   ? launch_pair<float, true>(mw, ma, out, M, N, K, ldc, bn, tiles_m, scratch, scratch_bytes, stream)
                   : launch_pair<bf16, true>(mw, ma, out, M, N, K, ldc, bn, tiles_m, scratch, scratch_bytes, stream);
    }
    return out_dtype == AP_F32
               ? launch_pair<float, false>(mw, ma, out, M, N, K, ldc, bn, tiles_m, scratch, scratch_bytes, stream)
               : launch_pair<bf16, false>(mw, ma, out, M, N, K, ldc, bn, tiles_m, scratch, scratch_bytes, stream);
}

// Whether this kernel is the one to use for a product of many rows.  Measured against the
// persistent kernel (one SM to a tile of 128 x 256, which takes in 48 KB per block of K where a
// CTA of a pair takes 32 KB) it is 3 to 12 % faster from 129 rows on, with two exceptions: products for which the kernel with two
// weight tiles to a CTA is chosen (2048 x 4096 x 14336: 173 against 184 us), and few tiles of a short K.
AP_EXPORT int ap_gemm_tc_prefers_pair(int M, int N, int K) {
    if (M <= 128 || N <= 0 || K <= 0 || K % 8) return 0;               // (160 x 28672 x 4096: 59 against 62 us)
    const int nkb = (K + PAIR_TILE_K - 1) / PAIR_TILE_K;
    {
        // the two-tile kernel's case: a long K and few enough of its waves (see ap_gemm_tc_prefers_persistent;
        // its other case, a badly filled last round of single tiles, is this kernel's: 2048 x 4096 x 4096
        // 56 us against 59)
        const long long rows = (M + PAIR_MAX_BN - 1) / PAIR_MAX_BN;
        const long long single = (long long)((N + PAIR_TILE_W - 1) / PAIR_TILE_W) * rows;
        const long long dual = (long long)((N + 2 * PAIR_TILE_W - 1) / (2 * PAIR_TILE_W)) * rows;
        if (K >= 8192 && ((dual + 147) / 148) * 180 < ((single + 147) / 148) * 100) return 0;
    }
    // fewer tiles of 256 x 256 than keep about half of the 74 pairs busy: with a long K they are shared
    // among several pairs (512 x 4096 x 14336: 61 us against the persistent kernel's 76, 544 x 2048 x
    // 8192: 35 against 46); with a short K one SM to a tile of 128 x 256 puts as many SMs to work
    // and is the faster (256 x 6144 x 4096: 28.4 against 30.6 us, 512 x 4096 x 4096: 30.7 against 34.7)
    const long long pair_tiles = (long long)((N + 2 * PAIR_TILE_W - 1) / (2 * PAIR_TILE_W)) * ((M + PAIR_MAX_BN - 1) / PAIR_MAX_BN);
    if (pair_tiles < 40) return (M > 256 && pair_tiles * 2 <= 74 && nkb >= 96) ? 1 : 0;
    return 1;
}

// 0 when every product on pairs of SMs so far ran to its end; else the code of the wait that
// expired (1 free stage, 2 operands, 3 accumulator, 4 the two CTAs' tensor memory differs).
AP_EXPORT int ap_gemm_tc_pair_status(void) {
    int v = -1;
    if (cudaMemcpyFromSymbol(&v, g_pair_status, sizeof(int)) != cudaSuccess) return -1;
    return v;
}

// Clear the status word so that products run again after a reported expiry.
AP_EXPORT int ap_gemm_tc_pair_reset_status(void) {
    const int zero = 0;
    return cudaMemcpyToSymbol(g_pair_status, &zero, sizeof(int)) == cudaSuccess ? AP_OK : AP_ERR_LAUNCH;
}
