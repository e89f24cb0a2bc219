// bfloat16 matrix product on the 5th-generation tensor cores:
//     out[M, N] = A[M, K] * W[N, K]^T        (activations times an [out, in] weight)
//
// The weight is the M side of the instruction: one CTA owns 128 weight rows (128 lanes
// of tensor memory) and BN rows of A (BN accumulator columns, BN in 16..256).  So a
// decode step with a handful of rows streams each weight tile once through a 128 x 16
// instruction, and a prompt portion uses 128 x 256.  Operands arrive by TMA into a ring
// of shared-memory stages (128-byte swizzle, K-major), one thread issues tcgen05.mma,
// the accumulator lives in tensor memory and four warps read it back with tcgen05.ld
// and write C transposed (lane = output feature, so a warp stores contiguous features).
// For few rows the K range is split over gridDim.z CTAs that write 32-bit partial sums
// [z, M, N]; consumers add them in order, which keeps results reproducible.
//
// Warps: 0 = TMA producer, 1 = tensor-memory owner and MMA issuer, 2..5 = epilogue.
// Every barrier wait has a time limit; on expiry the CTA raises a status word, lets its
// loads land, frees its tensor memory and returns.
//
// Reference counterpart: gemm_nt_kernel (cuda/src/kernels.cu:431-459), one thread per
// output element.
#include "common.cuh"
#include "tcgen05.cuh"

#define TILE_W 128          // weight rows per CTA (instruction M)
#define TILE_K 64           // bf16 elements per 128-byte swizzled row
#define A_TILE_BYTES (TILE_W * TILE_K * 2)

#define TC_ERR_EMPTY_WAIT 1
#define TC_ERR_FULL_WAIT 2
#define TC_ERR_ACCUM_WAIT 3

static __device__ int g_tc_status;

template <int BN, bool CLUSTER = false> struct TileCfg {
    static constexpr int kBBytes = BN * TILE_K * 2;
    static constexpr int kStageBytes = A_TILE_BYTES + kBBytes;
    static constexpr int kTmemCols = BN < 32 ? 32 : BN;
    static constexpr int kBarrierBytes = 256 + 1024;      // barriers, then the scale of each token column
    // cluster reduction buffer: [slices][BN][rows per slice], at most 136 rows in all
    static constexpr int kReduceBytes = (TILE_W + 8) * BN * 4;
    // 128 tokens and more: the reduction buffer lies over the stages, which are idle by then
    static constexpr bool kReduceOverStages = BN >= 128;
    static constexpr int kFixedBytes = 1024 /*alignment*/ + kBarrierBytes + ((CLUSTER && !kReduceOverStages) ? kReduceBytes : 0);
    // Up to 128 tokens: as many stages as let two CTAs share an SM (227 KB, 1 KB of each CTA the
    // system's), so that the CTAs of the next product can load their weights beside this one's.
    // One stage fewer or more than that costs 3 to 25 % of a decode step.
    static constexpr int kHalfSm = 232448 / 2 - 1024;
    static constexpr int kStages = BN >= 256 ? 4 : (kHalfSm - kFixedBytes) / kStageBytes;
    static constexpr int kSmemBytes = kStages * kStageBytes + 1024 + kBarrierBytes;
    static constexpr int kSmemBytesCluster = kSmemBytes + (kReduceOverStages ? 0 : kReduceBytes);
    static_assert(kStages >= 3 && kStages <= 8, "stage count out of range");
    static_assert(!kReduceOverStages || kReduceBytes <= kStages * kStageBytes, "the reduction buffer must fit the stages");
};

// What the epilogue does with the finished sums.
//   EPI_PLAIN     out[m, n] = sum                                  (32-bit or bfloat16 out)
//   EPI_PAIRS     the weight's rows alternate gate, up, gate, up ...; the sums of row 2i and 2i+1
//                 become out[m, i] = silu(gate) * up (out is [M, N/2]), so that the gated
//                 activation of a decode step needs no kernel of its own
//   EPI_RESIDUAL  out is the 32-bit residual stream: out[m, n] += sum; the updated value also goes
//                 to xb[m, n] in bfloat16 (the next product's input), and partial sums of squares
//                 of the updated rows go to ss_out[m, part] (every part is written, none added to)
//   EPI_ROPE      the weight is [W_q; W_k; W_v] of an attention layer: the sums of every pair of
//                 neighbouring rows of the Q and K heads are rotated by the row's position (the
//                 table of cosines and sines) and Q goes to q_out, K and V into the cache page and
//                 slot of the row's position.  pairing 0: the rows of each Q and K head were
//                 interleaved beforehand so that rows 2j and 2j+1 hold elements j and j + hd/2,
//                 and the results go back to their places; pairing 1: neighbouring elements pair
// PLAIN and PAIRS can scale token column m by 1/sqrt(mean square + eps) of the product's input
// row m, given as partial sums of squares (ss_in): an RMSNorm whose weight was multiplied into
// this product's weight beforehand then needs no kernel of its own either.
#define EPI_PLAIN 0
#define EPI_PAIRS 1
#define EPI_RESIDUAL 2
#define EPI_ROPE 3

struct EpiArgs {
    const float* ss_in;      // [M][ss_in_parts] or nullptr: no scale
    int ss_in_parts;
    float inv_width;         // 1 / (elements of an input row that the squares were summed over)
    float eps;
    bf16* xb;                // EPI_RESIDUAL: [M][ldxb]
    long long ldxb;
    float* ss_out;           // EPI_RESIDUAL: [M][ss_out_parts]
    int ss_out_parts;
    // EPI_ROPE
    bf16* q_out;             // [M][nh * hd]
    bf16* cache;             // one layer's pages [page][2][nkv][P][hd], or nullptr: store no K, V
    const int* positions;    // [M]
    const int* token_seq;    // [M] row of the block table
    const int* block_table;  // [.][max_blocks]
    const float2* cos_sin;   // [M][hd/2] (cos, sin), or nullptr: no rotation
    long long page_stride;
    int max_blocks, nh, nkv, hd, P, pairing;
};

// One pair of neighbouring rows (n even, n + 1) of the stacked Q, K, V projection for token m:
// a and b are the finished sums in the storage type's precision.
__device__ __forceinline__ void rope_store_pair(const EpiArgs& ea, int m, int n, float a, float b) {
    const int hd = ea.hd, half = hd >> 1;
    const int head = n / hd, r = n - head * hd, j = r >> 1;
    int ia = r, ib = r + 1;
    if (head < ea.nh + ea.nkv) {
        if (ea.pairing == 0) { ia = j; ib = j + half; }
        if (ea.cos_sin) {
            const float2 cs = ea.cos_sin[(size_t)m * half + j];
            const float ra = a * cs.x - b * cs.y, rb = a * cs.y + b * cs.x;
            a = ra;
            b = rb;
        }
    }
    bf16* dst;
    if (head < ea.nh) {
        dst = ea.q_out + (size_t)m * ea.nh * hd + (size_t)head * hd;
    } else {
        if (ea.cache == nullptr) return;
        const int pos = ea.positions[m];
        const int page = ea.block_table[(size_t)ea.token_seq[m] * ea.max_blocks + pos / ea.P];
        if (page < 0) return;
        const int kvh = head - ea.nh;                       // K heads, then V heads: the page's planes in order
        dst = ea.cache + (size_t)page * ea.page_stride + ((size_t)kvh * ea.P + pos % ea.P) * hd;
    }
    dst[ia] = __float2bfloat16_rn(a);
    dst[ib] = __float2bfloat16_rn(b);
}

__device__ __forceinline__ float gated(float gate, float up) { return __fdividef(gate, 1.0f + __expf(-gate)) * up; }
// the four epilogue warps among themselves (barrier 1; barrier 0 is __syncthreads)
__device__ __forceinline__ void epilogue_sync() { asm volatile("bar.sync 1, 128;" ::: "memory"); }

// CLUSTER: the gridDim.z K-slices of one output tile form a thread-block cluster and add
// their partial tiles through distributed shared memory, each CTA finishing a band of the
// 128 weight rows; `out` is then the finished matrix.  Otherwise slice z writes its
// partial sums to out + z * split_stride (EPI_PLAIN only).
template <int BN, typename TO, bool CLUSTER, int EPI = EPI_PLAIN>
__global__ void __launch_bounds__(192)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_a,
               TO* __restrict__ out, int M, int N, int K, long long ldc, int kb_per_split,
               long long split_stride, const EpiArgs ea) {
    using Cfg = TileCfg<BN, CLUSTER>;
    constexpr int STAGES = Cfg::kStages;
    constexpr bool PAIRS = EPI == EPI_PAIRS;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* w_tiles = smem;
    uint8_t* a_tiles = smem + STAGES * A_TILE_BYTES;
    uint64_t* full = (uint64_t*)(smem + STAGES * Cfg::kStageBytes);
    uint64_t* empty = full + STAGES;
    uint64_t* accum = empty + STAGES;
    uint32_t* tmem_slot = (uint32_t*)(accum + 1);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
    float* inv_s = (float*)(smem + STAGES * Cfg::kStageBytes + 256);      // [BN] scale of each token column
    // CLUSTER with 128 tokens or more: the buffer the slices' partial sums are gathered in lies
    // over the operand stages, and a cluster barrier makes sure every CTA is done with them
    constexpr bool REUSE = CLUSTER && Cfg::kReduceOverStages;
    float* reduce = REUSE ? (float*)smem : (float*)(smem + STAGES * Cfg::kStageBytes + Cfg::kBarrierBytes);
    bool have_acc = false;          // epilogue threads: the accumulator is complete and may be read
    float xin_first[16];            // epilogue threads, EPI_RESIDUAL in a cluster: see below

    // once a wait has expired anywhere, later CTAs do nothing: the product is void anyway.
    // (In a cluster every CTA still walks to the cluster barrier, or its peers would wait.)
    const bool skip = *(volatile int*)&g_tc_status != 0;
    if (!CLUSTER && skip) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    // blockIdx.x walks the row tiles: CTAs that share a weight tile run side by side, so the
    // weight comes from HBM once and from L2 for the others
    const int n0 = blockIdx.y * TILE_W;
    const int m0 = blockIdx.x * BN;
    const int kb_total = (K + TILE_K - 1) / TILE_K;
    const int kb0 = blockIdx.z * kb_per_split;
    const int kb1 = min(kb_total, kb0 + kb_per_split);
    const int nkb = skip ? 0 : max(0, kb1 - kb0);
    if (!CLUSTER) out += (size_t)blockIdx.z * split_stride;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            tc::mbar_init(&full[s], 1);
            tc::mbar_init(&empty[s], 1);
        }
        tc::mbar_init(accum, 1);
        *abort_flag = 0;
        tc::fence_barrier_init();
        tc::prefetch_tensormap(&tmap_w);
        tc::prefetch_tensormap(&tmap_a);
    }
    if (warp == 1) tc::tmem_alloc(tmem_slot, Cfg::kTmemCols);
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;
    // A grid that fits the GPU in one wave lets the next kernel start at once (it will only
    // prefetch until this one is done); a larger grid keeps the SMs to itself until its end.
    const bool one_wave = gridDim.x * gridDim.y * gridDim.z <= 2 * 148;
    if (one_wave) ap_pdl_trigger();

    if (warp == 0) {
        if (lane == 0) {
            // The weight does not depend on earlier kernels: fill the ring with weight tiles
            // first, then wait for the kernels that produce the activations.
            const int pre = min(nkb, STAGES);
            for (int i = 0; i < pre; ++i) {
                tc::mbar_expect_tx(&full[i], Cfg::kStageBytes);
                tc::tma_load_2d(w_tiles + i * A_TILE_BYTES, &tmap_w, (kb0 + i) * TILE_K, n0, &full[i]);
            }
            ap_pdl_wait();
            for (int i = 0; i < pre; ++i)
                tc::tma_load_2d(a_tiles + i * Cfg::kBBytes, &tmap_a, (kb0 + i) * TILE_K, m0, &full[i]);
            int issued = pre;
            for (int i = pre; i < nkb; ++i) {
                const int s = i % STAGES;
                const uint32_t ph = (i / STAGES) & 1;
                if (*abort_flag) break;
                if (!tc::mbar_wait(&empty[s], ph ^ 1)) {
                    *abort_flag = 1;
                    atomicExch(&g_tc_status, TC_ERR_EMPTY_WAIT);
                    break;
                }
                tc::mbar_expect_tx(&full[s], Cfg::kStageBytes);
                tc::tma_load_2d(w_tiles + s * A_TILE_BYTES, &tmap_w, (kb0 + i) * TILE_K, n0, &full[s]);
                tc::tma_load_2d(a_tiles + s * Cfg::kBBytes, &tmap_a, (kb0 + i) * TILE_K, m0, &full[s]);
                issued = i + 1;
            }
            if (*abort_flag) {
                // let the loads that are still in flight land before the CTA's memory goes away
                for (int i = max(0, issued - STAGES); i < issued; ++i)
                    tc::mbar_wait(&full[i % STAGES], (i / STAGES) & 1, 200000000LL);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = tc::instr_desc_bf16_f32(TILE_W, BN);
            bool ok = true;
            for (int i = 0; i < nkb; ++i) {
                const int s = i % STAGES;
                const uint32_t ph = (i / STAGES) & 1;
                if (*abort_flag) { ok = false; break; }
                if (!tc::mbar_wait(&full[s], ph)) {
                    *abort_flag = 1;
                    atomicExch(&g_tc_status, TC_ERR_FULL_WAIT);
                    ok = false;
                    break;
                }
                tc::fence_after_sync();
                const uint64_t wd = tc::smem_desc_k_major_sw128(w_tiles + s * A_TILE_BYTES);
                const uint64_t ad = tc::smem_desc_k_major_sw128(a_tiles + s * Cfg::kBBytes);
#pragma unroll
                for (int k = 0; k < TILE_K / 16; ++k) {
                    // 16 bf16 = 32 bytes further along the swizzled row: +2 in 16-byte units
                    tc::mma_bf16(tmem_base, wd + 2 * k, ad + 2 * k, idesc, (i > 0 || k > 0) ? 1u : 0u);
                }
                tc::mma_commit(&empty[s]);          // the stage is free once these MMAs are done
            }
            if (ok && nkb > 0) tc::mma_commit(accum);
        }
    } else {
        // epilogue: warp q reads lanes 32q..32q+31 = weight rows n0 + 32q + lane
        const int q = warp & 3;
        const int row = q * 32 + lane;
        const int n = n0 + row;
        const int et = (int)threadIdx.x - 64;
        ap_pdl_wait();          // `out` may still be read by an earlier kernel
        if (CLUSTER && EPI == EPI_RESIDUAL && !skip) {
            // The residual's old values at the first sixteen places this thread will finish
            // (nobody else writes the residual while this product runs): fetched now, long before
            // the sums are complete, so that their latency is not paid at the end.
            const int S = gridDim.z;
            const int band = (TILE_W + S - 1) / S;
            const int first = blockIdx.z * band;
            const int rows = max(1, min(band, TILE_W - first));
            const int total = rows * min(BN, M - m0);
#pragma unroll
            for (int u = 0; u < 16; ++u) {
                const int idx = u * 128 + et;
                const int c = idx / rows, i = idx - c * rows;
                xin_first[u] = (idx < total && n0 + first + i < N)
                                   ? reinterpret_cast<float*>(out)[(size_t)(m0 + c) * ldc + n0 + first + i] : 0.f;
            }
        }
        // the scale of every token column of this tile, from the partial sums of squares of the
        // product's input rows (1 where there is no deferred norm): 128 / BN threads share a
        // token's parts (each every TPT-th one) and add their sums up by butterfly
        {
            constexpr int TPT = BN >= 128 ? 1 : 128 / BN;               // threads per token: 1, 2, 4 or 8
            for (int c0 = 0; c0 < BN; c0 += 128 / TPT) {
                const int c = c0 + et / TPT, sub = et % TPT;
                float ss = 0.f;
                const bool live = ea.ss_in != nullptr && m0 + c < M;
                if (live) {
                    const float* p = ea.ss_in + (size_t)(m0 + c) * ea.ss_in_parts;
                    for (int i = sub; i < ea.ss_in_parts; i += TPT) ss += p[i];
                }
#pragma unroll
                for (int o = TPT >> 1; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
                if (sub == 0) inv_s[c] = live ? 1.0f / sqrtf(ss * ea.inv_width + ea.eps) : 1.0f;
            }
        }
        epilogue_sync();
        bool have = nkb > 0;
        if (have) {
            if (!tc::mbar_wait(accum, 0)) {
                if (!*abort_flag) {
                    *abort_flag = 1;
                    atomicExch(&g_tc_status, TC_ERR_ACCUM_WAIT);
                }
                have = false;
            }
            tc::fence_after_sync();
        }
        have_acc = have;
        if (REUSE) {
            // the hand-over follows below, once no CTA of the cluster reads its stages any more
        } else if (CLUSTER) {
            // hand this row's partial sums to the CTA that finishes its band of rows
            const int S = gridDim.z;
            const int band = (TILE_W + S - 1) / S;
            const int dest = row / band, slot = row - dest * band;
            const uint32_t base = tc::map_to_rank(tc::smem_addr(reduce), (uint32_t)dest) +
                                  (uint32_t)((blockIdx.z * BN) * band + slot) * 4u;
#pragma unroll 1
            for (int c = 0; c < BN; c += 16) {
                uint32_t v[16];
                if (have) {
                    tc::tmem_ld_x16(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)c, v);
                    tc::tmem_ld_wait();
                } else {
#pragma unroll
                    for (int j = 0; j < 16; ++j) v[j] = 0u;
                }
#pragma unroll
                for (int j = 0; j < 16; ++j)
                    tc::st_cluster_f32(base + (uint32_t)((c + j) * band) * 4u, __uint_as_float(v[j]));
            }
        } else if (__all_sync(0xffffffffu, have)) {
#pragma unroll 1
            for (int c = 0; c < BN; c += 16) {
                if (m0 + c >= M) break;
                uint32_t v[16];
                tc::tmem_ld_x16(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)c, v);
                tc::tmem_ld_wait();
                if (PAIRS) {
                    // even lane: gate of column n/2, odd lane: up.  The even lane finishes rows
                    // c..c+7, the odd lane rows c+8..c+15, each with the other's half; both values
                    // pass through the storage type, as when the activation is a kernel of its own.
                    const bool odd = lane & 1;
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const uint32_t other = __shfl_xor_sync(0xffffffffu, odd ? v[j] : v[8 + j], 1);
                        const int col = c + (odd ? 8 : 0) + j;
                        const float sc = inv_s[col];
                        const float gt = ap_to_float(ap_from_float<TO>(__uint_as_float(odd ? other : v[j]) * sc));
                        const float up = ap_to_float(ap_from_float<TO>(__uint_as_float(odd ? v[8 + j] : other) * sc));
                        const int m = m0 + col;
                        if (m < M && n < N) out[(size_t)m * ldc + (n >> 1)] = ap_from_float<TO>(gated(gt, up));
                    }
                } else if (EPI == EPI_ROPE) {
                    // even lane: row n, odd lane: row n + 1 of a pair; the even lane finishes token
                    // columns c..c+7, the odd lane c+8..c+15, each with the other's half
                    const bool odd = lane & 1;
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        const uint32_t other = __shfl_xor_sync(0xffffffffu, odd ? v[j] : v[8 + j], 1);
                        const int col = c + (odd ? 8 : 0) + j;
                        const float sc = inv_s[col];
                        const float a = ap_to_float(__float2bfloat16_rn(__uint_as_float(odd ? other : v[j]) * sc));
                        const float b = ap_to_float(__float2bfloat16_rn(__uint_as_float(odd ? v[8 + j] : other) * sc));
                        const int m = m0 + col;
                        if (m < M && n < N) rope_store_pair(ea, m, n & ~1, a, b);
                    }
                } else if (EPI == EPI_RESIDUAL) {
                    // lane = weight row n: add into the residual, keep its bfloat16 copy, and sum the
                    // squares of this warp's 32 rows for every token (lanes by butterfly: a fixed order)
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int m = m0 + c + j;
                        float xv = 0.f;
                        if (m < M && n < N) {
                            float* px = reinterpret_cast<float*>(out) + (size_t)m * ldc + n;
                            xv = *px + __uint_as_float(v[j]);
                            *px = xv;
                            ea.xb[(size_t)m * ea.ldxb + n] = __float2bfloat16_rn(xv);
                        }
                        const float sq = ap_warp_sum(xv * xv);
                        if (lane == 0 && m < M) ea.ss_out[(size_t)m * ea.ss_out_parts + blockIdx.y * 4 + q] = sq;
                    }
                } else if (n < N) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int m = m0 + c + j;
                        if (m < M) out[(size_t)m * ldc + n] = ap_from_float<TO>(__uint_as_float(v[j]) * inv_s[c + j]);
                    }
                }
            }
        } else if (nkb == 0 && EPI != EPI_RESIDUAL && EPI != EPI_ROPE && n < N && (!PAIRS || !(lane & 1))) {
            for (int c = 0; c < BN; ++c) {
                const int m = m0 + c;
                if (m < M) out[(size_t)m * ldc + (PAIRS ? n >> 1 : n)] = ap_from_float<TO>(0.f);
            }
        }
    }
    if (REUSE) {
        // The epilogue warps come here after the last MMA of this CTA has finished, that is,
        // after every load into its stages has been consumed: once all threads of the cluster
        // have arrived, every CTA's stages are free to receive partial sums.
        __syncwarp();
        tc::cluster_arrive();
        tc::cluster_wait();
        if (warp >= 2) {
            const int q = warp & 3;
            const int row = q * 32 + lane;
            const int S = gridDim.z;
            const int band = (TILE_W + S - 1) / S;
            const int dest = row / band, slot = row - dest * band;
            const uint32_t base = tc::map_to_rank(tc::smem_addr(reduce), (uint32_t)dest) +
                                  (uint32_t)((blockIdx.z * BN) * band + slot) * 4u;
            const int mcols = min(BN, M - m0);
#pragma unroll 1
            for (int c = 0; c < mcols; c += 16) {
                uint32_t v[16];
                if (have_acc) {
                    tc::tmem_ld_x16(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)c, v);
                    tc::tmem_ld_wait();
                } else {
#pragma unroll
                    for (int j = 0; j < 16; ++j) v[j] = 0u;
                }
#pragma unroll
                for (int j = 0; j < 16; ++j)
                    tc::st_cluster_f32(base + (uint32_t)((c + j) * band) * 4u, __uint_as_float(v[j]));
            }
        }
    }
    if (CLUSTER) {
        const int S = gridDim.z;
        const int band = (TILE_W + S - 1) / S;
        const int first = blockIdx.z * band;
        const int rows = max(0, min(band, TILE_W - first));
        const int e = (int)threadIdx.x - 64;              // the four epilogue warps add the band
        __syncwarp();
        tc::cluster_sync();                 // every slice has delivered its partial sums
        if (e >= 0 && !skip) {
            const int mcols = min(BN, M - m0);
            if (PAIRS) {
                // a band starts at an even row and has an even number of rows: pairs stay together
                const int prs = rows / 2;
                for (int idx = e; idx < prs * mcols; idx += 128) {
                    const int c = idx / prs, i = idx - c * prs;
                    float gt = 0.f, up = 0.f;
                    for (int s = 0; s < S; ++s) {                                          // slices in order
                        gt += reduce[(s * BN + c) * band + 2 * i];
                        up += reduce[(s * BN + c) * band + 2 * i + 1];
                    }
                    gt = ap_to_float(ap_from_float<TO>(gt * inv_s[c]));
                    up = ap_to_float(ap_from_float<TO>(up * inv_s[c]));
                    const int n = n0 + first + 2 * i;
                    if (n < N) out[(size_t)(m0 + c) * ldc + (n >> 1)] = ap_from_float<TO>(gated(gt, up));
                }
            } else if (EPI == EPI_ROPE) {
                const int prs = rows / 2;
                for (int idx = e; idx < prs * mcols; idx += 128) {
                    const int c = idx / prs, i = idx - c * prs;
                    float a = 0.f, b = 0.f;
                    for (int s = 0; s < S; ++s) {                                          // slices in order
                        a += reduce[(s * BN + c) * band + 2 * i];
                        b += reduce[(s * BN + c) * band + 2 * i + 1];
                    }
                    a = ap_to_float(__float2bfloat16_rn(a * inv_s[c]));
                    b = ap_to_float(__float2bfloat16_rn(b * inv_s[c]));
                    const int n = n0 + first + 2 * i;
                    if (n < N) rope_store_pair(ea, m0 + c, n, a, b);
                }
            } else if (EPI == EPI_RESIDUAL) {
                // Thread idx owns (token c, row i) of the band.  The squares of a token's rows are
                // summed over runs of min(rows, 32) lanes, which hold consecutive rows of one token
                // (rows is a power of two: 128 over 2, 4 or 8 slices), and every run writes one part.
                // The residual's old values are fetched sixteen at a time, the first sixteen before
                // the cluster barrier above (xin_first), so that their latency is not paid here.
                const int total = rows * mcols;
                const int width = rows < 32 ? rows : 32;
                const int groups = rows < 32 ? 1 : rows / 32;
                for (int base = 0; base < total; base += 128 * 16) {        // the same trips for every lane
                    float xin[16];
#pragma unroll
                    for (int u = 0; u < 16; ++u) {
                        const int idx = base + u * 128 + e;
                        const int c = idx / rows, i = idx - c * rows;
                        xin[u] = base == 0 ? xin_first[u]
                                           : ((idx < total && n0 + first + i < N)
                                                  ? reinterpret_cast<float*>(out)[(size_t)(m0 + c) * ldc + n0 + first + i] : 0.f);
                    }
#pragma unroll
                    for (int u = 0; u < 16; ++u) {
                        if (base + u * 128 >= total) break;                 // uniform
                        const int idx = base + u * 128 + e;
                        const bool valid = idx < total;
                        const int c = valid ? idx / rows : 0, i = valid ? idx - c * rows : 0;
                        const int n = n0 + first + i;
                        float xv = 0.f;
                        if (valid && n < N) {
                            float sum = 0.f;
                            for (int s = 0; s < S; ++s) sum += reduce[(s * BN + c) * band + i];   // slices in order
                            xv = xin[u] + sum;
                            reinterpret_cast<float*>(out)[(size_t)(m0 + c) * ldc + n] = xv;
                            ea.xb[(size_t)(m0 + c) * ea.ldxb + n] = __float2bfloat16_rn(xv);
                        }
                        float sq = xv * xv;
                        for (int o = width >> 1; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
                        if (valid && (lane & (width - 1)) == 0)
                            ea.ss_out[(size_t)(m0 + c) * ea.ss_out_parts +
                                      ((size_t)blockIdx.y * S + blockIdx.z) * groups + (i >> 5)] = sq;
                    }
                }
            } else {
                for (int idx = e; idx < rows * mcols; idx += 128) {
                    const int c = idx / rows, i = idx - c * rows;
                    float sum = 0.f;
                    for (int s = 0; s < S; ++s) sum += reduce[(s * BN + c) * band + i];   // slices in order
                    const int n = n0 + first + i;
                    if (n < N) out[(size_t)(m0 + c) * ldc + n] = ap_from_float<TO>(sum * inv_s[c]);
                }
            }
        }
    }
    tc::fence_before_sync();
    __syncthreads();
    if (!one_wave) ap_pdl_trigger();
    if (warp == 1) {
        __syncwarp();
        tc::tmem_dealloc(tmem_base, Cfg::kTmemCols);
    }
}

// ---------------------------------------------------------------------------
// Two weight tiles per CTA against the same activation tile: a 256 x BN output tile from
// two accumulators (2 * BN tensor-memory columns).  Every activation tile that reaches
// shared memory now feeds twice the FLOPs, which matters once many rows are in flight and
// the product is bound by what L2 can deliver to the SMs.  The second weight tile starts
// `w1_offset` (128) rows after the first.
// ---------------------------------------------------------------------------
template <int BN> struct DualCfg {
    static constexpr int kStages = BN >= 256 ? 3 : 4;
    static constexpr int kBBytes = BN * TILE_K * 2;
    static constexpr int kStageBytes = 2 * A_TILE_BYTES + kBBytes;
    static constexpr int kTmemCols = 2 * BN;
    static constexpr int kSmemBytes = kStages * kStageBytes + 1024 + 256;
};

template <int BN, typename TO>
__global__ void __launch_bounds__(192)
gemm_tc_dual_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_a,
                    TO* __restrict__ out, int M, int N, int K, long long ldc, int w1_offset) {
    using Cfg = DualCfg<BN>;
    constexpr int STAGES = Cfg::kStages;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* w_tiles = smem;                                   // [stage][2][128 x 64]
    uint8_t* a_tiles = smem + STAGES * 2 * A_TILE_BYTES;
    uint64_t* full = (uint64_t*)(smem + STAGES * Cfg::kStageBytes);
    uint64_t* empty = full + STAGES;
    uint64_t* accum = empty + STAGES;
    uint32_t* tmem_slot = (uint32_t*)(accum + 1);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

    if (*(volatile int*)&g_tc_status != 0) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.y * 2 * TILE_W;        // tile y covers 256 weight rows
    const int m0 = blockIdx.x * BN;            // row tiles side by side: they share the weight tiles
    const int nkb = (K + TILE_K - 1) / TILE_K;

    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            tc::mbar_init(&full[s], 1);
            tc::mbar_init(&empty[s], 1);
        }
        tc::mbar_init(accum, 1);
        *abort_flag = 0;
        tc::fence_barrier_init();
        tc::prefetch_tensormap(&tmap_w);
        tc::prefetch_tensormap(&tmap_a);
    }
    if (warp == 1) tc::tmem_alloc(tmem_slot, Cfg::kTmemCols);
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            ap_pdl_wait();
            int issued = 0;
            for (int i = 0; i < nkb; ++i) {
                const int s = i % STAGES;
                const uint32_t ph = (i / STAGES) & 1;
                if (*abort_flag) break;
                if (!tc::mbar_wait(&empty[s], ph ^ 1)) {
                    *abort_flag = 1;
                    atomicExch(&g_tc_status, TC_ERR_EMPTY_WAIT);
                    break;
                }
                tc::mbar_expect_tx(&full[s], Cfg::kStageBytes);
                tc::tma_load_2d(w_tiles + (2 * s) * A_TILE_BYTES, &tmap_w, i * TILE_K, n0, &full[s]);
                tc::tma_load_2d(w_tiles + (2 * s + 1) * A_TILE_BYTES, &tmap_w, i * TILE_K, n0 + w1_offset, &full[s]);
                tc::tma_load_2d(a_tiles + s * Cfg::kBBytes, &tmap_a, i * TILE_K, m0, &full[s]);
                issued = i + 1;
            }
            if (*abort_flag) {
                for (int i = max(0, issued - STAGES); i < issued; ++i)
                    tc::mbar_wait(&full[i % STAGES], (i / STAGES) & 1, 200000000LL);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = tc::instr_desc_bf16_f32(TILE_W, BN);
            bool ok = true;
            for (int i = 0; i < nkb; ++i) {
                const int s = i % STAGES;
                const uint32_t ph = (i / STAGES) & 1;
                if (*abort_flag) { ok = false; break; }
                if (!tc::mbar_wait(&full[s], ph)) {
                    *abort_flag = 1;
                    atomicExch(&g_tc_status, TC_ERR_FULL_WAIT);
                    ok = false;
                    break;
                }
                tc::fence_after_sync();
                const uint64_t w0 = tc::smem_desc_k_major_sw128(w_tiles + (2 * s) * A_TILE_BYTES);
                const uint64_t w1 = tc::smem_desc_k_major_sw128(w_tiles + (2 * s + 1) * A_TILE_BYTES);
                const uint64_t ad = tc::smem_desc_k_major_sw128(a_tiles + s * Cfg::kBBytes);
#pragma unroll
                for (int k = 0; k < TILE_K / 16; ++k) {
                    const uint32_t acc = (i > 0 || k > 0) ? 1u : 0u;
                    tc::mma_bf16(tmem_base, w0 + 2 * k, ad + 2 * k, idesc, acc);
                    tc::mma_bf16(tmem_base + BN, w1 + 2 * k, ad + 2 * k, idesc, acc);
                }
                tc::mma_commit(&empty[s]);
            }
            if (ok) tc::mma_commit(accum);
        }
    } else {
        const int q = warp & 3;
        const int row = q * 32 + lane;
        ap_pdl_wait();
        bool have = true;
        if (!tc::mbar_wait(accum, 0)) {
            if (!*abort_flag) {
                *abort_flag = 1;
                atomicExch(&g_tc_status, TC_ERR_ACCUM_WAIT);
            }
            have = false;
        }
        tc::fence_after_sync();
        if (have) {
            const uint32_t lane_base = tmem_base + ((uint32_t)(q * 32) << 16);
#pragma unroll 1
            for (int c = 0; c < BN; c += 16) {
                if (m0 + c >= M) break;
                uint32_t v0[16], v1[16];
                tc::tmem_ld_x16(lane_base + (uint32_t)c, v0);
                tc::tmem_ld_x16(lane_base + (uint32_t)(BN + c), v1);
                tc::tmem_ld_wait();
                {
                    const int na = n0 + row, nb = n0 + w1_offset + row;
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int m = m0 + c + j;
                        if (m >= M) break;
                        if (na < N) out[(size_t)m * ldc + na] = ap_from_float<TO>(__uint_as_float(v0[j]));
                        if (nb < N) out[(size_t)m * ldc + nb] = ap_from_float<TO>(__uint_as_float(v1[j]));
                    }
                }
            }
        }
    }
    tc::fence_before_sync();
    __syncthreads();
    ap_pdl_trigger();
    if (warp == 1) {
        __syncwarp();
        tc::tmem_dealloc(tmem_base, Cfg::kTmemCols);
    }
}

// ---------------------------------------------------------------------------
// host side
// ---------------------------------------------------------------------------
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                  const cuuint64_t*, const cuuint32_t*, const cuuint32_t*,
                                  CUtensorMapInterleave, CUtensorMapSwizzle, CUtensorMapL2promotion,
                                  CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    if (!fn) {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (EncodeTiledFn)p;
    }
    return fn;
}

// rows x K bf16 matrix with leading dimension ld (elements); box = box_rows x 64.
static bool make_map(CUtensorMap* map, const void* base, long long rows, long long K, long long ld, int box_rows) {
    EncodeTiledFn fn = encode_fn();
    if (!fn) return false;
    cuuint64_t dims[2] = {(cuuint64_t)K, (cuuint64_t)rows};
    cuuint64_t strides[1] = {(cuuint64_t)ld * 2};
    cuuint32_t box[2] = {TILE_K, (cuuint32_t)box_rows};
    cuuint32_t estr[2] = {1, 1};
    return fn(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
              CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
              CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS;
}

static int pick_bn(int M) { return M <= 16 ? 16 : M <= 32 ? 32 : M <= 64 ? 64 : M <= 128 ? 128 : 256; }

// How many K slices the kernel wants for this shape (1: none).  Few rows leave too few
// weight tiles to keep every SM loading, so K is split until about two CTAs per SM exist
// (at most 8: the slices of a tile form one thread-block cluster that adds them up).
AP_EXPORT int ap_gemm_tc_plan(int M, int N, int K) {
    if (M <= 0 || N <= 0 || K <= 0) return 1;
    const int kb_total = (K + TILE_K - 1) / TILE_K;
    const int bn = pick_bn(M);
    const long long tiles = (long long)((N + TILE_W - 1) / TILE_W) * ((M + bn - 1) / bn);
    const bool wide = bn > 128;             // a tile of 256 tokens fills an SM; narrower ones go two to an SM
    if (M > 256 || tiles >= (wide ? 148 : 288)) return 1;
    // as many slices as keep the whole grid resident at once, with a little slack so that the
    // clusters find room side by side.  Measured inside the decode step and alone, 8 to 128
    // rows: the 8B QKV weight (48 tiles) wants 4 slices, O and down (32 tiles) 8, at every row count.
    int ns = (int)((wide ? 148 : 288) / tiles);
    ns = min(ns, wide ? kb_total / 8 : kb_total / 4);
    ns = min(ns, 8);                       // one thread-block cluster adds the slices
    if (ns < 1) ns = 1;
    while (ns & (ns - 1)) ns &= ns - 1;    // clusters of 2, 4 or 8 CTAs find room side by side; odd sizes do not
    if (wide && ns < 4) return 1;          // two slices of a wide tile cost more to add than they save
    const int per = (kb_total + ns - 1) / ns;
    return (kb_total + per - 1) / per;
}

template <int BN, typename TO, bool CLUSTER, int EPI = EPI_PLAIN>
static int launch_tc(const CUtensorMap& mw, const CUtensorMap& ma, void* out, int M, int N, int K,
                     long long ldc, int nsplit, long long split_stride, const EpiArgs& ea, cudaStream_t stream) {
    using Cfg = TileCfg<BN, CLUSTER>;
    auto kern = gemm_tc_kernel<BN, TO, CLUSTER, EPI>;
    constexpr int smem = CLUSTER ? Cfg::kSmemBytesCluster : Cfg::kSmemBytes;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
        AP_REQUIRE(e == cudaSuccess, "gemm_tc: cannot reserve %d bytes of shared memory: %s", smem,
                   cudaGetErrorString(e));
        configured = true;
    }
    const int kb_total = (K + TILE_K - 1) / TILE_K;
    const int per = (kb_total + nsplit - 1) / nsplit;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3((M + BN - 1) / BN, (N + TILE_W - 1) / TILE_W, nsplit);
    cfg.blockDim = dim3(192);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[2];
    int nattr = 0;
    if (CLUSTER) {
        attr[nattr].id = cudaLaunchAttributeClusterDimension;
        attr[nattr].val.clusterDim.x = 1;
        attr[nattr].val.clusterDim.y = 1;
        attr[nattr].val.clusterDim.z = nsplit;
        ++nattr;
    }
    if (ap_pdl_enabled()) {
        attr[nattr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[nattr].val.programmaticStreamSerializationAllowed = 1;
        ++nattr;
    }
    cfg.attrs = attr;
    cfg.numAttrs = nattr;
    cudaError_t e = cudaLaunchKernelEx(&cfg, kern, mw, ma, (TO*)out, M, N, K, ldc, per, split_stride, ea);
    if (e != cudaSuccess) {
        ap_set_error("gemm_tc: launch failed: %s", cudaGetErrorString(e));
        return AP_ERR_LAUNCH;
    }
    return AP_OK;
}

#define AP_MAX_CLUSTER 8

// Parts of the sums of squares that ap_gemm_tc writes per row with epi == 2 (see there).
AP_EXPORT int ap_gemm_tc_residual_parts(int N, int nsplit) {
    const int tiles = (N + TILE_W - 1) / TILE_W;
    if (nsplit <= 1) return tiles * 4;
    const int band = (TILE_W + nsplit - 1) / nsplit;
    return tiles * nsplit * (band < 32 ? 1 : band / 32);
}

static int gemm_tc_run(const void* a, const void* w, void* out, int out_dtype, int M, int N, int K,
                       long long lda, long long ldw, long long ldc, int nsplit, long long split_stride,
                       int reduce, int epi, const float* ss_in, int ss_in_parts, float inv_width, float eps,
                       void* xb, long long ldxb, float* ss_out, int ss_out_parts, const EpiArgs* rope,
                       cudaStream_t stream);

// reduce != 0: the K slices add up inside a thread-block cluster and `out` is the finished
// matrix (nsplit <= 8, M <= 256); else slice z writes 32-bit partial sums at out + z * split_stride.
// epi: what becomes of the finished sums (nsplit == 1, or reduce):
//   0  out[M, N] = sums, 32-bit or bfloat16;
//   1  w's rows alternate gate and up, out[M, N/2] = silu(gate) * up (bfloat16, M <= 256);
//   2  out is the 32-bit residual [M, N] and is added to; xb [M, ldxb] receives its bfloat16
//      copy and ss_out [M, ap_gemm_tc_residual_parts(N, nsplit)] partial sums of squares of the
//      updated rows (nsplit 1, 2, 4 or 8; one tile of rows: M <= 256).
// ss_in (epi 0 and 1; nullptr: none): [M, ss_in_parts] partial sums of squares of the rows of
// the product's input before they were rounded to `a`; row m of the result is multiplied by
// 1/sqrt(sum(ss_in[m]) * inv_width + eps).
AP_EXPORT int ap_gemm_tc(const void* a, const void* w, void* out, int out_dtype, int M, int N, int K,
                         long long lda, long long ldw, long long ldc, int nsplit, long long split_stride,
                         int reduce, int epi, const float* ss_in, int ss_in_parts, float inv_width, float eps,
                         void* xb, long long ldxb, float* ss_out, int ss_out_parts, cudaStream_t stream) {
    AP_REQUIRE(M >= 0 && N > 0 && K > 0, "gemm_tc: bad sizes M=%d N=%d K=%d", M, N, K);
    if (M == 0) return AP_OK;
    AP_REQUIRE(K % 8 == 0 && lda % 8 == 0 && ldw % 8 == 0,
               "gemm_tc: K=%d and the leading dimensions must be multiples of 8 (16-byte rows for TMA)", K);
    AP_REQUIRE(((uintptr_t)a & 15) == 0 && ((uintptr_t)w & 15) == 0, "gemm_tc: operands must be 16-byte aligned");
    AP_REQUIRE(epi == EPI_PLAIN || epi == EPI_PAIRS || epi == EPI_RESIDUAL, "gemm_tc: unknown epilogue %d", epi);
    return gemm_tc_run(a, w, out, out_dtype, M, N, K, lda, ldw, ldc, nsplit, split_stride, reduce, epi, ss_in,
                       ss_in_parts, inv_width, eps, xb, ldxb, ss_out, ss_out_parts, nullptr, stream);
}

static int gemm_tc_run(const void* a, const void* w, void* out, int out_dtype, int M, int N, int K,
                       long long lda, long long ldw, long long ldc, int nsplit, long long split_stride,
                       int reduce, int epi, const float* ss_in, int ss_in_parts, float inv_width, float eps,
                       void* xb, long long ldxb, float* ss_out, int ss_out_parts, const EpiArgs* rope,
                       cudaStream_t stream) {
    const bool pairs = epi == EPI_PAIRS;
    AP_REQUIRE(lda >= K && ldw >= K && ldc >= (pairs ? N / 2 : N), "gemm_tc: a leading dimension is below its row length");
    const int kb_total = (K + TILE_K - 1) / TILE_K;
    AP_REQUIRE(nsplit >= 1 && nsplit <= kb_total && nsplit <= 65535, "gemm_tc: cannot split K=%d into %d", K, nsplit);
    AP_REQUIRE(!pairs || (N % 2 == 0 && M <= 256 && out_dtype == AP_BF16 && (nsplit == 1 || reduce)),
               "gemm_tc: the gated epilogue takes an even number of weight rows, at most 256 rows of a, "
               "bfloat16 output and finished sums");
    AP_REQUIRE((long long)(nsplit - 1) * ((kb_total + nsplit - 1) / nsplit) < kb_total,
               "gemm_tc: %d slices leave an empty one for K=%d", nsplit, K);
    AP_REQUIRE(out_dtype == AP_F32 || out_dtype == AP_BF16, "gemm_tc: unknown output dtype %d", out_dtype);
    const int bn = pick_bn(M);
    AP_REQUIRE((N + TILE_W - 1) / TILE_W <= 65535, "gemm_tc: %d output features exceed the grid", N);
    const bool cluster = reduce != 0 && nsplit > 1;
    AP_REQUIRE(!cluster || (nsplit <= AP_MAX_CLUSTER && M <= 256),
               "gemm_tc: slices are added in a cluster only for up to %d slices and 256 rows (got %d, %d)",
               AP_MAX_CLUSTER, nsplit, M);
    AP_REQUIRE(cluster || nsplit == 1 || out_dtype == AP_F32, "gemm_tc: partial sums must be 32-bit");
    AP_REQUIRE(ss_in == nullptr || ((nsplit == 1 || cluster) && ss_in_parts > 0 && inv_width > 0.f && epi != EPI_RESIDUAL),
               "gemm_tc: the scale of the rows applies to finished sums, and needs its parts and the rows' width");
    EpiArgs ea = {};
    if (rope) ea = *rope;
    ea.ss_in = ss_in; ea.ss_in_parts = ss_in_parts; ea.inv_width = inv_width; ea.eps = eps;
    if (epi == EPI_RESIDUAL) {
        AP_REQUIRE(out_dtype == AP_F32 && M <= 256 && (nsplit == 1 || (cluster && (nsplit == 2 || nsplit == 4 || nsplit == 8))),
                   "gemm_tc: the residual epilogue adds into a 32-bit matrix of at most 256 rows, with 1, 2, 4 or 8 "
                   "slices of K added in a cluster");
        AP_REQUIRE(xb && ss_out && ldxb >= N && ss_out_parts == ap_gemm_tc_residual_parts(N, nsplit),
                   "gemm_tc: the residual epilogue needs the bfloat16 copy and %d parts of sums of squares per row",
                   ap_gemm_tc_residual_parts(N, nsplit));
        ea.xb = (bf16*)xb; ea.ldxb = ldxb; ea.ss_out = ss_out; ea.ss_out_parts = ss_out_parts;
    }
    CUtensorMap mw, ma;
    AP_REQUIRE(make_map(&mw, w, N, K, ldw, TILE_W), "gemm_tc: cannot encode the weight's tensor map");
    AP_REQUIRE(make_map(&ma, a, M, K, lda, bn), "gemm_tc: cannot encode the activations' tensor map");
#define GO(BN, CL)                                                                                       \
    return out_dtype == AP_F32                                                                           \
               ? launch_tc<BN, float, CL>(mw, ma, out, M, N, K, ldc, nsplit, split_stride, ea, stream)   \
               : launch_tc<BN, bf16, CL>(mw, ma, out, M, N, K, ldc, nsplit, split_stride, ea, stream)
#define GOE(BN, CL, TT, EP) return launch_tc<BN, TT, CL, EP>(mw, ma, out, M, N, K, ldc, nsplit, split_stride, ea, stream)
#define BY_BN(MACRO, ...)                      \
    switch (bn) {                              \
        case 16: MACRO(16, __VA_ARGS__);       \
        case 32: MACRO(32, __VA_ARGS__);       \
        case 64: MACRO(64, __VA_ARGS__);       \
        case 128: MACRO(128, __VA_ARGS__);     \
        default: MACRO(256, __VA_ARGS__);      \
    }
    if (epi == EPI_PAIRS) {
        if (cluster) BY_BN(GOE, true, bf16, EPI_PAIRS)
        BY_BN(GOE, false, bf16, EPI_PAIRS)
    }
    if (epi == EPI_RESIDUAL) {
        if (cluster) BY_BN(GOE, true, float, EPI_RESIDUAL)
        BY_BN(GOE, false, float, EPI_RESIDUAL)
    }
    if (epi == EPI_ROPE) {
        if (cluster) BY_BN(GOE, true, bf16, EPI_ROPE)
        BY_BN(GOE, false, bf16, EPI_ROPE)
    }
    if (cluster) BY_BN(GO, true)
    BY_BN(GO, false)
#undef BY_BN
#undef GOE
#undef GO
}

// The stacked Q, K, V projection of an attention layer for at most 256 rows, with the rotation
// of Q and K and the store of K and V into the cache in its epilogue (EPI_ROPE): w is
// [(nh + 2 nkv) * hd, K]; q_out [M, nh * hd] bfloat16; cache one layer's pages
// [page][2][nkv][P][hd] bfloat16 (nullptr: K and V are not stored); cos_sin [M][hd/2] pairs
// (nullptr: no rotation); pairing 0: the rows of every Q and K head interleaved (2j: element j,
// 2j + 1: element j + hd/2), 1: neighbouring elements pair.  ss_in as for ap_gemm_tc.
AP_EXPORT int ap_gemm_tc_rope(const void* a, const void* w, int M, int K, long long lda, long long ldw, int nsplit,
                              const float* ss_in, int ss_in_parts, float inv_width, float eps, void* q_out,
                              void* cache, const int* positions, const int* token_seq, const int* block_table,
                              int max_blocks, const float* cos_sin, int pairing, int nh, int nkv, int hd, int P,
                              long long page_stride, cudaStream_t stream) {
    AP_REQUIRE(nh > 0 && nkv >= 0 && hd > 0 && hd % 2 == 0, "gemm_tc_rope: bad heads %d/%d of size %d", nh, nkv, hd);
    AP_REQUIRE(pairing == 0 || pairing == 1, "gemm_tc_rope: unknown pairing %d", pairing);
    AP_REQUIRE(q_out && positions, "gemm_tc_rope: the queries' destination and the positions are needed");
    AP_REQUIRE(cache == nullptr || (token_seq && block_table && max_blocks > 0 && P > 0 &&
                                    page_stride >= 2LL * nkv * P * hd),
               "gemm_tc_rope: storing needs the block table, the rows' sequences and whole pages");
    AP_REQUIRE(M <= 256, "gemm_tc_rope: at most 256 rows (got %d)", M);
    EpiArgs ea = {};
    ea.q_out = (bf16*)q_out; ea.cache = (bf16*)cache; ea.positions = positions; ea.token_seq = token_seq;
    ea.block_table = block_table; ea.cos_sin = (const float2*)cos_sin; ea.page_stride = page_stride;
    ea.max_blocks = max_blocks; ea.nh = nh; ea.nkv = nkv; ea.hd = hd; ea.P = P; ea.pairing = pairing;
    const int N = (nh + 2 * nkv) * hd;
    return gemm_tc_run(a, w, q_out, AP_BF16, M, N, K, lda, ldw, N, nsplit, 0, nsplit > 1 ? 1 : 0, EPI_ROPE, ss_in,
                       ss_in_parts, inv_width, eps, nullptr, 0, nullptr, 0, &ea, stream);
}

template <int BN, typename TO>
static int launch_dual(const CUtensorMap& mw, const CUtensorMap& ma, void* out, int M, int N, int K,
                       long long ldc, cudaStream_t stream) {
    using Cfg = DualCfg<BN>;
    auto kern = gemm_tc_dual_kernel<BN, TO>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
        AP_REQUIRE(e == cudaSuccess, "gemm_tc: cannot reserve %d bytes of shared memory: %s", Cfg::kSmemBytes,
                   cudaGetErrorString(e));
        configured = true;
    }
    dim3 grid((M + BN - 1) / BN, (N + 2 * TILE_W - 1) / (2 * TILE_W), 1);
    AP_CHECK_PDL_LAUNCH("gemm_tc_dual", ap_launch_pdl(kern, grid, dim3(192), (size_t)Cfg::kSmemBytes, stream, mw, ma,
                                                      (TO*)out, M, N, K, ldc, TILE_W));
    return AP_OK;
}

// Two weight tiles per CTA (see gemm_tc_dual_kernel), for products with more than 64 rows:
// out[M, N] = a * w^T for w [N, K].
AP_EXPORT int ap_gemm_tc_dual(const void* a, const void* w, void* out, int out_dtype, int M, int N, int K,
                              long long lda, long long ldw, long long ldc, cudaStream_t stream) {
    AP_REQUIRE(M >= 0 && N > 0 && K > 0, "gemm_tc: bad sizes M=%d N=%d K=%d", M, N, K);
    if (M == 0) return AP_OK;
    AP_REQUIRE(K % 8 == 0 && lda % 8 == 0 && ldw % 8 == 0,
               "gemm_tc: K=%d and the leading dimensions must be multiples of 8 (16-byte rows for TMA)", K);
    AP_REQUIRE(((uintptr_t)a & 15) == 0 && ((uintptr_t)w & 15) == 0, "gemm_tc: operands must be 16-byte aligned");
    AP_REQUIRE(lda >= K && ldw >= K && ldc >= N, "gemm_tc: a leading dimension is below its row length");
    AP_REQUIRE(out_dtype == AP_F32 || out_dtype == AP_BF16, "gemm_tc: unknown output dtype %d", out_dtype);
    const int bn = M <= 128 ? 128 : 256;
    AP_REQUIRE((N + TILE_W - 1) / TILE_W <= 65535, "gemm_tc: %d output features exceed the grid", N);
    CUtensorMap mw, ma;
    AP_REQUIRE(make_map(&mw, w, N, K, ldw, TILE_W), "gemm_tc: cannot encode the weight's tensor map");
    AP_REQUIRE(make_map(&ma, a, M, K, lda, bn), "gemm_tc: cannot encode the activations' tensor map");
#define GO(BN)                                                                             \
    return out_dtype == AP_F32 ? launch_dual<BN, float>(mw, ma, out, M, N, K, ldc, stream) \
                               : launch_dual<BN, bf16>(mw, ma, out, M, N, K, ldc, stream)
    if (bn == 128) GO(128);
    GO(256);
#undef GO
}

// Whether two weight tiles per CTA beat one for this shape: a dual tile takes about 1.65
// times as long as a single one, and either kind runs in waves of one CTA per SM.
AP_EXPORT int ap_gemm_tc_prefers_dual(int M, int N, int K) {
    (void)K;
    if (M <= 128) return 0;
    const int bn = M <= 128 ? 128 : 256;
    const long long rows = (M + bn - 1) / bn;
    const long long single = ((N + TILE_W - 1) / TILE_W) * rows, dual = ((N + 2 * TILE_W - 1) / (2 * TILE_W)) * rows;
    const long long ws = (single + 147) / 148, wd = (dual + 147) / 148;
    return wd * 165 < ws * 100 ? 1 : 0;
}

// ---------------------------------------------------------------------------
// Many rows (prompt portions): a persistent kernel, one CTA per SM, over output tiles of 128
// weight rows x BN tokens, dealt out round robin (consecutive tiles differ in the token tile
// first, so the CTAs that run side by side share weight tiles through L2).
//
// Fewer tiles than half the SMs and a long K (a portion of a few hundred tokens against the
// down projection): every tile is shared by `split` CTAs, each taking an equal range of K.  CTA g works on tile
// g % tiles and range g / tiles, so the CTAs of one range run side by side as before.  The
// CTAs of ranges 1.. hand their partial sums over in a scratch buffer ([token][weight row],
// 32-bit) and raise a flag; the CTA of range 0, which has worked just as long, adds them in
// range order and writes the tile.  The flags are left zero for the next product.
//
// The accumulator is double-buffered in tensor memory (2 x BN columns), so the four epilogue
// warps read one segment out while the tensor cores are on the next; the operand ring keeps
// running across segments.
//
// PAIRS: the weight's rows alternate gate, up, gate, up ... (row 2i and 2i+1 belong to output
// column i).  Neighbouring lanes exchange their values by shuffle and the epilogue writes
// silu(gate) * up to out[M, N/2]: the gated activation never makes a round trip to memory.
// ---------------------------------------------------------------------------
#define TC_ERR_PEER_WAIT 5
#define PERSIST_MAX_CTAS 256                 // flags at the head of the scratch buffer

template <int BN> struct PersistCfg {
    static constexpr int kStages = BN >= 256 ? 4 : 6;
    static constexpr int kBBytes = BN * TILE_K * 2;
    static constexpr int kStageBytes = A_TILE_BYTES + kBBytes;
    static constexpr int kTmemCols = 2 * BN;
    static constexpr int kSmemBytes = kStages * kStageBytes + 1024 + 256;
    static constexpr long long kPartialFloats = (long long)TILE_W * BN;       // per CTA
};

// A CTA's next piece of work: blocks [kb0, kb1) of K of one output tile.
struct Segment { int tile, kb0, kb1; };

// The work of CTA g of G in the order it is done.  split == 1: whole tiles g, g + G, ...;
// split > 1 (G == tiles * split): range g / tiles of the K blocks of tile g % tiles.
struct WorkList {
    int next_tile, tiles, G, nkb, split, g;
    bool done;
    __device__ __forceinline__ WorkList(int tiles_, int nkb_, int G_, int g_, int split_)
        : next_tile(g_), tiles(tiles_), G(G_), nkb(nkb_), split(split_), g(g_), done(false) {}
    __device__ __forceinline__ bool next(Segment& s) {
        if (split > 1) {
            if (done || g >= tiles * split) return false;
            done = true;
            const int slice = g / tiles;
            s.tile = g - slice * tiles;
            s.kb0 = (int)((long long)nkb * slice / split);
            s.kb1 = (int)((long long)nkb * (slice + 1) / split);
            return s.kb1 > s.kb0;
        }
        if (next_tile >= tiles) return false;
        s.tile = next_tile;
        s.kb0 = 0;
        s.kb1 = nkb;
        next_tile += G;
        return true;
    }
};

__device__ __forceinline__ int ld_acquire_gpu(const int* p) {
    int v;
    asm volatile("ld.acquire.gpu.global.s32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_gpu(int* p, int v) {
    asm volatile("st.release.gpu.global.s32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
template <int BN, typename TO, bool PAIRS>
__global__ void __launch_bounds__(192)
gemm_tc_persistent_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_a,
                          TO* __restrict__ out, int M, int N, int K, long long ldc, int tiles_m, int tiles_total,
                          int bn, int split, int* __restrict__ flags, float* __restrict__ partials) {
    using Cfg = PersistCfg<BN>;
    constexpr int STAGES = Cfg::kStages;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* w_tiles = smem;
    uint8_t* a_tiles = smem + STAGES * A_TILE_BYTES;
    uint64_t* full = (uint64_t*)(smem + STAGES * Cfg::kStageBytes);
    uint64_t* empty = full + STAGES;
    uint64_t* acc_full = empty + STAGES;       // [accumulator buffer]
    uint64_t* acc_empty = acc_full + 2;        // [accumulator buffer]
    uint32_t* tmem_slot = (uint32_t*)(acc_empty + 2);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);
    volatile int* peer_ok = (volatile int*)(tmem_slot + 2);

    if (*(volatile int*)&g_tc_status != 0) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int nkb = (K + TILE_K - 1) / TILE_K;
    // A tile holds `bn` <= BN tokens (a multiple of 16 chosen by the host so that the tiles of
    // a product are evenly filled); shared memory and tensor memory are laid out for BN.
    const uint32_t stage_bytes = (uint32_t)(A_TILE_BYTES + bn * TILE_K * 2);
    const int G = gridDim.x, g = blockIdx.x;
    if (threadIdx.x == 0) {
        for (int s = 0; s < STAGES; ++s) {
            tc::mbar_init(&full[s], 1);
            tc::mbar_init(&empty[s], 1);
        }
        for (int b = 0; b < 2; ++b) {
            tc::mbar_init(&acc_full[b], 1);
            tc::mbar_init(&acc_empty[b], 128);
        }
        *abort_flag = 0;
        tc::fence_barrier_init();
        tc::prefetch_tensormap(&tmap_w);
        tc::prefetch_tensormap(&tmap_a);
    }
    if (warp == 1) tc::tmem_alloc(tmem_slot, Cfg::kTmemCols);
    tc::fence_before_sync();
    __syncthreads();
    tc::fence_after_sync();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            WorkList work(tiles_total, nkb, G, g, split);
            Segment sg;
            long long idx = 0, issued = 0;
            bool first = true;
            while (!*abort_flag && work.next(sg)) {
                const int n0 = (sg.tile / tiles_m) * TILE_W, m0 = (sg.tile % tiles_m) * bn;
                int kb = sg.kb0;
                if (first) {
                    // the weight does not depend on earlier kernels: fill the ring with this
                    // segment's first weight blocks, then wait for the kernels that produce
                    // the activations
                    first = false;
                    const int pre = min(STAGES, sg.kb1 - sg.kb0);
                    for (int i = 0; i < pre; ++i) {
                        tc::mbar_expect_tx(&full[i], stage_bytes);
                        tc::tma_load_2d(w_tiles + i * A_TILE_BYTES, &tmap_w, (kb + i) * TILE_K, n0, &full[i]);
                    }
                    ap_pdl_wait();
                    for (int i = 0; i < pre; ++i)
                        tc::tma_load_2d(a_tiles + i * Cfg::kBBytes, &tmap_a, (kb + i) * TILE_K, m0, &full[i]);
                    kb += pre;
                    idx = issued = pre;
                }
                for (; kb < sg.kb1; ++kb, ++idx) {
                    const int s = (int)(idx % STAGES);
                    const uint32_t ph = (uint32_t)((idx / STAGES) & 1);
                    if (*abort_flag) break;
                    if (!tc::mbar_wait(&empty[s], ph ^ 1)) {
                        *abort_flag = 1;
                        atomicExch(&g_tc_status, TC_ERR_EMPTY_WAIT);
                        break;
                    }
                    tc::mbar_expect_tx(&full[s], stage_bytes);
                    tc::tma_load_2d(w_tiles + s * A_TILE_BYTES, &tmap_w, kb * TILE_K, n0, &full[s]);
                    tc::tma_load_2d(a_tiles + s * Cfg::kBBytes, &tmap_a, kb * TILE_K, m0, &full[s]);
                    issued = idx + 1;
                }
            }
            if (*abort_flag) {
                // let the loads that are still in flight land before the CTA's memory goes away
                for (long long i = max(0LL, issued - STAGES); i < issued; ++i)
                    tc::mbar_wait(&full[i % STAGES], (uint32_t)((i / STAGES) & 1), 200000000LL);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            const uint32_t idesc = tc::instr_desc_bf16_f32(TILE_W, bn);
            bool ok = true;
            long long idx = 0;
            WorkList work(tiles_total, nkb, G, g, split);
            Segment sg;
            for (int j = 0; ok && work.next(sg); ++j) {
                const int b = j & 1;
                // the epilogue warps have read this buffer's segment of two rounds ago
                if (!tc::mbar_wait(&acc_empty[b], (uint32_t)(((j >> 1) & 1) ^ 1))) {
                    *abort_flag = 1;
                    atomicExch(&g_tc_status, TC_ERR_ACCUM_WAIT);
                    ok = false;
                    break;
                }
                tc::fence_after_sync();
                const uint32_t acc = tmem_base + (uint32_t)(b * BN);
                for (int kb = sg.kb0; kb < sg.kb1; ++kb, ++idx) {
                    const int s = (int)(idx % STAGES);
                    const uint32_t ph = (uint32_t)((idx / STAGES) & 1);
                    if (*abort_flag) { ok = false; break; }
                    if (!tc::mbar_wait(&full[s], ph)) {
                        *abort_flag = 1;
                        atomicExch(&g_tc_status, TC_ERR_FULL_WAIT);
                        ok = false;
                        break;
                    }
                    tc::fence_after_sync();
                    const uint64_t wd = tc::smem_desc_k_major_sw128(w_tiles + s * A_TILE_BYTES);
                    const uint64_t ad = tc::smem_desc_k_major_sw128(a_tiles + s * Cfg::kBBytes);
#pragma unroll
                    for (int k = 0; k < TILE_K / 16; ++k)
                        tc::mma_bf16(acc, wd + 2 * k, ad + 2 * k, idesc, (kb > sg.kb0 || k > 0) ? 1u : 0u);
                    tc::mma_commit(&empty[s]);
                }
                if (ok) tc::mma_commit(&acc_full[b]);
            }
        }
    } else {
        // epilogue: warp q reads lanes 32q..32q+31 = weight rows n0 + 32q + lane
        const int q = warp & 3;
        const int row = q * 32 + lane;
        const int et = threadIdx.x - 64;                 // 0..127 among the epilogue threads
        ap_pdl_wait();          // `out` may still be read by an earlier kernel
        bool ok = true;
        WorkList work(tiles_total, nkb, G, g, split);
        Segment sg;
        for (int j = 0; ok && work.next(sg); ++j) {
            const int n0 = (sg.tile / tiles_m) * TILE_W, m0 = (sg.tile % tiles_m) * bn;
            const int b = j & 1;
            // tcgen05.ld is warp-wide: the whole warp goes on, or none of it
            if (!__all_sync(0xffffffffu, tc::mbar_wait(&acc_full[b], (uint32_t)((j >> 1) & 1)))) {
                if (!*abort_flag) {
                    *abort_flag = 1;
                    atomicExch(&g_tc_status, TC_ERR_ACCUM_WAIT);
                }
                ok = false;
                break;
            }
            tc::fence_after_sync();
            const uint32_t acc = tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)(b * BN);
            const int n = n0 + row;
            const int cols = min(bn, M - m0);           // token rows of this tile that exist
            if (sg.kb0 > 0) {
                // not the tile's first block: hand the partial sums over, [token][weight row]
                float* mine = partials + (size_t)g * Cfg::kPartialFloats;
#pragma unroll 1
                for (int c = 0; c < cols; c += 32) {
                    uint32_t v[32];
                    tc::tmem_ld_x32(acc + (uint32_t)c, v);
                    tc::tmem_ld_wait();
#pragma unroll
                    for (int jj = 0; jj < 32; ++jj) mine[(size_t)(c + jj) * TILE_W + row] = __uint_as_float(v[jj]);
                }
                __threadfence();
                tc::fence_before_sync();
                tc::mbar_arrive(&acc_empty[b]);
                epilogue_sync();
                if (et == 0) st_release_gpu(&flags[g], 1);
                continue;
            }
            // the tile's first blocks are here: CTAs g + tiles, g + 2 tiles, ... hold the rest of its K
            int peers = 0;
            if (sg.kb1 < nkb) {
                peers = split - 1;
                if (et == 0) {
                    int fine = 1;
                    const long long t0 = clock64();
                    for (int pi = 0; pi < peers && fine; ++pi) {
                        while (ld_acquire_gpu(&flags[g + (1 + pi) * tiles_total]) == 0) {
                            if (clock64() - t0 > 2000000000LL || *abort_flag) { fine = 0; break; }
                        }
                        if (fine) flags[g + (1 + pi) * tiles_total] = 0;          // ready for the next product
                    }
                    *peer_ok = fine;
                }
                epilogue_sync();
                if (!*peer_ok) {
                    if (et == 0 && !*abort_flag) {
                        *abort_flag = 1;
                        atomicExch(&g_tc_status, TC_ERR_PEER_WAIT);
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
                for (int pi = 0; pi < peers; ++pi) {
                    const float* theirs = partials + (size_t)(g + (1 + pi) * tiles_total) * Cfg::kPartialFloats +
                                          (size_t)c * TILE_W + row;
#pragma unroll
                    for (int jj = 0; jj < 32; ++jj)
                        v[jj] = __float_as_uint(__uint_as_float(v[jj]) + __ldcg(theirs + (size_t)jj * TILE_W));
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
            tc::fence_before_sync();
            tc::mbar_arrive(&acc_empty[b]);
        }
    }
    tc::fence_before_sync();
    __syncthreads();
    ap_pdl_trigger();
    if (warp == 1) {
        __syncwarp();
        tc::tmem_dealloc(tmem_base, Cfg::kTmemCols);
    }
}

template <int BN, typename TO, bool PAIRS>
static int launch_persistent(const CUtensorMap& mw, const CUtensorMap& ma, void* out, int M, int N, int K,
                             long long ldc, int bn, void* scratch, long long scratch_bytes, cudaStream_t stream) {
    using Cfg = PersistCfg<BN>;
    auto kern = gemm_tc_persistent_kernel<BN, TO, PAIRS>;
    static bool configured = false;
    static int sms = 0;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
        AP_REQUIRE(e == cudaSuccess, "gemm_tc: cannot reserve %d bytes of shared memory: %s", Cfg::kSmemBytes,
                   cudaGetErrorString(e));
        int dev = 0;
        AP_REQUIRE(cudaGetDevice(&dev) == cudaSuccess &&
                       cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) == cudaSuccess && sms > 0,
                   "gemm_tc: cannot read the number of SMs");
        configured = true;
    }
    const int tiles_m = (M + bn - 1) / bn;
    const long long tiles = (long long)tiles_m * ((N + TILE_W - 1) / TILE_W);
    AP_REQUIRE(tiles < (1LL << 30), "gemm_tc: too many output tiles");
    // Fewer tiles than half the SMs, a scratch buffer at hand and enough K to share: `split`
    // CTAs per tile.  Else whole tiles, round robin.
    const int max_ctas = min(sms, PERSIST_MAX_CTAS);
    const int nkb = (K + TILE_K - 1) / TILE_K;
    int split = 1;
    if (scratch && tiles * 2 <= max_ctas) {
        split = (int)min((long long)8, (long long)max_ctas / tiles);
        // handing partial sums over costs about as much as fifty blocks of K: share a tile only
        // where every CTA keeps about that many
        split = min(split, nkb / 48);
        if (split < 1) split = 1;
        const long long need = (long long)PERSIST_MAX_CTAS * 4 + tiles * split * Cfg::kPartialFloats * 4;
        if (split > 1 && scratch_bytes < need) split = 1;
    }
    const int ctas = split > 1 ? (int)tiles * split : (int)min((long long)max_ctas, tiles);
    int* flags = nullptr;
    float* partials = nullptr;
    if (split > 1) {
        AP_REQUIRE(((uintptr_t)scratch & 15) == 0, "gemm_tc: the scratch buffer must be 16-byte aligned");
        flags = (int*)scratch;
        partials = (float*)((char*)scratch + PERSIST_MAX_CTAS * 4);
    }
    dim3 grid((unsigned)ctas, 1, 1);
    AP_CHECK_PDL_LAUNCH("gemm_tc_persistent", ap_launch_pdl(kern, grid, dim3(192), (size_t)Cfg::kSmemBytes, stream, mw,
                                                            ma, (TO*)out, M, N, K, ldc, tiles_m, (int)tiles, bn,
                                                            split, flags, partials));
    return AP_OK;
}

// Bytes of scratch with which ap_gemm_tc_persistent shares few tiles among all SMs.  The
// buffer must be zero when first used and belongs to one stream; the kernel leaves its head
// (the flags) zero again.
AP_EXPORT long long ap_gemm_tc_persistent_scratch_bytes(void) {
    return (long long)PERSIST_MAX_CTAS * 4 + (long long)PERSIST_MAX_CTAS * PersistCfg<256>::kPartialFloats * 4;
}

// The persistent kernel (see gemm_tc_persistent_kernel), for products with more than 64 rows.
//   pairs == 0: out[M, N] = a * w^T for w [N, K].
//   pairs != 0: w [N, K] has gate and up rows alternating; out[M, N/2] = silu(gate) * up.
//   scratch: null, or ap_gemm_tc_persistent_scratch_bytes() bytes (see there).
AP_EXPORT int ap_gemm_tc_persistent(const void* a, const void* w, void* out, int out_dtype, int M, int N, int K,
                                    long long lda, long long ldw, long long ldc, int pairs, void* scratch,
                                    long long scratch_bytes, cudaStream_t stream) {
    AP_REQUIRE(M >= 0 && N > 0 && K > 0, "gemm_tc: bad sizes M=%d N=%d K=%d", M, N, K);
    if (M == 0) return AP_OK;
    AP_REQUIRE(K % 8 == 0 && lda % 8 == 0 && ldw % 8 == 0,
               "gemm_tc: K=%d and the leading dimensions must be multiples of 8 (16-byte rows for TMA)", K);
    AP_REQUIRE(((uintptr_t)a & 15) == 0 && ((uintptr_t)w & 15) == 0, "gemm_tc: operands must be 16-byte aligned");
    AP_REQUIRE(!pairs || N % 2 == 0, "gemm_tc: gate and up rows alternate, so the weight has an even number of rows");
    AP_REQUIRE(lda >= K && ldw >= K && ldc >= (pairs ? N / 2 : N), "gemm_tc: a leading dimension is below its row length");
    AP_REQUIRE(out_dtype == AP_F32 || out_dtype == AP_BF16, "gemm_tc: unknown output dtype %d", out_dtype);
    // token tiles: as many as tiles of the full width (128 for up to 128 rows, else 256) would
    // take, but evenly filled: their width is the smallest multiple of 16 that covers the rows
    const int cap = M <= 128 ? 128 : 256;
    int tiles_m = (M + cap - 1) / cap;
    {
        // One or two token tiles more, where that fills the SMs better: a tile's time is about that of
        // 150 + width token columns (the weight tile's 128 x K bytes cost the same at any width), and
        // the product takes as many of those as the busiest SM walks tiles.  Not where few tiles of a
        // long K are shared between CTAs instead (launch_persistent), and only for a clear gain.
        static int sms = 0;
        if (sms == 0) {
            int dev = 0;
            if (cudaGetDevice(&dev) != cudaSuccess ||
                cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0)
                sms = 148;
        }
        const long long tiles_n = (N + TILE_W - 1) / TILE_W;
        const bool shared = scratch && tiles_n * tiles_m * 2 <= sms && (K + TILE_K - 1) / TILE_K >= 96;
        auto cost = [&](int tm) {
            const int width = ((M + tm - 1) / tm + 15) / 16 * 16;
            return ((tiles_n * tm + sms - 1) / sms) * (150 + width);
        };
        const int base = tiles_m;
        for (int tm = base + 1; tm <= base + 2 && !shared; ++tm)
            if (cost(tm) * 100 < cost(tiles_m) * 95) tiles_m = tm;
    }
    const int bn = ((M + tiles_m - 1) / tiles_m + 15) / 16 * 16;
    CUtensorMap mw, ma;
    AP_REQUIRE(make_map(&mw, w, N, K, ldw, TILE_W), "gemm_tc: cannot encode the weight's tensor map");
    AP_REQUIRE(make_map(&ma, a, M, K, lda, bn), "gemm_tc: cannot encode the activations' tensor map");
#define GO(BN, PR)                                                                                                  \
    return out_dtype == AP_F32                                                                                      \
               ? launch_persistent<BN, float, PR>(mw, ma, out, M, N, K, ldc, bn, scratch, scratch_bytes, stream)    \
               : launch_persistent<BN, bf16, PR>(mw, ma, out, M, N, K, ldc, bn, scratch, scratch_bytes, stream)
    if (pairs) {
        if (cap == 128) GO(128, true);
        GO(256, true);
    }
    if (cap == 128) GO(128, false);
    GO(256, false);
#undef GO
}

// Whether the persistent kernel is the one to use for this shape.  It is, except where its
// tiles fill the last round of SMs badly while the kernel with two weight tiles per CTA
// covers the whole product in a single, well-filled wave.
AP_EXPORT int ap_gemm_tc_prefers_persistent(int M, int N, int K) {
    // up to 128 rows every weight tile is one CTA of the kernel above, two to an SM, all resident
    // at once: they stream the weight at one rate, where tiles dealt out to one CTA per SM leave
    // the SMs with one tile fewer idle (8B gate+up at 128 rows: 48 against 59 us)
    if (M <= 128) return 0;
    const int bn = M <= 128 ? 128 : 256;
    const long long rows = (M + bn - 1) / bn;
    const long long tiles = ((N + TILE_W - 1) / TILE_W) * rows, dual = ((N + 2 * TILE_W - 1) / (2 * TILE_W)) * rows;
    const long long rounds = (tiles + 147) / 148;
    const bool badly_filled = tiles * 100 < rounds * 148 * 90;
    const bool dual_one_wave = dual <= 148 && dual >= 118;
    if (badly_filled && dual_one_wave && rounds <= 2) return 0;
    // A long K: a wave of two-tile CTAs takes 1.8 times a round of single tiles (its epilogue is
    // paid once per two tiles and its two accumulators hide some of the instruction's latency;
    // at K = 4096 it is 2.0 and nothing is gained).  4096 x 4096 x 14336: 353 against 392 us.
    const long long waves = (dual + 147) / 148;
    if (K >= 8192 && waves * 180 < rounds * 100) return 0;
    return 1;
}

// 0 when every tensor-core product so far ran to its end; else the code of the wait that
// expired (1 free stage, 2 operands, 3 accumulator).  Synchronises the device.
AP_EXPORT int ap_gemm_tc_status(void) {
    int v = -1;
    if (cudaMemcpyFromSymbol(&v, g_tc_status, sizeof(int)) != cudaSuccess) return -1;
    return v;
}

// Clear the status word so that products run again after a reported expiry.
AP_EXPORT int ap_gemm_tc_reset_status(void) {
    const int zero = 0;
    return cudaMemcpyToSymbol(g_tc_status, &zero, sizeof(int)) == cudaSuccess ? AP_OK : AP_ERR_LAUNCH;
}
