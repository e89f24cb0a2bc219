// bfloat16 causal grouped-query attention over paged keys and values on the tensor
// cores, for one head size fixed at compile time (-DAP_HEAD_DIM=...).
//
// The query heads that share a KV head are packed into the rows of the MMA tile, so a
// tile of K and V loaded once serves all of them:
//
//   tile kernel   (prompt portions and mixed batches): a CTA owns up to 64 rows
//                 = tokens x heads-of-one-KV-head of one sequence; its 4 warps take 16
//                 rows each and walk the same 64-key tiles of the sequence.
//   split kernel  (decode: one row per sequence): a CTA owns the <= 16 heads of one KV
//                 head of one row and one slice of the keys; its 4 warps take 16 keys of
//                 every 64-key tile each and merge at the end; slices of several CTAs are
//                 written as partial results (value, running maximum, sum) to scratch
//                 memory and combined by attention_merge_kernel.
//
// Keys and values come through the block table straight from the pages (cp.async into
// padded shared-memory rows, double buffered); pages that were given back (id < 0) and
// keys outside a row's window are never read.  Scores, softmax statistics and the output
// accumulate in 32-bit; probabilities are rounded to bfloat16 for the second product.
//
// Reference counterparts (cuda/src/kernels.cu): attention_qtile_kernel :1801,
// attention_split_gqa_kernel :1874, attention_merge_kernel :1997, causal rule :1583-1585.
#include "common.cuh"
#include <float.h>
#include <math.h>

#ifndef AP_HEAD_DIM
#error "compile with -DAP_HEAD_DIM=<head size>"
#endif

#define HD AP_HEAD_DIM
#define BKV 64                         // keys per shared-memory tile
#define ROW_BYTES (HD * 2 + 16)        // padded row: conflict-free ldmatrix for any HD % 16 == 0
#define TILE_BYTES (BKV * ROW_BYTES)
#define KSTEPS (HD / 16)
#define DTILES (HD / 8)
#define CHUNKS_PER_ROW (HD / 8)        // 16-byte chunks in a row
#define ATC_THREADS 128
#define LOG2E 1.4426950408889634f

static_assert(HD % 16 == 0 && HD >= 16 && HD <= 256, "head size must be a multiple of 16 up to 256");

struct AttnTcParams {
    const bf16* q;
    bf16* out;
    const bf16* cache;
    const int* block_table;
    const int* seq_start;
    const int* positions;
    float* part_o;       // [nsplit][T][nh][HD]
    float* part_ml;      // [nsplit][T][nh][2]
    size_t page_stride;
    int max_blocks, nseq, T, nh, nkv, P, window;
    int tokens_per_tile, heads_per_chunk, n_chunks, nsplit;
    float scale_log2;    // softmax scale * log2(e)
};

__device__ __forceinline__ void cp_async16(uint32_t smem, const void* gmem) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(smem), "l"(gmem) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() {
    asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(addr));
}
__device__ __forceinline__ void mma_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

// Shared memory of both kernels: two stages of (K tile, V tile) and the row pointers of
// the tile being fetched.
struct SmemLayout {
    static constexpr int kStage = 2 * TILE_BYTES;
    static constexpr int kPtrs = 2 * kStage;
    static constexpr int kTotal = kPtrs + BKV * 8;
};

// Fetch keys k0 .. k0+63 of one KV head into a stage.  Keys outside [kmin, kmax] (or in a
// page that was given back) become zero rows.
__device__ __forceinline__ void fetch_tile(uint8_t* smem, int stage, int k0, int kmin, int kmax,
                                           const bf16* cache, const int* table, int P, size_t page_stride,
                                           size_t head_off, size_t v_off) {
    const bf16** ptrs = reinterpret_cast<const bf16**>(smem + SmemLayout::kPtrs);
    if (threadIdx.x < BKV) {
        const int kpos = k0 + threadIdx.x;
        const bf16* p = nullptr;
        if (kpos >= kmin && kpos <= kmax) {
            const int page = table[kpos / P];
            if (page >= 0) p = cache + (size_t)page * page_stride + head_off + (size_t)(kpos % P) * HD;
        }
        ptrs[threadIdx.x] = p;
    }
    __syncthreads();
    uint8_t* ks = smem + stage * SmemLayout::kStage;
    uint8_t* vs = ks + TILE_BYTES;
    for (int c = threadIdx.x; c < BKV * CHUNKS_PER_ROW; c += ATC_THREADS) {
        const int key = c / CHUNKS_PER_ROW, ch = c - key * CHUNKS_PER_ROW;
        const bf16* p = ptrs[key];
        const uint32_t off = key * ROW_BYTES + ch * 16;
        if (p) {
            cp_async16((uint32_t)__cvta_generic_to_shared(ks + off), p + ch * 8);
            cp_async16((uint32_t)__cvta_generic_to_shared(vs + off), p + v_off + ch * 8);
        } else {
            *reinterpret_cast<uint4*>(ks + off) = make_uint4(0, 0, 0, 0);
            *reinterpret_cast<uint4*>(vs + off) = make_uint4(0, 0, 0, 0);
        }
    }
}

// Where 16-byte chunk `chunk` of key `key` lies in a K or V tile.  Padded rows (filled by
// cp.async) or, SWZ, what TMA writes with the 128-byte swizzle: one [64 keys x 128 bytes]
// block per 64 columns of the head, the chunk index XORed with the key's low bits.  Both
// give conflict-free ldmatrix.
#define SWZ_HALF_BYTES (BKV * 128)
template <bool SWZ> __device__ __forceinline__ uint32_t tile_offset(int key, int chunk) {
    if (SWZ) return (uint32_t)((chunk >> 3) * SWZ_HALF_BYTES + key * 128 + (((chunk & 7) ^ (key & 7)) << 4));
    return (uint32_t)(key * ROW_BYTES + chunk * 16);
}

// One warp's share of a tile: NT n-tiles of 8 keys starting at key `key0` of the tile.
// Updates the running maximum (log2 domain), the per-thread partial sums and the output.
template <int NT, bool SWZ = false>
__device__ __forceinline__ void process_keys(const uint8_t* ks, const uint8_t* vs, int key0, int k0,
                                             const uint32_t (&qf)[KSTEPS][4], float (&o)[DTILES][4],
                                             float (&m)[2], float (&l)[2], const int (&qpos)[2],
                                             const bool (&rvalid)[2], int window, float scale_log2,
                                             bool all_visible = false) {
    const int lane = threadIdx.x & 31;
    const int mi = lane >> 3, r8 = lane & 7;
    float s[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j) s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.f;
    const uint32_t ks_base = (uint32_t)__cvta_generic_to_shared(ks);
    const uint32_t vs_base = (uint32_t)__cvta_generic_to_shared(vs);
#pragma unroll
    for (int kk = 0; kk < KSTEPS; ++kk) {
#pragma unroll
        for (int np = 0; np < NT / 2; ++np) {
            uint32_t b[4];
            const int key = key0 + np * 16 + (mi >> 1) * 8 + r8;
            ldmatrix_x4(b, ks_base + tile_offset<SWZ>(key, kk * 2 + (mi & 1)));
            mma_16816(s[2 * np], qf[kk], b[0], b[1]);
            mma_16816(s[2 * np + 1], qf[kk], b[2], b[3]);
        }
    }
    // scale, mask, running maximum (a tile every row of the warp sees whole needs no mask)
    float mx[2] = {-INFINITY, -INFINITY};
    if (all_visible) {
#pragma unroll
        for (int j = 0; j < NT; ++j) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float v = s[j][e] * scale_log2;
                s[j][e] = v;
                mx[e >> 1] = fmaxf(mx[e >> 1], v);
            }
        }
    } else {
#pragma unroll
        for (int j = 0; j < NT; ++j) {
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int h = e >> 1;
                const int kpos = k0 + key0 + j * 8 + (lane & 3) * 2 + (e & 1);
                const bool ok = rvalid[h] && kpos <= qpos[h] && (window <= 0 || qpos[h] - kpos < window);
                const float v = ok ? s[j][e] * scale_log2 : -INFINITY;
                s[j][e] = v;
                mx[h] = fmaxf(mx[h], v);
            }
        }
    }
    float alpha[2], muse[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
        mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
        const float mnew = fmaxf(m[h], mx[h]);
        muse[h] = mnew == -INFINITY ? 0.f : mnew;       // no visible key yet: keep everything at zero
        alpha[h] = exp2f(m[h] - muse[h]);               // m = -inf gives 0
        m[h] = mnew;
        l[h] *= alpha[h];
    }
#pragma unroll
    for (int j = 0; j < NT; ++j) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const float p = exp2f(s[j][e] - muse[e >> 1]);
            s[j][e] = p;
            l[e >> 1] += p;
        }
    }
#pragma unroll
    for (int j = 0; j < DTILES; ++j) {
        o[j][0] *= alpha[0];
        o[j][1] *= alpha[0];
        o[j][2] *= alpha[1];
        o[j][3] *= alpha[1];
    }
#pragma unroll
    for (int ksx = 0; ksx < NT / 2; ++ksx) {
        uint32_t a[4];
        a[0] = pack_bf16(s[2 * ksx][0], s[2 * ksx][1]);
        a[1] = pack_bf16(s[2 * ksx][2], s[2 * ksx][3]);
        a[2] = pack_bf16(s[2 * ksx + 1][0], s[2 * ksx + 1][1]);
        a[3] = pack_bf16(s[2 * ksx + 1][2], s[2 * ksx + 1][3]);
#pragma unroll
        for (int dp = 0; dp < DTILES / 2; ++dp) {
            uint32_t b[4];
            const int key = key0 + ksx * 16 + (mi & 1) * 8 + r8;
            ldmatrix_x4_trans(b, vs_base + tile_offset<SWZ>(key, dp * 2 + (mi >> 1)));
            mma_16816(o[2 * dp], a, b[0], b[1]);
            mma_16816(o[2 * dp + 1], a, b[2], b[3]);
        }
    }
}

__device__ __forceinline__ void load_q_frags(uint32_t (&qf)[KSTEPS][4], const bf16* qa, const bf16* qb) {
    const int lane = threadIdx.x & 31;
#pragma unroll
    for (int kk = 0; kk < KSTEPS; ++kk) {
        const int c = kk * 16 + (lane & 3) * 2;
        qf[kk][0] = qa ? *reinterpret_cast<const uint32_t*>(qa + c) : 0u;
        qf[kk][1] = qb ? *reinterpret_cast<const uint32_t*>(qb + c) : 0u;
        qf[kk][2] = qa ? *reinterpret_cast<const uint32_t*>(qa + c + 8) : 0u;
        qf[kk][3] = qb ? *reinterpret_cast<const uint32_t*>(qb + c + 8) : 0u;
    }
}

// ---------------------------------------------------------------------------
// tile kernel: grid (query tiles over all sequences, nkv * n_chunks)
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(ATC_THREADS)
attention_tile_kernel(const AttnTcParams p) {
    extern __shared__ __align__(16) uint8_t smem[];
    __shared__ int s_seq, s_tile;
    if (threadIdx.x == 0) {
        // late tiles of a sequence have the most keys to walk: hand them out first
        int t = gridDim.x - 1 - blockIdx.x, found = -1;
        for (int s = 0; s < p.nseq; ++s) {
            const int n = p.seq_start[s + 1] - p.seq_start[s];
            const int nt = (n + p.tokens_per_tile - 1) / p.tokens_per_tile;
            if (t < nt) { found = s; break; }
            t -= nt;
        }
        s_seq = found;
        s_tile = t;
    }
    __syncthreads();
    if (s_seq < 0) return;
    const int seq = s_seq;
    const int row0 = p.seq_start[seq] + s_tile * p.tokens_per_tile;
    const int ntok = min(p.tokens_per_tile, p.seq_start[seq + 1] - row0);
    const int reps = p.nh / p.nkv;
    const int kvh = blockIdx.y / p.n_chunks, chunk = blockIdx.y - kvh * p.n_chunks;
    const int HC = p.heads_per_chunk;
    const int head0 = kvh * reps + chunk * HC;
    const int nheads = min(HC, reps - chunk * HC);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;

    int qpos[2];
    bool rvalid[2];
    const bf16* qptr[2];
    bf16* optr[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int r = warp * 16 + (lane >> 2) + h * 8;
        const int tok = r / HC, hq = r - tok * HC;
        rvalid[h] = tok < ntok && hq < nheads;
        const int row = row0 + (rvalid[h] ? tok : 0);
        qpos[h] = p.positions[row];
        const size_t off = ((size_t)row * p.nh + head0 + (rvalid[h] ? hq : 0)) * HD;
        qptr[h] = rvalid[h] ? p.q + off : nullptr;
        optr[h] = rvalid[h] ? p.out + off : nullptr;
    }
    uint32_t qf[KSTEPS][4];
    load_q_frags(qf, qptr[0], qptr[1]);

    const int kmax = p.positions[row0 + ntok - 1];
    const int first = p.positions[row0];
    const int kmin = (p.window > 0 && first - p.window + 1 > 0) ? first - p.window + 1 : 0;
    const int* table = p.block_table + (size_t)seq * p.max_blocks;
    const size_t head_off = (size_t)kvh * p.P * HD;
    const size_t v_off = (size_t)p.nkv * p.P * HD;

    float o[DTILES][4];
#pragma unroll
    for (int j = 0; j < DTILES; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

    // the last position any row of this warp holds (-1: the warp has no valid row)
    int wm = max(rvalid[0] ? qpos[0] : -1, rvalid[1] ? qpos[1] : -1);
    wm = max(wm, __shfl_xor_sync(0xffffffffu, wm, 4));
    wm = max(wm, __shfl_xor_sync(0xffffffffu, wm, 8));
    wm = max(wm, __shfl_xor_sync(0xffffffffu, wm, 16));
    // ... and the first (-1 unless every row of the warp is valid): tiles that end at or
    // before it are visible to all rows of the warp and need no mask
    int wmin = (rvalid[0] && rvalid[1]) ? min(qpos[0], qpos[1]) : -1;
    wmin = min(wmin, __shfl_xor_sync(0xffffffffu, wmin, 4));
    wmin = min(wmin, __shfl_xor_sync(0xffffffffu, wmin, 8));
    wmin = min(wmin, __shfl_xor_sync(0xffffffffu, wmin, 16));

    const int t_lo = kmin / BKV, t_hi = kmax / BKV;
    fetch_tile(smem, 0, t_lo * BKV, kmin, kmax, p.cache, table, p.P, p.page_stride, head_off, v_off);
    cp_async_commit();
    __syncthreads();      // the row pointers of this fetch have been read: the next fetch may replace them
    for (int t = t_lo; t <= t_hi; ++t) {
        const int cur = (t - t_lo) & 1;
        if (t < t_hi)
            fetch_tile(smem, cur ^ 1, (t + 1) * BKV, kmin, kmax, p.cache, table, p.P, p.page_stride, head_off, v_off);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();
        const uint8_t* ks = smem + cur * SmemLayout::kStage;
        // a warp whose rows all sit before this tile has nothing to add (causal)
        if (wm >= t * BKV) {
            const bool all_visible = t * BKV + BKV - 1 <= wmin && (p.window <= 0 || wm - t * BKV < p.window);
            process_keys<8>(ks, ks + TILE_BYTES, 0, t * BKV, qf, o, m, l, qpos, rvalid, p.window, p.scale_log2,
                            all_visible);
        }
        __syncthreads();
    }
    cp_async_wait<0>();
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        l[h] += __shfl_xor_sync(0xffffffffu, l[h], 1);
        l[h] += __shfl_xor_sync(0xffffffffu, l[h], 2);
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        if (!optr[h]) continue;
        const float inv = l[h] > 0.f ? 1.0f / l[h] : 0.f;
#pragma unroll
        for (int j = 0; j < DTILES; ++j) {
            const int d = j * 8 + (lane & 3) * 2;
            *reinterpret_cast<uint32_t*>(optr[h] + d) = pack_bf16(o[j][2 * h] * inv, o[j][2 * h + 1] * inv);
        }
    }
}

// ---------------------------------------------------------------------------
// split kernel: grid (rows, nkv * n_chunks, nsplit); every sequence brings one row
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(ATC_THREADS)
attention_split_kernel(const AttnTcParams p) {
    extern __shared__ __align__(16) uint8_t smem[];
    ap_pdl_trigger();
    ap_pdl_wait();
    const int row = blockIdx.x;              // row == sequence index
    const int reps = p.nh / p.nkv;
    const int kvh = blockIdx.y / p.n_chunks, chunk = blockIdx.y - kvh * p.n_chunks;
    const int HC = p.heads_per_chunk;       // <= 16
    const int head0 = kvh * reps + chunk * HC;
    const int nheads = min(HC, reps - chunk * HC);
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int pos = p.positions[row];

    int qpos[2] = {pos, pos};
    bool rvalid[2];
    const bf16* qptr[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int r = (lane >> 2) + h * 8;
        rvalid[h] = r < nheads;
        qptr[h] = rvalid[h] ? p.q + ((size_t)row * p.nh + head0 + r) * HD : nullptr;
    }
    uint32_t qf[KSTEPS][4];
    load_q_frags(qf, qptr[0], qptr[1]);

    const int kmax = pos;
    const int kmin = (p.window > 0 && pos - p.window + 1 > 0) ? pos - p.window + 1 : 0;
    const int* table = p.block_table + (size_t)row * p.max_blocks;
    const size_t head_off = (size_t)kvh * p.P * HD;
    const size_t v_off = (size_t)p.nkv * p.P * HD;
    const int t_first = kmin / BKV, t_last = kmax / BKV;
    const int ntiles = t_last - t_first + 1;
    const int per = (ntiles + p.nsplit - 1) / p.nsplit;
    const int t_lo = t_first + blockIdx.z * per;
    const int t_hi = min(t_last, t_lo + per - 1);

    float o[DTILES][4];
#pragma unroll
    for (int j = 0; j < DTILES; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

    if (t_lo <= t_hi) {
        fetch_tile(smem, 0, t_lo * BKV, kmin, kmax, p.cache, table, p.P, p.page_stride, head_off, v_off);
        cp_async_commit();
        __syncthreads();  // the row pointers of this fetch have been read: the next fetch may replace them
        for (int t = t_lo; t <= t_hi; ++t) {
            const int cur = (t - t_lo) & 1;
            if (t < t_hi)
                fetch_tile(smem, cur ^ 1, (t + 1) * BKV, kmin, kmax, p.cache, table, p.P, p.page_stride, head_off,
                           v_off);
            cp_async_commit();
            cp_async_wait<1>();
            __syncthreads();
            const uint8_t* ks = smem + cur * SmemLayout::kStage;
            if (t * BKV + warp * 16 <= kmax)
                process_keys<2>(ks, ks + TILE_BYTES, warp * 16, t * BKV, qf, o, m, l, qpos, rvalid, p.window,
                                p.scale_log2);
            __syncthreads();
        }
        cp_async_wait<0>();
    }
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        l[h] += __shfl_xor_sync(0xffffffffu, l[h], 1);
        l[h] += __shfl_xor_sync(0xffffffffu, l[h], 2);
    }
    // merge the four warps (each saw a quarter of the keys) through shared memory
    __syncthreads();
    float* so = reinterpret_cast<float*>(smem);                 // [4][16][HD]
    float* sm = so + 4 * 16 * HD;                               // [4][16]
    float* sl = sm + 4 * 16;                                    // [4][16]
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const int r = (lane >> 2) + h * 8;
        float* dst = so + ((size_t)warp * 16 + r) * HD;
#pragma unroll
        for (int j = 0; j < DTILES; ++j) {
            const int d = j * 8 + (lane & 3) * 2;
            dst[d] = o[j][2 * h];
            dst[d + 1] = o[j][2 * h + 1];
        }
        if ((lane & 3) == 0) {
            sm[warp * 16 + r] = m[h];
            sl[warp * 16 + r] = l[h];
        }
    }
    __syncthreads();
    for (int idx = threadIdx.x; idx < nheads * HD; idx += ATC_THREADS) {
        const int r = idx / HD, d = idx - r * HD;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) M = fmaxf(M, sm[w * 16 + r]);
        float L = 0.f, O = 0.f;
        if (M != -INFINITY) {
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                const float f = exp2f(sm[w * 16 + r] - M);
                L += sl[w * 16 + r] * f;
                O += so[((size_t)w * 16 + r) * HD + d] * f;
            }
        }
        const float val = L > 0.f ? O / L : 0.f;
        const size_t orow = (size_t)row * p.nh + head0 + r;
        if (p.nsplit == 1) {
            p.out[orow * HD + d] = __float2bfloat16_rn(val);
        } else {
            const size_t prow = (size_t)blockIdx.z * p.T * p.nh + orow;
            p.part_o[prow * HD + d] = val;
            if (d == 0) {
                p.part_ml[prow * 2] = M;
                p.part_ml[prow * 2 + 1] = L;
            }
        }
    }
}

// combine the slices of the split kernel: grid (rows, heads)
__global__ void attention_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_ml,
                                       bf16* __restrict__ out, int T, int nh, int nsplit) {
    const size_t orow = (size_t)blockIdx.x * nh + blockIdx.y;
    ap_pdl_trigger();
    ap_pdl_wait();
    float M = -INFINITY;
    for (int z = 0; z < nsplit; ++z) M = fmaxf(M, part_ml[((size_t)z * T * nh + orow) * 2]);
    for (int d = threadIdx.x; d < HD; d += blockDim.x) {
        float L = 0.f, O = 0.f;
        if (M != -INFINITY) {
            for (int z = 0; z < nsplit; ++z) {
                const size_t prow = (size_t)z * T * nh + orow;
                const float lz = part_ml[prow * 2 + 1];
                if (lz <= 0.f) continue;
                const float f = lz * exp2f(part_ml[prow * 2] - M);
                L += f;
                O += part_o[prow * HD + d] * f;
            }
        }
        out[orow * HD + d] = __float2bfloat16_rn(L > 0.f ? O / L : 0.f);
    }
}

static int configure_smem(const void* kern, int bytes) {
    if (bytes > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
        if (e != cudaSuccess) {
            ap_set_error("attention: cannot reserve %d bytes of shared memory: %s", bytes, cudaGetErrorString(e));
            return AP_ERR_LAUNCH;
        }
    }
    return AP_OK;
}

// mode 0: tile kernel over `total_tiles` query tiles (prompt portions, mixed batches);
// mode 1: split kernel, one row per sequence, `nsplit` key slices; part_o/part_ml are
//         scratch of nsplit*T*nh*HD and nsplit*T*nh*2 floats (unused for nsplit == 1), which
//         a second kernel combines.
AP_EXPORT int ap_attention_tc(const void* q, void* out, const void* cache, const int* block_table,
                              int max_blocks, const int* seq_start, const int* positions, int nseq, int T,
                              int nh, int nkv, int hd, int P, long long page_stride, float scale, int window,
                              int mode, int total_tiles, int nsplit, float* part_o, float* part_ml,
                              cudaStream_t stream) {
    AP_REQUIRE(hd == HD, "attention: this library was compiled for head size %d, not %d", HD, hd);
    AP_REQUIRE(T >= 0 && nseq >= 0 && nh > 0 && nkv > 0 && nh % nkv == 0 && P > 0 && max_blocks > 0,
               "attention: bad sizes T=%d heads=%d kv_heads=%d page=%d", T, nh, nkv, P);
    if (T == 0 || nseq == 0) return AP_OK;
    AttnTcParams p;
    p.q = (const bf16*)q; p.out = (bf16*)out; p.cache = (const bf16*)cache;
    p.block_table = block_table; p.seq_start = seq_start; p.positions = positions;
    p.part_o = part_o; p.part_ml = part_ml; p.page_stride = (size_t)page_stride;
    p.max_blocks = max_blocks; p.nseq = nseq; p.T = T; p.nh = nh; p.nkv = nkv; p.P = P; p.window = window;
    p.scale_log2 = scale * LOG2E;
    const int reps = nh / nkv;
    static bool configured = false;
    const int merge_bytes = (4 * 16 * HD + 2 * 4 * 16) * (int)sizeof(float);
    const int smem_bytes = SmemLayout::kTotal > merge_bytes ? SmemLayout::kTotal : merge_bytes;
    if (!configured) {
        int rc = configure_smem((const void*)attention_tile_kernel, smem_bytes);
        if (rc != AP_OK) return rc;
        rc = configure_smem((const void*)attention_split_kernel, smem_bytes);
        if (rc != AP_OK) return rc;
        configured = true;
    }
    if (mode == 0) {
        p.heads_per_chunk = reps < 64 ? reps : 64;
        p.n_chunks = (reps + p.heads_per_chunk - 1) / p.heads_per_chunk;
        p.tokens_per_tile = 64 / p.heads_per_chunk;
        p.nsplit = 1;
        AP_REQUIRE(total_tiles > 0, "attention: the tile kernel needs the number of query tiles");
        AP_REQUIRE(nkv * p.n_chunks <= 65535, "attention: too many KV heads for the grid");
        dim3 grid(total_tiles, nkv * p.n_chunks);
        attention_tile_kernel<<<grid, ATC_THREADS, smem_bytes, stream>>>(p);
        AP_CHECK_LAUNCH("attention_tile");
        return AP_OK;
    }
    AP_REQUIRE(mode == 1, "attention: unknown mode %d", mode);
    AP_REQUIRE(nseq == T, "attention: the split kernel takes one row per sequence (T=%d, nseq=%d)", T, nseq);
    AP_REQUIRE(nsplit >= 1 && nsplit <= 65535, "attention: bad number of key slices %d", nsplit);
    AP_REQUIRE(nsplit == 1 || (part_o && part_ml), "attention: key slices need scratch memory");
    p.heads_per_chunk = reps < 16 ? reps : 16;
    p.n_chunks = (reps + p.heads_per_chunk - 1) / p.heads_per_chunk;
    p.tokens_per_tile = 1;
    p.nsplit = nsplit;
    AP_REQUIRE(nkv * p.n_chunks <= 65535, "attention: too many KV heads for the grid");
    dim3 grid(T, nkv * p.n_chunks, nsplit);
    AP_CHECK_PDL_LAUNCH("attention_split",
                        ap_launch_pdl(attention_split_kernel, grid, dim3(ATC_THREADS), smem_bytes, stream, p));
    if (nsplit > 1) {
        dim3 mgrid(T, nh);
        AP_CHECK_PDL_LAUNCH("attention_merge",
                            ap_launch_pdl(attention_merge_kernel, mgrid, dim3(HD < 128 ? 64 : 128), 0, stream,
                                          (const float*)part_o, (const float*)part_ml, (bf16*)out, T, nh, nsplit));
    }
    return AP_OK;
}

// how many query rows of one sequence a tile of the tile kernel holds
AP_EXPORT int ap_attention_tc_tokens_per_tile(int nh, int nkv) {
    const int reps = nh / nkv;
    const int hc = reps < 64 ? reps : 64;
    return 64 / hc;
}

// ---------------------------------------------------------------------------
// The split kernel fed by TMA, for head sizes 64 and 128 and pages of 8, 16, 32 or 64 keys.
// A decode step's attention only streams the cache, so what matters is how many bytes are in
// flight: here a producer warp (one lane per page of a tile, the page ids read from the block
// table one tile ahead) keeps a ring of three 64-key tiles of K and V loading by
// cp.async.bulk.tensor (128-byte swizzle), with no address arithmetic in the consumer warps
// and no round trip to the block table inside the loop.  The four consumer warps take 16 keys
// of every tile each, as in attention_split_kernel.  CLUSTER: the key slices of one row and KV
// head form a thread-block cluster (2, 4, 8 or 16 CTAs) and hand their results to its first CTA
// through distributed shared memory, which combines them and writes the row: no partial
// results in global memory and no second kernel.  Otherwise the slices are combined as for
// attention_split_kernel.
// Every barrier wait is bounded; on expiry a status word is raised and the CTA does no more
// (in a cluster it still walks to the cluster barriers, or its peers would wait).
// ---------------------------------------------------------------------------
#if (AP_HEAD_DIM == 64 || AP_HEAD_DIM == 128)
#include "tcgen05.cuh"
#include <cuda.h>

#define DT_STAGES 3
#define DT_THREADS 160                        // four consumer warps, one producer warp
#define DT_NHALF (HD / 64)
#define DT_KV_BYTES (DT_NHALF * SWZ_HALF_BYTES)   // K (or V) of one tile
#define DT_STAGE_BYTES (2 * DT_KV_BYTES)
#define DT_ERR_WAIT 6

static __device__ int g_dt_status;

struct DtSmem {
    static constexpr int kBars = DT_STAGES * DT_STAGE_BYTES;
    static constexpr int kUsed = kBars + 128;
    static constexpr int kMerge = (4 * 16 * HD + 2 * 4 * 16) * (int)sizeof(float);
    static constexpr int kTotal = (kUsed > kMerge ? kUsed : kMerge) + 1024;   // + alignment slack
    // cluster: the slices' results [slice][head][HD + 2] in the first CTA, behind its own merge
    // buffers and before the barriers
    static constexpr int kXchRow = HD + 2;
    static __host__ __device__ constexpr bool exchange_fits(int nsplit, int heads) {
        return kMerge + nsplit * heads * kXchRow * (int)sizeof(float) <= kBars;
    }
};

template <bool CLUSTER>
__global__ void __launch_bounds__(DT_THREADS)
attention_split_tma_kernel(const __grid_constant__ CUtensorMap tmap_kv, const __grid_constant__ CUtensorMap tmap_run,
                           const AttnTcParams p) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* full = (uint64_t*)(smem + DtSmem::kBars);
    uint64_t* empty = full + DT_STAGES;
    volatile int* abort_flag = (volatile int*)(empty + DT_STAGES);
    const bool skip = *(volatile int*)&g_dt_status != 0;
    if (!CLUSTER && skip) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    if (threadIdx.x == 0) {
        for (int s = 0; s < DT_STAGES; ++s) {
            tc::mbar_init(&full[s], 1);
            tc::mbar_init(&empty[s], 4);
        }
        *abort_flag = 0;
        tc::fence_barrier_init();
        tc::prefetch_tensormap(&tmap_kv);
        tc::prefetch_tensormap(&tmap_run);
    }
    // V starts as zeros: what a skipped page leaves in a stage must be finite, because a
    // probability of zero times a NaN would poison the row
    for (int s = 0; s < DT_STAGES; ++s)
        for (int i = threadIdx.x; i < DT_KV_BYTES / 16; i += DT_THREADS)
            reinterpret_cast<uint4*>(smem + s * DT_STAGE_BYTES + DT_KV_BYTES)[i] = make_uint4(0, 0, 0, 0);
    tc::fence_proxy_async();
    __syncthreads();
    ap_pdl_trigger();
    // The step's positions and block tables were uploaded before any kernel of the step ran,
    // and of the cache only the newest key of each row is written by the kernel before this
    // one: the producer starts loading older keys at once and waits for the kernels before
    // this one only where it comes to the tile that holds the newest key; the consumers wait
    // before they read the queries.

    const int row = blockIdx.x;              // row == sequence index
    const int reps = p.nh / p.nkv;
    const int kvh = blockIdx.y / p.n_chunks, chunk = blockIdx.y - kvh * p.n_chunks;
    const int HC = p.heads_per_chunk;       // <= 16
    const int head0 = kvh * reps + chunk * HC;
    const int nheads = min(HC, reps - chunk * HC);
    const int pos = p.positions[row];
    const int kmax = pos;
    const int kmin = (p.window > 0 && pos - p.window + 1 > 0) ? pos - p.window + 1 : 0;
    const int* table = p.block_table + (size_t)row * p.max_blocks;
    const int t_first = kmin / BKV, t_last = kmax / BKV;
    const int ntiles = t_last - t_first + 1;
    const int per = (ntiles + p.nsplit - 1) / p.nsplit;
    const int t_lo = t_first + blockIdx.z * per;
    const int t_hi = min(t_last, t_lo + per - 1);
    const int n = skip ? 0 : t_hi - t_lo + 1; // tiles of this slice (<= 0: none)

    float o[DTILES][4];
#pragma unroll
    for (int j = 0; j < DTILES; ++j) o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.f;
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.f, 0.f};

    if (warp == 4) {
        // producer: lane j owns page j of every tile; a page larger than a tile is lane 0's, and
        // the tile a part of it
        const bool big_pages = p.P > BKV;
        const int pages_per_tile = big_pages ? 1 : BKV / p.P;
        const int page_bytes = (big_pages ? BKV : p.P) * 128;   // one page (or tile), 64 columns of the head
        auto page_of = [&](int it) {
            if (big_pages) {
                const int lp = (t_lo + it) * BKV / p.P;
                return (it >= n || lane != 0 || lp >= p.max_blocks) ? -1 : table[lp];
            }
            const int lp = (t_lo + it) * pages_per_tile + lane;
            if (it >= n || lane >= pages_per_tile || lp >= p.max_blocks || lp * p.P > kmax ||
                lp * p.P + p.P - 1 < kmin)
                return -1;
            return table[lp];
        };
        int page = page_of(0);
        // tiles that may be loaded before the kernels ahead of this one are done: the first ring
        // fill, short of the tile with the newest key
        const int early = min(min(n, DT_STAGES), t_last - t_lo);
        bool waited = false;
        for (int it = 0; it < n; ++it) {
            const int s = it % DT_STAGES;
            const uint32_t ph = (uint32_t)((it / DT_STAGES) & 1);
            if (!waited && it >= early) {
                ap_pdl_wait();
                waited = true;
            }
            const int next_page = page_of(it + 1);        // in flight while this tile's loads go out
            const int valid = __popc(__ballot_sync(0xffffffffu, page >= 0));
            int fine = 1;
            if (lane == 0) {
                if (*abort_flag) fine = 0;
                if (fine && !tc::mbar_wait(&empty[s], ph ^ 1)) {
                    *abort_flag = 1;
                    atomicExch(&g_dt_status, DT_ERR_WAIT);
                    fine = 0;
                }
                if (fine) tc::mbar_expect_tx(&full[s], (uint32_t)(valid * page_bytes * DT_NHALF * 2));
            }
            fine = __shfl_sync(0xffffffffu, fine, 0);
            if (!fine) break;
            // pages of a tile that follow one another in memory (a sequence's pages are handed out
            // in rising order) come with one box per half: loads are issued at a limited rate
            const int page0 = __shfl_sync(0xffffffffu, page, 0);
            const bool run = !big_pages && page0 >= 0 &&
                             __all_sync(0xffffffffu, lane >= pages_per_tile || page == page0 + lane);
            if (run) {
                if (lane == 0) {
                    uint8_t* dst = smem + s * DT_STAGE_BYTES;
#pragma unroll
                    for (int h = 0; h < DT_NHALF; ++h) {
                        tc::tma_load_3d(dst + h * SWZ_HALF_BYTES, &tmap_run, h * 64, kvh * p.P, page0, &full[s]);
                        tc::tma_load_3d(dst + DT_KV_BYTES + h * SWZ_HALF_BYTES, &tmap_run, h * 64,
                                        (p.nkv + kvh) * p.P, page0, &full[s]);
                    }
                }
            } else if (page >= 0) {
                uint8_t* dst = smem + s * DT_STAGE_BYTES + lane * page_bytes;
                const int within = big_pages ? ((t_lo + it) * BKV) % p.P : 0;
                const int krow = ((page * 2 + 0) * p.nkv + kvh) * p.P + within;
                const int vrow = ((page * 2 + 1) * p.nkv + kvh) * p.P + within;
#pragma unroll
                for (int h = 0; h < DT_NHALF; ++h) {
                    tc::tma_load_2d(dst + h * SWZ_HALF_BYTES, &tmap_kv, h * 64, krow, &full[s]);
                    tc::tma_load_2d(dst + DT_KV_BYTES + h * SWZ_HALF_BYTES, &tmap_kv, h * 64, vrow, &full[s]);
                }
            }
            page = next_page;
        }
        if (!waited) ap_pdl_wait();
    } else {
        ap_pdl_wait();
        int qpos[2] = {pos, pos};
        bool rvalid[2];
        const bf16* qptr[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int r = (lane >> 2) + h * 8;
            rvalid[h] = r < nheads;
            qptr[h] = rvalid[h] ? p.q + ((size_t)row * p.nh + head0 + r) * HD : nullptr;
        }
        uint32_t qf[KSTEPS][4];
        load_q_frags(qf, qptr[0], qptr[1]);
        for (int it = 0; it < n; ++it) {
            const int s = it % DT_STAGES;
            const uint32_t ph = (uint32_t)((it / DT_STAGES) & 1);
            // ldmatrix and mma are warp-wide: the whole warp goes on, or none of it
            if (!__all_sync(0xffffffffu, tc::mbar_wait(&full[s], ph))) {
                if (!*abort_flag) {
                    *abort_flag = 1;
                    atomicExch(&g_dt_status, DT_ERR_WAIT);
                }
                break;
            }
            const int t = t_lo + it;
            const uint8_t* ks = smem + s * DT_STAGE_BYTES;
            if (t * BKV + warp * 16 <= kmax)
                process_keys<2, true>(ks, ks + DT_KV_BYTES, warp * 16, t * BKV, qf, o, m, l, qpos, rvalid, p.window,
                                      p.scale_log2);
            __syncwarp();
            if (lane == 0) tc::mbar_arrive(&empty[s]);
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            l[h] += __shfl_xor_sync(0xffffffffu, l[h], 1);
            l[h] += __shfl_xor_sync(0xffffffffu, l[h], 2);
        }
    }
    // merge the four consumer warps (each saw a quarter of the keys) through shared memory;
    // every load has landed (each was waited for), so the stages can be written over
    if (CLUSTER) tc::cluster_arrive();        // nothing is loaded into this CTA's shared memory any more
    __syncthreads();
    const bool dead = skip || *abort_flag != 0;
    if (!CLUSTER && dead) return;
    float* so = reinterpret_cast<float*>(smem);                 // [4][16][HD]
    float* sm = so + 4 * 16 * HD;                               // [4][16]
    float* sl = sm + 4 * 16;                                    // [4][16]
    float* xch = reinterpret_cast<float*>(smem + DtSmem::kMerge);   // cluster: [slice][head][HD + 2]
    if (warp < 4 && !dead) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int r = (lane >> 2) + h * 8;
            float* dst = so + ((size_t)warp * 16 + r) * HD;
#pragma unroll
            for (int j = 0; j < DTILES; ++j) {
                const int d = j * 8 + (lane & 3) * 2;
                dst[d] = o[j][2 * h];
                dst[d + 1] = o[j][2 * h + 1];
            }
            if ((lane & 3) == 0) {
                sm[warp * 16 + r] = m[h];
                sl[warp * 16 + r] = l[h];
            }
        }
    }
    __syncthreads();
    uint32_t xch0 = 0;
    if (CLUSTER) {
        tc::cluster_wait();                   // ... nor into any other CTA's of the cluster
        xch0 = tc::map_to_rank(tc::smem_addr(xch), 0u);
    }
    for (int idx = threadIdx.x; idx < nheads * HD && !dead; idx += DT_THREADS) {
        const int r = idx / HD, d = idx - r * HD;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < 4; ++w) M = fmaxf(M, sm[w * 16 + r]);
        float L = 0.f, O = 0.f;
        if (M != -INFINITY) {
#pragma unroll
            for (int w = 0; w < 4; ++w) {
                const float f = exp2f(sm[w * 16 + r] - M);
                L += sl[w * 16 + r] * f;
                O += so[((size_t)w * 16 + r) * HD + d] * f;
            }
        }
        const float val = L > 0.f ? O / L : 0.f;
        const size_t orow = (size_t)row * p.nh + head0 + r;
        if (CLUSTER) {
            const uint32_t at = xch0 + (uint32_t)((blockIdx.z * HC + r) * DtSmem::kXchRow) * 4u;
            tc::st_cluster_f32(at + (uint32_t)d * 4u, val);
            if (d == 0) {
                tc::st_cluster_f32(at + (uint32_t)HD * 4u, M);
                tc::st_cluster_f32(at + (uint32_t)(HD + 1) * 4u, L);
            }
        } else if (p.nsplit == 1) {
            p.out[orow * HD + d] = __float2bfloat16_rn(val);
        } else {
            const size_t prow = (size_t)blockIdx.z * p.T * p.nh + orow;
            p.part_o[prow * HD + d] = val;
            if (d == 0) {
                p.part_ml[prow * 2] = M;
                p.part_ml[prow * 2 + 1] = L;
            }
        }
    }
    if (CLUSTER) {
        tc::cluster_sync();                   // every slice has delivered
        if (blockIdx.z != 0 || dead) return;
        for (int idx = threadIdx.x; idx < nheads * HD; idx += DT_THREADS) {
            const int r = idx / HD, d = idx - r * HD;
            float M = -INFINITY;
            for (int z = 0; z < p.nsplit; ++z) M = fmaxf(M, xch[(z * HC + r) * DtSmem::kXchRow + HD]);
            float L = 0.f, O = 0.f;
            if (M != -INFINITY) {
                for (int z = 0; z < p.nsplit; ++z) {                      // slices in order
                    const float* rowz = xch + (z * HC + r) * DtSmem::kXchRow;
                    const float lz = rowz[HD + 1];
                    if (lz <= 0.f) continue;
                    const float f = lz * exp2f(rowz[HD] - M);
                    L += f;
                    O += rowz[d] * f;
                }
            }
            p.out[((size_t)row * p.nh + head0 + r) * HD + d] = __float2bfloat16_rn(L > 0.f ? O / L : 0.f);
        }
    }
}

typedef CUresult (*DtEncodeFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                               const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                               CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static DtEncodeFn dt_encode_fn() {
    static DtEncodeFn fn = nullptr;
    if (!fn) {
        void* ptr = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &ptr, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (DtEncodeFn)ptr;
    }
    return fn;
}

// 1 when ap_attention_decode_tma takes this shape, else 0 (the caller then uses ap_attention_tc)
AP_EXPORT int ap_attention_decode_tma_supports(int nh, int nkv, int hd, int P) {
    if (hd != HD || nkv <= 0 || nh % nkv) return 0;
    // pages that divide a key tile, or that whole key tiles divide
    if (P < 8 || (P <= BKV ? BKV % P : (P % BKV || P > 1024))) return 0;
    return dt_encode_fn() != nullptr;
}

// 1 when `nsplit` key slices are combined inside a thread-block cluster (no scratch needed)
AP_EXPORT int ap_attention_decode_tma_in_cluster(int nh, int nkv, int nsplit) {
    if (nkv <= 0 || nh % nkv) return 0;
    const int reps = nh / nkv;
    const int hc = reps < 16 ? reps : 16;
    return (nsplit == 2 || nsplit == 4 || nsplit == 8 || nsplit == 16) && DtSmem::exchange_fits(nsplit, hc);
}

// The split kernel with TMA loads: one row per sequence, `nsplit` key slices; part_o/part_ml
// as for ap_attention_tc (unused for nsplit == 1 and where the slices form a cluster).  `num_pages`: pages in `cache`, which must
// be contiguous ([page][2][nkv][P][hd]).  Unwritten slots of the cache must hold finite values.
AP_EXPORT int ap_attention_decode_tma(const void* q, void* out, const void* cache, long long num_pages,
                                      const int* block_table, int max_blocks, const int* positions, int T,
                                      int nh, int nkv, int hd, int P, long long page_stride, float scale,
                                      int window, int nsplit, float* part_o, float* part_ml, cudaStream_t stream) {
    AP_REQUIRE(ap_attention_decode_tma_supports(nh, nkv, hd, P), "attention (decode, TMA): shape not supported: "
               "heads=%d kv_heads=%d head_dim=%d page=%d", nh, nkv, hd, P);
    AP_REQUIRE(page_stride == 2LL * nkv * P * HD, "attention (decode, TMA): pages must be contiguous");
    AP_REQUIRE(T >= 0 && max_blocks > 0 && num_pages > 0, "attention (decode, TMA): bad sizes");
    if (T == 0) return AP_OK;
    AP_REQUIRE(((uintptr_t)cache & 15) == 0, "attention (decode, TMA): the cache must be 16-byte aligned");
    AP_REQUIRE(nsplit >= 1 && nsplit <= 65535, "attention: bad number of key slices %d", nsplit);
    const bool cluster = ap_attention_decode_tma_in_cluster(nh, nkv, nsplit) != 0;
    AP_REQUIRE(nsplit == 1 || cluster || (part_o && part_ml), "attention: key slices need scratch memory");
    CUtensorMap mkv;
    {
        cuuint64_t dims[2] = {(cuuint64_t)HD, (cuuint64_t)(num_pages * 2 * nkv * P)};
        cuuint64_t strides[1] = {(cuuint64_t)HD * 2};
        cuuint32_t box[2] = {64, (cuuint32_t)(P < BKV ? P : BKV)};
        cuuint32_t es[2] = {1, 1};
        AP_REQUIRE(dt_encode_fn()(&mkv, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(cache), dims, strides,
                                  box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS,
                   "attention (decode, TMA): cannot encode the cache tensor map");
    }
    CUtensorMap mrun;
    {
        // the same cache as [page][row within the page][column]: a box spans the pages of a key tile
        cuuint64_t dims[3] = {(cuuint64_t)HD, (cuuint64_t)(2 * nkv * P), (cuuint64_t)num_pages};
        cuuint64_t strides[2] = {(cuuint64_t)HD * 2, (cuuint64_t)page_stride * 2};
        // (pages larger than a tile are never loaded through this map)
        cuuint32_t box[3] = {64, (cuuint32_t)(P < BKV ? P : BKV), (cuuint32_t)(P < BKV ? BKV / P : 1)};
        cuuint32_t es[3] = {1, 1, 1};
        AP_REQUIRE(dt_encode_fn()(&mrun, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(cache), dims, strides,
                                  box, es, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                  CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) == CUDA_SUCCESS,
                   "attention (decode, TMA): cannot encode the tensor map of page runs");
    }
    static bool configured = false;
    if (!configured) {
        int rc = configure_smem((const void*)attention_split_tma_kernel<false>, DtSmem::kTotal);
        if (rc != AP_OK) return rc;
        rc = configure_smem((const void*)attention_split_tma_kernel<true>, DtSmem::kTotal);
        if (rc != AP_OK) return rc;
        configured = true;
    }
    AttnTcParams p;
    p.q = (const bf16*)q; p.out = (bf16*)out; p.cache = (const bf16*)cache;
    p.block_table = block_table; p.seq_start = nullptr; p.positions = positions;
    p.part_o = part_o; p.part_ml = part_ml; p.page_stride = (size_t)page_stride;
    p.max_blocks = max_blocks; p.nseq = T; p.T = T; p.nh = nh; p.nkv = nkv; p.P = P; p.window = window;
    p.scale_log2 = scale * LOG2E;
    const int reps = nh / nkv;
    p.heads_per_chunk = reps < 16 ? reps : 16;
    p.n_chunks = (reps + p.heads_per_chunk - 1) / p.heads_per_chunk;
    p.tokens_per_tile = 1;
    p.nsplit = nsplit;
    AP_REQUIRE(nkv * p.n_chunks <= 65535, "attention: too many KV heads for the grid");
    dim3 grid(T, nkv * p.n_chunks, nsplit);
    if (cluster) {
        static bool wide_clusters = false;
        if (nsplit > 8 && !wide_clusters) {
            // clusters of more than 8 CTAs are an opt-in of the kernel
            cudaError_t e = cudaFuncSetAttribute(attention_split_tma_kernel<true>, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
            AP_REQUIRE(e == cudaSuccess, "attention: clusters of %d CTAs are not available: %s", nsplit, cudaGetErrorString(e));
            wide_clusters = true;
        }
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = grid;
        cfg.blockDim = dim3(DT_THREADS);
        cfg.dynamicSmemBytes = DtSmem::kTotal;
        cfg.stream = stream;
        cudaLaunchAttribute attr[2];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = 1;
        attr[0].val.clusterDim.y = 1;
        attr[0].val.clusterDim.z = nsplit;
        attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[1].val.programmaticStreamSerializationAllowed = 1;
        cfg.attrs = attr;
        cfg.numAttrs = ap_pdl_enabled() ? 2 : 1;
        AP_CHECK_PDL_LAUNCH("attention_split_tma", cudaLaunchKernelEx(&cfg, attention_split_tma_kernel<true>, mkv, mrun, p));
        return AP_OK;
    }
    AP_CHECK_PDL_LAUNCH("attention_split_tma", ap_launch_pdl(attention_split_tma_kernel<false>, grid, dim3(DT_THREADS),
                                                             (size_t)DtSmem::kTotal, stream, mkv, mrun, p));
    if (nsplit > 1) {
        dim3 mgrid(T, nh);
        AP_CHECK_PDL_LAUNCH("attention_merge",
                            ap_launch_pdl(attention_merge_kernel, mgrid, dim3(HD < 128 ? 64 : 128), 0, stream,
                                          (const float*)part_o, (const float*)part_ml, (bf16*)out, T, nh, nsplit));
    }
    return AP_OK;
}

// CTAs of the TMA-fed decode kernel that the GPU holds at once (for planning the key slices)
AP_EXPORT int ap_attention_decode_tma_slots(void) {
    static int slots = 0;
    if (slots == 0) {
        int dev = 0, sms = 0, per_sm = 0;
        if (cudaGetDevice(&dev) != cudaSuccess ||
            cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess ||
            configure_smem((const void*)attention_split_tma_kernel<true>, DtSmem::kTotal) != AP_OK ||
            cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, attention_split_tma_kernel<true>, DT_THREADS,
                                                          DtSmem::kTotal) != cudaSuccess || per_sm <= 0)
            return 296;
        slots = sms * per_sm;
    }
    return slots;
}

AP_EXPORT int ap_attention_decode_tma_status(void) {
    int v = -1;
    if (cudaMemcpyFromSymbol(&v, g_dt_status, sizeof(int)) != cudaSuccess) return -1;
    return v;
}
#else
AP_EXPORT int ap_attention_decode_tma_supports(int, int, int, int) { return 0; }
AP_EXPORT int ap_attention_decode_tma_in_cluster(int, int, int) { return 0; }
AP_EXPORT int ap_attention_decode_tma_slots(void) { return 0; }
#endif

// ---------------------------------------------------------------------------
// The split kernel for callers that cannot allocate: its scratch is a fixed array in this
// library (see attention_noalloc.h for who needs this and what they must observe).
// ---------------------------------------------------------------------------
#include "attention_noalloc.h"

static __device__ __align__(256) float g_static_scratch[AP_ATTENTION_STATIC_SCRATCH_FLOATS];

#define AP_MAX_DEVICES 64
// Device address of g_static_scratch per device.  In host code the array's name is only a
// handle for the runtime, not an address a kernel could use, so the address is looked up.
static float* g_static_scratch_addr[AP_MAX_DEVICES];

AP_EXPORT int ap_attention_decode_static(const void* q, void* out, const void* cache, const int* block_table,
                                         int max_blocks, const int* positions, int T, int num_heads,
                                         int num_kv_heads, int head_dim, int page_size, long long page_stride,
                                         float scale, int window, int nsplit, cudaStream_t stream) {
    AP_REQUIRE(head_dim == HD, "attention: this library was compiled for head size %d, not %d", HD, head_dim);
    AP_REQUIRE(T >= 0 && num_heads > 0 && num_kv_heads > 0 && num_heads % num_kv_heads == 0 && page_size > 0 &&
                   max_blocks > 0 && nsplit >= 1 && nsplit <= 65535,
               "attention: bad sizes T=%d heads=%d kv_heads=%d page=%d slices=%d", T, num_heads, num_kv_heads,
               page_size, nsplit);
    if (T == 0) return AP_OK;
    const long long need = nsplit > 1 ? (long long)nsplit * T * num_heads * (HD + 2) : 0;
    AP_REQUIRE(need <= AP_ATTENTION_STATIC_SCRATCH_FLOATS,
               "attention: %d slices of %d rows x %d heads need %lld floats of scratch, the built-in array "
               "holds %d; use fewer slices or the entry point that takes scratch from the caller",
               nsplit, T, num_heads, need, AP_ATTENTION_STATIC_SCRATCH_FLOATS);
    int device = -1;
    AP_REQUIRE(cudaGetDevice(&device) == cudaSuccess && device >= 0 && device < AP_MAX_DEVICES,
               "attention: cannot tell the current device");
    if (!g_static_scratch_addr[device]) {
        // first call on this device: not inside a stream capture, please
        float* p = nullptr;
        cudaError_t e = cudaGetSymbolAddress((void**)&p, g_static_scratch);
        AP_REQUIRE(e == cudaSuccess && p != nullptr, "attention: cannot find the built-in scratch array: %s",
                   cudaGetErrorString(e));
        const int merge_bytes = (4 * 16 * HD + 2 * 4 * 16) * (int)sizeof(float);
        const int smem_bytes = SmemLayout::kTotal > merge_bytes ? SmemLayout::kTotal : merge_bytes;
        int rc = configure_smem((const void*)attention_split_kernel, smem_bytes);
        if (rc != AP_OK) return rc;
        g_static_scratch_addr[device] = p;
    }
    float* scratch = g_static_scratch_addr[device];
    const int reps = num_heads / num_kv_heads;
    AttnTcParams p;
    p.q = (const bf16*)q; p.out = (bf16*)out; p.cache = (const bf16*)cache;
    p.block_table = block_table; p.seq_start = nullptr; p.positions = positions;
    p.part_o = scratch;
    p.part_ml = scratch + (size_t)nsplit * T * num_heads * HD;
    p.page_stride = (size_t)page_stride;
    p.max_blocks = max_blocks; p.nseq = T; p.T = T; p.nh = num_heads; p.nkv = num_kv_heads; p.P = page_size;
    p.window = window; p.scale_log2 = scale * LOG2E;
    p.heads_per_chunk = reps < 16 ? reps : 16;
    p.n_chunks = (reps + p.heads_per_chunk - 1) / p.heads_per_chunk;
    p.tokens_per_tile = 1;
    p.nsplit = nsplit;
    AP_REQUIRE(num_kv_heads * p.n_chunks <= 65535, "attention: too many KV heads for the grid");
    const int merge_bytes = (4 * 16 * HD + 2 * 4 * 16) * (int)sizeof(float);
    const int smem_bytes = SmemLayout::kTotal > merge_bytes ? SmemLayout::kTotal : merge_bytes;
    dim3 grid(T, num_kv_heads * p.n_chunks, nsplit);
    attention_split_kernel<<<grid, ATC_THREADS, smem_bytes, stream>>>(p);
    AP_CHECK_LAUNCH("attention_split (built-in scratch)");
    if (nsplit > 1) {
        dim3 mgrid(T, num_heads);
        attention_merge_kernel<<<mgrid, HD < 128 ? 64 : 128, 0, stream>>>(p.part_o, p.part_ml, (bf16*)out, T,
                                                                           num_heads, nsplit);
        AP_CHECK_LAUNCH("attention_merge (built-in scratch)");
    }
    return AP_OK;
}
