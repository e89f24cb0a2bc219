// Causal grouped-query attention over paged keys and values, for one head size
// fixed at compile time (-DAP_HEAD_DIM=...).  One launch serves a whole step: rows
// of prompt portions and single decode rows alike, each row with its own sequence,
// position and block table.
//
//   q, out : [T, nh, HD]
//   cache  : one layer, [page][2][nkv][P][HD]   (keys then values of a page)
//   block_table : [nseq, max_blocks] page ids, < 0 where a page was given back
//   row r attends to keys at positions <= positions[r] of sequence token_seq[r]
//   (and > positions[r] - window when window > 0).
//
// Scores, softmax and the weighted sum are 32-bit.  This file holds the general
// kernel that also is the true 32-bit path.
//
// Reference counterparts (cuda/src/kernels.cu): attention_qtile_kernel :1801 and
// attention_split_gqa_kernel :1874 with the online softmax of attn_tile_step
// :1460-1552; the causal rule :1583-1585.  The reference packs pages into a
// contiguous buffer first (crates/allpaca-core/src/kv_tier.rs:1317-1417); here the
// kernel reads the block table itself.
#include "common.cuh"
#include <float.h>

#ifndef AP_HEAD_DIM
#error "compile with -DAP_HEAD_DIM=<head size>"
#endif

#define HD AP_HEAD_DIM
#define ATT_THREADS 128
#define ATT_CHUNK 128
#define ACC_PER_THREAD ((HD + ATT_THREADS - 1) / ATT_THREADS)

AP_EXPORT int ap_attention_head_dim(void) { return HD; }

template <typename T>
__global__ void __launch_bounds__(ATT_THREADS)
attention_rows_kernel(const T* __restrict__ q, T* __restrict__ out, const T* __restrict__ cache,
                      const int* __restrict__ block_table, int max_blocks,
                      const int* __restrict__ token_seq, const int* __restrict__ positions,
                      int nh, int nkv, int P, size_t page_stride, float scale, int window) {
    __shared__ float q_s[HD];
    __shared__ float p_s[ATT_CHUNK];
    __shared__ float red[32];
    const int t = blockIdx.x, h = blockIdx.y;
    const int kvh = h / (nh / nkv);
    const int seq = token_seq[t];
    const int qpos = positions[t];
    const int* table = block_table + (size_t)seq * max_blocks;
    const T* qr = q + ((size_t)t * nh + h) * HD;
    for (int d = threadIdx.x; d < HD; d += ATT_THREADS) q_s[d] = ap_to_float(qr[d]);
    __syncthreads();

    const size_t head_off = (size_t)kvh * P * HD;          // keys of this head inside a page
    const size_t v_off = (size_t)nkv * P * HD + head_off;  // values of this head inside a page
    float acc[ACC_PER_THREAD];
#pragma unroll
    for (int i = 0; i < ACC_PER_THREAD; ++i) acc[i] = 0.f;
    float m = -FLT_MAX, l = 0.f;

    const int kfirst = (window > 0 && qpos - window + 1 > 0) ? qpos - window + 1 : 0;
    for (int c0 = kfirst; c0 <= qpos; c0 += ATT_CHUNK) {
        const int kpos = c0 + threadIdx.x;
        float s = -FLT_MAX;
        if (kpos <= qpos) {
            const int page = table[kpos / P];
            const T* kr = cache + (size_t)page * page_stride + head_off + (size_t)(kpos % P) * HD;
            float dot = 0.f;
#pragma unroll 8
            for (int d = 0; d < HD; ++d) dot = fmaf(q_s[d], ap_to_float(kr[d]), dot);
            s = dot * scale;
        }
        const float cmax = ap_block_max(s, red);
        const float m_new = fmaxf(m, cmax);
        const float p = (kpos <= qpos) ? expf(s - m_new) : 0.f;
        p_s[threadIdx.x] = p;
        const float csum = ap_block_sum(p, red);   // also publishes p_s (it synchronises)
        const float alpha = expf(m - m_new);       // 0 on the first chunk (m = -FLT_MAX)
        l = l * alpha + csum;
        m = m_new;
        const int nk = min(ATT_CHUNK, qpos - c0 + 1);
#pragma unroll
        for (int i = 0; i < ACC_PER_THREAD; ++i) {
            const int d = threadIdx.x + i * ATT_THREADS;
            if (d < HD) {
                float a = acc[i] * alpha;
                for (int j = 0; j < nk; ++j) {
                    const int kp = c0 + j;
                    const int page = table[kp / P];
                    const T* vr = cache + (size_t)page * page_stride + v_off + (size_t)(kp % P) * HD;
                    a = fmaf(p_s[j], ap_to_float(vr[d]), a);
                }
                acc[i] = a;
            }
        }
        __syncthreads();   // p_s is rewritten by the next chunk
    }
    T* o = out + ((size_t)t * nh + h) * HD;
    const float inv = 1.0f / l;
#pragma unroll
    for (int i = 0; i < ACC_PER_THREAD; ++i) {
        const int d = threadIdx.x + i * ATT_THREADS;
        if (d < HD) o[d] = ap_from_float<T>(acc[i] * inv);
    }
}

AP_EXPORT int ap_attention_rows(const void* q, void* out, const void* cache, int dtype,
                                const int* block_table, int max_blocks, const int* token_seq,
                                const int* positions, int T, int nh, int nkv, int hd, int P,
                                long long page_stride, float scale, int window, cudaStream_t stream) {
    AP_REQUIRE(hd == HD, "attention: this library was compiled for head size %d, not %d", HD, hd);
    AP_REQUIRE(T >= 0 && nh > 0 && nkv > 0 && nh % nkv == 0 && P > 0 && max_blocks > 0,
               "attention: bad sizes T=%d heads=%d kv_heads=%d page=%d", T, nh, nkv, P);
    AP_REQUIRE(nh <= 65535, "attention: %d heads exceed the grid", nh);
    if (T == 0) return AP_OK;
    dim3 grid(T, nh);
    if (dtype == AP_F32)
        attention_rows_kernel<float><<<grid, ATT_THREADS, 0, stream>>>(
            (const float*)q, (float*)out, (const float*)cache, block_table, max_blocks, token_seq,
            positions, nh, nkv, P, (size_t)page_stride, scale, window);
    else if (dtype == AP_BF16)
        attention_rows_kernel<bf16><<<grid, ATT_THREADS, 0, stream>>>(
            (const bf16*)q, (bf16*)out, (const bf16*)cache, block_table, max_blocks, token_seq,
            positions, nh, nkv, P, (size_t)page_stride, scale, window);
    else
        AP_REQUIRE(false, "attention: unknown dtype %d", dtype);
    AP_CHECK_LAUNCH("attention_rows");
    return AP_OK;
}
