// Row-wise kernels of the decoder: embedding gather, residual add fused with
// RMSNorm (and with the reduction of split-K partial sums), rotary embedding
// fused with the write of keys and values into cache pages, and the gated
// activation.  Sums, norms and angles are computed in 32-bit floats whatever the
// storage type.
//
// Reference counterparts (cuda/src/kernels.cu): embed_gather_kernel :1198,
// rmsnorm_kernel :1152 with residual_add_kernel :649, rope_qk_kernel :1244 with the
// page writes of crates/allpaca-core/src/kv_tier.rs:1101-1203, silu_mul_kernel :775.
#include "common.cuh"

// ---------------------------------------------------------------------------
// embedding gather: x[t, :] = table[token[t], :]   (32-bit residual stream)
// ---------------------------------------------------------------------------
template <typename TW>
__global__ void embed_gather_kernel(const int* __restrict__ tokens, const TW* __restrict__ table,
                                    float* __restrict__ x, int H, int V, float scale) {
    const int t = blockIdx.x;
    ap_pdl_trigger();
    ap_pdl_wait();
    int tok = tokens[t];
    // The host rejects tokens outside the vocabulary; the clamp keeps a corrupted
    // id from reading outside the table.
    tok = tok < 0 ? 0 : (tok >= V ? V - 1 : tok);
    const TW* src = table + (size_t)tok * H;
    float* dst = x + (size_t)t * H;
    // blockIdx.y walks the row in runs of blockDim.x elements (or of four times as many where the
    // row can be moved four elements at a time)
    if (sizeof(TW) == 2 && H % 4 == 0 && (((uintptr_t)table | (uintptr_t)x) & 15) == 0) {
        for (int i = (blockIdx.y * blockDim.x + threadIdx.x) * 4; i < H; i += gridDim.y * blockDim.x * 4) {
            const uint2 v = *reinterpret_cast<const uint2*>(reinterpret_cast<const bf16*>(src) + i);
            const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.x));
            const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&v.y));
            *reinterpret_cast<float4*>(dst + i) = make_float4(a.x * scale, a.y * scale, b.x * scale, b.y * scale);
        }
        return;
    }
    for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < H; i += gridDim.y * blockDim.x)
        dst[i] = ap_to_float(src[i]) * scale;
}

AP_EXPORT int ap_embed_gather(const int* tokens, const void* table, int table_dtype, float* x,
                              int T, int H, int V, float scale, cudaStream_t stream) {
    AP_REQUIRE(T >= 0 && H > 0 && V > 0, "embed_gather: bad sizes T=%d H=%d V=%d", T, H, V);
    if (T == 0) return AP_OK;
    const int threads = H >= 1024 ? 256 : 128;
    // few rows: several blocks to a row, so that a decode step's handful of rows is not one
    // long chain of loads per thread
    const dim3 grid(T, T <= 64 ? (H + 4 * threads - 1) / (4 * threads) : 1);
    // The first kernel of a step is launched in plain stream order: it starts when everything
    // before it on the stream has finished.  Kernels later in the step may therefore read what
    // earlier steps wrote (the cache) ahead of their own dependency wait.
    if (table_dtype == AP_F32)
        embed_gather_kernel<float><<<grid, threads, 0, stream>>>(tokens, (const float*)table, x, H, V, scale);
    else if (table_dtype == AP_BF16)
        embed_gather_kernel<bf16><<<grid, threads, 0, stream>>>(tokens, (const bf16*)table, x, H, V, scale);
    else
        AP_REQUIRE(false, "embed_gather: unknown table dtype %d", table_dtype);
    AP_CHECK_LAUNCH("embed_gather");
    return AP_OK;
}

// ---------------------------------------------------------------------------
// add + RMSNorm:  v = x[row] + sum_s delta[s, row];  out = v * rsqrt(mean(v^2) + eps) * w
//   rows == nullptr: every row t < T, and x[t] is overwritten with v.
//   rows != nullptr: only the listed rows are normed into out[r]; x is left as it is.
// One block per row, the row kept in shared memory between the two passes.
// ---------------------------------------------------------------------------
// The block is sized to the row (up to 1024 threads) and works on float4 when the width
// allows, so that a decode step's few rows still have many loads in flight.
template <typename TW, typename TO, int VEC>
__global__ void __launch_bounds__(1024)
add_rmsnorm_kernel(float* __restrict__ x, const float* __restrict__ delta, int S, size_t delta_stride,
                   const TW* __restrict__ w, float eps, TO* __restrict__ out,
                   const int* __restrict__ rows, int H) {
    extern __shared__ __align__(16) float row_buf[];
    __shared__ float red[32];
    const int r = blockIdx.x;
    ap_pdl_trigger();
    ap_pdl_wait();
    const int t = rows ? rows[r] : r;
    float* xr = x + (size_t)t * H;
    const float* dr = delta + (size_t)t * H;
    float ss = 0.f;
    for (int i = threadIdx.x * VEC; i < H; i += blockDim.x * VEC) {
        float v[VEC];
        if (VEC == 4) {
            const float4 a = *reinterpret_cast<const float4*>(xr + i);
            v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
#pragma unroll 4
            for (int s = 0; s < S; ++s) {
                const float4 d = *reinterpret_cast<const float4*>(dr + (size_t)s * delta_stride + i);
                v[0] += d.x; v[1] += d.y; v[2] += d.z; v[3] += d.w;
            }
        } else {
            v[0] = xr[i];
#pragma unroll 4
            for (int s = 0; s < S; ++s) v[0] += dr[(size_t)s * delta_stride + i];
        }
#pragma unroll
        for (int e = 0; e < VEC; ++e) {
            row_buf[i + e] = v[e];
            ss = fmaf(v[e], v[e], ss);
        }
        if (!rows && S > 0) {
            if (VEC == 4) *reinterpret_cast<float4*>(xr + i) = make_float4(v[0], v[1], v[2], v[3]);
            else xr[i] = v[0];
        }
    }
    ss = ap_block_sum(ss, red);
    const float inv = 1.0f / sqrtf(ss / (float)H + eps);
    TO* o = out + (size_t)r * H;
    if (VEC == 4 && sizeof(TO) == 2 && sizeof(TW) == 2 && (((uintptr_t)o | (uintptr_t)w) & 7) == 0) {
        // four bfloat16 results per thread in one 8-byte store
        for (int i = threadIdx.x * 4; i < H; i += blockDim.x * 4) {
            const float4 v = *reinterpret_cast<const float4*>(row_buf + i);
            const uint2 wv = *reinterpret_cast<const uint2*>(reinterpret_cast<const bf16*>(w) + i);
            const float2 w01 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&wv.x));
            const float2 w23 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&wv.y));
            uint2 ov;
            *reinterpret_cast<__nv_bfloat162*>(&ov.x) = __floats2bfloat162_rn(v.x * inv * w01.x, v.y * inv * w01.y);
            *reinterpret_cast<__nv_bfloat162*>(&ov.y) = __floats2bfloat162_rn(v.z * inv * w23.x, v.w * inv * w23.y);
            *reinterpret_cast<uint2*>(reinterpret_cast<bf16*>(o) + i) = ov;
        }
        return;
    }
    for (int i = threadIdx.x; i < H; i += blockDim.x)
        o[i] = ap_from_float<TO>(row_buf[i] * inv * ap_to_float(w[i]));
}

template <typename TW, typename TO>
static int launch_add_rmsnorm(float* x, const float* delta, int S, size_t delta_stride, const void* w,
                              float eps, void* out, const int* rows, int R, int H, cudaStream_t stream) {
    const size_t smem = (size_t)H * sizeof(float);
    const bool vec = (H % 4 == 0) && (((uintptr_t)x & 15) == 0) && (((uintptr_t)delta & 15) == 0) &&
                     (delta_stride % 4 == 0);
    auto kern = vec ? add_rmsnorm_kernel<TW, TO, 4> : add_rmsnorm_kernel<TW, TO, 1>;
    if (smem > 48 * 1024) {
        AP_REQUIRE(smem <= 200 * 1024, "rmsnorm: width %d does not fit the shared-memory row buffer", H);
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        AP_REQUIRE(e == cudaSuccess, "rmsnorm: cannot reserve %zu bytes of shared memory", smem);
    }
    const int per = vec ? 4 : 1;
    int threads = ((H + per - 1) / per + 31) / 32 * 32;
    threads = threads < 64 ? 64 : (threads > 1024 ? 1024 : threads);
    // many rows: smaller blocks, so that an SM holds several rows and one row's reduction
    // does not leave it idle
    if (R >= 4 * 148 && threads > 256) threads = 256;
    AP_CHECK_PDL_LAUNCH("add_rmsnorm", ap_launch_pdl(kern, dim3(R), dim3(threads), smem, stream, x, delta, S,
                                                     delta_stride, (const TW*)w, eps, (TO*)out, rows, H));
    return AP_OK;
}

AP_EXPORT int ap_add_rmsnorm(float* x, const float* delta, int S, long long delta_stride,
                             const void* weight, int w_dtype, float eps, void* out, int out_dtype,
                             const int* rows, int R, int H, cudaStream_t stream) {
    AP_REQUIRE(R >= 0 && H > 0 && S >= 0, "rmsnorm: bad sizes R=%d H=%d S=%d", R, H, S);
    AP_REQUIRE(S == 0 || delta != nullptr, "rmsnorm: S=%d partial sums but no buffer", S);
    if (R == 0) return AP_OK;
    if (w_dtype == AP_F32 && out_dtype == AP_F32)
        return launch_add_rmsnorm<float, float>(x, delta, S, delta_stride, weight, eps, out, rows, R, H, stream);
    if (w_dtype == AP_BF16 && out_dtype == AP_BF16)
        return launch_add_rmsnorm<bf16, bf16>(x, delta, S, delta_stride, weight, eps, out, rows, R, H, stream);
    if (w_dtype == AP_F32 && out_dtype == AP_BF16)
        return launch_add_rmsnorm<float, bf16>(x, delta, S, delta_stride, weight, eps, out, rows, R, H, stream);
    if (w_dtype == AP_BF16 && out_dtype == AP_F32)
        return launch_add_rmsnorm<bf16, float>(x, delta, S, delta_stride, weight, eps, out, rows, R, H, stream);
    AP_REQUIRE(false, "rmsnorm: unknown dtypes w=%d out=%d", w_dtype, out_dtype);
}

// ---------------------------------------------------------------------------
// residual add alone: x[t] += sum_s delta[s, t]   (used where no norm follows)
// ---------------------------------------------------------------------------
__global__ void residual_add_kernel(float* __restrict__ x, const float* __restrict__ delta, int S,
                                    size_t delta_stride, size_t n) {
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        float v = x[i];
        for (int s = 0; s < S; ++s) v += delta[(size_t)s * delta_stride + i];
        x[i] = v;
    }
}

AP_EXPORT int ap_residual_add(float* x, const float* delta, int S, long long delta_stride,
                              long long n, cudaStream_t stream) {
    AP_REQUIRE(n >= 0 && S >= 0, "residual_add: bad sizes");
    if (n == 0 || S == 0) return AP_OK;
    const int threads = 256;
    long long blocks = (n + threads - 1) / threads;
    if (blocks > 148 * 16) blocks = 148 * 16;
    residual_add_kernel<<<(int)blocks, threads, 0, stream>>>(x, delta, S, (size_t)delta_stride, (size_t)n);
    AP_CHECK_LAUNCH("residual_add");
    return AP_OK;
}

// ---------------------------------------------------------------------------
// bias and logit transforms, for decoders that have them (none on the plain Llama path):
//   bias_add:        out[t, n] += bias[n]                       (out in 32-bit or bfloat16)
//   logit_transform: z = (logit + bias[n]) * scale;  z = cap * tanh(z / cap) when cap > 0
// ---------------------------------------------------------------------------
template <typename TO, typename TB>
__global__ void bias_add_kernel(TO* __restrict__ out, const TB* __restrict__ bias, size_t n, int N) {
    ap_pdl_trigger();
    ap_pdl_wait();
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
        out[i] = ap_from_float<TO>(ap_to_float(out[i]) + ap_to_float(bias[i % N]));
}

AP_EXPORT int ap_bias_add(void* out, int out_dtype, const void* bias, int bias_dtype, int T, int N,
                          cudaStream_t stream) {
    AP_REQUIRE(T >= 0 && N > 0 && out && bias, "bias_add: bad arguments T=%d N=%d", T, N);
    if (T == 0) return AP_OK;
    const size_t n = (size_t)T * N;
    const int threads = 256;
    size_t blocks = (n + threads - 1) / threads;
    if (blocks > 148 * 16) blocks = 148 * 16;
#define LAUNCH(TO, TB)                                                                                    \
    AP_CHECK_PDL_LAUNCH("bias_add", ap_launch_pdl(bias_add_kernel<TO, TB>, dim3((unsigned)blocks), dim3(threads), 0, \
                                                  stream, (TO*)out, (const TB*)bias, n, N))
    if (out_dtype == AP_F32 && bias_dtype == AP_F32) LAUNCH(float, float);
    else if (out_dtype == AP_F32 && bias_dtype == AP_BF16) LAUNCH(float, bf16);
    else if (out_dtype == AP_BF16 && bias_dtype == AP_F32) LAUNCH(bf16, float);
    else if (out_dtype == AP_BF16 && bias_dtype == AP_BF16) LAUNCH(bf16, bf16);
    else AP_REQUIRE(false, "bias_add: unknown dtypes out=%d bias=%d", out_dtype, bias_dtype);
#undef LAUNCH
    return AP_OK;
}

template <typename TB>
__global__ void logit_transform_kernel(float* __restrict__ logits, const TB* __restrict__ bias, size_t n, int V,
                                       float scale, float cap) {
    ap_pdl_trigger();
    ap_pdl_wait();
    for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        float z = logits[i];
        if (bias) z += ap_to_float(bias[i % V]);
        z *= scale;
        if (cap > 0.f) z = cap * tanhf(z / cap);
        logits[i] = z;
    }
}

AP_EXPORT int ap_logit_transform(float* logits, const void* bias, int bias_dtype, int R, int V, float scale,
                                 float softcap, cudaStream_t stream) {
    AP_REQUIRE(R >= 0 && V > 0 && logits, "logit_transform: bad arguments R=%d V=%d", R, V);
    if (R == 0) return AP_OK;
    const size_t n = (size_t)R * V;
    const int threads = 256;
    size_t blocks = (n + threads - 1) / threads;
    if (blocks > 148 * 16) blocks = 148 * 16;
    if (bias == nullptr || bias_dtype == AP_F32)
        AP_CHECK_PDL_LAUNCH("logit_transform", ap_launch_pdl(logit_transform_kernel<float>, dim3((unsigned)blocks),
                                                             dim3(threads), 0, stream, logits, (const float*)bias, n,
                                                             V, scale, softcap));
    else if (bias_dtype == AP_BF16)
        AP_CHECK_PDL_LAUNCH("logit_transform", ap_launch_pdl(logit_transform_kernel<bf16>, dim3((unsigned)blocks),
                                                             dim3(threads), 0, stream, logits, (const bf16*)bias, n,
                                                             V, scale, softcap));
    else
        AP_REQUIRE(false, "logit_transform: unknown bias dtype %d", bias_dtype);
    return AP_OK;
}

// ---------------------------------------------------------------------------
// rotary embedding of Q and K + write of K and V into cache pages.
//   in:  [S, T, (nh + 2*nkv) * hd]  (S partial sums in 32-bit, or S == 1 in TI)
//   q_out: [T, nh*hd]
//   cache (one layer): [page][2][nkv][P][hd]; the page of a row is
//       block_table[token_seq[t]][pos / P], its slot pos % P; cache == nullptr: store nothing
//   cos_sin: [T][hd/2] (cos, sin) pairs from rope_table_kernel, or nullptr for no rotation
//   pairing 0: pairs (i, i + hd/2)   (checkpoints in the Hugging Face layout)
//   pairing 1: pairs (2i, 2i + 1)    (checkpoints whose Q/K rows were permuted)
//   pairing 2: the input holds the pair (i, i + hd/2) side by side at (2i, 2i + 1) (the rows of
//              the projection's weight were interleaved so); the output is in the usual order
// ---------------------------------------------------------------------------
template <typename TI>
__device__ __forceinline__ float load_partial(const TI* in, int S, size_t stride, size_t idx) {
    float v = ap_to_float(in[idx]);
#pragma unroll 4
    for (int s = 1; s < S; ++s) v += ap_to_float(in[(size_t)s * stride + idx]);
    return v;
}

// cos and sin of pos * inv_freq[i] for every row of the step, computed once and shared by
// all layers with the same rotation: table[t][i] = (cos, sin).  The angle is a 32-bit
// product; sincosf is the accurate (not the fast-math) routine.
__global__ void rope_table_kernel(const int* __restrict__ positions, const float* __restrict__ inv_freq,
                                  float2* __restrict__ table, int half) {
    const int t = blockIdx.x;
    ap_pdl_trigger();
    ap_pdl_wait();
    const float pos = (float)positions[t];
    for (int i = threadIdx.x; i < half; i += blockDim.x) {
        float sn, cs;
        sincosf(pos * inv_freq[i], &sn, &cs);
        table[(size_t)t * half + i] = make_float2(cs, sn);
    }
}

AP_EXPORT int ap_rope_table(const int* positions, const float* inv_freq, float* table, int T, int half,
                            cudaStream_t stream) {
    AP_REQUIRE(T >= 0 && half > 0, "rope_table: bad sizes T=%d half=%d", T, half);
    if (T == 0) return AP_OK;
    AP_CHECK_PDL_LAUNCH("rope_table", ap_launch_pdl(rope_table_kernel, dim3(T), dim3(half < 128 ? 64 : 128), 0,
                                                    stream, positions, inv_freq, (float2*)table, half));
    return AP_OK;
}

// ---------------------------------------------------------------------------
// A page is first written at its slot 0 (a request's positions are contiguous).  Before the
// layers of a step run, the slots of such a page behind the last one this step writes are
// cleared in every run of the cache group: the attention kernels load whole pages and weigh
// what lies behind a row's position with a probability of exactly zero, which only gives zero
// if it is finite, and a page that was given back keeps its last owner's values, whatever they
// were.  pages: [runs][num_pages][outer][P][inner] of 1-, 2- or 4-byte elements.
// ---------------------------------------------------------------------------
template <typename T>
__global__ void clear_page_tails_kernel(T* __restrict__ pages, size_t run_stride, size_t page_stride, int runs,
                                        int outer, int P, int inner, const int* __restrict__ positions,
                                        const int* __restrict__ token_seq, const int* __restrict__ block_table,
                                        int max_blocks, const int* __restrict__ context_lens) {
    const int t = blockIdx.x;
    const int pos = positions[t];
    if (pos % P != 0) return;
    const int seq = token_seq[t];
    const int page = block_table[(size_t)seq * max_blocks + pos / P];
    const int first = context_lens[seq] - pos;          // slots 0 .. first-1 are written by this step's rows
    if (page < 0 || first >= P) return;
    const size_t per_plane = (size_t)(P - first) * inner;  // the cleared slots of one plane are contiguous
    const size_t total = (size_t)runs * outer * per_plane;
    for (size_t i = blockIdx.y * (size_t)blockDim.x + threadIdx.x; i < total; i += (size_t)gridDim.y * blockDim.x) {
        const size_t plane = i / per_plane, e = i - plane * per_plane;
        const size_t run = plane / outer, o = plane - run * outer;
        pages[run * run_stride + (size_t)page * page_stride + (o * P + first) * inner + e] = T(0);
    }
}

AP_EXPORT int ap_clear_page_tails(void* pages, int elem_bytes, long long run_stride, long long page_stride, int runs,
                                  int outer, int P, int inner, const int* positions, const int* token_seq,
                                  const int* block_table, int max_blocks, const int* context_lens, int T,
                                  cudaStream_t stream) {
    AP_REQUIRE(T >= 0 && runs > 0 && outer > 0 && P > 0 && inner > 0 && max_blocks > 0,
               "clear_page_tails: bad sizes runs=%d outer=%d page=%d inner=%d", runs, outer, P, inner);
    AP_REQUIRE(pages && positions && token_seq && block_table && context_lens, "clear_page_tails: a pointer is missing");
    if (T == 0) return AP_OK;
    // elements are cleared in the widest unit that divides a slot's bytes (zero is zero in every type)
    long long unit = elem_bytes;
    while (unit < 8 && ((long long)inner * elem_bytes) % (unit * 2) == 0 && ((uintptr_t)pages % (unit * 2)) == 0 &&
           (run_stride * elem_bytes) % (unit * 2) == 0 && (page_stride * elem_bytes) % (unit * 2) == 0)
        unit *= 2;
    const int scale = (int)(unit / elem_bytes);
    dim3 grid(T, 8);
#define LAUNCH(TT)                                                                                            \
    clear_page_tails_kernel<TT><<<grid, 256, 0, stream>>>((TT*)pages, (size_t)(run_stride / scale),          \
                                                          (size_t)(page_stride / scale), runs, outer, P,     \
                                                          inner / scale, positions, token_seq, block_table,   \
                                                          max_blocks, context_lens)
    if (unit == 8) LAUNCH(unsigned long long);
    else if (unit == 4) LAUNCH(unsigned int);
    else if (unit == 2) LAUNCH(unsigned short);
    else if (unit == 1) LAUNCH(unsigned char);
    else AP_REQUIRE(false, "clear_page_tails: elements of %d bytes", elem_bytes);
#undef LAUNCH
    AP_CHECK_LAUNCH("clear_page_tails");
    return AP_OK;
}

// One thread per pair of elements: (nh + nkv) * half rotated pairs, then nkv * half pairs of V.
#define ROPE_THREADS 256
template <typename TI, typename TO>
__global__ void __launch_bounds__(ROPE_THREADS)
rope_kv_store_kernel(const TI* __restrict__ in, int S, size_t in_stride,
                     TO* __restrict__ q_out, TO* __restrict__ cache,
                     const int* __restrict__ positions,
                     const int* __restrict__ token_seq,
                     const int* __restrict__ block_table, int max_blocks,
                     const float2* __restrict__ cos_sin, int pairing,
                     int nh, int nkv, int hd, int P, size_t page_stride) {
    const int t = blockIdx.x;
    const int half = hd >> 1;
    const int item = blockIdx.y * ROPE_THREADS + threadIdx.x;
    ap_pdl_trigger();
    ap_pdl_wait();
    const int rot_pairs = (nh + nkv) * half;
    const int v_pairs = cache ? nkv * half : 0;
    const size_t row = (size_t)t * (nh + 2 * nkv) * hd;
    int page = -1, off = 0;
    if (cache) {
        const int ipos = positions[t];
        page = block_table[(size_t)token_seq[t] * max_blocks + ipos / P];
        off = ipos % P;
    }
    if (item >= rot_pairs + v_pairs) return;
    if (item < rot_pairs) {
        const int head = item / half, i = item - head * half;
        if (head >= nh && page < 0) return;
        // where the pair lies in the input, and where it goes (pairing 2: neighbours in, halves out)
        const int ia = pairing == 1 ? 2 * i : i;
        const int ib = pairing == 1 ? 2 * i + 1 : i + half;
        const int ia_in = pairing == 0 ? i : 2 * i;
        const int ib_in = pairing == 0 ? i + half : 2 * i + 1;
        const size_t base = row + (size_t)head * hd;
        // partial sums are rounded to the storage type once they are complete
        const float a = ap_to_float(ap_from_float<TO>(load_partial(in, S, in_stride, base + ia_in)));
        const float b = ap_to_float(ap_from_float<TO>(load_partial(in, S, in_stride, base + ib_in)));
        float ra = a, rb = b;
        if (cos_sin) {
            const float2 cs = cos_sin[(size_t)t * half + i];
            ra = a * cs.x - b * cs.y;
            rb = a * cs.y + b * cs.x;
        }
        TO* dst = head < nh ? q_out + (size_t)t * nh * hd + (size_t)head * hd
                            : cache + (size_t)page * page_stride + ((size_t)(head - nh) * P + off) * hd;
        dst[ia] = ap_from_float<TO>(ra);
        dst[ib] = ap_from_float<TO>(rb);
    } else if (page >= 0) {
        const int e = (item - rot_pairs) * 2;              // hd is even: a pair never straddles heads
        const int kh = e / hd, d = e - kh * hd;
        const size_t vbase = row + (size_t)(nh + nkv) * hd + e;
        TO* dst = cache + (size_t)page * page_stride + (size_t)nkv * P * hd + ((size_t)kh * P + off) * hd + d;
        dst[0] = ap_from_float<TO>(load_partial(in, S, in_stride, vbase));
        dst[1] = ap_from_float<TO>(load_partial(in, S, in_stride, vbase + 1));
    }
}

// bfloat16, single input slice, half-split pairing: one thread rotates 8 pairs (elements
// i..i+7 with i+half..i+half+7) or copies 8 elements of V, in 16-byte accesses.
__global__ void __launch_bounds__(ROPE_THREADS)
rope_kv_store_bf16x8_kernel(const bf16* __restrict__ in, bf16* __restrict__ q_out, bf16* __restrict__ cache,
                            const int* __restrict__ positions, const int* __restrict__ token_seq,
                            const int* __restrict__ block_table, int max_blocks,
                            const float2* __restrict__ cos_sin, int nh, int nkv, int hd, int P,
                            size_t page_stride, int interleaved) {
    const int t = blockIdx.x;
    const int half = hd >> 1, h8 = half >> 3;             // groups of 8 pairs per head
    const int item = blockIdx.y * ROPE_THREADS + threadIdx.x;
    ap_pdl_trigger();
    ap_pdl_wait();
    const int rot_items = (nh + nkv) * h8;
    const int v_items = cache ? nkv * (hd >> 3) : 0;
    const size_t row = (size_t)t * (nh + 2 * nkv) * hd;
    int page = -1, off = 0;
    if (cache) {
        const int ipos = positions[t];
        page = block_table[(size_t)token_seq[t] * max_blocks + ipos / P];
        off = ipos % P;
    }
    if (item >= rot_items + v_items) return;
    if (item < rot_items) {
        const int head = item / h8, i = (item - head * h8) * 8;
        if (head >= nh && page < 0) return;
        const bf16* src = in + row + (size_t)head * hd;
        uint4 a4, b4;
        if (interleaved) {
            // elements 2i .. 2i+15 hold the pairs (a_k, b_k) side by side: split them
            const uint4 lo = *reinterpret_cast<const uint4*>(src + 2 * i);
            const uint4 hi = *reinterpret_cast<const uint4*>(src + 2 * i + 8);
            const uint32_t w[8] = {lo.x, lo.y, lo.z, lo.w, hi.x, hi.y, hi.z, hi.w};
            uint32_t aw[4], bw[4];
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                aw[k] = __byte_perm(w[2 * k], w[2 * k + 1], 0x5410);      // low halves: a_2k, a_2k+1
                bw[k] = __byte_perm(w[2 * k], w[2 * k + 1], 0x7632);      // high halves: b_2k, b_2k+1
            }
            a4 = make_uint4(aw[0], aw[1], aw[2], aw[3]);
            b4 = make_uint4(bw[0], bw[1], bw[2], bw[3]);
        } else {
            a4 = *reinterpret_cast<const uint4*>(src + i);
            b4 = *reinterpret_cast<const uint4*>(src + i + half);
        }
        const __nv_bfloat162* a2 = reinterpret_cast<const __nv_bfloat162*>(&a4);
        const __nv_bfloat162* b2 = reinterpret_cast<const __nv_bfloat162*>(&b4);
        uint4 ra4 = a4, rb4 = b4;
        if (cos_sin) {
            __nv_bfloat162* ra2 = reinterpret_cast<__nv_bfloat162*>(&ra4);
            __nv_bfloat162* rb2 = reinterpret_cast<__nv_bfloat162*>(&rb4);
            const float4* cs = reinterpret_cast<const float4*>(cos_sin + (size_t)t * half + i);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float4 c = cs[k];                   // (cos, sin) of pairs 2k and 2k+1
                const float2 a = __bfloat1622float2(a2[k]), b = __bfloat1622float2(b2[k]);
                ra2[k] = __floats2bfloat162_rn(a.x * c.x - b.x * c.y, a.y * c.z - b.y * c.w);
                rb2[k] = __floats2bfloat162_rn(a.x * c.y + b.x * c.x, a.y * c.w + b.y * c.z);
            }
        }
        bf16* dst = head < nh ? q_out + (size_t)t * nh * hd + (size_t)head * hd
                              : cache + (size_t)page * page_stride + ((size_t)(head - nh) * P + off) * hd;
        *reinterpret_cast<uint4*>(dst + i) = ra4;
        *reinterpret_cast<uint4*>(dst + i + half) = rb4;
    } else if (page >= 0) {
        const int e = (item - rot_items) * 8;
        const int kh = e / hd, d = e - kh * hd;
        const uint4 v4 = *reinterpret_cast<const uint4*>(in + row + (size_t)(nh + nkv) * hd + e);
        *reinterpret_cast<uint4*>(cache + (size_t)page * page_stride + (size_t)nkv * P * hd +
                                  ((size_t)kh * P + off) * hd + d) = v4;
    }
}

AP_EXPORT int ap_rope_kv_store(const void* in, int in_dtype, int S, long long in_stride, void* q_out,
                               void* cache, int act_dtype, const int* positions, const int* token_seq,
                               const int* block_table, int max_blocks, const float* cos_sin, int pairing,
                               int T, int nh, int nkv, int hd, int P, long long page_stride,
                               cudaStream_t stream) {
    AP_REQUIRE(T >= 0 && nh > 0 && nkv >= 0 && hd > 0 && (hd % 2) == 0 && S >= 1,
               "rope_kv_store: bad sizes T=%d heads=%d kv_heads=%d head_dim=%d S=%d", T, nh, nkv, hd, S);
    AP_REQUIRE(pairing >= 0 && pairing <= 2, "rope_kv_store: unknown pairing %d", pairing);
    AP_REQUIRE(cache == nullptr || (P > 0 && page_stride >= 2LL * nkv * P * hd),
               "rope_kv_store: page stride %lld is below one page of keys and values", page_stride);
    AP_REQUIRE(cache == nullptr || (token_seq && block_table && max_blocks > 0),
               "rope_kv_store: storing needs the block table and the rows' sequences");
    if (T == 0) return AP_OK;
    if (in_dtype == AP_BF16 && act_dtype == AP_BF16 && S == 1 && pairing != 1 && hd % 16 == 0 &&
        ((uintptr_t)in & 15) == 0 && ((uintptr_t)q_out & 15) == 0 && ((uintptr_t)cache & 15) == 0 &&
        page_stride % 8 == 0 && ((uintptr_t)cos_sin & 15) == 0) {
        const int items8 = (nh + nkv) * (hd / 16) + (cache ? nkv * (hd / 8) : 0);
        dim3 grid8(T, (items8 + ROPE_THREADS - 1) / ROPE_THREADS);
        AP_REQUIRE(grid8.y <= 65535, "rope_kv_store: too many heads for the grid");
        AP_CHECK_PDL_LAUNCH("rope_kv_store", ap_launch_pdl(
            rope_kv_store_bf16x8_kernel, grid8, dim3(ROPE_THREADS), 0, stream, (const bf16*)in, (bf16*)q_out,
            (bf16*)cache, positions, token_seq, block_table, max_blocks, (const float2*)cos_sin, nh, nkv, hd, P,
            (size_t)page_stride, pairing == 2 ? 1 : 0));
        return AP_OK;
    }
    const int items = (nh + nkv) * (hd / 2) + (cache ? nkv * (hd / 2) : 0);
    dim3 grid(T, (items + ROPE_THREADS - 1) / ROPE_THREADS);
    AP_REQUIRE(grid.y <= 65535, "rope_kv_store: too many heads for the grid");
#define LAUNCH(TI, TO)                                                                              \
    AP_CHECK_PDL_LAUNCH("rope_kv_store", ap_launch_pdl(                                             \
        rope_kv_store_kernel<TI, TO>, grid, dim3(ROPE_THREADS), 0, stream,                          \
        (const TI*)in, S, (size_t)in_stride, (TO*)q_out, (TO*)cache, positions, token_seq,         \
        block_table, max_blocks, (const float2*)cos_sin, pairing, nh, nkv, hd, P, (size_t)page_stride))
    if (in_dtype == AP_F32 && act_dtype == AP_F32) LAUNCH(float, float);
    else if (in_dtype == AP_F32 && act_dtype == AP_BF16) LAUNCH(float, bf16);
    else if (in_dtype == AP_BF16 && act_dtype == AP_BF16) {
        AP_REQUIRE(S == 1, "rope_kv_store: partial sums must be 32-bit");
        LAUNCH(bf16, bf16);
    } else AP_REQUIRE(false, "rope_kv_store: unsupported dtypes in=%d act=%d", in_dtype, act_dtype);
#undef LAUNCH
    return AP_OK;
}

// ---------------------------------------------------------------------------
// gated activation: out[t, j] = silu(g) * u,  g = in[t, j], u = in[t, I + j]; or, with gate and up
// columns alternating (`pairs`), g = in[t, 2j], u = in[t, 2j + 1]
// ---------------------------------------------------------------------------
template <typename TI, typename TO>
__global__ void swiglu_kernel(const TI* __restrict__ in, int S, size_t in_stride, TO* __restrict__ out,
                              int T, int I, int pairs) {
    const size_t n = (size_t)T * I;
    ap_pdl_trigger();
    ap_pdl_wait();
    for (size_t e = blockIdx.x * (size_t)blockDim.x + threadIdx.x; e < n; e += (size_t)gridDim.x * blockDim.x) {
        const size_t t = e / I, j = e - t * I;
        const size_t base = t * 2 * (size_t)I;
        const float g = ap_to_float(ap_from_float<TO>(load_partial(in, S, in_stride, pairs ? base + 2 * j : base + j)));
        const float u = ap_to_float(ap_from_float<TO>(load_partial(in, S, in_stride, pairs ? base + 2 * j + 1 : base + I + j)));
        const float a = g / (1.0f + expf(-g));
        out[e] = ap_from_float<TO>(a * u);
    }
}

// bfloat16 in and out, 8 elements (16 bytes) per thread
template <bool PAIRS>
__global__ void swiglu_bf16x8_kernel(const bf16* __restrict__ in, bf16* __restrict__ out, int T, int I) {
    const size_t n8 = (size_t)T * (I / 8);
    ap_pdl_trigger();
    ap_pdl_wait();
    for (size_t e = blockIdx.x * (size_t)blockDim.x + threadIdx.x; e < n8; e += (size_t)gridDim.x * blockDim.x) {
        const size_t t = e / (I / 8), j = (e - t * (I / 8)) * 8;
        // the 16 values that make these 8 outputs: two separate runs of 8, or one run of 16 pairs
        const uint4 g4 = *reinterpret_cast<const uint4*>(in + t * 2 * (size_t)I + (PAIRS ? 2 * j : j));
        const uint4 u4 = *reinterpret_cast<const uint4*>(in + t * 2 * (size_t)I + (PAIRS ? 2 * j + 8 : I + j));
        const __nv_bfloat162* g2 = reinterpret_cast<const __nv_bfloat162*>(&g4);
        const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&u4);
        uint4 o4;
        __nv_bfloat162* o2 = reinterpret_cast<__nv_bfloat162*>(&o4);
#pragma unroll
        for (int k = 0; k < 4; ++k) {
            float2 g, u;
            if (PAIRS) {
                // every bfloat162 is one (gate, up) pair; outputs 2k and 2k+1 come from pairs 2k, 2k+1
                const float2 p0 = __bfloat1622float2(k < 2 ? g2[2 * k] : u2[2 * k - 4]);
                const float2 p1 = __bfloat1622float2(k < 2 ? g2[2 * k + 1] : u2[2 * k - 3]);
                g = make_float2(p0.x, p1.x);
                u = make_float2(p0.y, p1.y);
            } else {
                g = __bfloat1622float2(g2[k]);
                u = __bfloat1622float2(u2[k]);
            }
            o2[k] = __floats2bfloat162_rn(g.x / (1.0f + expf(-g.x)) * u.x, g.y / (1.0f + expf(-g.y)) * u.y);
        }
        *reinterpret_cast<uint4*>(out + t * (size_t)I + j) = o4;
    }
}

AP_EXPORT int ap_swiglu(const void* in, int in_dtype, int S, long long in_stride, void* out, int out_dtype,
                        int T, int I, int pairs, cudaStream_t stream) {
    AP_REQUIRE(T >= 0 && I > 0 && S >= 1, "swiglu: bad sizes T=%d I=%d S=%d", T, I, S);
    if (T == 0) return AP_OK;
    const int threads = 256;
    long long blocks = ((long long)T * I + threads - 1) / threads;
    if (blocks > 148 * 32) blocks = 148 * 32;
    if (in_dtype == AP_BF16 && out_dtype == AP_BF16 && S == 1 && I % 8 == 0 && ((uintptr_t)in & 15) == 0 &&
        ((uintptr_t)out & 15) == 0) {
        long long b8 = ((long long)T * (I / 8) + threads - 1) / threads;
        if (b8 > 148 * 32) b8 = 148 * 32;
        if (pairs)
            AP_CHECK_PDL_LAUNCH("swiglu", ap_launch_pdl(swiglu_bf16x8_kernel<true>, dim3((unsigned)b8), dim3(threads), 0,
                                                        stream, (const bf16*)in, (bf16*)out, T, I));
        else
            AP_CHECK_PDL_LAUNCH("swiglu", ap_launch_pdl(swiglu_bf16x8_kernel<false>, dim3((unsigned)b8), dim3(threads), 0,
                                                        stream, (const bf16*)in, (bf16*)out, T, I));
        return AP_OK;
    }
#define LAUNCH(TI, TO) \
    AP_CHECK_PDL_LAUNCH("swiglu", ap_launch_pdl(swiglu_kernel<TI, TO>, dim3((unsigned)blocks), dim3(threads), 0, stream, \
                                                (const TI*)in, S, (size_t)in_stride, (TO*)out, T, I, pairs))
    if (in_dtype == AP_F32 && out_dtype == AP_F32) LAUNCH(float, float);
    else if (in_dtype == AP_F32 && out_dtype == AP_BF16) LAUNCH(float, bf16);
    else if (in_dtype == AP_BF16 && out_dtype == AP_BF16) {
        AP_REQUIRE(S == 1, "swiglu: partial sums must be 32-bit");
        LAUNCH(bf16, bf16);
    } else AP_REQUIRE(false, "swiglu: unsupported dtypes in=%d out=%d", in_dtype, out_dtype);
#undef LAUNCH
    return AP_OK;
}
