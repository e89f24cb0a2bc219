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

template <int BN> struct TileCfg {
    static constexpr int kStages = BN >= 256 ? 4 : (BN >= 128 ? 6 : 4);
    static constexpr int kBBytes = BN * TILE_K * 2;
    static constexpr int kStageBytes = A_TILE_BYTES + kBBytes;
    static constexpr int kTmemCols = BN < 32 ? 32 : BN;
    static constexpr int kSmemBytes = kStages * kStageBytes + 1024 /*alignment*/ + 256 /*barriers*/;
};

template <int BN, typename TO>
__global__ void __launch_bounds__(192)
gemm_tc_kernel(const __grid_constant__ CUtensorMap tmap_w, const __grid_constant__ CUtensorMap tmap_a,
               TO* __restrict__ out, int M, int N, int K, long long ldc, int kb_per_split,
               long long split_stride) {
    using Cfg = TileCfg<BN>;
    constexpr int STAGES = Cfg::kStages;
    extern __shared__ uint8_t smem_raw[];
    uint8_t* smem = (uint8_t*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint8_t* w_tiles = smem;
    uint8_t* a_tiles = smem + STAGES * A_TILE_BYTES;
    uint64_t* full = (uint64_t*)(smem + STAGES * Cfg::kStageBytes);
    uint64_t* empty = full + STAGES;
    uint64_t* accum = empty + STAGES;
    uint32_t* tmem_slot = (uint32_t*)(accum + 1);
    volatile int* abort_flag = (volatile int*)(tmem_slot + 1);

    // once a wait has expired anywhere, later CTAs do nothing: the product is void anyway
    if (*(volatile int*)&g_tc_status != 0) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * TILE_W;
    const int m0 = blockIdx.y * BN;
    const int kb_total = (K + TILE_K - 1) / TILE_K;
    const int kb0 = blockIdx.z * kb_per_split;
    const int kb1 = min(kb_total, kb0 + kb_per_split);
    const int nkb = max(0, kb1 - kb0);
    out += (size_t)blockIdx.z * split_stride;

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
        const int n = n0 + q * 32 + lane;
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
        if (have) {
#pragma unroll 1
            for (int c = 0; c < BN; c += 16) {
                if (m0 + c >= M) break;
                uint32_t v[16];
                tc::tmem_ld_x16(tmem_base + ((uint32_t)(q * 32) << 16) + (uint32_t)c, v);
                tc::tmem_ld_wait();
                if (n < N) {
#pragma unroll
                    for (int j = 0; j < 16; ++j) {
                        const int m = m0 + c + j;
                        if (m < M) out[(size_t)m * ldc + n] = ap_from_float<TO>(__uint_as_float(v[j]));
                    }
                }
            }
        } else if (nkb == 0 && n < N) {
            for (int c = 0; c < BN; ++c) {
                const int m = m0 + c;
                if (m < M) out[(size_t)m * ldc + n] = ap_from_float<TO>(0.f);
            }
        }
    }
    tc::fence_before_sync();
    __syncthreads();
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
// weight tiles to keep every SM loading, so K is split until about two CTAs per SM exist,
// as long as the partial sums stay small beside the weight itself.
AP_EXPORT int ap_gemm_tc_plan(int M, int N, int K) {
    if (M <= 0 || N <= 0 || K <= 0) return 1;
    const int kb_total = (K + TILE_K - 1) / TILE_K;
    const int bn = pick_bn(M);
    const long long tiles = (long long)((N + TILE_W - 1) / TILE_W) * ((M + bn - 1) / bn);
    if (M > 64 || tiles >= 148) return 1;
    int ns = (int)((296 + tiles - 1) / tiles);
    ns = min(ns, kb_total / 4);
    ns = min(ns, max(1, K / (16 * M)));
    ns = min(ns, 16);
    if (ns < 1) ns = 1;
    const int per = (kb_total + ns - 1) / ns;
    return (kb_total + per - 1) / per;
}

template <int BN, typename TO>
static int launch_tc(const CUtensorMap& mw, const CUtensorMap& ma, void* out, int M, int N, int K,
                     long long ldc, int nsplit, long long split_stride, cudaStream_t stream) {
    using Cfg = TileCfg<BN>;
    auto kern = gemm_tc_kernel<BN, TO>;
    static bool configured = false;
    if (!configured) {
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::kSmemBytes);
        AP_REQUIRE(e == cudaSuccess, "gemm_tc: cannot reserve %d bytes of shared memory: %s", Cfg::kSmemBytes,
                   cudaGetErrorString(e));
        configured = true;
    }
    const int kb_total = (K + TILE_K - 1) / TILE_K;
    const int per = (kb_total + nsplit - 1) / nsplit;
    dim3 grid((N + TILE_W - 1) / TILE_W, (M + BN - 1) / BN, nsplit);
    kern<<<grid, 192, Cfg::kSmemBytes, stream>>>(mw, ma, (TO*)out, M, N, K, ldc, per, split_stride);
    AP_CHECK_LAUNCH("gemm_tc");
    return AP_OK;
}

AP_EXPORT int ap_gemm_tc(const void* a, const void* w, void* out, int out_dtype, int M, int N, int K,
                         long long lda, long long ldw, long long ldc, int nsplit, long long split_stride,
                         cudaStream_t stream) {
    AP_REQUIRE(M >= 0 && N > 0 && K > 0, "gemm_tc: bad sizes M=%d N=%d K=%d", M, N, K);
    if (M == 0) return AP_OK;
    AP_REQUIRE(K % 8 == 0 && lda % 8 == 0 && ldw % 8 == 0,
               "gemm_tc: K=%d and the leading dimensions must be multiples of 8 (16-byte rows for TMA)", K);
    AP_REQUIRE(((uintptr_t)a & 15) == 0 && ((uintptr_t)w & 15) == 0, "gemm_tc: operands must be 16-byte aligned");
    AP_REQUIRE(lda >= K && ldw >= K && ldc >= N, "gemm_tc: a leading dimension is below its row length");
    const int kb_total = (K + TILE_K - 1) / TILE_K;
    AP_REQUIRE(nsplit >= 1 && nsplit <= kb_total && nsplit <= 65535, "gemm_tc: cannot split K=%d into %d", K, nsplit);
    AP_REQUIRE(nsplit == 1 || out_dtype == AP_F32, "gemm_tc: partial sums must be 32-bit");
    AP_REQUIRE((long long)(nsplit - 1) * ((kb_total + nsplit - 1) / nsplit) < kb_total,
               "gemm_tc: %d slices leave an empty one for K=%d", nsplit, K);
    const int bn = pick_bn(M);
    AP_REQUIRE((M + bn - 1) / bn <= 65535, "gemm_tc: %d rows exceed the grid", M);
    CUtensorMap mw, ma;
    AP_REQUIRE(make_map(&mw, w, N, K, ldw, TILE_W), "gemm_tc: cannot encode the weight's tensor map");
    AP_REQUIRE(make_map(&ma, a, M, K, lda, bn), "gemm_tc: cannot encode the activations' tensor map");
#define GO(BN)                                                                                          \
    return out_dtype == AP_F32                                                                          \
               ? launch_tc<BN, float>(mw, ma, out, M, N, K, ldc, nsplit, split_stride, stream)          \
               : launch_tc<BN, bf16>(mw, ma, out, M, N, K, ldc, nsplit, split_stride, stream)
    AP_REQUIRE(out_dtype == AP_F32 || out_dtype == AP_BF16, "gemm_tc: unknown output dtype %d", out_dtype);
    switch (bn) {
        case 16: GO(16);
        case 32: GO(32);
        case 64: GO(64);
        case 128: GO(128);
        default: GO(256);
    }
#undef GO
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
