// C[M,N] = A[M,K] * W[N,K]^T on the CUDA cores with 32-bit accumulation.
//
// This is the true 32-bit matrix product of the engine (no tensor cores, so no
// reduced-precision operand mode) and the fallback for bfloat16 shapes the
// tensor-core kernel refuses.  Each output element is one thread's sequential sum
// over k in ascending order, so a row's result does not depend on which other
// rows are in the batch.
//
// Reference counterpart: gemm_nt_kernel, one thread per output with a scalar K
// loop (cuda/src/kernels.cu:431-459).
#include "common.cuh"

#define BM 64
#define BN 64
#define BK 16
#define TM 4
#define TN 4

template <typename TA, typename TW, typename TO>
__global__ void __launch_bounds__(256)
gemm_nt_simt_kernel(const TA* __restrict__ A, const TW* __restrict__ W, TO* __restrict__ C,
                    int M, int N, int K, long long lda, long long ldw, long long ldc) {
    __shared__ float As[BK][BM + 4];
    __shared__ float Ws[BK][BN + 4];
    const int tid = threadIdx.x;
    const int tx = tid & 15, ty = tid >> 4;          // 16 x 16 threads, 4 x 4 outputs each
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;

    // each thread loads 4 elements of each tile per k-step: row = tid/4, k = (tid%4)*4..+3
    const int lrow = tid >> 2, lk = (tid & 3) * 4;
    for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
        for (int e = 0; e < 4; ++e) {
            const int k = k0 + lk + e;
            const int am = m0 + lrow, wn = n0 + lrow;
            As[lk + e][lrow] = (am < M && k < K) ? ap_to_float(A[(size_t)am * lda + k]) : 0.f;
            Ws[lk + e][lrow] = (wn < N && k < K) ? ap_to_float(W[(size_t)wn * ldw + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[TM], w[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) w[j] = Ws[kk][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int m = m0 + ty * TM + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int n = n0 + tx * TN + j;
            if (n < N) C[(size_t)m * ldc + n] = ap_from_float<TO>(acc[i][j]);
        }
    }
}

// The weight may be stored in 32-bit while activations are bfloat16 (a checkpoint tensor
// stored in 32-bit keeps its type); the output may be 32-bit for any operand type.
AP_EXPORT int ap_gemm_simt(const void* a, int a_dtype, const void* w, int w_dtype, void* out, int out_dtype,
                           int M, int N, int K, long long lda, long long ldw, long long ldc,
                           cudaStream_t stream) {
    AP_REQUIRE(M >= 0 && N > 0 && K > 0, "gemm: bad sizes M=%d N=%d K=%d", M, N, K);
    AP_REQUIRE(lda >= K && ldw >= K && ldc >= N, "gemm: a leading dimension is below its row length");
    if (M == 0) return AP_OK;
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    AP_REQUIRE(grid.y <= 65535, "gemm: %d rows exceed the grid of the CUDA-core kernel", M);
#define LAUNCH(TA, TW, TO)                                                      \
    gemm_nt_simt_kernel<TA, TW, TO><<<grid, 256, 0, stream>>>(                  \
        (const TA*)a, (const TW*)w, (TO*)out, M, N, K, lda, ldw, ldc)
    const int key = a_dtype * 100 + w_dtype * 10 + out_dtype;
    switch (key) {
        case 0: LAUNCH(float, float, float); break;
        case 111: LAUNCH(bf16, bf16, bf16); break;
        case 110: LAUNCH(bf16, bf16, float); break;
        case 101: LAUNCH(bf16, float, bf16); break;
        case 100: LAUNCH(bf16, float, float); break;
        default:
            AP_REQUIRE(false, "gemm: unsupported dtypes a=%d w=%d out=%d", a_dtype, w_dtype, out_dtype);
    }
#undef LAUNCH
    AP_CHECK_LAUNCH("gemm_simt");
    return AP_OK;
}
