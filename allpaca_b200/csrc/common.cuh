// Shared declarations of the kernel library: status codes, element types and
// small load/store helpers.  Every exported function is `extern "C"`, takes the
// stream it launches on as its last argument and returns one of the codes below;
// nothing here allocates device memory.
//
// Role in the reference: the flat C kernel ABI with status codes and one stream
// argument per call (cuda/include/allpaca_cuda_kernels.h:11-22).
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <stdint.h>

#define AP_OK 0
#define AP_ERR_INVALID 1      // an argument the kernel cannot take (size, alignment, dtype)
#define AP_ERR_LAUNCH 2       // the CUDA runtime refused the launch
#define AP_ERR_UNSUPPORTED 3  // a size outside what this build was compiled for

#define AP_F32 0
#define AP_BF16 1

#define AP_EXPORT extern "C" __attribute__((visibility("default")))

// The last error text of this thread, for the Python side to raise with.
void ap_set_error(const char* fmt, ...);

#define AP_REQUIRE(cond, ...)                 \
    do {                                      \
        if (!(cond)) {                        \
            ap_set_error(__VA_ARGS__);        \
            return AP_ERR_INVALID;            \
        }                                     \
    } while (0)

#define AP_CHECK_LAUNCH(name)                                              \
    do {                                                                   \
        cudaError_t e__ = cudaGetLastError();                              \
        if (e__ != cudaSuccess) {                                          \
            ap_set_error("%s: launch failed: %s", name, cudaGetErrorString(e__)); \
            return AP_ERR_LAUNCH;                                          \
        }                                                                  \
    } while (0)

typedef __nv_bfloat16 bf16;

// ---- programmatic dependent launch ---------------------------------------------------
// Kernels of the decode path are launched so that a kernel may start while the one before
// it on the stream is still running.  Such a kernel does only work that depends on nothing
// the earlier kernels write (set-up, prefetch of weights) until ap_pdl_wait() returns,
// which is when every earlier kernel has finished and its writes are visible; and it calls
// ap_pdl_trigger() once the kernel after it may start the same way.  Launched without the
// attribute both are no-ops.
__device__ __forceinline__ void ap_pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void ap_pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

bool ap_pdl_enabled();     // false when the environment sets ALLPACA_PDL=0

template <typename... KArgs, typename... Args>
static inline cudaError_t ap_launch_pdl(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem,
                                        cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = stream;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = ap_pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, KArgs(args)...);
}

#define AP_CHECK_PDL_LAUNCH(name, call)                                        \
    do {                                                                       \
        cudaError_t e__ = (call);                                              \
        if (e__ != cudaSuccess) {                                              \
            ap_set_error("%s: launch failed: %s", name, cudaGetErrorString(e__)); \
            return AP_ERR_LAUNCH;                                              \
        }                                                                      \
    } while (0)

__device__ __forceinline__ float ap_to_float(float v) { return v; }
__device__ __forceinline__ float ap_to_float(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T ap_from_float(float v);
template <> __device__ __forceinline__ float ap_from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 ap_from_float<bf16>(float v) { return __float2bfloat16_rn(v); }

__device__ __forceinline__ float ap_warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float ap_warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Block-wide sum with a fixed order: lanes by butterfly, then warps in index order.
// `scratch` holds at least 32 floats.  All threads get the result.
__device__ __forceinline__ float ap_block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = ap_warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float total = 0.f;
    for (int w = 0; w < nwarps; ++w) total += scratch[w];
    return total;
}
__device__ __forceinline__ float ap_block_max(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int nwarps = (blockDim.x + 31) >> 5;
    v = ap_warp_max(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    float total = scratch[0];
    for (int w = 1; w < nwarps; ++w) total = fmaxf(total, scratch[w]);
    return total;
}
