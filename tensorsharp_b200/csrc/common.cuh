// Shared device/host helpers for every kernel in this library (sm_100a only).
//
// Conventions
//  * Every exported entry point is `extern "C" int tsb_<name>(..., void* stream)` and returns
//    0 on success or a negative TSB_ERR_* code; tsb_last_error() returns the message.
//  * Activations are bf16 unless a name says otherwise; norm weights and biases are f32.
//  * No entry point allocates device memory unless its comment says so; scratch is passed in.
//  * Device-side waits are bounded and report through a status word; nothing traps.
#pragma once
#include <cuda_runtime.h>
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <stdint.h>

#define TSB_OK 0
#define TSB_ERR_ARG (-1)
#define TSB_ERR_CUDA (-2)
#define TSB_ERR_UNSUPPORTED (-3)
#define TSB_ERR_TIMEOUT (-4)

#ifdef __cplusplus
extern "C" {
#endif
const char* tsb_last_error();
#ifdef __cplusplus
}
#endif
void tsb_set_error(const char* fmt, ...);

#define TSB_CHECK_ARG(cond, ...)                      \
    do {                                              \
        if (!(cond)) {                                \
            tsb_set_error(__VA_ARGS__);               \
            return TSB_ERR_ARG;                       \
        }                                             \
    } while (0)

#define TSB_CHECK_CUDA(expr)                                                        \
    do {                                                                            \
        cudaError_t _e = (expr);                                                    \
        if (_e != cudaSuccess) {                                                    \
            tsb_set_error("%s failed: %s (%s:%d)", #expr, cudaGetErrorString(_e),   \
                          __FILE__, __LINE__);                                      \
            return TSB_ERR_CUDA;                                                    \
        }                                                                           \
    } while (0)

#define TSB_CHECK_LAUNCH() TSB_CHECK_CUDA(cudaGetLastError())

// GGML tensor type ids (fixed by the GGUF specification).
enum TsbGgmlType {
    TSB_F32 = 0, TSB_F16 = 1, TSB_Q4_0 = 2, TSB_Q4_1 = 3, TSB_Q5_0 = 6, TSB_Q5_1 = 7,
    TSB_Q8_0 = 8, TSB_Q2_K = 10, TSB_Q3_K = 11, TSB_Q4_K = 12, TSB_Q5_K = 13, TSB_Q6_K = 14,
    TSB_IQ4_NL = 20, TSB_BF16 = 30, TSB_MXFP4 = 39
};

#ifdef __CUDACC__
#include <utility>
typedef __nv_bfloat16 bf16;

// Programmatic dependent launch: every kernel of this library is launched with the
// programmatic-serialisation attribute, calls pdl_wait() before its first global access (it
// returns once every earlier kernel in the stream has completed and flushed) and
// pdl_trigger() right after, which lets the next kernel's blocks be scheduled and run up to
// their own pdl_wait() while this one is still executing.  This hides the launch latency
// between the several hundred small kernels of a decode step.  Both are no-ops for a kernel
// launched without the attribute.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

bool tsb_pdl_enabled();

template <typename... KArgs, typename... Args>
static inline cudaError_t tsb_launch(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s,
                                     Args&&... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = s;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = tsb_pdl_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

typedef __nv_bfloat162 bf162;

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
// Block-wide sum; `red` is shared scratch of >= 32 floats. All threads get the result.
__device__ __forceinline__ float block_sum(float v, float* red) {
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) red[w] = v;
    __syncthreads();
    float r = (lane < nw) ? red[lane] : 0.f;
    r = warp_sum(r);
    return r;
}
__device__ __forceinline__ float block_max(float v, float* red) {
    const int lane = threadIdx.x & 31, w = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_max(v);
    __syncthreads();
    if (lane == 0) red[w] = v;
    __syncthreads();
    float r = (lane < nw) ? red[lane] : -INFINITY;
    r = warp_max(r);
    return r;
}
__device__ __forceinline__ float bf2f(bf16 v) { return __bfloat162float(v); }
__device__ __forceinline__ bf16 f2bf(float v) { return __float2bfloat16(v); }
__device__ __forceinline__ float h2f_bits(uint16_t b) { return __half2float(__ushort_as_half(b)); }

// 16-byte streaming load that does not pollute L1 (weights are read exactly once per step).
__device__ __forceinline__ uint4 ld_stream_u4(const void* p) {
    uint4 v;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p));
    return v;
}
__device__ __forceinline__ uint32_t ld_stream_u32(const void* p) {
    uint32_t v;
    asm volatile("ld.global.nc.L1::no_allocate.u32 %0, [%1];" : "=r"(v) : "l"(p));
    return v;
}
__device__ __forceinline__ uint16_t ld_stream_u16(const void* p) {
    uint16_t v;
    asm volatile("ld.global.nc.L1::no_allocate.u16 %0, [%1];" : "=h"(v) : "l"(p));
    return v;
}
#endif  // __CUDACC__
