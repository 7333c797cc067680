// Shared helpers of the sm_100a kernel library: dtype codes, error reporting,
// loads that widen to float, warp and block reductions.
//
// Every entry point is extern "C", takes raw device pointers and a stream, and
// returns 0 or a non-zero code after recording a message that
// skv_last_error() returns.  Nothing here allocates device memory.
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <cstdint>
#include <cstdio>
#include <cstdlib>

#define SKV_F32 0
#define SKV_BF16 1

// Each build of the library serves one compute dtype and one head size.
#ifndef SKV_DTYPE
#error "compile with -DSKV_DTYPE=0 (float) or 1 (bfloat16)"
#endif
#ifndef SKV_HEAD_DIM
#error "compile with -DSKV_HEAD_DIM=<head size, a multiple of 16>"
#endif
#if SKV_DTYPE == SKV_BF16
typedef __nv_bfloat16 skv_t;
#else
typedef float skv_t;
#endif

#define SKV_EXPORT extern "C" __attribute__((visibility("default")))

namespace skv {

inline char* error_buffer() {
    static thread_local char buffer[512] = {0};
    return buffer;
}

inline int fail(const char* what, const char* detail = "") {
    snprintf(error_buffer(), 512, "%s%s%s", what, detail[0] ? ": " : "", detail);
    return 1;
}

inline int check_launch(const char* kernel) {
    cudaError_t status = cudaGetLastError();
    if (status != cudaSuccess) return fail(kernel, cudaGetErrorString(status));
    return 0;
}

// ---- programmatic dependent launch ------------------------------------------
// Kernels of a step are launched so that the next one may start while the
// previous one drains: it can fetch what does not depend on its predecessor
// (weights, tables) and then waits.  pdl_wait() returns once the preceding
// kernel on the stream has completed and its writes are visible; nothing that a
// predecessor writes may be read, and nothing a predecessor reads may be
// written, before it.  Set SKV_NO_PDL=1 in the environment to launch plainly.
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void pdl_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;"); }

inline bool pdl_enabled() {
    static const bool enabled = [] {
        const char* off = getenv("SKV_NO_PDL");
        return !(off && off[0] == '1');
    }();
    return enabled;
}

template <typename... KernelArgs, typename... Args>
inline int launch_pdl(const char* name, void (*kernel)(KernelArgs...), dim3 grid, dim3 block, size_t smem,
                      cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = smem;
    config.stream = stream;
    cudaLaunchAttribute attribute[1];
    attribute[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attribute[0].val.programmaticStreamSerializationAllowed = 1;
    config.attrs = attribute;
    config.numAttrs = pdl_enabled() ? 1 : 0;
    const cudaError_t status = cudaLaunchKernelEx(&config, kernel, static_cast<KernelArgs>(args)...);
    if (status != cudaSuccess) return fail(name, cudaGetErrorString(status));
    return 0;
}

// Number of SMs of the current device (asked once per process; a process drives one kind of GPU).
inline int sm_count() {
    static const int count = [] {
        int device = 0, value = 0;
        if (cudaGetDevice(&device) != cudaSuccess ||
            cudaDeviceGetAttribute(&value, cudaDevAttrMultiProcessorCount, device) != cudaSuccess || value <= 0)
            value = 1;
        return value;
    }();
    return count;
}

// Activations of a gated feed-forward's gate, chosen by the part's spec (ops.ACTIVATIONS has the names).
enum { ACT_SILU = 0, ACT_GELU_TANH = 1, ACT_COUNT = 2 };

// gelu(g) = g/2 * (1 + tanh(sqrt(2/pi) * (g + 0.044715 g^3))), the "tanh" form.
__device__ __forceinline__ float gelu_tanh(float g) {
    return 0.5f * g * (1.0f + tanhf(0.7978845608028654f * (g + 0.044715f * g * g * g)));
}

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ float to_float(float v) { return v; }
__device__ __forceinline__ float to_float(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_float(float v);
template <> __device__ __forceinline__ float from_float<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_float<__nv_bfloat16>(float v) {
    return __float2bfloat16_rn(v);
}

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) v += __shfl_xor_sync(0xffffffffu, v, offset);
    return v;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int offset = 16; offset > 0; offset >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, offset));
    return v;
}

// Sum over a block of up to 1024 threads; every thread gets the result.
// `scratch` holds 33 floats of shared memory.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int warps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < warps ? scratch[lane] : 0.0f;
        t = warp_sum(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

}  // namespace skv
