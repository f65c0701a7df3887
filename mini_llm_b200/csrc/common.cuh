// Shared helpers of the kernel sources: element types, conversions, the
// activation formulas and the C ABI's error convention.
//
// Every exported launcher returns 0 on success and a non-zero code otherwise;
// the text of the last failure is read with <lib>_last_error().  Launchers
// never allocate device memory, never synchronise and launch on the stream
// they are given.
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <math.h>
#include <stdint.h>
#include <stdio.h>

typedef __nv_bfloat16 bf16;

// Element type codes of the C ABI.
enum { DT_F32 = 0, DT_BF16 = 1 };

// Epilogue codes of the linear kernels.
//   EPI_STORE      out = acc + bias
//   EPI_GELU_TANH  out = gelu_tanh(acc + bias)
//   EPI_GELU_ERF   out = gelu_erf(acc + bias)
//   EPI_ADD        out(fp32) += acc + bias        (residual sum kept in 32-bit)
enum { EPI_STORE = 0, EPI_GELU_TANH = 1, EPI_GELU_ERF = 2, EPI_ADD = 3 };

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<bf16>(bf16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ bf16 from_f32<bf16>(float v) { return __float2bfloat16_rn(v); }

// gelu, tanh form: 0.5 u (1 + tanh(0.7978845608 (u + 0.044715 u^3))), the
// formula of the reference's feed-forward (engine/include/gelu_math.h:6-11).
__device__ __forceinline__ float gelu_tanh_f(float u) {
    const float c = 0.7978845608f;
    const float k = 0.044715f;
    float arg = c * (u + k * u * u * u);
    return 0.5f * u * (1.0f + tanhf(arg));
}

// gelu, exact form: 0.5 u (1 + erf(u / sqrt(2))) (engine/src/gelu.c:5-9).
__device__ __forceinline__ float gelu_erf_f(float u) {
    return 0.5f * u * (1.0f + erff(u / sqrtf(2.0f)));
}

// gelu, tanh form, with the hardware's approximate tanh (relative error about 2^-11): the
// result is rounded to bfloat16 (2^-9) right after, and an exact tanh for every element of a
// feed-forward product costs more SM time than the product itself.  For kernels whose output is
// bfloat16 only.
__device__ __forceinline__ float gelu_tanh_fast(float u) {
    float t;
    asm("tanh.approx.f32 %0, %1;" : "=f"(t) : "f"(0.7978845608f * (u + 0.044715f * u * u * u)));
    return 0.5f * u * (1.0f + t);
}

template <int EPI> __device__ __forceinline__ float apply_activation(float v) {
    if (EPI == EPI_GELU_TANH) return gelu_tanh_f(v);
    if (EPI == EPI_GELU_ERF) return gelu_erf_f(v);
    return v;
}

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

// Sum over a block of up to 1024 threads; every thread gets the result.
// `scratch` holds 33 floats of shared memory.
__device__ __forceinline__ float block_sum(float v, float* scratch) {
    int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int n_warps = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();                 // scratch may still be read from a previous call
    if (lane == 0) scratch[warp] = v;
    __syncthreads();
    if (warp == 0) {
        float t = lane < n_warps ? scratch[lane] : 0.0f;
        t = warp_sum(t);
        if (lane == 0) scratch[32] = t;
    }
    __syncthreads();
    return scratch[32];
}

#define MLLM_ERROR_BUFFER 512

// ---- programmatic dependent launch ---------------------------------------------------------
//
// A kernel launched with launch_kernel(true, ...) may be scheduled while the kernel before it
// on the stream still runs: its CTAs take the SMs that the earlier kernel's CTAs leave, set up
// what needs no memory of the step (barriers, tensor memory, index arithmetic) and then wait
// in wait_for_earlier_kernels(), which returns when every earlier kernel has completed and its
// writes are visible.  No thread reads or writes global memory that another kernel of the
// stream touches before it has passed that wait.  A kernel says with dependents_may_start(),
// at its start, that the next one may be scheduled as soon as all of its own CTAs run.  Both
// calls do nothing in a kernel that was launched the ordinary way, and stream capture keeps the
// dependency as an edge of the graph.
__device__ __forceinline__ void dependents_may_start() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void wait_for_earlier_kernels() { asm volatile("griddepcontrol.wait;" ::: "memory"); }

// (cluster: the CTAs of a thread block cluster, or x = 0 for a launch without clusters)
template <typename... Params, typename... Args>
static cudaError_t launch_kernel_in_clusters(bool dependent, dim3 cluster, void (*kernel)(Params...), dim3 grid, dim3 block,
                                             size_t shared_bytes, cudaStream_t stream, Args... args) {
    cudaLaunchConfig_t config = {};
    config.gridDim = grid;
    config.blockDim = block;
    config.dynamicSmemBytes = shared_bytes;
    config.stream = stream;
    cudaLaunchAttribute attributes[2];
    unsigned count = 0;
    if (dependent) {
        attributes[count].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attributes[count].val.programmaticStreamSerializationAllowed = 1;
        count++;
    }
    if (cluster.x != 0) {
        attributes[count].id = cudaLaunchAttributeClusterDimension;
        attributes[count].val.clusterDim.x = cluster.x;
        attributes[count].val.clusterDim.y = cluster.y;
        attributes[count].val.clusterDim.z = cluster.z;
        count++;
    }
    config.attrs = attributes;
    config.numAttrs = count;
    return cudaLaunchKernelEx(&config, kernel, Params(args)...);
}
template <typename... Params, typename... Args>
static cudaError_t launch_kernel(bool dependent, void (*kernel)(Params...), dim3 grid, dim3 block, size_t shared_bytes,
                                 cudaStream_t stream, Args... args) {
    return launch_kernel_in_clusters(dependent, dim3(0, 1, 1), kernel, grid, block, shared_bytes, stream, args...);
}

#define MLLM_DEFINE_ERROR_API(prefix)                                              \
    static thread_local char g_error_text[MLLM_ERROR_BUFFER] = "";                 \
    extern "C" const char* prefix##_last_error(void) { return g_error_text; }      \
    static int fail(const char* what) {                                            \
        snprintf(g_error_text, MLLM_ERROR_BUFFER, "%s", what);                     \
        return 1;                                                                  \
    }                                                                              \
    static int check_launch(const char* kernel) {                                  \
        cudaError_t e = cudaGetLastError();                                        \
        if (e == cudaSuccess) return 0;                                            \
        snprintf(g_error_text, MLLM_ERROR_BUFFER, "%s: %s", kernel,                \
                 cudaGetErrorString(e));                                           \
        return 2;                                                                  \
    }                                                                              \
    /* whether this library's kernels are launched as dependents (see above) */    \
    static int g_dependent_launch = 1;                                             \
    extern "C" void prefix##_set_dependent_launch(int on) { g_dependent_launch = on; } \
    static int launched(cudaError_t e, const char* kernel) {                       \
        if (e == cudaSuccess) return check_launch(kernel);                         \
        snprintf(g_error_text, MLLM_ERROR_BUFFER, "%s: %s", kernel,                \
                 cudaGetErrorString(e));                                           \
        return 2;                                                                  \
    }
