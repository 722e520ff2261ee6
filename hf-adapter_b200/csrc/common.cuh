// Shared device/host helpers for the rwkv7_b200 kernels (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <atomic>

#include <cstdlib>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>

#include "../../include/rwkv7_b200.h"

namespace rwkv7 {

// ---- error plumbing -------------------------------------------------------
void set_error(const char* fmt, ...);  // defined in capi.cu (thread-local buffer)
constexpr int kMaxDevices = 64;        // device indices the per-device address caches cover

#define RWKV7_REQUIRE(cond, code, ...)  \
    do {                                \
        if (!(cond)) {                  \
            rwkv7::set_error(__VA_ARGS__); \
            return (code);              \
        }                               \
    } while (0)

inline int check_launch(const char* what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        set_error("%s: %s", what, cudaGetErrorString(e));
        return RWKV7_ERR_CUDA;
    }
    return RWKV7_OK;
}

inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) & (a - 1)) == 0; }

// Programmatic dependent launch of the projection kernels is on unless RWKV7_B200_NO_PDL is set (read once).
inline bool programmatic_launch_enabled() {
    static const bool on = [] {
        const char* v = getenv("RWKV7_B200_NO_PDL");
        return !(v && *v && *v != '0');
    }();
    return on;
}

// Launch with the programmatic-stream-serialization attribute: the kernel may become resident while its predecessor
// in the stream still runs and must call grid_dependency_wait() before touching anything that kernel writes.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_programmatic(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args&&... args) {
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = grid;
    cfg.blockDim = block;
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = programmatic_launch_enabled() ? 1 : 0;
    return cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...);
}

// ---- scalar conversion ----------------------------------------------------
template <typename T> __device__ __forceinline__ float to_f(T v);
template <> __device__ __forceinline__ float to_f<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f<__half>(__half v) { return __half2float(v); }
template <> __device__ __forceinline__ float to_f<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }

template <typename T> __device__ __forceinline__ T from_f(float v);
template <> __device__ __forceinline__ float from_f<float>(float v) { return v; }
template <> __device__ __forceinline__ __half from_f<__half>(float v) { return __float2half_rn(v); }
template <> __device__ __forceinline__ __nv_bfloat16 from_f<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// round a float through the storage type (models an HBM round trip without making one)
template <typename T> __device__ __forceinline__ float round_to(float v) { return to_f<T>(from_f<T>(v)); }

// ---- vectors of 4 / 8 elements ---------------------------------------------
template <typename T> struct Vec4 { T v[4]; };
template <typename T> struct alignas(16) Vec8 { T v[8]; };

template <typename T>
__device__ __forceinline__ void load4(const T* p, float (&o)[4]) {
    if constexpr (sizeof(T) == 4) {
        float4 t = *reinterpret_cast<const float4*>(p);
        o[0] = t.x; o[1] = t.y; o[2] = t.z; o[3] = t.w;
    } else {
        uint2 t = *reinterpret_cast<const uint2*>(p);
        const T* h = reinterpret_cast<const T*>(&t);
#pragma unroll
        for (int i = 0; i < 4; ++i) o[i] = to_f<T>(h[i]);
    }
}

template <typename T>
__device__ __forceinline__ void store4(T* p, const float (&o)[4]) {
    if constexpr (sizeof(T) == 4) {
        *reinterpret_cast<float4*>(p) = make_float4(o[0], o[1], o[2], o[3]);
    } else {
        uint2 t;
        T* h = reinterpret_cast<T*>(&t);
#pragma unroll
        for (int i = 0; i < 4; ++i) h[i] = from_f<T>(o[i]);
        *reinterpret_cast<uint2*>(p) = t;
    }
}

template <typename T>
__device__ __forceinline__ void load8(const T* p, float (&o)[8]) {
    if constexpr (sizeof(T) == 4) {
        float4 t0 = reinterpret_cast<const float4*>(p)[0];
        float4 t1 = reinterpret_cast<const float4*>(p)[1];
        o[0] = t0.x; o[1] = t0.y; o[2] = t0.z; o[3] = t0.w;
        o[4] = t1.x; o[5] = t1.y; o[6] = t1.z; o[7] = t1.w;
    } else {
        uint4 t = *reinterpret_cast<const uint4*>(p);
        const T* h = reinterpret_cast<const T*>(&t);
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] = to_f<T>(h[i]);
    }
}

template <typename T>
__device__ __forceinline__ void store8(T* p, const float (&o)[8]) {
    if constexpr (sizeof(T) == 4) {
        reinterpret_cast<float4*>(p)[0] = make_float4(o[0], o[1], o[2], o[3]);
        reinterpret_cast<float4*>(p)[1] = make_float4(o[4], o[5], o[6], o[7]);
    } else {
        uint4 t;
        T* h = reinterpret_cast<T*>(&t);
#pragma unroll
        for (int i = 0; i < 8; ++i) h[i] = from_f<T>(o[i]);
        *reinterpret_cast<uint4*>(p) = t;
    }
}

// ---- programmatic dependent launch ------------------------------------------
// A kernel launched with the programmatic-stream-serialization attribute may start while its predecessor in the
// stream is still running; it must not touch anything the predecessor writes before grid_dependency_wait() returns
// (which also makes the predecessor's writes visible).  Without the attribute both instructions are no-ops.
// grid_launch_dependents() lets the successor start once every CTA of this grid has issued it (or exited).
__device__ __forceinline__ void grid_dependency_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_launch_dependents() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// ---- math -----------------------------------------------------------------
__device__ __forceinline__ float sigmoidf_(float x) { return 1.0f / (1.0f + expf(-x)); }
// The reference's decay constant (rwkv7_hf/native.py:52), not exp(-0.5) to full precision.
__device__ __forceinline__ float decay_from_raw(float w_raw) { return expf(-0.606531f * sigmoidf_(w_raw)); }

// ---- reductions -----------------------------------------------------------
template <int WIDTH>
__device__ __forceinline__ float group_sum(float v) {
#pragma unroll
    for (int o = WIDTH / 2; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
template <int WIDTH>
__device__ __forceinline__ float group_max(float v) {
#pragma unroll
    for (int o = WIDTH / 2; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}

// Sum over a whole CTA (blockDim.x multiple of 32, <= 1024).  `red` holds >= 32 floats.
__device__ __forceinline__ float block_sum(float v, float* red) {
    v = group_sum<32>(v);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    __syncthreads();  // protect `red` from the previous use
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float t = (lane < nw) ? red[lane] : 0.0f;
    return group_sum<32>(t);
}
__device__ __forceinline__ float block_max(float v, float* red) {
    v = group_max<32>(v);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    __syncthreads();
    if (lane == 0) red[warp] = v;
    __syncthreads();
    float t = (lane < nw) ? red[lane] : -INFINITY;
    return group_max<32>(t);
}

// ---- dtype dispatch ---------------------------------------------------------
#define RWKV7_DISPATCH_DTYPE(dtype, T, ...)                           \
    switch (dtype) {                                                  \
        case RWKV7_F16: { using T = __half; __VA_ARGS__; break; }     \
        case RWKV7_BF16: { using T = __nv_bfloat16; __VA_ARGS__; break; } \
        case RWKV7_F32: { using T = float; __VA_ARGS__; break; }      \
        default: rwkv7::set_error("unknown dtype %d", dtype); return RWKV7_ERR_INVALID; \
    }

inline size_t dtype_size(int dtype) { return dtype == RWKV7_F32 ? 4 : 2; }

}  // namespace rwkv7
