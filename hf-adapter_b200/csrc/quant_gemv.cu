// Weight-streaming GEMV for the decode-time quantised projections (M <= 64 rows of
// activations against an int4 group-wise or int8 per-channel weight matrix).
//
// One warp owns one output channel and streams its weight row with 128-bit
// coalesced loads (a warp instruction reads 512 contiguous bytes), dequantises in
// registers exactly as the reference materialises the weight -- value =
// round_T((q - zero) * scale) -- and accumulates in fp32 against MB activation rows
// at a time; activations come from L1/L2 (they are M*K*2 bytes, shared by every
// warp).  The lane partial sums are combined with warp shuffles.  HBM-bound for
// small M; for larger M the FMA rate takes over and the tensor-core kernel on the tiled
// weight copy (w4g_umma.cu, rwkv7_w4g_gemv_tiled) is the one the model uses.
#include "common.cuh"

namespace rwkv7 {

struct GemvArgs {
    const void* x;
    const uint8_t* packed;  // int4: [Nout, K/2]; int8: [Nout, K] (as bytes)
    const void* scales;     // int4: [Nout, K/group]; int8: [Nout]
    const uint8_t* zeros;   // int4 only, optional
    const void* residual;
    void* out;
    int M, K, Nout, group, epilogue;
};

template <typename T>
__device__ __forceinline__ void epilogue_store(const GemvArgs& p, int m, int n, float acc) {
    float y = round_to<T>(acc);
    if (p.epilogue == RWKV7_EPI_RELU2) {
        y = fmaxf(y, 0.f);
        y = y * y;
    } else if (p.epilogue == RWKV7_EPI_ADD) {
        y += to_f<T>(reinterpret_cast<const T*>(p.residual)[(size_t)m * p.Nout + n]);
    }
    reinterpret_cast<T*>(p.out)[(size_t)m * p.Nout + n] = from_f<T>(y);
}

// W4: each lane takes 16 bytes = 32 consecutive k per iteration; 1024 k per warp iteration.
template <typename T, int MB>
__global__ void __launch_bounds__(256) w4g_gemv_kernel(const GemvArgs p) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = blockIdx.x * 8 + warp;
    if (n >= p.Nout) return;
    const int K = p.K, ngroups = K / p.group;
    const uint8_t* wrow = p.packed + (size_t)n * (K / 2);
    const T* srow = reinterpret_cast<const T*>(p.scales) + (size_t)n * ngroups;
    const uint8_t* zrow = p.zeros ? p.zeros + (size_t)n * ngroups : nullptr;
    const T* x = reinterpret_cast<const T*>(p.x);
    for (int m0 = 0; m0 < p.M; m0 += MB) {
        float acc[MB];
#pragma unroll
        for (int r = 0; r < MB; ++r) acc[r] = 0.f;
        for (int k0 = lane * 32; k0 < K; k0 += 1024) {
            const uint4 pk = *reinterpret_cast<const uint4*>(wrow + k0 / 2);
            const int gi = k0 / p.group;
            const float sc = to_f<T>(srow[gi]);
            const float z = zrow ? (float)zrow[gi] : 8.0f;
            float w[32];
            const uint32_t words[4] = {pk.x, pk.y, pk.z, pk.w};
#pragma unroll
            for (int q = 0; q < 4; ++q)
#pragma unroll
                for (int e = 0; e < 8; ++e)
                    w[q * 8 + e] = round_to<T>(((float)((words[q] >> (4 * e)) & 15u) - z) * sc);
#pragma unroll
            for (int r = 0; r < MB; ++r) {
                if (m0 + r < p.M) {
                    const T* xr = x + (size_t)(m0 + r) * K + k0;
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        float xv[8];
                        load8(xr + q * 8, xv);
#pragma unroll
                        for (int e = 0; e < 8; ++e) acc[r] = fmaf(xv[e], w[q * 8 + e], acc[r]);
                    }
                }
            }
        }
#pragma unroll
        for (int r = 0; r < MB; ++r) {
            const float s = group_sum<32>(acc[r]);
            if (lane == 0 && m0 + r < p.M) epilogue_store<T>(p, m0 + r, n, s);
        }
    }
}

// W8: each lane takes 16 bytes = 16 consecutive k per iteration; 512 k per warp iteration.
template <typename T, int MB>
__global__ void __launch_bounds__(256) w8_gemv_kernel(const GemvArgs p) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = blockIdx.x * 8 + warp;
    if (n >= p.Nout) return;
    const int K = p.K;
    const int8_t* wrow = reinterpret_cast<const int8_t*>(p.packed) + (size_t)n * K;
    const float sc = to_f<T>(reinterpret_cast<const T*>(p.scales)[n]);
    const T* x = reinterpret_cast<const T*>(p.x);
    for (int m0 = 0; m0 < p.M; m0 += MB) {
        float acc[MB];
#pragma unroll
        for (int r = 0; r < MB; ++r) acc[r] = 0.f;
        for (int k0 = lane * 16; k0 < K; k0 += 512) {
            const int4 pk = *reinterpret_cast<const int4*>(wrow + k0);
            const int8_t* qb = reinterpret_cast<const int8_t*>(&pk);
            float w[16];
#pragma unroll
            for (int e = 0; e < 16; ++e) w[e] = round_to<T>((float)qb[e] * sc);
#pragma unroll
            for (int r = 0; r < MB; ++r) {
                if (m0 + r < p.M) {
                    const T* xr = x + (size_t)(m0 + r) * K + k0;
#pragma unroll
                    for (int q = 0; q < 2; ++q) {
                        float xv[8];
                        load8(xr + q * 8, xv);
#pragma unroll
                        for (int e = 0; e < 8; ++e) acc[r] = fmaf(xv[e], w[q * 8 + e], acc[r]);
                    }
                }
            }
        }
#pragma unroll
        for (int r = 0; r < MB; ++r) {
            const float s = group_sum<32>(acc[r]);
            if (lane == 0 && m0 + r < p.M) epilogue_store<T>(p, m0 + r, n, s);
        }
    }
}

// ---------------------------------------------------------------- weight materialisation (prefill)
// W[n,k] = round_T((q - zero) * scale): the dense weight the reference hands to its GEMM for
// many-row inputs.  One thread per 16 packed bytes (int4) / 16 weights (int8).
template <typename T>
__global__ void __launch_bounds__(256) w4g_dequant_kernel(const uint8_t* __restrict__ packed, const T* __restrict__ scales,
                                                          const uint8_t* __restrict__ zeros, T* __restrict__ W,
                                                          int K, int group, long long total_chunks) {
    const long long c = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= total_chunks) return;
    const int chunks_per_row = K / 32;
    const long long n = c / chunks_per_row;
    const int k0 = (int)(c % chunks_per_row) * 32;
    const uint4 pk = *reinterpret_cast<const uint4*>(packed + n * (K / 2) + k0 / 2);
    const long long gi = n * (K / group) + k0 / group;
    const float sc = to_f<T>(scales[gi]);
    const float z = zeros ? (float)zeros[gi] : 8.0f;
    const uint32_t words[4] = {pk.x, pk.y, pk.z, pk.w};
#pragma unroll
    for (int q = 0; q < 4; ++q) {
        float w[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) w[e] = ((float)((words[q] >> (4 * e)) & 15u) - z) * sc;
        store8(W + n * K + k0 + q * 8, w);
    }
}

template <typename T>
__global__ void __launch_bounds__(256) w8_dequant_kernel(const int8_t* __restrict__ q, const T* __restrict__ scale,
                                                         T* __restrict__ W, int K, long long total_chunks) {
    const long long c = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= total_chunks) return;
    const int chunks_per_row = K / 16;
    const long long n = c / chunks_per_row;
    const int k0 = (int)(c % chunks_per_row) * 16;
    const int4 pk = *reinterpret_cast<const int4*>(q + n * K + k0);
    const int8_t* qb = reinterpret_cast<const int8_t*>(&pk);
    const float sc = to_f<T>(scale[n]);
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        float w[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) w[e] = (float)qb[h * 8 + e] * sc;
        store8(W + n * K + k0 + h * 8, w);
    }
}

static int check_gemv(const char* what, const GemvArgs& p, int kalign) {
    RWKV7_REQUIRE(p.M > 0 && p.K > 0 && p.Nout > 0, RWKV7_ERR_INVALID, "%s: sizes must be positive", what);
    RWKV7_REQUIRE(p.K % kalign == 0, RWKV7_ERR_UNSUPPORTED, "%s: K must be a multiple of %d (got %d)", what, kalign, p.K);
    RWKV7_REQUIRE(p.x && p.packed && p.scales && p.out, RWKV7_ERR_INVALID, "%s: null pointer", what);
    RWKV7_REQUIRE(p.epilogue >= 0 && p.epilogue <= 2, RWKV7_ERR_INVALID, "%s: bad epilogue code %d", what, p.epilogue);
    RWKV7_REQUIRE(p.epilogue != RWKV7_EPI_ADD || p.residual, RWKV7_ERR_INVALID, "%s: residual is required for the add epilogue", what);
    RWKV7_REQUIRE(aligned(p.x, 16) && aligned(p.packed, 16), RWKV7_ERR_ALIGN, "%s: x and weights must be 16-byte aligned", what);
    return RWKV7_OK;
}

}  // namespace rwkv7

using namespace rwkv7;

#define RWKV7_GEMV_LAUNCH(KERNEL)                                                           \
    do {                                                                                    \
        const int grid = (Nout + 7) / 8;                                                    \
        if (M == 1) KERNEL<T, 1><<<grid, 256, 0, st>>>(p);                                  \
        else if (M == 2) KERNEL<T, 2><<<grid, 256, 0, st>>>(p);                             \
        else if (M <= 4) KERNEL<T, 4><<<grid, 256, 0, st>>>(p);                             \
        else KERNEL<T, 8><<<grid, 256, 0, st>>>(p);                                         \
    } while (0)

extern "C" int rwkv7_w4g_gemv(const void* x, const uint8_t* packed, const void* scales, const uint8_t* zeros,
                              const void* residual, void* out, int M, int K, int Nout, int group, int epilogue,
                              int dtype, void* stream) {
    GemvArgs p{x, packed, scales, zeros, residual, out, M, K, Nout, group, epilogue};
    if (int e = check_gemv("w4g_gemv", p, 32)) return e;
    RWKV7_REQUIRE(group > 0 && group % 32 == 0 && K % group == 0, RWKV7_ERR_UNSUPPORTED,
                  "w4g_gemv: group must be a multiple of 32 dividing K (group=%d K=%d)", group, K);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    RWKV7_DISPATCH_DTYPE(dtype, T, {
        RWKV7_GEMV_LAUNCH(w4g_gemv_kernel);
        return check_launch("w4g_gemv_kernel");
    });
    return RWKV7_OK;
}

extern "C" int rwkv7_w8_gemv(const void* x, const int8_t* q, const void* scale, const void* residual, void* out,
                             int M, int K, int Nout, int epilogue, int dtype, void* stream) {
    GemvArgs p{x, reinterpret_cast<const uint8_t*>(q), scale, nullptr, residual, out, M, K, Nout, 0, epilogue};
    if (int e = check_gemv("w8_gemv", p, 16)) return e;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    RWKV7_DISPATCH_DTYPE(dtype, T, {
        RWKV7_GEMV_LAUNCH(w8_gemv_kernel);
        return check_launch("w8_gemv_kernel");
    });
    return RWKV7_OK;
}

extern "C" int rwkv7_w4g_dequant(const uint8_t* packed, const void* scales, const uint8_t* zeros, void* W, int K,
                                 int Nout, int group, int dtype, void* stream) {
    RWKV7_REQUIRE(K > 0 && Nout > 0, RWKV7_ERR_INVALID, "w4g_dequant: sizes must be positive");
    RWKV7_REQUIRE(K % 32 == 0 && group > 0 && group % 32 == 0 && K % group == 0, RWKV7_ERR_UNSUPPORTED,
                  "w4g_dequant: K and group must be multiples of 32 with group dividing K");
    RWKV7_REQUIRE(packed && scales && W, RWKV7_ERR_INVALID, "w4g_dequant: null pointer");
    RWKV7_REQUIRE(aligned(packed, 16) && aligned(W, 16), RWKV7_ERR_ALIGN, "w4g_dequant: unaligned pointer");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const long long chunks = (long long)Nout * (K / 32);
    RWKV7_DISPATCH_DTYPE(dtype, T, {
        w4g_dequant_kernel<T><<<(unsigned)((chunks + 255) / 256), 256, 0, st>>>(
            packed, reinterpret_cast<const T*>(scales), zeros, reinterpret_cast<T*>(W), K, group, chunks);
        return check_launch("w4g_dequant_kernel");
    });
    return RWKV7_OK;
}

extern "C" int rwkv7_w8_dequant(const int8_t* q, const void* scale, void* W, int K, int Nout, int dtype, void* stream) {
    RWKV7_REQUIRE(K > 0 && Nout > 0, RWKV7_ERR_INVALID, "w8_dequant: sizes must be positive");
    RWKV7_REQUIRE(K % 16 == 0, RWKV7_ERR_UNSUPPORTED, "w8_dequant: K must be a multiple of 16");
    RWKV7_REQUIRE(q && scale && W, RWKV7_ERR_INVALID, "w8_dequant: null pointer");
    RWKV7_REQUIRE(aligned(q, 16) && aligned(W, 16), RWKV7_ERR_ALIGN, "w8_dequant: unaligned pointer");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const long long chunks = (long long)Nout * (K / 16);
    RWKV7_DISPATCH_DTYPE(dtype, T, {
        w8_dequant_kernel<T><<<(unsigned)((chunks + 255) / 256), 256, 0, st>>>(
            q, reinterpret_cast<const T*>(scale), reinterpret_cast<T*>(W), K, chunks);
        return check_launch("w8_dequant_kernel");
    });
    return RWKV7_OK;
}
