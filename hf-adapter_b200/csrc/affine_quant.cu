// Affine 8-bit ("fp16i8") and 4-bit projections in the reference's layouts
// (rwkv7_hf/native_quant_mm8.py:62-110, rwkv7_hf/native_quant_mm4.py:77-125):
//
//   W[k, n] = (q[k, n] + 0.5) * ry[k] * rx[n] + my[k] + mx[n]          q: u8 [K, Nout]  or  u4 packed [K, Np/2]
//                                                                      (low nibble = even n), rx/mx [Nout], ry/my [K]
//   y[b, n] = sum_k x[b, k] W[k, n]
//           = rx[n] * sum_k (x[b,k] ry[k]) (q[k,n] + 0.5)  +  sum_k x[b,k] my[k]  +  mx[n] * sum_k x[b,k]
//
// Decode (up to 8 rows per pass): the weight bytes stream from HBM once, split over K so that every SM has work;
// fp32 partial sums go to a caller-provided workspace and a second kernel adds them in fixed order and applies the
// affine terms (deterministic, no atomics).  Many rows: materialise W in the activation dtype with the reference's
// operation order and rounding, then the caller runs one library GEMM (what the reference does above four rows).
#include "common.cuh"

namespace rwkv7 {

constexpr int kAffRows = 8;      // activation rows per pass
constexpr int kAffTileN = 256;   // output channels per CTA (8 per lane)
constexpr int kAffWarps = 8;

template <int BITS>
__device__ __forceinline__ void load_q8(const uint8_t* row, int n, float (&q)[8]) {
    if constexpr (BITS == 8) {
        const uint2 v = *reinterpret_cast<const uint2*>(row + n);
        const uint32_t w[2] = {v.x, v.y};
#pragma unroll
        for (int e = 0; e < 8; ++e) q[e] = (float)((w[e >> 2] >> (8 * (e & 3))) & 0xFFu) + 0.5f;
    } else {
        const uint32_t v = *reinterpret_cast<const uint32_t*>(row + (n >> 1));
#pragma unroll
        for (int e = 0; e < 8; ++e) q[e] = (float)((v >> (4 * e)) & 0xFu) + 0.5f;  // byte j: low nibble = n+2j, high = n+2j+1
    }
}

struct AffArgs {
    const void* x;
    const uint8_t* q;
    const void *mx, *rx, *my, *ry;
    float* partial;  // [S][M][Nout]
    void* out;
    int M, K, Nout, row_bytes, S, kslice;
};

template <typename T, int BITS>
__global__ void __launch_bounds__(kAffWarps * 32) affine_partial_kernel(const AffArgs p) {
    extern __shared__ float sm[];  // [warps][rows][tile]
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n0 = blockIdx.x * kAffTileN, n = n0 + lane * 8;
    const int kbeg = blockIdx.y * p.kslice, kend = min(p.K, kbeg + p.kslice);
    const T* x = reinterpret_cast<const T*>(p.x);
    const T* ry = reinterpret_cast<const T*>(p.ry);
    float acc[kAffRows][8];
#pragma unroll
    for (int b = 0; b < kAffRows; ++b)
#pragma unroll
        for (int e = 0; e < 8; ++e) acc[b][e] = 0.f;
    if (n < p.Nout) {
#pragma unroll 2
        for (int k = kbeg + warp; k < kend; k += kAffWarps) {
            float q[8];
            load_q8<BITS>(p.q + (size_t)k * p.row_bytes, n, q);
            const float r = to_f<T>(ry[k]);
#pragma unroll
            for (int b = 0; b < kAffRows; ++b) {
                if (b < p.M) {
                    const float xs = to_f<T>(x[(size_t)b * p.K + k]) * r;
#pragma unroll
                    for (int e = 0; e < 8; ++e) acc[b][e] = fmaf(xs, q[e], acc[b][e]);
                }
            }
        }
    }
#pragma unroll
    for (int b = 0; b < kAffRows; ++b)
#pragma unroll
        for (int e = 0; e < 8; ++e) sm[(warp * kAffRows + b) * kAffTileN + lane * 8 + e] = acc[b][e];
    __syncthreads();
    for (int idx = threadIdx.x; idx < p.M * kAffTileN; idx += kAffWarps * 32) {
        const int b = idx / kAffTileN, c = idx % kAffTileN;
        if (n0 + c >= p.Nout) continue;
        float s = 0.f;
#pragma unroll
        for (int w = 0; w < kAffWarps; ++w) s += sm[(w * kAffRows + b) * kAffTileN + c];
        p.partial[((size_t)blockIdx.y * p.M + b) * p.Nout + n0 + c] = s;
    }
}

// grid (tiles, M): sums the K-slices in order and applies the affine terms
template <typename T>
__global__ void __launch_bounds__(256) affine_finish_kernel(const AffArgs p) {
    __shared__ float red[32];
    const int b = blockIdx.y;
    const T* x = reinterpret_cast<const T*>(p.x) + (size_t)b * p.K;
    const T* my = reinterpret_cast<const T*>(p.my);
    float sx = 0.f, sxm = 0.f;
    for (int k = threadIdx.x; k < p.K; k += 256) {
        const float xv = to_f<T>(x[k]);
        sx += xv;
        sxm = fmaf(xv, to_f<T>(my[k]), sxm);
    }
    sx = block_sum(sx, red);
    sxm = block_sum(sxm, red);
    const int n = blockIdx.x * 256 + threadIdx.x;
    if (n < p.Nout) {
        float s = 0.f;
        for (int sl = 0; sl < p.S; ++sl) s += p.partial[((size_t)sl * p.M + b) * p.Nout + n];
        const float y = s * to_f<T>(reinterpret_cast<const T*>(p.rx)[n]) + sxm + sx * to_f<T>(reinterpret_cast<const T*>(p.mx)[n]);
        reinterpret_cast<T*>(p.out)[(size_t)b * p.Nout + n] = from_f<T>(y);
    }
}

// W[k][n] in T with the reference's operation order, each operation rounded to T
template <typename T, int BITS>
__global__ void __launch_bounds__(256) affine_dequant_kernel(const uint8_t* __restrict__ q, const T* __restrict__ mx,
                                                             const T* __restrict__ rx, const T* __restrict__ my,
                                                             const T* __restrict__ ry, T* __restrict__ W, int K, int Nout,
                                                             int row_bytes) {
    const int groups = (Nout + 7) / 8;
    const long long total = (long long)K * groups;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int k = (int)(i / groups), n = (int)(i % groups) * 8;
        const float ryk = to_f<T>(ry[k]), myk = to_f<T>(my[k]);
        const uint8_t* row = q + (size_t)k * row_bytes;
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            if (n + e >= Nout) break;
            float u;
            if constexpr (BITS == 8) u = (float)row[n + e];
            else u = (float)((row[(n + e) >> 1] >> (4 * ((n + e) & 1))) & 0xFu);
            float v = round_to<T>(u + 0.5f);
            v = round_to<T>(v * ryk);
            v = round_to<T>(v * to_f<T>(rx[n + e]));
            v = round_to<T>(v + myk);
            v = round_to<T>(v + to_f<T>(mx[n + e]));
            W[(size_t)k * Nout + n + e] = from_f<T>(v);
        }
    }
}

static int affine_splits(int K, int Nout) {
    const int tiles = (Nout + kAffTileN - 1) / kAffTileN;
    int S = (148 * 2 + tiles - 1) / tiles;
    if (S > 32) S = 32;
    while (S > 1 && K / S < 64) --S;
    return S < 1 ? 1 : S;
}

}  // namespace rwkv7

using namespace rwkv7;

extern "C" int64_t rwkv7_affine_gemv_workspace_bytes(int M, int K, int Nout) {
    if (M <= 0 || K <= 0 || Nout <= 0) return 0;
    const int rows = M < kAffRows ? M : kAffRows;
    return (int64_t)affine_splits(K, Nout) * rows * Nout * 4;
}

// bits = 8: q [K, Nout] u8;  bits = 4: q [K, Np/2] u8 with Np = Nout rounded up to even (row_bytes = Np / 2).
extern "C" int rwkv7_affine_gemv(const void* x, const uint8_t* q, const void* mx, const void* rx, const void* my,
                                 const void* ry, void* out, float* workspace, int64_t workspace_bytes, int M, int K,
                                 int Nout, int bits, int dtype, void* stream) {
    RWKV7_REQUIRE(bits == 8 || bits == 4, RWKV7_ERR_INVALID, "affine_gemv: bits must be 8 or 4 (got %d)", bits);
    RWKV7_REQUIRE(M >= 1 && M <= kAffRows, RWKV7_ERR_UNSUPPORTED, "affine_gemv: 1..%d rows per call (got %d)", kAffRows, M);
    RWKV7_REQUIRE(K > 0 && Nout > 0 && Nout % 8 == 0, RWKV7_ERR_UNSUPPORTED, "affine_gemv: Nout must be a positive multiple of 8 (got %d)", Nout);
    RWKV7_REQUIRE(x && q && mx && rx && my && ry && out && workspace, RWKV7_ERR_INVALID, "affine_gemv: null pointer");
    RWKV7_REQUIRE(aligned(q, 8) && aligned(workspace, 16), RWKV7_ERR_ALIGN, "affine_gemv: unaligned pointer");
    RWKV7_REQUIRE(workspace_bytes >= rwkv7_affine_gemv_workspace_bytes(M, K, Nout), RWKV7_ERR_WORKSPACE,
                  "affine_gemv: workspace of %lld bytes is smaller than the %lld required", (long long)workspace_bytes,
                  (long long)rwkv7_affine_gemv_workspace_bytes(M, K, Nout));
    AffArgs p{x, q, mx, rx, my, ry, workspace, out, M, K, Nout, bits == 8 ? Nout : Nout / 2, affine_splits(K, Nout), 0};
    p.kslice = ((K + p.S - 1) / p.S + kAffWarps - 1) / kAffWarps * kAffWarps;
    p.S = (K + p.kslice - 1) / p.kslice;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const int tiles = (Nout + kAffTileN - 1) / kAffTileN;
    const size_t smem = (size_t)kAffWarps * kAffRows * kAffTileN * sizeof(float);
    RWKV7_DISPATCH_DTYPE(dtype, T, {
        if (bits == 8) {
            cudaFuncSetAttribute(affine_partial_kernel<T, 8>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            affine_partial_kernel<T, 8><<<dim3(tiles, p.S), kAffWarps * 32, smem, st>>>(p);
        } else {
            cudaFuncSetAttribute(affine_partial_kernel<T, 4>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
            affine_partial_kernel<T, 4><<<dim3(tiles, p.S), kAffWarps * 32, smem, st>>>(p);
        }
        if (int e = check_launch("affine_partial_kernel")) return e;
        affine_finish_kernel<T><<<dim3((Nout + 255) / 256, M), 256, 0, st>>>(p);
        return check_launch("affine_finish_kernel");
    });
    return RWKV7_OK;
}

extern "C" int rwkv7_affine_dequant(const uint8_t* q, const void* mx, const void* rx, const void* my, const void* ry,
                                    void* W, int K, int Nout, int bits, int dtype, void* stream) {
    RWKV7_REQUIRE(bits == 8 || bits == 4, RWKV7_ERR_INVALID, "affine_dequant: bits must be 8 or 4 (got %d)", bits);
    RWKV7_REQUIRE(K > 0 && Nout > 0, RWKV7_ERR_INVALID, "affine_dequant: sizes must be positive");
    RWKV7_REQUIRE(q && mx && rx && my && ry && W, RWKV7_ERR_INVALID, "affine_dequant: null pointer");
    const int row_bytes = bits == 8 ? Nout : (Nout + 1) / 2;
    const long long total = (long long)K * ((Nout + 7) / 8);
    const int grid = (int)((total + 255) / 256 < 148LL * 32 ? (total + 255) / 256 : 148LL * 32);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    RWKV7_DISPATCH_DTYPE(dtype, T, {
        if (bits == 8)
            affine_dequant_kernel<T, 8><<<grid, 256, 0, st>>>(q, reinterpret_cast<const T*>(mx), reinterpret_cast<const T*>(rx),
                                                             reinterpret_cast<const T*>(my), reinterpret_cast<const T*>(ry),
                                                             reinterpret_cast<T*>(W), K, Nout, row_bytes);
        else
            affine_dequant_kernel<T, 4><<<grid, 256, 0, st>>>(q, reinterpret_cast<const T*>(mx), reinterpret_cast<const T*>(rx),
                                                             reinterpret_cast<const T*>(my), reinterpret_cast<const T*>(ry),
                                                             reinterpret_cast<T*>(W), K, Nout, row_bytes);
        return check_launch("affine_dequant_kernel");
    });
    return RWKV7_OK;
}
