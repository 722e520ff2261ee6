// A8W8 projection for prefill: dynamic per-row int8 activation quantiser, int8 x int8
// -> int32 GEMM (bit-exact integer accumulators), fp32 dequant epilogue.
//
// This file holds the quantiser, the epilogue and a warp-level mma.sync (IMMA
// m16n8k32) GEMM used for shapes the tcgen05 kernel (gemm_umma.cu) does not take
// (ragged M/N/K) and as the comparison baseline for it.
#include "common.cuh"

namespace rwkv7 {

// ---------------------------------------------------------------- quantiser
// one CTA per row; s = max(amax/127, 1e-5); q = clamp(round_half_away(x / s), +-127).  The row is read from memory
// ONCE: each thread keeps its 8-element chunks in registers between the amax pass and the quantising pass (rows up to
// 256 * 8 * kQuantChunks elements; longer rows re-read the tail, which then comes from L2).
constexpr int kQuantChunks = 8;

__device__ __forceinline__ int8_t quant_one(float v, float s) {
    const float t = __fdiv_rn(v, s);
    float r = (t >= 0.f) ? floorf(t + 0.5f) : ceilf(t - 0.5f);
    r = fminf(fmaxf(r, -127.f), 127.f);
    return (int8_t)(int)r;
}

template <typename T>
__global__ void __launch_bounds__(256) a8_quant_kernel(const T* __restrict__ x, int8_t* __restrict__ q,
                                                       float* __restrict__ scale, int K) {
    __shared__ float red[32];
    const size_t row = blockIdx.x;
    const T* xr = x + row * K;
    Vec8<T> keep[kQuantChunks];  // the row's chunks in their storage type: 4 registers per chunk for 16-bit inputs
    float amax = 0.f;
#pragma unroll
    for (int c = 0; c < kQuantChunks; ++c) {
        const int k = (c * 256 + threadIdx.x) * 8;
        if (k < K) {
            keep[c] = *reinterpret_cast<const Vec8<T>*>(xr + k);
#pragma unroll
            for (int e = 0; e < 8; ++e) amax = fmaxf(amax, fabsf(to_f<T>(keep[c].v[e])));
        }
    }
    for (int k = (kQuantChunks * 256 + threadIdx.x) * 8; k < K; k += 256 * 8) {
        float v[8];
        load8(xr + k, v);
#pragma unroll
        for (int e = 0; e < 8; ++e) amax = fmaxf(amax, fabsf(v[e]));
    }
    amax = block_max(amax, red);
    const float s = fmaxf(__fdiv_rn(amax, 127.0f), 1.0e-5f);
    if (threadIdx.x == 0) scale[row] = s;
#pragma unroll
    for (int c = 0; c < kQuantChunks; ++c) {
        const int k = (c * 256 + threadIdx.x) * 8;
        if (k < K) {
            alignas(8) int8_t o[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) o[e] = quant_one(to_f<T>(keep[c].v[e]), s);
            *reinterpret_cast<uint2*>(q + row * K + k) = *reinterpret_cast<const uint2*>(o);
        }
    }
    for (int k = (kQuantChunks * 256 + threadIdx.x) * 8; k < K; k += 256 * 8) {
        float v[8];
        load8(xr + k, v);
        alignas(8) int8_t o[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) o[e] = quant_one(v[e], s);
        *reinterpret_cast<uint2*>(q + row * K + k) = *reinterpret_cast<const uint2*>(o);
    }
}

// ---------------------------------------------------------------- FFN boundary: dequantise, relu^2, requantise
// one CTA per row: h = fp16(acc * sa[row] * sw[n] (+ bias)); r = fp16(max(h, 0)^2); then the activation quantiser on r
// (rwkv7_hf/native_quant_a8w8.py:189-232).  The hidden activation never exists in fp16 in memory.
template <typename T>
__global__ void __launch_bounds__(256) a8w8_relu2_requant_kernel(const int32_t* __restrict__ acc, const float* __restrict__ sa,
                                                                 const float* __restrict__ sw, const T* __restrict__ bias,
                                                                 int8_t* __restrict__ q, float* __restrict__ scale, int N) {
    __shared__ float red[32];
    const size_t row = blockIdx.x;
    const int32_t* ar = acc + row * N;
    const float a_s = sa[row];
    auto value = [&](int n) {
        float pre = (float)ar[n] * a_s * sw[n];
        if (bias) pre += to_f<T>(bias[n]);
        pre = __half2float(__float2half_rn(pre));
        const float act = fmaxf(pre, 0.f);
        return __half2float(__float2half_rn(act * act));
    };
    float amax = 0.f;
    for (int n = threadIdx.x; n < N; n += 256) amax = fmaxf(amax, fabsf(value(n)));
    amax = block_max(amax, red);
    const float s = fmaxf(__fdiv_rn(amax, 127.0f), 1.0e-5f);
    if (threadIdx.x == 0) scale[row] = s;
    for (int n = threadIdx.x; n < N; n += 256) {
        const float t = __fdiv_rn(value(n), s);
        float r = (t >= 0.f) ? floorf(t + 0.5f) : ceilf(t - 0.5f);
        r = fminf(fmaxf(r, -127.f), 127.f);
        q[row * N + n] = (int8_t)(int)r;
    }
}

// ---------------------------------------------------------------- dequant epilogue
template <typename T>
__global__ void __launch_bounds__(256) a8w8_dequant_kernel(const int32_t* __restrict__ acc, const float* __restrict__ sa,
                                                           const float* __restrict__ sw, const T* __restrict__ bias,
                                                           const T* __restrict__ residual, T* __restrict__ out,
                                                           int M, int Nout, int relu2) {
    const long long total = (long long)M * Nout;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (long long)gridDim.x * blockDim.x) {
        const int m = (int)(i / Nout), n = (int)(i % Nout);
        // every step rounded on its own (no fused multiply-add): the tensor-core GEMM's fused epilogue does the same
        float v = __fmul_rn(__fmul_rn((float)acc[i], sa[m]), sw[n]);
        if (bias) v = __fadd_rn(v, to_f<T>(bias[n]));
        if (relu2) {
            const float a = fmaxf(round_to<T>(v), 0.f);
            v = a * a;
        } else if (residual) {
            v = __fadd_rn(v, to_f<T>(residual[i]));
        }
        out[i] = from_f<T>(v);
    }
}

// ---------------------------------------------------------------- mma.sync int8 GEMM
// C[M,N] (i32) = A[M,K] (i8, row-major) . B[N,K]^T (i8, row-major).  CTA tile 128x128x64,
// 8 warps as 2 (M) x 4 (N), warp tile 64x32, cp.async double buffering, 16-byte-chunk XOR
// swizzle in shared memory so ldmatrix is conflict-free.
constexpr int BM = 128, BN = 128, BK = 64;

__device__ __forceinline__ void cp_async16_zfill(void* smem, const void* gmem, bool valid) {
    unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    int sz = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(gmem), "r"(sz));
}
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], const void* smem) {
    unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
__device__ __forceinline__ void mma_s8(int (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+r"(c[0]), "+r"(c[1]), "+r"(c[2]), "+r"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// smem tile: rows of 64 bytes = 4 chunks of 16 B; chunk c of row r is stored at chunk (c ^ ((r >> 1) & 3))
__device__ __forceinline__ int swz(int row, int chunk) { return row * 64 + ((chunk ^ ((row >> 1) & 3)) << 4); }

__global__ void __launch_bounds__(256) i8_gemm_mma_kernel(const int8_t* __restrict__ A, const int8_t* __restrict__ Bm,
                                                          int32_t* __restrict__ C, int M, int K, int N) {
    __shared__ __align__(128) int8_t sA[2][BM * BK];
    __shared__ __align__(128) int8_t sB[2][BN * BK];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int wm = warp >> 2, wn = warp & 3;  // 2 x 4
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;

    int acc[4][4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[i][j][e] = 0;

    auto load_tile = [&](int buf, int k0) {
        // 128 rows x 4 chunks for A and for B: 512 chunks each, 256 threads -> 2 + 2
#pragma unroll
        for (int it = 0; it < 2; ++it) {
            const int idx = tid + it * 256;
            const int row = idx >> 2, ch = idx & 3;
            const bool kin = (k0 + ch * 16) < K;
            const bool va = kin && (m0 + row) < M;
            const bool vb = kin && (n0 + row) < N;
            cp_async16_zfill(&sA[buf][swz(row, ch)], va ? A + (size_t)(m0 + row) * K + k0 + ch * 16 : A, va);
            cp_async16_zfill(&sB[buf][swz(row, ch)], vb ? Bm + (size_t)(n0 + row) * K + k0 + ch * 16 : Bm, vb);
        }
        asm volatile("cp.async.commit_group;\n" ::);
    };

    const int nk = (K + BK - 1) / BK;
    load_tile(0, 0);
    for (int kt = 0; kt < nk; ++kt) {
        const int buf = kt & 1;
        if (kt + 1 < nk) {
            load_tile(buf ^ 1, (kt + 1) * BK);
            asm volatile("cp.async.wait_group 1;\n" ::);
        } else {
            asm volatile("cp.async.wait_group 0;\n" ::);
        }
        __syncthreads();
#pragma unroll
        for (int ks = 0; ks < 2; ++ks) {  // two k32 steps per BK = 64
            uint32_t af[4][4], bf[2][4];
            // A: x4 = (rows 0-7, k lo), (rows 8-15, k lo), (rows 0-7, k hi), (rows 8-15, k hi)
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                const int row = wm * 64 + i * 16 + (lane & 7) + ((lane >> 3) & 1) * 8;
                const int ch = ks * 2 + (lane >> 4);
                ldmatrix_x4(af[i], &sA[buf][swz(row, ch)]);
            }
            // B: x4 = (n 0-7, k lo), (n 0-7, k hi), (n 8-15, k lo), (n 8-15, k hi)
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int row = wn * 32 + j * 16 + (lane & 7) + (lane >> 4) * 8;
                const int ch = ks * 2 + ((lane >> 3) & 1);
                ldmatrix_x4(bf[j], &sB[buf][swz(row, ch)]);
            }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) mma_s8(acc[i][j], af[i], bf[j >> 1][(j & 1) * 2], bf[j >> 1][(j & 1) * 2 + 1]);
        }
        __syncthreads();
    }

    const int gid = lane >> 2, tig = lane & 3;
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int row = m0 + wm * 64 + i * 16 + gid;
            const int col = n0 + wn * 32 + j * 8 + tig * 2;
#pragma unroll
            for (int hh = 0; hh < 2; ++hh) {
                const int rr = row + hh * 8;
                if (rr < M) {
                    if (col + 1 < N && (N & 1) == 0) {
                        *reinterpret_cast<int2*>(C + (size_t)rr * N + col) = make_int2(acc[i][j][hh * 2], acc[i][j][hh * 2 + 1]);
                    } else {
                        if (col < N) C[(size_t)rr * N + col] = acc[i][j][hh * 2];
                        if (col + 1 < N) C[(size_t)rr * N + col + 1] = acc[i][j][hh * 2 + 1];
                    }
                }
            }
        }
}

int launch_i8_gemm_mma(const int8_t* qa, const int8_t* qw, int32_t* acc, int M, int K, int Nout, cudaStream_t st) {
    dim3 grid((Nout + BN - 1) / BN, (M + BM - 1) / BM);
    i8_gemm_mma_kernel<<<grid, 256, 0, st>>>(qa, qw, acc, M, K, Nout);
    return check_launch("i8_gemm_mma_kernel");
}

// implemented in gemm_umma.cu; returns RWKV7_ERR_UNSUPPORTED when the shape is not eligible
int launch_i8_gemm_umma(const int8_t* qa, const int8_t* qw, int32_t* acc, int M, int K, int Nout, cudaStream_t st);
int launch_i8_gemm_dequant_umma(const int8_t* qa, const float* sa, const int8_t* qw, const float* sw, const void* bias,
                                const void* residual, void* out, int M, int K, int Nout, int relu2, int dtype,
                                cudaStream_t st);

static inline int64_t align_up(int64_t v, int64_t a) { return (v + a - 1) / a * a; }

}  // namespace rwkv7

using namespace rwkv7;

extern "C" int rwkv7_a8_quant(const void* x, int8_t* q, float* scale, int rows, int K, int dtype, void* stream) {
    RWKV7_REQUIRE(rows > 0 && K > 0, RWKV7_ERR_INVALID, "a8_quant: sizes must be positive");
    RWKV7_REQUIRE(K % 8 == 0, RWKV7_ERR_UNSUPPORTED, "a8_quant: K must be a multiple of 8 (got %d)", K);
    RWKV7_REQUIRE(x && q && scale, RWKV7_ERR_INVALID, "a8_quant: null pointer");
    RWKV7_REQUIRE(aligned(x, 16) && aligned(q, 8), RWKV7_ERR_ALIGN, "a8_quant: unaligned pointer");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    RWKV7_DISPATCH_DTYPE(dtype, T, {
        a8_quant_kernel<T><<<rows, 256, 0, st>>>(reinterpret_cast<const T*>(x), q, scale, K);
        return check_launch("a8_quant_kernel");
    });
    return RWKV7_OK;
}

extern "C" int rwkv7_i8_gemm(const int8_t* qa, const int8_t* qw, int32_t* acc, int M, int K, int Nout, void* stream) {
    RWKV7_REQUIRE(M > 0 && K > 0 && Nout > 0, RWKV7_ERR_INVALID, "i8_gemm: sizes must be positive");
    RWKV7_REQUIRE(K % 16 == 0, RWKV7_ERR_UNSUPPORTED, "i8_gemm: K must be a multiple of 16 (got %d)", K);
    RWKV7_REQUIRE(qa && qw && acc, RWKV7_ERR_INVALID, "i8_gemm: null pointer");
    RWKV7_REQUIRE(aligned(qa, 16) && aligned(qw, 16) && aligned(acc, 16), RWKV7_ERR_ALIGN, "i8_gemm: unaligned pointer");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int e = launch_i8_gemm_umma(qa, qw, acc, M, K, Nout, st);
    if (e != RWKV7_ERR_UNSUPPORTED) return e;
    return launch_i8_gemm_mma(qa, qw, acc, M, K, Nout, st);
}

static int a8w8_dequant_impl(const int32_t* acc, const float* sa, const float* sw, const void* bias, const void* residual,
                             void* out, int M, int Nout, int relu2, int dtype, void* stream) {
    RWKV7_REQUIRE(M > 0 && Nout > 0, RWKV7_ERR_INVALID, "a8w8_dequant: sizes must be positive");
    RWKV7_REQUIRE(acc && sa && sw && out, RWKV7_ERR_INVALID, "a8w8_dequant: null pointer");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const long long total = (long long)M * Nout;
    const int grid = (int)((total + 255) / 256 < 148LL * 16 ? (total + 255) / 256 : 148LL * 16);
    RWKV7_DISPATCH_DTYPE(dtype, T, {
        a8w8_dequant_kernel<T><<<grid, 256, 0, st>>>(acc, sa, sw, reinterpret_cast<const T*>(bias),
                                                    reinterpret_cast<const T*>(residual), reinterpret_cast<T*>(out), M, Nout, relu2);
        return check_launch("a8w8_dequant_kernel");
    });
    return RWKV7_OK;
}

extern "C" int rwkv7_a8w8_dequant(const int32_t* acc, const float* sa, const float* sw, const void* bias,
                                  const void* residual, void* out, int M, int Nout, int dtype, void* stream) {
    return a8w8_dequant_impl(acc, sa, sw, bias, residual, out, M, Nout, 0, dtype, stream);
}

extern "C" int rwkv7_a8w8_relu2_requant(const int32_t* acc, const float* sa, const float* sw, const void* bias, int8_t* q,
                                        float* scale, int M, int N, int dtype, void* stream) {
    RWKV7_REQUIRE(M > 0 && N > 0, RWKV7_ERR_INVALID, "a8w8_relu2_requant: sizes must be positive");
    RWKV7_REQUIRE(acc && sa && sw && q && scale, RWKV7_ERR_INVALID, "a8w8_relu2_requant: null pointer");
    RWKV7_REQUIRE(dtype == RWKV7_F16, RWKV7_ERR_UNSUPPORTED, "a8w8_relu2_requant: the fused FFN boundary is defined for fp16 activations");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    a8w8_relu2_requant_kernel<__half><<<M, 256, 0, st>>>(acc, sa, sw, reinterpret_cast<const __half*>(bias), q, scale, N);
    return check_launch("a8w8_relu2_requant_kernel");
}

extern "C" int64_t rwkv7_a8w8_workspace_bytes(int M, int K, int Nout) {
    if (M <= 0 || K <= 0 || Nout <= 0) return 0;
    return align_up((int64_t)M * K, 256) + align_up((int64_t)M * 4, 256) + align_up((int64_t)M * Nout * 4, 256);
}

static int a8w8_linear_impl(const void* x, const int8_t* qw, const float* sw, const void* bias, const void* residual,
                            void* out, void* workspace, int64_t workspace_bytes, int M, int K, int Nout, int relu2,
                            int dtype, void* stream) {
    RWKV7_REQUIRE(M > 0 && K > 0 && Nout > 0, RWKV7_ERR_INVALID, "a8w8_linear: sizes must be positive");
    RWKV7_REQUIRE(workspace && aligned(workspace, 256), RWKV7_ERR_ALIGN, "a8w8_linear: workspace must be 256-byte aligned");
    RWKV7_REQUIRE(workspace_bytes >= rwkv7_a8w8_workspace_bytes(M, K, Nout), RWKV7_ERR_WORKSPACE,
                  "a8w8_linear: workspace of %lld bytes is smaller than the %lld required", (long long)workspace_bytes,
                  (long long)rwkv7_a8w8_workspace_bytes(M, K, Nout));
    char* ws = static_cast<char*>(workspace);
    int8_t* qa = reinterpret_cast<int8_t*>(ws);
    float* sa = reinterpret_cast<float*>(ws + align_up((int64_t)M * K, 256));
    int32_t* acc = reinterpret_cast<int32_t*>(ws + align_up((int64_t)M * K, 256) + align_up((int64_t)M * 4, 256));
    if (int e = rwkv7_a8_quant(x, qa, sa, M, K, dtype, stream)) return e;
    // tensor-core route: the dequantisation rides in the GEMM's epilogue, the int32 accumulators never reach memory
    RWKV7_REQUIRE(sw && out, RWKV7_ERR_INVALID, "a8w8_linear: null pointer");
    int e = launch_i8_gemm_dequant_umma(qa, sa, qw, sw, bias, residual, out, M, K, Nout, relu2, dtype, static_cast<cudaStream_t>(stream));
    if (e != RWKV7_ERR_UNSUPPORTED) return e;
    if (int e2 = rwkv7_i8_gemm(qa, qw, acc, M, K, Nout, stream)) return e2;
    return a8w8_dequant_impl(acc, sa, sw, bias, residual, out, M, Nout, relu2, dtype, stream);
}

extern "C" int rwkv7_a8w8_linear(const void* x, const int8_t* qw, const float* sw, const void* bias,
                                 const void* residual, void* out, void* workspace, int64_t workspace_bytes, int M,
                                 int K, int Nout, int dtype, void* stream) {
    return a8w8_linear_impl(x, qw, sw, bias, residual, out, workspace, workspace_bytes, M, K, Nout, 0, dtype, stream);
}

extern "C" int rwkv7_a8w8_linear_relu2(const void* x, const int8_t* qw, const float* sw, const void* bias, void* out,
                                       void* workspace, int64_t workspace_bytes, int M, int K, int Nout, int dtype,
                                       void* stream) {
    return a8w8_linear_impl(x, qw, sw, bias, nullptr, out, workspace, workspace_bytes, M, K, Nout, 1, dtype, stream);
}

// ---------------------------------------------------------------- no-allocation variant
// Some callers cannot obtain device memory at call time: a serving process that has handed the whole GPU
// memory pool to its own arena, a real-time or signal-restricted thread that must not enter the CUDA
// allocator, a plugin host that forbids cudaMalloc inside operator calls.  For them the scratch that
// rwkv7_a8w8_linear takes from the caller (quantised rows, row scales, int32 accumulators) lives in a
// fixed array inside the library instead.  Every GPU that loads the library holds kStaticScratchBytes of
// it until the process exits.
constexpr long long kStaticScratchBytes = 8ll << 20;  // 8 MiB
static __device__ __align__(256) unsigned char g_a8w8_static_scratch[kStaticScratchBytes];

namespace {
// In host code the array's name is only a handle for the runtime: the device address has to be asked
// for, once per device, with that device current.
void* static_scratch_ptr() {
    static std::atomic<void*> cache[rwkv7::kMaxDevices];  // racing first callers store the same address
    int dev = -1;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0) {
        rwkv7::set_error("a8w8_linear_static: cannot query the current device");
        return nullptr;
    }
    if (dev >= rwkv7::kMaxDevices) {
        rwkv7::set_error("a8w8_linear_static: device index %d is beyond the %d devices this library keeps per-device addresses for",
                         dev, rwkv7::kMaxDevices);
        return nullptr;
    }
    void* p = cache[dev].load(std::memory_order_acquire);
    if (p == nullptr) {
        cudaError_t e = cudaGetSymbolAddress(&p, g_a8w8_static_scratch);
        if (e != cudaSuccess || p == nullptr) {
            rwkv7::set_error("a8w8_linear_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(e));
            return nullptr;
        }
        cache[dev].store(p, std::memory_order_release);
    }
    return p;
}
}  // namespace

extern "C" int64_t rwkv7_a8w8_static_capacity_bytes(void) { return kStaticScratchBytes; }

extern "C" int rwkv7_a8w8_linear_static(const void* x, const int8_t* qw, const float* sw, const void* bias,
                                        const void* residual, void* out, int M, int K, int Nout, int dtype,
                                        void* stream) {
    RWKV7_REQUIRE(M > 0 && K > 0 && Nout > 0, RWKV7_ERR_INVALID, "a8w8_linear_static: sizes must be positive");
    const int64_t need = rwkv7_a8w8_workspace_bytes(M, K, Nout);
    RWKV7_REQUIRE(need <= kStaticScratchBytes, RWKV7_ERR_WORKSPACE,
                  "a8w8_linear_static: M=%d K=%d Nout=%d needs %lld bytes of scratch, the built-in array holds %lld; "
                  "use rwkv7_a8w8_linear with a caller-provided workspace",
                  M, K, Nout, (long long)need, (long long)kStaticScratchBytes);
    void* ws = static_scratch_ptr();
    if (ws == nullptr) return RWKV7_ERR_CUDA;
    // nothing in the scratch has to start at zero: the quantiser, the GEMM and the epilogue each overwrite
    // every element they later read
    return rwkv7_a8w8_linear(x, qw, sw, bias, residual, out, ws, kStaticScratchBytes, M, K, Nout, dtype, stream);
}
