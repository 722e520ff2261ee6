// Grouped small GEMM for the LoRA projections of a decode step (up to 64 activation rows):
//
//   out_p[M, Nout_p] = act_p( x_p[M, K_p] . W_p[Nout_p, K_p]^T + bias_p )      p = 0..n_problems-1
//
// One launch covers the four rank-R "down" projections (K = d_model, Nout = rank) or the four "up"
// projections (K = rank, Nout = attention width) of a layer.  These matrices are tiny (a few MB per
// layer in total), so the kernel is built for latency: warp-level HMMA (mma.sync m16n8k16, fp32
// accumulate) on 64 x 64 output tiles, cp.async double-buffered 64-wide K chunks with an XOR swizzle
// for conflict-free ldmatrix, and split-K across a thread-block cluster whose partial tiles are
// reduced through distributed shared memory in fixed rank order (deterministic, no scratch memory).
#include <cooperative_groups.h>

#include "common.cuh"

namespace cg = cooperative_groups;

namespace rwkv7 {

constexpr int kMaxProblems = 4;
constexpr int LT = 64;         // tile rows (activations) and tile columns (outputs)
constexpr int LK = 64;         // K chunk
constexpr int LTHREADS = 128;  // 4 warps as 2 x 2, warp tile 32 x 32

struct GroupArgs {
    const void* x[kMaxProblems];
    const void* W[kMaxProblems];
    const void* bias[kMaxProblems];
    void* out[kMaxProblems];
    int K[kMaxProblems], Nout[kMaxProblems], act[kMaxProblems];
    int M, splits, max_tiles;
};

__device__ __forceinline__ void lcp16(void* smem, const void* g, bool valid) {
    unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    int sz = valid ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(s), "l"(g), "r"(sz));
}
__device__ __forceinline__ void lldm4(uint32_t (&r)[4], const void* smem) {
    unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];\n"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(s));
}
template <typename T> __device__ __forceinline__ void hmma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1);
template <> __device__ __forceinline__ void hmma<__half>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
template <> __device__ __forceinline__ void hmma<__nv_bfloat16>(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};\n"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// tile of 64 rows x 64 k (2-byte elements): rows of 128 bytes = 8 chunks; chunk c of row r at chunk c ^ (r & 7)
__device__ __forceinline__ int lswz(int row, int chunk) { return row * 128 + ((chunk ^ (row & 7)) << 4); }

__device__ __forceinline__ float lora_act(float v, int act) {
    if (act == 1) return tanhf(v);
    if (act == 2) return sigmoidf_(v);
    return v;
}

template <typename T>
__global__ void __launch_bounds__(LTHREADS) small_gemm_group_kernel(const GroupArgs p) {
    __shared__ __align__(128) unsigned char sX[2][LT * 128];
    __shared__ __align__(128) unsigned char sW[2][LT * 128];
    __shared__ __align__(16) float sP[LT * LT];  // partial tile for the split-K reduction

    // launched programmatically: resident under the tail of the preceding kernel of the stream, everything below after it
    grid_dependency_wait();
    if (threadIdx.x == 0) grid_launch_dependents();
    const int prob = blockIdx.y;
    const int K = p.K[prob], Nout = p.Nout[prob];
    const int n0 = (blockIdx.x % p.max_tiles) * LT;
    const int r0 = (blockIdx.x / p.max_tiles) * LT;  // activation row block
    if (n0 >= Nout) return;  // whole cluster shares blockIdx.x / y, so it leaves together
    const int split = blockIdx.z, S = p.splits;
    const int chunks_total = (K + LK - 1) / LK;
    const int chunks_per = (chunks_total + S - 1) / S;
    const int c_begin = split * chunks_per;
    const int c_end = min(chunks_total, c_begin + chunks_per);
    const T* X = reinterpret_cast<const T*>(p.x[prob]);
    const T* W = reinterpret_cast<const T*>(p.W[prob]);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int wm = warp >> 1, wn = warp & 1;

    float acc[2][4][4];
#pragma unroll
    for (int i = 0; i < 2; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int e = 0; e < 4; ++e) acc[i][j][e] = 0.f;

    auto load_chunk = [&](int buf, int c) {
        const int k0 = c * LK;
#pragma unroll
        for (int it = 0; it < 4; ++it) {  // 64 rows x 8 chunks = 512 chunks per operand, 128 threads
            const int idx = tid + it * LTHREADS;
            const int row = idx >> 3, ch = idx & 7;
            const bool kin = (k0 + ch * 8) < K;
            const bool vx = kin && (r0 + row) < p.M;
            const bool vw = kin && (n0 + row) < Nout;
            lcp16(&sX[buf][lswz(row, ch)], vx ? X + (size_t)(r0 + row) * K + k0 + ch * 8 : X, vx);
            lcp16(&sW[buf][lswz(row, ch)], vw ? W + (size_t)(n0 + row) * K + k0 + ch * 8 : W, vw);
        }
        asm volatile("cp.async.commit_group;\n" ::);
    };

    if (c_begin < c_end) load_chunk(0, c_begin);
    for (int c = c_begin; c < c_end; ++c) {
        const int buf = (c - c_begin) & 1;
        if (c + 1 < c_end) {
            load_chunk(buf ^ 1, c + 1);
            asm volatile("cp.async.wait_group 1;\n" ::);
        } else {
            asm volatile("cp.async.wait_group 0;\n" ::);
        }
        __syncthreads();
#pragma unroll
        for (int ks = 0; ks < LK / 16; ++ks) {
            uint32_t af[2][4], bf[2][4];
#pragma unroll
            for (int i = 0; i < 2; ++i) {
                const int row = wm * 32 + i * 16 + (lane & 15);
                lldm4(af[i], &sX[buf][lswz(row, ks * 2 + (lane >> 4))]);
            }
#pragma unroll
            for (int j = 0; j < 2; ++j) {
                const int row = wn * 32 + j * 16 + (lane & 7) + ((lane >> 4) << 3);
                lldm4(bf[j], &sW[buf][lswz(row, ks * 2 + ((lane >> 3) & 1))]);
            }
#pragma unroll
            for (int i = 0; i < 2; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) hmma<T>(acc[i][j], af[i], bf[j >> 1][(j & 1) * 2], bf[j >> 1][(j & 1) * 2 + 1]);
        }
        __syncthreads();
    }

    const int gid = lane >> 2, tig = lane & 3;
    cg::cluster_group cluster = cg::this_cluster();
    if (S > 1) {
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j)
#pragma unroll
                for (int hh = 0; hh < 2; ++hh) {
                    const int r = wm * 32 + i * 16 + gid + hh * 8, cidx = wn * 32 + j * 8 + tig * 2;
                    *reinterpret_cast<float2*>(&sP[r * LT + cidx]) = make_float2(acc[i][j][hh * 2], acc[i][j][hh * 2 + 1]);
                }
        cluster.sync();
        // rank `split` finishes rows [split*LT/S, (split+1)*LT/S)
        const int rows_per = LT / S;
        const T* bias = reinterpret_cast<const T*>(p.bias[prob]);
        T* out = reinterpret_cast<T*>(p.out[prob]);
        for (int idx = tid; idx < rows_per * LT; idx += LTHREADS) {
            const int r = split * rows_per + idx / LT, cidx = idx % LT;
            float v = 0.f;
            for (int q = 0; q < S; ++q) v += cluster.map_shared_rank(sP, q)[r * LT + cidx];
            if (r0 + r < p.M && n0 + cidx < Nout) {
                if (bias) v += to_f<T>(bias[n0 + cidx]);
                v = round_to<T>(v);
                if (p.act[prob]) v = lora_act(v, p.act[prob]);
                out[(size_t)(r0 + r) * Nout + n0 + cidx] = from_f<T>(v);
            }
        }
        cluster.sync();
    } else {
        const T* bias = reinterpret_cast<const T*>(p.bias[prob]);
        T* out = reinterpret_cast<T*>(p.out[prob]);
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
            for (int j = 0; j < 4; ++j)
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const int r = wm * 32 + i * 16 + gid + (e >> 1) * 8, cidx = n0 + wn * 32 + j * 8 + tig * 2 + (e & 1);
                    if (r0 + r < p.M && cidx < Nout) {
                        float v = acc[i][j][e];
                        if (bias) v += to_f<T>(bias[cidx]);
                        v = round_to<T>(v);
                        if (p.act[prob]) v = lora_act(v, p.act[prob]);
                        out[(size_t)(r0 + r) * Nout + cidx] = from_f<T>(v);
                    }
                }
    }
}

}  // namespace rwkv7

using namespace rwkv7;

extern "C" int rwkv7_small_gemm_group(int n_problems, const void* const* x, const void* const* W, const void* const* bias,
                                      void* const* out, const int* K, const int* Nout, const int* act_out, int M, int dtype,
                                      void* stream) {
    RWKV7_REQUIRE(n_problems >= 1 && n_problems <= kMaxProblems, RWKV7_ERR_INVALID, "small_gemm_group: 1..%d problems", kMaxProblems);
    RWKV7_REQUIRE(M >= 1 && M <= 16384, RWKV7_ERR_UNSUPPORTED, "small_gemm_group: M must be in 1..16384 (got %d)", M);
    const int row_blocks = (M + LT - 1) / LT;
    RWKV7_REQUIRE(dtype == RWKV7_F16 || dtype == RWKV7_BF16, RWKV7_ERR_UNSUPPORTED, "small_gemm_group: fp16 / bf16 only");
    RWKV7_REQUIRE(x && W && out && K && Nout && act_out, RWKV7_ERR_INVALID, "small_gemm_group: null argument array");
    GroupArgs a{};
    int max_tiles = 0, max_k = 0;
    for (int i = 0; i < n_problems; ++i) {
        RWKV7_REQUIRE(x[i] && W[i] && out[i], RWKV7_ERR_INVALID, "small_gemm_group: null pointer in problem %d", i);
        RWKV7_REQUIRE(K[i] > 0 && Nout[i] > 0 && K[i] % 8 == 0, RWKV7_ERR_UNSUPPORTED,
                      "small_gemm_group: K must be a positive multiple of 8 (problem %d: K=%d Nout=%d)", i, K[i], Nout[i]);
        RWKV7_REQUIRE(act_out[i] >= 0 && act_out[i] <= 2, RWKV7_ERR_INVALID, "small_gemm_group: bad activation code");
        RWKV7_REQUIRE(aligned(x[i], 16) && aligned(W[i], 16), RWKV7_ERR_ALIGN, "small_gemm_group: x and W must be 16-byte aligned");
        a.x[i] = x[i]; a.W[i] = W[i]; a.bias[i] = bias ? bias[i] : nullptr; a.out[i] = out[i];
        a.K[i] = K[i]; a.Nout[i] = Nout[i]; a.act[i] = act_out[i];
        max_tiles = max_tiles > (Nout[i] + LT - 1) / LT ? max_tiles : (Nout[i] + LT - 1) / LT;
        max_k = max_k > K[i] ? max_k : K[i];
    }
    a.M = M;
    // split K across a cluster when there are few output tiles and a long K (the "down" projections)
    int splits = 1;
    const int chunks = (max_k + LK - 1) / LK;
    while (splits < 8 && max_tiles * row_blocks * n_problems * splits * 2 <= 160 && chunks / (splits * 2) >= 4) splits *= 2;
    a.splits = splits;
    a.max_tiles = max_tiles;
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(max_tiles * row_blocks, n_problems, splits);
    cfg.blockDim = dim3(LTHREADS);
    cfg.dynamicSmemBytes = 0;
    cfg.stream = static_cast<cudaStream_t>(stream);
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = splits;
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = programmatic_launch_enabled() ? 2 : 1;
    cudaError_t e;
    if (dtype == RWKV7_F16) e = cudaLaunchKernelEx(&cfg, small_gemm_group_kernel<__half>, a);
    else e = cudaLaunchKernelEx(&cfg, small_gemm_group_kernel<__nv_bfloat16>, a);
    RWKV7_REQUIRE(e == cudaSuccess, RWKV7_ERR_CUDA, "small_gemm_group launch: %s", cudaGetErrorString(e));
    return RWKV7_OK;
}
