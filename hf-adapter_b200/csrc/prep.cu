// Small fused element/row kernels around the recurrence: the rank-R LoRA linears with
// their activations, prefill state preparation, and attention-output preparation.
#include "common.cuh"

namespace rwkv7 {

// ---------------------------------------------------------------- dense_small
// out[rows,Nout] = act_out(act_in(x) . W^T + bias).  One warp per (row-block, output);
// the K loop is split across the 32 lanes with 128-bit loads.  ROWS rows share each
// weight load.  Used for the rank-R LoRA projections, where either K or Nout is small.
__device__ __forceinline__ float apply_act(float v, int act) {
    if (act == 1) return tanhf(v);
    if (act == 2) return sigmoidf_(v);
    return v;
}

struct DenseArgs {
    const void *x, *W, *bias;
    void* out;
    int rows, K, Nout, act_in, act_out;
};

template <typename T, int ROWS>
__global__ void __launch_bounds__(256) dense_small_kernel(const DenseArgs p) {
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n = blockIdx.x * 8 + warp;
    const int r0 = blockIdx.y * ROWS;
    if (n >= p.Nout) return;
    const T* W = reinterpret_cast<const T*>(p.W) + (size_t)n * p.K;
    const T* x = reinterpret_cast<const T*>(p.x);
    float acc[ROWS];
#pragma unroll
    for (int r = 0; r < ROWS; ++r) acc[r] = 0.f;
    for (int k0 = lane * 8; k0 < p.K; k0 += 256) {
        float w[8];
        load8(W + k0, w);
#pragma unroll
        for (int r = 0; r < ROWS; ++r) {
            if (r0 + r < p.rows) {
                float xv[8];
                load8(x + (size_t)(r0 + r) * p.K + k0, xv);
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    float t = xv[e];
                    if (p.act_in) t = round_to<T>(apply_act(t, p.act_in));
                    acc[r] = fmaf(t, w[e], acc[r]);
                }
            }
        }
    }
    const float bias = p.bias ? to_f<T>(reinterpret_cast<const T*>(p.bias)[n]) : 0.f;
#pragma unroll
    for (int r = 0; r < ROWS; ++r) {
        const float s = group_sum<32>(acc[r]);
        if (lane == 0 && r0 + r < p.rows) {
            float o = s + bias;
            if (p.act_out) o = apply_act(round_to<T>(o), p.act_out);
            reinterpret_cast<T*>(p.out)[(size_t)(r0 + r) * p.Nout + n] = from_f<T>(o);
        }
    }
}

// ---------------------------------------------------------------- prefill_state_prep
struct PrepArgs {
    const void *w_raw, *k_raw, *v_raw, *a, *k_k, *k_a, *v_first, *v_gate;
    float* w_out;
    void *k_out, *v_out, *kk_out;
    int H, a_is_raw, v_gate_is_raw, log_decay;
    long long total_heads;  // rows * H
};

// one 16-lane group per (row, head): 4 columns per lane
template <typename T>
__global__ void __launch_bounds__(256) state_prep_kernel(const PrepArgs p) {
    const long long gidx = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 4;
    const int l16 = threadIdx.x & 15;
    const bool active = gidx < p.total_heads;
    const long long g = active ? gidx : p.total_heads - 1;  // keep the shuffle groups converged
    const int h = (int)(g % p.H);
    const size_t off = (size_t)g * 64 + l16 * 4;
    const int hoff = h * 64 + l16 * 4;
    float w[4] = {0.f, 0.f, 0.f, 0.f}, k[4], v[4], a[4], ks[4], ka[4];
    if (p.w_raw) load4(reinterpret_cast<const T*>(p.w_raw) + off, w);  // absent: K / V / KK only (the scan takes raw w)
    load4(reinterpret_cast<const T*>(p.k_raw) + off, k);
    load4(reinterpret_cast<const T*>(p.v_raw) + off, v);
    load4(reinterpret_cast<const T*>(p.a) + off, a);
    load4(reinterpret_cast<const T*>(p.k_k) + hoff, ks);
    load4(reinterpret_cast<const T*>(p.k_a) + hoff, ka);
    float kk[4], n2 = 0.f;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        if (p.a_is_raw) a[c] = sigmoidf_(a[c]);
        kk[c] = k[c] * ks[c];
        n2 += kk[c] * kk[c];
    }
    n2 = group_sum<16>(n2);
    const float inv = 1.0f / fmaxf(sqrtf(n2), 1e-12f);
    float wo[4], ko[4];
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        kk[c] *= inv;
        ko[c] = k[c] * (1.0f + (a[c] - 1.0f) * ka[c]);
        const float lw = -0.606531f * sigmoidf_(w[c]);
        wo[c] = p.log_decay ? lw : expf(lw);
    }
    if (p.v_first && p.v_gate) {
        float vf[4], vg[4];
        load4(reinterpret_cast<const T*>(p.v_first) + off, vf);
        load4(reinterpret_cast<const T*>(p.v_gate) + off, vg);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            if (p.v_gate_is_raw) vg[c] = sigmoidf_(vg[c]);
            v[c] = v[c] + (vf[c] - v[c]) * vg[c];
        }
    }
    if (active) {
        if (p.w_out) *reinterpret_cast<float4*>(p.w_out + off) = make_float4(wo[0], wo[1], wo[2], wo[3]);
        store4(reinterpret_cast<T*>(p.k_out) + off, ko);
        store4(reinterpret_cast<T*>(p.v_out) + off, v);
        store4(reinterpret_cast<T*>(p.kk_out) + off, kk);
    }
}

// ---------------------------------------------------------------- attn_output_prepare
struct OutPrepArgs {
    const void *rec, *r, *k, *v, *g, *r_k, *gn_w, *gn_b;
    void* out;
    int H;
    float eps;
    long long total_heads;
};

template <typename T>
__global__ void __launch_bounds__(256) output_prepare_kernel(const OutPrepArgs p) {
    const long long gidx = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 4;
    const int l16 = threadIdx.x & 15;
    const bool active = gidx < p.total_heads;
    const long long g = active ? gidx : p.total_heads - 1;
    const int h = (int)(g % p.H);
    const size_t off = (size_t)g * 64 + l16 * 4;
    const int hoff = h * 64 + l16 * 4;
    float y[4], r[4], k[4], v[4], gt[4], rk[4], gw[4], gb[4];
    load4(reinterpret_cast<const T*>(p.rec) + off, y);
    load4(reinterpret_cast<const T*>(p.r) + off, r);
    load4(reinterpret_cast<const T*>(p.k) + off, k);
    load4(reinterpret_cast<const T*>(p.v) + off, v);
    load4(reinterpret_cast<const T*>(p.g) + off, gt);
    load4(reinterpret_cast<const T*>(p.r_k) + hoff, rk);
    load4(reinterpret_cast<const T*>(p.gn_w) + hoff, gw);
    load4(reinterpret_cast<const T*>(p.gn_b) + hoff, gb);
    const float mean = group_sum<16>(y[0] + y[1] + y[2] + y[3]) * (1.0f / 64);
    float q = 0.f, corr = 0.f;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
        y[c] -= mean;
        q += y[c] * y[c];
        corr += r[c] * k[c] * rk[c];
    }
    const float rstd = rsqrtf(group_sum<16>(q) * (1.0f / 64) + p.eps);
    corr = group_sum<16>(corr);
    float o[4];
#pragma unroll
    for (int c = 0; c < 4; ++c) o[c] = (y[c] * rstd * gw[c] + gb[c] + corr * v[c]) * gt[c];
    if (active) store4(reinterpret_cast<T*>(p.out) + off, o);
}

}  // namespace rwkv7

using namespace rwkv7;

extern "C" int rwkv7_dense_small(const void* x, const void* W, const void* bias, void* out, int rows, int K, int Nout,
                                 int act_in, int act_out, int dtype, void* stream) {
    RWKV7_REQUIRE(rows > 0 && K > 0 && Nout > 0, RWKV7_ERR_INVALID, "dense_small: sizes must be positive");
    RWKV7_REQUIRE(K % 8 == 0, RWKV7_ERR_UNSUPPORTED, "dense_small: K must be a multiple of 8 (got %d)", K);
    RWKV7_REQUIRE(x && W && out, RWKV7_ERR_INVALID, "dense_small: null pointer");
    RWKV7_REQUIRE(act_in >= 0 && act_in <= 2 && act_out >= 0 && act_out <= 2, RWKV7_ERR_INVALID, "dense_small: bad activation code");
    RWKV7_REQUIRE(aligned(x, 16) && aligned(W, 16), RWKV7_ERR_ALIGN, "dense_small: x and W must be 16-byte aligned");
    DenseArgs p{x, W, bias, out, rows, K, Nout, act_in, act_out};
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    constexpr int ROWS = 8;
    dim3 grid((Nout + 7) / 8, (rows + ROWS - 1) / ROWS);
    RWKV7_DISPATCH_DTYPE(dtype, T, {
        dense_small_kernel<T, ROWS><<<grid, 256, 0, st>>>(p);
        return check_launch("dense_small_kernel");
    });
    return RWKV7_OK;
}

extern "C" int rwkv7_prefill_state_prep(const void* w_raw, const void* k_raw, const void* v_raw, const void* a,
                                        const void* k_k, const void* k_a, const void* v_first, const void* v_gate,
                                        float* w_out, void* k_out, void* v_out, void* kk_out, int rows, int H, int N,
                                        int a_is_raw, int v_gate_is_raw, int log_decay, int dtype, void* stream) {
    RWKV7_REQUIRE(N == 64, RWKV7_ERR_UNSUPPORTED, "prefill_state_prep: head size must be 64, got %d", N);
    RWKV7_REQUIRE(rows > 0 && H > 0, RWKV7_ERR_INVALID, "prefill_state_prep: sizes must be positive");
    RWKV7_REQUIRE(k_raw && v_raw && a && k_k && k_a && k_out && v_out && kk_out, RWKV7_ERR_INVALID,
                  "prefill_state_prep: null pointer");
    RWKV7_REQUIRE((w_raw == nullptr) == (w_out == nullptr), RWKV7_ERR_INVALID,
                  "prefill_state_prep: w_raw and w_out must be given together (both NULL = no decay output)");
    RWKV7_REQUIRE((v_first == nullptr) == (v_gate == nullptr), RWKV7_ERR_INVALID,
                  "prefill_state_prep: v_first and v_gate must be given together");
    const void* ptrs[] = {w_raw, k_raw, v_raw, a, k_k, k_a, v_first, v_gate, w_out, k_out, v_out, kk_out};
    for (const void* q : ptrs) RWKV7_REQUIRE(aligned(q, 16), RWKV7_ERR_ALIGN, "prefill_state_prep: unaligned pointer");
    PrepArgs p{w_raw, k_raw, v_raw, a, k_k, k_a, v_first, v_gate, w_out, k_out, v_out, kk_out,
               H, a_is_raw, v_gate_is_raw, log_decay, (long long)rows * H};
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const long long threads = p.total_heads * 16;
    const int grid = (int)((threads + 255) / 256);
    RWKV7_DISPATCH_DTYPE(dtype, T, {
        state_prep_kernel<T><<<grid, 256, 0, st>>>(p);
        return check_launch("state_prep_kernel");
    });
    return RWKV7_OK;
}

// y = max(x, 0)^2 elementwise (in place allowed), 8 elements per thread
template <typename T>
__global__ void __launch_bounds__(256) relu2_kernel(const T* __restrict__ x, T* __restrict__ y, long long nvec) {
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < nvec; i += (long long)gridDim.x * blockDim.x) {
        float v[8];
        load8(x + i * 8, v);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
            const float r = fmaxf(round_to<T>(v[e]), 0.f);
            v[e] = r * r;
        }
        store8(y + i * 8, v);
    }
}

extern "C" int rwkv7_relu2(const void* x, void* y, long long n, int dtype, void* stream) {
    RWKV7_REQUIRE(n > 0 && n % 8 == 0, RWKV7_ERR_UNSUPPORTED, "relu2: element count must be a positive multiple of 8");
    RWKV7_REQUIRE(x && y, RWKV7_ERR_INVALID, "relu2: null pointer");
    RWKV7_REQUIRE(aligned(x, 16) && aligned(y, 16), RWKV7_ERR_ALIGN, "relu2: unaligned pointer");
    const long long nvec = n / 8;
    const int grid = (int)((nvec + 255) / 256 < 148LL * 32 ? (nvec + 255) / 256 : 148LL * 32);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    RWKV7_DISPATCH_DTYPE(dtype, T, {
        relu2_kernel<T><<<grid, 256, 0, st>>>(reinterpret_cast<const T*>(x), reinterpret_cast<T*>(y), nvec);
        return check_launch("relu2_kernel");
    });
    return RWKV7_OK;
}

extern "C" int rwkv7_attn_output_prepare(const void* recurrent, const void* r, const void* k, const void* v,
                                         const void* g, const void* r_k, const void* gn_w, const void* gn_b, void* out,
                                         int rows, int H, int N, float eps, int dtype, void* stream) {
    RWKV7_REQUIRE(N == 64, RWKV7_ERR_UNSUPPORTED, "attn_output_prepare: head size must be 64, got %d", N);
    RWKV7_REQUIRE(rows > 0 && H > 0, RWKV7_ERR_INVALID, "attn_output_prepare: sizes must be positive");
    RWKV7_REQUIRE(recurrent && r && k && v && g && r_k && gn_w && gn_b && out, RWKV7_ERR_INVALID,
                  "attn_output_prepare: null pointer");
    const void* ptrs[] = {recurrent, r, k, v, g, r_k, gn_w, gn_b, out};
    for (const void* q : ptrs) RWKV7_REQUIRE(aligned(q, 16), RWKV7_ERR_ALIGN, "attn_output_prepare: unaligned pointer");
    OutPrepArgs p{recurrent, r, k, v, g, r_k, gn_w, gn_b, out, H, eps, (long long)rows * H};
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const long long threads = p.total_heads * 16;
    const int grid = (int)((threads + 255) / 256);
    RWKV7_DISPATCH_DTYPE(dtype, T, {
        output_prepare_kernel<T><<<grid, 256, 0, st>>>(p);
        return check_launch("output_prepare_kernel");
    });
    return RWKV7_OK;
}
