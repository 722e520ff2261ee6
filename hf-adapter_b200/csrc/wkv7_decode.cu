// WKV-7 single-token recurrence for decode: one CTA per (sequence, head).
//
// The 64x64 fp32 state tile is streamed HBM -> registers -> HBM exactly once
// (16 KiB in, 16 KiB out); everything else the decode layer does around the
// recurrence (decay, kk normalisation, k adjustment, v interpolation, a/w LoRA
// biases, GroupNorm, bonus term, output gate) is folded into the same pass so
// no intermediate vector touches HBM.  The kernel is HBM-bound: algorithmic
// traffic is 2*64*64*4 + ~7*64*sizeof(T) bytes per (sequence, head).
//
// The state may also be stored in fp16 (the reference's opt-in FP16-state lanes: the Triton output-prepare kernels
// load it to fp32 and round the result back, rwkv7_hf/fused_recurrent_update.py:655-699; the native_wkv_fp16
// extension additionally dithers the decay, rwkv7_hf/native_wkv_fp16.py:118-128): the arithmetic stays fp32, the
// traffic halves.
//
// Thread map (128 threads): lane16 = tid & 15 owns columns 4*lane16..+3 (key
// index j), rowgroup = tid >> 4 owns rows rowgroup + 8*it (value index i), so a
// warp instruction touches two full 256-byte state rows = 512 contiguous bytes.
#include "common.cuh"

namespace rwkv7 {

constexpr int kN = 64;
constexpr int kStepThreads = 128;

enum StepMode { kUpdate = 0, kPrepare = 1, kRaw = 2 };

struct StepArgs {
    const void *r, *w, *k, *v, *kk, *a;
    const void* state_in;  // fp32 or fp16 [B,H,64,64]
    void* state_out;
    void* out;
    const void *g, *r_k, *gn_w, *gn_b;
    const void *k_k, *k_a;
    const void *w_bias, *a_bias, *v_first, *v_gate, *v_gate_bias;
    void* v_out;
    int a_is_raw, v_gate_is_raw;
    int H;
    float eps;
    int prefetch_state;  // load the state tile before the grid-dependency wait (state_prefetch argument of the raw entry point)
    const int* slots;    // state pool: row b of the batch lives in pool row slots[b] (state, v_first / v_out, elapsed); NULL = row b
    const int* elapsed;  // fp16 state, raw mode: per-sequence step counters [B] that phase the decay dither (NULL = no dither)
};

// Deterministic zero-mean rotator of the reference's FP16-state kernel (rwkv7_hf/native_wkv_fp16.py:118-121): the
// decay of a half-precision state is often smaller than half an ulp of the entry it multiplies, which would freeze it
// under round-to-nearest; a pseudo-random offset of up to +-2^-10 on (decay - 1), different for every channel and
// step, makes the rounding unbiased on average.
__device__ __forceinline__ float rotator1(int x) {
    const uint32_t bits = 2654435769u * static_cast<uint32_t>(x);
    return 4.547473508864641e-13f * static_cast<float>(static_cast<int32_t>(bits));
}

template <typename TS> struct StateIO;
template <> struct StateIO<float> {
    static __device__ __forceinline__ float4 load(const void* base, size_t off) {
        return *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(base) + off);  // plain load: may alias state_out
    }
    // streaming store: the new state is not read again before the next token, so it should not linger in L2 and
    // be written back under the kernels that follow (measured: -8 % time)
    static __device__ __forceinline__ void store(void* base, size_t off, const float4& s) {
        __stcs(reinterpret_cast<float4*>(reinterpret_cast<float*>(base) + off), s);
    }
};
template <> struct StateIO<__half> {
    static __device__ __forceinline__ float4 load(const void* base, size_t off) {
        const uint2 u = *reinterpret_cast<const uint2*>(reinterpret_cast<const __half*>(base) + off);
        const float2 a = __half22float2(*reinterpret_cast<const __half2*>(&u.x));
        const float2 b = __half22float2(*reinterpret_cast<const __half2*>(&u.y));
        return make_float4(a.x, a.y, b.x, b.y);
    }
    static __device__ __forceinline__ void store(void* base, size_t off, const float4& s) {
        const __half2 a = __floats2half2_rn(s.x, s.y), b = __floats2half2_rn(s.z, s.w);
        uint2 u;
        u.x = *reinterpret_cast<const uint32_t*>(&a);
        u.y = *reinterpret_cast<const uint32_t*>(&b);
        __stcs(reinterpret_cast<uint2*>(reinterpret_cast<__half*>(base) + off), u);
    }
};

template <typename T, typename TW, int MODE, typename TS, bool POOL = false>
__global__ void __launch_bounds__(kStepThreads, 8) wkv7_step_kernel(const StepArgs p) {  // 64 registers: 8 CTAs per SM (measured: 7 -> 8 CTAs is -9 % time)
    const int bh = blockIdx.x;
    const int h = bh % p.H;
    const int tid = threadIdx.x;
    const int l16 = tid & 15;
    const int rg = tid >> 4;
    const size_t vbase = (size_t)bh * kN;
    // with a state pool the recurrent rows of sequence b sit at pool row slots[b]; the step's operands stay batch-ordered
    // (a template parameter, not a run-time test: the dense kernel keeps its exact instruction stream and registers)
    const int srow = POOL ? __ldg(p.slots + bh / p.H) : bh / p.H;
    const size_t sbh = POOL ? (size_t)srow * p.H + h : (size_t)bh;
    const size_t vsbase = sbh * kN;
    const int hbase = h * kN;
    const int c0 = l16 * 4;

    __shared__ float s_v[kN];
    __shared__ float s_y[kN];

    // Launched programmatically: resident under the tail of the preceding kernel.  By default everything waits for it.
    if (!p.prefetch_state) grid_dependency_wait();
    // ---- state tile: issue all 8 row loads first (memory-level parallelism)
    const size_t sbase = sbh * kN * kN;
    float4 S[8];
#pragma unroll
    for (int it = 0; it < 8; ++it) S[it] = StateIO<TS>::load(p.state_in, sbase + (size_t)(it * 8 + rg) * kN + c0);

    // With the state-prefetch option the loads above are already in flight while the preceding kernel (the r/k/v
    // projection of a decode step) finishes: the caller promises that kernel does not write the state, and every
    // kernel of this library releases its successor only after its own wait, so whatever wrote the state earlier has
    // completed.  Everything below reads the preceding kernel's output.
    if (p.prefetch_state) grid_dependency_wait();
    if (tid == 0) grid_launch_dependents();  // the output projection sets up and streams weights under this grid's tail

    // ---- column-indexed vectors (4 columns per thread)
    float r[4], w[4], k[4], kk[4], a[4];
    load4(reinterpret_cast<const T*>(p.r) + vbase + c0, r);
    load4(reinterpret_cast<const T*>(p.a) + vbase + c0, a);
    if constexpr (MODE == kRaw) {
        float wr[4], kr[4], ks[4], ka[4];
        load4(reinterpret_cast<const T*>(p.w) + vbase + c0, wr);
        load4(reinterpret_cast<const T*>(p.k) + vbase + c0, kr);
        load4(reinterpret_cast<const T*>(p.k_k) + hbase + c0, ks);
        load4(reinterpret_cast<const T*>(p.k_a) + hbase + c0, ka);
        if (p.w_bias) {
            float wb[4];
            load4(reinterpret_cast<const T*>(p.w_bias) + hbase + c0, wb);
#pragma unroll
            for (int c = 0; c < 4; ++c) wr[c] = round_to<T>(wr[c] + wb[c]);
        }
        if (p.a_is_raw) {
            float ab[4] = {0.f, 0.f, 0.f, 0.f};
            if (p.a_bias) load4(reinterpret_cast<const T*>(p.a_bias) + hbase + c0, ab);
#pragma unroll
            for (int c = 0; c < 4; ++c) a[c] = round_to<T>(sigmoidf_(round_to<T>(a[c] + ab[c])));
        }
        float n2 = 0.f;
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            kk[c] = kr[c] * ks[c];
            n2 += kk[c] * kk[c];
        }
        n2 = group_sum<16>(n2);
        const float inv = 1.0f / fmaxf(sqrtf(n2), 1e-12f);
#pragma unroll
        for (int c = 0; c < 4; ++c) {
            kk[c] *= inv;
            k[c] = kr[c] * (1.0f + (a[c] - 1.0f) * ka[c]);
            w[c] = decay_from_raw(wr[c]);
        }
        if constexpr (sizeof(TS) == 2) {
            if (p.elapsed != nullptr) {  // (decay - 1 + rotator) rounded to fp16, as the reference's FP16-state kernel forms it
                const int phase = p.elapsed[srow] + hbase + c0;
#pragma unroll
                for (int c = 0; c < 4; ++c) w[c] = 1.0f + __half2float(__float2half_rn(w[c] - 1.0f + rotator1(phase + c)));
            }
        }
    } else {
        load4(reinterpret_cast<const TW*>(p.w) + vbase + c0, w);
        load4(reinterpret_cast<const T*>(p.k) + vbase + c0, k);
        load4(reinterpret_cast<const T*>(p.kk) + vbase + c0, kk);
    }
    float kka[4];
#pragma unroll
    for (int c = 0; c < 4; ++c) kka[c] = kk[c] * a[c];

    // ---- row-indexed value vector (with the optional v_first interpolation)
    if (tid < kN) {
        float vv = to_f<T>(reinterpret_cast<const T*>(p.v)[vbase + tid]);
        if constexpr (MODE == kRaw) {
            if (p.v_first != nullptr && p.v_gate != nullptr) {
                float gate = to_f<T>(reinterpret_cast<const T*>(p.v_gate)[vbase + tid]);
                if (p.v_gate_is_raw) {
                    const float gb = p.v_gate_bias ? to_f<T>(reinterpret_cast<const T*>(p.v_gate_bias)[hbase + tid]) : 0.f;
                    gate = round_to<T>(sigmoidf_(round_to<T>(gate + gb)));
                }
                const float vf = to_f<T>(reinterpret_cast<const T*>(p.v_first)[vsbase + tid]);
                vv = round_to<T>(vv + (vf - vv) * gate);
            }
            if (p.v_out) reinterpret_cast<T*>(p.v_out)[vsbase + tid] = from_f<T>(vv);
        }
        s_v[tid] = vv;
    }
    __syncthreads();

    // ---- the recurrence, row by row
#pragma unroll
    for (int it = 0; it < 8; ++it) {
        const int i = it * 8 + rg;
        float4 s = S[it];
        float sa = s.x * kk[0] + s.y * kk[1] + s.z * kk[2] + s.w * kk[3];
        sa = group_sum<16>(sa);
        const float vi = s_v[i];
        s.x = s.x * w[0] + vi * k[0] - sa * kka[0];
        s.y = s.y * w[1] + vi * k[1] - sa * kka[1];
        s.z = s.z * w[2] + vi * k[2] - sa * kka[2];
        s.w = s.w * w[3] + vi * k[3] - sa * kka[3];
        StateIO<TS>::store(p.state_out, sbase + (size_t)i * kN + c0, s);
        if constexpr (sizeof(TS) == 2) {  // the output is formed from the state as stored
            s.x = round_to<__half>(s.x); s.y = round_to<__half>(s.y); s.z = round_to<__half>(s.z); s.w = round_to<__half>(s.w);
        }
        float y = s.x * r[0] + s.y * r[1] + s.z * r[2] + s.w * r[3];
        y = group_sum<16>(y);
        if (l16 == 0) s_y[i] = y;
    }

    float corr = 0.f;
    if constexpr (MODE != kUpdate) {
        float rk[4];
        load4(reinterpret_cast<const T*>(p.r_k) + hbase + c0, rk);
#pragma unroll
        for (int c = 0; c < 4; ++c) corr += r[c] * k[c] * rk[c];
        corr = group_sum<16>(corr);
    }
    __syncthreads();

    if (tid < kN) {
        T* out = reinterpret_cast<T*>(p.out) + vbase;
        const float y = s_y[tid];
        if constexpr (MODE == kUpdate) {
            out[tid] = from_f<T>(y);
        } else {
            // both warps 0 and 1 compute the head statistics redundantly from shared memory
            const int lane = tid & 31;
            const float y0 = s_y[lane], y1 = s_y[lane + 32];
            const float mean = group_sum<32>(y0 + y1) * (1.0f / kN);
            const float d0 = y0 - mean, d1 = y1 - mean;
            const float var = group_sum<32>(d0 * d0 + d1 * d1) * (1.0f / kN);
            const float normed = (y - mean) * rsqrtf(var + p.eps);
            const float gw = to_f<T>(reinterpret_cast<const T*>(p.gn_w)[hbase + tid]);
            const float gb = to_f<T>(reinterpret_cast<const T*>(p.gn_b)[hbase + tid]);
            const float gate = to_f<T>(reinterpret_cast<const T*>(p.g)[vbase + tid]);
            out[tid] = from_f<T>((normed * gw + gb + corr * s_v[tid]) * gate);
        }
    }
}

template <typename T, typename TW, int MODE, typename TS = float, bool POOL = false>
static int launch_step(StepArgs p, int B, cudaStream_t st) {
    launch_programmatic(wkv7_step_kernel<T, TW, MODE, TS, POOL>, dim3(B * p.H), dim3(kStepThreads), 0, st, p);
    return check_launch("wkv7_step_kernel");
}

__global__ void advance_elapsed_kernel(int* elapsed, int B) {
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b < B) elapsed[b] += 1;
}

static int check_step_common(const StepArgs& p, int B, int H, int N) {
    RWKV7_REQUIRE(N == kN, RWKV7_ERR_UNSUPPORTED, "wkv7: head size must be 64, got %d", N);
    RWKV7_REQUIRE(B > 0 && H > 0, RWKV7_ERR_INVALID, "wkv7: B and H must be positive (B=%d H=%d)", B, H);
    RWKV7_REQUIRE(p.r && p.w && p.k && p.v && p.a && p.state_in && p.state_out && p.out, RWKV7_ERR_INVALID,
                  "wkv7: null tensor pointer");
    const void* ptrs[] = {p.r, p.w, p.k, p.v, p.a, p.kk, p.state_in, p.state_out, p.out, p.g, p.r_k, p.gn_w,
                          p.gn_b, p.k_k, p.k_a, p.w_bias, p.a_bias, p.v_first, p.v_gate, p.v_gate_bias, p.v_out};
    for (const void* q : ptrs) RWKV7_REQUIRE(aligned(q, 16), RWKV7_ERR_ALIGN, "wkv7: pointers must be 16-byte aligned");
    return RWKV7_OK;
}

}  // namespace rwkv7

using namespace rwkv7;

extern "C" int rwkv7_wkv7_update(const void* r, const void* w, const void* k, const void* v, const void* kk,
                                 const void* a, const float* state_in, float* state_out, void* y, int B, int H,
                                 int N, int dtype, int w_is_f32, void* stream) {
    StepArgs p{};
    p.r = r; p.w = w; p.k = k; p.v = v; p.kk = kk; p.a = a;
    p.state_in = state_in; p.state_out = state_out; p.out = y; p.H = H;
    RWKV7_REQUIRE(kk != nullptr, RWKV7_ERR_INVALID, "wkv7_update: kk is null");
    if (int e = check_step_common(p, B, H, N)) return e;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    RWKV7_DISPATCH_DTYPE(dtype, T, {
        if (w_is_f32) return launch_step<T, float, kUpdate>(p, B, st);
        return launch_step<T, T, kUpdate>(p, B, st);
    });
    return RWKV7_OK;
}

extern "C" int rwkv7_wkv7_output_prepare(const void* r, const void* w, const void* k, const void* v, const void* kk,
                                         const void* a, const float* state_in, float* state_out, const void* g,
                                         const void* r_k, const void* gn_w, const void* gn_b, void* out, int B,
                                         int H, int N, float eps, int dtype, int w_is_f32, void* stream) {
    StepArgs p{};
    p.r = r; p.w = w; p.k = k; p.v = v; p.kk = kk; p.a = a;
    p.state_in = state_in; p.state_out = state_out; p.out = out; p.H = H;
    p.g = g; p.r_k = r_k; p.gn_w = gn_w; p.gn_b = gn_b; p.eps = eps;
    RWKV7_REQUIRE(kk && g && r_k && gn_w && gn_b, RWKV7_ERR_INVALID, "wkv7_output_prepare: null tensor pointer");
    if (int e = check_step_common(p, B, H, N)) return e;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    RWKV7_DISPATCH_DTYPE(dtype, T, {
        if (w_is_f32) return launch_step<T, float, kPrepare>(p, B, st);
        return launch_step<T, T, kPrepare>(p, B, st);
    });
    return RWKV7_OK;
}

extern "C" int rwkv7_wkv7_output_prepare_raw(const void* r, const void* w_raw, const void* k_raw, const void* v,
                                             const void* a, const float* state_in, float* state_out, const void* g,
                                             const void* k_k, const void* k_a, const void* r_k, const void* gn_w,
                                             const void* gn_b, void* out, const void* w_bias, const void* a_bias,
                                             int a_is_raw, const void* v_first, const void* v_gate,
                                             const void* v_gate_bias, int v_gate_is_raw, void* v_out, int state_prefetch,
                                             int B, int H, int N, float eps, int dtype, void* stream) {
    StepArgs p{};
    p.r = r; p.w = w_raw; p.k = k_raw; p.v = v; p.a = a;
    p.state_in = state_in; p.state_out = state_out; p.out = out; p.H = H;
    p.g = g; p.r_k = r_k; p.gn_w = gn_w; p.gn_b = gn_b; p.eps = eps;
    p.k_k = k_k; p.k_a = k_a;
    p.w_bias = w_bias; p.a_bias = a_bias; p.a_is_raw = a_is_raw;
    p.v_first = v_first; p.v_gate = v_gate; p.v_gate_bias = v_gate_bias; p.v_gate_is_raw = v_gate_is_raw;
    p.v_out = v_out;
    p.prefetch_state = state_prefetch != 0;
    RWKV7_REQUIRE(g && r_k && gn_w && gn_b && k_k && k_a, RWKV7_ERR_INVALID,
                  "wkv7_output_prepare_raw: null tensor pointer");
    RWKV7_REQUIRE((v_first == nullptr) == (v_gate == nullptr), RWKV7_ERR_INVALID,
                  "wkv7_output_prepare_raw: v_first and v_gate must be given together");
    if (int e = check_step_common(p, B, H, N)) return e;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    RWKV7_DISPATCH_DTYPE(dtype, T, { return launch_step<T, T, kRaw>(p, B, st); });
    return RWKV7_OK;
}

// ---------------------------------------------------------------- state pool
extern "C" int rwkv7_wkv7_output_prepare_raw_pool(const void* r, const void* w_raw, const void* k_raw, const void* v,
                                                  const void* a, float* state_pool, const int32_t* slot_ids, const void* g,
                                                  const void* k_k, const void* k_a, const void* r_k, const void* gn_w,
                                                  const void* gn_b, void* out, const void* w_bias, const void* a_bias,
                                                  int a_is_raw, const void* v_first_pool, const void* v_gate,
                                                  const void* v_gate_bias, int v_gate_is_raw, void* v_out_pool,
                                                  int state_prefetch, int B, int H, int N, float eps, int dtype, void* stream) {
    StepArgs p{};
    p.r = r; p.w = w_raw; p.k = k_raw; p.v = v; p.a = a;
    p.state_in = state_pool; p.state_out = state_pool; p.out = out; p.H = H;
    p.g = g; p.r_k = r_k; p.gn_w = gn_w; p.gn_b = gn_b; p.eps = eps;
    p.k_k = k_k; p.k_a = k_a;
    p.w_bias = w_bias; p.a_bias = a_bias; p.a_is_raw = a_is_raw;
    p.v_first = v_first_pool; p.v_gate = v_gate; p.v_gate_bias = v_gate_bias; p.v_gate_is_raw = v_gate_is_raw;
    p.v_out = v_out_pool;
    p.prefetch_state = state_prefetch != 0;
    p.slots = slot_ids;
    RWKV7_REQUIRE(slot_ids && g && r_k && gn_w && gn_b && k_k && k_a, RWKV7_ERR_INVALID,
                  "wkv7_output_prepare_raw_pool: null tensor pointer");
    RWKV7_REQUIRE((v_first_pool == nullptr) == (v_gate == nullptr), RWKV7_ERR_INVALID,
                  "wkv7_output_prepare_raw_pool: v_first_pool and v_gate must be given together");
    if (int e = check_step_common(p, B, H, N)) return e;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    RWKV7_DISPATCH_DTYPE(dtype, T, { return launch_step<T, T, kRaw, float, true>(p, B, st); });
    return RWKV7_OK;
}

// ---------------------------------------------------------------- fp16 recurrent state
extern "C" int rwkv7_wkv7_output_prepare_f16state(const void* r, const void* w, const void* k, const void* v, const void* kk,
                                                  const void* a, const void* state_in, void* state_out, const void* g,
                                                  const void* r_k, const void* gn_w, const void* gn_b, void* out, int B,
                                                  int H, int N, float eps, int dtype, int w_is_f32, void* stream) {
    StepArgs p{};
    p.r = r; p.w = w; p.k = k; p.v = v; p.kk = kk; p.a = a;
    p.state_in = state_in; p.state_out = state_out; p.out = out; p.H = H;
    p.g = g; p.r_k = r_k; p.gn_w = gn_w; p.gn_b = gn_b; p.eps = eps;
    RWKV7_REQUIRE(kk && g && r_k && gn_w && gn_b, RWKV7_ERR_INVALID, "wkv7_output_prepare_f16state: null tensor pointer");
    if (int e = check_step_common(p, B, H, N)) return e;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    RWKV7_DISPATCH_DTYPE(dtype, T, {
        if (w_is_f32) return launch_step<T, float, kPrepare, __half>(p, B, st);
        return launch_step<T, T, kPrepare, __half>(p, B, st);
    });
    return RWKV7_OK;
}

extern "C" int rwkv7_wkv7_output_prepare_raw_f16state(const void* r, const void* w_raw, const void* k_raw, const void* v,
                                                      const void* a, const void* state_in, void* state_out, const void* g,
                                                      const void* k_k, const void* k_a, const void* r_k, const void* gn_w,
                                                      const void* gn_b, void* out, const void* w_bias, const void* a_bias,
                                                      int a_is_raw, const void* v_first, const void* v_gate,
                                                      const void* v_gate_bias, int v_gate_is_raw, void* v_out,
                                                      int* elapsed, int advance_elapsed, int state_prefetch, int B, int H,
                                                      int N, float eps, int dtype, void* stream) {
    StepArgs p{};
    p.r = r; p.w = w_raw; p.k = k_raw; p.v = v; p.a = a;
    p.state_in = state_in; p.state_out = state_out; p.out = out; p.H = H;
    p.g = g; p.r_k = r_k; p.gn_w = gn_w; p.gn_b = gn_b; p.eps = eps;
    p.k_k = k_k; p.k_a = k_a;
    p.w_bias = w_bias; p.a_bias = a_bias; p.a_is_raw = a_is_raw;
    p.v_first = v_first; p.v_gate = v_gate; p.v_gate_bias = v_gate_bias; p.v_gate_is_raw = v_gate_is_raw;
    p.v_out = v_out;
    p.prefetch_state = state_prefetch != 0;
    p.elapsed = elapsed;
    RWKV7_REQUIRE(g && r_k && gn_w && gn_b && k_k && k_a, RWKV7_ERR_INVALID,
                  "wkv7_output_prepare_raw_f16state: null tensor pointer");
    RWKV7_REQUIRE((v_first == nullptr) == (v_gate == nullptr), RWKV7_ERR_INVALID,
                  "wkv7_output_prepare_raw_f16state: v_first and v_gate must be given together");
    RWKV7_REQUIRE(!advance_elapsed || elapsed, RWKV7_ERR_INVALID, "wkv7_output_prepare_raw_f16state: advance_elapsed needs elapsed");
    if (int e = check_step_common(p, B, H, N)) return e;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    RWKV7_DISPATCH_DTYPE(dtype, T, {
        if (int e = launch_step<T, T, kRaw, __half>(p, B, st)) return e;
        if (advance_elapsed) {  // after the step, in stream order: no CTA of the step can see the new count
            advance_elapsed_kernel<<<(B + 127) / 128, 128, 0, st>>>(elapsed, B);
            return check_launch("advance_elapsed_kernel");
        }
        return RWKV7_OK;
    });
    return RWKV7_OK;
}
