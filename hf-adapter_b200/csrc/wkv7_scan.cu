// WKV-7 sequential scan over T tokens: one CTA per (sequence, head), the 64x64
// fp32 state lives in registers for the whole sequence (two threads per state
// row, 32 columns each), token vectors are staged through shared memory in
// blocks of kTS tokens with cp.async double buffering and converted to fp32 once
// per block.  HBM traffic is the algorithmic minimum (each token vector read
// once, y written once, state read/written once); the kernel is bound by the
// CUDA-core FMA rate (4*64*64 FMAs per token-head), which is what the chunked
// tensor-core form in wkv7_chunk.cu removes.
#include "common.cuh"

namespace rwkv7 {

constexpr int kSN = 64;
constexpr int kScanThreads = 128;
constexpr int kTS = 16;  // tokens per shared-memory stage

struct ScanArgs {
    const void *r, *w, *k, *v, *kk, *a;
    const void* state_in;  // fp32, or fp16 when state_f16
    void* state_out;
    void* y;
    const void *g, *r_k, *gn_w, *gn_b;
    float eps;
    int T, H;
    int w_mode;  // 0: decay in T, 1: decay fp32, 2: raw w in T
    // the reference's FP16-state sequence lane (rwkv7_hf/native_wkv_fp16.py:335-452)
    int state_f16;       // the state is stored in fp16 (loaded to fp32 registers, rounded back once at the end)
    int ab_mode;         // `kk` holds -kk and `a` holds kk*a (the lane's neg_kk / kka operands)
    const void* w0;      // w_mode 2: per-channel bias [H*64] added to raw w before the decay (may be NULL)
    const int* elapsed;  // w_mode 2: per-sequence step counters [B]; token t uses the dither phase elapsed + channel + t
};

// zero-mean pseudo-random offset of the reference's FP16-state kernels (rwkv7_hf/native_wkv_fp16.py:118-121)
__device__ __forceinline__ float scan_rotator1(int x) {
    const uint32_t bits = 2654435769u * static_cast<uint32_t>(x);
    return 4.547473508864641e-13f * static_cast<float>(static_cast<int32_t>(bits));
}

__device__ __forceinline__ void cp_async16(void* smem, const void* gmem) {
    unsigned s = (unsigned)__cvta_generic_to_shared(smem);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;\n" ::"r"(s), "l"(gmem));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

// Raw staging buffer for one block of tokens: six vectors (r,k,v,kk,a in T; w in T or fp32).
template <typename T>
struct RawStage {
    T r[kTS][kSN], k[kTS][kSN], v[kTS][kSN], kk[kTS][kSN], a[kTS][kSN];
    float w[kTS][kSN];  // sized for the fp32 case; the T case uses a prefix of it
};

template <typename T, bool PREP>
__global__ void __launch_bounds__(kScanThreads) wkv7_scan_kernel(const ScanArgs p) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    RawStage<T>* raw = reinterpret_cast<RawStage<T>*>(smem_raw);  // [2]
    float* f = reinterpret_cast<float*>(smem_raw + 2 * sizeof(RawStage<T>));
    // fp32 working set of the current stage
    float(*fr)[kSN] = reinterpret_cast<float(*)[kSN]>(f);
    float(*fw)[kSN] = fr + kTS;
    float(*fk)[kSN] = fw + kTS;
    float(*fkk)[kSN] = fk + kTS;
    float(*fkka)[kSN] = fkk + kTS;
    float(*fv)[kSN] = fkka + kTS;
    float(*fy)[kSN] = fv + kTS;

    const int bh = blockIdx.x;
    const int b = bh / p.H, h = bh % p.H;
    const int tid = threadIdx.x;
    const int row = tid >> 1, half = tid & 1, c0 = half * 32;
    const int T_ = p.T;
    const size_t tok_stride = (size_t)p.H * kSN;              // elements between consecutive tokens
    const size_t base = ((size_t)b * T_ * p.H + h) * kSN;     // element offset of token 0
    const int wbytes = (p.w_mode == 1) ? 4 : (int)sizeof(T);

    float S[32];
    const size_t soff = ((size_t)bh * kSN + row) * kSN + c0;
    if (p.state_f16) {
        const __half* sin = reinterpret_cast<const __half*>(p.state_in) + soff;
#pragma unroll
        for (int c = 0; c < 32; c += 8) {
            const uint4 t = *reinterpret_cast<const uint4*>(sin + c);
            const __half2* h2 = reinterpret_cast<const __half2*>(&t);
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const float2 f2 = __half22float2(h2[e]);
                S[c + 2 * e] = f2.x; S[c + 2 * e + 1] = f2.y;
            }
        }
    } else {
        const float* sin = reinterpret_cast<const float*>(p.state_in) + soff;
#pragma unroll
        for (int c = 0; c < 32; c += 4) {
            float4 t = *reinterpret_cast<const float4*>(sin + c);
            S[c] = t.x; S[c + 1] = t.y; S[c + 2] = t.z; S[c + 3] = t.w;
        }
    }
    const int phase0 = p.elapsed ? p.elapsed[b] + h * kSN : 0;

    // 16-byte chunks per token vector
    constexpr int CH_T = kSN * sizeof(T) / 16;
    auto issue_stage = [&](int stage, int t0) {
        RawStage<T>& rs = raw[stage & 1];
        const int nt = min(kTS, T_ - t0);
        const int ch_w = kSN * wbytes / 16;
        const int per_tok = 5 * CH_T + ch_w;
        for (int idx = tid; idx < nt * per_tok; idx += kScanThreads) {
            const int tt = idx / per_tok, q = idx % per_tok;
            const size_t goff = base + (size_t)(t0 + tt) * tok_stride;
            if (q < 5 * CH_T) {
                const int which = q / CH_T, ch = q % CH_T;
                const T* src;
                T* dst;
                switch (which) {
                    case 0: src = reinterpret_cast<const T*>(p.r); dst = rs.r[tt]; break;
                    case 1: src = reinterpret_cast<const T*>(p.k); dst = rs.k[tt]; break;
                    case 2: src = reinterpret_cast<const T*>(p.v); dst = rs.v[tt]; break;
                    case 3: src = reinterpret_cast<const T*>(p.kk); dst = rs.kk[tt]; break;
                    default: src = reinterpret_cast<const T*>(p.a); dst = rs.a[tt]; break;
                }
                cp_async16(reinterpret_cast<char*>(dst) + ch * 16, reinterpret_cast<const char*>(src + goff) + ch * 16);
            } else {
                const int ch = q - 5 * CH_T;
                cp_async16(reinterpret_cast<char*>(rs.w[tt]) + ch * 16,
                           reinterpret_cast<const char*>(p.w) + goff * wbytes + ch * 16);
            }
        }
        cp_async_commit();
    };

    const int nstages = (T_ + kTS - 1) / kTS;
    issue_stage(0, 0);
    for (int s = 0; s < nstages; ++s) {
        const int t0 = s * kTS;
        const int nt = min(kTS, T_ - t0);
        if (s + 1 < nstages) {
            issue_stage(s + 1, t0 + kTS);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();  // raw stage s visible; previous stage's fy flush finished
        {
            RawStage<T>& rs = raw[s & 1];
            for (int idx = tid; idx < nt * kSN; idx += kScanThreads) {
                const int tt = idx / kSN, c = idx % kSN;
                const float kkv = to_f<T>(rs.kk[tt][c]);
                fr[tt][c] = to_f<T>(rs.r[tt][c]);
                fk[tt][c] = to_f<T>(rs.k[tt][c]);
                fv[tt][c] = to_f<T>(rs.v[tt][c]);
                fkk[tt][c] = p.ab_mode ? -kkv : kkv;
                fkka[tt][c] = p.ab_mode ? to_f<T>(rs.a[tt][c]) : kkv * to_f<T>(rs.a[tt][c]);
                float wv;
                if (p.w_mode == 1) wv = rs.w[tt][c];
                else {
                    wv = to_f<T>(reinterpret_cast<const T*>(rs.w[tt])[c]);
                    if (p.w_mode == 2) {
                        if (p.w0) wv += to_f<T>(reinterpret_cast<const T*>(p.w0)[h * kSN + c]);
                        wv = decay_from_raw(wv);
                        // (decay - 1 + rotator) rounded to fp16, as the reference's kernel forms its decay operand
                        if (p.elapsed) wv = 1.0f + __half2float(__float2half_rn(wv - 1.0f + scan_rotator1(phase0 + c + t0 + tt)));
                    }
                }
                fw[tt][c] = wv;
            }
        }
        __syncthreads();
        for (int tt = 0; tt < nt; ++tt) {
            float sa0 = 0.f, sa1 = 0.f;
#pragma unroll
            for (int c = 0; c < 32; c += 4) {
                const float4 q = *reinterpret_cast<const float4*>(&fkk[tt][c0 + c]);
                sa0 = fmaf(S[c], q.x, sa0); sa1 = fmaf(S[c + 1], q.y, sa1);
                sa0 = fmaf(S[c + 2], q.z, sa0); sa1 = fmaf(S[c + 3], q.w, sa1);
            }
            float sa = sa0 + sa1;
            sa += __shfl_xor_sync(0xffffffffu, sa, 1);
            const float vi = fv[tt][row];
            float y0 = 0.f, y1 = 0.f;
#pragma unroll
            for (int c = 0; c < 32; c += 4) {
                const float4 wq = *reinterpret_cast<const float4*>(&fw[tt][c0 + c]);
                const float4 kq = *reinterpret_cast<const float4*>(&fk[tt][c0 + c]);
                const float4 bq = *reinterpret_cast<const float4*>(&fkka[tt][c0 + c]);
                const float4 rq = *reinterpret_cast<const float4*>(&fr[tt][c0 + c]);
                S[c] = fmaf(-sa, bq.x, fmaf(vi, kq.x, S[c] * wq.x));
                S[c + 1] = fmaf(-sa, bq.y, fmaf(vi, kq.y, S[c + 1] * wq.y));
                S[c + 2] = fmaf(-sa, bq.z, fmaf(vi, kq.z, S[c + 2] * wq.z));
                S[c + 3] = fmaf(-sa, bq.w, fmaf(vi, kq.w, S[c + 3] * wq.w));
                y0 = fmaf(S[c], rq.x, y0); y1 = fmaf(S[c + 1], rq.y, y1);
                y0 = fmaf(S[c + 2], rq.z, y0); y1 = fmaf(S[c + 3], rq.w, y1);
            }
            float y = y0 + y1;
            y += __shfl_xor_sync(0xffffffffu, y, 1);
            if (half == 0) fy[tt][row] = y;
        }
        __syncthreads();
        // flush y of this stage (optionally with GroupNorm / bonus / gate)
        T* yout = reinterpret_cast<T*>(p.y);
        if constexpr (!PREP) {
            for (int idx = tid; idx < nt * kSN; idx += kScanThreads) {
                const int tt = idx / kSN, c = idx % kSN;
                yout[base + (size_t)(t0 + tt) * tok_stride + c] = from_f<T>(fy[tt][c]);
            }
        } else {
            const int warp = tid >> 5, lane = tid & 31;
            for (int tt = warp; tt < nt; tt += kScanThreads / 32) {
                const float y0 = fy[tt][lane], y1 = fy[tt][lane + 32];
                const float mean = group_sum<32>(y0 + y1) * (1.0f / kSN);
                const float d0 = y0 - mean, d1 = y1 - mean;
                const float rstd = rsqrtf(group_sum<32>(d0 * d0 + d1 * d1) * (1.0f / kSN) + p.eps);
                const T* rk = reinterpret_cast<const T*>(p.r_k) + h * kSN;
                float corr = fr[tt][lane] * fk[tt][lane] * to_f<T>(rk[lane]) +
                             fr[tt][lane + 32] * fk[tt][lane + 32] * to_f<T>(rk[lane + 32]);
                corr = group_sum<32>(corr);
                const size_t o = base + (size_t)(t0 + tt) * tok_stride;
                const T* gw = reinterpret_cast<const T*>(p.gn_w) + h * kSN;
                const T* gb = reinterpret_cast<const T*>(p.gn_b) + h * kSN;
                const T* gg = reinterpret_cast<const T*>(p.g) + o;
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                    const int c = lane + 32 * u;
                    const float d = u ? d1 : d0;
                    const float val = (d * rstd * to_f<T>(gw[c]) + to_f<T>(gb[c]) + corr * fv[tt][c]) * to_f<T>(gg[c]);
                    yout[o + c] = from_f<T>(val);
                }
            }
        }
        // the next iteration's first __syncthreads orders this flush before fy/f* are overwritten
    }

    if (p.state_f16) {
        __half* sout = reinterpret_cast<__half*>(p.state_out) + soff;
#pragma unroll
        for (int c = 0; c < 32; c += 8) {
            uint4 t;
            __half2* h2 = reinterpret_cast<__half2*>(&t);
#pragma unroll
            for (int e = 0; e < 4; ++e) h2[e] = __floats2half2_rn(S[c + 2 * e], S[c + 2 * e + 1]);
            *reinterpret_cast<uint4*>(sout + c) = t;
        }
    } else {
        float* sout = reinterpret_cast<float*>(p.state_out) + soff;
#pragma unroll
        for (int c = 0; c < 32; c += 4)
            *reinterpret_cast<float4*>(sout + c) = make_float4(S[c], S[c + 1], S[c + 2], S[c + 3]);
    }
}

template <typename T>
static size_t scan_smem_bytes() { return 2 * sizeof(RawStage<T>) + 7 * kTS * kSN * sizeof(float); }

}  // namespace rwkv7

using namespace rwkv7;

static int scan_impl(const void* r, const void* w, const void* k, const void* v, const void* kk, const void* a,
                     const void* state_in, void* state_out, void* y, const void* g, const void* r_k, const void* gn_w,
                     const void* gn_b, float eps, int B, int T, int H, int N, int dtype, int w_mode, int state_f16,
                     int ab_mode, const void* w0, const int* elapsed, void* stream) {
    RWKV7_REQUIRE(N == kSN, RWKV7_ERR_UNSUPPORTED, "wkv7_scan: head size must be 64, got %d", N);
    RWKV7_REQUIRE(B > 0 && H > 0 && T >= 0, RWKV7_ERR_INVALID, "wkv7_scan: bad sizes B=%d T=%d H=%d", B, T, H);
    RWKV7_REQUIRE(w_mode >= 0 && w_mode <= 2, RWKV7_ERR_INVALID, "wkv7_scan: w_mode must be 0, 1 or 2");
    RWKV7_REQUIRE(state_in && state_out, RWKV7_ERR_INVALID, "wkv7_scan: null state pointer");
    const bool prep = g || r_k || gn_w || gn_b;
    if (prep) RWKV7_REQUIRE(g && r_k && gn_w && gn_b, RWKV7_ERR_INVALID, "wkv7_scan: g, r_k, gn_w, gn_b go together");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (T == 0) {  // empty sequence: the state passes through
        if (state_out != state_in) {
            cudaError_t e = cudaMemcpyAsync(state_out, state_in, (size_t)B * H * N * N * (state_f16 ? 2 : 4),
                                            cudaMemcpyDeviceToDevice, st);
            RWKV7_REQUIRE(e == cudaSuccess, RWKV7_ERR_CUDA, "wkv7_scan: %s", cudaGetErrorString(e));
        }
        return RWKV7_OK;
    }
    RWKV7_REQUIRE(r && w && k && v && kk && a && y, RWKV7_ERR_INVALID, "wkv7_scan: null tensor pointer");
    const void* ptrs[] = {r, w, k, v, kk, a, state_in, state_out, y, g};
    for (const void* q : ptrs) RWKV7_REQUIRE(aligned(q, 16), RWKV7_ERR_ALIGN, "wkv7_scan: pointers must be 16-byte aligned");
    RWKV7_REQUIRE((!w0 && !elapsed) || w_mode == 2, RWKV7_ERR_INVALID, "wkv7_scan: w0 / elapsed apply to raw w (w_mode 2)");
    ScanArgs p{r, w, k, v, kk, a, state_in, state_out, y, g, r_k, gn_w, gn_b, eps, T, H, w_mode, state_f16 != 0, ab_mode != 0, w0, elapsed};
    RWKV7_DISPATCH_DTYPE(dtype, TT, {
        const size_t smem = scan_smem_bytes<TT>();
        auto kern = prep ? wkv7_scan_kernel<TT, true> : wkv7_scan_kernel<TT, false>;
        cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        RWKV7_REQUIRE(e == cudaSuccess, RWKV7_ERR_CUDA, "wkv7_scan: %s", cudaGetErrorString(e));
        kern<<<B * H, kScanThreads, smem, st>>>(p);
        return check_launch("wkv7_scan_kernel");
    });
    return RWKV7_OK;
}

extern "C" int rwkv7_wkv7_scan(const void* r, const void* w, const void* k, const void* v, const void* kk,
                               const void* a, const float* state_in, float* state_out, void* y, const void* g,
                               const void* r_k, const void* gn_w, const void* gn_b, float eps, int B, int T, int H,
                               int N, int dtype, int w_mode, void* stream) {
    return scan_impl(r, w, k, v, kk, a, state_in, state_out, y, g, r_k, gn_w, gn_b, eps, B, T, H, N, dtype, w_mode, 0, 0,
                     nullptr, nullptr, stream);
}

extern "C" int rwkv7_wkv7_scan_f16state(const void* r, const void* w, const void* k, const void* v, const void* kk,
                                        const void* a, const void* state_in, void* state_out, void* y, const void* g,
                                        const void* r_k, const void* gn_w, const void* gn_b, float eps, int B, int T,
                                        int H, int N, int dtype, int w_mode, int ab_mode, const void* w0,
                                        const int* elapsed, void* stream) {
    return scan_impl(r, w, k, v, kk, a, state_in, state_out, y, g, r_k, gn_w, gn_b, eps, B, T, H, N, dtype, w_mode, 1,
                     ab_mode, w0, elapsed, stream);
}
