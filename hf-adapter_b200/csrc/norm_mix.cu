// LayerNorm + token-shift mixing kernels (memory-bound, one CTA per row).
// Each row is read once into registers (128-bit loads), normalised in fp32 with a
// centred two-pass variance, and every consumer of the normalised row (the six
// time-mix streams, the shift state) is written from registers in the same pass.
#include <atomic>

#include "common.cuh"

namespace rwkv7 {

constexpr int kNMThreads = 256;
constexpr int kNMMaxVec = 4;  // 8-element vectors per thread -> D <= 8192

// Eight elements in storage type, fetched with one 16- or 32-byte load and converted where they are used: the
// per-channel constants of a row kernel (norm weight / bias, mix vectors) are fetched BEFORE the grid-dependency wait
// and before the row statistics, so their latency hides under the preceding kernel's tail and the reductions.
template <typename T>
struct alignas(sizeof(T) * 8) Raw8 {
    T v[8];
};
template <typename T>
__device__ __forceinline__ Raw8<T> ld_raw8(const T* p) { return *reinterpret_cast<const Raw8<T>*>(p); }
template <typename T>
__device__ __forceinline__ void cvt8(const Raw8<T>& r, float (&o)[8]) {
#pragma unroll
    for (int e = 0; e < 8; ++e) o[e] = to_f<T>(r.v[e]);
}

template <typename T>
struct RowStats {
    float x[kNMMaxVec][8];
    float mean, rstd;
};

// loads row (optionally + add row) into registers, returns mean / rstd
template <typename T, bool ADD>
__device__ __forceinline__ void load_row_stats(const T* x, const T* add, T* sum_out, int D, float eps, RowStats<T>& rs,
                                               float* red) {
    const int nvec = D / 8;
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < kNMMaxVec; ++i) {
        const int vi = threadIdx.x + i * kNMThreads;
        if (vi < nvec) {
            load8(x + vi * 8, rs.x[i]);
            if constexpr (ADD) {
                float t[8];
                load8(add + vi * 8, t);
#pragma unroll
                for (int e = 0; e < 8; ++e) rs.x[i][e] += t[e];
                if (sum_out) store8(sum_out + vi * 8, rs.x[i]);  // the norm below sees the unrounded fp32 sum
            }
#pragma unroll
            for (int e = 0; e < 8; ++e) s += rs.x[i][e];
        }
    }
    rs.mean = block_sum(s, red) / (float)D;
    float q = 0.f;
#pragma unroll
    for (int i = 0; i < kNMMaxVec; ++i) {
        const int vi = threadIdx.x + i * kNMThreads;
        if (vi < nvec) {
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const float d = rs.x[i][e] - rs.mean;
                q += d * d;
            }
        }
    }
    rs.rstd = rsqrtf(block_sum(q, red) / (float)D + eps);
}

struct Mix6Args {
    const void *x, *nw, *nb;
    void* prev;
    const void* mix[6];
    void* out[6];
    int D;
    float eps;
    const int* slots;  // state pool: the shift state of batch row b is row slots[b] of `prev`; NULL = row b
};

template <typename T>
__global__ void __launch_bounds__(kNMThreads) attn_norm_mix6_kernel(const Mix6Args p) {
    __shared__ float red[32];
    const size_t row = blockIdx.x;
    const int D = p.D;
    const int nvec = D / 8;
    Raw8<T> cw[kNMMaxVec], cb[kNMMaxVec], cm[6][kNMMaxVec];
#pragma unroll
    for (int i = 0; i < kNMMaxVec; ++i) {
        const int vi = threadIdx.x + i * kNMThreads;
        if (vi < nvec) {
            cw[i] = ld_raw8(reinterpret_cast<const T*>(p.nw) + vi * 8);
            cb[i] = ld_raw8(reinterpret_cast<const T*>(p.nb) + vi * 8);
#pragma unroll
            for (int m = 0; m < 6; ++m) cm[m][i] = ld_raw8(reinterpret_cast<const T*>(p.mix[m]) + vi * 8);
        }
    }
    // Resident under the tail of the preceding kernel; the wait orders every access below after it, and only then may
    // the projections that follow start (they stream their weights meanwhile).
    grid_dependency_wait();
    if (threadIdx.x == 0) grid_launch_dependents();
    RowStats<T> rs;
    load_row_stats<T, false>(reinterpret_cast<const T*>(p.x) + row * D, nullptr, nullptr, D, p.eps, rs, red);
    T* prev = reinterpret_cast<T*>(p.prev) + (p.slots ? (size_t)__ldg(p.slots + row) : row) * D;
#pragma unroll
    for (int i = 0; i < kNMMaxVec; ++i) {
        const int vi = threadIdx.x + i * kNMThreads;
        if (vi < nvec) {
            float w[8], b[8], pv[8], h[8], d[8];
            cvt8(cw[i], w);
            cvt8(cb[i], b);
            load8(prev + vi * 8, pv);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                h[e] = (rs.x[i][e] - rs.mean) * rs.rstd * w[e] + b[e];
                d[e] = pv[e] - h[e];
            }
            store8(prev + vi * 8, h);
#pragma unroll
            for (int m = 0; m < 6; ++m) {
                float mx[8], o[8];
                cvt8(cm[m][i], mx);
#pragma unroll
                for (int e = 0; e < 8; ++e) o[e] = h[e] + d[e] * mx[e];
                store8(reinterpret_cast<T*>(p.out[m]) + row * D + vi * 8, o);
            }
        }
    }
}

struct FfnMixArgs {
    const void *res, *attn, *nw, *nb, *mix;
    void *prev, *res_out, *mixed;
    int D;
    float eps;
    const int* slots;  // as in Mix6Args
};

// ADD: x = res + attn (stored to res_out; normalised from the fp32 sum like the reference's fused kernel)
// MIX: emit mixed + update prev; otherwise plain LayerNorm into `mixed`.
template <typename T, bool ADD, bool MIX>
__global__ void __launch_bounds__(kNMThreads) ffn_add_norm_mix_kernel(const FfnMixArgs p) {
    __shared__ float red[32];
    const size_t row = blockIdx.x;
    const int D = p.D;
    const int nvec = D / 8;
    Raw8<T> cw[kNMMaxVec], cb[kNMMaxVec], cm[kNMMaxVec];
#pragma unroll
    for (int i = 0; i < kNMMaxVec; ++i) {
        const int vi = threadIdx.x + i * kNMThreads;
        if (vi < nvec) {
            cw[i] = ld_raw8(reinterpret_cast<const T*>(p.nw) + vi * 8);
            cb[i] = ld_raw8(reinterpret_cast<const T*>(p.nb) + vi * 8);
            if constexpr (MIX) cm[i] = ld_raw8(reinterpret_cast<const T*>(p.mix) + vi * 8);
        }
    }
    grid_dependency_wait();
    if (threadIdx.x == 0) grid_launch_dependents();
    RowStats<T> rs;
    load_row_stats<T, ADD>(reinterpret_cast<const T*>(p.res) + row * D,
                           ADD ? reinterpret_cast<const T*>(p.attn) + row * D : nullptr,
                           ADD ? reinterpret_cast<T*>(p.res_out) + row * D : nullptr, D, p.eps, rs, red);
#pragma unroll
    for (int i = 0; i < kNMMaxVec; ++i) {
        const int vi = threadIdx.x + i * kNMThreads;
        if (vi < nvec) {
            float w[8], b[8], h[8];
            cvt8(cw[i], w);
            cvt8(cb[i], b);
#pragma unroll
            for (int e = 0; e < 8; ++e) h[e] = (rs.x[i][e] - rs.mean) * rs.rstd * w[e] + b[e];
            if constexpr (MIX) {
                float pv[8], mx[8], o[8];
                T* prev = reinterpret_cast<T*>(p.prev) + (p.slots ? (size_t)__ldg(p.slots + row) : row) * D;
                load8(prev + vi * 8, pv);
                cvt8(cm[i], mx);
#pragma unroll
                for (int e = 0; e < 8; ++e) o[e] = h[e] + (pv[e] - h[e]) * mx[e];
                store8(prev + vi * 8, h);
                store8(reinterpret_cast<T*>(p.mixed) + row * D + vi * 8, o);
            } else {
                store8(reinterpret_cast<T*>(p.mixed) + row * D + vi * 8, h);
            }
        }
    }
}

struct SeqMixArgs {
    const void *x, *init_prev;
    const void* mix[6];
    void* out[6];
    void* next_state;
    int T, D, n_mix;
    long long total_vec;
    bool strict;  // fp16: round the difference and the product separately (the reference's strict_fp16_rounding)
};

template <typename T>
__global__ void __launch_bounds__(256) seq_shift_mix_kernel(const SeqMixArgs p) {
    const int D = p.D, vecD = D / 8;
    for (long long v = (long long)blockIdx.x * blockDim.x + threadIdx.x; v < p.total_vec;
         v += (long long)gridDim.x * blockDim.x) {
        const long long rowi = v / vecD;  // b*T + t
        const int c = (int)(v % vecD) * 8;
        const int t = (int)(rowi % p.T);
        const long long b = rowi / p.T;
        float x[8], pv[8];
        const T* xp = reinterpret_cast<const T*>(p.x) + rowi * D + c;
        load8(xp, x);
        if (t == 0) load8(reinterpret_cast<const T*>(p.init_prev) + b * D + c, pv);
        else load8(xp - D, pv);
#pragma unroll
        for (int e = 0; e < 8; ++e) pv[e] -= x[e];
        for (int m = 0; m < p.n_mix; ++m) {
            float mx[8], o[8];
            load8(reinterpret_cast<const T*>(p.mix[m]) + c, mx);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                // strict: the difference and the product are each rounded to the storage type (fp32 arithmetic on
                // 11-bit significands followed by one rounding equals the fp16 instruction: 24 >= 2*11 + 2)
                if (p.strict) o[e] = __fadd_rn(x[e], round_to<T>(__fmul_rn(round_to<T>(pv[e]), mx[e])));
                else o[e] = x[e] + pv[e] * mx[e];
            }
            store8(reinterpret_cast<T*>(p.out[m]) + rowi * D + c, o);
        }
        if (t == p.T - 1 && p.next_state) store8(reinterpret_cast<T*>(p.next_state) + b * D + c, x);
    }
}

static int check_row_shape(const char* what, int rows, int D) {
    RWKV7_REQUIRE(rows > 0 && D > 0, RWKV7_ERR_INVALID, "%s: rows and D must be positive", what);
    RWKV7_REQUIRE(D % 8 == 0 && D <= 8 * kNMThreads * kNMMaxVec, RWKV7_ERR_UNSUPPORTED,
                  "%s: D must be a multiple of 8 and <= %d (got %d)", what, 8 * kNMThreads * kNMMaxVec, D);
    return RWKV7_OK;
}

}  // namespace rwkv7

using namespace rwkv7;

static int attn_norm_mix6_impl(const void* x, void* prev, const int32_t* slots, const void* norm_w, const void* norm_b,
                               const void* const mixes[6], void* const outs[6], int rows, int D, float eps, int dtype,
                               void* stream) {
    if (int e = check_row_shape("attn_norm_mix6", rows, D)) return e;
    RWKV7_REQUIRE(x && prev && norm_w && norm_b && mixes && outs, RWKV7_ERR_INVALID, "attn_norm_mix6: null pointer");
    RWKV7_REQUIRE(x != prev, RWKV7_ERR_INVALID, "attn_norm_mix6: x and prev must not alias");
    Mix6Args p{x, norm_w, norm_b, prev, {}, {}, D, eps, slots};
    for (int m = 0; m < 6; ++m) {
        RWKV7_REQUIRE(mixes[m] && outs[m], RWKV7_ERR_INVALID, "attn_norm_mix6: null mix/out pointer %d", m);
        RWKV7_REQUIRE(aligned(mixes[m], 16) && aligned(outs[m], 16), RWKV7_ERR_ALIGN, "attn_norm_mix6: unaligned pointer");
        p.mix[m] = mixes[m];
        p.out[m] = outs[m];
    }
    RWKV7_REQUIRE(aligned(x, 16) && aligned(prev, 16) && aligned(norm_w, 16) && aligned(norm_b, 16), RWKV7_ERR_ALIGN,
                  "attn_norm_mix6: unaligned pointer");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    RWKV7_DISPATCH_DTYPE(dtype, T, {
        launch_programmatic(attn_norm_mix6_kernel<T>, dim3(rows), dim3(kNMThreads), 0, st, p);
        return check_launch("attn_norm_mix6_kernel");
    });
    return RWKV7_OK;
}

extern "C" int rwkv7_attn_norm_mix6(const void* x, void* prev, const void* norm_w, const void* norm_b,
                                    const void* const mixes[6], void* const outs[6], int rows, int D, float eps,
                                    int dtype, void* stream) {
    return attn_norm_mix6_impl(x, prev, nullptr, norm_w, norm_b, mixes, outs, rows, D, eps, dtype, stream);
}

extern "C" int rwkv7_attn_norm_mix6_pool(const void* x, void* prev_pool, const int32_t* slot_ids, const void* norm_w,
                                         const void* norm_b, const void* const mixes[6], void* const outs[6], int rows,
                                         int D, float eps, int dtype, void* stream) {
    RWKV7_REQUIRE(slot_ids != nullptr, RWKV7_ERR_INVALID, "attn_norm_mix6_pool: null slot_ids");
    return attn_norm_mix6_impl(x, prev_pool, slot_ids, norm_w, norm_b, mixes, outs, rows, D, eps, dtype, stream);
}

static int ffn_add_norm_mix_impl(const void* residual, const void* attn_out, void* prev, const int32_t* slots,
                                 const void* norm_w, const void* norm_b, const void* mix, void* residual_out, void* mixed,
                                 int rows, int D, float eps, int dtype, void* stream) {
    if (int e = check_row_shape("ffn_add_norm_mix", rows, D)) return e;
    RWKV7_REQUIRE(residual && prev && norm_w && norm_b && mix && mixed, RWKV7_ERR_INVALID, "ffn_add_norm_mix: null pointer");
    RWKV7_REQUIRE(attn_out == nullptr || residual_out != nullptr, RWKV7_ERR_INVALID,
                  "ffn_add_norm_mix: residual_out is required when attn_out is given");
    const void* ptrs[] = {residual, attn_out, prev, norm_w, norm_b, mix, residual_out, mixed};
    for (const void* q : ptrs) RWKV7_REQUIRE(aligned(q, 16), RWKV7_ERR_ALIGN, "ffn_add_norm_mix: unaligned pointer");
    FfnMixArgs p{residual, attn_out, norm_w, norm_b, mix, prev, residual_out, mixed, D, eps, slots};
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    RWKV7_DISPATCH_DTYPE(dtype, T, {
        if (attn_out) launch_programmatic(ffn_add_norm_mix_kernel<T, true, true>, dim3(rows), dim3(kNMThreads), 0, st, p);
        else launch_programmatic(ffn_add_norm_mix_kernel<T, false, true>, dim3(rows), dim3(kNMThreads), 0, st, p);
        return check_launch("ffn_add_norm_mix_kernel");
    });
    return RWKV7_OK;
}

extern "C" int rwkv7_ffn_add_norm_mix(const void* residual, const void* attn_out, void* prev, const void* norm_w,
                                      const void* norm_b, const void* mix, void* residual_out, void* mixed, int rows,
                                      int D, float eps, int dtype, void* stream) {
    return ffn_add_norm_mix_impl(residual, attn_out, prev, nullptr, norm_w, norm_b, mix, residual_out, mixed, rows, D, eps,
                                 dtype, stream);
}

extern "C" int rwkv7_ffn_add_norm_mix_pool(const void* residual, const void* attn_out, void* prev_pool,
                                           const int32_t* slot_ids, const void* norm_w, const void* norm_b,
                                           const void* mix, void* residual_out, void* mixed, int rows, int D, float eps,
                                           int dtype, void* stream) {
    RWKV7_REQUIRE(slot_ids != nullptr, RWKV7_ERR_INVALID, "ffn_add_norm_mix_pool: null slot_ids");
    return ffn_add_norm_mix_impl(residual, attn_out, prev_pool, slot_ids, norm_w, norm_b, mix, residual_out, mixed, rows, D,
                                 eps, dtype, stream);
}

extern "C" int rwkv7_layer_norm(const void* x, const void* norm_w, const void* norm_b, void* out, int rows, int D,
                                float eps, int dtype, void* stream) {
    if (int e = check_row_shape("layer_norm", rows, D)) return e;
    RWKV7_REQUIRE(x && norm_w && norm_b && out, RWKV7_ERR_INVALID, "layer_norm: null pointer");
    const void* ptrs[] = {x, norm_w, norm_b, out};
    for (const void* q : ptrs) RWKV7_REQUIRE(aligned(q, 16), RWKV7_ERR_ALIGN, "layer_norm: unaligned pointer");
    FfnMixArgs p{x, nullptr, norm_w, norm_b, nullptr, nullptr, nullptr, out, D, eps, nullptr};
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    RWKV7_DISPATCH_DTYPE(dtype, T, {
        launch_programmatic(ffn_add_norm_mix_kernel<T, false, false>, dim3(rows), dim3(kNMThreads), 0, st, p);
        return check_launch("layer_norm_kernel");
    });
    return RWKV7_OK;
}

extern "C" int rwkv7_seq_shift_mix(const void* x, const void* initial_prev, const void* const* mixes,
                                   void* const* outs, void* next_state, int B, int T, int D, int n_mix, int strict_rounding,
                                   int dtype, void* stream) {
    RWKV7_REQUIRE(B > 0 && T > 0 && D > 0, RWKV7_ERR_INVALID, "seq_shift_mix: sizes must be positive");
    RWKV7_REQUIRE(D % 8 == 0, RWKV7_ERR_UNSUPPORTED, "seq_shift_mix: D must be a multiple of 8");
    RWKV7_REQUIRE(n_mix >= 1 && n_mix <= 6, RWKV7_ERR_INVALID, "seq_shift_mix: n_mix must be in 1..6");
    RWKV7_REQUIRE(x && initial_prev && mixes && outs, RWKV7_ERR_INVALID, "seq_shift_mix: null pointer");
    RWKV7_REQUIRE(!strict_rounding || dtype == RWKV7_F16, RWKV7_ERR_UNSUPPORTED, "seq_shift_mix: strict rounding is defined for fp16 only");
    SeqMixArgs p{x, initial_prev, {}, {}, next_state, T, D, n_mix, (long long)B * T * (D / 8), strict_rounding != 0};
    for (int m = 0; m < n_mix; ++m) {
        RWKV7_REQUIRE(mixes[m] && outs[m], RWKV7_ERR_INVALID, "seq_shift_mix: null mix/out pointer %d", m);
        RWKV7_REQUIRE(aligned(mixes[m], 16) && aligned(outs[m], 16), RWKV7_ERR_ALIGN, "seq_shift_mix: unaligned pointer");
        p.mix[m] = mixes[m];
        p.out[m] = outs[m];
    }
    RWKV7_REQUIRE(aligned(x, 16) && aligned(initial_prev, 16) && aligned(next_state, 16), RWKV7_ERR_ALIGN,
                  "seq_shift_mix: unaligned pointer");
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    const long long blocks = (p.total_vec + 255) / 256;
    const int grid = (int)(blocks < 148LL * 16 ? blocks : 148LL * 16);
    RWKV7_DISPATCH_DTYPE(dtype, TT, {
        seq_shift_mix_kernel<TT><<<grid, 256, 0, st>>>(p);
        return check_launch("seq_shift_mix_kernel");
    });
    return RWKV7_OK;
}

namespace rwkv7 {

unsigned int* kernel_error_word();  // capi.cu

// ---- tensor-parallel forms: the sum over ranks happens inside the row kernel -----------------------------------------
// Under head-sharded tensor parallelism the [rows, D] outputs of o_proj and ffn.value are partial sums, and the kernel
// that consumes each of them is one of the two row kernels above.  These forms take this rank's PARTIAL instead of the
// summed tensor.  The CTA of row r
//   1. stores its partial row into slot [rank] of every peer's inbox, every 4 bytes of payload paired with the 4-byte
//      call number in one 8-byte unit (plain 16-byte peer stores of two such units),
//   2. polls its own inbox until every unit of row r from every peer carries the call number (bounded),
//   3. adds the P rows in rank order in fp32 and rounds the sum to the storage type (bit for bit what the stand-alone
//      all-reduce kernel stores), and carries on with LayerNorm and the mixes from registers.
// An aligned 8-byte store arrives whole, so a unit that shows the call number holds this call's payload: no fence, no
// separate flag, and the exchange costs ONE trip over the link instead of three (data, acknowledgement, flag).  One
// launch and one pass over the row replace the all-reduce kernel, its [rows, D] round trip and a kernel boundary.
// Two inbox buffers alternate by call number (a rank that starts call e + 2 has finished call e + 1, whose wait
// proves that every peer had started e + 1, i.e. finished reading e); the call counter lives on the device; the sum
// runs in rank order on every rank; a wait that runs out raises error word 7 and the kernel stores nothing.  A CTA
// waits for the same row's CTA on every peer: the host admits only row counts whose CTAs are all resident at once, so
// no CTA waits for one that cannot start.
constexpr int kTpMaxRanks = 8;
constexpr unsigned kErrPeerWait = 7;

struct TpRowsArgs {
    const void* partial;            // this rank's [rows, D] partial sums
    uint4* inbox[kTpMaxRanks];      // per rank: [2][P][slot_elems / 2] units of {payload word, call number}, two per uint4
    uint32_t* counters;             // local: [0] completed calls, [1] CTAs of the current call that are through
    unsigned int* error;
    int rank, world, rows;
    long long slot_elems;           // payload values per inbox slot (a multiple of 8)
    unsigned long long wait_ns;
};

__device__ __forceinline__ void st_volatile_v4(uint4* p, uint32_t a, uint32_t b, uint32_t c, uint32_t d) {
    asm volatile("st.volatile.global.v4.u32 [%0], {%1, %2, %3, %4};" ::"l"(p), "r"(a), "r"(b), "r"(c), "r"(d) : "memory");
}
__device__ __forceinline__ uint4 ld_volatile_v4(const uint4* p) {
    uint4 v;
    asm volatile("ld.volatile.global.v4.u32 {%0, %1, %2, %3}, [%4];" : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w) : "l"(p) : "memory");
    return v;
}
template <typename T> __device__ __forceinline__ T word_lo(uint32_t w);
template <typename T> __device__ __forceinline__ T word_hi(uint32_t w);
template <> __device__ __forceinline__ __half word_lo<__half>(uint32_t w) { return __ushort_as_half((unsigned short)(w & 0xffffu)); }
template <> __device__ __forceinline__ __half word_hi<__half>(uint32_t w) { return __ushort_as_half((unsigned short)(w >> 16)); }
template <> __device__ __forceinline__ __nv_bfloat16 word_lo<__nv_bfloat16>(uint32_t w) { return __ushort_as_bfloat16((unsigned short)(w & 0xffffu)); }
template <> __device__ __forceinline__ __nv_bfloat16 word_hi<__nv_bfloat16>(uint32_t w) { return __ushort_as_bfloat16((unsigned short)(w >> 16)); }
__device__ __forceinline__ unsigned long long timer_ns() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}

// inbox[r] without indexing the kernel parameters dynamically (which would copy the argument block to local memory)
__device__ __forceinline__ uint4* tp_inbox(const TpRowsArgs& t, int r) {
    uint4* p = t.inbox[0];
#pragma unroll
    for (int k = 1; k < kTpMaxRanks; ++k)
        if (r == k) p = t.inbox[k];
    return p;
}

// The call number of this launch (every thread of the CTA gets it) - read before any row is pushed.
__device__ __forceinline__ uint32_t tp_rows_begin(const TpRowsArgs& t, uint32_t* s_epoch) {
    if (threadIdx.x == 0) *s_epoch = *reinterpret_cast<volatile uint32_t*>(t.counters) + 1u;
    __syncthreads();
    return *s_epoch;
}

template <typename T, int NV>
__device__ __forceinline__ void tp_load_own(const TpRowsArgs& t, size_t row, int D, uint4 (&own)[NV]) {
    const uint4* mine = reinterpret_cast<const uint4*>(reinterpret_cast<const T*>(t.partial) + row * D);
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int vi = threadIdx.x + i * kNMThreads;
        if (vi < D / 8) own[i] = mine[vi];
    }
}

// Step 1 for one row.
template <typename T, int NV>
__device__ __forceinline__ void tp_rows_push(const TpRowsArgs& t, uint32_t e, size_t row, int D) {
    static_assert(sizeof(T) == 2, "the inbox holds 2-byte values");
    const uint32_t tag = e ? e : 1u;  // never 0 (fresh memory); calls 0 and 1 use different buffers
    const long long slot_u4 = t.slot_elems / 4;  // uint4 per slot: 2 per 8 payload values
    uint4 own[NV];
    tp_load_own<T, NV>(t, row, D, own);
    for (int s = 1; s < t.world; ++s) {
        const int peer = (t.rank + s) % t.world;  // start with the next rank: the peers' links are loaded evenly
        uint4* dst = tp_inbox(t, peer) + ((long long)(e & 1u) * t.world + t.rank) * slot_u4 + (long long)row * (D / 4);
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int vi = threadIdx.x + i * kNMThreads;
            if (vi < D / 8) {
                st_volatile_v4(dst + 2 * vi, own[i].x, tag, own[i].y, tag);
                st_volatile_v4(dst + 2 * vi + 1, own[i].z, tag, own[i].w, tag);
            }
        }
    }
}

// Steps 2-3 for one row: x[i][e] receives the rounded sum.  Returns false when a wait ran out (the caller stores
// nothing more and still calls tp_rows_finish).
template <typename T, int NV>
__device__ __forceinline__ bool tp_rows_sum(const TpRowsArgs& t, uint32_t e, size_t row, int D, float (&x)[kNMMaxVec][8]) {
    const int tid = threadIdx.x, nvec = D / 8;
    const uint32_t tag = e ? e : 1u;
    const long long slot_u4 = t.slot_elems / 4;
    uint4 own[NV];
    tp_load_own<T, NV>(t, row, D, own);
    float acc[NV][8];
#pragma unroll
    for (int i = 0; i < NV; ++i)
#pragma unroll
        for (int q = 0; q < 8; ++q) acc[i][q] = 0.f;
    bool gave_up = false;
    const unsigned long long t0 = timer_ns();
    const uint4* box = tp_inbox(t, t.rank) + (long long)(e & 1u) * t.world * slot_u4 + (long long)row * (D / 4);
    for (int s = 0; s < t.world; ++s) {
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int vi = tid + i * kNMThreads;
            if (vi < nvec) {
                uint4 raw = own[i];
                if (s != t.rank) {
                    const uint4* src = box + (long long)s * slot_u4 + 2 * vi;
                    uint4 lo = ld_volatile_v4(src), hi = ld_volatile_v4(src + 1);
                    for (uint32_t spin = 1; !gave_up && (lo.y != tag || lo.w != tag || hi.y != tag || hi.w != tag); ++spin) {
                        if ((spin & 15u) == 0 && timer_ns() - t0 > t.wait_ns) gave_up = true;
                        lo = ld_volatile_v4(src);
                        hi = ld_volatile_v4(src + 1);
                    }
                    raw = make_uint4(lo.x, lo.z, hi.x, hi.z);
                }
                const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
                for (int q = 0; q < 4; ++q) {
                    acc[i][2 * q] += to_f<T>(word_lo<T>(w[q]));
                    acc[i][2 * q + 1] += to_f<T>(word_hi<T>(w[q]));
                }
            }
        }
    }
    if (__syncthreads_or(gave_up ? 1 : 0)) {
        if (tid == 0) atomicCAS(t.error, 0u, kErrPeerWait);
        return false;
    }
#pragma unroll
    for (int i = 0; i < NV; ++i)
#pragma unroll
        for (int q = 0; q < 8; ++q) x[i][q] = round_to<T>(acc[i][q]);
    return true;
}

// The call counter advances when the last CTA of the launch is through (every CTA read it at its start).
__device__ __forceinline__ void tp_rows_finish(const TpRowsArgs& t, uint32_t* s_epoch) {
    __syncthreads();
    if (threadIdx.x == 0 && atomicAdd(t.counters + 1, 1u) == gridDim.x - 1) {
        t.counters[1] = 0;
        __threadfence();
        *reinterpret_cast<volatile uint32_t*>(t.counters) = *s_epoch;
    }
}

template <typename T, int NV>
__device__ __forceinline__ void row_stats(RowStats<T>& rs, int D, float eps, float* red) {
    const int nvec = D / 8;
    float s = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i)
        if (threadIdx.x + i * kNMThreads < nvec) {
#pragma unroll
            for (int e = 0; e < 8; ++e) s += rs.x[i][e];
        }
    rs.mean = block_sum(s, red) / (float)D;
    float q = 0.f;
#pragma unroll
    for (int i = 0; i < NV; ++i)
        if (threadIdx.x + i * kNMThreads < nvec) {
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const float d = rs.x[i][e] - rs.mean;
                q += d * d;
            }
        }
    rs.rstd = rsqrtf(block_sum(q, red) / (float)D + eps);
}

// attn_norm_mix6 of (sum over ranks of partial); the summed row is also stored to x_out (the residual stream).
template <typename T, int NV>
__global__ void __launch_bounds__(kNMThreads, NV <= 2 ? 2 : 1) tp_attn_norm_mix6_kernel(const Mix6Args p, const TpRowsArgs t, void* x_out) {
    __shared__ float red[32];
    __shared__ uint32_t s_epoch;
    const int D = p.D, nvec = D / 8;
    Raw8<T> cw[NV], cb[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int vi = threadIdx.x + i * kNMThreads;
        if (vi < nvec) {
            cw[i] = ld_raw8(reinterpret_cast<const T*>(p.nw) + vi * 8);
            cb[i] = ld_raw8(reinterpret_cast<const T*>(p.nb) + vi * 8);
        }
    }
    grid_dependency_wait();
    if (threadIdx.x == 0) grid_launch_dependents();
    const uint32_t call = tp_rows_begin(t, &s_epoch);
#pragma unroll 1
    for (size_t row = blockIdx.x; row < (size_t)t.rows; row += gridDim.x) tp_rows_push<T, NV>(t, call, row, D);
#pragma unroll 1
    for (size_t row = blockIdx.x; row < (size_t)t.rows; row += gridDim.x) {
        // the six mix vectors are fetched per row, ahead of the wait for the peers, which hides their latency; held
        // across the row loop they would not fit the registers of two CTAs per SM
        Raw8<T> cm[6][NV];
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int vi = threadIdx.x + i * kNMThreads;
            if (vi < nvec) {
#pragma unroll
                for (int m = 0; m < 6; ++m) cm[m][i] = ld_raw8(reinterpret_cast<const T*>(p.mix[m]) + vi * 8);
            }
        }
        RowStats<T> rs;
        if (!tp_rows_sum<T, NV>(t, call, row, D, rs.x)) break;
        row_stats<T, NV>(rs, D, p.eps, red);
        T* prev = reinterpret_cast<T*>(p.prev) + (p.slots ? (size_t)__ldg(p.slots + row) : row) * D;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int vi = threadIdx.x + i * kNMThreads;
            if (vi < nvec) {
                float w[8], b[8], pv[8], h[8], d[8];
                cvt8(cw[i], w);
                cvt8(cb[i], b);
                load8(prev + vi * 8, pv);
                store8(reinterpret_cast<T*>(x_out) + row * D + vi * 8, rs.x[i]);
#pragma unroll
                for (int e = 0; e < 8; ++e) {
                    h[e] = (rs.x[i][e] - rs.mean) * rs.rstd * w[e] + b[e];
                    d[e] = pv[e] - h[e];
                }
                store8(prev + vi * 8, h);
#pragma unroll
                for (int m = 0; m < 6; ++m) {
                    float mx[8], o[8];
                    cvt8(cm[m][i], mx);
#pragma unroll
                    for (int e = 0; e < 8; ++e) o[e] = h[e] + d[e] * mx[e];
                    store8(reinterpret_cast<T*>(p.out[m]) + row * D + vi * 8, o);
                }
            }
        }
    }
    tp_rows_finish(t, &s_epoch);
}

// ffn_add_norm_mix with attn = sum over ranks of partial: res_out = res + attn (normalised from the fp32 sum).
template <typename T, int NV>
__global__ void __launch_bounds__(kNMThreads, NV <= 2 ? 2 : 1) tp_ffn_add_norm_mix_kernel(const FfnMixArgs p, const TpRowsArgs t) {
    __shared__ float red[32];
    __shared__ uint32_t s_epoch;
    const int D = p.D, nvec = D / 8;
    Raw8<T> cw[NV], cb[NV], cm[NV];
#pragma unroll
    for (int i = 0; i < NV; ++i) {
        const int vi = threadIdx.x + i * kNMThreads;
        if (vi < nvec) {
            cw[i] = ld_raw8(reinterpret_cast<const T*>(p.nw) + vi * 8);
            cb[i] = ld_raw8(reinterpret_cast<const T*>(p.nb) + vi * 8);
            cm[i] = ld_raw8(reinterpret_cast<const T*>(p.mix) + vi * 8);
        }
    }
    grid_dependency_wait();
    if (threadIdx.x == 0) grid_launch_dependents();
    const uint32_t call = tp_rows_begin(t, &s_epoch);
#pragma unroll 1
    for (size_t row = blockIdx.x; row < (size_t)t.rows; row += gridDim.x) tp_rows_push<T, NV>(t, call, row, D);
#pragma unroll 1
    for (size_t row = blockIdx.x; row < (size_t)t.rows; row += gridDim.x) {
        RowStats<T> rs;
        if (!tp_rows_sum<T, NV>(t, call, row, D, rs.x)) break;
        const T* res = reinterpret_cast<const T*>(p.res) + row * D;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int vi = threadIdx.x + i * kNMThreads;
            if (vi < nvec) {
                float r[8];
                load8(res + vi * 8, r);
#pragma unroll
                for (int e = 0; e < 8; ++e) rs.x[i][e] = r[e] + rs.x[i][e];
                store8(reinterpret_cast<T*>(p.res_out) + row * D + vi * 8, rs.x[i]);
            }
        }
        row_stats<T, NV>(rs, D, p.eps, red);
        T* prev = reinterpret_cast<T*>(p.prev) + (p.slots ? (size_t)__ldg(p.slots + row) : row) * D;
#pragma unroll
        for (int i = 0; i < NV; ++i) {
            const int vi = threadIdx.x + i * kNMThreads;
            if (vi < nvec) {
                float w[8], b[8], h[8], pv[8], mx[8], o[8];
                cvt8(cw[i], w);
                cvt8(cb[i], b);
#pragma unroll
                for (int e = 0; e < 8; ++e) h[e] = (rs.x[i][e] - rs.mean) * rs.rstd * w[e] + b[e];
                load8(prev + vi * 8, pv);
                cvt8(cm[i], mx);
#pragma unroll
                for (int e = 0; e < 8; ++e) o[e] = h[e] + (pv[e] - h[e]) * mx[e];
                store8(prev + vi * 8, h);
                store8(reinterpret_cast<T*>(p.mixed) + row * D + vi * 8, o);
            }
        }
    }
    tp_rows_finish(t, &s_epoch);
}

// How many CTAs of a row kernel are resident at once on this device (0 on error): the largest grid of the
// tensor-parallel forms, whose CTAs wait for the peers' CTAs of the same index.
template <auto kernel>  // (a template VALUE: every kernel has its own cache; all of them share one pointer type)
static int resident_ctas() {
    static std::atomic<int> cached{0};
    int n = cached.load(std::memory_order_relaxed);
    if (n > 0) return n;
    int dev = 0, sms = 0, per_sm = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 0;
    if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) return 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, kernel, kNMThreads, 0) != cudaSuccess) return 0;
    n = sms * per_sm;
    cached.store(n, std::memory_order_relaxed);
    return n;
}

static int fill_tp_args(const char* what, TpRowsArgs& t, const void* partial, void* const* inbox_ptrs, void* counters,
                        int rank, int world, int rows, int D, long long slot_elems, int wait_ms) {
    RWKV7_REQUIRE(world >= 2 && world <= kTpMaxRanks && rank >= 0 && rank < world, RWKV7_ERR_INVALID,
                  "%s: world must be 2..%d and rank inside it (world=%d rank=%d)", what, kTpMaxRanks, world, rank);
    RWKV7_REQUIRE(partial && inbox_ptrs && counters, RWKV7_ERR_INVALID, "%s: null pointer", what);
    RWKV7_REQUIRE(slot_elems % 8 == 0 && (long long)rows * D <= slot_elems, RWKV7_ERR_WORKSPACE,
                  "%s: %d x %d values do not fit an inbox slot of %lld", what, rows, D, slot_elems);
    RWKV7_REQUIRE(aligned(partial, 16) && aligned(counters, 8), RWKV7_ERR_ALIGN, "%s: unaligned pointer", what);
    t.partial = partial;
    for (int r = 0; r < world; ++r) {
        RWKV7_REQUIRE(inbox_ptrs[r] && aligned(inbox_ptrs[r], 16), RWKV7_ERR_INVALID, "%s: bad inbox pointer of rank %d", what, r);
        t.inbox[r] = reinterpret_cast<uint4*>(inbox_ptrs[r]);
    }
    t.counters = reinterpret_cast<uint32_t*>(counters);
    t.error = kernel_error_word();
    RWKV7_REQUIRE(t.error != nullptr, RWKV7_ERR_CUDA, "%s: cannot resolve the device error word", what);
    t.rank = rank;
    t.world = world;
    t.rows = rows;
    t.slot_elems = slot_elems;
    t.wait_ns = (unsigned long long)(wait_ms > 0 ? wait_ms : 2000) * 1000000ull;
    return RWKV7_OK;
}

}  // namespace rwkv7

using namespace rwkv7;

// vectors per thread for a row of D values: rows of <= 4096 values keep half the registers, so two CTAs share an SM
static int tp_vectors(int D) { return D <= 8 * kNMThreads ? 1 : (D <= 16 * kNMThreads ? 2 : 4); }

// Every CTA pushes all of its rows before it waits for any, and CTA c of one rank waits for CTA c of the others only:
// with the whole grid resident (on every rank alike: same kernel, same device type) nobody waits for a CTA that
// cannot start.  max_ctas > 0 lowers the bound (two such kernels side by side on two streams share the SMs).
static int tp_grid(const char* what, int rows, int resident, int max_ctas, int* grid) {
    RWKV7_REQUIRE(resident > 0, RWKV7_ERR_CUDA, "%s: cannot determine how many CTAs are resident", what);
    int g = max_ctas > 0 && max_ctas < resident ? max_ctas : resident;
    *grid = rows < g ? rows : g;
    return RWKV7_OK;
}

template <typename T>
static int tp_mix6_launch(int nv, int rows, int max_ctas, cudaStream_t st, const Mix6Args& p, const TpRowsArgs& t, void* x_out) {
    int grid = 0;
#define RWKV7_TP_MIX6(NV)                                                                                         \
    {                                                                                                             \
        if (int e = tp_grid("tp_attn_norm_mix6", rows, resident_ctas<tp_attn_norm_mix6_kernel<T, NV>>(), max_ctas, &grid)) return e; \
        launch_programmatic(tp_attn_norm_mix6_kernel<T, NV>, dim3(grid), dim3(kNMThreads), 0, st, p, t, x_out);   \
    }
    if (nv == 1) RWKV7_TP_MIX6(1) else if (nv == 2) RWKV7_TP_MIX6(2) else RWKV7_TP_MIX6(4)
#undef RWKV7_TP_MIX6
    return check_launch("tp_attn_norm_mix6_kernel");
}

template <typename T>
static int tp_ffn_launch(int nv, int rows, int max_ctas, cudaStream_t st, const FfnMixArgs& p, const TpRowsArgs& t) {
    int grid = 0;
#define RWKV7_TP_FFN(NV)                                                                                          \
    {                                                                                                             \
        if (int e = tp_grid("tp_ffn_add_norm_mix", rows, resident_ctas<tp_ffn_add_norm_mix_kernel<T, NV>>(), max_ctas, &grid)) return e; \
        launch_programmatic(tp_ffn_add_norm_mix_kernel<T, NV>, dim3(grid), dim3(kNMThreads), 0, st, p, t);        \
    }
    if (nv == 1) RWKV7_TP_FFN(1) else if (nv == 2) RWKV7_TP_FFN(2) else RWKV7_TP_FFN(4)
#undef RWKV7_TP_FFN
    return check_launch("tp_ffn_add_norm_mix_kernel");
}

extern "C" int rwkv7_tp_rows_resident(int D, int dtype) {
    if (D <= 0 || D % 8 || D > 8 * kNMThreads * kNMMaxVec) return 0;
    const int nv = tp_vectors(D);
    int a = 0, b = 0;
    if (dtype == RWKV7_F16) {
        a = nv == 1 ? resident_ctas<tp_attn_norm_mix6_kernel<__half, 1>>() : nv == 2 ? resident_ctas<tp_attn_norm_mix6_kernel<__half, 2>>() : resident_ctas<tp_attn_norm_mix6_kernel<__half, 4>>();
        b = nv == 1 ? resident_ctas<tp_ffn_add_norm_mix_kernel<__half, 1>>() : nv == 2 ? resident_ctas<tp_ffn_add_norm_mix_kernel<__half, 2>>() : resident_ctas<tp_ffn_add_norm_mix_kernel<__half, 4>>();
    } else if (dtype == RWKV7_BF16) {
        a = nv == 1 ? resident_ctas<tp_attn_norm_mix6_kernel<__nv_bfloat16, 1>>() : nv == 2 ? resident_ctas<tp_attn_norm_mix6_kernel<__nv_bfloat16, 2>>() : resident_ctas<tp_attn_norm_mix6_kernel<__nv_bfloat16, 4>>();
        b = nv == 1 ? resident_ctas<tp_ffn_add_norm_mix_kernel<__nv_bfloat16, 1>>() : nv == 2 ? resident_ctas<tp_ffn_add_norm_mix_kernel<__nv_bfloat16, 2>>() : resident_ctas<tp_ffn_add_norm_mix_kernel<__nv_bfloat16, 4>>();
    }
    return a < b ? a : b;
}

extern "C" int rwkv7_tp_attn_norm_mix6(const void* partial, void* x_out, void* prev, const int32_t* slot_ids,
                                       const void* norm_w, const void* norm_b, const void* const mixes[6],
                                       void* const outs[6], void* const* inbox_ptrs, void* counters, int rank, int world,
                                       int rows, int D, long long slot_elems, int max_ctas, float eps, int wait_ms,
                                       int dtype, void* stream) {
    if (int e = check_row_shape("tp_attn_norm_mix6", rows, D)) return e;
    RWKV7_REQUIRE(dtype == RWKV7_F16 || dtype == RWKV7_BF16, RWKV7_ERR_UNSUPPORTED, "tp_attn_norm_mix6: fp16 or bf16");
    RWKV7_REQUIRE(x_out && prev && norm_w && norm_b && mixes && outs, RWKV7_ERR_INVALID, "tp_attn_norm_mix6: null pointer");
    Mix6Args p{nullptr, norm_w, norm_b, prev, {}, {}, D, eps, slot_ids};
    for (int m = 0; m < 6; ++m) {
        RWKV7_REQUIRE(mixes[m] && outs[m] && aligned(mixes[m], 16) && aligned(outs[m], 16), RWKV7_ERR_INVALID,
                      "tp_attn_norm_mix6: bad mix / out pointer %d", m);
        p.mix[m] = mixes[m];
        p.out[m] = outs[m];
    }
    const void* ptrs[] = {x_out, prev, norm_w, norm_b};
    for (const void* q : ptrs) RWKV7_REQUIRE(aligned(q, 16), RWKV7_ERR_ALIGN, "tp_attn_norm_mix6: unaligned pointer");
    TpRowsArgs t{};
    if (int e = fill_tp_args("tp_attn_norm_mix6", t, partial, inbox_ptrs, counters, rank, world, rows, D, slot_elems, wait_ms))
        return e;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return dtype == RWKV7_F16 ? tp_mix6_launch<__half>(tp_vectors(D), rows, max_ctas, st, p, t, x_out)
                              : tp_mix6_launch<__nv_bfloat16>(tp_vectors(D), rows, max_ctas, st, p, t, x_out);
}

extern "C" int rwkv7_tp_ffn_add_norm_mix(const void* residual, const void* partial, void* prev, const int32_t* slot_ids,
                                         const void* norm_w, const void* norm_b, const void* mix, void* residual_out,
                                         void* mixed, void* const* inbox_ptrs, void* counters, int rank, int world, int rows,
                                         int D, long long slot_elems, int max_ctas, float eps, int wait_ms, int dtype,
                                         void* stream) {
    if (int e = check_row_shape("tp_ffn_add_norm_mix", rows, D)) return e;
    RWKV7_REQUIRE(dtype == RWKV7_F16 || dtype == RWKV7_BF16, RWKV7_ERR_UNSUPPORTED, "tp_ffn_add_norm_mix: fp16 or bf16");
    RWKV7_REQUIRE(residual && prev && norm_w && norm_b && mix && residual_out && mixed, RWKV7_ERR_INVALID,
                  "tp_ffn_add_norm_mix: null pointer");
    const void* ptrs[] = {residual, prev, norm_w, norm_b, mix, residual_out, mixed};
    for (const void* q : ptrs) RWKV7_REQUIRE(aligned(q, 16), RWKV7_ERR_ALIGN, "tp_ffn_add_norm_mix: unaligned pointer");
    FfnMixArgs p{residual, nullptr, norm_w, norm_b, mix, prev, residual_out, mixed, D, eps, slot_ids};
    TpRowsArgs t{};
    if (int e = fill_tp_args("tp_ffn_add_norm_mix", t, partial, inbox_ptrs, counters, rank, world, rows, D, slot_elems, wait_ms))
        return e;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    return dtype == RWKV7_F16 ? tp_ffn_launch<__half>(tp_vectors(D), rows, max_ctas, st, p, t)
                              : tp_ffn_launch<__nv_bfloat16>(tp_vectors(D), rows, max_ctas, st, p, t);
}
