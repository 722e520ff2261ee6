// Chunked (WY / DPLR) WKV-7 prefill scan with the intra-chunk contractions on tcgen05 tensor cores.
//
// One CTA per (sequence, head) walks the sequence in tiles of 64 tokens (the result does not depend on the
// tile length, so the caller's chunk size is only validated).  With a~ = -kk, b~ = kk*a, per-channel log-decay
// sums gi (inclusive) / ge (exclusive), gl = gi at the tile end and a centring point gref = gi at token 31:
//
//   A1 = [ a~ e^{ge-gref} ; r e^{gi-gref} ]   (128 x 64, tf32)      B1 = [ k e^{gref-gi} ; b~ e^{gref-gi} ]  (128 x 64)
//   D1 = A1 B1^T = [[A_ak A_ab],[A_qk A_qb]]  (128 x 128)           D2 = A1 (S0 e^{gref})^T = [ a~E S0^T ; rP S0^T ]
//   rhs = D2[0:64] + tril_strict(A_ak) V      (fp16 MMA)            U = (I - tril_strict(A_ab))^-1 rhs   (CUDA cores)
//   Y   = D2[64:128] + [tril(A_qk) tril(A_qb)] [V ; U]              S' = S0 e^{gl} + [V^T U^T] [k e^{gl-gi} ; b~ e^{gl-gi}]
//
// The decay-scaled factors span many orders of magnitude, so the products that contain them run as kind::tf32 on
// operands rounded to tf32 in shared memory; the products of bounded quantities (A_* against V, U and the
// end-of-tile-decayed keys) run as kind::f16.  All operands are written by the CTA's threads straight into
// K-major 128-byte-swizzled tiles; accumulators D1/D2/D3 live in tensor memory (256 columns); the state row of
// each value index stays in registers between tiles.  Every mbarrier wait is bounded (umma.cuh).
#include "umma.cuh"

namespace rwkv7 {
namespace ck {
constexpr int C = 64, N = 64, THREADS = 512;  // warps 0-7 own the TMEM lanes; warps 8-15 help in the CUDA-core phases
constexpr int ABS = 68;  // row stride (floats) of the fp32 A_ab / rhs arrays: 16-byte aligned, conflict-free
// shared-memory regions (bytes)
constexpr int R_A = 0;                      // A1 (tf32 128x64) | later AE (fp16 128 x 128)
constexpr int R_B = R_A + 32768;            // B1 (tf32 128x64) | later AB + RH (fp32 64 x 68 each)
constexpr int R_S0 = R_B + 36864;           // S0 e^{gref} (tf32 64 x 64)
constexpr int R_AK = R_S0 + 16384;          // tril_strict(A_ak) (fp16 128 x 64, rows 64.. zero)
constexpr int R_VU = R_AK + 16384;          // [V^T | U^T] (fp16 128 x 128, rows 64.. zero)
constexpr int R_KB = R_VU + 32768;          // [kD ; bD]^T (fp16 64 x 128)
constexpr int R_RAW = R_KB + 16384;         // r,k,v,kk,a (T 64x64 each) + w (fp32 64x64)
constexpr int R_SMALL = R_RAW + 5 * 8192 + 16384;
constexpr int R_INV = R_SMALL + 4096;     // inverses of the four 16 x 16 diagonal blocks of I - tril_strict(A_ab) (fp32)
constexpr int INVS = 20;                  // row stride (floats) of one inverse block: conflict-free 16-byte row reads
constexpr int SMEM_BYTES = R_INV + 4 * 16 * INVS * 4 + 1024;
constexpr int D1_COL = 0, D2_COL = 128, D3_COL = 192, TMEM_COLS = 256;
}  // namespace ck

struct ChunkArgs {
    const __half *r, *k, *v, *kk, *a;
    const void* w;
    const float* state_in;
    float* state_out;
    __half* y;
    int T, H, w_mode;
    unsigned int* error;
};

// Round to tf32 (nearest, ties away) with one integer add: the tensor core ignores the 13 low mantissa bits, so adding
// half an ulp of tf32 to the bit pattern is all the rounding needs (cvt.rna.tf32 runs on the quarter-rate conversion
// pipe, and this kernel rounds 16k values per tile).
__device__ __forceinline__ float to_tf32(float x) { return __uint_as_float(__float_as_uint(x) + 0x1000u); }
__device__ __forceinline__ float fast_rcp(float x) {
    float y;
    asm("rcp.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

struct ChunkMaps {
    CUtensorMap m[6];  // r, k, v, kk, a, w viewed as (64 channels, H, B*T tokens)
};

__global__ void __launch_bounds__(ck::THREADS, 1) wkv7_chunk_kernel(const __grid_constant__ ChunkMaps maps, const ChunkArgs p) {
    using namespace ck;
    extern __shared__ unsigned char smem_unaligned[];
    unsigned char* sm = smem_unaligned + ((1024u - (smem_u32(smem_unaligned) & 1023u)) & 1023u);
    float* AB = reinterpret_cast<float*>(sm + R_B);
    float* RH = AB + C * ABS;
    float* UU = reinterpret_cast<float*>(sm + R_S0);   // U (fp32 64 x 64) during the solve; the S0 tile is dead by then
    float* INV = reinterpret_cast<float*>(sm + R_INV);
    __half* raw_r = reinterpret_cast<__half*>(sm + R_RAW);
    __half* raw_k = raw_r + 4096;
    __half* raw_v = raw_k + 4096;
    __half* raw_kk = raw_v + 4096;
    __half* raw_a = raw_kk + 4096;
    float* raw_w = reinterpret_cast<float*>(raw_a + 4096);
    float* part = reinterpret_cast<float*>(sm + R_SMALL);  // [8][64] partial log-decay sums
    float* gref = part + 512;                              // [64]
    float* gl = gref + 64;                                 // [64]
    float* egref = gl + 64;                                // [64] e^{gref}
    float* egl = egref + 64;                               // [64] e^{gl}
    uint64_t* bar = reinterpret_cast<uint64_t*>(egl + 64);
    uint64_t* raw_bar = bar + 1;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(raw_bar + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    const AbortCtx actx{abort_flag, p.error};

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const bool main_warp = warp < 8;
    const int q = warp & 3, hi = (warp >> 2) & 1;  // TMEM lane quarter / column half (main warps)
    const int tl = q * 32 + lane;            // TMEM lane = accumulator row of this thread
    const int bh = blockIdx.x, b = bh / p.H, h = bh % p.H;
    const size_t tok_stride = (size_t)p.H * N;
    const size_t base = ((size_t)b * p.T * p.H + h) * N;
    const int wbytes = p.w_mode == 1 ? 4 : 2;

    if (tid == 0) {
        mbar_init(bar, 1);
        mbar_init(raw_bar, 1);
        *abort_flag = 0;
        mbar_fence_init();
        for (int i = 0; i < 6; ++i) tma_prefetch_desc(&maps.m[i]);
    }
    if (warp == 0) tmem_alloc(tmem_slot, TMEM_COLS);
    // rows 64..127 of the fp16 A-operand tiles stay zero for the whole kernel
    for (int i = tid; i < (16384 + 32768) / 16; i += THREADS) reinterpret_cast<uint4*>(sm + R_AK)[i] = make_uint4(0, 0, 0, 0);

    // state row of value index i = tl (< 64), columns hi*32..+31, kept in registers across tiles
    float S[32];
    if (main_warp && tl < 64) {
        const float* sp = p.state_in + ((size_t)bh * N + tl) * N + hi * 32;
#pragma unroll
        for (int c = 0; c < 32; c += 4) {
            const float4 t4 = *reinterpret_cast<const float4*>(sp + c);
            S[c] = t4.x; S[c + 1] = t4.y; S[c + 2] = t4.z; S[c + 3] = t4.w;
        }
    }

    // one thread fetches the six [64 tokens x 64 channels] slices of a tile with TMA (rows of the other heads are
    // skipped by the tensor map); tokens past T in the last tile are masked where they are consumed
    auto load_raw = [&](int t0) {
        mbar_expect_tx(raw_bar, 5 * 8192 + 64 * 64 * wbytes);
        const int row = b * p.T + t0;
        tma_load_3d(raw_r, &maps.m[0], raw_bar, 0, h, row);
        tma_load_3d(raw_k, &maps.m[1], raw_bar, 0, h, row);
        tma_load_3d(raw_v, &maps.m[2], raw_bar, 0, h, row);
        tma_load_3d(raw_kk, &maps.m[3], raw_bar, 0, h, row);
        tma_load_3d(raw_a, &maps.m[4], raw_bar, 0, h, row);
        tma_load_3d(raw_w, &maps.m[5], raw_bar, 0, h, row);
    };

    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;
    const uint32_t lane_addr = tmem + ((uint32_t)(q * 32) << 16);
    uint32_t phase = 0;
    bool ok = true;
    auto wait_mma = [&]() {  // one polling lane per warp; result broadcast
        if (lane == 0) ok = mbar_wait(bar, phase, actx, kErrWaitDFull);
        ok = __shfl_sync(0xffffffffu, ok, 0);
        phase ^= 1;
        tc_fence_after();
    };

    const int ntiles = (p.T + C - 1) / C;
    if (tid == 0) load_raw(0);
    uint32_t raw_phase = 0;
    for (int tile = 0; tile < ntiles && ok; ++tile) {
        const int t0 = tile * C;
        if (lane == 0) ok = mbar_wait(raw_bar, raw_phase, actx, kErrWaitFull);
        ok = __shfl_sync(0xffffffffu, ok, 0);
        raw_phase ^= 1;
        if (!ok) break;
        // ---------------- phase A: log-decay prefix sums, decay factors, operand tiles
        // step 1, thread = (channel n, token quarter tq): prefix sums along tokens, f1 = e^{gi-gref} to shared memory,
        // and the token-transposed fp16 tiles (rows = channel) with 16-byte stores
        const int n = tid & 63, tq = tid >> 6;  // tq = 0..7: tokens tq*8 .. tq*8+7
        float* F1 = reinterpret_cast<float*>(sm + R_S0);  // [64 tokens][64 channels]; the S0 tile is written after phase A
        float lw[8];
        {
            float wv[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int t = tq * 8 + j;
                wv[j] = p.w_mode == 1 ? raw_w[t * 64 + n] : __half2float(reinterpret_cast<const __half*>(raw_w)[t * 64 + n]);
            }
            float run = 0.f;
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                float v = p.w_mode == 2 ? -0.606531f * sigmoidf_(wv[j]) : __logf(wv[j]);
                v = (t0 + tq * 8 + j < p.T) ? v : 0.f;
                run += v;
                lw[j] = v;
            }
            part[tq * 64 + n] = run;
        }
        __syncthreads();
        {
            float gi = 0.f, g_ref = 0.f, g_l = 0.f;
#pragma unroll
            for (int qq = 0; qq < 8; ++qq) {
                const float pv = part[qq * 64 + n];
                gi += qq < tq ? pv : 0.f;
                g_ref += qq < 4 ? pv : 0.f;
                g_l += pv;
            }
            if (tq == 0) {
                gref[n] = g_ref;
                gl[n] = g_l;
                egref[n] = __expf(g_ref);
                egl[n] = __expf(g_l);
            }
            // e^{gref-gi} = 1/f1 and e^{gl-gi} = e^{gl-gref}/f1
            const float e_lr = __expf(g_l - g_ref);
            float kx[8], bx[8];
            __half vx[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const int t = tq * 8 + j;
                const bool valid = t0 + t < p.T;
                const float kv = __half2float(raw_k[t * 64 + n]);
                const float bv = __half2float(raw_kk[t * 64 + n]) * __half2float(raw_a[t * 64 + n]);
                const __half vv = raw_v[t * 64 + n];
                kx[j] = valid ? kv : 0.f;
                bx[j] = valid ? bv : 0.f;
                vx[j] = valid ? vv : __float2half(0.f);
            }
            uint32_t kdp[4], bdp[4], vvp[4];
#pragma unroll
            for (int j = 0; j < 8; j += 2) {
                float f4[2];
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                    gi += lw[j + u];
                    const float f1 = __expf(gi - g_ref);
                    F1[(tq * 8 + j + u) * 64 + n] = f1;
                    f4[u] = e_lr * fast_rcp(f1);
                }
                const __half2 hk = __floats2half2_rn(kx[j] * f4[0], kx[j + 1] * f4[1]);
                const __half2 hb = __floats2half2_rn(bx[j] * f4[0], bx[j + 1] * f4[1]);
                const __half2 hv = __halves2half2(vx[j], vx[j + 1]);
                kdp[j >> 1] = *reinterpret_cast<const uint32_t*>(&hk);
                bdp[j >> 1] = *reinterpret_cast<const uint32_t*>(&hb);
                vvp[j >> 1] = *reinterpret_cast<const uint32_t*>(&hv);
            }
            // 8 tokens = one 16-byte chunk of row n
            const uint32_t kb = tq * 16;
            *reinterpret_cast<uint4*>(sm + R_KB + sw128_offset(n, kb, 64)) = make_uint4(kdp[0], kdp[1], kdp[2], kdp[3]);
            *reinterpret_cast<uint4*>(sm + R_KB + sw128_offset(n, 128 + kb, 64)) = make_uint4(bdp[0], bdp[1], bdp[2], bdp[3]);
            *reinterpret_cast<uint4*>(sm + R_VU + sw128_offset(n, kb, 128)) = make_uint4(vvp[0], vvp[1], vvp[2], vvp[3]);
        }
        __syncthreads();  // F1, gref visible
        // step 2, thread = (token t, 8 channels): the token-major tf32 tiles with 16-byte loads and stores
        {
            const int t = tid >> 3, nb = (tid & 7) * 8;
            const float m = t0 + t < p.T ? 1.f : 0.f;
            float r8[8], k8[8], kk8[8], a8[8], f1v[8], f2v[8];
            load8(raw_r + t * 64 + nb, r8);
            load8(raw_k + t * 64 + nb, k8);
            load8(raw_kk + t * 64 + nb, kk8);
            load8(raw_a + t * 64 + nb, a8);
            load8(F1 + t * 64 + nb, f1v);
            // e^{ge-gref}: f1 of the previous token; e^{-gref} for the first one
            if (t > 0) load8(F1 + (t - 1) * 64 + nb, f2v);
            else {
                load8(egref + nb, f2v);
#pragma unroll
                for (int e = 0; e < 8; ++e) f2v[e] = fast_rcp(f2v[e]);
            }
            float ae[8], rp[8], ki[8], bi[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const float f3 = fast_rcp(f1v[e]) * m;
                const float kkm = kk8[e] * m;
                ae[e] = to_tf32(-kkm * f2v[e]);
                rp[e] = to_tf32(r8[e] * f1v[e] * m);
                ki[e] = to_tf32(k8[e] * f3);
                bi[e] = to_tf32(kk8[e] * a8[e] * f3);
            }
#pragma unroll
            for (int c = 0; c < 8; c += 4) {
                const uint32_t kb = (nb + c) * 4;
                *reinterpret_cast<float4*>(sm + R_A + sw128_offset(t, kb, 128)) = make_float4(ae[c], ae[c + 1], ae[c + 2], ae[c + 3]);
                *reinterpret_cast<float4*>(sm + R_A + sw128_offset(64 + t, kb, 128)) = make_float4(rp[c], rp[c + 1], rp[c + 2], rp[c + 3]);
                *reinterpret_cast<float4*>(sm + R_B + sw128_offset(t, kb, 128)) = make_float4(ki[c], ki[c + 1], ki[c + 2], ki[c + 3]);
                *reinterpret_cast<float4*>(sm + R_B + sw128_offset(64 + t, kb, 128)) = make_float4(bi[c], bi[c + 1], bi[c + 2], bi[c + 3]);
            }
        }
        __syncthreads();  // raw buffers and F1 consumed
        if (tid == 0 && tile + 1 < ntiles) {
            fence_proxy_async_smem();  // generic reads of the raw buffers are ordered before the refill
            load_raw(t0 + C);
        }
        if (main_warp && tl < 64) {  // S0 e^{gref} operand tile and the D3 accumulator initialised with S0 e^{gl}
            uint32_t d3[32];
#pragma unroll
            for (int c = 0; c < 32; c += 4) {
                float4 o;
                const float4 er = *reinterpret_cast<const float4*>(egref + hi * 32 + c);
                o.x = to_tf32(S[c] * er.x);
                o.y = to_tf32(S[c + 1] * er.y);
                o.z = to_tf32(S[c + 2] * er.z);
                o.w = to_tf32(S[c + 3] * er.w);
                *reinterpret_cast<float4*>(sm + R_S0 + sw128_offset(tl, (hi * 32 + c) * 4, 64)) = o;
#pragma unroll
                for (int e = 0; e < 4; ++e) d3[c + e] = __float_as_uint(S[c + e] * egl[hi * 32 + c + e]);
            }
            tmem_st16(lane_addr + D3_COL + hi * 32, reinterpret_cast<uint32_t(&)[16]>(d3[0]));
            tmem_st16(lane_addr + D3_COL + hi * 32 + 16, reinterpret_cast<uint32_t(&)[16]>(d3[16]));
            tc_wait_st();
        }
        fence_proxy_async_smem();
        tc_fence_before();
        __syncthreads();
        // ---------------- phase B: D1 = A1 B1^T, D2 = A1 S0^T (tf32)
        if (tid == 0) {
            tc_fence_after();
            constexpr uint32_t id128 = make_idesc(128, 128, 1, 2, 2), id64 = make_idesc(128, 64, 1, 2, 2);
            const uint64_t da = make_sw128_kmajor_desc(smem_u32(sm + R_A));
            const uint64_t db = make_sw128_kmajor_desc(smem_u32(sm + R_B));
            const uint64_t ds = make_sw128_kmajor_desc(smem_u32(sm + R_S0));
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const uint64_t oa = (uint64_t)(((j >> 2) * 128 * 128 + (j & 3) * 32) >> 4);
                const uint64_t os = (uint64_t)(((j >> 2) * 64 * 128 + (j & 3) * 32) >> 4);
                umma_tf32_ss(tmem + D1_COL, da + oa, db + oa, id128, j > 0);
                umma_tf32_ss(tmem + D2_COL, da + oa, ds + os, id64, j > 0);
            }
            tc_commit(bar);
        }
        wait_mma();
        if (!ok) break;
        // ---------------- phase C: mask D1 into tril_strict(A_ak) (fp16), tril_strict(A_ab) (fp32), [tril A_qk | tril A_qb] (fp16)
        for (int i = tid; i < 1024; i += THREADS) {  // rows 0..63 of both AE atoms are zero
            const int atom = i >> 9, rem = i & 511;
            reinterpret_cast<uint4*>(sm + R_A + atom * 16384)[rem] = make_uint4(0, 0, 0, 0);
        }
        if (main_warp) {
            const int t = tl & 63;
            const bool low = tl < 64;  // rows of a~E (low) or rP (high)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                uint32_t v[16];
                tmem_ld16(lane_addr + D1_COL + hi * 64 + c * 16, v);
                tc_wait_ld();
                if (low && hi == 1) {  // A_ab, strict lower triangle, fp32
#pragma unroll
                    for (int e = 0; e < 16; e += 4) {
                        const int s = c * 16 + e;
                        float4 o;
                        o.x = (s + 0 < t) ? __uint_as_float(v[e + 0]) : 0.f;
                        o.y = (s + 1 < t) ? __uint_as_float(v[e + 1]) : 0.f;
                        o.z = (s + 2 < t) ? __uint_as_float(v[e + 2]) : 0.f;
                        o.w = (s + 3 < t) ? __uint_as_float(v[e + 3]) : 0.f;
                        *reinterpret_cast<float4*>(AB + t * ABS + s) = o;
                    }
                } else {
                    uint32_t pk[8];
#pragma unroll
                    for (int e = 0; e < 16; e += 2) {
                        const int s = c * 16 + e;
                        const bool k0 = low ? (s < t) : (s <= t), k1 = low ? (s + 1 < t) : (s + 1 <= t);
                        const __half2 h2 = __floats2half2_rn(k0 ? __uint_as_float(v[e]) : 0.f, k1 ? __uint_as_float(v[e + 1]) : 0.f);
                        pk[e >> 1] = *reinterpret_cast<const uint32_t*>(&h2);
                    }
                    unsigned char* dst = low ? sm + R_AK + sw128_offset(t, c * 32, 128)
                                             : sm + R_A + sw128_offset(64 + t, (hi * 64 + c * 16) * 2, 128);
                    // 16 halves = two 16-byte chunks (chunk index differs by one: separate swizzled addresses)
                    *reinterpret_cast<uint4*>(dst) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                    unsigned char* dst2 = low ? sm + R_AK + sw128_offset(t, c * 32 + 16, 128)
                                              : sm + R_A + sw128_offset(64 + t, (hi * 64 + c * 16) * 2 + 16, 128);
                    *reinterpret_cast<uint4*>(dst2) = make_uint4(pk[4], pk[5], pk[6], pk[7]);
                }
            }
        }
        // ---------------- phase C2: rhs = D2[0:64] += tril_strict(A_ak) V   (fp16, K = 64)
        // Warps 0 and 1 wrote tril_strict(A_ak): they hand it to the tensor core at once (named barrier of 64 threads),
        // so the product runs under the other warps' masks and the block inverses below.
        if (warp < 2) {
            fence_proxy_async_smem();
            tc_fence_before();
            asm volatile("bar.sync 1, 64;" ::: "memory");
            if (tid == 0) {
                tc_fence_after();
                constexpr uint32_t idh = make_idesc(128, 64, 1, 0, 0);
                const uint64_t da = make_sw128_kmajor_desc(smem_u32(sm + R_AK));
                const uint64_t db = make_sw128_kmajor_desc(smem_u32(sm + R_VU));
#pragma unroll
                for (int j = 0; j < 4; ++j) umma_f16_ss(tmem + D2_COL, da + (uint64_t)(j * 2), db + (uint64_t)(j * 2), idh, 1);
                tc_commit(bar);
            }
        }
        fence_proxy_async_smem();
        tc_fence_before();
        __syncthreads();
        // While that product runs, four helper warps invert the 16 x 16 diagonal blocks of I - tril_strict(A_ab):
        // lane c of warp 8 + b builds column c of block b by forward substitution in registers.
        if (warp >= 8 && warp < 12 && lane < 16) {
            const int blk = warp - 8;
            const float* L = AB + (blk * 16) * ABS + blk * 16;
            float x[16];
#pragma unroll
            for (int t = 0; t < 16; ++t) {
                float a0 = t == lane ? 1.f : 0.f, a1 = 0.f;
#pragma unroll
                for (int ss = 0; ss + 1 < t; ss += 2) {
                    a0 = fmaf(L[t * ABS + ss], x[ss], a0);
                    a1 = fmaf(L[t * ABS + ss + 1], x[ss + 1], a1);
                }
                if (t & 1) a0 = fmaf(L[t * ABS + t - 1], x[t - 1], a0);
                x[t] = a0 + a1;
                INV[(blk * 16 + t) * INVS + lane] = x[t];
            }
        }
        wait_mma();
        if (!ok) break;
        // ---------------- phase D: U = (I - tril_strict(A_ab))^-1 rhs
        if (main_warp && tl < 64) {
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                uint32_t v[16];
                tmem_ld16(lane_addr + D2_COL + hi * 32 + c * 16, v);
                tc_wait_ld();
#pragma unroll
                for (int e = 0; e < 16; e += 4)
                    *reinterpret_cast<float4*>(RH + tl * ABS + hi * 32 + c * 16 + e) =
                        make_float4(__uint_as_float(v[e]), __uint_as_float(v[e + 1]), __uint_as_float(v[e + 2]), __uint_as_float(v[e + 3]));
            }
        }
        tc_fence_before();
        __syncthreads();
        // Blocked forward substitution on 16-row blocks.  Value columns are independent, so each sweeping warp takes a
        // group of columns through all four blocks with warp-level syncs only; a lane owns rows rg, rg+4, rg+8, rg+12
        // of the block and CW columns:
        //   (a) rhs_b += L[b][0..b) U[0..b)        (b) U_b = inv(I - L_bb) rhs_b
        constexpr int CW = 2;                   // value columns per lane (measured: 2 columns on 4 warps 1.17 ms, 1 column on 8 warps 1.22 ms)
        constexpr int SWEEP_WARPS = 8 / CW;     // 8 lanes x CW columns per warp
        if (warp < SWEEP_WARPS) {
            const int rg = lane >> 3, col = warp * (8 * CW) + (lane & 7) * CW;
#pragma unroll 1
            for (int blk = 0; blk < 4; ++blk) {
                const int r0 = blk * 16 + rg;
                if (blk > 0) {
                    float acc[4][CW];
#pragma unroll
                    for (int rr = 0; rr < 4; ++rr)
#pragma unroll
                        for (int c = 0; c < CW; ++c) acc[rr][c] = RH[(r0 + 4 * rr) * ABS + col + c];
#pragma unroll 2
                    for (int s0 = 0; s0 < blk * 16; s0 += 4) {
                        float u[4][CW];
#pragma unroll
                        for (int e = 0; e < 4; ++e)
#pragma unroll
                            for (int c = 0; c < CW; ++c) u[e][c] = UU[(s0 + e) * 64 + col + c];
#pragma unroll
                        for (int rr = 0; rr < 4; ++rr) {
                            const float4 m = *reinterpret_cast<const float4*>(AB + (r0 + 4 * rr) * ABS + s0);
#pragma unroll
                            for (int c = 0; c < CW; ++c)
                                acc[rr][c] = fmaf(m.x, u[0][c], fmaf(m.y, u[1][c], fmaf(m.z, u[2][c], fmaf(m.w, u[3][c], acc[rr][c]))));
                        }
                    }
#pragma unroll
                    for (int rr = 0; rr < 4; ++rr)
#pragma unroll
                        for (int c = 0; c < CW; ++c) RH[(r0 + 4 * rr) * ABS + col + c] = acc[rr][c];
                    __syncwarp();
                }
                float o[4][CW];
#pragma unroll
                for (int rr = 0; rr < 4; ++rr)
#pragma unroll
                    for (int c = 0; c < CW; ++c) o[rr][c] = 0.f;
#pragma unroll
                for (int s0 = 0; s0 < 16; s0 += 4) {
                    float x[4][CW];
#pragma unroll
                    for (int e = 0; e < 4; ++e)
#pragma unroll
                        for (int c = 0; c < CW; ++c) x[e][c] = RH[(blk * 16 + s0 + e) * ABS + col + c];
#pragma unroll
                    for (int rr = 0; rr < 4; ++rr) {
                        const float4 m = *reinterpret_cast<const float4*>(INV + (r0 + 4 * rr) * INVS + s0);
#pragma unroll
                        for (int c = 0; c < CW; ++c)
                            o[rr][c] = fmaf(m.x, x[0][c], fmaf(m.y, x[1][c], fmaf(m.z, x[2][c], fmaf(m.w, x[3][c], o[rr][c]))));
                    }
                }
#pragma unroll
                for (int rr = 0; rr < 4; ++rr)
#pragma unroll
                    for (int c = 0; c < CW; ++c) UU[(r0 + 4 * rr) * 64 + col + c] = o[rr][c];
                __syncwarp();
            }
        }
        __syncthreads();
        {
            const int i = tid & 63, tg = tid >> 6;
            // U^T into the second K atom of [V^T | U^T]: row = value index i, k = 64 + token; thread (i, tg) packs 8 tokens
            uint32_t pk[4];
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const __half2 h2 = __floats2half2_rn(UU[(tg * 8 + 2 * e) * 64 + i], UU[(tg * 8 + 2 * e + 1) * 64 + i]);
                pk[e] = *reinterpret_cast<const uint32_t*>(&h2);
            }
            *reinterpret_cast<uint4*>(sm + R_VU + sw128_offset(i, (64 + tg * 8) * 2, 128)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
        }
        fence_proxy_async_smem();
        __syncthreads();
        // ---------------- phase E / F: Y = D2[64:128] += [A_qk A_qb][V;U];  S' = D3 += [V^T U^T][kD;bD]   (fp16, K = 128)
        if (tid == 0) {
            tc_fence_after();
            constexpr uint32_t idh = make_idesc(128, 64, 1, 0, 0);
            const uint64_t dae = make_sw128_kmajor_desc(smem_u32(sm + R_A));
            const uint64_t dvu = make_sw128_kmajor_desc(smem_u32(sm + R_VU));
            const uint64_t dkb = make_sw128_kmajor_desc(smem_u32(sm + R_KB));
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const uint64_t o128 = (uint64_t)(((j >> 2) * 128 * 128 + (j & 3) * 32) >> 4);
                const uint64_t o64 = (uint64_t)(((j >> 2) * 64 * 128 + (j & 3) * 32) >> 4);
                umma_f16_ss(tmem + D2_COL, dae + o128, dvu + o128, idh, 1);
                umma_f16_ss(tmem + D3_COL, dvu + o128, dkb + o64, idh, 1);
            }
            tc_commit(bar);
        }
        wait_mma();
        if (!ok) break;
        // ---------------- phase G: outputs of the tile, new state rows back to registers
        if (main_warp) {
            uint32_t v[32];
            const uint32_t col = (tl < 64 ? D3_COL : D2_COL) + hi * 32;
            tmem_ld16(lane_addr + col, reinterpret_cast<uint32_t(&)[16]>(v[0]));
            tmem_ld16(lane_addr + col + 16, reinterpret_cast<uint32_t(&)[16]>(v[16]));
            tc_wait_ld();
            if (tl < 64) {
#pragma unroll
                for (int c = 0; c < 32; ++c) S[c] = __uint_as_float(v[c]);
            } else {
                const int t = tl - 64;
                if (t0 + t < p.T) {
                    __half* yp = p.y + base + (size_t)(t0 + t) * tok_stride + hi * 32;
#pragma unroll
                    for (int c = 0; c < 32; c += 8) {
                        uint32_t pk[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e) {
                            const __half2 h2 = __floats2half2_rn(__uint_as_float(v[c + 2 * e]), __uint_as_float(v[c + 2 * e + 1]));
                            pk[e] = *reinterpret_cast<const uint32_t*>(&h2);
                        }
                        *reinterpret_cast<uint4*>(yp + c) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                    }
                }
            }
        }
        tc_fence_before();
        __syncthreads();  // accumulators and operand tiles are free for the next tile
    }

    if (main_warp && tl < 64 && *abort_flag == 0) {
        float* sp = p.state_out + ((size_t)bh * N + tl) * N + hi * 32;
#pragma unroll
        for (int c = 0; c < 32; c += 4) *reinterpret_cast<float4*>(sp + c) = make_float4(S[c], S[c + 1], S[c + 2], S[c + 3]);
    }
    tc_fence_before();
    __syncthreads();
    if (warp == 0) {
        tc_fence_after();
        tmem_dealloc(tmem, TMEM_COLS);
    }
}

}  // namespace rwkv7

using namespace rwkv7;

extern "C" int rwkv7_wkv7_chunk_scan(const void* r, const void* w, const void* k, const void* v, const void* kk, const void* a,
                                     const float* state_in, float* state_out, void* y, int B, int T, int H, int N, int chunk,
                                     int dtype, int w_mode, void* stream) {
    RWKV7_REQUIRE(N == 64, RWKV7_ERR_UNSUPPORTED, "wkv7_chunk_scan: head size must be 64, got %d", N);
    RWKV7_REQUIRE(dtype == RWKV7_F16, RWKV7_ERR_UNSUPPORTED, "wkv7_chunk_scan: fp16 activations only");
    RWKV7_REQUIRE(chunk == 16 || chunk == 32 || chunk == 64, RWKV7_ERR_UNSUPPORTED, "wkv7_chunk_scan: chunk must be 16, 32 or 64");
    RWKV7_REQUIRE(B > 0 && H > 0 && T > 0 && T % chunk == 0, RWKV7_ERR_INVALID,
                  "wkv7_chunk_scan: B, H, T must be positive and T a multiple of chunk (B=%d T=%d H=%d chunk=%d)", B, T, H, chunk);
    RWKV7_REQUIRE(w_mode >= 0 && w_mode <= 2, RWKV7_ERR_INVALID, "wkv7_chunk_scan: w_mode must be 0, 1 or 2");
    RWKV7_REQUIRE(r && w && k && v && kk && a && state_in && state_out && y, RWKV7_ERR_INVALID, "wkv7_chunk_scan: null pointer");
    const void* ptrs[] = {r, w, k, v, kk, a, state_in, state_out, y};
    for (const void* q : ptrs) RWKV7_REQUIRE(aligned(q, 16), RWKV7_ERR_ALIGN, "wkv7_chunk_scan: pointers must be 16-byte aligned");
    ChunkArgs p{reinterpret_cast<const __half*>(r), reinterpret_cast<const __half*>(k), reinterpret_cast<const __half*>(v),
                reinterpret_cast<const __half*>(kk), reinterpret_cast<const __half*>(a), w, state_in, state_out,
                reinterpret_cast<__half*>(y), T, H, w_mode, kernel_error_word()};
    RWKV7_REQUIRE(p.error != nullptr, RWKV7_ERR_CUDA, "wkv7_chunk_scan: cannot resolve the device error word");
    ChunkMaps maps;
    const void* srcs[6] = {r, k, v, kk, a, w};
    for (int i = 0; i < 6; ++i) {
        const bool f32 = (i == 5 && w_mode == 1);
        if (int e2 = make_tmap_tokens(&maps.m[i], srcs[i], f32 ? 4 : 2, (uint64_t)B * T, H)) return e2;
    }
    cudaError_t e = cudaFuncSetAttribute(wkv7_chunk_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, ck::SMEM_BYTES);
    RWKV7_REQUIRE(e == cudaSuccess, RWKV7_ERR_CUDA, "wkv7_chunk_scan: %s", cudaGetErrorString(e));
    wkv7_chunk_kernel<<<B * H, ck::THREADS, ck::SMEM_BYTES, static_cast<cudaStream_t>(stream)>>>(maps, p);
    return check_launch("wkv7_chunk_kernel");
}
