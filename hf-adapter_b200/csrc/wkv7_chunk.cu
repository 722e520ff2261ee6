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
constexpr int C = 64, N = 64, THREADS = 256;
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
constexpr int SMEM_BYTES = R_SMALL + 2048 + 1024;
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

__device__ __forceinline__ float to_tf32(float x) {
    uint32_t u;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(u) : "f"(x));
    return __uint_as_float(u);
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
    __half* raw_r = reinterpret_cast<__half*>(sm + R_RAW);
    __half* raw_k = raw_r + 4096;
    __half* raw_v = raw_k + 4096;
    __half* raw_kk = raw_v + 4096;
    __half* raw_a = raw_kk + 4096;
    float* raw_w = reinterpret_cast<float*>(raw_a + 4096);
    float* part = reinterpret_cast<float*>(sm + R_SMALL);  // [4][64] partial log-decay sums
    float* gref = part + 256;                              // [64]
    float* gl = gref + 64;                                 // [64]
    float* egref = gl + 64;                                // [64] e^{gref}
    float* egl = egref + 64;                               // [64] e^{gl}
    uint64_t* bar = reinterpret_cast<uint64_t*>(egl + 64);
    uint64_t* raw_bar = bar + 1;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(raw_bar + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    const AbortCtx actx{abort_flag, p.error};

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int q = warp & 3, hi = warp >> 2;  // TMEM lane quarter / column half
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
    if (tl < 64) {
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
        const int n = tid & 63, tq = tid >> 6;
        float* F1 = reinterpret_cast<float*>(sm + R_S0);  // [64 tokens][64 channels]; the S0 tile is written after phase A
        float lw[16];
        {
            float run = 0.f;
#pragma unroll
            for (int j = 0; j < 16; ++j) {
                const int t = tq * 16 + j;
                float v = 0.f;
                if (t0 + t < p.T) {
                    if (p.w_mode == 1) v = __logf(raw_w[t * 64 + n]);
                    else {
                        const float wv = __half2float(reinterpret_cast<const __half*>(raw_w)[t * 64 + n]);
                        v = p.w_mode == 2 ? -0.606531f * sigmoidf_(wv) : __logf(wv);
                    }
                }
                run += v;
                lw[j] = v;
            }
            part[tq * 64 + n] = run;
        }
        __syncthreads();
        {
            const float p0 = part[n], p1 = part[64 + n], p2 = part[128 + n], p3 = part[192 + n];
            const float g_ref = p0 + p1, g_l = p0 + p1 + p2 + p3;
            if (tq == 0) {
                gref[n] = g_ref;
                gl[n] = g_l;
                egref[n] = __expf(g_ref);
                egl[n] = __expf(g_l);
            }
            float gi = tq == 0 ? 0.f : tq == 1 ? p0 : tq == 2 ? p0 + p1 : p0 + p1 + p2;
            // e^{gref-gi} = 1/f1 and e^{gl-gi} = e^{gl-gref}/f1
            const float e_lr = __expf(g_l - g_ref);
            uint32_t kdp[8], bdp[8], vvp[8];
#pragma unroll
            for (int j = 0; j < 16; j += 2) {
                float kd[2], bd[2];
                __half vv[2];
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                    const int t = tq * 16 + j + u;
                    const bool valid = t0 + t < p.T;
                    gi += lw[j + u];
                    const float f1 = __expf(gi - g_ref);
                    F1[t * 64 + n] = f1;
                    const float f4 = e_lr * __frcp_rn(f1);
                    const float kx = valid ? __half2float(raw_k[t * 64 + n]) : 0.f;
                    const float bx = valid ? __half2float(raw_kk[t * 64 + n]) * __half2float(raw_a[t * 64 + n]) : 0.f;
                    kd[u] = kx * f4;
                    bd[u] = bx * f4;
                    vv[u] = valid ? raw_v[t * 64 + n] : __float2half(0.f);
                }
                const __half2 hk = __floats2half2_rn(kd[0], kd[1]), hb = __floats2half2_rn(bd[0], bd[1]), hv = __halves2half2(vv[0], vv[1]);
                kdp[j >> 1] = *reinterpret_cast<const uint32_t*>(&hk);
                bdp[j >> 1] = *reinterpret_cast<const uint32_t*>(&hb);
                vvp[j >> 1] = *reinterpret_cast<const uint32_t*>(&hv);
            }
            // 16 tokens = 32 bytes = two 16-byte chunks of row n
#pragma unroll
            for (int c = 0; c < 2; ++c) {
                const uint32_t kb = (tq * 16 + c * 8) * 2;
                *reinterpret_cast<uint4*>(sm + R_KB + sw128_offset(n, kb, 64)) = make_uint4(kdp[c * 4], kdp[c * 4 + 1], kdp[c * 4 + 2], kdp[c * 4 + 3]);
                *reinterpret_cast<uint4*>(sm + R_KB + sw128_offset(n, 128 + kb, 64)) = make_uint4(bdp[c * 4], bdp[c * 4 + 1], bdp[c * 4 + 2], bdp[c * 4 + 3]);
                *reinterpret_cast<uint4*>(sm + R_VU + sw128_offset(n, kb, 128)) = make_uint4(vvp[c * 4], vvp[c * 4 + 1], vvp[c * 4 + 2], vvp[c * 4 + 3]);
            }
        }
        __syncthreads();  // F1, gref visible
        // step 2, thread = (token t, 16 channels): the token-major tf32 tiles with 16-byte loads and stores
        {
            const int t = tid >> 2, nb = (tid & 3) * 16;
            const bool valid = t0 + t < p.T;
            float r16[16], k16[16], kk16[16], a16[16];
            load8(raw_r + t * 64 + nb, reinterpret_cast<float(&)[8]>(r16[0]));
            load8(raw_r + t * 64 + nb + 8, reinterpret_cast<float(&)[8]>(r16[8]));
            load8(raw_k + t * 64 + nb, reinterpret_cast<float(&)[8]>(k16[0]));
            load8(raw_k + t * 64 + nb + 8, reinterpret_cast<float(&)[8]>(k16[8]));
            load8(raw_kk + t * 64 + nb, reinterpret_cast<float(&)[8]>(kk16[0]));
            load8(raw_kk + t * 64 + nb + 8, reinterpret_cast<float(&)[8]>(kk16[8]));
            load8(raw_a + t * 64 + nb, reinterpret_cast<float(&)[8]>(a16[0]));
            load8(raw_a + t * 64 + nb + 8, reinterpret_cast<float(&)[8]>(a16[8]));
#pragma unroll
            for (int c = 0; c < 16; c += 4) {
                const float4 f1 = *reinterpret_cast<const float4*>(F1 + t * 64 + nb + c);
                float4 f2;  // e^{ge-gref}: f1 of the previous token; e^{-gref} for the first one
                if (t > 0) f2 = *reinterpret_cast<const float4*>(F1 + (t - 1) * 64 + nb + c);
                else {
                    const float4 er = *reinterpret_cast<const float4*>(egref + nb + c);
                    f2 = make_float4(__frcp_rn(er.x), __frcp_rn(er.y), __frcp_rn(er.z), __frcp_rn(er.w));
                }
                const float f1v[4] = {f1.x, f1.y, f1.z, f1.w}, f2v[4] = {f2.x, f2.y, f2.z, f2.w};
                float ae[4], rp[4], ki[4], bi[4];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float m = valid ? 1.f : 0.f;
                    const float f3 = __frcp_rn(f1v[e]);
                    ae[e] = to_tf32(-kk16[c + e] * f2v[e] * m);
                    rp[e] = to_tf32(r16[c + e] * f1v[e] * m);
                    ki[e] = to_tf32(k16[c + e] * f3 * m);
                    bi[e] = to_tf32(kk16[c + e] * a16[c + e] * f3 * m);
                }
                const uint32_t kb = (nb + c) * 4;
                *reinterpret_cast<float4*>(sm + R_A + sw128_offset(t, kb, 128)) = make_float4(ae[0], ae[1], ae[2], ae[3]);
                *reinterpret_cast<float4*>(sm + R_A + sw128_offset(64 + t, kb, 128)) = make_float4(rp[0], rp[1], rp[2], rp[3]);
                *reinterpret_cast<float4*>(sm + R_B + sw128_offset(t, kb, 128)) = make_float4(ki[0], ki[1], ki[2], ki[3]);
                *reinterpret_cast<float4*>(sm + R_B + sw128_offset(64 + t, kb, 128)) = make_float4(bi[0], bi[1], bi[2], bi[3]);
            }
        }
        __syncthreads();  // raw buffers and F1 consumed
        if (tid == 0 && tile + 1 < ntiles) {
            fence_proxy_async_smem();  // generic reads of the raw buffers are ordered before the refill
            load_raw(t0 + C);
        }
        if (tl < 64) {  // S0 e^{gref} operand tile and the D3 accumulator initialised with S0 e^{gl}
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
        {
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
        fence_proxy_async_smem();
        tc_fence_before();
        __syncthreads();
        // ---------------- phase C2: rhs = D2[0:64] += tril_strict(A_ak) V   (fp16, K = 64)
        if (tid == 0) {
            tc_fence_after();
            constexpr uint32_t idh = make_idesc(128, 64, 1, 0, 0);
            const uint64_t da = make_sw128_kmajor_desc(smem_u32(sm + R_AK));
            const uint64_t db = make_sw128_kmajor_desc(smem_u32(sm + R_VU));
#pragma unroll
            for (int j = 0; j < 4; ++j) umma_f16_ss(tmem + D2_COL, da + (uint64_t)(j * 2), db + (uint64_t)(j * 2), idh, 1);
            tc_commit(bar);
        }
        wait_mma();
        if (!ok) break;
        // ---------------- phase D: U = (I - tril_strict(A_ab))^-1 rhs
        if (tl < 64) {
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
        // Blocked forward substitution on 16-row blocks, U overwriting rhs in RH: the off-diagonal update
        // rhs_b += L[b][0..b) U[0..b) is spread over all threads, the 16-step in-block solve runs one thread per
        // value column.
        {
            const int i = tid & 63, tg = tid >> 6;
#pragma unroll 1
            for (int blk = 0; blk < 4; ++blk) {
                if (blk > 0) {
                    float acc[4] = {0.f, 0.f, 0.f, 0.f};
                    const int tr = blk * 16 + tg * 4;  // this thread's four rows
                    for (int s0 = 0; s0 < blk * 16; s0 += 4) {
                        const float u0 = RH[(s0 + 0) * ABS + i], u1 = RH[(s0 + 1) * ABS + i];
                        const float u2 = RH[(s0 + 2) * ABS + i], u3 = RH[(s0 + 3) * ABS + i];
#pragma unroll
                        for (int rr = 0; rr < 4; ++rr) {
                            const float4 m = *reinterpret_cast<const float4*>(AB + (tr + rr) * ABS + s0);
                            acc[rr] = fmaf(m.x, u0, fmaf(m.y, u1, fmaf(m.z, u2, fmaf(m.w, u3, acc[rr]))));
                        }
                    }
#pragma unroll
                    for (int rr = 0; rr < 4; ++rr) RH[(tr + rr) * ABS + i] += acc[rr];
                    __syncthreads();
                }
                if (tid < 64) {
                    float u[16];
#pragma unroll
                    for (int tt = 0; tt < 16; ++tt) {
                        const int t = blk * 16 + tt;
                        float a0 = RH[t * ABS + tid], a1 = 0.f;
#pragma unroll
                        for (int ss = 0; ss + 1 < tt; ss += 2) {
                            a0 = fmaf(AB[t * ABS + blk * 16 + ss], u[ss], a0);
                            a1 = fmaf(AB[t * ABS + blk * 16 + ss + 1], u[ss + 1], a1);
                        }
                        if (tt & 1) a0 = fmaf(AB[t * ABS + blk * 16 + tt - 1], u[tt - 1], a0);
                        u[tt] = a0 + a1;
                        RH[t * ABS + tid] = u[tt];
                    }
                }
                __syncthreads();
            }
            // U^T into the second K atom of [V^T | U^T]: row = value index i, k = 64 + token; thread (i, tg) packs 16 tokens
            uint32_t pk[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const __half2 h2 = __floats2half2_rn(RH[(tg * 16 + 2 * e) * ABS + i], RH[(tg * 16 + 2 * e + 1) * ABS + i]);
                pk[e] = *reinterpret_cast<const uint32_t*>(&h2);
            }
            *reinterpret_cast<uint4*>(sm + R_VU + sw128_offset(i, (64 + tg * 16) * 2, 128)) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
            *reinterpret_cast<uint4*>(sm + R_VU + sw128_offset(i, (64 + tg * 16 + 8) * 2, 128)) = make_uint4(pk[4], pk[5], pk[6], pk[7]);
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
        {
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

    if (tl < 64 && *abort_flag == 0) {
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
