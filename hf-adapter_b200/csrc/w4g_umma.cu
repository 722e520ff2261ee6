// Decode-time int4 group-wise projection on the 5th-generation tensor cores (M = 9..64 activation rows).
//
//   out[M, Nout] = epilogue( x[M, K] . W[Nout, K]^T ),  W = round_f16((nibble - zero) * scale)
//
// At these batch sizes the CUDA-core GEMV is FMA-bound (M*K*Nout MACs) while the weights still have
// to stream from HBM exactly once, so the contraction goes to tcgen05.mma and the kernel is built
// around keeping shared-memory traffic low, which is what otherwise caps a dequantising GEMM:
//
//   * the weights are read from a TILED copy of the reference's [Nout, K/2] array (rwkv7_w4g_repack, built once
//     at load): one 8 KiB block per [128 channels x 128 k] tile, blocks of a channel tile consecutive in memory,
//     so every CTA streams one contiguous region with 8 KiB bulk copies -- row-strided 64-byte pieces of the
//     row-major array reach under 1 TB/s on HBM3e, contiguous blocks run at copy speed;
//   * four dequant warps (thread = output channel) read their 64 packed bytes, expand them to 128
//     fp16 values in registers (lop3 magic-number conversion, exact (q - zero), one fp16 rounding
//     for the scale product = the reference's materialised weight) and write them with tcgen05.st
//     straight into TENSOR MEMORY as the A operand -- the 4x larger fp16 tile never touches shared
//     memory;
//   * the activation tile [64 rows x 128 k] arrives by TMA (128-byte swizzle) and is the B operand
//     from shared memory; D [128 x 64] fp32 accumulates in tensor memory;
//   * split-K runs as a thread-block cluster along z; partial tiles are reduced through distributed
//     shared memory in a fixed order (deterministic, no scratch buffer, no atomics), then the
//     relu^2 / residual epilogue is applied and fp16 results are stored coalesced.
//
// Warp roles (192 threads): warp 0 = TMA producer, warp 1 = TMEM allocator + MMA issuer, warps 2-5 =
// dequantise + epilogue.  All mbarrier waits are bounded (umma.cuh).
#include <cooperative_groups.h>

#include "umma.cuh"

namespace cg = cooperative_groups;

namespace rwkv7 {

namespace w4 {
constexpr int TILE_N = 128;  // output channels per CTA = UMMA M
constexpr int KB = 128;      // k elements per pipeline stage
constexpr int NB = 64;       // activation rows per MMA = UMMA N
constexpr int STAGES = 6;
constexpr int RAW_BYTES = TILE_N * KB / 2;  // 8192
constexpr int SC_BYTES = TILE_N * 2;        // per-channel fp16 scale of the k-block
constexpr int Z_BYTES = TILE_N;             // per-channel zero-point of the k-block
constexpr int META_BYTES = 512;             // scales + zeros, padded
constexpr int XATOM_BYTES = NB * 128;       // one 64-k swizzle atom of the activation tile
constexpr int X_BYTES = 2 * XATOM_BYTES;    // 16384
constexpr int STAGE_BYTES = RAW_BYTES + SC_BYTES + Z_BYTES + X_BYTES;  // bytes that land per stage
constexpr int TMEM_COLS = 256;  // A: 2 x 64 columns, D: 64 columns
constexpr int D_COL = 128;
constexpr int THREADS = 192;
}  // namespace w4

struct W4UmmaArgs {
    const uint8_t* tw;   // tiled weights  [tiles][K/128][4 chunks][128 channels][16 B]
    const __half* ts;    // tiled scales   [tiles][K/128][128]
    const uint8_t* tz;   // tiled zeros    [tiles][K/128][128]
    const __half* residual;
    __half* out;
    int M, K, Nout, epilogue, nkb, kbt, splits;  // kbt = K / 128 (k-blocks per channel tile)
    unsigned int* error;
};

// One 32-bit word of the tiled format holds 8 consecutive k in the nibble order [k0 k2 k4 k6 k1 k3 k5 k7]
// (nibble i at bits 4i), so the two-nibble masks below yield (k0,k1) (k2,k3) (k4,k5) (k6,k7) directly.
// 0x6400 | q is the fp16 number 1024 + q; the high-nibble form 1024 + 16 q is brought back with an exact fma.
__device__ __forceinline__ void dequant_word(uint32_t w, __half2 zlo, __half2 zhi, __half2 sc, uint32_t* out) {
    const __half2 sixteenth = __float2half2_rn(0.0625f);
    uint32_t t0 = (w & 0x000F000Fu) | 0x64006400u;   // 1024 + (k0, k1)
    uint32_t t1 = (w & 0x00F000F0u) | 0x64006400u;   // 1024 + 16*(k2, k3)
    const uint32_t w2 = w >> 8;
    uint32_t t2 = (w2 & 0x000F000Fu) | 0x64006400u;  // 1024 + (k4, k5)
    uint32_t t3 = (w2 & 0x00F000F0u) | 0x64006400u;  // 1024 + 16*(k6, k7)
    const __half2 v0 = __hmul2(__hsub2(*reinterpret_cast<__half2*>(&t0), zlo), sc);
    const __half2 v1 = __hmul2(__hfma2(*reinterpret_cast<__half2*>(&t1), sixteenth, zhi), sc);
    const __half2 v2 = __hmul2(__hsub2(*reinterpret_cast<__half2*>(&t2), zlo), sc);
    const __half2 v3 = __hmul2(__hfma2(*reinterpret_cast<__half2*>(&t3), sixteenth, zhi), sc);
    out[0] = *reinterpret_cast<const uint32_t*>(&v0);
    out[1] = *reinterpret_cast<const uint32_t*>(&v1);
    out[2] = *reinterpret_cast<const uint32_t*>(&v2);
    out[3] = *reinterpret_cast<const uint32_t*>(&v3);
}

__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

__global__ void __launch_bounds__(w4::THREADS, 1)
w4g_umma_kernel(const __grid_constant__ CUtensorMap tm_x, const W4UmmaArgs p) {
    using namespace w4;
    extern __shared__ unsigned char smem_unaligned[];
    // the swizzled TMA / UMMA tiles need 1024-byte alignment; the offset is the same in every CTA
    unsigned char* smem = smem_unaligned + ((1024u - (smem_u32(smem_unaligned) & 1023u)) & 1023u);
    // [stage][x atom 0 | x atom 1] | [stage][raw] | [stage][scales | zeros] | barriers
    unsigned char* xs = smem;
    unsigned char* raws = smem + STAGES * X_BYTES;
    unsigned char* metas = raws + STAGES * RAW_BYTES;
    uint64_t* bars = reinterpret_cast<uint64_t*>(metas + STAGES * META_BYTES);
    uint64_t* full = bars;                   // [STAGES]
    uint64_t* empty = bars + STAGES;         // [STAGES]
    uint64_t* a_ready = bars + 2 * STAGES;   // [2]
    uint64_t* a_free = a_ready + 2;          // [2]
    uint64_t* d_full = a_free + 2;           // [1]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(d_full + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    const AbortCtx actx{abort_flag, p.error};
    float* P = reinterpret_cast<float*>(smem);  // [NB][TILE_N] partial tile, reuses the x stages after the main loop

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n0 = blockIdx.x * TILE_N;
    const int split = blockIdx.z;
    const int kb0 = split * p.nkb;
    const int nkb = p.nkb;

    if (tid == 0) {
        tma_prefetch_desc(&tm_x);
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 4 + 1);  // 4 dequant warps + the MMA commit
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(&a_ready[a], 4);
            mbar_init(&a_free[a], 1);
        }
        mbar_init(d_full, 1);
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 1) tmem_alloc(tmem_slot, TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            for (int i = 0; i < nkb; ++i) {
                const int s = i % STAGES;
                if (i >= STAGES && !mbar_wait(&empty[s], ((i / STAGES) - 1) & 1, actx, kErrWaitEmpty)) break;
                mbar_expect_tx(&full[s], STAGE_BYTES);
                const int kblk = kb0 + i;
                const size_t blk = (size_t)blockIdx.x * p.kbt + kblk;  // tile-major block index
                bulk_load(raws + s * RAW_BYTES, p.tw + blk * RAW_BYTES, RAW_BYTES, &full[s]);
                bulk_load(metas + s * META_BYTES, p.ts + blk * TILE_N, SC_BYTES, &full[s]);
                bulk_load(metas + s * META_BYTES + SC_BYTES, p.tz + blk * TILE_N, Z_BYTES, &full[s]);
                tma_load_2d(xs + s * X_BYTES, &tm_x, &full[s], kblk * KB, 0);
                tma_load_2d(xs + s * X_BYTES + XATOM_BYTES, &tm_x, &full[s], kblk * KB + 64, 0);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc(TILE_N, NB, /*F32*/ 1, /*F16*/ 0, /*F16*/ 0);
            const uint32_t d_tmem = tmem_base + D_COL;
            bool ok = true;
            for (int i = 0; i < nkb && ok; ++i) {
                const int s = i % STAGES, a = i & 1;
                ok = mbar_wait(&full[s], (i / STAGES) & 1, actx, kErrWaitFull) &&
                     mbar_wait(&a_ready[a], (i / 2) & 1, actx, kErrWaitAReady);
                if (!ok) break;
                tc_fence_after();
                const uint32_t xbase = smem_u32(xs + s * X_BYTES);
#pragma unroll
                for (int j = 0; j < KB / 16; ++j) {
                    const uint64_t bdesc = make_sw128_kmajor_desc(xbase + (j >> 2) * XATOM_BYTES + (j & 3) * 32);
                    umma_f16_ts(d_tmem, tmem_base + a * 64 + j * 8, bdesc, idesc, (i > 0 || j > 0) ? 1u : 0u);
                }
                tc_commit(&a_free[a]);
                tc_commit(&empty[s]);
            }
            tc_commit(d_full);
        }
    } else {
        const int q = warp & 3;
        const int row = q * 32 + lane;
        const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
        bool ok = true;
        for (int i = 0; i < nkb && ok; ++i) {
            const int s = i % STAGES, a = i & 1;
            ok = mbar_wait(&full[s], (i / STAGES) & 1, actx, kErrWaitFull);
            if (!ok) break;
            // this channel's 64 packed bytes: chunk c (32 k) of all 128 channels is one 2 KiB slab, so the
            // threads of a warp read consecutive 16-byte pieces (no bank conflicts, no swizzle)
            const unsigned char* rrow = raws + s * RAW_BYTES + row * 16;
            uint4 pk[4];
#pragma unroll
            for (int c = 0; c < 4; ++c) pk[c] = *reinterpret_cast<const uint4*>(rrow + c * 2048);
            const __half sch = reinterpret_cast<const __half*>(metas + s * META_BYTES)[row];
            const float z = (float)(metas + s * META_BYTES + SC_BYTES)[row];
            __syncwarp();
            if (lane == 0) mbar_arrive(&empty[s]);
            if (i >= 2) {
                ok = mbar_wait(&a_free[a], ((i / 2) - 1) & 1, actx, kErrWaitAFree);
                if (!ok) break;
            }
            tc_fence_after();
            const __half2 sc = __half2half2(sch);
            const __half2 zlo = __float2half2_rn(1024.0f + z);
            const __half2 zhi = __float2half2_rn(-(64.0f + z));
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                uint32_t v[16];
                dequant_word(pk[c].x, zlo, zhi, sc, v + 0);
                dequant_word(pk[c].y, zlo, zhi, sc, v + 4);
                dequant_word(pk[c].z, zlo, zhi, sc, v + 8);
                dequant_word(pk[c].w, zlo, zhi, sc, v + 12);
                tmem_st16(lane_addr + a * 64 + c * 16, v);
            }
            tc_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&a_ready[a]);
        }
        // ---- accumulator tile -> shared memory partial P[m][n]
        if (ok) ok = mbar_wait(d_full, 0, actx, kErrWaitDFull);
        if (ok) {
            tc_fence_after();
#pragma unroll
            for (int c = 0; c < NB / 16; ++c) {
                uint32_t v[16];
                tmem_ld16(lane_addr + D_COL + c * 16, v);
                tc_wait_ld();
#pragma unroll
                for (int e = 0; e < 16; ++e) P[(c * 16 + e) * TILE_N + row] = __uint_as_float(v[e]);
            }
            tc_fence_before();
        }
    }

    // ---- split-K reduction across the cluster (fixed rank order) + epilogue
    cg::cluster_group cluster = cg::this_cluster();
    __syncthreads();
    if (p.splits > 1) cluster.sync();
    const bool aborted = (*abort_flag != 0);
    if (warp >= 2 && !aborted && n0 + (warp & 3) * 32 + lane < p.Nout) {
        const int n = (warp & 3) * 32 + lane;
        const int rows_per_rank = NB / p.splits;
        const int m_begin = split * rows_per_rank;
        const int m_end = min(p.M, m_begin + rows_per_rank);
        const float* Pr[8];
        for (int r = 0; r < 8; ++r) Pr[r] = (r < p.splits && p.splits > 1) ? cluster.map_shared_rank(P, r) : P;
        for (int mb = m_begin; mb < m_end; mb += 8) {  // 8 rows at a time: all loads in flight before any store
            float acc[8], res[8];
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                acc[u] = 0.f;
                res[u] = 0.f;
            }
            for (int r = 0; r < p.splits; ++r) {
#pragma unroll
                for (int u = 0; u < 8; ++u)
                    if (mb + u < m_end) acc[u] += Pr[r][(mb + u) * TILE_N + n];
            }
            if (p.epilogue == RWKV7_EPI_ADD) {
#pragma unroll
                for (int u = 0; u < 8; ++u)
                    if (mb + u < m_end) res[u] = __half2float(p.residual[(size_t)(mb + u) * p.Nout + n0 + n]);
            }
#pragma unroll
            for (int u = 0; u < 8; ++u) {
                if (mb + u < m_end) {
                    float y = __half2float(__float2half_rn(acc[u]));
                    if (p.epilogue == RWKV7_EPI_RELU2) {
                        y = fmaxf(y, 0.f);
                        y = y * y;
                    } else if (p.epilogue == RWKV7_EPI_ADD) {
                        y += res[u];
                    }
                    p.out[(size_t)(mb + u) * p.Nout + n0 + n] = __float2half_rn(y);
                }
            }
        }
    }
    if (p.splits > 1) cluster.sync();  // peers may still be reading this CTA's partial tile
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}

// ---------------------------------------------------------------- repack (load time)
// reference layout -> tiled layout described at the top of this file
template <typename T>
__global__ void w4g_repack_kernel(const uint8_t* __restrict__ packed, const T* __restrict__ scales, const uint8_t* __restrict__ zeros,
                                  uint32_t* __restrict__ tw, T* __restrict__ ts, uint8_t* __restrict__ tz,
                                  int K, int Nout, int group, long long total_words) {
    const long long widx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (widx >= total_words) return;
    // widx = (((tile * kbt + b) * 4 + c) * 128 + r) * 4 + j
    const int j = (int)(widx & 3);
    const int r = (int)((widx >> 2) & 127);
    const int c = (int)((widx >> 9) & 3);
    const long long blk = widx >> 11;
    const int kbt = K / 128;
    const int b = (int)(blk % kbt);
    const long long tile = blk / kbt;
    const long long n = tile * 128 + r;
    const int k = b * 128 + c * 32 + j * 8;
    uint32_t out = 0x88888888u;
    if (n < Nout) {
        const uint32_t w = *reinterpret_cast<const uint32_t*>(packed + n * (K / 2) + k / 2);  // nibble i = k + i
        out = 0;
        const int order[8] = {0, 2, 4, 6, 1, 3, 5, 7};
#pragma unroll
        for (int i = 0; i < 8; ++i) out |= ((w >> (4 * order[i])) & 15u) << (4 * i);
    }
    tw[widx] = out;
    if (c == 0 && j == 0) {
        const long long gi = n * (K / group) + (b * 128) / group;
        ts[blk * 128 + r] = (n < Nout) ? scales[gi] : from_f<T>(0.f);
        tz[blk * 128 + r] = (n < Nout && zeros) ? zeros[gi] : (uint8_t)8;
    }
}

int launch_w4g_umma_tiled(const void* x, const uint8_t* tw, const void* ts, const uint8_t* tz, const void* residual,
                          void* out, int M, int K, int Nout, int epilogue, cudaStream_t st) {
    using namespace w4;
    RWKV7_REQUIRE(M >= 1 && M <= NB, RWKV7_ERR_UNSUPPORTED, "w4g_gemv_tiled: M must be in 1..%d (got %d)", NB, M);
    RWKV7_REQUIRE(K % KB == 0, RWKV7_ERR_UNSUPPORTED, "w4g_gemv_tiled: K must be a multiple of %d (got %d)", KB, K);
    const int tiles = (Nout + TILE_N - 1) / TILE_N;
    const int total_kb = K / KB;
    int splits = 1;
    for (int s = 8; s >= 2; s >>= 1) {
        if (tiles * s <= 160 && total_kb % s == 0 && (total_kb / s) >= 4) {
            splits = s;
            break;
        }
    }
    const int nkb = total_kb / splits;
    CUtensorMap tm_x;
    if (int e = make_tmap_2d(&tm_x, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, x, M, K, NB, 64, CU_TENSOR_MAP_SWIZZLE_128B)) return e;
    W4UmmaArgs a{tw, reinterpret_cast<const __half*>(ts), tz, reinterpret_cast<const __half*>(residual),
                 reinterpret_cast<__half*>(out), M, K, Nout, epilogue, nkb, total_kb, splits, kernel_error_word()};
    RWKV7_REQUIRE(a.error != nullptr, RWKV7_ERR_CUDA, "w4g_gemv_tiled: cannot resolve the device error word");
    const size_t smem = (size_t)STAGES * (X_BYTES + RAW_BYTES + META_BYTES) + (2 * STAGES + 5) * 8 + 16 + 1024;
    cudaError_t e = cudaFuncSetAttribute(w4g_umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    RWKV7_REQUIRE(e == cudaSuccess, RWKV7_ERR_CUDA, "w4g_gemv_tiled: %s", cudaGetErrorString(e));
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(tiles, 1, splits);
    cfg.blockDim = dim3(THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = splits;
    cfg.attrs = attr;
    cfg.numAttrs = 1;
    e = cudaLaunchKernelEx(&cfg, w4g_umma_kernel, tm_x, a);
    RWKV7_REQUIRE(e == cudaSuccess, RWKV7_ERR_CUDA, "w4g_gemv_tiled launch: %s", cudaGetErrorString(e));
    return RWKV7_OK;
}

}  // namespace rwkv7

using namespace rwkv7;

extern "C" int64_t rwkv7_w4g_tiled_bytes(int K, int Nout, int64_t* scale_elems) {
    if (K <= 0 || Nout <= 0 || K % 128) return 0;
    const int64_t tiles = (Nout + 127) / 128, kbt = K / 128;
    if (scale_elems) *scale_elems = tiles * kbt * 128;
    return tiles * kbt * 8192;
}

extern "C" int rwkv7_w4g_repack(const uint8_t* packed, const void* scales, const uint8_t* zeros, uint8_t* tiled_w,
                                void* tiled_scales, uint8_t* tiled_zeros, int K, int Nout, int group, int dtype, void* stream) {
    RWKV7_REQUIRE(K > 0 && Nout > 0 && K % 128 == 0, RWKV7_ERR_UNSUPPORTED, "w4g_repack: K must be a positive multiple of 128");
    RWKV7_REQUIRE(group > 0 && group % 128 == 0 && K % group == 0, RWKV7_ERR_UNSUPPORTED,
                  "w4g_repack: group must be a multiple of 128 dividing K (group=%d K=%d)", group, K);
    RWKV7_REQUIRE(packed && scales && tiled_w && tiled_scales && tiled_zeros, RWKV7_ERR_INVALID, "w4g_repack: null pointer");
    RWKV7_REQUIRE(dtype == RWKV7_F16, RWKV7_ERR_UNSUPPORTED, "w4g_repack: the tiled format holds fp16 scales");
    RWKV7_REQUIRE(aligned(packed, 4) && aligned(tiled_w, 16) && aligned(tiled_scales, 16) && aligned(tiled_zeros, 16),
                  RWKV7_ERR_ALIGN, "w4g_repack: unaligned pointer");
    const long long tiles = (Nout + 127) / 128;
    const long long words = tiles * (K / 128) * 2048;
    w4g_repack_kernel<__half><<<(unsigned)((words + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        packed, reinterpret_cast<const __half*>(scales), zeros, reinterpret_cast<uint32_t*>(tiled_w),
        reinterpret_cast<__half*>(tiled_scales), tiled_zeros, K, Nout, group, words);
    return check_launch("w4g_repack_kernel");
}

extern "C" int rwkv7_w4g_gemv_tiled(const void* x, const uint8_t* tiled_w, const void* tiled_scales, const uint8_t* tiled_zeros,
                                    const void* residual, void* out, int M, int K, int Nout, int epilogue, int dtype,
                                    void* stream) {
    RWKV7_REQUIRE(x && tiled_w && tiled_scales && tiled_zeros && out, RWKV7_ERR_INVALID, "w4g_gemv_tiled: null pointer");
    RWKV7_REQUIRE(dtype == RWKV7_F16, RWKV7_ERR_UNSUPPORTED, "w4g_gemv_tiled: fp16 activations only");
    RWKV7_REQUIRE(epilogue >= 0 && epilogue <= 2, RWKV7_ERR_INVALID, "w4g_gemv_tiled: bad epilogue code %d", epilogue);
    RWKV7_REQUIRE(epilogue != RWKV7_EPI_ADD || residual, RWKV7_ERR_INVALID, "w4g_gemv_tiled: residual is required for the add epilogue");
    RWKV7_REQUIRE(aligned(x, 16) && aligned(tiled_w, 16) && aligned(tiled_scales, 16) && aligned(tiled_zeros, 16),
                  RWKV7_ERR_ALIGN, "w4g_gemv_tiled: pointers must be 16-byte aligned");
    return launch_w4g_umma_tiled(x, tiled_w, tiled_scales, tiled_zeros, residual, out, M, K, Nout, epilogue,
                                 static_cast<cudaStream_t>(stream));
}
