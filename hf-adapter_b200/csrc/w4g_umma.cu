// Decode-time int4 group-wise projection on the 5th-generation tensor cores (M = 9..64 activation rows).
//
//   out[M, Nout] = epilogue( x[M, K] . W[Nout, K]^T ),  W = round_f16((nibble - zero) * scale)
//
// At these batch sizes the CUDA-core GEMV is FMA-bound (M*K*Nout MACs) while the weights still have
// to stream from HBM exactly once, so the contraction goes to tcgen05.mma and the kernel is built
// around keeping shared-memory traffic low, which is what otherwise caps a dequantising GEMM:
//
//   * the weights are read from a TILED copy of the reference's [Nout, K/2] array (rwkv7_w4g_repack, built once
//     at load): one 8.5 KiB block per [128 channels x 128 k] tile (nibbles, then the tile's scales and zero-points),
//     blocks of a channel tile consecutive in memory, so every CTA streams one contiguous region, one bulk copy per block -- row-strided 64-byte pieces of the
//     row-major array reach under 1 TB/s on HBM3e, contiguous blocks run at copy speed;
//   * four dequant warps (thread = output channel) read their 64 packed bytes, expand them to 128
//     fp16 values in registers (lop3 magic-number conversion, exact (q - zero), one fp16 rounding
//     for the scale product = the reference's materialised weight) and write them with tcgen05.st
//     straight into TENSOR MEMORY as the A operand -- the 4x larger fp16 tile never touches shared
//     memory;
//   * the activation tile [64 rows x 128 k] arrives by TMA (128-byte swizzle) and is the B operand
//     from shared memory; D [128 x 64] fp32 accumulates in tensor memory;
//   * split-K runs as a thread-block cluster along z; every CTA PUSHES the rows of its partial tile that belong to
//     rank k straight from the accumulator registers into slot [own rank] of rank k's shared memory (remote
//     stores are fire-and-forget, remote loads would cost a round trip), one cluster barrier, then each rank sums
//     its slots in fixed rank order (deterministic, no scratch buffer, no atomics), applies the relu^2 / residual
//     epilogue and stores fp16 results coalesced.
//
// Warp roles: warp 0 = weight-stream producer, last warp = activation-tile producer, warp 1 and the last but one =
// MMA issuers (warp 1 also owns the TMEM allocation), warps 2..2+4*SB-1 = SB dequantise groups (k-block i of a
// super-block goes to group i) + epilogue.  All mbarrier waits are bounded (umma.cuh).
#include <cooperative_groups.h>

#include <mutex>
#include <unordered_set>

#include "umma.cuh"

namespace cg = cooperative_groups;

namespace rwkv7 {

namespace w4 {
constexpr int TILE_N = 128;  // output channels per CTA = UMMA M
constexpr int KB = 128;      // k elements per pipeline stage
constexpr int WB = 2;        // tile blocks per bulk copy (17 KiB requests: a bare copy ring of this shape moved 33.5 MB in
                             // 6.9 us against 9.5-10.6 us with 8.5 KiB ones; in this kernel, whose ring is kept full
                             // by the slower consumer side, the step time did not change)
constexpr int RAW_BYTES = TILE_N * KB / 2;  // 8192 packed nibbles
constexpr int SC_OFF = RAW_BYTES;           // then 128 fp16 scales of the k-block
constexpr int Z_OFF = SC_OFF + TILE_N * 2;  // then 128 u8 zero-points, then padding
constexpr int BLOCK_BYTES = 8704;           // one tile block in memory = one bulk copy (68 x 128 B)
constexpr int SB = 3;            // dequant warp groups: group g expands copies g, g + SB, g + 2 SB, ...
constexpr int TMEM_COLS = 512;   // A: NAB x 64 columns, D: NISS x NB columns
constexpr int ISS2_WARP = 2 + SB * 4;           // second issuer = last warp
constexpr int XPROD_WARP = ISS2_WARP + 1;       // activation-tile producer
constexpr int THREADS = 64 + SB * 128 + 64;

// Two shapes of the same kernel: 64 activation rows per weight pass (decode batches up to 64: deep rings, six A buffers)
// and 128 rows per pass (larger batches, e.g. tensor-parallel decode: every dequantised block feeds an MMA twice as
// wide, so the dequantisation and the weight stream are paid once per 128 rows; shorter rings pay for the wider tiles).
template <int NB_>
struct Cfg;
// NISS = MMA issuer warps, each with its own accumulator (summed in the epilogue), taking k-blocks i = me (mod NISS).
// A waiter must see every phase of a barrier it waits on, so the activation ring and the A buffers, which are indexed
// by i, need a length that is a multiple of NISS: then a stage or buffer always belongs to the same issuer.  (With
// three stages and two issuers an issuer skips every other phase of a stage's barrier, a parity wait passes a phase
// early and the ring runs out of step until a wait never completes.)  The same holds for the dequant groups: the
// weight ring (in copies) is a multiple of SB and the A buffers a multiple of WB * SB.
template <>
struct Cfg<64> {
    static constexpr int NB = 64, STAGES = 4, WSTAGES = 6, NAB = 6, NISS = 2;
};
template <>
struct Cfg<128> {
    static constexpr int NB = 128, STAGES = 3, WSTAGES = 3, NAB = 6, NISS = 1;
};
template <int NB_>
constexpr size_t smem_bytes() {
    using C = Cfg<NB_>;
    return (size_t)C::STAGES * 2 * C::NB * 128 + (size_t)C::WSTAGES * WB * BLOCK_BYTES + (size_t)C::NB * TILE_N * 4 +
           (2 * C::STAGES + 2 * C::WSTAGES + 2 * C::NAB + 1) * 8 + 16 + 1024;
}
}  // namespace w4

constexpr int kW4MaxGroup = 4;  // projections of equal shape served by one launch (r / k / v of a layer)

struct W4UmmaArgs {
    const uint8_t* tw[kW4MaxGroup];  // tiled weights: [tiles][K/128] blocks of BLOCK_BYTES = [4 chunks][128 channels][16 B] | scales | zeros
    __half* out[kW4MaxGroup];
    const __half* residual;          // add epilogue (single projection only)
    int M, K, Nout, epilogue, nkb, kbt, splits, row_blocks;  // kbt = K / 128 (k-blocks per channel tile)
    unsigned int* error;
};

struct W4Maps {
    CUtensorMap x[kW4MaxGroup];  // activations of each projection as (k_in 64, row, k_out)
};

// One 32-bit word of the tiled format holds 8 consecutive k in the nibble order [k0 k2 k4 k6 k1 k3 k5 k7]
// (nibble i at bits 4i), so the two-nibble masks below yield (k0,k1) (k2,k3) (k4,k5) (k6,k7) directly.
// 0x6400 | q is the fp16 number 1024 + q; the high-nibble form 1024 + 16 q is brought back with an exact fma.
// All in 32-bit registers (packed fp16 pairs), one instruction per step: lop3 (w & mask) | magic, then
// sub / fma and mul on f16x2.
__device__ __forceinline__ uint32_t and_or(uint32_t a, uint32_t mask, uint32_t orv) {
    uint32_t d;
    asm("lop3.b32 %0, %1, %2, %3, 0xEA;" : "=r"(d) : "r"(a), "r"(mask), "r"(orv));
    return d;
}
__device__ __forceinline__ uint32_t sub_mul_h2(uint32_t t, uint32_t z, uint32_t sc) {
    uint32_t d;
    asm("{\n\t.reg .b32 u;\n\tsub.f16x2 u, %1, %2;\n\tmul.f16x2 %0, u, %3;\n\t}" : "=r"(d) : "r"(t), "r"(z), "r"(sc));
    return d;
}
__device__ __forceinline__ uint32_t fma_mul_h2(uint32_t t, uint32_t m, uint32_t z, uint32_t sc) {
    uint32_t d;
    asm("{\n\t.reg .b32 u;\n\tfma.rn.f16x2 u, %1, %2, %3;\n\tmul.f16x2 %0, u, %4;\n\t}" : "=r"(d) : "r"(t), "r"(m), "r"(z), "r"(sc));
    return d;
}
__device__ __forceinline__ void dequant_word(uint32_t w, uint32_t zlo, uint32_t zhi, uint32_t sc, uint32_t* out) {
    constexpr uint32_t kSixteenth = 0x2C002C00u;  // (1/16, 1/16) in fp16
    constexpr uint32_t kMagic = 0x64006400u;      // (1024, 1024)
    const uint32_t w2 = w >> 8;
    out[0] = sub_mul_h2(and_or(w, 0x000F000Fu, kMagic), zlo, sc);               // 1024 + (k0, k1)
    out[1] = fma_mul_h2(and_or(w, 0x00F000F0u, kMagic), kSixteenth, zhi, sc);   // 1024 + 16*(k2, k3)
    out[2] = sub_mul_h2(and_or(w2, 0x000F000Fu, kMagic), zlo, sc);              // 1024 + (k4, k5)
    out[3] = fma_mul_h2(and_or(w2, 0x00F000F0u, kMagic), kSixteenth, zhi, sc);  // 1024 + 16*(k6, k7)
}

__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

template <int NBT>
__global__ void __launch_bounds__(w4::THREADS, 1)
w4g_umma_kernel(const __grid_constant__ W4Maps maps, const W4UmmaArgs p) {
    using namespace w4;
    using C = Cfg<NBT>;
    constexpr int NB = C::NB;            // activation rows per MMA = UMMA N
    constexpr int STAGES = C::STAGES;    // activation-tile ring (L2-resident source, freed by the MMA commit)
    constexpr int WSTAGES = C::WSTAGES;  // weight ring, in copies (HBM source, freed as soon as the dequant warps have read both blocks)
    constexpr int NAB = C::NAB;          // dequantised-A buffers in tensor memory (one k-block = 64 columns each)
    constexpr int NA = NAB;              // barrier pairs for the A buffers
    constexpr int WRING_BYTES = WSTAGES * WB * BLOCK_BYTES;
    constexpr int XATOM_BYTES = NB * 128;     // one 64-k swizzle atom of the activation tile
    constexpr int X_BYTES = 2 * XATOM_BYTES;
    constexpr int D_COL = NAB * 64;
    constexpr int Q_BYTES = NB * TILE_N * 4;  // split-K exchange: [rank slot][rows of this rank][128 channels] fp32
    constexpr int NISS = C::NISS;
    static_assert(D_COL + NISS * NB <= TMEM_COLS, "tensor memory capacity");
    static_assert(STAGES % NISS == 0 && NAB % NISS == 0, "a stage / A buffer must always belong to the same issuer");
    static_assert(WSTAGES % SB == 0 && NAB % (WB * SB) == 0, "a weight stage / A buffer must always belong to the same dequant group");
    extern __shared__ unsigned char smem_unaligned[];
    // the swizzled TMA / UMMA tiles need 1024-byte alignment; the offset is the same in every CTA
    unsigned char* smem = smem_unaligned + ((1024u - (smem_u32(smem_unaligned) & 1023u)) & 1023u);
    // [x stage][atom 0 | atom 1] | [weight stage][nibbles | scales | zeros] | barriers.  Two independent rings: the
    // recycle latency of a stage (consumer release -> producer wake-up -> copy latency) bounds the throughput of
    // a ring, and a weight block can be released ~10x earlier than the activation tile the MMAs still read.
    unsigned char* xs = smem;
    unsigned char* raws = smem + STAGES * X_BYTES;
    float* Q = reinterpret_cast<float*>(raws + WRING_BYTES);  // never aliased: peers write it while this CTA still streams
    uint64_t* bars = reinterpret_cast<uint64_t*>(raws + WRING_BYTES + Q_BYTES);
    uint64_t* full = bars;                   // [STAGES]  activation tile landed
    uint64_t* empty = bars + STAGES;         // [STAGES]  MMAs that read it completed
    uint64_t* wfull = bars + 2 * STAGES;     // [WSTAGES] weight block landed
    uint64_t* wempty = wfull + WSTAGES;      // [WSTAGES] the four dequant warps of its group have read it
    uint64_t* a_ready = wempty + WSTAGES;    // [NA]
    uint64_t* a_free = a_ready + NA;         // [NA]
    uint64_t* d_full = a_free + NA;          // [1]
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(d_full + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    const AbortCtx actx{abort_flag, p.error};

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n0 = blockIdx.x * TILE_N;
    const int grp_idx = blockIdx.y / p.row_blocks;  // which projection of the group
    const CUtensorMap* tm_x = &maps.x[grp_idx];
    const uint8_t* tw = p.tw[grp_idx];
    __half* outp = p.out[grp_idx];
    const int m0 = (blockIdx.y % p.row_blocks) * NB;  // activation row block of this CTA
    const int m_rows = min(NB, p.M - m0);           // valid rows in the block
    const int split = blockIdx.z;
    const int kb0 = split * p.nkb;
    const int nkb = p.nkb;

    if (tid == 0) {
        tma_prefetch_desc(tm_x);
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int s = 0; s < WSTAGES; ++s) {
            mbar_init(&wfull[s], 1);
            mbar_init(&wempty[s], 4 * WB);  // the four warps of each block's dequant group
        }
        for (int a = 0; a < NA; ++a) {
            mbar_init(&a_ready[a], 4);  // the four warps of the group that filled the buffer
            mbar_init(&a_free[a], 1);
        }
        mbar_init(d_full, NISS);
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 1) tmem_alloc(tmem_slot, TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    // Cluster barrier phase 0 = "every CTA of the cluster runs" (precondition of remote shared-memory stores): arrive
    // now, wait only just before the first push.  Phase 1 orders the pushes before the reduction.
    cg::cluster_group cluster = cg::this_cluster();
    const bool clustered = p.splits > 1;
    const int rows_per_rank = NB / p.splits;
    // The two producer threads have work that does not depend on anything; everybody else would only idle until the
    // first weight block lands, so they take the phase-0 wait now, off the tail of the kernel.
    if (clustered) cluster_arrive_relaxed();
    bool waited0 = false;
    if (clustered && !((warp == 0 || warp == XPROD_WARP) && lane == 0)) {
        cluster_wait();
        waited0 = true;
    }

    if (warp == 0) {
        if (lane == 0) {  // weight stream: one bulk copy per WB consecutive blocks (nibbles + scales + zero-points each)
            const int ncopy = (nkb + WB - 1) / WB;
            for (int c = 0; c < ncopy; ++c) {
                const int s = c % WSTAGES;
                if (c >= WSTAGES && !mbar_wait(&wempty[s], ((c / WSTAGES) - 1) & 1, actx, kErrWaitEmpty)) break;
                const uint32_t bytes = (uint32_t)min(WB, nkb - c * WB) * BLOCK_BYTES;
                mbar_expect_tx(&wfull[s], bytes);
                const size_t blk = (size_t)blockIdx.x * p.kbt + kb0 + c * WB;  // tile-major block index
                bulk_load(raws + s * (WB * BLOCK_BYTES), tw + blk * BLOCK_BYTES, bytes, &wfull[s]);
            }
        }
    } else if (warp == XPROD_WARP) {
        if (lane == 0) {  // activation tiles: both 64-k atoms of a block through one 3-D map (k_in, row, k_out)
            // The activations are the only input the preceding kernel of the stream may still be writing: under a
            // programmatic launch the weight stream, the dequantisation and the tensor-memory A buffers above run
            // ahead of this point, in the shadow of that kernel.
            grid_dependency_wait();
            // Only now may the next kernel of the stream start: every kernel of this library releases its successor
            // after its own wait, so a programmatically launched kernel knows that everything before its immediate
            // predecessor has completed.
            grid_launch_dependents();
            for (int i = 0; i < nkb; ++i) {
                const int s = i % STAGES;
                if (i >= STAGES && !mbar_wait(&empty[s], ((i / STAGES) - 1) & 1, actx, kErrWaitEmpty)) break;
                mbar_expect_tx(&full[s], X_BYTES);
                tma_load_3d(xs + s * X_BYTES, tm_x, &full[s], 0, m0, (kb0 + i) * 2);
            }
        }
    } else if (warp == 1 || (NISS == 2 && warp == ISS2_WARP)) {
        if (lane == 0) {
            // Throughput of the A path = (buffers in flight) / (dequantise + barrier hop + MMA + commit + hop), so
            // tensor memory holds six single-block A buffers; every mbarrier hop costs this thread ~150-200 cycles
            // against ~55 per 128x64x16 MMA, so two issuer threads take alternate k-blocks (separate accumulators,
            // summed in the epilogue): one issues while the other waits.
            constexpr uint32_t idesc = make_idesc(TILE_N, NB, /*F32*/ 1, /*F16*/ 0, /*F16*/ 0);
            const int me = warp == 1 ? 0 : 1;
            const uint32_t d_tmem = tmem_base + D_COL + me * NB;
            for (int i = me; i < nkb; i += NISS) {
                const int ab = i % NAB, s = i % STAGES;
                if (!mbar_wait_hot(&a_ready[ab], (i / NAB) & 1, actx, kErrWaitAReady)) break;
                if (!mbar_wait_hot(&full[s], (i / STAGES) & 1, actx, kErrWaitFull)) break;
                tc_fence_after();
                // descriptor of the stage's first atom; the start-address field counts 16-byte units
                const uint64_t bdesc0 = make_sw128_kmajor_desc(smem_u32(xs + s * X_BYTES));
                const uint32_t a_tmem = tmem_base + ab * 64;
#pragma unroll
                for (int j = 0; j < KB / 16; ++j) {
                    const uint64_t bdesc = bdesc0 + (uint64_t)(((j >> 2) * XATOM_BYTES + (j & 3) * 32) >> 4);
                    umma_f16_ts(d_tmem, a_tmem + j * 8, bdesc, idesc, (i == me && j == 0) ? 0u : 1u);
                }
                tc_commit(&empty[s]);
                tc_commit(&a_free[ab]);
            }
            tc_commit(d_full);
        }
    } else if (warp >= 2 && warp < ISS2_WARP) {
        const int q = warp & 3;            // TMEM lane quarter this warp may access
        const int grp = (warp - 2) >> 2;   // dequant group
        const int row = q * 32 + lane;
        const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
        bool ok = true;
        // a group takes whole copies (WB consecutive blocks): one poll of the copy's barrier serves all of them
        for (int i = grp * WB; i < nkb && ok; i += ((i % WB) == WB - 1) ? (SB - 1) * WB + 1 : 1) {
            const int ab = i % NAB, wc = i / WB, ws = wc % WSTAGES;
            const unsigned char* wblk = raws + (ws * WB + (i - wc * WB)) * BLOCK_BYTES;
            if (i == wc * WB) {
                // one lane per warp polls; the others wait at the shuffle
                if (lane == 0) ok = mbar_wait(&wfull[ws], (wc / WSTAGES) & 1, actx, kErrWaitFull);
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) break;
            }
            // this channel's 64 packed bytes: chunk c (32 k) of all 128 channels is one 2 KiB slab, so the
            // threads of a warp read consecutive 16-byte pieces (no bank conflicts, no swizzle)
            const unsigned char* rrow = wblk + row * 16;
            uint4 pk[4];
#pragma unroll
            for (int c = 0; c < 4; ++c) pk[c] = *reinterpret_cast<const uint4*>(rrow + c * 2048);
            const __half sch = reinterpret_cast<const __half*>(wblk + SC_OFF)[row];
            const float z = (float)(wblk + Z_OFF)[row];
            __syncwarp();
            if (lane == 0) mbar_arrive(&wempty[ws]);
            if (i >= NAB) {
                if (lane == 0) ok = mbar_wait(&a_free[ab], ((i / NAB) - 1) & 1, actx, kErrWaitAFree);
                ok = __shfl_sync(0xffffffffu, ok, 0);
                if (!ok) break;
            }
            tc_fence_after();
            const __half2 sc2 = __half2half2(sch), zlo2 = __float2half2_rn(1024.0f + z), zhi2 = __float2half2_rn(-(64.0f + z));
            const uint32_t sc = *reinterpret_cast<const uint32_t*>(&sc2), zlo = *reinterpret_cast<const uint32_t*>(&zlo2),
                           zhi = *reinterpret_cast<const uint32_t*>(&zhi2);
            const uint32_t a_addr = lane_addr + ab * 64;
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                uint32_t v[16];
                dequant_word(pk[c].x, zlo, zhi, sc, v + 0);
                dequant_word(pk[c].y, zlo, zhi, sc, v + 4);
                dequant_word(pk[c].z, zlo, zhi, sc, v + 8);
                dequant_word(pk[c].w, zlo, zhi, sc, v + 12);
                tmem_st16(a_addr + c * 16, v);
            }
            tc_wait_st();
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&a_ready[ab]);
        }
        // ---- accumulator tile -> slot [this rank] of the owning rank's exchange buffer; groups 0 and 1 split the 64 columns
        if (ok && lane == 0) ok = mbar_wait(d_full, 0, actx, kErrWaitDFull);
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (grp < 2) {
            if (ok) {
                tc_fence_after();
                constexpr int CPG = NB / 2;  // accumulator columns (activation rows) per reading group
#pragma unroll
                for (int c = 0; c < CPG / 16; ++c) {
                    uint32_t v[16], v2[16];
                    const int col0 = grp * CPG + c * 16;
                    tmem_ld16(lane_addr + D_COL + col0, v);
                    if (NISS == 2 && nkb > 1) tmem_ld16(lane_addr + D_COL + NB + col0, v2);  // second issuer's accumulator (unused when it had no work)
                    tc_wait_ld();
                    if (!clustered) {
                        // No split-K: nothing to exchange, so the accumulator goes straight to global memory (fp16
                        // rounding, epilogue, 2-byte stores: the 32 lanes of a warp cover 64 contiguous bytes of a row).
                        // The activations arrived after the grid-dependency wait of the producer thread, so the
                        // preceding kernel has completed; the residual it may have written is read here.
                        const int nn = n0 + row;
                        grid_dependency_wait();  // returns at once (see above); keeps the ordering explicit
                        if (nn < p.Nout) {
#pragma unroll
                            for (int e = 0; e < 16; ++e) {
                                const int m = col0 + e;
                                if (m >= m_rows) break;
                                const float a = __uint_as_float(v[e]) + ((NISS == 2 && nkb > 1) ? __uint_as_float(v2[e]) : 0.f);
                                const size_t o = (size_t)(m0 + m) * p.Nout + nn;
                                float y = __half2float(__float2half_rn(a));
                                if (p.epilogue == RWKV7_EPI_RELU2) {
                                    y = fmaxf(y, 0.f);
                                    y *= y;
                                } else if (p.epilogue == RWKV7_EPI_ADD) {
                                    y += __half2float(p.residual[o]);
                                }
                                outp[o] = __float2half_rn(y);
                            }
                        }
                    } else if (col0 < m_rows) {
                        // 16 consecutive rows never straddle two ranks (rows_per_rank is 8, 16, 32 or 64)
#pragma unroll
                        for (int h8 = 0; h8 < 2; ++h8) {
                            const int m = col0 + h8 * 8;
                            const int dst = m / rows_per_rank;
                            float* q = (clustered ? cluster.map_shared_rank(Q, dst) : Q) +
                                       ((size_t)split * rows_per_rank + (m - dst * rows_per_rank)) * TILE_N + row;
#pragma unroll
                            for (int e = 0; e < 8; ++e)
                                q[e * TILE_N] = __uint_as_float(v[h8 * 8 + e]) + ((NISS == 2 && nkb > 1) ? __uint_as_float(v2[h8 * 8 + e]) : 0.f);
                        }
                    }
                }
                tc_fence_before();
            }
        }
    }

    // ---- split-K reduction (fixed rank order) + epilogue, from this CTA's own shared memory
    if (clustered) {
        if (!waited0) cluster_wait();
        cluster_arrive_release();
        cluster_wait();
    } else {
        __syncthreads();
    }
    const bool aborted = (*abort_flag != 0);
    grid_dependency_wait();  // residual reads and output writes are ordered after the preceding kernel (returns at once here:
                             // the accumulators already depend on the activations)
    if (!aborted && clustered) {
        // Each thread owns one channel pair (n, n+1) and walks the rows of this rank's share in steps of
        // THREADS/64, four rows per batch: float2 loads of the rank slots in fixed order, fp16 rounding, epilogue,
        // one 4-byte store; 64 consecutive threads cover one 256-byte output row segment.
        const int m_begin = split * rows_per_rank;
        const int m_end = min(m_rows, m_begin + rows_per_rank);
        const int n = (tid & 63) * 2;
        const bool n_ok = n0 + n < p.Nout;
        const bool pair = (n0 + n + 1 < p.Nout) && ((p.Nout & 1) == 0);
        constexpr int RSTEP = (THREADS - 64) / 64;  // the last two warps (second issuer, x producer) sit the epilogue out
        const float* Q0 = Q + n - (size_t)m_begin * TILE_N;  // slot r, global row m: Q0[(r * rows_per_rank + m) * TILE_N]
        const int slot = rows_per_rank * TILE_N;
        for (int mb = m_begin + (tid >> 6); mb < m_end && n_ok && tid < RSTEP * 64; mb += 4 * RSTEP) {
            float2 acc[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int m = mb + u * RSTEP;
                acc[u] = make_float2(0.f, 0.f);
                if (m < m_end) {
                    const float* q = Q0 + m * TILE_N;
                    acc[u] = *reinterpret_cast<const float2*>(q);
                    if (p.splits == 4) {  // the common plan: all four loads in flight, summed in rank order
                        const float2 v1 = *reinterpret_cast<const float2*>(q + slot);
                        const float2 v2 = *reinterpret_cast<const float2*>(q + 2 * slot);
                        const float2 v3 = *reinterpret_cast<const float2*>(q + 3 * slot);
                        acc[u].x = ((acc[u].x + v1.x) + v2.x) + v3.x;
                        acc[u].y = ((acc[u].y + v1.y) + v2.y) + v3.y;
                    } else {
                        for (int r = 1; r < p.splits; ++r) {
                            const float2 v = *reinterpret_cast<const float2*>(q + r * slot);
                            acc[u].x += v.x; acc[u].y += v.y;
                        }
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int m = mb + u * RSTEP;
                if (m >= m_end) continue;
                const size_t o = (size_t)(m0 + m) * p.Nout + n0 + n;
                float y0 = __half2float(__float2half_rn(acc[u].x)), y1 = __half2float(__float2half_rn(acc[u].y));
                if (p.epilogue == RWKV7_EPI_RELU2) {
                    y0 = fmaxf(y0, 0.f); y0 *= y0;
                    y1 = fmaxf(y1, 0.f); y1 *= y1;
                } else if (p.epilogue == RWKV7_EPI_ADD) {
                    if (pair) {
                        const float2 rr = __half22float2(*reinterpret_cast<const __half2*>(p.residual + o));
                        y0 += rr.x;
                        y1 += rr.y;
                    } else {
                        y0 += __half2float(p.residual[o]);
                        if (n0 + n + 1 < p.Nout) y1 += __half2float(p.residual[o + 1]);
                    }
                }
                if (pair) {
                    *reinterpret_cast<__half2*>(outp + o) = __floats2half2_rn(y0, y1);
                } else {
                    outp[o] = __float2half_rn(y0);
                    if (n0 + n + 1 < p.Nout) outp[o + 1] = __float2half_rn(y1);
                }
            }
        }
    }
    __syncthreads();  // nothing remote is touched after the barrier above, so the CTA may leave on its own
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem_base, TMEM_COLS);
    }
}


// ================================================================ 64 activation rows: self-issuing dequant groups
// The kernel above hands every dequantised block from a dequant group to a separate MMA-issuer warp and back (two
// mbarrier hops of 150-200 cycles each per block, two polling issuer threads, six A buffers to cover the round trip)
// and spends about as many warp instructions on that plumbing as on the dequantisation itself.  This variant for
// batches up to 64 rows removes the hand-off:
//
//   * four dequant groups (four warps each = the 128 tensor-memory lanes); group g owns k-blocks g, g+4, ... of the
//     CTA's k range, ONE A buffer (64 columns) and ONE accumulator (64 columns) in tensor memory;
//   * a group loads its block from the weight ring, expands it into 64 registers per thread, waits until the MMAs of
//     its previous block have completed (they were issued a whole block-time earlier), stores the registers into its
//     A buffer, meets at a 128-thread named barrier and one of its threads issues the eight MMAs itself; the commit of
//     those MMAs releases both the A buffer and the activation stage;
//   * the four accumulators are summed in the epilogue (fixed order), where group g takes activation rows
//     16 g .. 16 g + 15 of all of them.
//
// Rings: weights 8 stages of one block (two per group, released as soon as the block is in registers), activations 8
// stages (two per group).  A stage always belongs to the same group (ring lengths are multiples of the group count),
// so every waiter sees every phase of the barriers it waits on.  The split-K exchange buffer aliases the weight ring:
// a CTA announces the end of its main loop with a cluster-barrier arrive and peers wait for that phase before they
// push, so nobody writes into a ring that is still being read.
namespace w4b {
using namespace w4;
constexpr int G = 4;                      // dequant groups
constexpr int NB = 64;                    // activation rows = UMMA N
constexpr int WST = 8, XST = 8;           // ring lengths (stages)
constexpr int XATOM = NB * 128, X_BYTES = 2 * XATOM;
constexpr int NTHREADS = 64 + G * 128;    // warp 0: weight producer, warp 1: activation producer + TMEM owner, then the groups
constexpr int A_COL = 0, D_COL = G * 64;  // tensor memory: A buffers | accumulators
constexpr int Q_BYTES = NB * TILE_N * 4;
constexpr int WRING_BYTES = WST * BLOCK_BYTES;
static_assert(WST % G == 0 && XST % G == 0, "a stage must always belong to the same group");
static_assert(Q_BYTES <= WRING_BYTES, "the exchange buffer aliases the weight ring");
static_assert(D_COL + G * NB <= TMEM_COLS, "tensor memory capacity");
constexpr size_t SMEM = (size_t)XST * X_BYTES + WRING_BYTES + (2 * XST + 2 * WST + 1) * 8 + 16 + 1024;
}  // namespace w4b

// Named barrier of one dequant group that also agrees on whether every thread is still healthy.
__device__ __forceinline__ bool group_barrier_and(int id, bool ok) {
    uint32_t r;
    asm volatile(
        "{\n\t.reg .pred p, q;\n\t"
        "setp.ne.b32 p, %1, 0;\n\t"
        "barrier.cta.red.and.pred q, %2, 128, p;\n\t"
        "selp.b32 %0, 1, 0, q;\n\t}"
        : "=r"(r) : "r"((uint32_t)ok), "r"(id) : "memory");
    return r != 0;
}

__global__ void __launch_bounds__(w4b::NTHREADS, 1)
w4g_umma64_kernel(const __grid_constant__ W4Maps maps, const W4UmmaArgs p) {
    using namespace w4b;
    extern __shared__ unsigned char smem_unaligned[];
    unsigned char* smem = smem_unaligned + ((1024u - (smem_u32(smem_unaligned) & 1023u)) & 1023u);
    unsigned char* xs = smem;                                   // [XST][atom 0 | atom 1]
    unsigned char* raws = smem + XST * X_BYTES;                 // [WST][nibbles | scales | zeros]
    float* Q = reinterpret_cast<float*>(raws);                  // split-K exchange (after the main loop)
    uint64_t* bars = reinterpret_cast<uint64_t*>(raws + WRING_BYTES);
    uint64_t* full = bars;               // [XST] activation tile landed
    uint64_t* done = bars + XST;         // [XST] the MMAs that read the tile (and the group's A buffer) completed
    uint64_t* wfull = done + XST;        // [WST] weight block landed
    uint64_t* wempty = wfull + WST;      // [WST] the group's four warps hold the block in registers
    uint64_t* d_full = wempty + WST;     // [1]   every group's last MMA completed
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(d_full + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    const AbortCtx actx{abort_flag, p.error};

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int n0 = blockIdx.x * TILE_N;
    const int grp_idx = blockIdx.y / p.row_blocks;
    const CUtensorMap* tm_x = &maps.x[grp_idx];
    const uint8_t* tw = p.tw[grp_idx];
    __half* outp = p.out[grp_idx];
    const int m0 = (blockIdx.y % p.row_blocks) * NB;
    const int m_rows = min(NB, p.M - m0);
    const int split = blockIdx.z;
    const int kb0 = split * p.nkb;
    const int nkb = p.nkb;
    const bool clustered = p.splits > 1;
    const int rows_per_rank = NB / p.splits;
    const uint8_t* wsrc = tw + ((size_t)blockIdx.x * p.kbt + kb0) * BLOCK_BYTES;

    if (tid == 0) {
        for (int s = 0; s < XST; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&done[s], 1);
        }
        for (int s = 0; s < WST; ++s) {
            mbar_init(&wfull[s], 1);
            mbar_init(&wempty[s], 4);
        }
        mbar_init(d_full, G);
        *abort_flag = 0;
        mbar_fence_init();
        // the first ring fill does not depend on anything: start it before the tensor-memory allocation
        const int pre = min(WST, nkb);
        for (int c = 0; c < pre; ++c) {
            mbar_expect_tx(&wfull[c], BLOCK_BYTES);
            bulk_load(raws + c * BLOCK_BYTES, wsrc + (size_t)c * BLOCK_BYTES, BLOCK_BYTES, &wfull[c]);
        }
    }
    if (warp == 1) {
        if (lane == 0) tma_prefetch_desc(tm_x);
        __syncwarp();
        tmem_alloc(tmem_slot, TMEM_COLS);
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;
    cg::cluster_group cluster = cg::this_cluster();

    if (warp == 0) {
        if (lane == 0) {  // weight stream, one block per copy
            for (int c = WST; c < nkb; ++c) {
                const int s = c % WST;
                if (!mbar_wait(&wempty[s], ((c / WST) - 1) & 1, actx, kErrWaitEmpty)) break;
                mbar_expect_tx(&wfull[s], BLOCK_BYTES);
                bulk_load(raws + s * BLOCK_BYTES, wsrc + (size_t)c * BLOCK_BYTES, BLOCK_BYTES, &wfull[s]);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {  // activation tiles: the only input the preceding kernel of the stream may still be writing
            grid_dependency_wait();
            grid_launch_dependents();
            for (int i = 0; i < nkb; ++i) {
                const int s = i % XST;
                if (i >= XST && !mbar_wait(&done[s], ((i / XST) - 1) & 1, actx, kErrWaitEmpty)) break;
                mbar_expect_tx(&full[s], X_BYTES);
                tma_load_3d(xs + s * X_BYTES, tm_x, &full[s], 0, m0, (kb0 + i) * 2);
            }
        }
    } else {
        const int q = warp & 3;                // TMEM lane quarter this warp may access
        const int g = (warp - 2) >> 2;         // dequant group
        const int wig = (warp - 2) & 3;        // warp within the group
        const int row = q * 32 + lane;
        const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
        const uint32_t a_addr = lane_addr + A_COL + g * 64;
        const uint32_t a_tmem = tmem_base + A_COL + g * 64;
        const uint32_t d_tmem = tmem_base + D_COL + g * NB;
        constexpr uint32_t idesc = make_idesc(TILE_N, NB, /*F32*/ 1, /*F16*/ 0, /*F16*/ 0);
        bool ok = true;
        for (int i = g; i < nkb; i += G) {
            const int ws = i % WST, xst = i % XST;
            const unsigned char* wblk = raws + ws * BLOCK_BYTES;
            if (lane == 0 && ok) ok = mbar_wait(&wfull[ws], (i / WST) & 1, actx, kErrWaitFull);
            ok = __shfl_sync(0xffffffffu, ok, 0);
            uint4 pk[4];
            uint32_t sc = 0, zlo = 0, zhi = 0;
            if (ok) {
                const unsigned char* rrow = wblk + row * 16;
#pragma unroll
                for (int c = 0; c < 4; ++c) pk[c] = *reinterpret_cast<const uint4*>(rrow + c * 2048);
                const uint32_t s16 = reinterpret_cast<const unsigned short*>(wblk + SC_OFF)[row];
                const uint32_t z = (wblk + Z_OFF)[row];
                sc = s16 * 0x00010001u;               // (scale, scale)
                zlo = z * 0x00010001u + 0x64006400u;  // 1024 + z as fp16: 0x6400 | z
                zhi = z * 0x00100010u + 0xD400D400u;  // -(64 + z) as fp16: 0xD400 | (z << 4)
            }
            __syncwarp();
            if (lane == 0 && ok) mbar_arrive(&wempty[ws]);
            uint32_t v[4][16];
            if (ok) {
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    dequant_word(pk[c].x, zlo, zhi, sc, v[c] + 0);
                    dequant_word(pk[c].y, zlo, zhi, sc, v[c] + 4);
                    dequant_word(pk[c].z, zlo, zhi, sc, v[c] + 8);
                    dequant_word(pk[c].w, zlo, zhi, sc, v[c] + 12);
                }
            }
            if (i >= G && ok) {  // the MMAs of this group's previous block (A buffer, stage xst - G) completed
                const int ps = (i - G) % XST;
                if (lane == 0) ok = mbar_wait(&done[ps], ((i - G) / XST) & 1, actx, kErrWaitAFree);
                ok = __shfl_sync(0xffffffffu, ok, 0);
            }
            if (ok) {
                tc_fence_after();
#pragma unroll
                for (int c = 0; c < 4; ++c) tmem_st16(a_addr + c * 16, v[c]);
                tc_wait_st();
                tc_fence_before();
            }
            ok = group_barrier_and(1 + g, ok);
            if (!ok) break;
            if (wig == ((i / G) & 3)) {  // the issuing warp rotates
                if (lane == 0) {
                    ok = mbar_wait(&full[xst], (i / XST) & 1, actx, kErrWaitFull);
                    if (ok) {
                        tc_fence_after();
                        const uint64_t bdesc0 = make_sw128_kmajor_desc(smem_u32(xs + xst * X_BYTES));
#pragma unroll
                        for (int j = 0; j < KB / 16; ++j) {
                            const uint64_t bdesc = bdesc0 + (uint64_t)(((j >> 2) * XATOM + (j & 3) * 32) >> 4);
                            umma_f16_ts(d_tmem, a_tmem + j * 8, bdesc, idesc, (i == g && j == 0) ? 0u : 1u);
                        }
                        tc_commit(&done[xst]);
                        if (i + G >= nkb) tc_commit(d_full);
                    }
                }
                ok = __shfl_sync(0xffffffffu, ok, 0);
            }
        }
        // groups that issued nothing (fewer blocks than groups) or gave up still owe their arrival
        ok = group_barrier_and(1 + g, ok);
        if (wig == 0 && lane == 0 && (g >= nkb || !ok)) mbar_arrive(d_full);

        // ---- the main loop of this CTA has released the weight ring: peers may push into the exchange buffer
        if (clustered) cluster_arrive_release();
        if (ok && lane == 0) ok = mbar_wait(d_full, 0, actx, kErrWaitDFull);
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (clustered) cluster_wait();
        if (ok && *abort_flag == 0) {
            tc_fence_after();
            const int nacc = min(G, nkb);
            const int col0 = g * 16;  // activation rows of this group in every accumulator
            uint32_t v[16], t[16];
            tmem_ld16(lane_addr + D_COL + col0, v);
            tc_wait_ld();
            for (int a = 1; a < nacc; ++a) {
                tmem_ld16(lane_addr + D_COL + a * NB + col0, t);
                tc_wait_ld();
#pragma unroll
                for (int e = 0; e < 16; ++e) v[e] = __float_as_uint(__uint_as_float(v[e]) + __uint_as_float(t[e]));
            }
            if (!clustered) {
                const int nn = n0 + row;
                grid_dependency_wait();  // returns at once (the accumulators already depend on the activations)
                if (nn < p.Nout) {
#pragma unroll
                    for (int e = 0; e < 16; ++e) {
                        const int m = col0 + e;
                        if (m >= m_rows) break;
                        const size_t o = (size_t)(m0 + m) * p.Nout + nn;
                        float y = __half2float(__float2half_rn(__uint_as_float(v[e])));
                        if (p.epilogue == RWKV7_EPI_RELU2) {
                            y = fmaxf(y, 0.f);
                            y *= y;
                        } else if (p.epilogue == RWKV7_EPI_ADD) {
                            y += __half2float(p.residual[o]);
                        }
                        outp[o] = __float2half_rn(y);
                    }
                }
            } else if (col0 < m_rows) {
                // 8 consecutive rows never straddle two ranks (rows_per_rank is 8, 16 or 32)
#pragma unroll
                for (int h8 = 0; h8 < 2; ++h8) {
                    const int m = col0 + h8 * 8;
                    const int dst = m / rows_per_rank;
                    float* qd = cluster.map_shared_rank(Q, dst) + ((size_t)split * rows_per_rank + (m - dst * rows_per_rank)) * TILE_N + row;
#pragma unroll
                    for (int e = 0; e < 8; ++e) qd[e * TILE_N] = __uint_as_float(v[h8 * 8 + e]);
                }
            }
            tc_fence_before();
        }
    }
    if (warp < 2 && clustered) {  // the producer warps take part in the same cluster-barrier phases
        cluster_arrive_release();
        cluster_wait();
    }

    // ---- split-K reduction (fixed rank order) + epilogue, from this CTA's own shared memory
    if (clustered) {
        cluster_arrive_release();
        cluster_wait();
    } else {
        __syncthreads();
    }
    const bool aborted = (*abort_flag != 0);
    grid_dependency_wait();
    if (!aborted && clustered) {
        const int m_begin = split * rows_per_rank;
        const int m_end = min(m_rows, m_begin + rows_per_rank);
        const int n = (tid & 63) * 2;
        const bool n_ok = n0 + n < p.Nout;
        const bool pair = (n0 + n + 1 < p.Nout) && ((p.Nout & 1) == 0);
        constexpr int RSTEP = NTHREADS / 64;
        const float* Q0 = Q + n - (size_t)m_begin * TILE_N;
        const int slot = rows_per_rank * TILE_N;
        for (int m = m_begin + (tid >> 6); m < m_end && n_ok; m += RSTEP) {
            const float* qq = Q0 + m * TILE_N;
            float2 acc = *reinterpret_cast<const float2*>(qq);
            for (int r = 1; r < p.splits; ++r) {
                const float2 t2 = *reinterpret_cast<const float2*>(qq + r * slot);
                acc.x += t2.x;
                acc.y += t2.y;
            }
            const size_t o = (size_t)(m0 + m) * p.Nout + n0 + n;
            float y0 = __half2float(__float2half_rn(acc.x)), y1 = __half2float(__float2half_rn(acc.y));
            if (p.epilogue == RWKV7_EPI_RELU2) {
                y0 = fmaxf(y0, 0.f); y0 *= y0;
                y1 = fmaxf(y1, 0.f); y1 *= y1;
            } else if (p.epilogue == RWKV7_EPI_ADD) {
                if (pair) {
                    const float2 rr = __half22float2(*reinterpret_cast<const __half2*>(p.residual + o));
                    y0 += rr.x;
                    y1 += rr.y;
                } else {
                    y0 += __half2float(p.residual[o]);
                    if (n0 + n + 1 < p.Nout) y1 += __half2float(p.residual[o + 1]);
                }
            }
            if (pair) {
                *reinterpret_cast<__half2*>(outp + o) = __floats2half2_rn(y0, y1);
            } else {
                outp[o] = __float2half_rn(y0);
                if (n0 + n + 1 < p.Nout) outp[o + 1] = __float2half_rn(y1);
            }
        }
    }
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
                                  uint8_t* __restrict__ tiled, int K, int Nout, int group, long long total_words) {
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
    uint8_t* block = tiled + blk * w4::BLOCK_BYTES;
    reinterpret_cast<uint32_t*>(block)[widx & 2047] = out;
    if (c == 0 && j == 0) {
        const long long gi = n * (K / group) + (b * 128) / group;
        reinterpret_cast<T*>(block + w4::SC_OFF)[r] = (n < Nout) ? scales[gi] : from_f<T>(0.f);
        (block + w4::Z_OFF)[r] = (n < Nout && zeros) ? zeros[gi] : (uint8_t)8;
    }
}

// Tiled buffers written by rwkv7_w4g_repack and not yet read by a projection.  The projection kernel streams the
// weights BEFORE its grid-dependency wait, so the first projection after a repack is launched with full stream
// ordering (it may directly follow the repack kernel); every later one is ordered behind that launch.
static std::mutex g_fresh_mu;
static std::unordered_set<const void*> g_fresh_tiled;

static void mark_tiled_fresh(const void* tiled) {
    std::lock_guard<std::mutex> lk(g_fresh_mu);
    g_fresh_tiled.insert(tiled);
}
static bool take_tiled_fresh(const void* tiled) {
    std::lock_guard<std::mutex> lk(g_fresh_mu);
    return g_fresh_tiled.erase(tiled) != 0;
}

// G projections of equal shape (their own activations, weights and outputs) in one launch.
int launch_w4g_umma_tiled(const void* const* xs, const uint8_t* const* tws, const void* residual, void* const* outs, int G,
                          int M, int K, int Nout, int epilogue, cudaStream_t st) {
    using namespace w4;
    RWKV7_REQUIRE(G >= 1 && G <= kW4MaxGroup, RWKV7_ERR_UNSUPPORTED, "w4g_gemv_tiled: 1..%d projections per launch (got %d)", kW4MaxGroup, G);
    const int NB = M > 64 ? 128 : 64;          // activation rows per pass over the weights
    RWKV7_REQUIRE(M >= 1 && (long long)G * ((M + NB - 1) / NB) <= 65535, RWKV7_ERR_UNSUPPORTED, "w4g_gemv_tiled: M out of range (got %d)", M);
    const int row_blocks = (M + NB - 1) / NB;
    RWKV7_REQUIRE(K % KB == 0, RWKV7_ERR_UNSUPPORTED, "w4g_gemv_tiled: K must be a multiple of %d (got %d)", KB, K);
    const int tiles = (Nout + TILE_N - 1) / TILE_N;
    const int total_kb = K / KB;
    int splits = 1;
    for (int s = 8; s >= 2; s >>= 1) {
        if (tiles * row_blocks * G * s <= 160 && total_kb % s == 0 && (total_kb / s) >= 4) {
            splits = s;
            break;
        }
    }
    const int nkb = total_kb / splits;
    W4Maps maps;
    W4UmmaArgs a{};
    bool fresh = false;
    for (int g = 0; g < G; ++g) {
        if (int e = make_tmap_x3d(&maps.x[g], xs[g], M, K, NB)) return e;
        a.tw[g] = tws[g];
        a.out[g] = reinterpret_cast<__half*>(outs[g]);
        fresh |= take_tiled_fresh(tws[g]);
    }
    for (int g = G; g < kW4MaxGroup; ++g) maps.x[g] = maps.x[0];
    a.residual = reinterpret_cast<const __half*>(residual);
    a.M = M; a.K = K; a.Nout = Nout; a.epilogue = epilogue; a.nkb = nkb; a.kbt = total_kb; a.splits = splits;
    a.row_blocks = row_blocks;
    a.error = kernel_error_word();
    RWKV7_REQUIRE(a.error != nullptr, RWKV7_ERR_CUDA, "w4g_gemv_tiled: cannot resolve the device error word");
    // up to 64 rows: the self-issuing dequant-group kernel; RWKV7_B200_W4G_HANDOFF=1 keeps the hand-off kernel for A/B timing
    static const bool handoff = [] {
        const char* v = getenv("RWKV7_B200_W4G_HANDOFF");
        return v && *v && *v != '0';
    }();
    const bool v64 = NB == 64 && !handoff;
    const size_t smem = v64 ? w4b::SMEM : NB == 128 ? smem_bytes<128>() : smem_bytes<64>();
    cudaError_t e = v64 ? cudaFuncSetAttribute(w4g_umma64_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)
        : NB == 128 ? cudaFuncSetAttribute(w4g_umma_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)
                    : cudaFuncSetAttribute(w4g_umma_kernel<64>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    RWKV7_REQUIRE(e == cudaSuccess, RWKV7_ERR_CUDA, "w4g_gemv_tiled: %s", cudaGetErrorString(e));
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(tiles, row_blocks * G, splits);
    cfg.blockDim = dim3(v64 ? w4b::NTHREADS : w4::THREADS);
    cfg.dynamicSmemBytes = smem;
    cfg.stream = st;
    cudaLaunchAttribute attr[2];
    attr[0].id = cudaLaunchAttributeClusterDimension;
    attr[0].val.clusterDim.x = 1;
    attr[0].val.clusterDim.y = 1;
    attr[0].val.clusterDim.z = splits;
    // programmatic dependent launch: start under the tail of the preceding kernel (see grid_dependency_wait in the kernel)
    attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[1].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = (programmatic_launch_enabled() && !fresh) ? 2 : 1;
    e = v64 ? cudaLaunchKernelEx(&cfg, w4g_umma64_kernel, maps, a)
        : NB == 128 ? cudaLaunchKernelEx(&cfg, w4g_umma_kernel<128>, maps, a) : cudaLaunchKernelEx(&cfg, w4g_umma_kernel<64>, maps, a);
    RWKV7_REQUIRE(e == cudaSuccess, RWKV7_ERR_CUDA, "w4g_gemv_tiled launch: %s", cudaGetErrorString(e));
    return RWKV7_OK;
}

}  // namespace rwkv7

using namespace rwkv7;

extern "C" int64_t rwkv7_w4g_tiled_bytes(int K, int Nout) {
    if (K <= 0 || Nout <= 0 || K % 128) return 0;
    const int64_t tiles = (Nout + 127) / 128, kbt = K / 128;
    return tiles * kbt * w4::BLOCK_BYTES;
}

extern "C" int rwkv7_w4g_repack(const uint8_t* packed, const void* scales, const uint8_t* zeros, uint8_t* tiled, int K,
                                int Nout, int group, int dtype, void* stream) {
    RWKV7_REQUIRE(K > 0 && Nout > 0 && K % 128 == 0, RWKV7_ERR_UNSUPPORTED, "w4g_repack: K must be a positive multiple of 128");
    RWKV7_REQUIRE(group > 0 && group % 128 == 0 && K % group == 0, RWKV7_ERR_UNSUPPORTED,
                  "w4g_repack: group must be a multiple of 128 dividing K (group=%d K=%d)", group, K);
    RWKV7_REQUIRE(packed && scales && tiled, RWKV7_ERR_INVALID, "w4g_repack: null pointer");
    RWKV7_REQUIRE(dtype == RWKV7_F16, RWKV7_ERR_UNSUPPORTED, "w4g_repack: the tiled format holds fp16 scales");
    RWKV7_REQUIRE(aligned(packed, 4) && aligned(tiled, 16), RWKV7_ERR_ALIGN, "w4g_repack: unaligned pointer");
    const long long tiles = (Nout + 127) / 128;
    const long long words = tiles * (K / 128) * 2048;
    w4g_repack_kernel<__half><<<(unsigned)((words + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(
        packed, reinterpret_cast<const __half*>(scales), zeros, tiled, K, Nout, group, words);
    mark_tiled_fresh(tiled);
    return check_launch("w4g_repack_kernel");
}

extern "C" int rwkv7_w4g_gemv_tiled(const void* x, const uint8_t* tiled, const void* residual, void* out, int M, int K,
                                    int Nout, int epilogue, int dtype, void* stream) {
    RWKV7_REQUIRE(x && tiled && out, RWKV7_ERR_INVALID, "w4g_gemv_tiled: null pointer");
    RWKV7_REQUIRE(dtype == RWKV7_F16, RWKV7_ERR_UNSUPPORTED, "w4g_gemv_tiled: fp16 activations only");
    RWKV7_REQUIRE(epilogue >= 0 && epilogue <= 2, RWKV7_ERR_INVALID, "w4g_gemv_tiled: bad epilogue code %d", epilogue);
    RWKV7_REQUIRE(epilogue != RWKV7_EPI_ADD || residual, RWKV7_ERR_INVALID, "w4g_gemv_tiled: residual is required for the add epilogue");
    RWKV7_REQUIRE(aligned(x, 16) && aligned(tiled, 16), RWKV7_ERR_ALIGN, "w4g_gemv_tiled: pointers must be 16-byte aligned");
    return launch_w4g_umma_tiled(&x, &tiled, residual, &out, 1, M, K, Nout, epilogue, static_cast<cudaStream_t>(stream));
}

extern "C" int rwkv7_w4g_gemv_tiled_group(const void* const* xs, const uint8_t* const* tiled, void* const* outs, int G, int M,
                                          int K, int Nout, int epilogue, int dtype, void* stream) {
    RWKV7_REQUIRE(xs && tiled && outs, RWKV7_ERR_INVALID, "w4g_gemv_tiled_group: null pointer");
    RWKV7_REQUIRE(G >= 1 && G <= kW4MaxGroup, RWKV7_ERR_UNSUPPORTED, "w4g_gemv_tiled_group: 1..%d projections (got %d)", kW4MaxGroup, G);
    RWKV7_REQUIRE(dtype == RWKV7_F16, RWKV7_ERR_UNSUPPORTED, "w4g_gemv_tiled_group: fp16 activations only");
    RWKV7_REQUIRE(epilogue == RWKV7_EPI_NONE || epilogue == RWKV7_EPI_RELU2, RWKV7_ERR_INVALID,
                  "w4g_gemv_tiled_group: epilogue must be none or relu^2 (got %d)", epilogue);
    for (int g = 0; g < G; ++g) {
        RWKV7_REQUIRE(xs[g] && tiled[g] && outs[g], RWKV7_ERR_INVALID, "w4g_gemv_tiled_group: null pointer in projection %d", g);
        RWKV7_REQUIRE(aligned(xs[g], 16) && aligned(tiled[g], 16), RWKV7_ERR_ALIGN, "w4g_gemv_tiled_group: pointers must be 16-byte aligned");
    }
    return launch_w4g_umma_tiled(xs, tiled, nullptr, outs, G, M, K, Nout, epilogue, static_cast<cudaStream_t>(stream));
}
