// Decode-time int4 group-wise projection on the 5th-generation tensor cores (any row count; one pass over the
// weights per 64 activation rows up to 64 rows, per 128 rows above).
//
//   out[M, Nout] = epilogue( x[M, K] . W[Nout, K]^T ),  W = round_f16((nibble - zero) * scale)
//
// At these batch sizes a CUDA-core GEMV is FMA-bound (M*K*Nout MACs) while the weights still have to stream from
// HBM exactly once, so the contraction goes to tcgen05.mma:
//
//   * the weights are read from a TILED copy of the reference's [Nout, K/2] array (rwkv7_w4g_repack, built once at
//     load): one 8.5 KiB block per [128 channels x 128 k] tile (nibbles, then the tile's scales and zero-points),
//     blocks of a channel tile consecutive in memory, so every CTA streams one contiguous region, one bulk copy per
//     block -- row-strided 64-byte pieces of the row-major array reach under 1 TB/s on HBM3e, contiguous blocks run
//     at copy speed;
//   * dequant warps (thread = output channel) read their 64 packed bytes, expand them to 128 fp16 values in
//     registers (lop3 magic-number conversion, exact (q - zero), one fp16 rounding for the scale product = the
//     reference's materialised weight) and write them with tcgen05.st straight into TENSOR MEMORY as the A operand:
//     the 4x larger fp16 tile never touches shared memory;
//   * the activation tile [NB rows x 128 k] arrives by TMA (128-byte swizzle) and is the B operand from shared
//     memory; D [128 x NB] fp32 accumulates in tensor memory;
//   * split-K runs as a thread-block cluster along z; every CTA PUSHES the rows of its partial tile that belong to
//     rank k straight from the accumulator registers into slot [own rank] of rank k's shared memory (remote stores
//     are fire-and-forget, remote loads would cost a round trip), one cluster barrier, then each rank sums its slots
//     in fixed rank order (deterministic, no scratch buffer, no atomics), applies the relu^2 / residual epilogue and
//     stores fp16 results coalesced.
//
// What shapes the pipeline (clock64 traces and micro-benchmarks on this part):
//
//   * a 128 x N x 16 MMA occupies the tensor pipe for about 64 cycles for every N up to 128, so at 64 rows a
//     [128 x 128] weight block costs 512 cycles: 17 bytes of int4 weights per clock and SM, about 4.2 TB/s over 128
//     CTAs.  That is the ceiling of this kernel at batch 64, below the HBM roofline; 128 rows per pass pay the same
//     cycles for twice the rows;
//   * a tcgen05.mma issue holds its thread while the pipe digests the previous one, so the eight MMAs of a block
//     cost the issuing thread those 512 cycles whoever it is: dedicated issuer warps, and two of them on alternate
//     blocks (own accumulators, summed in the epilogue) so that one's barrier / commit overhead hides under the
//     other's MMAs.  The issue loop runs under elect.sync with a warp-uniform warp index (descriptors in uniform
//     registers);
//   * polling an mbarrier whose phase completed long ago cost 175-350 cycles as "try_wait with a suspend hint by one
//     lane, then a shuffle" and 20 as test_wait: every wait tests first (mbar_wait in umma.cuh);
//   * the "A buffer ready" hand-off from a dequant group to its issuer is a hardware named barrier (bar.arrive by
//     the group's 128 threads, bar.sync by the issuer warp: tens of cycles) instead of an mbarrier, whose completion
//     takes about 175 cycles to become visible to a waiter.
//
// Warps: 0 weight-stream producer, 1 activation producer + tensor-memory owner, 2..1+NISS issuers, then three dequant
// groups of four warps (group g takes k-blocks g, g+3, ...).  Six A buffers (two per group): a group waits for the
// MMAs of its block before last, never for the previous one.  Weight ring: six stages of one block (two per group,
// released as soon as the block is in registers).  Stage, A buffer and "done" barrier of block i have index i mod 6
// and always belong to group i mod 3 and issuer i mod NISS: every waiter sees every phase of the barriers it waits on
// (a waiter that skips phases passes a parity wait one phase early).  The split-K exchange buffer aliases the
// activation ring: a CTA announces that its last MMA completed with a cluster-barrier arrive and peers wait for that
// phase before they push.
//
// Named barriers have no time-out, so nobody may skip one: after a bounded mbarrier wait gave up (abort flag raised)
// every role keeps walking its blocks, skipping the waits and the work but not the bar.arrive / bar.sync.
#include <cooperative_groups.h>

#include <mutex>
#include <unordered_set>

#include "umma.cuh"

namespace cg = cooperative_groups;

namespace rwkv7 {

namespace w4 {
constexpr int TILE_N = 128;  // output channels per CTA = UMMA M
constexpr int KB = 128;      // k elements per block
constexpr int RAW_BYTES = TILE_N * KB / 2;  // 8192 packed nibbles
constexpr int SC_OFF = RAW_BYTES;           // then 128 fp16 scales of the k-block
constexpr int Z_OFF = SC_OFF + TILE_N * 2;  // then 128 u8 zero-points, then padding
constexpr int W4_BLOCK_BYTES = 8704;        // one int4 tile block in memory = one bulk copy (68 x 128 B)
constexpr int W8_BLOCK_BYTES = TILE_N * KB;  // int8 per-channel format: 16 KiB of offset-binary bytes (q + 128), scales apart
constexpr int TMEM_COLS = 512;
constexpr int G = 3;                        // dequant groups (four groups with one A buffer each measured the same)
constexpr int NA = 6;                       // A buffers (two per group) = weight stages = "done" barriers
constexpr int HANDOFF_THREADS = 128 + 32;   // a dequant group arrives, its issuer warp syncs

// NB = activation rows per weight pass = UMMA N.  64: two issuers, six activation stages sharing the "done" barriers
// with the A buffers.  128: one issuer (tensor memory holds 6 A buffers + one 128-column accumulator), three
// activation stages of 32 KiB with their own barriers.
// FMT 0 = int4 group-128 (scales and zero-points inside the block), FMT 1 = int8 with one scale per output channel.
template <int NB_, int FMT_>
struct Cfg {
    static constexpr int NB = NB_, FMT = FMT_;
    static constexpr int BLOCK_BYTES = FMT_ == 0 ? W4_BLOCK_BYTES : W8_BLOCK_BYTES;
    static constexpr int WRING_BYTES = NA * BLOCK_BYTES;
    static constexpr int NISS = NB_ == 64 ? 2 : 1;
    static constexpr int XST = NB_ == 64 ? 6 : 3;
    static constexpr bool SHARED_DONE = XST == NA;  // one commit per block releases the activation stage and the A buffer
    static constexpr int XATOM = NB_ * 128, X_BYTES = 2 * XATOM;
    static constexpr int FIRST_DQ_WARP = 2 + NISS;
    static constexpr int NTHREADS = (FIRST_DQ_WARP + G * 4) * 32;
    static constexpr int A_COL = 0, D_COL = NA * 64;
    static constexpr int Q_BYTES = NB_ * TILE_N * 4;
    static constexpr int NBARS = 2 * XST + 3 * NA + 1;
    static constexpr size_t SMEM = (size_t)XST * X_BYTES + WRING_BYTES + NBARS * 8 + 16 + 1024;
    static_assert(SMEM <= 227 * 1024, "shared memory capacity");
    static_assert(NA % G == 0 && NA % NISS == 0, "an A buffer must always belong to the same group and issuer");
    static_assert(Q_BYTES <= XST * X_BYTES, "the exchange buffer aliases the activation ring");
    static_assert(D_COL + NISS * NB_ <= TMEM_COLS, "tensor memory capacity");
};
}  // namespace w4

constexpr int kW4MaxGroup = 4;  // projections of equal shape served by one launch (r / k / v of a layer)

struct W4UmmaArgs {
    const uint8_t* tw[kW4MaxGroup];  // tiled weights: [tiles][K/128] blocks; int4: [4 chunks][128 channels][16 B] | scales | zeros,
                                     // int8: [8 chunks][128 channels][16 B]
    const __half* rscale[kW4MaxGroup];  // int8 format: one scale per output channel
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

// int8 format: a word holds the offset-binary bytes (q + 128) of four consecutive k.  prmt puts each byte under the high
// byte 0x64, which is the fp16 number 1024 + byte; subtracting 1152 leaves q exactly.  The per-channel scale is applied
// to the fp32 accumulator in the epilogue.
__device__ __forceinline__ void dequant_word8(uint32_t w, uint32_t* out) {
    constexpr uint32_t kHi = 0x64646464u, kOff = 0x64806480u;  // (1152, 1152)
    uint32_t a, b;
    asm("prmt.b32 %0, %1, %2, 0x4140;" : "=r"(a) : "r"(w), "r"(kHi));
    asm("prmt.b32 %0, %1, %2, 0x4342;" : "=r"(b) : "r"(w), "r"(kHi));
    asm("sub.f16x2 %0, %1, %2;" : "=r"(out[0]) : "r"(a), "r"(kOff));
    asm("sub.f16x2 %0, %1, %2;" : "=r"(out[1]) : "r"(b), "r"(kOff));
}

__device__ __forceinline__ void bulk_load(void* smem_dst, const void* gsrc, uint32_t bytes, uint64_t* bar) {
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];"
                 ::"r"(smem_u32(smem_dst)), "l"(gsrc), "r"(bytes), "r"(smem_u32(bar)) : "memory");
}

__device__ __forceinline__ bool elect_one() {
    uint32_t pred;
    asm volatile("{\n\t.reg .pred P;\n\telect.sync _|P, 0xffffffff;\n\tselp.b32 %0, 1, 0, P;\n\t}" : "=r"(pred));
    return pred != 0;
}
__device__ __forceinline__ void named_arrive(int id, int threads) { asm volatile("bar.arrive %0, %1;" ::"r"(id), "r"(threads) : "memory"); }
__device__ __forceinline__ void named_sync(int id, int threads) { asm volatile("bar.sync %0, %1;" ::"r"(id), "r"(threads) : "memory"); }

template <int NBT, int FMT>
__global__ void __launch_bounds__(w4::Cfg<NBT, FMT>::NTHREADS, 1)
w4g_umma_kernel(const __grid_constant__ W4Maps maps, const W4UmmaArgs p) {
    using namespace w4;
    using C = Cfg<NBT, FMT>;
    constexpr int BLOCK_BYTES = C::BLOCK_BYTES, WRING_BYTES = C::WRING_BYTES;
    constexpr int NB = C::NB, NISS = C::NISS, XST = C::XST, X_BYTES = C::X_BYTES, XATOM = C::XATOM;
    constexpr int FIRST_DQ_WARP = C::FIRST_DQ_WARP, NTHREADS = C::NTHREADS, A_COL = C::A_COL, D_COL = C::D_COL;
    extern __shared__ unsigned char smem_unaligned[];
    // the swizzled TMA / UMMA tiles need 1024-byte alignment; the offset is the same in every CTA
    unsigned char* smem = smem_unaligned + ((1024u - (smem_u32(smem_unaligned) & 1023u)) & 1023u);
    unsigned char* xs = smem;                                   // [XST][atom 0 | atom 1]
    unsigned char* raws = smem + XST * X_BYTES;                 // [NA][nibbles | scales | zeros]
    float* Q = reinterpret_cast<float*>(xs);                    // split-K exchange (after the last MMA)
    uint64_t* bars = reinterpret_cast<uint64_t*>(raws + WRING_BYTES);
    uint64_t* full = bars;               // [XST] activation tile landed
    uint64_t* xfree = bars + XST;        // [XST] the MMAs that read the tile completed (unused when SHARED_DONE)
    uint64_t* done = xfree + XST;        // [NA]  the MMAs of the block completed: its A buffer is free
    uint64_t* wfull = done + NA;         // [NA]  weight block landed
    uint64_t* wempty = wfull + NA;       // [NA]  the group's four warps hold the block in registers
    uint64_t* d_full = wempty + NA;      // [1]   every issuer's last MMA completed
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(d_full + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    const AbortCtx actx{abort_flag, p.error};
    uint64_t* const xdone = C::SHARED_DONE ? done : xfree;  // what the activation producer waits on

    // the shuffle makes the warp index provably warp-uniform for the compiler (uniform registers, uniform branches)
    const int tid = threadIdx.x, warp = __shfl_sync(0xffffffffu, threadIdx.x >> 5, 0), lane = tid & 31;
    const int n0 = blockIdx.x * TILE_N;
    const int grp_idx = blockIdx.y / p.row_blocks;  // which projection of the group
    const CUtensorMap* tm_x = &maps.x[grp_idx];
    const uint8_t* tw = p.tw[grp_idx];
    __half* outp = p.out[grp_idx];
    const int m0 = (blockIdx.y % p.row_blocks) * NB;  // activation row block of this CTA
    const int m_rows = min(NB, p.M - m0);             // valid rows in the block
    const int split = blockIdx.z;
    const int kb0 = split * p.nkb;
    const int nkb = p.nkb;
    const bool clustered = p.splits > 1;
    const int rows_per_rank = NB / p.splits;
    const uint8_t* wsrc = tw + ((size_t)blockIdx.x * p.kbt + kb0) * BLOCK_BYTES;  // this CTA's contiguous weight stream

    if (tid == 0) {
        for (int s = 0; s < XST; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&xfree[s], 1);
        }
        for (int s = 0; s < NA; ++s) {
            mbar_init(&done[s], 1);
            mbar_init(&wfull[s], 1);
            mbar_init(&wempty[s], 4);  // the four warps of the block's dequant group
        }
        mbar_init(d_full, NISS);
        *abort_flag = 0;
        mbar_fence_init();
        // the first ring fill does not depend on anything: start it before the tensor-memory allocation
        const int pre = min(NA, nkb);
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
        if (lane == 0) {  // weight stream, one block per copy (nibbles + scales + zero-points)
            for (int c = NA; c < nkb; ++c) {
                const int s = c % NA;
                if (!mbar_wait(&wempty[s], ((c / NA) - 1) & 1, actx, kErrWaitEmpty)) break;
                mbar_expect_tx(&wfull[s], BLOCK_BYTES);
                bulk_load(raws + s * BLOCK_BYTES, wsrc + (size_t)c * BLOCK_BYTES, BLOCK_BYTES, &wfull[s]);
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {  // activation tiles: both 64-k atoms of a block through one 3-D map (k_in, row, k_out)
            // The activations are the only input the preceding kernel of the stream may still be writing: under a
            // programmatic launch the weight stream, the dequantisation and the tensor-memory A buffers run ahead
            // of this point, in the shadow of that kernel.
            grid_dependency_wait();
            // Only now may the next kernel of the stream start: every kernel of this library releases its successor
            // after its own wait, so a programmatically launched kernel knows that everything before its immediate
            // predecessor has completed.
            grid_launch_dependents();
            for (int i = 0; i < nkb; ++i) {
                const int s = i % XST;
                if (i >= XST && !mbar_wait(&xdone[s], ((i / XST) - 1) & 1, actx, kErrWaitEmpty)) break;
                mbar_expect_tx(&full[s], X_BYTES);
                tma_load_3d(xs + s * X_BYTES, tm_x, &full[s], 0, m0, (kb0 + i) * 2);
            }
        }
    } else if (warp < FIRST_DQ_WARP) {
        // ---- issuers: per block, meet the group at the A buffer's named barrier, then one elected lane issues
        constexpr uint32_t idesc = make_idesc(TILE_N, NB, /*F32*/ 1, /*F16*/ 0, /*F16*/ 0);
        const int me = warp - 2;
        const uint32_t d_tmem = tmem_base + D_COL + me * NB;
        bool ok = true;
        for (int i = me; i < nkb; i += NISS) {
            const int xst = i % XST, aa = i % NA;
            if (elect_one()) {  // the activation tile has usually landed long before the A buffer is ready
                if (ok && *abort_flag == 0) ok = mbar_wait(&full[xst], (i / XST) & 1, actx, kErrWaitFull);
                else ok = false;
            }
            ok = __all_sync(0xffffffffu, ok);
            named_sync(1 + aa, HANDOFF_THREADS);  // never skipped
            if (elect_one()) {
                if (ok) {
                    tc_fence_after();
                    // descriptor of the stage's first atom; the start-address field counts 16-byte units
                    const uint64_t bdesc0 = make_sw128_kmajor_desc(smem_u32(xs + xst * X_BYTES));
                    const uint32_t a_tmem = tmem_base + A_COL + aa * 64;
#pragma unroll
                    for (int j = 0; j < KB / 16; ++j) {
                        const uint64_t bdesc = bdesc0 + (uint64_t)(((j >> 2) * XATOM + (j & 3) * 32) >> 4);
                        umma_f16_ts(d_tmem, a_tmem + j * 8, bdesc, idesc, (i == me && j == 0) ? 0u : 1u);
                    }
                }
                // committed even when nothing was issued: the waiters of these barriers are released either way
                tc_commit(&done[aa]);
                if (!C::SHARED_DONE) tc_commit(&xfree[xst]);
                if (i + NISS >= nkb) tc_commit(d_full);
            }
        }
        if (me >= nkb && lane == 0) mbar_arrive(d_full);  // an issuer without any block still owes its arrival
    } else {
        const int q = warp & 3;                      // TMEM lane quarter this warp may access
        const int g = (warp - FIRST_DQ_WARP) >> 2;   // dequant group
        const int row = q * 32 + lane;
        const uint32_t lane_addr = tmem_base + ((uint32_t)(q * 32) << 16);
        bool ok = true;
        for (int i = g; i < nkb; i += G) {
            const int aa = i % NA;
            const unsigned char* wblk = raws + aa * BLOCK_BYTES;
            // one lane per warp polls; the others wait at the shuffle
            if (lane == 0 && ok) ok = mbar_wait(&wfull[aa], (i / NA) & 1, actx, kErrWaitFull);
            ok = __shfl_sync(0xffffffffu, ok, 0);
            uint32_t v[4][16];
            if (ok) {
                // this channel's 64 packed bytes: chunk c (32 k) of all 128 channels is one 2 KiB slab, so the
                // threads of a warp read consecutive 16-byte pieces (no bank conflicts, no swizzle)
                const unsigned char* rrow = wblk + row * 16;
                if constexpr (FMT == 0) {
                    uint4 pk[4];
#pragma unroll
                    for (int c = 0; c < 4; ++c) pk[c] = *reinterpret_cast<const uint4*>(rrow + c * 2048);
                    const uint32_t s16 = reinterpret_cast<const unsigned short*>(wblk + SC_OFF)[row];
                    const uint32_t z = (wblk + Z_OFF)[row];
                    const uint32_t sc = s16 * 0x00010001u;               // (scale, scale)
                    const uint32_t zlo = z * 0x00010001u + 0x64006400u;  // 1024 + z as fp16: 0x6400 | z
                    const uint32_t zhi = z * 0x00100010u + 0xD400D400u;  // -(64 + z) as fp16: 0xD400 | (z << 4)
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&wempty[aa]);
#pragma unroll
                    for (int c = 0; c < 4; ++c) {
                        dequant_word(pk[c].x, zlo, zhi, sc, v[c] + 0);
                        dequant_word(pk[c].y, zlo, zhi, sc, v[c] + 4);
                        dequant_word(pk[c].z, zlo, zhi, sc, v[c] + 8);
                        dequant_word(pk[c].w, zlo, zhi, sc, v[c] + 12);
                    }
                } else {
                    // 128 bytes per channel: chunk c (16 k) of all 128 channels is one 2 KiB slab
                    uint4 pk[8];
#pragma unroll
                    for (int c = 0; c < 8; ++c) pk[c] = *reinterpret_cast<const uint4*>(rrow + c * 2048);
                    __syncwarp();
                    if (lane == 0) mbar_arrive(&wempty[aa]);
#pragma unroll
                    for (int c = 0; c < 8; ++c) {
                        uint32_t* o = v[c >> 1] + (c & 1) * 8;
                        dequant_word8(pk[c].x, o + 0);
                        dequant_word8(pk[c].y, o + 2);
                        dequant_word8(pk[c].z, o + 4);
                        dequant_word8(pk[c].w, o + 6);
                    }
                }
            }
            if (i >= NA && ok) {  // the MMAs of the block that used this A buffer before completed
                if (lane == 0) ok = mbar_wait(&done[aa], ((i / NA) - 1) & 1, actx, kErrWaitAFree);
                ok = __shfl_sync(0xffffffffu, ok, 0);
            }
            if (ok) {
                tc_fence_after();
                const uint32_t a_addr = lane_addr + A_COL + aa * 64;
#pragma unroll
                for (int c = 0; c < 4; ++c) tmem_st16(a_addr + c * 16, v[c]);
                tc_wait_st();
                tc_fence_before();
            }
            named_arrive(1 + aa, HANDOFF_THREADS);  // never skipped
        }

        if (lane == 0) ok = (*abort_flag == 0) && mbar_wait(d_full, 0, actx, kErrWaitDFull);
        ok = __shfl_sync(0xffffffffu, ok, 0);
        // ---- every MMA of this CTA has completed: its activation ring is free, peers may push into the exchange buffer
        if (clustered) {
            cluster_arrive_release();
            cluster_wait();
        }
        if (ok && *abort_flag == 0) {
            tc_fence_after();
            // 16-column chunks of the accumulator (activation rows) are dealt to the groups in turn
            for (int c = g; c < NB / 16; c += G) {
                const int col0 = c * 16;
                uint32_t v[16];
                tmem_ld16(lane_addr + D_COL + col0, v);
                tc_wait_ld();
                if (NISS == 2 && nkb > 1) {  // the second issuer's accumulator
                    uint32_t t[16];
                    tmem_ld16(lane_addr + D_COL + NB + col0, t);
                    tc_wait_ld();
#pragma unroll
                    for (int e = 0; e < 16; ++e) v[e] = __float_as_uint(__uint_as_float(v[e]) + __uint_as_float(t[e]));
                }
                if (!clustered) {
                    // No split-K: nothing to exchange, so the accumulator goes straight to global memory (fp16
                    // rounding, epilogue, 2-byte stores: the 32 lanes of a warp cover 64 contiguous bytes of a row).
                    const int nn = n0 + row;
                    grid_dependency_wait();  // returns at once (the accumulator already depends on the activations)
                    if (nn < p.Nout) {
                        const float rs = FMT == 1 ? __half2float(p.rscale[grp_idx][nn]) : 1.f;
#pragma unroll
                        for (int e = 0; e < 16; ++e) {
                            const int m = col0 + e;
                            if (m >= m_rows) break;
                            const size_t o = (size_t)(m0 + m) * p.Nout + nn;
                            float y = __half2float(__float2half_rn(__uint_as_float(v[e]) * rs));
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
                    // 8 consecutive rows never straddle two ranks (rows_per_rank is a multiple of 8)
#pragma unroll
                    for (int h8 = 0; h8 < 2; ++h8) {
                        const int m = col0 + h8 * 8;
                        const int dst = m / rows_per_rank;
                        float* qd = cluster.map_shared_rank(Q, dst) + ((size_t)split * rows_per_rank + (m - dst * rows_per_rank)) * TILE_N + row;
#pragma unroll
                        for (int e = 0; e < 8; ++e) qd[e * TILE_N] = __uint_as_float(v[h8 * 8 + e]);
                    }
                }
            }
            tc_fence_before();
        }
    }
    if (warp < FIRST_DQ_WARP && clustered) {  // the producer and issuer warps take part in the same cluster-barrier phases
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
    grid_dependency_wait();  // residual reads and output writes are ordered after the preceding kernel (returns at once here)
    if (!aborted && clustered) {
        // Each thread owns one channel pair (n, n+1) and walks the rows of this rank's share: float2 loads of the rank
        // slots in fixed order, fp16 rounding, epilogue, one 4-byte store; 64 consecutive threads cover one 256-byte
        // output row segment.
        const int m_begin = split * rows_per_rank;
        const int m_end = min(m_rows, m_begin + rows_per_rank);
        const int n = (tid & 63) * 2;
        const bool n_ok = n0 + n < p.Nout;
        const bool pair = (n0 + n + 1 < p.Nout) && ((p.Nout & 1) == 0);
        constexpr int RSTEP = NTHREADS / 64;  // full 64-thread row teams (a trailing half team sits out)
        const float* Q0 = Q + n - (size_t)m_begin * TILE_N;  // slot r, global row m: Q0[(r * rows_per_rank + m) * TILE_N]
        const int slot = rows_per_rank * TILE_N;
        float rs0 = 1.f, rs1 = 1.f;
        if (FMT == 1 && n_ok) {
            rs0 = __half2float(p.rscale[grp_idx][n0 + n]);
            if (n0 + n + 1 < p.Nout) rs1 = __half2float(p.rscale[grp_idx][n0 + n + 1]);
        }
        for (int m = m_begin + (tid >> 6); m < m_end && n_ok && (tid >> 6) < RSTEP; m += RSTEP) {
            const float* qq = Q0 + m * TILE_N;
            float2 acc = *reinterpret_cast<const float2*>(qq);
            for (int r = 1; r < p.splits; ++r) {
                const float2 t2 = *reinterpret_cast<const float2*>(qq + r * slot);
                acc.x += t2.x;
                acc.y += t2.y;
            }
            const size_t o = (size_t)(m0 + m) * p.Nout + n0 + n;
            float y0 = __half2float(__float2half_rn(acc.x * rs0)), y1 = __half2float(__float2half_rn(acc.y * rs1));
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
    __syncthreads();  // nothing remote is touched after the barrier above, so the CTA may leave on its own
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
    uint8_t* block = tiled + blk * w4::W4_BLOCK_BYTES;
    reinterpret_cast<uint32_t*>(block)[widx & 2047] = out;
    if (c == 0 && j == 0) {
        const long long gi = n * (K / group) + (b * 128) / group;
        reinterpret_cast<T*>(block + w4::SC_OFF)[r] = (n < Nout) ? scales[gi] : from_f<T>(0.f);
        (block + w4::Z_OFF)[r] = (n < Nout && zeros) ? zeros[gi] : (uint8_t)8;
    }
}

// int8 per-channel weights q [Nout, K] -> [tiles][K/128] blocks of [8 chunks][128 channels][16 B], bytes stored as
// q + 128 (offset binary: the kernel's byte -> fp16 conversion needs no sign handling).  One thread per 16-byte piece.
__global__ void w8_repack_kernel(const int8_t* __restrict__ q, uint8_t* __restrict__ tiled, int K, int Nout, long long total_pieces) {
    const long long pidx = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (pidx >= total_pieces) return;
    // pidx = ((tile * kbt + b) * 8 + c) * 128 + r
    const int r = (int)(pidx & 127);
    const int c = (int)((pidx >> 7) & 7);
    const long long blk = pidx >> 10;
    const int kbt = K / 128;
    const int b = (int)(blk % kbt);
    const long long n = (blk / kbt) * 128 + r;
    uint4 v = make_uint4(0x80808080u, 0x80808080u, 0x80808080u, 0x80808080u);  // padding channels: q = 0
    if (n < Nout) {
        v = *reinterpret_cast<const uint4*>(q + n * K + b * 128 + c * 16);
        v.x ^= 0x80808080u; v.y ^= 0x80808080u; v.z ^= 0x80808080u; v.w ^= 0x80808080u;
    }
    reinterpret_cast<uint4*>(tiled)[pidx] = v;
}

// Tiled buffers written by rwkv7_w4g_repack / rwkv7_w8_repack and not yet read by a projection.  The projection kernel streams the
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
template <int NBT, int FMT>
static cudaError_t launch_variant(cudaLaunchConfig_t& cfg, const W4Maps& maps, const W4UmmaArgs& a) {
    using C = w4::Cfg<NBT, FMT>;
    cudaError_t e = cudaFuncSetAttribute(w4g_umma_kernel<NBT, FMT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)C::SMEM);
    if (e != cudaSuccess) return e;
    cfg.blockDim = dim3(C::NTHREADS);
    cfg.dynamicSmemBytes = C::SMEM;
    return cudaLaunchKernelEx(&cfg, w4g_umma_kernel<NBT, FMT>, maps, a);
}

// fmt 0: int4 group-wise tiled weights; fmt 1: int8 tiled weights with per-channel scales rscales[g] [Nout].
int launch_w4g_umma_tiled(const void* const* xs, const uint8_t* const* tws, const void* const* rscales, const void* residual,
                          void* const* outs, int G, int M, int K, int Nout, int epilogue, int fmt, cudaStream_t st) {
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
        if (tiles * row_blocks * G * s <= 148 && total_kb % s == 0 && (total_kb / s) >= 4) {
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
        a.rscale[g] = rscales ? reinterpret_cast<const __half*>(rscales[g]) : nullptr;
        a.out[g] = reinterpret_cast<__half*>(outs[g]);
        fresh |= take_tiled_fresh(tws[g]);
    }
    for (int g = G; g < kW4MaxGroup; ++g) maps.x[g] = maps.x[0];
    a.residual = reinterpret_cast<const __half*>(residual);
    a.M = M; a.K = K; a.Nout = Nout; a.epilogue = epilogue; a.nkb = nkb; a.kbt = total_kb; a.splits = splits;
    a.row_blocks = row_blocks;
    a.error = kernel_error_word();
    RWKV7_REQUIRE(a.error != nullptr, RWKV7_ERR_CUDA, "w4g_gemv_tiled: cannot resolve the device error word");
    cudaLaunchConfig_t cfg{};
    cfg.gridDim = dim3(tiles, row_blocks * G, splits);
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
    const cudaError_t e = NB == 64 ? (fmt == 0 ? launch_variant<64, 0>(cfg, maps, a) : launch_variant<64, 1>(cfg, maps, a))
                                   : (fmt == 0 ? launch_variant<128, 0>(cfg, maps, a) : launch_variant<128, 1>(cfg, maps, a));
    RWKV7_REQUIRE(e == cudaSuccess, RWKV7_ERR_CUDA, "w4g_gemv_tiled launch: %s", cudaGetErrorString(e));
    return RWKV7_OK;
}

}  // namespace rwkv7

using namespace rwkv7;

extern "C" int64_t rwkv7_w4g_tiled_bytes(int K, int Nout) {
    if (K <= 0 || Nout <= 0 || K % 128) return 0;
    const int64_t tiles = (Nout + 127) / 128, kbt = K / 128;
    return tiles * kbt * w4::W4_BLOCK_BYTES;
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
    return launch_w4g_umma_tiled(&x, &tiled, nullptr, residual, &out, 1, M, K, Nout, epilogue, 0, static_cast<cudaStream_t>(stream));
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
    return launch_w4g_umma_tiled(xs, tiled, nullptr, nullptr, outs, G, M, K, Nout, epilogue, 0, static_cast<cudaStream_t>(stream));
}

// ---------------------------------------------------------------- int8 per-output-channel weights
extern "C" int64_t rwkv7_w8_tiled_bytes(int K, int Nout) {
    if (K <= 0 || Nout <= 0 || K % 128) return 0;
    const int64_t tiles = (Nout + 127) / 128, kbt = K / 128;
    return tiles * kbt * w4::W8_BLOCK_BYTES;
}

extern "C" int rwkv7_w8_repack(const int8_t* q, uint8_t* tiled, int K, int Nout, void* stream) {
    RWKV7_REQUIRE(K > 0 && Nout > 0 && K % 128 == 0, RWKV7_ERR_UNSUPPORTED, "w8_repack: K must be a positive multiple of 128");
    RWKV7_REQUIRE(q && tiled, RWKV7_ERR_INVALID, "w8_repack: null pointer");
    RWKV7_REQUIRE(aligned(q, 16) && aligned(tiled, 16), RWKV7_ERR_ALIGN, "w8_repack: unaligned pointer");
    const long long pieces = (long long)((Nout + 127) / 128) * (K / 128) * 1024;
    w8_repack_kernel<<<(unsigned)((pieces + 255) / 256), 256, 0, static_cast<cudaStream_t>(stream)>>>(q, tiled, K, Nout, pieces);
    mark_tiled_fresh(tiled);
    return check_launch("w8_repack_kernel");
}

extern "C" int rwkv7_w8_gemv_tiled_group(const void* const* xs, const uint8_t* const* tiled, const void* const* scales,
                                         const void* residual, void* const* outs, int G, int M, int K, int Nout, int epilogue,
                                         int dtype, void* stream) {
    RWKV7_REQUIRE(xs && tiled && scales && outs, RWKV7_ERR_INVALID, "w8_gemv_tiled_group: null pointer");
    RWKV7_REQUIRE(G >= 1 && G <= kW4MaxGroup, RWKV7_ERR_UNSUPPORTED, "w8_gemv_tiled_group: 1..%d projections (got %d)", kW4MaxGroup, G);
    RWKV7_REQUIRE(dtype == RWKV7_F16, RWKV7_ERR_UNSUPPORTED, "w8_gemv_tiled_group: fp16 activations only");
    RWKV7_REQUIRE(epilogue >= 0 && epilogue <= 2, RWKV7_ERR_INVALID, "w8_gemv_tiled_group: bad epilogue code %d", epilogue);
    RWKV7_REQUIRE(epilogue != RWKV7_EPI_ADD || (residual && G == 1), RWKV7_ERR_INVALID,
                  "w8_gemv_tiled_group: the add epilogue takes one projection and a residual");
    for (int g = 0; g < G; ++g) {
        RWKV7_REQUIRE(xs[g] && tiled[g] && scales[g] && outs[g], RWKV7_ERR_INVALID, "w8_gemv_tiled_group: null pointer in projection %d", g);
        RWKV7_REQUIRE(aligned(xs[g], 16) && aligned(tiled[g], 16), RWKV7_ERR_ALIGN, "w8_gemv_tiled_group: pointers must be 16-byte aligned");
    }
    return launch_w4g_umma_tiled(xs, tiled, scales, residual, outs, G, M, K, Nout, epilogue, 1, static_cast<cudaStream_t>(stream));
}
