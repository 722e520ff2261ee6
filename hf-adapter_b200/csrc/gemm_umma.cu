// Persistent tensor-core GEMM with fused epilogues, for the many-row (prefill) side of the projections:
//
//   C[M, N] = epilogue( A[M, K] . B[N, K]^T )        A, B K-major (row-major activations, [out, in] weights)
//
//   kind f16 / bf16 : fp32 accumulation; epilogue (+ bias) then relu^2 or (+ residual), output in the operand type
//   kind i8         : int32 accumulation (exact); epilogue raw int32, or the A8W8 dequantisation
//                     acc * sa[row] * sw[col] (+ bias) (+ residual) in fp32 with every step rounded, output T
//
// One CTA per SM walks output tiles of 128 x 256 in an order that keeps a band of 16 row-tiles of A in L2 while the
// B tiles stream.  TMA (128-byte swizzle, 128 bytes of K per box) lands both operands in the layout the MMA
// descriptors read; a 4-stage ring feeds tcgen05.mma (one issuing thread); TWO accumulators of 256 columns live in
// tensor memory, so the epilogue warps drain tile i while the tensor pipe already works on tile i + 1.
// Warp 0 = TMA producer, warp 1 = MMA issuer + TMEM owner, warps 2-5 = epilogue (TMEM -> staging -> global); the CTA-pair
// kernel has a second form with eight epilogue warps for products with a tiny K, which are all epilogue.
// Ragged M / N / K edges are zero-filled by TMA and masked at the store.  All waits are bounded (umma.cuh).
// With more than 128 rows the same roles run as CTA pairs on 256 x 256 tiles (second kernel below).
#include "umma.cuh"

namespace rwkv7 {
namespace gm {
constexpr int BM = 128, BN = 256, BKB = 128, STAGES = 4, THREADS = 192;
constexpr int A_BYTES = BM * BKB, B_BYTES = BN * BKB, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int TMEM_COLS = 512;
constexpr int EPI_WARPS = 4;                        // one per TMEM lane quadrant
constexpr int STG_WARP_BYTES = 32 * 64 * 4;         // epilogue staging per epilogue warp: 32 rows x 64 fp32 columns
constexpr int STG_BYTES = EPI_WARPS * STG_WARP_BYTES;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 256 + STG_BYTES + 1024;
constexpr int GROUP_M = 16;
enum { KIND_F16 = 0, KIND_BF16 = 1, KIND_I8 = 2 };
enum { EPI_STORE = 0, EPI_RELU2 = 1, EPI_DEQUANT = 2, EPI_RAW_I32 = 3, EPI_ARGMAX = 4 };
}  // namespace gm

struct GemmArgs {
    void* C;
    const void* bias;      // [N] in the output type, or null
    const void* residual;  // [M, N] in the output type, or null
    const float* sa;       // [M] row scales (dequant epilogue)
    const float* sw;       // [N] channel scales (dequant epilogue)
    int M, N, K;
    int tiles_m, tiles_n;
    int epi;
    int relu2;  // with EPI_DEQUANT: relu^2 of the dequantised value rounded to the output type (instead of + residual)
    int vec;  // 1: N % 8 == 0 and every pointer the epilogue touches is 16-byte aligned
    unsigned int* error;
    // arg-max epilogue: per (row, column tile) the best value rounded to the output type and its column, [M, tiles_n] each
    float* part_val;
    int* part_idx;
};

// tile -> (row tile, column tile): bands of GROUP_M row tiles, row tile fastest inside a band
__device__ __forceinline__ void tile_coords(int tile, int tiles_m, int tiles_n, int& tm, int& tn) {
    const int per_band = gm::GROUP_M * tiles_n;
    const int band = tile / per_band, within = tile - band * per_band;
    const int rows = min(gm::GROUP_M, tiles_m - band * gm::GROUP_M);
    tn = within / rows;
    tm = band * gm::GROUP_M + (within - tn * rows);
}

// The epilogue of one warp for 64 columns of its 32 accumulator rows.  A thread owns one TMEM lane (= one row), so
// storing straight from the registers tcgen05.ld fills would write 32-byte pieces of 32 different rows per instruction:
// a quarter of every 128-byte line at a time and 32 wavefronts per store.  Instead the raw accumulators go through a
// per-warp staging tile in shared memory (16-byte units, unit index XORed with the row so both passes are
// conflict-free) and come back with eight lanes on the eight 16-byte pieces of one row: scales, bias and residual
// are then loaded, and the result stored, as whole 128-byte row segments, four rows per instruction.
template <int KIND, typename TOut>
__device__ __forceinline__ void epilogue_group(const GemmArgs& p, uint32_t* stg, uint32_t taddr, int row0, int col0, int lane) {
    using namespace gm;
    const int j8 = (lane & 7) * 8;  // this lane's eight columns inside the group
    const int col = col0 + j8;
    const TOut* res = reinterpret_cast<const TOut*>(p.residual);
    const bool full = p.vec && col + 8 <= p.N;
    // the residual does not depend on the accumulators: its eight row pieces are requested before the TMEM loads
    Vec8<TOut> rres[8];
    const bool pre_res = res != nullptr && full && !(p.epi == EPI_RELU2 || p.relu2);
    if (pre_res) {
#pragma unroll
        for (int i = 0; i < 8; ++i) {
            const int row = row0 + (lane >> 3) + 4 * i;
            if (row < p.M) rres[i] = *reinterpret_cast<const Vec8<TOut>*>(res + (size_t)row * p.N + col);
        }
    }
    // so do the tile-constant vectors of this lane's eight columns (bias, channel scales)
    const TOut* bias = reinterpret_cast<const TOut*>(p.bias);
    float bv[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f}, sv[8];
    if (col < p.N) {
        if (full) {
            if (bias) load8(bias + col, bv);
            if constexpr (KIND == KIND_I8) {
                if (p.epi == EPI_DEQUANT) load8(p.sw + col, sv);
            }
        } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                bv[e] = (bias && col + e < p.N) ? to_f<TOut>(bias[col + e]) : 0.f;
                if constexpr (KIND == KIND_I8) sv[e] = (p.epi == EPI_DEQUANT && col + e < p.N) ? p.sw[col + e] : 0.f;
            }
        }
    }
    {
        uint32_t v[64];
        tmem_ld64(taddr, v);
        tc_wait_ld();
#pragma unroll
        for (int u = 0; u < 16; ++u) {  // 16-byte units of this row
            const int pos = (u & 8) | ((u & 7) ^ (lane & 7));
            *reinterpret_cast<uint4*>(stg + lane * 64 + pos * 4) = make_uint4(v[4 * u], v[4 * u + 1], v[4 * u + 2], v[4 * u + 3]);
        }
    }
    __syncwarp();
#pragma unroll
    for (int i = 0; i < 8; ++i) {
        const int r = (lane >> 3) + 4 * i, row = row0 + r;
        const int u0 = (lane & 7) * 2;
        const uint4 a0 = *reinterpret_cast<const uint4*>(stg + r * 64 + ((u0 & 8) | ((u0 & 7) ^ (r & 7))) * 4);
        const uint4 a1 = *reinterpret_cast<const uint4*>(stg + r * 64 + (((u0 + 1) & 8) | (((u0 + 1) & 7) ^ (r & 7))) * 4);
        if (row >= p.M || col >= p.N) continue;
        const uint32_t raw[8] = {a0.x, a0.y, a0.z, a0.w, a1.x, a1.y, a1.z, a1.w};
        const size_t off = (size_t)row * p.N + col;
        if constexpr (KIND == KIND_I8) {
            if (p.epi == EPI_RAW_I32) {
                int32_t* dst = reinterpret_cast<int32_t*>(p.C) + off;
                if (full) {
                    *reinterpret_cast<uint4*>(dst) = a0;
                    *reinterpret_cast<uint4*>(dst + 4) = a1;
                } else {
                    for (int e = 0; e < 8 && col + e < p.N; ++e) dst[e] = (int)raw[e];
                }
                continue;
            }
        }
        float f[8];
        if constexpr (KIND == KIND_I8) {
            const float a_s = p.sa[row];
#pragma unroll
            for (int e = 0; e < 8; ++e) f[e] = __fmul_rn(__fmul_rn((float)(int)raw[e], a_s), sv[e]);
        } else {
#pragma unroll
            for (int e = 0; e < 8; ++e) f[e] = __uint_as_float(raw[e]);
        }
        if (bias) {
#pragma unroll
            for (int e = 0; e < 8; ++e) f[e] = __fadd_rn(f[e], bv[e]);
        }
        if (p.epi == EPI_RELU2 || p.relu2) {
#pragma unroll
            for (int e = 0; e < 8; ++e) {
                const float a = fmaxf(round_to<TOut>(f[e]), 0.f);
                f[e] = a * a;
            }
        } else if (res) {
            if (full) {
#pragma unroll
                for (int e = 0; e < 8; ++e) f[e] = __fadd_rn(f[e], to_f<TOut>(rres[i].v[e]));
            } else {
                for (int e = 0; e < 8 && col + e < p.N; ++e) f[e] = __fadd_rn(f[e], to_f<TOut>(res[off + e]));
            }
        }
        TOut* dst = reinterpret_cast<TOut*>(p.C) + off;
        if (full) {
            store8(dst, f);
        } else {
            for (int e = 0; e < 8 && col + e < p.N; ++e) dst[e] = from_f<TOut>(f[e]);
        }
    }
    __syncwarp();  // the staging tile is overwritten by the next group
}

// Arg-max epilogue: nothing of the product is stored.  A thread owns one row of the tile and folds its 256 columns
// into (best value, lowest column holding it); values are first rounded to the output type, so the winner is the one
// torch.argmax picks on the stored logits.
template <typename TOut>
__device__ __forceinline__ void argmax_chunk(const GemmArgs& p, const uint32_t (&v)[16], int col, float& best, int& best_col) {
#pragma unroll
    for (int e = 0; e < 16; ++e) {
        const float x = round_to<TOut>(__uint_as_float(v[e]));
        if (col + e < p.N && x > best) {
            best = x;
            best_col = col + e;
        }
    }
}

template <int KIND, typename TOut>
__global__ void __launch_bounds__(gm::THREADS, 1)
gemm_umma_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b, const GemmArgs p) {
    using namespace gm;
    extern __shared__ unsigned char smem_unaligned[];
    unsigned char* sm = smem_unaligned + ((1024u - (smem_u32(smem_unaligned) & 1023u)) & 1023u);
    uint64_t* full = reinterpret_cast<uint64_t*>(sm + STAGES * STAGE_BYTES);
    uint64_t* empty = full + STAGES;
    uint64_t* acc_full = empty + STAGES;
    uint64_t* acc_empty = acc_full + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    const AbortCtx actx{abort_flag, p.error};
    uint32_t* stg = reinterpret_cast<uint32_t*>(sm + STAGES * STAGE_BYTES + 256) + ((threadIdx.x >> 5) & 3) * (32 * 64);

    constexpr int ES = (KIND == KIND_I8) ? 1 : 2;
    constexpr int BK = BKB / ES;  // elements of K per stage
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nk = (p.K + BK - 1) / BK;
    const int ntiles = p.tiles_m * p.tiles_n;

    if (tid == 0) {
        tma_prefetch_desc(&tm_a);
        tma_prefetch_desc(&tm_b);
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(&acc_full[a], 1);
            mbar_init(&acc_empty[a], EPI_WARPS);  // one arrival per epilogue warp
        }
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 1) tmem_alloc(tmem_slot, TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            int it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < ntiles; tile += gridDim.x) {
                int tm, tn;
                tile_coords(tile, p.tiles_m, p.tiles_n, tm, tn);
                for (int kb = 0; kb < nk; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (it >= STAGES && !mbar_wait(&empty[s], ((it / STAGES) - 1) & 1, actx, kErrWaitEmpty)) {
                        ok = false;
                        break;
                    }
                    mbar_expect_tx(&full[s], STAGE_BYTES);
                    unsigned char* st = sm + s * STAGE_BYTES;
                    tma_load_2d(st, &tm_a, &full[s], kb * BK, tm * BM);
                    tma_load_2d(st + A_BYTES, &tm_b, &full[s], kb * BK, tn * BN);
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = (KIND == KIND_I8)    ? make_idesc(BM, BN, /*S32*/ 2, /*S8*/ 1, /*S8*/ 1)
                                       : (KIND == KIND_F16) ? make_idesc(BM, BN, /*F32*/ 1, /*F16*/ 0, /*F16*/ 0)
                                                            : make_idesc(BM, BN, /*F32*/ 1, /*BF16*/ 1, /*BF16*/ 1);
            int it = 0, li = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < ntiles; tile += gridDim.x, ++li) {
                const int as = li & 1;
                // the epilogue must have drained this accumulator's previous tile
                if (li >= 2 && !mbar_wait(&acc_empty[as], ((li >> 1) - 1) & 1, actx, kErrWaitDFull)) break;
                tc_fence_after();
                const uint32_t d = tmem + (uint32_t)(as * BN);
                for (int kb = 0; kb < nk; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (!mbar_wait_hot(&full[s], (it / STAGES) & 1, actx, kErrWaitFull)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint64_t da = make_sw128_kmajor_desc(smem_u32(sm + s * STAGE_BYTES));
                    const uint64_t db = make_sw128_kmajor_desc(smem_u32(sm + s * STAGE_BYTES + A_BYTES));
#pragma unroll
                    for (int j = 0; j < BKB / 32; ++j) {  // 32 bytes of K per instruction
                        const uint32_t accumulate = (kb > 0 || j > 0) ? 1u : 0u;
                        if constexpr (KIND == KIND_I8)
                            umma_i8_ss(d, da + (uint64_t)(j * 2), db + (uint64_t)(j * 2), idesc, accumulate);
                        else
                            umma_f16_ss(d, da + (uint64_t)(j * 2), db + (uint64_t)(j * 2), idesc, accumulate);
                    }
                    tc_commit(&empty[s]);
                }
                if (ok) tc_commit(&acc_full[as]);
            }
        }
    } else {
        const int q = warp & 3;  // the TMEM lane quadrant this warp may read
        int li = 0;
        for (int tile = blockIdx.x; tile < ntiles; tile += gridDim.x, ++li) {
            const int as = li & 1;
            int tm, tn;
            tile_coords(tile, p.tiles_m, p.tiles_n, tm, tn);
            bool ok = true;
            if (lane == 0) ok = mbar_wait(&acc_full[as], (li >> 1) & 1, actx, kErrWaitDFull);
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) break;
            tc_fence_after();
            const int row = tm * BM + q * 32 + lane;
            const uint32_t lane_addr = tmem + ((uint32_t)(q * 32) << 16) + (uint32_t)(as * BN);
            constexpr int half = 0;  // (the CTA-pair kernel splits the columns over two warps per quadrant)
            if (KIND != KIND_I8 && p.epi == EPI_ARGMAX) {
                if (half == 0) {
                float best = -INFINITY;
                int best_col = tn * BN;
#pragma unroll 1
                for (int c = 0; c < BN / 16; ++c) {
                    uint32_t v[16];
                    tmem_ld16(lane_addr + c * 16, v);
                    tc_wait_ld();
                    argmax_chunk<TOut>(p, v, tn * BN + c * 16, best, best_col);
                }
                if (row < p.M) {
                    p.part_val[(size_t)row * p.tiles_n + tn] = best;
                    p.part_idx[(size_t)row * p.tiles_n + tn] = best_col;
                }
                }
            } else {
#pragma unroll 1
                for (int gidx = 0; gidx < BN / 64; ++gidx)
                    epilogue_group<KIND, TOut>(p, stg, lane_addr + gidx * 64, tm * BM + q * 32, tn * BN + gidx * 64, lane);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[as]);
        }
    }
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem, TMEM_COLS);
    }
}

// ---------------------------------------------------------------- CTA-pair variant (tcgen05 cta_group::2)
// Two CTAs of a cluster share one 256 x 256 output tile.  Each stages its own 128 rows of A and 128 of the 256 rows
// of B (32 KB per 128 bytes of K instead of 48 KB, so the shared-memory fill per MMA cycle drops by a third); the
// even CTA issues MMAs of M = 256 that read both CTAs' shared memory and write each CTA's 128 result rows into that
// CTA's tensor memory.  Barrier protocol: both producers' TMA loads complete on the LEADER's full[s]
// (armed by the leader with the byte count of both); the leader's commits arrive on empty[s] / acc_full[a] in BOTH
// CTAs; the epilogue warps of both CTAs arrive on the leader's acc_empty[a].  No TMA multicast.
namespace gp {
constexpr int BM = 128, PAIR_M = 256, BN = 256, HALF_N = 128, BKB = 128;
constexpr int A_BYTES = BM * BKB, B_BYTES = HALF_N * BKB;
constexpr int TMEM_COLS = 512;
// Two forms, chosen by the number of epilogue warps EW.  EW = 4 (one per TMEM lane quadrant): a stage holds two
// 128-byte K slices of both operands, [A slices][B slices], three stages.  EW = 8 (two per quadrant, each on half of the
// tile's columns) for products whose K is so short that the epilogue is all there is (the LoRA up-projections of a
// prefill): the larger staging area leaves room for five one-slice stages.
constexpr int kbox(int ew) { return ew == 8 ? 1 : 2; }
constexpr int stages(int ew) { return ew == 8 ? 5 : 3; }
constexpr int threads(int ew) { return 64 + 32 * ew; }
constexpr int stage_bytes(int ew) { return kbox(ew) * (A_BYTES + B_BYTES); }
constexpr int smem_bytes(int ew) { return stages(ew) * stage_bytes(ew) + 256 + ew * gm::STG_WARP_BYTES + 1024; }
}  // namespace gp

template <int KIND, typename TOut, int EW>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(gp::threads(EW), 1)
gemm_umma_pair_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b, const GemmArgs p) {
    using namespace gp;
    constexpr int KBOX = kbox(EW), STAGES = stages(EW), STAGE_BYTES = stage_bytes(EW);
    extern __shared__ unsigned char smem_unaligned[];
    unsigned char* sm = smem_unaligned + ((1024u - (smem_u32(smem_unaligned) & 1023u)) & 1023u);
    uint64_t* full = reinterpret_cast<uint64_t*>(sm + STAGES * STAGE_BYTES);
    uint64_t* empty = full + STAGES;
    uint64_t* acc_full = empty + STAGES;
    uint64_t* acc_empty = acc_full + 2;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(acc_empty + 2);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    const AbortCtx actx{abort_flag, p.error};
    uint32_t* stg = reinterpret_cast<uint32_t*>(sm + STAGES * STAGE_BYTES + 256) + (threadIdx.x >= 64 ? (threadIdx.x >> 5) - 2 : 0) * (32 * 64);

    constexpr int ES = (KIND == gm::KIND_I8) ? 1 : 2;
    constexpr int BK = BKB / ES;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t rank = cluster_ctarank();
    const bool leader = rank == 0;
    const int pair = blockIdx.x >> 1, npairs = gridDim.x >> 1;
    const int nk = (p.K + KBOX * BK - 1) / (KBOX * BK);  // stages per tile (a ragged last stage is zero-filled by TMA)
    const int ntiles = p.tiles_m * p.tiles_n;  // tiles of 256 x 256

    if (tid == 0) {
        tma_prefetch_desc(&tm_a);
        tma_prefetch_desc(&tm_b);
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full[s], 1);   // used in the leader only
            mbar_init(&empty[s], 1);
        }
        for (int a = 0; a < 2; ++a) {
            mbar_init(&acc_full[a], 1);
            mbar_init(&acc_empty[a], 2 * EW);  // used in the leader only: the epilogue warps of both CTAs
        }
        *abort_flag = 0;
        mbar_fence_init();
    }
    if (warp == 1) tmem_alloc_pair(tmem_slot, TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    // the peer's barriers must exist before anything of this CTA signals them
    cluster_arrive_release();
    cluster_wait();
    tc_fence_after();
    const uint32_t tmem = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {
            int it = 0;
            bool ok = true;
            for (int tile = pair; ok && tile < ntiles; tile += npairs) {
                int tm, tn;
                tile_coords(tile, p.tiles_m, p.tiles_n, tm, tn);
                const int row_a = tm * PAIR_M + (int)rank * BM, row_b = tn * BN + (int)rank * HALF_N;
                for (int kb = 0; kb < nk; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (it >= STAGES && !mbar_wait(&empty[s], ((it / STAGES) - 1) & 1, actx, kErrWaitEmpty)) {
                        ok = false;
                        break;
                    }
                    if (leader) mbar_expect_tx(&full[s], 2 * STAGE_BYTES);
                    const uint32_t bar = mapa_shared(smem_u32(&full[s]), 0);
                    unsigned char* st = sm + s * STAGE_BYTES;
#pragma unroll
                    for (int x = 0; x < KBOX; ++x) {
                        tma_load_2d_pair(st + x * A_BYTES, &tm_a, bar, (kb * KBOX + x) * BK, row_a);
                        tma_load_2d_pair(st + KBOX * A_BYTES + x * B_BYTES, &tm_b, bar, (kb * KBOX + x) * BK, row_b);
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (leader && lane == 0) {
            constexpr uint32_t idesc = (KIND == gm::KIND_I8)    ? make_idesc(PAIR_M, BN, /*S32*/ 2, /*S8*/ 1, /*S8*/ 1)
                                       : (KIND == gm::KIND_F16) ? make_idesc(PAIR_M, BN, /*F32*/ 1, /*F16*/ 0, /*F16*/ 0)
                                                                : make_idesc(PAIR_M, BN, /*F32*/ 1, /*BF16*/ 1, /*BF16*/ 1);
            int it = 0, li = 0;
            bool ok = true;
            for (int tile = pair; ok && tile < ntiles; tile += npairs, ++li) {
                const int as = li & 1;
                if (li >= 2 && !mbar_wait(&acc_empty[as], ((li >> 1) - 1) & 1, actx, kErrWaitDFull)) break;
                tc_fence_after();
                const uint32_t d = tmem + (uint32_t)(as * BN);
                for (int kb = 0; kb < nk; ++kb, ++it) {
                    const int s = it % STAGES;
                    if (!mbar_wait_hot(&full[s], (it / STAGES) & 1, actx, kErrWaitFull)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
#pragma unroll
                    for (int x = 0; x < KBOX; ++x) {
                        const uint64_t da = make_sw128_kmajor_desc(smem_u32(sm + s * STAGE_BYTES + x * A_BYTES));
                        const uint64_t db = make_sw128_kmajor_desc(smem_u32(sm + s * STAGE_BYTES + KBOX * A_BYTES + x * B_BYTES));
#pragma unroll
                        for (int j = 0; j < BKB / 32; ++j) {
                            const uint32_t accumulate = (kb > 0 || x > 0 || j > 0) ? 1u : 0u;
                            if constexpr (KIND == gm::KIND_I8)
                                umma_i8_ss_pair(d, da + (uint64_t)(j * 2), db + (uint64_t)(j * 2), idesc, accumulate);
                            else
                                umma_f16_ss_pair(d, da + (uint64_t)(j * 2), db + (uint64_t)(j * 2), idesc, accumulate);
                        }
                    }
                    tc_commit_pair(&empty[s]);
                }
                if (ok) tc_commit_pair(&acc_full[as]);
            }
        }
    } else {
        const int q = warp & 3;
        int li = 0;
        for (int tile = pair; tile < ntiles; tile += npairs, ++li) {
            const int as = li & 1;
            int tm, tn;
            tile_coords(tile, p.tiles_m, p.tiles_n, tm, tn);
            bool ok = true;
            if (lane == 0) ok = mbar_wait(&acc_full[as], (li >> 1) & 1, actx, kErrWaitDFull);
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) break;
            tc_fence_after();
            const int row = tm * PAIR_M + (int)rank * BM + q * 32 + lane;
            const uint32_t lane_addr = tmem + ((uint32_t)(q * 32) << 16) + (uint32_t)(as * BN);
            constexpr int GPW = 16 / EW;  // 64-column groups per epilogue warp
            const int half = (warp - 2) >> 2;
            if (KIND != gm::KIND_I8 && p.epi == gm::EPI_ARGMAX) {
                if (half == 0) {
                float best = -INFINITY;
                int best_col = tn * BN;
#pragma unroll 1
                for (int c = 0; c < BN / 16; ++c) {
                    uint32_t v[16];
                    tmem_ld16(lane_addr + c * 16, v);
                    tc_wait_ld();
                    argmax_chunk<TOut>(p, v, tn * BN + c * 16, best, best_col);
                }
                if (row < p.M) {
                    p.part_val[(size_t)row * p.tiles_n + tn] = best;
                    p.part_idx[(size_t)row * p.tiles_n + tn] = best_col;
                }
                }
            } else {
#pragma unroll 1
                for (int gidx = half * GPW; gidx < half * GPW + GPW; ++gidx)
                    epilogue_group<KIND, TOut>(p, stg, lane_addr + gidx * 64, tm * PAIR_M + (int)rank * BM + q * 32, tn * BN + gidx * 64, lane);
            }
            tc_fence_before();
            __syncwarp();
            if (lane == 0) {
                if (leader) mbar_arrive(&acc_empty[as]);
                else mbar_arrive_cluster(mapa_shared(smem_u32(&acc_empty[as]), 0));
            }
        }
    }
    // neither CTA may free its tensor memory or leave while the other can still touch its memory
    tc_fence_before();
    __syncthreads();
    cluster_arrive_release();
    cluster_wait();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc_pair(tmem, TMEM_COLS);
    }
}

// number of SMs of the current device (cached per device; racing first callers store the same value)
static int sm_count() {
    static std::atomic<int> cache[kMaxDevices];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= kMaxDevices) return 148;
    int n = cache[dev].load(std::memory_order_relaxed);
    if (n == 0) {
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cache[dev].store(n, std::memory_order_relaxed);
    }
    return n;
}

template <int KIND, typename TOut>
static int launch_gemm(const void* a, const void* b, GemmArgs g, cudaStream_t st) {
    using namespace gm;
    constexpr int ES = (KIND == KIND_I8) ? 1 : 2;
    constexpr CUtensorMapDataType dt = (KIND == KIND_I8)    ? CU_TENSOR_MAP_DATA_TYPE_UINT8
                                       : (KIND == KIND_F16) ? CU_TENSOR_MAP_DATA_TYPE_FLOAT16
                                                            : CU_TENSOR_MAP_DATA_TYPE_BFLOAT16;
    CUtensorMap tm_a, tm_b;
    g.error = kernel_error_word();
    RWKV7_REQUIRE(g.error != nullptr, RWKV7_ERR_CUDA, "gemm: cannot resolve the device error word");
    if (g.M > BM) {
        // more than one 128-row tile: CTA pairs on 256 x 256 tiles
        if (int e = make_tmap_2d(&tm_a, dt, ES, a, g.M, g.K, gp::BM, BKB / ES, CU_TENSOR_MAP_SWIZZLE_128B)) return e;
        if (int e = make_tmap_2d(&tm_b, dt, ES, b, g.N, g.K, gp::HALF_N, BKB / ES, CU_TENSOR_MAP_SWIZZLE_128B)) return e;
        g.tiles_m = (g.M + gp::PAIR_M - 1) / gp::PAIR_M;
        g.tiles_n = (g.N + gp::BN - 1) / gp::BN;
        const long long pairs_wanted = (long long)g.tiles_m * g.tiles_n;
        const int pairs_fit = sm_count() / 2;
        const int pairs = (int)(pairs_wanted < pairs_fit ? pairs_wanted : pairs_fit);
        // up to four 128-byte K slices the tile's mainloop is shorter than its epilogue: eight epilogue warps
        if ((long long)g.K * ES <= 4 * BKB) {
            auto pk = gemm_umma_pair_kernel<KIND, TOut, 8>;
            cudaError_t pe = cudaFuncSetAttribute(pk, cudaFuncAttributeMaxDynamicSharedMemorySize, gp::smem_bytes(8));
            RWKV7_REQUIRE(pe == cudaSuccess, RWKV7_ERR_CUDA, "gemm: %s", cudaGetErrorString(pe));
            pk<<<2 * pairs, gp::threads(8), gp::smem_bytes(8), st>>>(tm_a, tm_b, g);
        } else {
            auto pk = gemm_umma_pair_kernel<KIND, TOut, 4>;
            cudaError_t pe = cudaFuncSetAttribute(pk, cudaFuncAttributeMaxDynamicSharedMemorySize, gp::smem_bytes(4));
            RWKV7_REQUIRE(pe == cudaSuccess, RWKV7_ERR_CUDA, "gemm: %s", cudaGetErrorString(pe));
            pk<<<2 * pairs, gp::threads(4), gp::smem_bytes(4), st>>>(tm_a, tm_b, g);
        }
        return check_launch("gemm_umma_pair_kernel");
    }
    if (int e = make_tmap_2d(&tm_a, dt, ES, a, g.M, g.K, BM, BKB / ES, CU_TENSOR_MAP_SWIZZLE_128B)) return e;
    if (int e = make_tmap_2d(&tm_b, dt, ES, b, g.N, g.K, BN, BKB / ES, CU_TENSOR_MAP_SWIZZLE_128B)) return e;
    g.tiles_m = (g.M + BM - 1) / BM;
    g.tiles_n = (g.N + BN - 1) / BN;
    auto kernel = gemm_umma_kernel<KIND, TOut>;
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    RWKV7_REQUIRE(e == cudaSuccess, RWKV7_ERR_CUDA, "gemm: %s", cudaGetErrorString(e));
    const long long tiles = (long long)g.tiles_m * g.tiles_n;
    const int grid = (int)(tiles < sm_count() ? tiles : sm_count());
    kernel<<<grid, THREADS, SMEM_BYTES, st>>>(tm_a, tm_b, g);
    return check_launch("gemm_umma_kernel");
}

static bool epilogue_vectorisable(const GemmArgs& g) {
    return g.N % 8 == 0 && aligned(g.C, 16) && (!g.bias || aligned(g.bias, 16)) && (!g.residual || aligned(g.residual, 16)) &&
           (!g.sw || aligned(g.sw, 16));
}

// int8 x int8 -> raw int32 accumulators.  RWKV7_ERR_UNSUPPORTED = shape / alignment not eligible (the caller falls
// back to the mma.sync kernel).
int launch_i8_gemm_umma(const int8_t* qa, const int8_t* qw, int32_t* acc, int M, int K, int Nout, cudaStream_t st) {
    if (M < 64 || K % 16 || !aligned(qa, 16) || !aligned(qw, 16) || !aligned(acc, 16)) return RWKV7_ERR_UNSUPPORTED;
    GemmArgs g{};
    g.C = acc;
    g.M = M, g.N = Nout, g.K = K;
    g.epi = gm::EPI_RAW_I32;
    g.vec = (Nout % 4 == 0);
    return launch_gemm<gm::KIND_I8, float>(qa, qw, g, st);
}

// int8 GEMM with the A8W8 dequantisation fused into its epilogue; same eligibility rule
int launch_i8_gemm_dequant_umma(const int8_t* qa, const float* sa, const int8_t* qw, const float* sw, const void* bias,
                                const void* residual, void* out, int M, int K, int Nout, int relu2, int dtype,
                                cudaStream_t st) {
    if (M < 64 || K % 16 || !aligned(qa, 16) || !aligned(qw, 16)) return RWKV7_ERR_UNSUPPORTED;
    GemmArgs g{};
    g.C = out, g.bias = bias, g.residual = residual, g.sa = sa, g.sw = sw;
    g.M = M, g.N = Nout, g.K = K;
    g.epi = gm::EPI_DEQUANT;
    g.relu2 = relu2;
    g.vec = epilogue_vectorisable(g);
    RWKV7_DISPATCH_DTYPE(dtype, T, { return launch_gemm<gm::KIND_I8, T>(qa, qw, g, st); });
    return RWKV7_OK;
}

// one CTA per row: fold the per-tile winners; among equal values the lowest column wins (torch.argmax's rule)
__global__ void __launch_bounds__(256) argmax_reduce_kernel(const float* __restrict__ part_val, const int* __restrict__ part_idx,
                                                            int tiles_n, float* __restrict__ out_val, long long* __restrict__ out_idx) {
    __shared__ float s_val[256];
    __shared__ int s_idx[256];
    const size_t row = blockIdx.x;
    float best = -INFINITY;
    int idx = 0x7fffffff;
    for (int t = threadIdx.x; t < tiles_n; t += 256) {
        const float v = part_val[row * tiles_n + t];
        const int i = part_idx[row * tiles_n + t];
        if (v > best || (v == best && i < idx)) best = v, idx = i;
    }
    s_val[threadIdx.x] = best;
    s_idx[threadIdx.x] = idx;
    __syncthreads();
    for (int w = 128; w > 0; w >>= 1) {
        if ((int)threadIdx.x < w) {
            const float v = s_val[threadIdx.x + w];
            const int i = s_idx[threadIdx.x + w];
            if (v > s_val[threadIdx.x] || (v == s_val[threadIdx.x] && i < s_idx[threadIdx.x])) s_val[threadIdx.x] = v, s_idx[threadIdx.x] = i;
        }
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        if (out_val) out_val[row] = s_val[0];
        out_idx[row] = s_idx[0];
    }
}

}  // namespace rwkv7

using namespace rwkv7;

extern "C" int64_t rwkv7_gemm_argmax_workspace_bytes(int M, int N) {
    if (M <= 0 || N <= 0) return 0;
    return (int64_t)M * ((N + gm::BN - 1) / gm::BN) * 8;
}

extern "C" int rwkv7_gemm_argmax(const void* a, const void* b, void* workspace, int64_t workspace_bytes, float* best_value,
                                 long long* best_index, int M, int K, int N, int dtype, void* stream) {
    RWKV7_REQUIRE(M > 0 && K > 0 && N > 0, RWKV7_ERR_INVALID, "gemm_argmax: sizes must be positive");
    RWKV7_REQUIRE(dtype == RWKV7_F16 || dtype == RWKV7_BF16, RWKV7_ERR_UNSUPPORTED, "gemm_argmax: fp16 or bf16 operands only");
    RWKV7_REQUIRE(K % 8 == 0, RWKV7_ERR_UNSUPPORTED, "gemm_argmax: K must be a multiple of 8 (got %d)", K);
    RWKV7_REQUIRE(a && b && workspace && best_index, RWKV7_ERR_INVALID, "gemm_argmax: null pointer");
    RWKV7_REQUIRE(aligned(a, 16) && aligned(b, 16) && aligned(workspace, 16), RWKV7_ERR_ALIGN, "gemm_argmax: operands must be 16-byte aligned");
    RWKV7_REQUIRE(workspace_bytes >= rwkv7_gemm_argmax_workspace_bytes(M, N), RWKV7_ERR_WORKSPACE,
                  "gemm_argmax: workspace of %lld bytes is smaller than the %lld required", (long long)workspace_bytes,
                  (long long)rwkv7_gemm_argmax_workspace_bytes(M, N));
    const int tiles_n = (N + gm::BN - 1) / gm::BN;
    GemmArgs g{};
    g.M = M, g.N = N, g.K = K;
    g.epi = gm::EPI_ARGMAX;
    g.part_val = reinterpret_cast<float*>(workspace);
    g.part_idx = reinterpret_cast<int*>(workspace) + (size_t)M * tiles_n;
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    int e = dtype == RWKV7_F16 ? launch_gemm<gm::KIND_F16, __half>(a, b, g, st) : launch_gemm<gm::KIND_BF16, __nv_bfloat16>(a, b, g, st);
    if (e) return e;
    argmax_reduce_kernel<<<M, 256, 0, st>>>(g.part_val, g.part_idx, tiles_n, best_value, best_index);
    return check_launch("argmax_reduce_kernel");
}

extern "C" int rwkv7_gemm(const void* a, const void* b, const void* bias, const void* residual, void* c, int M, int K,
                          int N, int epilogue, int dtype, void* stream) {
    RWKV7_REQUIRE(M > 0 && K > 0 && N > 0, RWKV7_ERR_INVALID, "gemm: sizes must be positive");
    RWKV7_REQUIRE(dtype == RWKV7_F16 || dtype == RWKV7_BF16, RWKV7_ERR_UNSUPPORTED, "gemm: fp16 or bf16 operands only");
    RWKV7_REQUIRE(K % 8 == 0, RWKV7_ERR_UNSUPPORTED, "gemm: K must be a multiple of 8 (got %d)", K);
    RWKV7_REQUIRE(a && b && c, RWKV7_ERR_INVALID, "gemm: null pointer");
    RWKV7_REQUIRE(aligned(a, 16) && aligned(b, 16), RWKV7_ERR_ALIGN, "gemm: operands must be 16-byte aligned");
    RWKV7_REQUIRE(epilogue == 0 || epilogue == 1, RWKV7_ERR_INVALID, "gemm: epilogue must be 0 (store / add) or 1 (relu^2)");
    RWKV7_REQUIRE(!(epilogue == 1 && residual), RWKV7_ERR_INVALID, "gemm: the relu^2 epilogue takes no residual");
    GemmArgs g{};
    g.C = c, g.bias = bias, g.residual = residual;
    g.M = M, g.N = N, g.K = K;
    g.epi = epilogue == 1 ? gm::EPI_RELU2 : gm::EPI_STORE;
    g.vec = epilogue_vectorisable(g);
    cudaStream_t st = static_cast<cudaStream_t>(stream);
    if (dtype == RWKV7_F16) return launch_gemm<gm::KIND_F16, __half>(a, b, g, st);
    return launch_gemm<gm::KIND_BF16, __nv_bfloat16>(a, b, g, st);
}
