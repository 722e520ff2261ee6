// int8 x int8 -> int32 GEMM on the 5th-generation tensor cores (tcgen05.mma kind::i8), for the A8W8 prefill path.
//
//   C[M, N] (i32) = A[M, K] (i8, row-major) . B[N, K]^T (i8, row-major)
//
// Both operands are K-major, so TMA (128-byte swizzle, 128 k per box) lands them in shared memory exactly in the
// layout the MMA descriptors read; the accumulator tile [128 x 256] int32 lives in tensor memory; integer
// accumulation is exact, so the result is bit-identical to any correct integer GEMM (torch._int_mm in the
// reference).  CTA tile 128 x 256 x 128, 4-stage TMA ring; warp 0 = TMA producer, warp 1 = MMA issuer (one
// thread), warps 2-5 = epilogue (tensor memory -> registers -> global).  Ragged M / N / K edges are zero-filled
// by TMA and masked at the store.  All waits are bounded (umma.cuh).
#include "umma.cuh"

namespace rwkv7 {
namespace i8g {
constexpr int BM = 128, BN = 256, BK = 128, STAGES = 4, THREADS = 192;
constexpr int A_BYTES = BM * BK, B_BYTES = BN * BK, STAGE_BYTES = A_BYTES + B_BYTES;
constexpr int TMEM_COLS = 256;
constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + 256 + 1024;
}  // namespace i8g

struct I8Args {
    int32_t* C;
    int M, N, K;
    unsigned int* error;
};

__global__ void __launch_bounds__(i8g::THREADS, 1)
i8_gemm_umma_kernel(const __grid_constant__ CUtensorMap tm_a, const __grid_constant__ CUtensorMap tm_b, const I8Args p) {
    using namespace i8g;
    extern __shared__ unsigned char smem_unaligned[];
    unsigned char* sm = smem_unaligned + ((1024u - (smem_u32(smem_unaligned) & 1023u)) & 1023u);
    uint64_t* full = reinterpret_cast<uint64_t*>(sm + STAGES * STAGE_BYTES);
    uint64_t* empty = full + STAGES;
    uint64_t* d_full = empty + STAGES;
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(d_full + 1);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    const AbortCtx actx{abort_flag, p.error};

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    const int nk = (p.K + BK - 1) / BK;

    if (tid == 0) {
        tma_prefetch_desc(&tm_a);
        tma_prefetch_desc(&tm_b);
        for (int s = 0; s < STAGES; ++s) {
            mbar_init(&full[s], 1);
            mbar_init(&empty[s], 1);
        }
        mbar_init(d_full, 1);
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
            for (int i = 0; i < nk; ++i) {
                const int s = i % STAGES;
                if (i >= STAGES && !mbar_wait(&empty[s], ((i / STAGES) - 1) & 1, actx, kErrWaitEmpty)) break;
                mbar_expect_tx(&full[s], STAGE_BYTES);
                unsigned char* st = sm + s * STAGE_BYTES;
                tma_load_2d(st, &tm_a, &full[s], i * BK, m0);
                tma_load_2d(st + A_BYTES, &tm_b, &full[s], i * BK, n0);              // rows n0 .. n0+127
                tma_load_2d(st + A_BYTES + 128 * BK, &tm_b, &full[s], i * BK, n0 + 128);  // rows n0+128 .. n0+255
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            constexpr uint32_t idesc = make_idesc(BM, BN, /*S32*/ 2, /*S8*/ 1, /*S8*/ 1);
            for (int i = 0; i < nk; ++i) {
                const int s = i % STAGES;
                if (!mbar_wait_hot(&full[s], (i / STAGES) & 1, actx, kErrWaitFull)) break;
                tc_fence_after();
                const uint64_t da = make_sw128_kmajor_desc(smem_u32(sm + s * STAGE_BYTES));
                const uint64_t db = make_sw128_kmajor_desc(smem_u32(sm + s * STAGE_BYTES + A_BYTES));
#pragma unroll
                for (int j = 0; j < BK / 32; ++j)  // 32 k (= 32 bytes) per instruction
                    umma_i8_ss(tmem, da + (uint64_t)(j * 2), db + (uint64_t)(j * 2), idesc, (i > 0 || j > 0) ? 1u : 0u);
                tc_commit(&empty[s]);
            }
            tc_commit(d_full);
        }
    } else {
        const int q = warp & 3;
        const int row = m0 + q * 32 + lane;
        bool ok = true;
        if (lane == 0) ok = mbar_wait(d_full, 0, actx, kErrWaitDFull);
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (ok) {
            tc_fence_after();
            const uint32_t lane_addr = tmem + ((uint32_t)(q * 32) << 16);
            const bool vec = (p.N & 3) == 0;
#pragma unroll 1
            for (int c = 0; c < BN / 16; ++c) {
                uint32_t v[16];
                tmem_ld16(lane_addr + c * 16, v);
                tc_wait_ld();
                const int col = n0 + c * 16;
                if (row < p.M && col < p.N) {
                    int32_t* dst = p.C + (size_t)row * p.N + col;
                    if (vec && col + 16 <= p.N) {
#pragma unroll
                        for (int e = 0; e < 16; e += 4)
                            *reinterpret_cast<int4*>(dst + e) = make_int4((int)v[e], (int)v[e + 1], (int)v[e + 2], (int)v[e + 3]);
                    } else {
                        for (int e = 0; e < 16 && col + e < p.N; ++e) dst[e] = (int)v[e];
                    }
                }
            }
            tc_fence_before();
        }
    }
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem, TMEM_COLS);
    }
}

// RWKV7_ERR_UNSUPPORTED = shape / alignment not eligible (the caller falls back to the mma.sync kernel).
int launch_i8_gemm_umma(const int8_t* qa, const int8_t* qw, int32_t* acc, int M, int K, int Nout, cudaStream_t st) {
    using namespace i8g;
    if (M < 64 || K % 16 || !aligned(qa, 16) || !aligned(qw, 16) || !aligned(acc, 16)) return RWKV7_ERR_UNSUPPORTED;
    CUtensorMap tm_a, tm_b;
    if (int e = make_tmap_2d(&tm_a, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, qa, M, K, BM, BK, CU_TENSOR_MAP_SWIZZLE_128B)) return e;
    if (int e = make_tmap_2d(&tm_b, CU_TENSOR_MAP_DATA_TYPE_UINT8, 1, qw, Nout, K, 128, BK, CU_TENSOR_MAP_SWIZZLE_128B)) return e;
    I8Args a{acc, M, Nout, K, kernel_error_word()};
    RWKV7_REQUIRE(a.error != nullptr, RWKV7_ERR_CUDA, "i8_gemm: cannot resolve the device error word");
    cudaError_t e = cudaFuncSetAttribute(i8_gemm_umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, SMEM_BYTES);
    RWKV7_REQUIRE(e == cudaSuccess, RWKV7_ERR_CUDA, "i8_gemm: %s", cudaGetErrorString(e));
    dim3 grid((Nout + BN - 1) / BN, (M + BM - 1) / BM);
    i8_gemm_umma_kernel<<<grid, THREADS, SMEM_BYTES, st>>>(tm_a, tm_b, a);
    return check_launch("i8_gemm_umma_kernel");
}

}  // namespace rwkv7
