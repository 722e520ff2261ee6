// Blackwell (sm_100a) building blocks used by the tensor-core kernels: mbarriers with BOUNDED waits,
// TMA tensor maps and tiled bulk copies, tensor-memory allocation, tcgen05.mma / ld / st / commit,
// and the shared-memory / instruction descriptors.  Bit layouts follow the PTX ISA tables for
// tcgen05 matrix descriptors (checked against the field definitions in CUTLASS's
// cute/arch/mma_sm100_desc.hpp).
//
// Every wait has an iteration cap.  A wait that gives up records a code in the device-side error
// word (readable through rwkv7_kernel_status) and sets a CTA-wide abort flag;
// all later waits of the CTA return immediately, the kernel skips its stores, releases tensor
// memory and returns, so the context stays usable.
#pragma once

#include <cuda.h>

#include "common.cuh"

namespace rwkv7 {

// error codes written to the device error word
enum : unsigned {
    kErrWaitFull = 1, kErrWaitEmpty = 2, kErrWaitAReady = 3, kErrWaitAFree = 4, kErrWaitDFull = 5, kErrWaitOther = 6
};
// Host: device address of the error word of the current device (capi.cu); passed to kernels as an argument
// because device symbols are private to their translation unit without relocatable device code.
unsigned int* kernel_error_word();

struct AbortCtx {
    volatile int* flag;   // CTA-wide abort flag in shared memory
    unsigned int* error;  // device-global error word
};


__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

// ---------------------------------------------------------------- mbarrier
__device__ __forceinline__ void mbar_init(uint64_t* bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_fence_init() { asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory"); }
__device__ __forceinline__ void mbar_arrive(uint64_t* bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t* bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// try_wait with a suspend-time hint: the hardware parks the thread until the phase completes (or the hint runs out), so
// a waiting warp issues no instructions.  Spinning on plain try_wait instead more than doubled the instruction count
// of the int4 kernel and competed with its dequantising warps for the integer pipe.
__device__ __forceinline__ bool mbar_try_wait(uint64_t* bar, uint32_t parity, uint32_t suspend_ns) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity), "r"(suspend_ns) : "memory");
    return ok != 0;
}
__device__ __forceinline__ uint64_t global_timer_ns() {
    uint64_t t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
// Non-blocking test of a phase.  On a phase that has already completed this returns in about 20 cycles, while
// try_wait with a suspend-time hint takes 50 (175 when one lane polls and the warp then reconverges on a shuffle),
// measured on one idle SM: every wait below tests first and only parks when the phase is still open.
__device__ __forceinline__ bool mbar_test_wait(uint64_t* bar, uint32_t parity) {
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.b32 %0, 1, 0, p;\n\t}"
        : "=r"(ok) : "r"(smem_u32(bar)), "r"(parity) : "memory");
    return ok != 0;
}
constexpr uint32_t kSuspendNs = 20000;            // per try_wait
constexpr uint64_t kWaitLimitNs = 2000000000ull;  // a wait gives up after two seconds

// Bounded wait.  Returns false (and raises the CTA abort flag) if the phase never completes.
__device__ __forceinline__ bool mbar_wait(uint64_t* bar, uint32_t parity, const AbortCtx& ctx, unsigned code) {
    if (mbar_test_wait(bar, parity)) return true;
    if (*ctx.flag) return false;  // the CTA is already giving up: do not park
    if (mbar_try_wait(bar, parity, kSuspendNs)) return true;
    const uint64_t t0 = global_timer_ns();
    for (;;) {
        if (mbar_try_wait(bar, parity, kSuspendNs)) return true;
        if (*ctx.flag) return false;
        if (global_timer_ns() - t0 > kWaitLimitNs) break;
    }
    *ctx.flag = 1;
    atomicCAS(ctx.error, 0u, code);
    return false;
}

// Kept as a separate name for the threads whose wake-up latency is on the critical path (MMA issuers).
__device__ __forceinline__ bool mbar_wait_hot(uint64_t* bar, uint32_t parity, const AbortCtx& ctx, unsigned code) {
    return mbar_wait(bar, parity, ctx, code);
}

// ---------------------------------------------------------------- cluster barrier, split into arrive / wait
// Every thread of every CTA of the cluster runs arrive and wait alternately, the same number of times.
__device__ __forceinline__ void cluster_arrive_relaxed() { asm volatile("barrier.cluster.arrive.relaxed;" ::: "memory"); }
__device__ __forceinline__ void cluster_arrive_release() { asm volatile("barrier.cluster.arrive.release;" ::: "memory"); }
__device__ __forceinline__ void cluster_wait() { asm volatile("barrier.cluster.wait.acquire;" ::: "memory"); }

// ---------------------------------------------------------------- TMA
__device__ __forceinline__ void tma_load_2d(void* smem_dst, const CUtensorMap* tmap, uint64_t* bar, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(tmap), "r"(smem_u32(bar)), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tma_load_3d(void* smem_dst, const CUtensorMap* tmap, uint64_t* bar, int c0, int c1, int c2) {
    asm volatile(
        "cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(tmap), "r"(smem_u32(bar)), "r"(c0), "r"(c1), "r"(c2) : "memory");
}
__device__ __forceinline__ void tma_prefetch_desc(const CUtensorMap* tmap) {
    asm volatile("prefetch.tensormap [%0];" ::"l"(tmap) : "memory");
}
__device__ __forceinline__ void fence_proxy_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }

// ---------------------------------------------------------------- tensor memory
__device__ __forceinline__ void tmem_alloc(uint32_t* smem_slot, uint32_t ncols) {  // one full warp
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_slot)), "r"(ncols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t ncols) {  // the same full warp
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(uint64_t* bar) {  // one thread
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}

// 16 consecutive 32-bit columns of this thread's TMEM lane
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};"
        ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]),
          "r"(v[8]), "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]) : "memory");
}
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, uint32_t (&v)[16]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x16.b32 {%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
          "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15])
        : "r"(taddr) : "memory");
}

// 64 consecutive 32-bit columns of this thread's TMEM lane in one instruction (one wait instead of four)
__device__ __forceinline__ void tmem_ld64(uint32_t taddr, uint32_t (&v)[64]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x64.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31,"
        "%32,%33,%34,%35,%36,%37,%38,%39,%40,%41,%42,%43,%44,%45,%46,%47,%48,%49,%50,%51,%52,%53,%54,%55,%56,%57,%58,%59,%60,%61,%62,%63}, [%64];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
          "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]),
          "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]),
          "=r"(v[30]), "=r"(v[31]), "=r"(v[32]), "=r"(v[33]), "=r"(v[34]), "=r"(v[35]), "=r"(v[36]), "=r"(v[37]), "=r"(v[38]), "=r"(v[39]),
          "=r"(v[40]), "=r"(v[41]), "=r"(v[42]), "=r"(v[43]), "=r"(v[44]), "=r"(v[45]), "=r"(v[46]), "=r"(v[47]), "=r"(v[48]), "=r"(v[49]),
          "=r"(v[50]), "=r"(v[51]), "=r"(v[52]), "=r"(v[53]), "=r"(v[54]), "=r"(v[55]), "=r"(v[56]), "=r"(v[57]), "=r"(v[58]), "=r"(v[59]),
          "=r"(v[60]), "=r"(v[61]), "=r"(v[62]), "=r"(v[63])
        : "r"(taddr) : "memory");
}

// ---------------------------------------------------------------- CTA pairs (cta_group::2)
// Two CTAs of a cluster (ranks 2i and 2i + 1) work on one 256-row tile: the even ("leader") CTA issues the MMAs,
// each CTA stages its own 128 rows of A and its half of B, and each CTA's tensor memory receives its own 128
// rows of the result.  Every tcgen05 instruction with a cta_group qualifier in such a kernel uses cta_group::2.
__device__ __forceinline__ uint32_t cluster_ctarank() {
    uint32_t r;
    asm volatile("mov.u32 %0, %%cluster_ctarank;" : "=r"(r));
    return r;
}
// shared::cluster address of the location `smem_addr` (a shared::cta address of this CTA) inside CTA `rank`
__device__ __forceinline__ uint32_t mapa_shared(uint32_t smem_addr, uint32_t rank) {
    uint32_t r;
    asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(smem_addr), "r"(rank));
    return r;
}
__device__ __forceinline__ void mbar_arrive_cluster(uint32_t bar_cluster_addr) {
    asm volatile("mbarrier.arrive.release.cluster.shared::cluster.b64 _, [%0];" ::"r"(bar_cluster_addr) : "memory");
}
// TMA load (no multicast) whose completion is signalled on a barrier that may live in the peer CTA of the pair
__device__ __forceinline__ void tma_load_2d_pair(void* smem_dst, const CUtensorMap* tmap, uint32_t bar_cluster_addr, int c0, int c1) {
    asm volatile(
        "cp.async.bulk.tensor.2d.cta_group::2.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];"
        ::"r"(smem_u32(smem_dst)), "l"(tmap), "r"(bar_cluster_addr), "r"(c0), "r"(c1) : "memory");
}
__device__ __forceinline__ void tmem_alloc_pair(uint32_t* smem_slot, uint32_t ncols) {  // one full warp in EACH CTA of the pair
    asm volatile("tcgen05.alloc.cta_group::2.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_slot)), "r"(ncols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::2.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc_pair(uint32_t taddr, uint32_t ncols) {  // the same warps
    asm volatile("tcgen05.dealloc.cta_group::2.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(ncols) : "memory");
}
// arrive on the barrier at this shared-memory offset in BOTH CTAs of the pair once the MMAs issued so far are done
__device__ __forceinline__ void tc_commit_pair(uint64_t* bar) {  // one thread of the leader CTA
    const uint16_t mask = 3;
    asm volatile("tcgen05.commit.cta_group::2.mbarrier::arrive::one.shared::cluster.multicast::cluster.b64 [%0], %1;"
                 ::"r"(smem_u32(bar)), "h"(mask) : "memory");
}
__device__ __forceinline__ void umma_f16_ss_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_i8_ss_pair(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::2.kind::i8 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}

// ---------------------------------------------------------------- descriptors
// Shared-memory matrix descriptor for a K-major operand tile stored as rows of 128 bytes with the
// 128-byte swizzle (what a TMA box of 64 x 16-bit / 128 x 8-bit inner elements produces): 8-row
// groups are 1024 bytes apart (stride byte offset), the leading byte offset is unused for swizzled
// K-major layouts, descriptor version 1 (Blackwell), layout type 2 (SWIZZLE_128B).
__device__ __forceinline__ uint64_t make_sw128_kmajor_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);       // [0,14)  start address
    d |= (uint64_t)1 << 16;                            // [16,30) leading byte offset (ignored) = 16 B
    d |= (uint64_t)(1024 >> 4) << 32;                  // [32,46) stride byte offset = 1024 B
    d |= (uint64_t)1 << 46;                            // [46,48) descriptor version
    d |= (uint64_t)2 << 61;                            // [61,64) SWIZZLE_128B
    return d;
}

// Instruction descriptor for kind::f16 / kind::i8 (dense, no negate, K-major A and B).
//   c_format: 1 = F32, 2 = S32; a/b format: f16 kind 0 = F16, 1 = BF16; tf32 kind 2 = TF32; i8 kind 0 = U8, 1 = S8.
__host__ __device__ constexpr uint32_t make_idesc(int M, int N, int c_format, int a_format, int b_format) {
    return ((uint32_t)c_format << 4) | ((uint32_t)a_format << 7) | ((uint32_t)b_format << 10) |
           ((uint32_t)(N >> 3) << 17) | ((uint32_t)(M >> 4) << 24);
}

// D[tmem] (+)= A[tmem] . B[smem]   (A from tensor memory)
__device__ __forceinline__ void umma_f16_ts(uint32_t d_tmem, uint32_t a_tmem, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
        ::"r"(d_tmem), "r"(a_tmem), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
// D[tmem] (+)= A[smem] . B[smem]
__device__ __forceinline__ void umma_f16_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_tf32_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}
__device__ __forceinline__ void umma_i8_ss(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(d_tmem), "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate) : "memory");
}

// Byte offset of element (row, byte position kbyte along K) inside a K-major SWIZZLE_128B tile of `rows` rows:
// the tile is a sequence of 128-byte-wide "atoms" along K (rows*128 bytes each); inside an atom the 16-byte chunk
// index is XORed with (row & 7).  This is the layout make_sw128_kmajor_desc describes.
__device__ __forceinline__ uint32_t sw128_offset(uint32_t row, uint32_t kbyte, uint32_t rows) {
    const uint32_t atom = kbyte >> 7, inb = kbyte & 127u;
    return atom * rows * 128u + row * 128u + ((((inb >> 4) ^ (row & 7u)) << 4) | (inb & 15u));
}

// ---------------------------------------------------------------- host: tensor maps
// cuTensorMapEncodeTiled is resolved through the runtime so the library has no link-time
// dependency on libcuda (it must load on machines without a driver).
typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline EncodeTiledFn get_encode_tiled() {
    static EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) != cudaSuccess) return (EncodeTiledFn) nullptr;
        return (EncodeTiledFn)p;
    }();
    return fn;
}

// 2-D row-major tensor [rows, cols] of `elem_bytes`-byte elements; box = [box_rows, box_cols].
inline int make_tmap_2d(CUtensorMap* map, CUtensorMapDataType dt, int elem_bytes, const void* base, uint64_t rows, uint64_t cols,
                        uint32_t box_rows, uint32_t box_cols, CUtensorMapSwizzle swz) {
    EncodeTiledFn fn = get_encode_tiled();
    if (!fn) {
        set_error("cuTensorMapEncodeTiled is unavailable (no CUDA driver?)");
        return RWKV7_ERR_CUDA;
    }
    cuuint64_t dims[2] = {cols, rows};
    cuuint64_t strides[1] = {cols * (uint64_t)elem_bytes};
    cuuint32_t box[2] = {box_cols, box_rows};
    cuuint32_t estr[2] = {1, 1};
    CUresult r = fn(map, dt, 2, const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, swz,
                    CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_error("cuTensorMapEncodeTiled failed with code %d (rows=%llu cols=%llu box=%ux%u)", (int)r,
                  (unsigned long long)rows, (unsigned long long)cols, box_rows, box_cols);
        return RWKV7_ERR_CUDA;
    }
    return RWKV7_OK;
}

// fp16 activations x[rows, K] viewed as (k_in = 64, row, k_out = K/64) so that ONE box {64, box_rows, 2} lands two
// consecutive 64-k swizzle atoms [k_out][row][128 B] -- the K-major SW128 operand layout for 128 k.
inline int make_tmap_x3d(CUtensorMap* map, const void* base, uint64_t rows, uint64_t K, uint32_t box_rows) {
    EncodeTiledFn fn = get_encode_tiled();
    if (!fn) {
        set_error("cuTensorMapEncodeTiled is unavailable (no CUDA driver?)");
        return RWKV7_ERR_CUDA;
    }
    cuuint64_t dims[3] = {64, rows, K / 64};
    cuuint64_t strides[2] = {K * 2, 128};
    cuuint32_t box[3] = {64, box_rows, 2};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3, const_cast<void*>(base), dims, strides, box, estr,
                    CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                    CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_error("cuTensorMapEncodeTiled (3-D activation map) failed with code %d (rows=%llu K=%llu)", (int)r,
                  (unsigned long long)rows, (unsigned long long)K);
        return RWKV7_ERR_CUDA;
    }
    return RWKV7_OK;
}

// Token vectors [tokens, H, 64] of 2- or 4-byte elements viewed as (64 channels, H, tokens): a box {64, 1, 64} at
// (0, h, t0) lands the 64-token slice of one head densely ([token][channel], no swizzle).
inline int make_tmap_tokens(CUtensorMap* map, const void* base, int elem_bytes, uint64_t tokens, uint64_t H) {
    EncodeTiledFn fn = get_encode_tiled();
    if (!fn) {
        set_error("cuTensorMapEncodeTiled is unavailable (no CUDA driver?)");
        return RWKV7_ERR_CUDA;
    }
    cuuint64_t dims[3] = {64, H, tokens};
    cuuint64_t strides[2] = {(cuuint64_t)64 * elem_bytes, (cuuint64_t)64 * elem_bytes * H};
    cuuint32_t box[3] = {64, 1, 64};
    cuuint32_t estr[3] = {1, 1, 1};
    CUresult r = fn(map, elem_bytes == 4 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 3,
                    const_cast<void*>(base), dims, strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                    CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_error("cuTensorMapEncodeTiled (token map) failed with code %d (tokens=%llu H=%llu)", (int)r,
                  (unsigned long long)tokens, (unsigned long long)H);
        return RWKV7_ERR_CUDA;
    }
    return RWKV7_OK;
}

}  // namespace rwkv7
