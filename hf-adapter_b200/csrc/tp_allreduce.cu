// Sum of the [rows, D] fp16 partial outputs of a row-sharded projection over the P GPUs of a tensor-parallel group,
// written for the decode step's payloads (0.5 - 4 MB, where a library all-reduce costs 25 - 50 us of mostly latency):
// ONE kernel per GPU, plain peer stores over NVLink into the consumer GPU's own memory, per-CTA flags, bounded waits.
//
//   every rank owns an "inbox" in peer-mapped memory: [2 buffers][P slots][slot_elems] fp16, and a flag array
//   [2][P][kMaxCtas] u32.  Call number e (counted on the device, the same on every rank because all ranks run the same
//   sequence of calls) uses buffer e & 1.  CTA c of rank r
//     1. copies its chunk of r's partial into slot r of every peer's inbox (16-byte stores to peer memory),
//     2. fences at system scope and writes e into flag [e & 1][r][c] of every peer,
//     3. waits until the flags [e & 1][s][c] in its OWN memory show e for every peer s (CTA c of rank s wrote them),
//     4. sums the P chunks in rank order (own partial + inbox slots, fp32 accumulation) and stores the fp16 result.
//   Rank order is the same everywhere, so all ranks hold bit-identical sums.  Two buffers suffice: a rank that starts
//   call e + 2 has finished call e + 1, whose wait proves that every peer had started e + 1, i.e. finished reading e.
//
// No multicast, no tensor maps over peer memory, no library kernel touches the peer pointers.  A wait that runs out
// (a peer that died or never launched) raises the device error word (rwkv7_kernel_status) and the kernel returns
// without storing; the context stays usable, the communicator state does not.
#include "umma.cuh"

namespace rwkv7 {

constexpr int kArMaxRanks = 8;
constexpr int kArMaxCtas = 64;
constexpr int kArThreads = 256;
constexpr unsigned kErrPeerWait = 7;

struct AllReduceArgs {
    const uint4* partial;            // local [rows * D / 8] vectors of 8 halves
    uint4* out;                      // local
    uint4* inbox[kArMaxRanks];       // inbox base of every rank as mapped into this process
    uint32_t* flags[kArMaxRanks];    // flag base of every rank as mapped into this process
    uint32_t* counters;              // local: [0] number of completed calls, [1] CTAs of the current call that finished
    unsigned int* error;
    int rank, world;
    long long total_vec, slot_vec;   // vectors per call / per inbox slot
    unsigned long long wait_ns;
};

__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
    uint32_t v;
    asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
    asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}

__device__ __forceinline__ void add8(float (&acc)[8], const uint4& v) {
    const __half2* h = reinterpret_cast<const __half2*>(&v);
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const float2 f = __half22float2(h[i]);
        acc[2 * i] += f.x;
        acc[2 * i + 1] += f.y;
    }
}

__global__ void __launch_bounds__(kArThreads) tp_allreduce_kernel(const AllReduceArgs p) {
    __shared__ uint32_t s_epoch;
    __shared__ int s_abort;
    const int tid = threadIdx.x, cta = blockIdx.x;
    if (tid == 0) {
        s_epoch = *reinterpret_cast<volatile uint32_t*>(p.counters) + 1u;
        s_abort = 0;
    }
    __syncthreads();
    const uint32_t e = s_epoch;
    const int buf = (int)(e & 1u);
    const long long chunk = (p.total_vec + gridDim.x - 1) / gridDim.x;
    const long long v0 = (long long)cta * chunk, v1 = min(p.total_vec, v0 + chunk);

    // 1. push this rank's chunk into slot [rank] of every peer's inbox
    for (int s = 1; s < p.world; ++s) {
        const int peer = (p.rank + s) % p.world;  // start with the next rank: the peers' links are loaded evenly
        uint4* dst = p.inbox[peer] + ((long long)buf * p.world + p.rank) * p.slot_vec;
        for (long long v = v0 + tid; v < v1; v += kArThreads) dst[v] = p.partial[v];
    }
    // 2. publish: every thread's peer stores are ordered before the flags at system scope
    __threadfence_system();
    __syncthreads();
    if (tid < p.world && tid != p.rank)
        st_release_sys(p.flags[tid] + ((long long)buf * p.world + p.rank) * kArMaxCtas + cta, e);
    // 3. wait for the same CTA of every peer (bounded)
    if (tid < p.world && tid != p.rank) {
        const uint32_t* f = p.flags[p.rank] + ((long long)buf * p.world + tid) * kArMaxCtas + cta;
        const uint64_t t0 = global_timer_ns();
        while ((int32_t)(ld_acquire_sys(f) - e) < 0) {
            if (global_timer_ns() - t0 > p.wait_ns) {
                s_abort = 1;
                atomicCAS(p.error, 0u, kErrPeerWait);
                break;
            }
            __nanosleep(64);
        }
    }
    __syncthreads();
    // 4. reduce in rank order
    if (!s_abort) {
        const uint4* mine = p.inbox[p.rank] + (long long)buf * p.world * p.slot_vec;
        for (long long v = v0 + tid; v < v1; v += kArThreads) {
            float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
            // inbox slots were written by other GPUs: read them past L1 (which is not coherent with peer writes)
            for (int s = 0; s < p.world; ++s) add8(acc, s == p.rank ? p.partial[v] : __ldcg(mine + (long long)s * p.slot_vec + v));
            uint4 o;
            __half2* h = reinterpret_cast<__half2*>(&o);
#pragma unroll
            for (int i = 0; i < 4; ++i) h[i] = __floats2half2_rn(acc[2 * i], acc[2 * i + 1]);
            p.out[v] = o;
        }
    }
    // the call counter advances when the last CTA of this launch is through (every CTA read it at its start)
    __syncthreads();
    if (tid == 0 && atomicAdd(p.counters + 1, 1u) == gridDim.x - 1) {
        p.counters[1] = 0;
        __threadfence();
        *reinterpret_cast<volatile uint32_t*>(p.counters) = e;
    }
}

}  // namespace rwkv7

using namespace rwkv7;

extern "C" int rwkv7_tp_allreduce_max_ctas(void) { return kArMaxCtas; }

extern "C" int rwkv7_tp_allreduce(const void* partial, void* out, void* const* inbox_ptrs, void* const* flag_ptrs,
                                  void* counters, int rank, int world, int rows, int D, long long slot_elems, int wait_ms,
                                  int dtype, void* stream) {
    RWKV7_REQUIRE(dtype == RWKV7_F16, RWKV7_ERR_UNSUPPORTED, "tp_allreduce: fp16 only");
    RWKV7_REQUIRE(world >= 2 && world <= kArMaxRanks && rank >= 0 && rank < world, RWKV7_ERR_INVALID,
                  "tp_allreduce: world must be 2..%d and rank inside it (world=%d rank=%d)", kArMaxRanks, world, rank);
    RWKV7_REQUIRE(rows > 0 && D > 0 && D % 8 == 0, RWKV7_ERR_UNSUPPORTED, "tp_allreduce: D must be a positive multiple of 8");
    RWKV7_REQUIRE(slot_elems % 8 == 0 && (long long)rows * D <= slot_elems, RWKV7_ERR_WORKSPACE,
                  "tp_allreduce: %d x %d values do not fit an inbox slot of %lld", rows, D, slot_elems);
    RWKV7_REQUIRE(partial && out && inbox_ptrs && flag_ptrs && counters, RWKV7_ERR_INVALID, "tp_allreduce: null pointer");
    RWKV7_REQUIRE(aligned(partial, 16) && aligned(out, 16) && aligned(counters, 8), RWKV7_ERR_ALIGN, "tp_allreduce: unaligned pointer");
    AllReduceArgs a{};
    a.partial = reinterpret_cast<const uint4*>(partial);
    a.out = reinterpret_cast<uint4*>(out);
    for (int r = 0; r < world; ++r) {
        RWKV7_REQUIRE(inbox_ptrs[r] && flag_ptrs[r] && aligned(inbox_ptrs[r], 16) && aligned(flag_ptrs[r], 4), RWKV7_ERR_INVALID,
                      "tp_allreduce: bad inbox / flag pointer of rank %d", r);
        a.inbox[r] = reinterpret_cast<uint4*>(inbox_ptrs[r]);
        a.flags[r] = reinterpret_cast<uint32_t*>(flag_ptrs[r]);
    }
    a.counters = reinterpret_cast<uint32_t*>(counters);
    a.error = kernel_error_word();
    RWKV7_REQUIRE(a.error != nullptr, RWKV7_ERR_CUDA, "tp_allreduce: cannot resolve the device error word");
    a.rank = rank;
    a.world = world;
    a.total_vec = (long long)rows * D / 8;
    a.slot_vec = slot_elems / 8;
    a.wait_ns = (unsigned long long)(wait_ms > 0 ? wait_ms : 2000) * 1000000ull;
    // the same grid on every rank: CTA c of one rank pairs with CTA c of the others
    long long ctas = a.total_vec / 1024;
    ctas = ctas < 1 ? 1 : (ctas > kArMaxCtas ? kArMaxCtas : ctas);
    tp_allreduce_kernel<<<(unsigned)ctas, kArThreads, 0, static_cast<cudaStream_t>(stream)>>>(a);
    return check_launch("tp_allreduce_kernel");
}
