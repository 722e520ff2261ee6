// int8 GEMM on the 5th-generation tensor cores (tcgen05.mma kind::i8) -- placeholder
// until the kernel lands: reports "unsupported" so rwkv7_i8_gemm takes the mma.sync path.
#include "common.cuh"

namespace rwkv7 {
int launch_i8_gemm_umma(const int8_t*, const int8_t*, int32_t*, int, int, int, cudaStream_t) {
    return RWKV7_ERR_UNSUPPORTED;
}
}  // namespace rwkv7
