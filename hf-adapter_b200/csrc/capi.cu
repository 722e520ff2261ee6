// Error buffer and version of the C ABI.
#include <atomic>

#include "common.cuh"

namespace rwkv7 {
static thread_local char g_err[512] = "";
void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}
// Set (first code wins) by a tensor-core kernel whose bounded wait gave up; see umma.cuh.
__device__ unsigned int rwkv7_kernel_error = 0;

// Device address of the word on the current device.  The per-device cache is filled by whichever thread asks
// first; the slots are atomics, so two threads that race both store the same address and neither reads a torn one.
unsigned int* kernel_error_word() {
    static std::atomic<unsigned int*> cache[kMaxDevices];
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0) return nullptr;
    if (dev >= kMaxDevices) {
        set_error("device index %d is beyond the %d devices this library keeps per-device addresses for", dev, kMaxDevices);
        return nullptr;
    }
    unsigned int* p = cache[dev].load(std::memory_order_acquire);
    if (p == nullptr) {
        void* q = nullptr;
        if (cudaGetSymbolAddress(&q, rwkv7_kernel_error) != cudaSuccess) return nullptr;
        p = static_cast<unsigned int*>(q);
        cache[dev].store(p, std::memory_order_release);
    }
    return p;
}
}  // namespace rwkv7

extern "C" int rwkv7_kernel_status(int reset) {
    unsigned int v = 0;
    cudaError_t e = cudaMemcpyFromSymbol(&v, rwkv7::rwkv7_kernel_error, sizeof(v));
    if (e != cudaSuccess) {
        rwkv7::set_error("kernel_status: %s", cudaGetErrorString(e));
        return RWKV7_ERR_CUDA;
    }
    if (reset && v) {
        unsigned int z = 0;
        cudaMemcpyToSymbol(rwkv7::rwkv7_kernel_error, &z, sizeof(z));
    }
    return (int)v;
}

extern "C" int rwkv7_abi_version(void) { return 1; }
extern "C" const char* rwkv7_last_error(void) { return rwkv7::g_err; }
