// Error buffer and version of the C ABI.
#include "common.cuh"

namespace rwkv7 {
static thread_local char g_err[512] = "";
void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}
}  // namespace rwkv7

extern "C" int rwkv7_abi_version(void) { return 1; }
extern "C" const char* rwkv7_last_error(void) { return rwkv7::g_err; }
