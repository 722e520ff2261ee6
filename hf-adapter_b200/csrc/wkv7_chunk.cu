// Chunked (WY / DPLR) WKV-7 scan on tensor cores -- placeholder until the kernel lands.
#include "common.cuh"

extern "C" int rwkv7_wkv7_chunk_scan(const void*, const void*, const void*, const void*, const void*, const void*,
                                     const float*, float*, void*, int, int, int, int, int, int, int, void*) {
    rwkv7::set_error("wkv7_chunk_scan: not built in this library version");
    return RWKV7_ERR_UNSUPPORTED;
}
