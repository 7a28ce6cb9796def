// Library-wide host helpers of the C ABI: status strings, version, launch counter, SM count cache.
#include "gemm_dispatch.cuh"
#include <atomic>

namespace rg {
static std::atomic<uint64_t> g_launches{0};
void count_launch(unsigned n) { g_launches.fetch_add(n, std::memory_order_relaxed); }

int sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}
}// namespace rg

extern "C" {
const char *rg_b200_status_string(int s) {
    switch (s) {
        case RG_OK: return "ok";
        case RG_ERR_NULL: return "null pointer";
        case RG_ERR_SHAPE: return "unsupported shape";
        case RG_ERR_DTYPE: return "unsupported data type";
        case RG_ERR_ALIGN: return "misaligned pointer or stride";
        case RG_ERR_CUDA: return "CUDA error";
        case RG_ERR_TIMEOUT: return "bounded wait expired";
        case RG_ERR_UNSUPPORTED: return "no kernel for this request";
        case RG_ERR_LIMIT: return "size beyond a fixed maximum";
        default: return "unknown status";
    }
}
int rg_b200_version(void) { return 2; }
uint64_t rg_b200_launch_count(void) { return rg::g_launches.load(std::memory_order_relaxed); }
static int error_state(bool clear) {
    if (cudaDeviceSynchronize() != cudaSuccess) return -1;
    const int a = rg::linear_error_word(clear) | rg::skinny_error_word(clear), b = rg::attn_error_word(clear) | rg::attn_tc_error_word(clear), c = rg::gemm_tc_error_word(clear), d = rg::all_reduce_error_word(clear),
              e = rg::mega_error_word(clear);
    const int i0 = rg::linear_index_error_word(clear), i1 = rg::elementwise_index_error_word(clear), i2 = rg::gemm_tc_index_error_word(clear),
              i3 = rg::mega_index_error_word(clear), i4 = rg::attn_index_error_word(clear), i5 = rg::gqa_index_error_word(clear) | rg::skinny_index_error_word(clear);
    if (a < 0 || b < 0 || c < 0 || d < 0 || e < 0 || i0 < 0 || i1 < 0 || i2 < 0 || i3 < 0 || i4 < 0 || i5 < 0) return -1;
    return (a ? 1 : 0) | (b ? 2 : 0) | (c ? 4 : 0) | (d ? 8 : 0) | (e ? 16 : 0) | ((i0 | i1 | i2 | i3 | i4 | i5) ? 32 : 0);
}
int rg_b200_error_state(void) { return error_state(false); }
int rg_b200_error_clear(void) { return error_state(true) < 0 ? RG_ERR_CUDA : RG_OK; }
}
