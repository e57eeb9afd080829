// Error plumbing, version and workspace helpers of the C ABI.
#include <cstdlib>
#include <mutex>
#include <unordered_map>

#include "sl_common.cuh"

namespace sl {

static thread_local char g_err[512] = "";

char* err_buf() { return g_err; }

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

static int g_pdl = 1, g_l2pf = 1, g_lru_fill = 1;

bool pdl_enabled() { return g_pdl != 0; }
bool l2_prefetch_enabled() { return g_l2pf != 0; }
bool lru_fused_fill() { return g_lru_fill != 0; }

// cudaFuncSetAttribute costs a microsecond or two; a decode loop launches thousands of kernels per
// second, so the largest dynamic shared-memory size set per (device, kernel) is remembered.
cudaError_t ensure_dyn_smem(const void* func, size_t bytes) {
    static std::mutex mu;
    static std::unordered_map<unsigned long long, size_t> seen;
    int dev = 0;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return e;
    const unsigned long long key = (unsigned long long)reinterpret_cast<uintptr_t>(func) * 64ull + (unsigned)dev;
    std::lock_guard<std::mutex> lock(mu);
    auto it = seen.find(key);
    if (it != seen.end() && it->second >= bytes) return cudaSuccess;
    e = cudaFuncSetAttribute(func, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes);
    if (e == cudaSuccess) seen[key] = bytes;
    return e;
}

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

}  // namespace sl

extern "C" int sl_version(void) { return 100; }

extern "C" int sl_set_device(int device) {
    SL_CUDA_OK(cudaSetDevice(device));
    return SL_OK;
}

extern "C" const char* sl_last_error_string(void) { return sl::err_buf(); }

extern "C" int sl_workspace_init(void* d_workspace, size_t bytes, void* stream) {
    SL_REQUIRE(d_workspace != nullptr, SL_EINVAL, "sl_workspace_init: null workspace");
    SL_CUDA_OK(cudaMemsetAsync(d_workspace, 0, bytes, static_cast<cudaStream_t>(stream)));
    return SL_OK;
}

namespace slscan { void set_scan_kernel(int v); }
namespace sl { void set_attn_warps(int v); void set_peer_spin_limit(unsigned v); void set_hash_kernel(int mode); int take_hash_status(); void set_attn_cluster(int v); int attn_cluster_capacity(int warps, int cs); void set_lru_multi(int v); }

extern "C" int sl_configure(int option, int value) {
    switch (option) {
        case SL_OPT_PDL: sl::g_pdl = value ? 1 : 0; return SL_OK;
        case SL_OPT_L2_PREFETCH: sl::g_l2pf = value ? 1 : 0; return SL_OK;
        case SL_OPT_SCAN_KERNEL:
            SL_REQUIRE(value >= 0 && value <= 2, SL_EINVAL, "sl_configure: SL_OPT_SCAN_KERNEL takes 0, 1 or 2");
            slscan::set_scan_kernel(value);
            return SL_OK;
        case SL_OPT_ATTN_WARPS:
            SL_REQUIRE(value == 0 || value == 4 || value == 8, SL_EINVAL, "sl_configure: SL_OPT_ATTN_WARPS takes 0, 4 or 8");
            sl::set_attn_warps(value);
            return SL_OK;
        case SL_OPT_PEER_SPIN_LIMIT:
            SL_REQUIRE(value >= 1, SL_EINVAL, "sl_configure: SL_OPT_PEER_SPIN_LIMIT takes a positive number of polls");
            sl::set_peer_spin_limit((unsigned)value);
            return SL_OK;
        case SL_OPT_LRU_MULTI_CTA: sl::set_lru_multi(value); return SL_OK;
        case SL_OPT_LRU_FUSED_FILL: sl::g_lru_fill = value ? 1 : 0; return SL_OK;
        case SL_OPT_ATTN_CLUSTER: sl::set_attn_cluster(value ? 1 : 0); return SL_OK;
        case SL_OPT_HASH_KERNEL:
            SL_REQUIRE(value >= 0 && value <= 2, SL_EINVAL, "sl_configure: SL_OPT_HASH_KERNEL takes 0, 1 or 2");
            sl::set_hash_kernel(value);
            return SL_OK;
        default: return sl::fail(SL_EINVAL, "sl_configure: unknown option %d", option);
    }
}

extern "C" int sl_hash_status(void) { return sl::take_hash_status(); }

extern "C" int sl_attn_cluster_capacity(int warps_per_cta, int cluster_size) {
    SL_REQUIRE(warps_per_cta == 4 || warps_per_cta == 8, SL_EINVAL, "sl_attn_cluster_capacity: warps_per_cta is 4 or 8");
    return sl::attn_cluster_capacity(warps_per_cta, cluster_size);
}
