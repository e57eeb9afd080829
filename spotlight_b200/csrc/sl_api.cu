// Error plumbing, version and workspace helpers of the C ABI.
#include <cstdlib>
#include <mutex>
#include <unordered_map>

#include "sl_common.cuh"

namespace sl {
void set_pdl(int on);

static thread_local char g_err[512] = "";

char* err_buf() { return g_err; }

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

static int g_pdl = -1;

bool pdl_enabled() {
    if (g_pdl < 0) {
        const char* e = getenv("SL_PDL");
        g_pdl = (e && e[0] == '0') ? 0 : 1;
    }
    return g_pdl != 0;
}

void set_pdl(int on) { g_pdl = on ? 1 : 0; }

static int g_l2pf = -1;

bool l2_prefetch_enabled() {
    if (g_l2pf < 0) {
        const char* e = getenv("SL_L2_PREFETCH");
        g_l2pf = (e && e[0] == '0') ? 0 : 1;
    }
    return g_l2pf != 0;
}

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

// Development switch, not part of the public header: turns programmatic dependent launch of the
// decode-path kernels on or off (default on; the environment variable SL_PDL=0 turns it off).
extern "C" void sl_debug_set_pdl(int on) { sl::set_pdl(on); }
