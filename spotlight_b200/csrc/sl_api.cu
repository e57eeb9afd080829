// Error plumbing, version and workspace helpers of the C ABI.
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
