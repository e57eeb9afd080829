// Shared host/device helpers of libspotlight_b200 (sm_100a only).
#pragma once
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include <cstdarg>
#include <cstdio>
#include <algorithm>

#include "../../include/spotlight_b200.h"

namespace sl {

// ---- host-side error plumbing ---------------------------------------------------------
char* err_buf();
int fail(int code, const char* fmt, ...);
int sm_count();          // SMs of the current device (cached per device)
cudaError_t ensure_dyn_smem(const void* func, size_t bytes);   // opt-in to `bytes` of dynamic shared memory, once
bool pdl_enabled();      // programmatic dependent launch on (default) / off (sl_configure)
bool l2_prefetch_enabled();   // the decode-step hash warms L2 with the code cache (sl_configure)
bool lru_fused_fill();        // the decode step lets the attention launch fetch and fill the LRU misses (sl_configure)

#define SL_CUDA_OK(expr)                                                                    \
    do {                                                                                    \
        cudaError_t e__ = (expr);                                                           \
        if (e__ != cudaSuccess)                                                             \
            return sl::fail(SL_ECUDA, "%s failed: %s", #expr, cudaGetErrorString(e__));     \
    } while (0)

#define SL_REQUIRE(cond, code, ...)                                                         \
    do {                                                                                    \
        if (!(cond)) return sl::fail(code, __VA_ARGS__);                                    \
    } while (0)

static inline bool aligned16(const void* p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

// ---- entry points with a device-side position (one captured launch serves every decode token) ----
struct DevPos {
    const long long* d_pos;        // position of the decode token; the context is *d_pos + 1 keys
    const void* cos_tab;           // [rows,128] of the run dtype, row r = position tab_pos0 + r (or null: no rotation)
    const void* sin_tab;
    long long tab_pos0;
};
int scan_topk_impl(const uint32_t* d_q_codes, const uint32_t* d_k_codes, int64_t k_batch_stride, int B, int64_t N,
                   int KH, int QH, int gqa_layout, int k, int sink, int recent, int32_t* d_idx, int idx_capacity,
                   int32_t* d_cnt, int16_t* d_scores_out, void* d_workspace, size_t workspace_bytes,
                   int32_t* d_status, const long long* d_pos, double mask_out, int min_remain, void* stream);
int decode_prepare_impl(const void* d_q, const void* d_k, const void* d_v, int dtype, int B, int QH, int KH,
                        const void* d_cos, const void* d_sin, const sl_hash_params* hash_q, const sl_hash_params* hash_k,
                        void* d_q_rot, uint32_t* d_q_codes, uint32_t* d_code_cache, int64_t code_batch_stride,
                        void* d_k_cache, void* d_v_cache, const sl_kv_layout* kv, int64_t pos, const DevPos* dp,
                        void* stream);

// ---- launches ----------------------------------------------------------------------------
// Kernels of the decode path are launched with programmatic stream serialisation: a kernel may
// start while its predecessor in the stream drains, does whatever does not depend on it, and
// blocks in pdl_wait() until the predecessor has completed and flushed. Every such kernel
// executes pdl_wait() on every path before it touches data other kernels produce or consume, so
// completion stays transitive along the stream. pdl_trigger() lets the successor begin.
template <typename... KArgs, typename... Args>
inline cudaError_t launch_kernel(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t s,
                                 bool cooperative, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = s;
    cudaLaunchAttribute attrs[2];
    unsigned n = 0;
    if (pdl_enabled()) {
        attrs[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attrs[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    if (cooperative) {
        attrs[n].id = cudaLaunchAttributeCooperative;
        attrs[n].val.cooperative = 1;
        ++n;
    }
    cfg.attrs = attrs; cfg.numAttrs = n;
    return cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
}

// ---- device helpers -------------------------------------------------------------------
__device__ __forceinline__ void pdl_trigger() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }
__device__ __forceinline__ void pdl_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
// Streaming 128-bit load that bypasses L1 allocation: the code stream is read once.
__device__ __forceinline__ uint4 ld_stream_v4(const uint4* p) {
    uint4 r;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
                 : "l"(p));
    return r;
}
// Gathered 128-bit load (rows are touched once per launch; keep them out of L1).
__device__ __forceinline__ uint4 ld_gather_v4(const void* p) {
    uint4 r;
    asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
                 : "l"(p));
    return r;
}
__device__ __forceinline__ unsigned ld_acquire_u32(const unsigned* p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}
__device__ __forceinline__ void red_release_add_u32(unsigned* p, unsigned v) {
    asm volatile("red.release.gpu.global.add.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ int popc4(uint4 a) {
    return __popc(a.x) + __popc(a.y) + __popc(a.z) + __popc(a.w);
}
__device__ __forceinline__ uint4 xor4(uint4 a, uint4 b) {
    return make_uint4(a.x ^ b.x, a.y ^ b.y, a.z ^ b.z, a.w ^ b.w);
}

// value type traits: load/round in the run dtype
template <typename T> struct VT;
template <> struct VT<__nv_bfloat16> {
    static __device__ __forceinline__ float to_f(__nv_bfloat16 v) { return __bfloat162float(v); }
    static __device__ __forceinline__ __nv_bfloat16 from_f(float f) { return __float2bfloat16_rn(f); }
    static __device__ __forceinline__ float round(float f) { return __bfloat162float(__float2bfloat16_rn(f)); }
};
template <> struct VT<__half> {
    static __device__ __forceinline__ float to_f(__half v) { return __half2float(v); }
    static __device__ __forceinline__ __half from_f(float f) { return __float2half_rn(f); }
    static __device__ __forceinline__ float round(float f) { return __half2float(__float2half_rn(f)); }
};
template <> struct VT<float> {
    static __device__ __forceinline__ float to_f(float v) { return v; }
    static __device__ __forceinline__ float from_f(float f) { return f; }
    static __device__ __forceinline__ float round(float f) { return f; }
};

// A bounded grid-wide barrier over `n_ctas` co-resident CTAs. `counter` counts arrivals and
// only grows during a launch (target of the j-th barrier is (j+1)*n_ctas). Thread 0 fences
// (ordering the CTA's earlier global writes, which the bar.sync made visible to it), arrives
// with a relaxed add, polls with relaxed loads and fences again once the poll has succeeded; data
// published before the barrier is read with L2-coherent loads (__ldcg) after it. Measured on B200: ~1.2 us, against ~1.5 us
// for the release-add / acquire-poll form. Gives up after `limit` polls, sets *status and
// returns false; callers carry on with bounded work.
__device__ __forceinline__ bool grid_barrier(unsigned* counter, unsigned target, int* status,
                                             unsigned limit = 4000000u) {
    __shared__ int ok_s;
    __syncthreads();
    if (threadIdx.x == 0) {
        __threadfence();
        asm volatile("red.relaxed.gpu.global.add.u32 [%0], %1;" ::"l"(counter), "r"(1u) : "memory");
        unsigned it = 0, v;
        int ok = 1;
        for (;;) {
            asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(counter) : "memory");
            if (v >= target) break;
            if (++it > limit) { ok = 0; break; }
        }
        __threadfence();     // acquire side: the CTA's later reads are ordered after the successful poll
        if (!ok && status) atomicExch(status, 1);
        ok_s = ok;
    }
    __syncthreads();
    return ok_s != 0;
}

}  // namespace sl
