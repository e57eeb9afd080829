// All-gather of small messages between the GPUs of one node over peer memory (NVLink), for the
// two exchanges of a sequence-sharded decode step (score histograms, attention partials). Every
// rank owns one exchange buffer
//     [R slots of slot_stride bytes][R flag words][one epoch word]
// allocated with cudaMalloc and opened by its peers through CUDA IPC. One kernel per exchange:
// every rank stores its message into slot `rank` of EVERY rank's buffer (plain peer stores),
// fences at system scope, writes its epoch into flag `rank` of every buffer, and then waits
// (bounded) until all R flags of its own buffer carry the epoch. The ranks run in lockstep, so the
// epoch is a device-side counter that every launch increments: nothing changes between launches
// and the kernel can sit in a replayed CUDA graph. A buffer is reused only after the OTHER exchange
// of the step has completed on every rank, which orders the overwrite of a slot after its readers.
// No multimem, no TMA; the ranks are different GPUs, never co-resident kernels of one GPU.
#include <cstring>

#include "sl_common.cuh"

namespace {

constexpr int MAX_RANKS = 8;
constexpr int PT = 512;

struct PeerArgs {
    unsigned char* base[MAX_RANKS];   // exchange buffer of every rank (own one included)
    const uint4* src;
    int R, rank;
    unsigned n16;                     // message size in 16-byte units
    unsigned long long slot_stride, flags_off;
    int* status;
};

__global__ void __launch_bounds__(PT) peer_allgather_kernel(const PeerArgs a) {
    __shared__ unsigned s_epoch;
    sl::pdl_trigger();
    sl::pdl_wait();                  // the message is the preceding kernel's output
    const int tid = threadIdx.x;
    for (int r = 0; r < a.R; ++r) {
        uint4* dst = reinterpret_cast<uint4*>(a.base[r] + (unsigned long long)a.rank * a.slot_stride);
        for (unsigned i = tid; i < a.n16; i += PT) dst[i] = a.src[i];
    }
    __syncthreads();
    if (tid == 0) {
        unsigned* epoch = reinterpret_cast<unsigned*>(a.base[a.rank] + a.flags_off) + a.R;
        const unsigned e = *epoch + 1u;
        *epoch = e;
        s_epoch = e;
        __threadfence_system();      // the CTA's stores (ordered before this by the barrier) before the flags
        for (int r = 0; r < a.R; ++r) {
            unsigned* pf = reinterpret_cast<unsigned*>(a.base[r] + a.flags_off) + a.rank;
            asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(pf), "r"(e) : "memory");
        }
    }
    __syncthreads();
    if (tid < a.R) {
        const unsigned e = s_epoch;
        const unsigned* lf = reinterpret_cast<const unsigned*>(a.base[a.rank] + a.flags_off) + tid;
        unsigned v = 0, it = 0;
        for (;;) {
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(lf) : "memory");
            if ((int)(v - e) >= 0) break;
            if (++it > 400000u) {    // about a second: give up, tell the host, let the stream go on
                if (a.status) atomicExch(a.status, 3);
                break;
            }
            __nanosleep(100);
        }
    }
    __syncthreads();
}

}  // namespace

extern "C" int sl_peer_alloc(size_t bytes, void** d_ptr) {
    SL_REQUIRE(d_ptr != nullptr && bytes > 0, SL_EINVAL, "sl_peer_alloc: bad arguments");
    SL_CUDA_OK(cudaMalloc(d_ptr, bytes));
    SL_CUDA_OK(cudaMemset(*d_ptr, 0, bytes));
    SL_CUDA_OK(cudaDeviceSynchronize());
    return SL_OK;
}

extern "C" int sl_peer_free(void* d_ptr) {
    if (d_ptr) SL_CUDA_OK(cudaFree(d_ptr));
    return SL_OK;
}

extern "C" int sl_peer_export(const void* d_ptr, unsigned char* handle64) {
    SL_REQUIRE(d_ptr && handle64, SL_EINVAL, "sl_peer_export: null pointer");
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    cudaIpcMemHandle_t h;
    SL_CUDA_OK(cudaIpcGetMemHandle(&h, const_cast<void*>(d_ptr)));
    memcpy(handle64, &h, 64);
    return SL_OK;
}

extern "C" int sl_peer_open(const unsigned char* handle64, void** d_ptr) {
    SL_REQUIRE(d_ptr && handle64, SL_EINVAL, "sl_peer_open: null pointer");
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, 64);
    SL_CUDA_OK(cudaIpcOpenMemHandle(d_ptr, h, cudaIpcMemLazyEnablePeerAccess));
    return SL_OK;
}

extern "C" int sl_peer_close(void* d_ptr) {
    if (d_ptr) SL_CUDA_OK(cudaIpcCloseMemHandle(d_ptr));
    return SL_OK;
}

extern "C" size_t sl_peer_buffer_bytes(int R, size_t slot_stride) {
    if (R <= 0 || R > MAX_RANKS) return 0;
    return (size_t)R * slot_stride + (size_t)(R + 1) * 4 + 60;
}

extern "C" int sl_peer_allgather(const void* d_src, size_t bytes, void* const* peer_bufs, int rank, int R,
                                 size_t slot_stride, int32_t* d_status, void* stream) {
    SL_REQUIRE(d_src && peer_bufs, SL_EINVAL, "sl_peer_allgather: null pointer");
    SL_REQUIRE(R >= 1 && R <= MAX_RANKS && rank >= 0 && rank < R, SL_EINVAL, "sl_peer_allgather: bad rank %d of %d", rank, R);
    SL_REQUIRE(bytes > 0 && bytes % 16 == 0 && bytes <= slot_stride && slot_stride % 16 == 0, SL_ESHAPE,
               "sl_peer_allgather: message of %zu bytes (slot %zu) must be a multiple of 16 bytes", bytes, slot_stride);
    SL_REQUIRE(sl::aligned16(d_src), SL_EALIGN, "sl_peer_allgather: source not 16-byte aligned");
    PeerArgs a = {};
    for (int r = 0; r < R; ++r) {
        SL_REQUIRE(peer_bufs[r] != nullptr && sl::aligned16(peer_bufs[r]), SL_EINVAL, "sl_peer_allgather: bad buffer of rank %d", r);
        a.base[r] = static_cast<unsigned char*>(peer_bufs[r]);
    }
    a.src = static_cast<const uint4*>(d_src);
    a.R = R; a.rank = rank;
    a.n16 = (unsigned)(bytes / 16);
    a.slot_stride = slot_stride;
    a.flags_off = (unsigned long long)R * slot_stride;
    a.status = d_status;
    SL_CUDA_OK(sl::launch_kernel(peer_allgather_kernel, dim3(1), dim3(PT), 0, static_cast<cudaStream_t>(stream), false, a));
    return SL_OK;
}
