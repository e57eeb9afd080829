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
unsigned g_peer_spin_limit = 400000u;   // polls of 100 ns: about a second (sl_configure shortens it for tests)

struct PeerArgs {
    unsigned char* base[MAX_RANKS];   // exchange buffer of every rank (own one included)
    const uint4* src;
    int R, rank;
    unsigned n16;                     // message size in 16-byte units
    unsigned long long slot_stride, flags_off;
    int* status;
    unsigned spin_limit;              // polls of a peer's flag before the wait gives up
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
            if (++it > a.spin_limit) {    // about a second by default: give up, tell the host, let the stream go on
                if (a.status) atomicExch(a.status, 3);
                break;
            }
            __nanosleep(100);
        }
    }
    __syncthreads();
}

// The second exchange of a sharded step in one launch: pack this rank's partial (o rounded to the
// run dtype as sl_sparse_attn_decode leaves it, lse in fp32) as rows*129 floats, send it to every rank
// ([rows][128] floats, then lse [rows]), and merge the R partials by log-sum-exp into out [rows][128].
// Several CTAs, MERGE_ROWS rows each: a CTA stores its rows into slot `rank` of every rank's buffer, fences at
// system scope and adds its share to an arrival counter in every buffer; when its own buffer's counter shows
// that every CTA of every rank has arrived (bounded wait), it merges its rows from the R slots. The flag area
// of such a buffer holds, after the R flag words of sl_peer_allgather (unused here): [R] launches completed,
// [R+1] arrival counter, [R+2] CTAs of the running launch that have finished.
constexpr int MERGE_ROWS = 4;      // rows per CTA: 128 threads per row
template <typename T>
__global__ void __launch_bounds__(PT) peer_merge_lse_kernel(const PeerArgs a, const T* __restrict__ o,
                                                            const float* __restrict__ lse, int rows, T* __restrict__ out) {
    sl::pdl_trigger();
    sl::pdl_wait();
    const int tid = threadIdx.x, ncta = gridDim.x;
    const int row = blockIdx.x * MERGE_ROWS + (tid >> 7), col = tid & 127;
    const bool live = row < rows;
    unsigned* own_words = reinterpret_cast<unsigned*>(a.base[a.rank] + a.flags_off) + a.R;
    const unsigned ep = __ldcg(own_words);                        // launches completed on this buffer
    if (live) {
        const float v = sl::VT<T>::to_f(o[row * 128 + col]);
        for (int r = 0; r < a.R; ++r)
            reinterpret_cast<float*>(a.base[r] + (unsigned long long)a.rank * a.slot_stride)[row * 128 + col] = v;
        if (col == 0) {
            const float l = lse[row];
            for (int r = 0; r < a.R; ++r)
                reinterpret_cast<float*>(a.base[r] + (unsigned long long)a.rank * a.slot_stride)[rows * 128 + row] = l;
        }
    }
    __syncthreads();
    if (tid == 0) {
        const unsigned share = (unsigned)(((unsigned long long)(blockIdx.x + 1) << 16) / ncta - ((unsigned long long)blockIdx.x << 16) / ncta);
        __threadfence_system();          // the CTA's stores (ordered before this by the barrier) before its arrival
        for (int r = 0; r < a.R; ++r) {
            unsigned* pf = reinterpret_cast<unsigned*>(a.base[r] + a.flags_off) + a.R + 1;
            asm volatile("red.relaxed.sys.global.add.u32 [%0], %1;" ::"l"(pf), "r"(share) : "memory");
        }
        const unsigned target = (ep + 1u) * (unsigned)a.R * 65536u;
        unsigned v = 0, it = 0;
        for (;;) {
            asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(own_words + 1) : "memory");
            if ((int)(v - target) >= 0) break;
            if (++it > a.spin_limit) {
                if (a.status) atomicExch(a.status, 3);
                break;
            }
            __nanosleep(100);
        }
    }
    __syncthreads();
    if (live) {
        const float* own = reinterpret_cast<const float*>(a.base[a.rank]);
        const long long sstr = (long long)(a.slot_stride >> 2);
        float lv[MAX_RANKS], ov[MAX_RANKS];
#pragma unroll
        for (int r = 0; r < MAX_RANKS; ++r) {                    // every load in flight at once
            lv[r] = r < a.R ? __ldcg(own + r * sstr + rows * 128 + row) : -INFINITY;
            ov[r] = r < a.R ? __ldcg(own + r * sstr + row * 128 + col) : 0.0f;
        }
        float M = -INFINITY;
#pragma unroll
        for (int r = 0; r < MAX_RANKS; ++r) M = fmaxf(M, lv[r]);
        float L = 0.0f, O = 0.0f;
        if (M != -INFINITY) {
#pragma unroll
            for (int r = 0; r < MAX_RANKS; ++r) {
                if (r < a.R) {
                    const float w = expf(lv[r] - M);
                    L += w;
                    O += w * ov[r];
                }
            }
        }
        out[row * 128 + col] = sl::VT<T>::from_f(L > 0.0f ? O / L : 0.0f);
    }
    // the last CTA to finish closes the launch: every CTA has read the launch count by now
    __syncthreads();
    if (tid == 0) {
        __threadfence();
        const unsigned old = atomicAdd(own_words + 2, 1u);
        if (old == (unsigned)ncta - 1u) {
            own_words[2] = 0u;
            own_words[0] = ep + 1u;
            __threadfence();
        }
    }
}

int fill_args(PeerArgs& a, void* const* peer_bufs, int rank, int R, size_t slot_stride, int32_t* d_status, const char* fn) {
    SL_REQUIRE(peer_bufs, SL_EINVAL, "%s: null pointer", fn);
    SL_REQUIRE(R >= 1 && R <= MAX_RANKS && rank >= 0 && rank < R, SL_EINVAL, "%s: bad rank %d of %d", fn, rank, R);
    SL_REQUIRE(slot_stride % 16 == 0, SL_ESHAPE, "%s: slot stride must be a multiple of 16 bytes", fn);
    for (int r = 0; r < R; ++r) {
        SL_REQUIRE(peer_bufs[r] != nullptr && sl::aligned16(peer_bufs[r]), SL_EINVAL, "%s: bad buffer of rank %d", fn, r);
        a.base[r] = static_cast<unsigned char*>(peer_bufs[r]);
    }
    a.R = R; a.rank = rank;
    a.slot_stride = slot_stride;
    a.flags_off = (unsigned long long)R * slot_stride;
    a.status = d_status;
    a.spin_limit = g_peer_spin_limit;
    return SL_OK;
}

}  // namespace

namespace sl { void set_peer_spin_limit(unsigned v) { g_peer_spin_limit = v; } }

extern "C" int sl_peer_merge_lse(const void* d_o, const float* d_lse, int dtype, int64_t rows, void* const* peer_bufs,
                                 int rank, int R, size_t slot_stride, void* d_out, int32_t* d_status, void* stream) {
    SL_REQUIRE(d_o && d_lse && d_out, SL_EINVAL, "sl_peer_merge_lse: null pointer");
    SL_REQUIRE(rows > 0 && rows <= (1 << 20), SL_ESHAPE, "sl_peer_merge_lse: bad row count");
    SL_REQUIRE((size_t)rows * 129 * 4 <= slot_stride, SL_ESHAPE, "sl_peer_merge_lse: slot of %zu bytes < %lld rows x 129 floats",
               slot_stride, (long long)rows);
    PeerArgs a = {};
    if (int rc = fill_args(a, peer_bufs, rank, R, slot_stride, d_status, "sl_peer_merge_lse")) return rc;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const dim3 grid((unsigned)((rows + MERGE_ROWS - 1) / MERGE_ROWS));
    switch (dtype) {
        case SL_BF16:
            SL_CUDA_OK(sl::launch_kernel(peer_merge_lse_kernel<__nv_bfloat16>, grid, dim3(PT), 0, s, false, a,
                                         static_cast<const __nv_bfloat16*>(d_o), d_lse, (int)rows, static_cast<__nv_bfloat16*>(d_out)));
            break;
        case SL_F16:
            SL_CUDA_OK(sl::launch_kernel(peer_merge_lse_kernel<__half>, grid, dim3(PT), 0, s, false, a,
                                         static_cast<const __half*>(d_o), d_lse, (int)rows, static_cast<__half*>(d_out)));
            break;
        case SL_F32:
            SL_CUDA_OK(sl::launch_kernel(peer_merge_lse_kernel<float>, grid, dim3(PT), 0, s, false, a,
                                         static_cast<const float*>(d_o), d_lse, (int)rows, static_cast<float*>(d_out)));
            break;
        default: return sl::fail(SL_EINVAL, "sl_peer_merge_lse: unsupported dtype %d", dtype);
    }
    return SL_OK;
}

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
    return (size_t)R * slot_stride + 8192;      // slots, then 8 KB of flag and epoch words
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
    a.spin_limit = g_peer_spin_limit;
    SL_CUDA_OK(sl::launch_kernel(peer_allgather_kernel, dim3(1), dim3(PT), 0, static_cast<cudaStream_t>(stream), false, a));
    return SL_OK;
}
