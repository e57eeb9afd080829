// Code-cache build at prefill on the 5th-generation tensor cores: hash MLP 128 -> 256 -> 128 (bf16),
// sign and pack of many rows of one head per CTA. This is the one dense contraction of the retrieval path
// (reference math: spotlight/modifiers/spotlight_generation.py:229-255).
//
// One persistent CTA per SM works on 128-row tiles of one head. The head's weights stay in shared memory
// for the whole launch, transposed to K-major rows in the 128-byte-swizzled layout tcgen05.mma reads; the
// accumulators live in tensor memory (TMEM); input tiles arrive by TMA (cp.async.bulk.tensor, no multicast,
// this GPU's own memory) straight into the same swizzled layout.
//
// Two pipelines share the SM, each with 256 TMEM columns, one stage of input rows, four epilogue warps
// (a thread owns one row = one TMEM lane) and one issuing thread:
//   TMA   X tile [128 x 128]                                   -> x_full
//   MMA1  D1[128 x 256] = X W1            (8 x  M128 N256 K16)  -> d1_full   (the input stage is free again)
//   EPI1  D1 -> registers, torch's rounding points (matmul -> bf16, + bias -> bf16, SiLU -> bf16), packed
//         pairs of bf16 written back to TMEM over the columns already read: the A operand of layer 2
//                                                               -> h_full
//   MMA2  D2[128 x 128] = H W2            (16 x M128 N128 K16, A from TMEM) -> d2_full
//   EPI2  D2 -> registers, rounding points, sign bit of every value: the thread holds its row's 128 bits
//         and stores them as one 16-byte code                   -> d_free
// While one pipeline's warps are in an epilogue the tensor core runs the other's contraction. The epilogue
// (one exp and one division per hidden value on the special-function units) takes longer than the
// contraction, so the kernel is bound by it. Every wait on an mbarrier is bounded; a wait that runs out
// raises the library's hash status word, the CTA drains what it has in flight, frees its TMEM and returns.
// Same arithmetic as the warp-level kernel in sl_hash_mma.cu up to the order of the fp32 additions.
#include <cuda.h>

#include "sl_common.cuh"

namespace {

constexpr int TC_EPI_WARPS = 8;                 // 2 pipelines x 4 warps
constexpr int TC_THREADS = (TC_EPI_WARPS + 2) * 32;
constexpr int TC_TILE = 128;
constexpr unsigned W1_BYTES = 128 * 256 * 2, W2_BYTES = 256 * 128 * 2, X_BYTES = TC_TILE * 128 * 2;
constexpr unsigned OFF_W1 = 0, OFF_W2 = W1_BYTES, OFF_X = W1_BYTES + W2_BYTES, OFF_B1 = OFF_X + 2 * X_BYTES,
                   OFF_B2 = OFF_B1 + 512, OFF_BAR = OFF_B2 + 256, OFF_MISC = OFF_BAR + 2 * 5 * 8, TC_SMEM = OFF_MISC + 16 + 1024;
constexpr unsigned WAIT_FAST = 1u << 14, WAIT_LIMIT = 1u << 22;   // polls (non-blocking test_wait) without / with a 256 ns pause: about a second in all

struct HashTcArgs {
    long long T; int H; int B;
    const __nv_bfloat16* w1; const __nv_bfloat16* w2; const __nv_bfloat16* b1; const __nv_bfloat16* b2;
    uint32_t* codes; long long cs_b;
    long long tiles_per_b, n_tiles;
    int* status;                                  // mapped host word: 3 = a wait ran out
};

__device__ __forceinline__ float bfr(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }
__device__ __forceinline__ unsigned pack2(float lo, float hi) {
    return (unsigned)__bfloat16_as_ushort(__float2bfloat16_rn(lo)) | ((unsigned)__bfloat16_as_ushort(__float2bfloat16_rn(hi)) << 16);
}

// ---- mbarrier, TMA, tcgen05 in PTX
__device__ __forceinline__ void mbar_init(unsigned bar, unsigned count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_arrive(unsigned bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(bar) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(unsigned bar, unsigned bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_test(unsigned bar, unsigned parity) {
    unsigned ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
    return ok != 0;
}
// Bounded wait: false when the limit ran out or another thread of the CTA has already given up.
__device__ __forceinline__ bool mbar_wait(unsigned bar, unsigned parity, volatile int* abort_flag) {
    for (unsigned i = 0; i < WAIT_LIMIT; ++i) {
        if (mbar_test(bar, parity)) return true;
        if (i >= WAIT_FAST) {
            if (*abort_flag) return false;
            __nanosleep(256);
        }
    }
    return false;
}
__device__ __forceinline__ void tma_load_4d(unsigned dst, const CUtensorMap* map, unsigned bar, int c0, int c1, int c2, int c3) {
    asm volatile("cp.async.bulk.tensor.4d.shared::cluster.global.tile.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4, %5, %6}], [%2];"
                 ::"r"(dst), "l"(map), "r"(bar), "r"(c0), "r"(c1), "r"(c2), "r"(c3) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_commit(unsigned bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(bar) : "memory");
}
// D[tmem] (+)= A[smem] B[smem]
__device__ __forceinline__ void mma_ss(unsigned d, unsigned long long adesc, unsigned long long bdesc, unsigned idesc, unsigned acc) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                 ::"r"(d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc) : "memory");
}
// D[tmem] (+)= A[tmem] B[smem]
__device__ __forceinline__ void mma_ts(unsigned d, unsigned a, unsigned long long bdesc, unsigned idesc, unsigned acc) {
    asm volatile("{\n\t.reg .pred p;\n\tsetp.ne.b32 p, %4, 0;\n\ttcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n\t}"
                 ::"r"(d), "r"(a), "l"(bdesc), "r"(idesc), "r"(acc) : "memory");
}
__device__ __forceinline__ void tmem_ld32(unsigned taddr, unsigned (&v)[32]) {
    asm volatile("tcgen05.ld.sync.aligned.32x32b.x32.b32 {%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                 "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                 : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]),
                   "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]),
                   "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]),
                   "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                 : "r"(taddr) : "memory");
}
__device__ __forceinline__ void tmem_st16(unsigned taddr, const unsigned (&v)[16]) {
    asm volatile("tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, %16};"
                 ::"r"(taddr), "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
                   "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15]) : "memory");
}
__device__ __forceinline__ void tmem_wait_ld() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ void tmem_wait_st() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

// Shared-memory matrix descriptor: K-major rows of 128 bytes (64 bf16), 128-byte swizzle, groups of 8 rows
// 1024 bytes apart. A K step of 16 elements inside a swizzle row advances the start address by 32 bytes.
__device__ __forceinline__ unsigned long long smem_desc(unsigned addr) {
    return (unsigned long long)((addr >> 4) & 0x3fffu) | (1ull << 16) | (64ull << 32) | (1ull << 46) | (2ull << 61);
}
// Instruction descriptor: fp32 accumulators, bf16 A and B, both K-major, M = 128.
__host__ __device__ constexpr unsigned instr_desc(int n) { return (1u << 4) | (1u << 7) | (1u << 10) | ((unsigned)(n >> 3) << 17) | (8u << 24); }

// byte offset of element (row, k) of a K-major operand: slabs of 64 k, rows of 128 bytes, 16-byte chunks XORed with row % 8
__device__ __forceinline__ unsigned kmajor_off(int row, int k, int rows) {
    return (unsigned)((k >> 6) * rows * 128 + row * 128 + ((((k & 63) >> 3) ^ (row & 7)) << 4) + (k & 7) * 2);
}

__global__ void __launch_bounds__(TC_THREADS, 1) hash_encode_tc_kernel(const __grid_constant__ CUtensorMap xmap, const HashTcArgs a) {
    extern __shared__ unsigned char smem_raw[];
    const unsigned raw = (unsigned)__cvta_generic_to_shared(smem_raw);
    const unsigned base = (raw + 1023u) & ~1023u;             // operand slabs start on 1024-byte boundaries
    unsigned char* g = smem_raw + (base - raw);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int h = blockIdx.y;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(g + OFF_MISC + 4);
    unsigned* tmem_slot = reinterpret_cast<unsigned*>(g + OFF_MISC);
    auto bar = [&](int p, int i) { return base + OFF_BAR + (unsigned)(p * 5 + i) * 8u; };   // 0 x_full 1 d1_full 2 h_full 3 d2_full 4 d_free

    // ---- set-up: barriers, TMEM, this head's weights (transposed to K-major) and biases
    if (tid == 0) {
        *abort_flag = 0;
        for (int p = 0; p < 2; ++p) {
            mbar_init(bar(p, 0), 1); mbar_init(bar(p, 1), 1); mbar_init(bar(p, 2), 128); mbar_init(bar(p, 3), 1); mbar_init(bar(p, 4), 128);
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == TC_EPI_WARPS) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(base + OFF_MISC) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    {
        const unsigned* w1 = reinterpret_cast<const unsigned*>(a.w1 + (long long)h * 128 * 256);   // [k][n], pairs of n
        for (int i = tid; i < 128 * 128; i += TC_THREADS) {
            const int k = i >> 7, n = (i & 127) * 2;
            const unsigned v = w1[i];
            *reinterpret_cast<unsigned short*>(g + OFF_W1 + kmajor_off(n, k, 256)) = (unsigned short)(v & 0xffffu);
            *reinterpret_cast<unsigned short*>(g + OFF_W1 + kmajor_off(n + 1, k, 256)) = (unsigned short)(v >> 16);
        }
        const unsigned* w2 = reinterpret_cast<const unsigned*>(a.w2 + (long long)h * 256 * 128);
        for (int i = tid; i < 256 * 64; i += TC_THREADS) {
            const int k = i >> 6, n = (i & 63) * 2;
            const unsigned v = w2[i];
            *reinterpret_cast<unsigned short*>(g + OFF_W2 + kmajor_off(n, k, 128)) = (unsigned short)(v & 0xffffu);
            *reinterpret_cast<unsigned short*>(g + OFF_W2 + kmajor_off(n + 1, k, 128)) = (unsigned short)(v >> 16);
        }
        __nv_bfloat16* sb1 = reinterpret_cast<__nv_bfloat16*>(g + OFF_B1);
        __nv_bfloat16* sb2 = reinterpret_cast<__nv_bfloat16*>(g + OFF_B2);
        for (int i = tid; i < 256; i += TC_THREADS) sb1[i] = a.b1 ? a.b1[(long long)h * 256 + i] : __float2bfloat16_rn(0.0f);
        for (int i = tid; i < 128; i += TC_THREADS) sb2[i] = a.b2 ? a.b2[(long long)h * 128 + i] : __float2bfloat16_rn(0.0f);
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // the weights were written by ordinary stores, the tensor core reads them
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem = *tmem_slot;

    const int p = warp < TC_EPI_WARPS ? warp >> 2 : warp - TC_EPI_WARPS;          // pipeline of this warp
    const long long first = (long long)blockIdx.x + (long long)p * gridDim.x, step = 2ll * gridDim.x;
    bool failed = false;

    if (warp < TC_EPI_WARPS) {
        // ================= epilogue warps: thread = row = TMEM lane =================
        const int q = warp & 3, row = q * 32 + lane;
        const unsigned t_d1 = tmem + ((unsigned)(q * 32) << 16) + (unsigned)p * 256u;   // D1 columns [0,256), H over [0,128), D2 [128,256)
        const __nv_bfloat16* sb1 = reinterpret_cast<const __nv_bfloat16*>(g + OFF_B1);
        const __nv_bfloat16* sb2 = reinterpret_cast<const __nv_bfloat16*>(g + OFF_B2);
        const bool has_b1 = a.b1 != nullptr, has_b2 = a.b2 != nullptr;
        unsigned it = 0;
        for (long long tile = first; tile < a.n_tiles; tile += step, ++it) {
            const unsigned par = it & 1u;
            if (!__all_sync(0xffffffffu, mbar_wait(bar(p, 1), par, abort_flag))) { failed = true; break; }   // warp-uniform: the TMEM accesses below are warp-wide
            tc_fence_after();
#pragma unroll 1
            for (int j = 0; j < 8; ++j) {
                unsigned v[32], pk[16];
                tmem_ld32(t_d1 + 32u * j, v);
                tmem_wait_ld();
#pragma unroll
                for (int e = 0; e < 32; e += 2) {
                    float y0 = bfr(__uint_as_float(v[e])), y1 = bfr(__uint_as_float(v[e + 1]));
                    if (has_b1) {
                        y0 = bfr(y0 + __bfloat162float(sb1[32 * j + e]));
                        y1 = bfr(y1 + __bfloat162float(sb1[32 * j + e + 1]));
                    }
                    y0 = y0 / (1.0f + expf(-y0));
                    y1 = y1 / (1.0f + expf(-y1));
                    pk[e >> 1] = pack2(y0, y1);
                }
                tmem_st16(t_d1 + 16u * j, pk);
            }
            tmem_wait_st();
            tc_fence_before();
            mbar_arrive(bar(p, 2));

            if (!__all_sync(0xffffffffu, mbar_wait(bar(p, 3), par, abort_flag))) { failed = true; break; }
            tc_fence_after();
            unsigned word[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                unsigned v[32];
                tmem_ld32(t_d1 + 128u + 32u * j, v);
                tmem_wait_ld();
                unsigned bits = 0u;
#pragma unroll
                for (int e = 0; e < 32; ++e) {
                    float y = bfr(__uint_as_float(v[e]));
                    if (has_b2) y = bfr(y + __bfloat162float(sb2[32 * j + e]));
                    bits |= (y > 0.0f ? 1u : 0u) << e;
                }
                word[j] = bits;
            }
            tc_fence_before();
            mbar_arrive(bar(p, 4));
            const long long b = tile / a.tiles_per_b, t = (tile - b * a.tiles_per_b) * TC_TILE + row;
            if (t < a.T)
                *reinterpret_cast<uint4*>(a.codes + b * a.cs_b + (t * a.H + h) * 4) = make_uint4(word[0], word[1], word[2], word[3]);
        }
    } else if (lane == 0) {
        // ================= issuing thread of pipeline p: TMA loads and tensor-core instructions =================
        const unsigned x_s = base + OFF_X + (unsigned)p * X_BYTES;
        const unsigned t_d1 = tmem + (unsigned)p * 256u;
        constexpr unsigned I1 = instr_desc(256), I2 = instr_desc(128);
        bool load_pending = false;
        auto load = [&](long long tile) {
            const long long b = tile / a.tiles_per_b;
            const int t0 = (int)((tile - b * a.tiles_per_b) * TC_TILE);
            mbar_expect_tx(bar(p, 0), X_BYTES);
            tma_load_4d(x_s, &xmap, bar(p, 0), 0, t0, h, (int)b);                 // k 0..63 of the 128 rows
            tma_load_4d(x_s + X_BYTES / 2, &xmap, bar(p, 0), 64, t0, h, (int)b);  // k 64..127
            load_pending = true;
        };
        if (first < a.n_tiles) load(first);
        unsigned it = 0;
        for (long long tile = first; tile < a.n_tiles; tile += step, ++it) {
            const unsigned par = it & 1u;
            if (!mbar_wait(bar(p, 0), par, abort_flag)) { failed = true; break; }
            load_pending = false;
            if (it > 0 && !mbar_wait(bar(p, 4), par ^ 1u, abort_flag)) { failed = true; break; }   // D2 of the previous tile has been read
            tc_fence_after();
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
                const unsigned ao = (unsigned)(ks >> 2) * (X_BYTES / 2) + (unsigned)(ks & 3) * 32u;
                const unsigned bo = (unsigned)(ks >> 2) * (256u * 128u) + (unsigned)(ks & 3) * 32u;
                mma_ss(t_d1, smem_desc(x_s + ao), smem_desc(base + OFF_W1 + bo), I1, ks > 0 ? 1u : 0u);
            }
            tc_commit(bar(p, 1));
            if (!mbar_wait(bar(p, 1), par, abort_flag)) { failed = true; break; }                  // the input stage is free
            if (tile + step < a.n_tiles) load(tile + step);
            if (!mbar_wait(bar(p, 2), par, abort_flag)) { failed = true; break; }                  // H is in TMEM
            tc_fence_after();
#pragma unroll
            for (int ks = 0; ks < 16; ++ks) {
                const unsigned bo = (unsigned)(ks >> 2) * (128u * 128u) + (unsigned)(ks & 3) * 32u;
                mma_ts(t_d1 + 128u, t_d1 + 8u * ks, smem_desc(base + OFF_W2 + bo), I2, ks > 0 ? 1u : 0u);
            }
            tc_commit(bar(p, 3));
        }
        if (failed && load_pending) mbar_wait(bar(p, 0), it & 1u, abort_flag);    // a copy of ours is still in flight: let it land (bounded)
    }
    if (failed) {
        *abort_flag = 1;
        if (a.status) *reinterpret_cast<volatile int*>(a.status) = 3;
    }
    __syncwarp();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == TC_EPI_WARPS) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 512;" ::"r"(tmem) : "memory");
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = [] {
        void* p = nullptr;
        cudaDriverEntryPointQueryResult qres;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) != cudaSuccess || qres != cudaDriverEntryPointSuccess)
            p = nullptr;
        return reinterpret_cast<EncodeTiledFn>(p);
    }();
    return fn;
}

int* g_status_host = nullptr;     // one mapped host word for the process: any device may raise it
int g_hash_kernel = 0;            // 0 by shape, 1 warp-level kernel only, 2 this kernel whenever it covers the shape

}  // namespace

namespace sl {

void set_hash_kernel(int mode) { g_hash_kernel = mode; }

// Returns the hash status word (0, or 3 after a device-side wait ran out) and clears it. The caller synchronises first.
int take_hash_status() {
    if (!g_status_host) return 0;
    const int v = *reinterpret_cast<volatile int*>(g_status_host);
    *reinterpret_cast<volatile int*>(g_status_host) = 0;
    return v;
}

// Returns SL_OK after launching, 1 when the shape is not one this kernel covers (the caller falls through to the
// warp-level kernel), or an error code.
int launch_hash_encode_tc(const void* x, long long xs_b, long long xs_tok, long long xs_h, int B, long long T, int H, const sl_hash_params* hp,
                          uint32_t* codes, long long cs_b, cudaStream_t s) {
    if (g_hash_kernel == 1) return 1;
    if (hp->n_layers != 2 || hp->dims[0] != 128 || hp->dims[1] != 256 || hp->dims[2] != 128 || hp->residue) return 1;
    if (H > 65535 || B > 65535 || T > 0x7fffff00ll) return 1;
    if (g_hash_kernel == 0 && (long long)B * T * H < 32768) return 1;           // too few tiles to pay for the set-up
    if (!sl::aligned16(x) || !sl::aligned16(codes) || cs_b % 4 != 0) return 1;
    if (xs_tok % 8 != 0 || xs_h % 8 != 0 || (B > 1 && (xs_b % 8 != 0 || xs_b <= 0))) return 1;
    EncodeTiledFn enc = encode_fn();
    if (!enc) return 1;
    if (!g_status_host) {
        int* p = nullptr;
        if (cudaHostAlloc(reinterpret_cast<void**>(&p), sizeof(int), cudaHostAllocMapped | cudaHostAllocPortable) != cudaSuccess) { cudaGetLastError(); return 1; }
        *p = 0;
        g_status_host = p;
    }
    int* d_status = nullptr;
    if (cudaHostGetDevicePointer(reinterpret_cast<void**>(&d_status), g_status_host, 0) != cudaSuccess) { cudaGetLastError(); return 1; }

    CUtensorMap map;
    const cuuint64_t gdim[4] = {128, (cuuint64_t)T, (cuuint64_t)H, (cuuint64_t)B};
    const cuuint64_t gstr[3] = {(cuuint64_t)xs_tok * 2, (cuuint64_t)xs_h * 2, (cuuint64_t)(B > 1 ? xs_b : (long long)T * xs_tok) * 2};
    const cuuint32_t box[4] = {64, TC_TILE, 1, 1}, estr[4] = {1, 1, 1, 1};
    if (enc(&map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(x), gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
            CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS)
        return 1;

    HashTcArgs a = {};
    a.T = T; a.H = H; a.B = B;
    a.w1 = static_cast<const __nv_bfloat16*>(hp->d_w[0]); a.w2 = static_cast<const __nv_bfloat16*>(hp->d_w[1]);
    a.b1 = static_cast<const __nv_bfloat16*>(hp->d_b[0]); a.b2 = static_cast<const __nv_bfloat16*>(hp->d_b[1]);
    a.codes = codes; a.cs_b = cs_b;
    a.tiles_per_b = (T + TC_TILE - 1) / TC_TILE;
    a.n_tiles = a.tiles_per_b * B;
    a.status = d_status;
    SL_CUDA_OK(cudaFuncSetAttribute(hash_encode_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TC_SMEM));
    const long long per_head = std::max<long long>(1, (long long)sl::sm_count() / H);
    const unsigned gx = (unsigned)std::min<long long>(a.n_tiles, per_head);
    hash_encode_tc_kernel<<<dim3(gx, (unsigned)H), TC_THREADS, TC_SMEM, s>>>(map, a);
    SL_CUDA_OK(cudaGetLastError());
    return SL_OK;
}

}  // namespace sl
