// Code-cache build at prefill on the 5th-generation tensor cores: hash MLP 128 -> {256, 128} -> 128 (the narrow one also
// in the reference's residual form) and linear hash 128 -> 128 (bf16),
// sign and pack of many rows of one head per CTA. This is the one dense contraction of the retrieval path
// (reference math: spotlight/modifiers/spotlight_generation.py:229-255).
//
// One persistent CTA per SM works on 128-row tiles of one head, one tile after the other. The head's weights stay in shared memory
// for the whole launch, transposed to K-major rows in the 128-byte-swizzled layout tcgen05.mma reads; the
// accumulators live in tensor memory (TMEM); input tiles arrive by TMA (cp.async.bulk.tensor, one CTA per copy,
// this GPU's own memory) straight into the same swizzled layout.
//
// The MLP kernel (written for a hidden width D1 of 256; 128 halves the pieces). TMEM columns: D1 [0,D1) fp32, H [256,256+D1/2)
// packed bf16 pairs, D2 [384,512) fp32. Sixteen epilogue warps (a thread owns one row = one TMEM lane and a quarter
// of the columns) and one issuing thread:
//   TMA   X tile [128 x 128] into one of two stages            -> x_full[stage]
//   MMA1  D1[128 x D1] = X W1             (8 x  M128 N=D1 K16)  -> d1_full
//   EPI1  D1 -> registers, torch's rounding points (matmul -> bf16, + bias -> bf16, SiLU -> bf16, + input -> bf16 in the
//         residual form), packed pairs of bf16 written to H: the A operand of layer 2
//                                                               -> h_full, h_full2 (a warp's columns in two halves:
//         MMA2 starts on the first; after the second D1 is free and the input stage takes the next rows; MMA1 of the
//         next tile, issued behind MMA2 of this one, runs under EPI2)
//   MMA2  D2[128 x 128] = H W2            (D1/16 x M128 N128 K16, A from TMEM) -> d2_full
//   EPI2  D2 -> registers, rounding points, sign bit of every value: a thread holds one 32-bit word of its
//         row's code and stores it                              -> d2_free
// SiLU of a bf16 is a function of 16 bits: a table in shared memory, filled by the formula (accurate exp, IEEE division)
// at the start of the kernel, serves all but exact zeros and outliers, which call the formula; so the codes equal the
// other kernels' up to the order of the fp32 additions. Still the epilogue takes longer than the contraction: the
// kernel is bound by instruction issue of the epilogue warps, not by the tensor core. The linear hash has a kernel of
// its own further down (one contraction per tile, bound by the stream of its input rows). Every wait on an mbarrier is
// bounded; a wait that runs out raises the library's hash status word, the CTA lets its copies in flight land, frees
// its TMEM and returns.
// Same arithmetic as the warp-level kernel in sl_hash_mma.cu up to the order of the fp32 additions.
#include <cuda.h>

#include "sl_common.cuh"

namespace {

constexpr int TC_EPI_WARPS = 16;                // 4 lane quadrants x 4 column groups
constexpr int TC_THREADS = (TC_EPI_WARPS + 1) * 32;
constexpr int TC_TILE = 128;
constexpr unsigned W1_BYTES = 128 * 256 * 2, W2_BYTES = 256 * 128 * 2, X_BYTES = TC_TILE * 128 * 2;
constexpr unsigned OFF_W1 = 0, OFF_W2 = W1_BYTES, OFF_X = W1_BYTES + W2_BYTES, OFF_B1 = OFF_X + 2 * X_BYTES,
                   OFF_B2 = OFF_B1 + 512, OFF_LUT = OFF_B2 + 256, OFF_BAR = OFF_LUT + 16384, OFF_MISC = OFF_BAR + 8 * 8, TC_SMEM = OFF_MISC + 16 + 1024;
constexpr unsigned WAIT_NS = 20000u, WAIT_TRIES = 50000u, WAIT_LIMIT = 1u << 22;

struct HashTcArgs {
    long long T; int H; int B;
    const __nv_bfloat16* w1; const __nv_bfloat16* w2; const __nv_bfloat16* b1; const __nv_bfloat16* b2;
    uint32_t* codes; long long cs_b;
    long long tiles_per_b, n_tiles;
    int* status;                                  // mapped host word: 3 = a wait ran out
};

__device__ __forceinline__ unsigned pack2(float lo, float hi) {      // two fp32 -> two bf16, round to nearest even, one instruction
    unsigned r;
    asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(hi), "f"(lo));
    return r;
}

// sum of two pairs of bf16, each rounded to nearest even once: equal to the fp32 sum rounded to bf16
__device__ __forceinline__ unsigned add_bf16x2(unsigned x, unsigned y) {
    unsigned r;
    asm("add.rn.bf16x2 %0, %1, %2;" : "=r"(r) : "r"(x), "r"(y));
    return r;
}

// SiLU of a bf16 at torch's rounding point: fp32 x / (1 + exp(-x)) with the accurate exp and the IEEE division, rounded once.
__device__ __forceinline__ unsigned short silu_bf16(unsigned short u) {
    const float y = __uint_as_float((unsigned)u << 16);
    return __bfloat16_as_ushort(__float2bfloat16_rn(y / (1.0f + expf(-y))));
}
// The activation has one bf16 argument, so it is a function of 16 bits. Its values for 2^-28 <= |x| < 16 (both signs:
// 8192 arguments, where all of a layer's values lie but exact zeros and outliers) are tabulated in shared memory at the
// start of the kernel with the formula above; the other arguments go through the formula itself. Either way the
// result is the formula's, bit for bit.
constexpr unsigned LUT_LO = 99u << 7;       // 2^-28

__device__ __noinline__ unsigned silu_pair(unsigned y) {
    return (unsigned)silu_bf16((unsigned short)(y & 0xffffu)) | ((unsigned)silu_bf16((unsigned short)(y >> 16)) << 16);
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
// Suspends the thread until the phase completes or about `ns` nanoseconds have passed (no spinning on shared memory,
// which the tensor core is reading its operands from).
__device__ __forceinline__ bool mbar_try(unsigned bar, unsigned parity, unsigned ns) {
    unsigned ok;
    asm volatile("{\n\t.reg .pred p;\n\tmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\tselp.u32 %0, 1, 0, p;\n\t}"
                 : "=r"(ok) : "r"(bar), "r"(parity), "r"(ns) : "memory");
    return ok != 0;
}
// Bounded wait: false when the limit ran out (WAIT_TRIES suspensions of at most WAIT_NS each and a pause between them:
// about a second) or another thread of the CTA has already given up.
__device__ __forceinline__ bool mbar_wait(unsigned bar, unsigned parity, volatile int* abort_flag) {
    for (unsigned i = 0; i < WAIT_TRIES; ++i) {
        if (mbar_try(bar, parity, WAIT_NS)) return true;
        if (*abort_flag) return false;
        __nanosleep(64);
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

// Phase stamps exist only in profiling builds (-DSL_TC_TIMING): CTA (0,0) stores the SM cycle counter at its phase boundaries.
#ifdef SL_TC_TIMING
__device__ unsigned long long g_tc_dbg[2][64][4];
__device__ unsigned long long g_tc_dbgw[16][4];
#define TC_STAMPW(k) if (blockIdx.x == 0 && blockIdx.y == 0 && it == 3 && lane == 0) g_tc_dbgw[warp][k] = (unsigned long long)clock64();
#define TC_STAMP(who, i, k) if (blockIdx.x == 0 && blockIdx.y == 0 && (i) < 64) g_tc_dbg[who][i][k] = (unsigned long long)clock64();
#else
#define TC_STAMP(who, i, k)
#define TC_STAMPW(k)
#endif

// D1: width of the hidden layer (256, or 128: then a warp's columns are one piece and both halves of H arrive together).
// RES (D1 == 128): the reference's residual form, layer output = f(x W + b) + input, rounded once more to bf16.
template <int D1, bool RES>
__global__ void __launch_bounds__(TC_THREADS, 1) hash_encode_tc_kernel(const __grid_constant__ CUtensorMap xmap, const HashTcArgs a) {
    static_assert(D1 == 256 || (D1 == 128), "hidden width");
    static_assert(!RES || D1 == 128, "a residual layer keeps its width");
    constexpr int NCH = D1 / 128;                             // 32-column pieces of D1 per epilogue warp
    extern __shared__ unsigned char smem_raw[];
    const unsigned raw = (unsigned)__cvta_generic_to_shared(smem_raw);
    const unsigned base = (raw + 1023u) & ~1023u;             // operand slabs start on 1024-byte boundaries
    unsigned char* g = smem_raw + (base - raw);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int h = blockIdx.y;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(g + OFF_MISC + 4);
    unsigned* tmem_slot = reinterpret_cast<unsigned*>(g + OFF_MISC);
    auto bar = [&](int i) { return base + OFF_BAR + (unsigned)i * 8u; };
    constexpr int X_FULL = 0 /* and 1 */, D1_FULL = 2, H_FULL = 3 /* first half of every warp's columns */, D2_FULL = 4, D2_FREE = 5, H_FULL2 = 6;

    // ---- set-up: barriers, TMEM, this head's weights (transposed to K-major) and biases
    if (tid == 0) {
        *abort_flag = 0;
        mbar_init(bar(X_FULL), 1); mbar_init(bar(X_FULL + 1), 1); mbar_init(bar(D1_FULL), 1);
        mbar_init(bar(H_FULL), TC_EPI_WARPS * 32); mbar_init(bar(H_FULL2), TC_EPI_WARPS * 32); mbar_init(bar(D2_FULL), 1); mbar_init(bar(D2_FREE), TC_EPI_WARPS * 32);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == TC_EPI_WARPS) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 512;" ::"r"(base + OFF_MISC) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    {
        // a warp takes 32 consecutive k of 8 columns: each lane reads 16 bytes of its row and writes 8 halfwords; the
        // 32 lanes of a store fall into distinct banks (k runs along the swizzled 128-byte row)
        const int NWARP = TC_THREADS / 32;
        constexpr int NG1 = D1 / 8;                                                               // groups of 8 n per row of W1
        const uint4* w1 = reinterpret_cast<const uint4*>(a.w1 + (long long)h * 128 * D1);         // [k][n]
        for (int task = warp; task < 4 * NG1; task += NWARP) {
            const int k = (task / NG1) * 32 + lane, n0 = (task % NG1) * 8;
            const uint4 v = w1[k * NG1 + (task % NG1)];
            const unsigned short* e = reinterpret_cast<const unsigned short*>(&v);
#pragma unroll
            for (int c = 0; c < 8; ++c) *reinterpret_cast<unsigned short*>(g + OFF_W1 + kmajor_off(n0 + c, k, D1)) = e[c];
        }
        const uint4* w2 = reinterpret_cast<const uint4*>(a.w2 + (long long)h * D1 * 128);         // [k][n], 16 groups of 8 n per row
        for (int task = warp; task < (D1 / 32) * 16; task += NWARP) {
            const int k = (task >> 4) * 32 + lane, n0 = (task & 15) * 8;
            const uint4 v = w2[k * 16 + (task & 15)];
            const unsigned short* e = reinterpret_cast<const unsigned short*>(&v);
#pragma unroll
            for (int c = 0; c < 8; ++c) *reinterpret_cast<unsigned short*>(g + OFF_W2 + kmajor_off(n0 + c, k, 128)) = e[c];
        }
        __nv_bfloat16* sb1 = reinterpret_cast<__nv_bfloat16*>(g + OFF_B1);
        __nv_bfloat16* sb2 = reinterpret_cast<__nv_bfloat16*>(g + OFF_B2);
        for (int i = tid; i < D1; i += TC_THREADS) sb1[i] = a.b1 ? a.b1[(long long)h * D1 + i] : __float2bfloat16_rn(0.0f);
        for (int i = tid; i < 128; i += TC_THREADS) sb2[i] = a.b2 ? a.b2[(long long)h * 128 + i] : __float2bfloat16_rn(0.0f);
        unsigned short* lut = reinterpret_cast<unsigned short*>(g + OFF_LUT);
        for (unsigned i = tid; i < 8192u; i += TC_THREADS)
            lut[i] = silu_bf16((unsigned short)(((i & 0xfffu) + LUT_LO) | ((i & 0x1000u) << 3)));
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // the weights were written by ordinary stores, the tensor core reads them
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem = *tmem_slot;

    const long long first = blockIdx.x, step = gridDim.x;
    bool failed = false;

    if (warp < TC_EPI_WARPS) {
        // ================= epilogue warps: thread = row = TMEM lane, warp group cg = a quarter of the columns =================
        const int q = warp & 3, cg = warp >> 2, row = q * 32 + lane;
        const unsigned t_row = tmem + ((unsigned)(q * 32) << 16);
        const unsigned t_d1 = t_row + (unsigned)(D1 / 4) * cg, t_h = t_row + 256u + (unsigned)(D1 / 8) * cg, t_d2 = t_row + 384u + 32u * cg;
        const unsigned* sb1 = reinterpret_cast<const unsigned*>(g + OFF_B1) + (D1 / 8) * cg;     // pairs of bf16
        unsigned hk[16];                                       // RES: this thread's 32 hidden values, the residual of layer 2
        const unsigned* sb2 = reinterpret_cast<const unsigned*>(g + OFF_B2) + 16 * cg;
        const unsigned char* lutb = g + OFF_LUT;
        unsigned it = 0;
        for (long long tile = first; tile < a.n_tiles; tile += step, ++it) {
            const unsigned par = it & 1u;
            if (!__all_sync(0xffffffffu, mbar_wait(bar(D1_FULL), par, abort_flag))) { failed = true; break; }   // warp-uniform: the TMEM accesses below are warp-wide
            tc_fence_after();
            if (tid == 0) { TC_STAMP(0, it, 0) }
            TC_STAMPW(0)
            unsigned v[1][32];
#pragma unroll 1
            for (int jj = 0; jj < NCH; ++jj) {
                constexpr int j = 0;
                unsigned pk[16], oob = 0u;
                tmem_ld32(t_d1 + 32u * jj, v[0]);
                tmem_wait_ld();
#pragma unroll
                for (int e = 0; e < 16; ++e) {
                    unsigned y = pack2(__uint_as_float(v[j][2 * e]), __uint_as_float(v[j][2 * e + 1]));   // matmul -> bf16
                    y = add_bf16x2(y, sb1[16 * jj + e]);                                                   // + bias -> bf16 (a null bias is a row of zeros)
                    v[j][e] = y;
                    // both halves at once: a half outside the table's range leaves bits in 0x7000 (a borrow from the low half can
                    // only come from such a half), and then the pair goes through the formula below
                    const unsigned d = y - (LUT_LO | (LUT_LO << 16)), dh = d >> 16;
                    oob |= d;
                    const unsigned i0 = ((d << 1) & 0x1ffeu) | ((d >> 2) & 0x2000u), i1 = ((dh << 1) & 0x1ffeu) | ((dh >> 2) & 0x2000u);
                    pk[e] = (unsigned)*reinterpret_cast<const unsigned short*>(lutb + i0) |
                            ((unsigned)*reinterpret_cast<const unsigned short*>(lutb + i1) << 16);         // SiLU -> bf16
                }
                if (oob & 0x70007000u) {
#pragma unroll
                    for (int e = 0; e < 16; ++e)                                  // only the pairs that need it (an exact zero, mostly: a sum that
                        if ((v[j][e] - (LUT_LO | (LUT_LO << 16))) & 0x70007000u)  // cancelled its bias); a call each, so the arrays stay in registers
                            pk[e] = silu_pair(v[j][e]);
                }
                if (RES) {                  // + input -> bf16: the thread's own row of the tile, still in its input stage
                    const unsigned char* xrow = g + OFF_X + (it & 1u) * X_BYTES;
#pragma unroll
                    for (int e = 0; e < 16; ++e) {
                        pk[e] = add_bf16x2(pk[e], *reinterpret_cast<const unsigned*>(xrow + kmajor_off(row, 32 * cg + 2 * e, TC_TILE)));
                        hk[e] = pk[e];
                    }
                }
                tmem_st16(t_h + 16u * jj, pk);
                tmem_wait_st();
                tc_fence_before();
                if (NCH == 1 || jj == 0) mbar_arrive(bar(H_FULL));     // layer 2 starts on the half that is there
                if (NCH == 1 || jj == 1) mbar_arrive(bar(H_FULL2));
            }
            if (tid == 0) { TC_STAMP(0, it, 1) }
            TC_STAMPW(1)

            if (!__all_sync(0xffffffffu, mbar_wait(bar(D2_FULL), par, abort_flag))) { failed = true; break; }
            tc_fence_after();
            if (tid == 0) { TC_STAMP(0, it, 2) }
            TC_STAMPW(2)
            tmem_ld32(t_d2, v[0]);
            tmem_wait_ld();
            tc_fence_before();
            mbar_arrive(bar(D2_FREE));
            unsigned bits = 0u;
#pragma unroll
            for (int e = 0; e < 16; ++e) {
                unsigned y = pack2(__uint_as_float(v[0][2 * e]), __uint_as_float(v[0][2 * e + 1]));
                y = add_bf16x2(y, sb2[e]);
                if (RES) y = add_bf16x2(y, hk[e]);              // + the layer's input (the hidden values of the same columns)
                const float y0 = __uint_as_float(y << 16), y1 = __uint_as_float(y & 0xffff0000u);
                bits |= ((y0 > 0.0f ? 1u : 0u) | (y1 > 0.0f ? 2u : 0u)) << (2 * e);
            }
            const long long b = tile / a.tiles_per_b, t = (tile - b * a.tiles_per_b) * TC_TILE + row;
            if (t < a.T) a.codes[b * a.cs_b + (t * a.H + h) * 4 + cg] = bits;
            if (tid == 0) { TC_STAMP(0, it, 3) }
            TC_STAMPW(3)
        }
    } else if (lane == 0) {
        // ================= issuing thread: TMA loads and tensor-core instructions =================
        const unsigned x_s = base + OFF_X;
        constexpr unsigned I1 = instr_desc(D1), I2 = instr_desc(128);
        bool pending[2] = {false, false};                     // a copy into this stage is in flight
        auto load = [&](long long tile, int st) {
            const long long b = tile / a.tiles_per_b;
            const int t0 = (int)((tile - b * a.tiles_per_b) * TC_TILE);
            const unsigned dst = x_s + (unsigned)st * X_BYTES;
            mbar_expect_tx(bar(X_FULL + st), X_BYTES);
            tma_load_4d(dst, &xmap, bar(X_FULL + st), 0, t0, h, (int)b);                 // k 0..63 of the 128 rows
            tma_load_4d(dst + X_BYTES / 2, &xmap, bar(X_FULL + st), 64, t0, h, (int)b);  // k 64..127
            pending[st] = true;
        };
        auto mma1 = [&](unsigned n) -> bool {                 // layer 1 of this CTA's n-th tile, once its rows have landed
            const int st = (int)(n & 1u);
            if (!mbar_wait(bar(X_FULL + st), (n >> 1) & 1u, abort_flag)) return false;
            pending[st] = false;
            tc_fence_after();
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
                const unsigned ao = (unsigned)st * X_BYTES + (unsigned)(ks >> 2) * (X_BYTES / 2) + (unsigned)(ks & 3) * 32u;
                const unsigned bo = (unsigned)(ks >> 2) * ((unsigned)D1 * 128u) + (unsigned)(ks & 3) * 32u;
                mma_ss(tmem, smem_desc(x_s + ao), smem_desc(base + OFF_W1 + bo), I1, ks > 0 ? 1u : 0u);
            }
            tc_commit(bar(D1_FULL));
            return true;
        };
        if (first < a.n_tiles) load(first, 0);
        if (first + step < a.n_tiles) load(first + step, 1);
        if (first < a.n_tiles && !mma1(0)) failed = true;
        unsigned it = 0;
        for (long long tile = first; tile < a.n_tiles && !failed; tile += step, ++it) {
            const unsigned par = it & 1u;
            TC_STAMP(1, it, 0)
            if (!mbar_wait(bar(H_FULL), par, abort_flag)) { failed = true; break; }        // the first half of every warp's H columns is written
            TC_STAMP(1, it, 1)
            if (it > 0 && !mbar_wait(bar(D2_FREE), par ^ 1u, abort_flag)) { failed = true; break; }   // D2 of the previous tile has been read
            tc_fence_after();
#pragma unroll
            for (int half = 0; half < 2; ++half) {
                if (half == 1) {
                    if (!mbar_wait(bar(H_FULL2), par, abort_flag)) { failed = true; break; }   // the rest of H is written, all of D1 read
                    tc_fence_after();
                    // layer 1 of this tile is over and (RES) its input rows have been added: the input stage takes the next rows
                    if (tile + 2 * step < a.n_tiles) load(tile + 2 * step, (int)par);
                }
                if (NCH == 2 || half == 0) {
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        // D1 = 256: warp group cg wrote K [64 cg + 32 half, + 32); D1 = 128: K [32 cg, + 32), all there at once
                        const int ks = NCH == 2 ? 4 * (i >> 1) + 2 * half + (i & 1) : i;
                        const unsigned bo = (unsigned)(ks >> 2) * (128u * 128u) + (unsigned)(ks & 3) * 32u;
                        mma_ts(tmem + 384u, tmem + 256u + 8u * ks, smem_desc(base + OFF_W2 + bo), I2, (half | i) ? 1u : 0u);
                    }
                }
            }
            if (failed) break;
            tc_commit(bar(D2_FULL));
            TC_STAMP(1, it, 2)
            if (tile + step < a.n_tiles && !mma1(it + 1)) { failed = true; break; }         // runs under the second epilogue of this tile
        }
        TC_STAMP(1, 63, 3)
        if (failed) {                                         // copies of ours still in flight: let them land (bounded)
            for (int st = 0; st < 2; ++st)
                if (pending[st]) {
                    for (unsigned i = 0; i < WAIT_LIMIT && !(mbar_test(bar(X_FULL + st), 0u) || mbar_test(bar(X_FULL + st), 1u)); ++i) __nanosleep(256);
                }
        }
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

// ---- the linear hash 128 -> 128 (one contraction per tile): bound by the stream of the input rows, so the kernel
// keeps four input stages in flight and two accumulators in TMEM; two teams of four epilogue warps take alternate
// tiles (a thread reads its row's 128 columns, adds the bias, takes the sign bits and stores the row's 16-byte code).
constexpr int L1_NS = 4;                        // input stages
constexpr int L1_THREADS = (8 + 1) * 32;
constexpr unsigned L1_W = 128 * 128 * 2, L1_OFF_X = L1_W, L1_OFF_B = L1_OFF_X + L1_NS * X_BYTES, L1_OFF_BAR = L1_OFF_B + 256,
                   L1_OFF_MISC = L1_OFF_BAR + 8 * 8, L1_SMEM = L1_OFF_MISC + 16 + 1024;

__global__ void __launch_bounds__(L1_THREADS, 1) hash_encode_tc_linear_kernel(const __grid_constant__ CUtensorMap xmap, const HashTcArgs a) {
    extern __shared__ unsigned char smem_raw[];
    const unsigned raw = (unsigned)__cvta_generic_to_shared(smem_raw);
    const unsigned base = (raw + 1023u) & ~1023u;
    unsigned char* g = smem_raw + (base - raw);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int h = blockIdx.y;
    volatile int* abort_flag = reinterpret_cast<volatile int*>(g + L1_OFF_MISC + 4);
    unsigned* tmem_slot = reinterpret_cast<unsigned*>(g + L1_OFF_MISC);
    auto bar = [&](int i) { return base + L1_OFF_BAR + (unsigned)i * 8u; };
    constexpr int X_FULL = 0 /* .. 3 */, D_FULL = 4 /* , 5 */, D_FREE = 6 /* , 7 */;

    if (tid == 0) {
        *abort_flag = 0;
        for (int i = 0; i < L1_NS; ++i) mbar_init(bar(X_FULL + i), 1);
        for (int i = 0; i < 2; ++i) { mbar_init(bar(D_FULL + i), 1); mbar_init(bar(D_FREE + i), 128); }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 8) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], 256;" ::"r"(base + L1_OFF_MISC) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    {
        const uint4* w1 = reinterpret_cast<const uint4*>(a.w1 + (long long)h * 128 * 128);        // [k][n], 16 groups of 8 n per row
        for (int task = warp; task < 4 * 16; task += L1_THREADS / 32) {
            const int k = (task >> 4) * 32 + lane, n0 = (task & 15) * 8;
            const uint4 v = w1[k * 16 + (task & 15)];
            const unsigned short* e = reinterpret_cast<const unsigned short*>(&v);
#pragma unroll
            for (int c = 0; c < 8; ++c) *reinterpret_cast<unsigned short*>(g + kmajor_off(n0 + c, k, 128)) = e[c];
        }
        __nv_bfloat16* sb = reinterpret_cast<__nv_bfloat16*>(g + L1_OFF_B);
        for (int i = tid; i < 128; i += L1_THREADS) sb[i] = a.b1 ? a.b1[(long long)h * 128 + i] : __float2bfloat16_rn(0.0f);
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const unsigned tmem = *tmem_slot;
    const long long first = blockIdx.x, step = gridDim.x;
    bool failed = false;

    if (warp < 8) {
        // ================= epilogue team `team` takes the CTA's tiles team, team + 2, ... =================
        const int team = warp >> 2, q = warp & 3, row = q * 32 + lane;
        const unsigned t_d = tmem + ((unsigned)(q * 32) << 16) + 128u * team;
        const unsigned* sb = reinterpret_cast<const unsigned*>(g + L1_OFF_B);
        unsigned it = team;
        for (long long tile = first + team * step; tile < a.n_tiles; tile += 2 * step, it += 2) {
            if (!__all_sync(0xffffffffu, mbar_wait(bar(D_FULL + team), (it >> 1) & 1u, abort_flag))) { failed = true; break; }
            tc_fence_after();
            unsigned v[4][32];
#pragma unroll
            for (int j = 0; j < 4; ++j) tmem_ld32(t_d + 32u * j, v[j]);
            tmem_wait_ld();
            tc_fence_before();
            mbar_arrive(bar(D_FREE + team));
            unsigned word[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                unsigned bits = 0u;
#pragma unroll
                for (int e = 0; e < 16; ++e) {
                    unsigned y = pack2(__uint_as_float(v[j][2 * e]), __uint_as_float(v[j][2 * e + 1]));   // matmul -> bf16
                    y = add_bf16x2(y, sb[16 * j + e]);                                                     // + bias -> bf16
                    const float y0 = __uint_as_float(y << 16), y1 = __uint_as_float(y & 0xffff0000u);
                    bits |= ((y0 > 0.0f ? 1u : 0u) | (y1 > 0.0f ? 2u : 0u)) << (2 * e);
                }
                word[j] = bits;
            }
            const long long b = tile / a.tiles_per_b, t = (tile - b * a.tiles_per_b) * TC_TILE + row;
            if (t < a.T) *reinterpret_cast<uint4*>(a.codes + b * a.cs_b + (t * a.H + h) * 4) = make_uint4(word[0], word[1], word[2], word[3]);
        }
    } else if (lane == 0) {
        // ================= issuing thread =================
        const unsigned x_s = base + L1_OFF_X;
        constexpr unsigned I1 = instr_desc(128);
        bool pending[L1_NS] = {false, false, false, false};
        auto load = [&](long long tile, int st) {
            const long long b = tile / a.tiles_per_b;
            const int t0 = (int)((tile - b * a.tiles_per_b) * TC_TILE);
            const unsigned dst = x_s + (unsigned)st * X_BYTES;
            mbar_expect_tx(bar(X_FULL + st), X_BYTES);
            tma_load_4d(dst, &xmap, bar(X_FULL + st), 0, t0, h, (int)b);
            tma_load_4d(dst + X_BYTES / 2, &xmap, bar(X_FULL + st), 64, t0, h, (int)b);
            pending[st] = true;
        };
        for (int i = 0; i < L1_NS; ++i)
            if (first + i * step < a.n_tiles) load(first + i * step, i);
        unsigned it = 0;
        for (long long tile = first; tile < a.n_tiles; tile += step, ++it) {
            const int st = (int)(it % L1_NS), buf = (int)(it & 1u);
            if (!mbar_wait(bar(X_FULL + st), (it / L1_NS) & 1u, abort_flag)) { failed = true; break; }
            pending[st] = false;
            if (it >= 2 && !mbar_wait(bar(D_FREE + buf), ((it >> 1) - 1u) & 1u, abort_flag)) { failed = true; break; }   // the accumulator has been read
            tc_fence_after();
#pragma unroll
            for (int ks = 0; ks < 8; ++ks) {
                const unsigned ao = (unsigned)st * X_BYTES + (unsigned)(ks >> 2) * (X_BYTES / 2) + (unsigned)(ks & 3) * 32u;
                const unsigned bo = (unsigned)(ks >> 2) * (128u * 128u) + (unsigned)(ks & 3) * 32u;
                mma_ss(tmem + 128u * buf, smem_desc(x_s + ao), smem_desc(base + bo), I1, ks > 0 ? 1u : 0u);
            }
            tc_commit(bar(D_FULL + buf));
            if (it >= 1) {       // the contraction of the tile before this one is over by now or soon: its input stage takes the next rows
                if (!mbar_wait(bar(D_FULL + (buf ^ 1)), ((it - 1u) >> 1) & 1u, abort_flag)) { failed = true; break; }
                const long long nxt = tile + (long long)(L1_NS - 1) * step;
                if (nxt < a.n_tiles) load(nxt, (int)((it - 1u) % L1_NS));
            }
        }
        if (failed) {
            for (int st = 0; st < L1_NS; ++st)
                if (pending[st]) {
                    for (unsigned i = 0; i < WAIT_LIMIT && !(mbar_test(bar(X_FULL + st), 0u) || mbar_test(bar(X_FULL + st), 1u)); ++i) __nanosleep(256);
                }
        }
    }
    if (failed) {
        *abort_flag = 1;
        if (a.status) *reinterpret_cast<volatile int*>(a.status) = 3;
    }
    __syncwarp();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    if (warp == 8) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, 256;" ::"r"(tmem) : "memory");
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

#ifdef SL_TC_TIMING
extern "C" int sl_profile_tc_timing(unsigned long long* host_out) {
    if (cudaMemcpyFromSymbol(host_out + 2 * 64 * 4, g_tc_dbgw, sizeof(g_tc_dbgw)) != cudaSuccess) return 1;
    return cudaMemcpyFromSymbol(host_out, g_tc_dbg, sizeof(g_tc_dbg)) == cudaSuccess ? 0 : 1;
}
#endif

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
    const bool mlp = hp->n_layers == 2 && hp->dims[0] == 128 && (hp->dims[1] == 256 || hp->dims[1] == 128) && hp->dims[2] == 128;
    const bool linear = hp->n_layers == 1 && hp->dims[0] == 128 && hp->dims[1] == 128;
    if ((!mlp && !linear) || (hp->residue && (linear || hp->dims[1] != 128))) return 1;
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
    a.w1 = static_cast<const __nv_bfloat16*>(hp->d_w[0]); a.b1 = static_cast<const __nv_bfloat16*>(hp->d_b[0]);
    if (mlp) { a.w2 = static_cast<const __nv_bfloat16*>(hp->d_w[1]); a.b2 = static_cast<const __nv_bfloat16*>(hp->d_b[1]); }
    a.codes = codes; a.cs_b = cs_b;
    a.tiles_per_b = (T + TC_TILE - 1) / TC_TILE;
    a.n_tiles = a.tiles_per_b * B;
    a.status = d_status;
    const long long per_head = std::max<long long>(1, (long long)sl::sm_count() / H);
    const unsigned gx = (unsigned)std::min<long long>(a.n_tiles, per_head);
    if (mlp) {
        void (*kern)(const CUtensorMap, const HashTcArgs) = hp->dims[1] == 256 ? hash_encode_tc_kernel<256, false>
                                                          : hp->residue       ? hash_encode_tc_kernel<128, true>
                                                                              : hash_encode_tc_kernel<128, false>;
        SL_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)TC_SMEM));
        kern<<<dim3(gx, (unsigned)H), TC_THREADS, TC_SMEM, s>>>(map, a);
    } else {
        SL_CUDA_OK(cudaFuncSetAttribute(hash_encode_tc_linear_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)L1_SMEM));
        hash_encode_tc_linear_kernel<<<dim3(gx, (unsigned)H), L1_THREADS, L1_SMEM, s>>>(map, a);
    }
    SL_CUDA_OK(cudaGetLastError());
    return SL_OK;
}

}  // namespace sl
