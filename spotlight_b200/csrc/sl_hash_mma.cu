// Code-cache build at prefill on the warp-level tensor-core path: hash + sign + pack of many
// rows of one head per CTA (bf16; shapes 128 -> 128 and 128 -> {128,256} -> 128).
//
// This is the one dense contraction of the retrieval path (N*H rows x the hash MLP). The
// weights of the CTA's head stay in shared memory (XOR-swizzled rows, read with ldmatrix.trans),
// input rows arrive in double-buffered 128-row tiles by cp.async, every warp owns 16 rows:
//   layer 1  C1[16 x D1] = X[16 x 128] W1       (two 128-column passes when D1 = 256)
//            epilogue at torch's rounding points (matmul -> bf16, + bias -> bf16, SiLU -> bf16,
//            + residual -> bf16); the rounded values are re-packed IN REGISTERS as the A
//            fragments of layer 2 (accumulator tiles 2j, 2j+1 are exactly k-step j)
//   layer 2  C2[16 x 128] = H[16 x D1] W2, epilogue, sign bit of every value, 128 bits per row
//            gathered across the four lanes of a group and stored as four uint32 words.
// Same arithmetic as the scalar kernel in sl_hash.cu up to the order of the fp32 additions.
#include "sl_mma.cuh"

namespace {

constexpr int HM_THREADS = 256;
constexpr int HM_TILE = 128;             // rows per CTA tile = 8 warps x 16 rows

struct HashMmaArgs {
    const __nv_bfloat16* x; long long xs_b, xs_tok, xs_h; long long T; int H; int B;
    const __nv_bfloat16* w[2]; const __nv_bfloat16* bias[2]; int residue;
    uint32_t* codes; long long cs_b; long long n_tiles;
};

// byte offset of 16-byte chunk c of row r when a row holds CH chunks (CH a multiple of 8)
__device__ __forceinline__ unsigned wz(int r, int c, int CH) { return (unsigned)((r * CH + ((c & ~7) | ((c ^ r) & 7))) << 4); }

__device__ __forceinline__ float bfr(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

// one layer's epilogue for one value: torch's operator sequence in bf16
__device__ __forceinline__ float finish(float c, const __nv_bfloat16* bias, int col, bool act, bool residue, float xres) {
    float y = bfr(c);
    if (bias) y = bfr(y + __bfloat162float(bias[col]));
    if (act) y = bfr(y / (1.0f + expf(-y)));
    if (residue) y = bfr(y + xres);
    return y;
}

__device__ __forceinline__ float bf_lo(unsigned v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf_hi(unsigned v) { return __uint_as_float(v & 0xffff0000u); }

template <int NL, int D1>   // NL layers; D1 = width after layer 1 (128 when NL == 1)
__global__ void __launch_bounds__(HM_THREADS, 1) hash_encode_mma_kernel(const HashMmaArgs a) {
    extern __shared__ __align__(128) unsigned char smem[];
    constexpr int CH1 = D1 / 8;                              // 16-byte chunks per row of W1
    constexpr int W1_BYTES = 128 * D1 * 2, W2_BYTES = NL == 2 ? D1 * 128 * 2 : 0;
    const unsigned s_w1 = (unsigned)__cvta_generic_to_shared(smem);
    const unsigned s_w2 = s_w1 + W1_BYTES;
    const unsigned s_x = s_w2 + W2_BYTES;                    // [2][128 rows][256 B]
    unsigned char* g_x = smem + W1_BYTES + W2_BYTES;

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, grp = lane >> 2, tig = lane & 3;
    const int h = blockIdx.y;
    const long long rows = (long long)a.B * a.T;

    // ---- this head's weights -> shared memory (swizzled rows)
    {
        const uint4* w1 = reinterpret_cast<const uint4*>(a.w[0] + (long long)h * 128 * D1);
        for (int i = tid; i < 128 * CH1; i += HM_THREADS) {
            const int r = i / CH1, c = i % CH1;
            *reinterpret_cast<uint4*>(smem + wz(r, c, CH1)) = w1[i];
        }
        if (NL == 2) {
            const uint4* w2 = reinterpret_cast<const uint4*>(a.w[1] + (long long)h * D1 * 128);
            for (int i = tid; i < D1 * 16; i += HM_THREADS) {
                const int r = i >> 4, c = i & 15;
                *reinterpret_cast<uint4*>(smem + W1_BYTES + wz(r, c, 16)) = w2[i];
            }
        }
    }
    const __nv_bfloat16* b1 = a.bias[0] ? a.bias[0] + (long long)h * D1 : nullptr;
    const __nv_bfloat16* b2 = (NL == 2 && a.bias[1]) ? a.bias[1] + (long long)h * 128 : nullptr;

    auto issue_tile = [&](long long tile, int buf) {         // 128 rows x 16 chunks, 8 per thread
#pragma unroll
        for (int it = 0; it < 8; ++it) {
            const int id = it * HM_THREADS + tid, r = id >> 4, c = id & 15;
            long long rg = tile * HM_TILE + r;
            if (rg >= rows) rg = rows - 1;
            const long long b = rg / a.T, t = rg - b * a.T;
            cp_async16(s_x + buf * (HM_TILE * 256) + wz(r, c, 16), a.x + b * a.xs_b + t * a.xs_tok + h * a.xs_h + c * 8);
        }
    };

    long long tile = blockIdx.x;
    int buf = 0;
    if (tile < a.n_tiles) issue_tile(tile, 0);
    cp_async_commit();
    for (; tile < a.n_tiles; tile += gridDim.x, buf ^= 1) {
        if (tile + gridDim.x < a.n_tiles) issue_tile(tile + gridDim.x, buf ^ 1);
        cp_async_commit();
        cp_async_wait<1>();
        __syncthreads();                                     // tile `buf` (and, first time, the weights) visible
        const unsigned xw = s_x + buf * (HM_TILE * 256) + warp * (16 * 256);   // this warp's 16 rows
        const unsigned char* xg = g_x + buf * (HM_TILE * 256) + warp * (16 * 256);

        // ---- A fragments of the 16 input rows, all 8 k-steps
        unsigned xa[8][4];
#pragma unroll
        for (int s = 0; s < 8; ++s)
            ldsm_x4(xa[s], xw + wz(((lane >> 3) & 1) * 8 + (lane & 7), 2 * s + (lane >> 4), 16));

        unsigned ha[NL == 2 ? D1 / 16 : 1][4];               // layer-2 A fragments (rounded layer-1 output)
        unsigned bits0[4] = {0u, 0u, 0u, 0u}, bits1[4] = {0u, 0u, 0u, 0u};   // rows grp / grp + 8, NL == 1
#pragma unroll
        for (int half = 0; half < D1 / 128; ++half) {
            float acc[16][4];
#pragma unroll
            for (int t = 0; t < 16; ++t) { acc[t][0] = acc[t][1] = acc[t][2] = acc[t][3] = 0.0f; }
#pragma unroll
            for (int s = 0; s < 8; ++s) {
#pragma unroll
                for (int t2 = 0; t2 < 8; ++t2) {
                    unsigned bf[4];
                    ldsm_x4_trans(bf, s_w1 + wz(16 * s + ((lane >> 3) & 1) * 8 + (lane & 7), half * 16 + 2 * t2 + (lane >> 4), CH1));
                    mma_bf16(acc[2 * t2], xa[s][0], xa[s][1], xa[s][2], xa[s][3], bf[0], bf[1]);
                    mma_bf16(acc[2 * t2 + 1], xa[s][0], xa[s][1], xa[s][2], xa[s][3], bf[2], bf[3]);
                }
            }
#pragma unroll
            for (int t = 0; t < 16; ++t) {
                const int col = half * 128 + 8 * t + 2 * tig;
                float r00 = 0.f, r01 = 0.f, r10 = 0.f, r11 = 0.f;   // residual x[row][col], D1 == 128 only
                if (a.residue) {
                    const unsigned v0 = *reinterpret_cast<const unsigned*>(xg + wz(grp, col >> 3, 16) + (col & 7) * 2);
                    const unsigned v1 = *reinterpret_cast<const unsigned*>(xg + wz(grp + 8, col >> 3, 16) + (col & 7) * 2);
                    r00 = bf_lo(v0); r01 = bf_hi(v0); r10 = bf_lo(v1); r11 = bf_hi(v1);
                }
                const bool act = NL == 2;
                const float y00 = finish(acc[t][0], b1, col, act, a.residue, r00);
                const float y01 = finish(acc[t][1], b1, col + 1, act, a.residue, r01);
                const float y10 = finish(acc[t][2], b1, col, act, a.residue, r10);
                const float y11 = finish(acc[t][3], b1, col + 1, act, a.residue, r11);
                if (NL == 2) {
                    const int j = (half * 16 + t) >> 1, o = (t & 1) * 2;
                    ha[j][o] = pack_bf16(y00, y01);
                    ha[j][o + 1] = pack_bf16(y10, y11);
                } else {
                    const int sh = 8 * (t & 3) + 2 * tig;
                    bits0[t >> 2] |= ((y00 > 0.f ? 1u : 0u) | (y01 > 0.f ? 2u : 0u)) << sh;
                    bits1[t >> 2] |= ((y10 > 0.f ? 1u : 0u) | (y11 > 0.f ? 2u : 0u)) << sh;
                }
            }
        }
        if (NL == 2) {
            float acc[16][4];
#pragma unroll
            for (int t = 0; t < 16; ++t) { acc[t][0] = acc[t][1] = acc[t][2] = acc[t][3] = 0.0f; }
#pragma unroll
            for (int j = 0; j < D1 / 16; ++j) {
#pragma unroll
                for (int t2 = 0; t2 < 8; ++t2) {
                    unsigned bf[4];
                    ldsm_x4_trans(bf, s_w2 + wz(16 * j + ((lane >> 3) & 1) * 8 + (lane & 7), 2 * t2 + (lane >> 4), 16));
                    mma_bf16(acc[2 * t2], ha[j][0], ha[j][1], ha[j][2], ha[j][3], bf[0], bf[1]);
                    mma_bf16(acc[2 * t2 + 1], ha[j][0], ha[j][1], ha[j][2], ha[j][3], bf[2], bf[3]);
                }
            }
#pragma unroll
            for (int t = 0; t < 16; ++t) {
                const int col = 8 * t + 2 * tig;
                float r00 = 0.f, r01 = 0.f, r10 = 0.f, r11 = 0.f;   // residual = layer-1 output (D1 == 128)
                if (a.residue) {
                    const unsigned v0 = ha[t >> 1][(t & 1) * 2], v1 = ha[t >> 1][(t & 1) * 2 + 1];
                    r00 = bf_lo(v0); r01 = bf_hi(v0); r10 = bf_lo(v1); r11 = bf_hi(v1);
                }
                const float y00 = finish(acc[t][0], b2, col, false, a.residue, r00);
                const float y01 = finish(acc[t][1], b2, col + 1, false, a.residue, r01);
                const float y10 = finish(acc[t][2], b2, col, false, a.residue, r10);
                const float y11 = finish(acc[t][3], b2, col + 1, false, a.residue, r11);
                const int sh = 8 * (t & 3) + 2 * tig;
                bits0[t >> 2] |= ((y00 > 0.f ? 1u : 0u) | (y01 > 0.f ? 2u : 0u)) << sh;
                bits1[t >> 2] |= ((y10 > 0.f ? 1u : 0u) | (y11 > 0.f ? 2u : 0u)) << sh;
            }
        }
        // ---- the four lanes of a group hold disjoint bits of the same rows: OR them together
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            bits0[w] |= __shfl_xor_sync(0xffffffffu, bits0[w], 1);
            bits0[w] |= __shfl_xor_sync(0xffffffffu, bits0[w], 2);
            bits1[w] |= __shfl_xor_sync(0xffffffffu, bits1[w], 1);
            bits1[w] |= __shfl_xor_sync(0xffffffffu, bits1[w], 2);
        }
#pragma unroll
        for (int half = 0; half < 2; ++half) {               // lane tig stores word tig of rows grp and grp + 8
            const long long rg = tile * HM_TILE + warp * 16 + grp + 8 * half;
            if (rg < rows) {
                const long long b = rg / a.T, t = rg - b * a.T;
                const unsigned* bb = half ? bits1 : bits0;
                const unsigned word = tig == 0 ? bb[0] : tig == 1 ? bb[1] : tig == 2 ? bb[2] : bb[3];
                a.codes[b * a.cs_b + (t * a.H + h) * 4 + tig] = word;
            }
        }
        __syncthreads();                                     // everyone is done with tile `buf` before it is refilled
    }
    cp_async_wait<0>();
}

template <int NL, int D1>
int launch_one(const HashMmaArgs& a, cudaStream_t s) {
    const size_t smem = (size_t)128 * D1 * 2 + (NL == 2 ? (size_t)D1 * 128 * 2 : 0) + 2 * HM_TILE * 256;
    SL_CUDA_OK(cudaFuncSetAttribute(hash_encode_mma_kernel<NL, D1>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const long long per_head = std::max<long long>(1, (long long)sl::sm_count() / a.H);
    const unsigned gx = (unsigned)std::min<long long>(a.n_tiles, per_head);
    hash_encode_mma_kernel<NL, D1><<<dim3(gx, (unsigned)a.H), HM_THREADS, smem, s>>>(a);
    SL_CUDA_OK(cudaGetLastError());
    return SL_OK;
}

}  // namespace

namespace sl {

// Returns SL_OK after launching, or 1 when the shape is not one the tensor-core kernel covers.
int launch_hash_encode_mma(const void* x, long long xs_b, long long xs_tok, long long xs_h, int B, long long T, int H, const sl_hash_params* hp,
                           uint32_t* codes, long long cs_b, cudaStream_t s) {
    if (hp->dims[0] != 128 || hp->dims[hp->n_layers] != 128 || hp->n_layers > 2) return 1;
    if (hp->n_layers == 2 && hp->dims[1] != 128 && hp->dims[1] != 256) return 1;
    if (H > 65535) return 1;
    HashMmaArgs a = {};
    a.x = static_cast<const __nv_bfloat16*>(x); a.xs_b = xs_b; a.xs_tok = xs_tok; a.xs_h = xs_h; a.T = T; a.H = H; a.B = B;
    for (int i = 0; i < hp->n_layers; ++i) {
        a.w[i] = static_cast<const __nv_bfloat16*>(hp->d_w[i]);
        a.bias[i] = static_cast<const __nv_bfloat16*>(hp->d_b[i]);
    }
    a.residue = hp->residue;
    a.codes = codes; a.cs_b = cs_b;
    a.n_tiles = ((long long)B * T + HM_TILE - 1) / HM_TILE;
    if (hp->n_layers == 1) return launch_one<1, 128>(a, s);
    if (hp->dims[1] == 128) return launch_one<2, 128>(a, s);
    return launch_one<2, 256>(a, s);
}

}  // namespace sl
