// Sign-bit packing and the plain Hamming match-count kernels (the parity shims for the
// reference's pack_* / attn_* entry points).
#include "sl_common.cuh"
#include "sl_sliced.cuh"

namespace {

// One thread packs 8 consecutive values into one byte; a warp reads 32 x 16 B (bf16/fp16),
// 32 x 32 B (fp32) or 32 x 8 B (bool) contiguous bytes and writes 32 contiguous bytes.
template <typename T>
__global__ void __launch_bounds__(256) pack_kernel(const T* __restrict__ x, uint8_t* __restrict__ out,
                                                   int64_t n_bytes) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    const int64_t stride = (int64_t)gridDim.x * blockDim.x;
    for (; i < n_bytes; i += stride) {
        unsigned byte = 0;
        if constexpr (sizeof(T) == 2) {
            uint4 raw = sl::ld_stream_v4(reinterpret_cast<const uint4*>(x) + i);
            const T* v = reinterpret_cast<const T*>(&raw);
#pragma unroll
            for (int j = 0; j < 8; ++j) byte |= (sl::VT<T>::to_f(v[j]) > 0.0f ? 1u : 0u) << j;
        } else if constexpr (sizeof(T) == 4) {
            uint4 r0 = sl::ld_stream_v4(reinterpret_cast<const uint4*>(x) + 2 * i);
            uint4 r1 = sl::ld_stream_v4(reinterpret_cast<const uint4*>(x) + 2 * i + 1);
            const float* a = reinterpret_cast<const float*>(&r0);
            const float* b = reinterpret_cast<const float*>(&r1);
#pragma unroll
            for (int j = 0; j < 4; ++j) byte |= (a[j] > 0.0f ? 1u : 0u) << j;
#pragma unroll
            for (int j = 0; j < 4; ++j) byte |= (b[j] > 0.0f ? 1u : 0u) << (4 + j);
        } else {
            uint2 raw = *(reinterpret_cast<const uint2*>(x) + i);
            const uint8_t* v = reinterpret_cast<const uint8_t*>(&raw);
#pragma unroll
            for (int j = 0; j < 8; ++j) byte |= (v[j] != 0 ? 1u : 0u) << j;
        }
        out[i] = (uint8_t)byte;
    }
}

// One thread scores one (token, kv head) code of W words; q codes staged in shared memory.
template <int W>
__global__ void __launch_bounds__(256) scores_kernel(const uint32_t* __restrict__ q, const uint32_t* __restrict__ k,
                                                     int64_t k_bstride, int16_t* __restrict__ out, int64_t N,
                                                     int KH, int G, int layout) {
    extern __shared__ uint32_t qs[];  // [KH][G][W]
    const int b = blockIdx.y;
    const int QH = KH * G;
    for (int i = threadIdx.x; i < QH * W; i += blockDim.x) {
        int w = i % W, hg = i / W, g = hg % G, h = hg / G;
        int qh = layout == SL_GQA_INTERLEAVED ? g * KH + h : h * G + g;
        qs[i] = q[((int64_t)b * QH + qh) * W + w];
    }
    __syncthreads();
    const int64_t total = N * KH;
    const uint32_t* kb = k + (int64_t)b * k_bstride;
    int16_t* ob = out + (int64_t)b * total;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int h = (int)(i % KH);
        uint32_t c[W];
        if constexpr (W == 4) {
            uint4 v = sl::ld_stream_v4(reinterpret_cast<const uint4*>(kb) + i);
            c[0] = v.x; c[1] = v.y; c[2] = v.z; c[3] = v.w;
        } else {
#pragma unroll
            for (int w = 0; w < W; ++w) c[w] = kb[i * W + w];
        }
        int acc = 0;
        const uint32_t* qh = qs + h * G * W;
        for (int g = 0; g < G; ++g) {
#pragma unroll
            for (int w = 0; w < W; ++w) acc += __popc(~(qh[g * W + w] ^ c[w]));
        }
        ob[i] = (int16_t)acc;
    }
}

// 128-bit codes with the kv heads dividing the block size: every thread keeps one head, scores
// with the bit-sliced carry-save scorer (P + 2 popcounts per key instead of 4*G) and streams
// four 16-byte loads at a time.
template <int P>
__global__ void __launch_bounds__(256) scores_sliced_kernel(const uint32_t* __restrict__ q, const uint4* __restrict__ k,
                                                            int64_t k_bstride16, int16_t* __restrict__ out, int64_t N,
                                                            int KH, int G, int layout) {
    __shared__ __align__(16) uint32_t planes[32 * 2 * 4 * 4];          // [KH][2][P][4], KH <= 32
    __shared__ __align__(16) int pbase[32 * 4];
    const int b = blockIdx.y;
    stage_planes<P>(q + (int64_t)b * KH * G * 4, KH, G, layout, planes, pbase, threadIdx.x >> 5, 8, threadIdx.x & 31);
    __syncthreads();
    uint32_t M[P][4], Mp[P][4];
    const int base = load_planes<P>(planes, pbase, threadIdx.x % KH, M, Mp);
    const int sh = sliced_shift(G);
    const int64_t total = N * KH, stride = (int64_t)gridDim.x * 256;
    const uint4* kb = k + (int64_t)b * k_bstride16;
    int16_t* ob = out + (int64_t)b * total;
    for (int64_t i0 = (int64_t)blockIdx.x * 256 + threadIdx.x; i0 < total; i0 += 4 * stride) {
        uint4 c[4];
#pragma unroll
        for (int u = 0; u < 4; ++u)
            if (i0 + u * stride < total) c[u] = sl::ld_stream_v4(kb + i0 + u * stride);
#pragma unroll
        for (int u = 0; u < 4; ++u)
            if (i0 + u * stride < total) ob[i0 + u * stride] = (int16_t)(base + (sliced_score<P>(c[u], M, Mp) << sh));
    }
}

__global__ void __launch_bounds__(256) scores_u8_kernel(const uint8_t* __restrict__ q, const uint8_t* __restrict__ k,
                                                        uint8_t* __restrict__ out, int64_t R, int64_t N, int D) {
    const int64_t total = R * N;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t r = i / N;
        const uint8_t* qr = q + r * D;
        const uint8_t* kr = k + i * D;
        unsigned acc = 0;
        for (int d = 0; d < D; ++d) acc += __popc((unsigned)(uint8_t)(~(qr[d] ^ kr[d])));
        out[i] = (uint8_t)acc;
    }
}

}  // namespace

extern "C" int sl_pack_signbits(const void* d_x, int dtype, int64_t n_elems, void* d_out, void* stream) {
    SL_REQUIRE(d_x && d_out, SL_EINVAL, "sl_pack_signbits: null pointer");
    SL_REQUIRE(n_elems >= 0 && n_elems % 8 == 0, SL_ESHAPE, "sl_pack_signbits: n_elems=%lld not a multiple of 8",
               (long long)n_elems);
    SL_REQUIRE(sl::aligned16(d_x), SL_EALIGN, "sl_pack_signbits: input not 16-byte aligned");
    if (n_elems == 0) return SL_OK;
    const int64_t n_bytes = n_elems / 8;
    int64_t blocks = (n_bytes + 255) / 256;
    const int64_t cap = (int64_t)sl::sm_count() * 16;
    if (blocks > cap) blocks = cap;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    uint8_t* o = static_cast<uint8_t*>(d_out);
    switch (dtype) {
        case SL_BF16: pack_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, s>>>((const __nv_bfloat16*)d_x, o, n_bytes); break;
        case SL_F16: pack_kernel<__half><<<(unsigned)blocks, 256, 0, s>>>((const __half*)d_x, o, n_bytes); break;
        case SL_F32: pack_kernel<float><<<(unsigned)blocks, 256, 0, s>>>((const float*)d_x, o, n_bytes); break;
        case SL_BOOL: pack_kernel<uint8_t><<<(unsigned)blocks, 256, 0, s>>>((const uint8_t*)d_x, o, n_bytes); break;
        default: return sl::fail(SL_EINVAL, "sl_pack_signbits: unknown dtype %d", dtype);
    }
    SL_CUDA_OK(cudaGetLastError());
    return SL_OK;
}

extern "C" int sl_hamming_scores(const uint32_t* d_q, const uint32_t* d_k, int64_t k_batch_stride, int16_t* d_out,
                                 int B, int64_t N, int KH, int QH, int W, int gqa_layout, void* stream) {
    SL_REQUIRE(d_q && d_k && d_out, SL_EINVAL, "sl_hamming_scores: null pointer");
    SL_REQUIRE(B > 0 && N >= 0 && KH > 0 && QH > 0 && QH % KH == 0, SL_ESHAPE,
               "sl_hamming_scores: bad shape B=%d N=%lld KH=%d QH=%d", B, (long long)N, KH, QH);
    SL_REQUIRE(W == 1 || W == 2 || W == 4 || W == 8, SL_ESHAPE, "sl_hamming_scores: W=%d not in {1,2,4,8}", W);
    SL_REQUIRE(gqa_layout == SL_GQA_INTERLEAVED || gqa_layout == SL_GQA_BLOCKED, SL_EINVAL,
               "sl_hamming_scores: unknown gqa_layout %d", gqa_layout);
    SL_REQUIRE(k_batch_stride == 0 || k_batch_stride >= N * KH * W, SL_ESHAPE, "sl_hamming_scores: batch stride shorter than a batch row");
    SL_REQUIRE((int64_t)QH * W * 4 <= 48 * 1024, SL_ESHAPE, "sl_hamming_scores: QH*W too large");
    SL_REQUIRE(B <= 65535, SL_ESHAPE, "sl_hamming_scores: B > 65535");
    if (W == 4) SL_REQUIRE(sl::aligned16(d_k) && (k_batch_stride % 4 == 0), SL_EALIGN, "sl_hamming_scores: codes not 16-byte aligned");
    if (N == 0) return SL_OK;
    const int G = QH / KH;
    const int64_t total = N * KH;
    int64_t bx = (total + 255) / 256;
    const int64_t cap = std::max<int64_t>(1, (int64_t)sl::sm_count() * 8 / B);
    if (bx > cap) bx = cap;
    dim3 grid((unsigned)bx, (unsigned)B);
    const size_t smem = (size_t)QH * W * 4;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (W == 4 && KH <= 32 && 32 % KH == 0 && sliced_planes(G) > 0) {
        const uint4* k16 = reinterpret_cast<const uint4*>(d_k);
        const int64_t kb16 = k_batch_stride / 4;
        switch (sliced_planes(G)) {
            case 1: scores_sliced_kernel<1><<<grid, 256, 0, s>>>(d_q, k16, kb16, d_out, N, KH, G, gqa_layout); break;
            case 2: scores_sliced_kernel<2><<<grid, 256, 0, s>>>(d_q, k16, kb16, d_out, N, KH, G, gqa_layout); break;
            case 3: scores_sliced_kernel<3><<<grid, 256, 0, s>>>(d_q, k16, kb16, d_out, N, KH, G, gqa_layout); break;
            default: scores_sliced_kernel<4><<<grid, 256, 0, s>>>(d_q, k16, kb16, d_out, N, KH, G, gqa_layout); break;
        }
        SL_CUDA_OK(cudaGetLastError());
        return SL_OK;
    }
    switch (W) {
        case 1: scores_kernel<1><<<grid, 256, smem, s>>>(d_q, d_k, k_batch_stride, d_out, N, KH, G, gqa_layout); break;
        case 2: scores_kernel<2><<<grid, 256, smem, s>>>(d_q, d_k, k_batch_stride, d_out, N, KH, G, gqa_layout); break;
        case 4: scores_kernel<4><<<grid, 256, smem, s>>>(d_q, d_k, k_batch_stride, d_out, N, KH, G, gqa_layout); break;
        default: scores_kernel<8><<<grid, 256, smem, s>>>(d_q, d_k, k_batch_stride, d_out, N, KH, G, gqa_layout); break;
    }
    SL_CUDA_OK(cudaGetLastError());
    return SL_OK;
}

extern "C" int sl_hamming_scores_u8(const uint8_t* d_q, const uint8_t* d_k, uint8_t* d_out, int64_t R, int64_t N,
                                    int D, void* stream) {
    SL_REQUIRE(d_q && d_k && d_out, SL_EINVAL, "sl_hamming_scores_u8: null pointer");
    SL_REQUIRE(R > 0 && N >= 0 && D > 0, SL_ESHAPE, "sl_hamming_scores_u8: bad shape");
    if (N == 0) return SL_OK;
    int64_t blocks = (R * N + 255) / 256;
    const int64_t cap = (int64_t)sl::sm_count() * 8;
    if (blocks > cap) blocks = cap;
    scores_u8_kernel<<<(unsigned)blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(d_q, d_k, d_out, R, N, D);
    SL_CUDA_OK(cudaGetLastError());
    return SL_OK;
}
