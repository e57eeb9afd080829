// Sparse GQA decode attention over an index list: rows are gathered straight from the K/V
// caches (16-byte loads, one 256-byte row = half a warp for 2-byte types), online softmax in
// fp32, split over the list (flash-decoding style) with a small merge kernel combining the
// per-split partials. Also the LSE merge across sequence shards and the row-gather shim.
#include <type_traits>

#include "sl_attn.cuh"

namespace {

constexpr int AT = 256;            // threads per CTA
constexpr int AW = AT / 32;        // warps
constexpr int PF = 4;              // row groups in flight per warp
constexpr int MAX_SPLITS = sl::ATTN_MAX_SPLITS;
constexpr float LOG2E = 1.4426950408889634f;
constexpr float LN2 = 0.6931471805599453f;

using sl::AttnArgs;

__device__ __forceinline__ float ex2(float x) { return exp2f(x); }

template <typename T, int G>
__global__ void __launch_bounds__(AT, (G * (16 / sizeof(T)) > 32) ? 1 : 2) sparse_attn_kernel(const AttnArgs a) {
    constexpr int EPL = 16 / sizeof(T);       // elements per lane
    constexpr int LPR = 128 / EPL;            // lanes per row
    constexpr int RPW = 32 / LPR;             // rows per warp step
    __shared__ float sm_acc[AW][G][128];
    __shared__ float sm_m[AW][G], sm_l[AW][G];

    sl::pdl_trigger();
    sl::pdl_wait();
    const int sp = blockIdx.x, h = blockIdx.y, b = blockIdx.z, KH = a.KH;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int sub = lane % LPR, rs = lane / LPR;
    const int n = a.cnt[b * KH + h];
    const int per = (n + a.splits - 1) / a.splits;
    const int lo = min(n, sp * per), hi = min(n, lo + per);
    const int* list = a.idx + ((long long)b * KH + h) * a.cap;
    const long long hoff = (long long)b * a.kv_b + (long long)(h / a.kv_div) * a.head_stride + sub * EPL;
    const T* kb = reinterpret_cast<const T*>(a.k) + hoff;
    const T* vb = reinterpret_cast<const T*>(a.v) + hoff;
    const long long row_stride = a.tok_stride;

    float qf[G][EPL];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        const int qh = a.layout == SL_GQA_INTERLEAVED ? g * KH + h : h * G + g;
        const T* qp = reinterpret_cast<const T*>(a.q) + ((long long)b * KH * G + qh) * 128 + sub * EPL;
        const uint4 raw = *reinterpret_cast<const uint4*>(qp);
        const T* qv = reinterpret_cast<const T*>(&raw);
#pragma unroll
        for (int e = 0; e < EPL; ++e) qf[g][e] = sl::VT<T>::to_f(qv[e]) * (0.08838834764831845f * LOG2E);
    }
    float m[G], l[G], acc[G][EPL];
#pragma unroll
    for (int g = 0; g < G; ++g) {
        m[g] = -INFINITY; l[g] = 0.0f;
#pragma unroll
        for (int e = 0; e < EPL; ++e) acc[g][e] = 0.0f;
    }

    const int step = AW * RPW;
    const int nit = (hi - lo + step - 1) / step;
    uint4 kbuf[PF], vbuf[PF];
    bool okb[PF];
    auto issue = [&](int it, int slot) {
        const int j = lo + it * step + warp * RPW + rs;
        const bool ok = it < nit && j < hi;
        okb[slot] = ok;
        if (ok) {
            const long long tok = list[j];
            kbuf[slot] = sl::ld_gather_v4(kb + tok * row_stride);
            vbuf[slot] = sl::ld_gather_v4(vb + tok * row_stride);
        }
    };
#pragma unroll
    for (int p = 0; p < PF; ++p) issue(p, p);
    for (int it0 = 0; it0 < nit; it0 += PF) {
#pragma unroll
        for (int p = 0; p < PF; ++p) {
            if (it0 + p < nit) {   // warp-uniform
                const bool ok = okb[p];
                const T* kv = reinterpret_cast<const T*>(&kbuf[p]);
                const T* vv = reinterpret_cast<const T*>(&vbuf[p]);
                float kf[EPL], vf[EPL];
#pragma unroll
                for (int e = 0; e < EPL; ++e) {
                    kf[e] = ok ? sl::VT<T>::to_f(kv[e]) : 0.0f;
                    vf[e] = ok ? sl::VT<T>::to_f(vv[e]) : 0.0f;
                }
#pragma unroll
                for (int g = 0; g < G; ++g) {
                    float s = 0.0f;
#pragma unroll
                    for (int e = 0; e < EPL; ++e) s = fmaf(qf[g][e], kf[e], s);
#pragma unroll
                    for (int d = LPR / 2; d > 0; d >>= 1) s += __shfl_xor_sync(0xffffffffu, s, d);
                    if (ok) {
                        const float mn = fmaxf(m[g], s);
                        const float corr = ex2(m[g] - mn);      // m = -inf -> 0
                        const float p_ = ex2(s - mn);
                        l[g] = l[g] * corr + p_;
#pragma unroll
                        for (int e = 0; e < EPL; ++e) acc[g][e] = fmaf(acc[g][e], corr, p_ * vf[e]);
                        m[g] = mn;
                    }
                }
                issue(it0 + p + PF, p);
            }
        }
    }

    // ---- merge the row slots of a warp (lanes holding the same columns)
#pragma unroll
    for (int d = LPR; d < 32; d <<= 1) {
#pragma unroll
        for (int g = 0; g < G; ++g) {
            const float mo = __shfl_xor_sync(0xffffffffu, m[g], d);
            const float lo_ = __shfl_xor_sync(0xffffffffu, l[g], d);
            const float mn = fmaxf(m[g], mo);
            const float c0 = mn == -INFINITY ? 0.0f : ex2(m[g] - mn);
            const float c1 = mn == -INFINITY ? 0.0f : ex2(mo - mn);
            l[g] = l[g] * c0 + lo_ * c1;
#pragma unroll
            for (int e = 0; e < EPL; ++e) {
                const float ao = __shfl_xor_sync(0xffffffffu, acc[g][e], d);
                acc[g][e] = acc[g][e] * c0 + ao * c1;
            }
            m[g] = mn;
        }
    }
    if (rs == 0) {
#pragma unroll
        for (int g = 0; g < G; ++g) {
#pragma unroll
            for (int e = 0; e < EPL; ++e) sm_acc[warp][g][sub * EPL + e] = acc[g][e];
            if (sub == 0) { sm_m[warp][g] = m[g]; sm_l[warp][g] = l[g]; }
        }
    }
    __syncthreads();

    // ---- merge the warps of the CTA
    const long long bh = (long long)b * KH + h;
    float* part = a.part + (bh * a.splits + sp) * G * 130;
    for (int e = tid; e < G * 128; e += AT) {
        const int g = e >> 7, col = e & 127;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < AW; ++w) M = fmaxf(M, sm_m[w][g]);
        float L = 0.0f, O = 0.0f;
        if (M != -INFINITY) {
#pragma unroll
            for (int w = 0; w < AW; ++w) {
                const float c = ex2(sm_m[w][g] - M);
                L += sm_l[w][g] * c;
                O += sm_acc[w][g][col] * c;
            }
        }
        if (a.splits == 1) {
            const int qh = a.layout == SL_GQA_INTERLEAVED ? g * KH + h : h * G + g;
            const long long o = ((long long)b * KH * G + qh) * 128 + col;
            reinterpret_cast<T*>(a.out)[o] = sl::VT<T>::from_f(L > 0.0f ? O / L : 0.0f);
            if (a.lse && col == 0) a.lse[(long long)b * KH * G + qh] = L > 0.0f ? (M + log2f(L)) * LN2 : -INFINITY;
        } else {
            part[g * 130 + col] = O;
            if (col == 0) { part[g * 130 + 128] = M; part[g * 130 + 129] = L; }
        }
    }
}

// One CTA per query head merges the partials of its splits: thread (grp, col) accumulates the
// splits s = grp (mod 4) of output column col with every load in flight at once.
template <typename T>
__global__ void __launch_bounds__(512) attn_merge_kernel(const float* __restrict__ part, int splits, int G, int KH,
                                                         int layout, T* __restrict__ out, float* __restrict__ lse) {
    __shared__ float s_m[sl::ATTN_MAX_SPLITS], s_l[sl::ATTN_MAX_SPLITS], s_w[sl::ATTN_MAX_SPLITS];
    __shared__ float red[4][128];
    sl::pdl_trigger();
    sl::pdl_wait();
    const int g = blockIdx.x % G;
    const long long bh = blockIdx.x / G;
    const int h = (int)(bh % KH);
    const long long b = bh / KH;
    const int tid = threadIdx.x, col = tid & 127, grp = tid >> 7;
    const float* pb = part + (bh * splits * G + g) * 130;             // split s at pb + s*G*130
    const long long sstride = (long long)G * 130;
    float v[sl::ATTN_MAX_SPLITS / 4];
#pragma unroll
    for (int j = 0; j < sl::ATTN_MAX_SPLITS / 4; ++j) {
        const int s = grp + 4 * j;
        v[j] = s < splits ? __ldcg(pb + s * sstride + col) : 0.0f;
    }
    if (tid < splits) {
        s_m[tid] = __ldcg(pb + tid * sstride + 128);
        s_l[tid] = __ldcg(pb + tid * sstride + 129);
    }
    __syncthreads();
    float M = -INFINITY;
    for (int s = 0; s < splits; ++s) M = fmaxf(M, s_m[s]);
    if (tid < splits) s_w[tid] = M == -INFINITY ? 0.0f : exp2f(s_m[tid] - M);
    __syncthreads();
    float acc = 0.0f;
#pragma unroll
    for (int j = 0; j < sl::ATTN_MAX_SPLITS / 4; ++j) {
        const int s = grp + 4 * j;
        if (s < splits) acc = fmaf(v[j], s_w[s], acc);
    }
    red[grp][col] = acc;
    __syncthreads();
    if (grp == 0) {
        float L = 0.0f;
        for (int s = 0; s < splits; ++s) L = fmaf(s_l[s], s_w[s], L);
        const float O = (red[0][col] + red[1][col]) + (red[2][col] + red[3][col]);
        const int qh = layout == SL_GQA_INTERLEAVED ? g * KH + h : h * G + g;
        const long long o = ((long long)b * KH * G + qh) * 128 + col;
        out[o] = sl::VT<T>::from_f(L > 0.0f ? O / L : 0.0f);
        if (lse && col == 0) lse[(long long)b * KH * G + qh] = L > 0.0f ? (M + log2f(L)) * LN2 : -INFINITY;
    }
}

template <typename T>
__global__ void __launch_bounds__(128) merge_lse_kernel(const float* __restrict__ o, const float* __restrict__ lse,
                                                        int R, long long rows, T* __restrict__ out) {
    const long long row = blockIdx.x;
    const int col = threadIdx.x;
    float M = -INFINITY;
    for (int r = 0; r < R; ++r) M = fmaxf(M, lse[r * rows + row]);
    float L = 0.0f, O = 0.0f;
    if (M != -INFINITY) {
        for (int r = 0; r < R; ++r) {
            const float w = expf(lse[r * rows + row] - M);
            L += w;
            O += w * o[(r * rows + row) * 128 + col];
        }
    }
    out[row * 128 + col] = sl::VT<T>::from_f(L > 0.0f ? O / L : 0.0f);
}

__global__ void __launch_bounds__(256) gather_rows_kernel(const unsigned char* __restrict__ cache, long long bstride_bytes,
                                                          int row_bytes, const int* __restrict__ idx, int cap, int KH,
                                                          int budget, unsigned char* __restrict__ out) {
    // one warp-group of row_bytes/16 lanes copies one row
    const int lanes = row_bytes / 16;
    const int rows_per_block = 256 / lanes;
    const int b = blockIdx.y;
    const long long r = (long long)blockIdx.x * rows_per_block + threadIdx.x / lanes;   // r = j*KH + h
    if (threadIdx.x / lanes >= rows_per_block || r >= (long long)budget * KH) return;
    const int j = (int)(r / KH), h = (int)(r % KH);
    const long long tok = idx[((long long)b * KH + h) * cap + j];
    const uint4 v = sl::ld_gather_v4(cache + b * bstride_bytes + (tok * KH + h) * row_bytes + (threadIdx.x % lanes) * 16);
    *reinterpret_cast<uint4*>(out + (((long long)b * budget + j) * KH + h) * row_bytes + (threadIdx.x % lanes) * 16) = v;
}

int pick_splits(int B, int KH, int cap) {
    const int ctas = B * KH;
    int s = (4 * sl::sm_count() + ctas - 1) / ctas;
    const int by_rows = std::max(1, cap / 64);
    s = std::min(s, std::min(by_rows, MAX_SPLITS));
    return std::max(s, 1);
}

template <typename T, int G>
int launch_attn(const AttnArgs& a, cudaStream_t s) {
    dim3 grid((unsigned)a.splits, (unsigned)a.KH, (unsigned)a.B);
    SL_CUDA_OK(sl::launch_kernel(sparse_attn_kernel<T, G>, grid, dim3(AT), 0, s, false, a));
    if (a.splits > 1) return sl::launch_attn_merge(a, G, sizeof(T) == 4 ? SL_F32 : (std::is_same<T, __half>::value ? SL_F16 : SL_BF16), s);
    return SL_OK;
}

template <typename T>
int dispatch_g(const AttnArgs& a, int G, cudaStream_t s) {
    switch (G) {
        case 1: return launch_attn<T, 1>(a, s);
        case 2: return launch_attn<T, 2>(a, s);
        case 3: return launch_attn<T, 3>(a, s);
        case 4: return launch_attn<T, 4>(a, s);
        case 5: return launch_attn<T, 5>(a, s);
        case 6: return launch_attn<T, 6>(a, s);
        case 7: return launch_attn<T, 7>(a, s);
        case 8: return launch_attn<T, 8>(a, s);
        default: return sl::fail(SL_ESHAPE, "sl_sparse_attn_decode: group size %d not in 1..8", G);
    }
}

}  // namespace

namespace sl {
int launch_attn_merge(const AttnArgs& a, int G, int dtype, cudaStream_t s) {
    const unsigned blocks = (unsigned)(a.B * a.KH * G);
    switch (dtype) {
        case SL_BF16: SL_CUDA_OK(launch_kernel(attn_merge_kernel<__nv_bfloat16>, dim3(blocks), dim3(512), 0, s, false, (const float*)a.part, a.splits, G, a.KH, a.layout, (__nv_bfloat16*)a.out, a.lse)); break;
        case SL_F16: SL_CUDA_OK(launch_kernel(attn_merge_kernel<__half>, dim3(blocks), dim3(512), 0, s, false, (const float*)a.part, a.splits, G, a.KH, a.layout, (__half*)a.out, a.lse)); break;
        default: SL_CUDA_OK(launch_kernel(attn_merge_kernel<float>, dim3(blocks), dim3(512), 0, s, false, (const float*)a.part, a.splits, G, a.KH, a.layout, (float*)a.out, a.lse)); break;
    }
    return SL_OK;
}
}  // namespace sl

extern "C" size_t sl_sparse_attn_workspace_bytes(int B, int KH, int QH) {
    if (B <= 0 || KH <= 0 || QH <= 0) return 0;
    (void)KH;
    return (size_t)B * QH * MAX_SPLITS * 130 * 4;
}

static int attn_decode(const void* d_q, const void* d_k, const void* d_v, int dtype, const sl_kv_layout* kv,
                       const int32_t* d_idx, int idx_capacity, const int32_t* d_cnt, int B, int KH, int QH,
                       int gqa_layout, void* d_out, float* d_lse, void* d_workspace, size_t workspace_bytes,
                       const sl_attn_fill* fill, void* stream) {
    SL_REQUIRE(d_q && d_k && d_v && kv && d_idx && d_cnt && d_out && d_workspace, SL_EINVAL, "sl_sparse_attn_decode: null pointer");
    SL_REQUIRE(B > 0 && KH > 0 && QH > 0 && QH % KH == 0 && idx_capacity > 0, SL_ESHAPE, "sl_sparse_attn_decode: bad shape");
    SL_REQUIRE(B <= 65535 && KH <= 65535, SL_ESHAPE, "sl_sparse_attn_decode: B or KH > 65535");
    SL_REQUIRE(gqa_layout == SL_GQA_INTERLEAVED || gqa_layout == SL_GQA_BLOCKED, SL_EINVAL,
               "sl_sparse_attn_decode: unknown gqa_layout %d", gqa_layout);
    SL_REQUIRE(dtype == SL_BF16 || dtype == SL_F32 || dtype == SL_F16, SL_EINVAL, "sl_sparse_attn_decode: unsupported dtype %d", dtype);
    SL_REQUIRE(kv->list_heads_per_kv_head >= 1 && KH % kv->list_heads_per_kv_head == 0, SL_ESHAPE,
               "sl_sparse_attn_decode: %d list heads do not divide into groups of %d per kv head", KH, kv->list_heads_per_kv_head);
    SL_REQUIRE(kv->batch_stride >= 0 && kv->token_stride >= 128 && kv->head_stride >= 128, SL_ESHAPE,
               "sl_sparse_attn_decode: cache strides must leave room for a 128-value row");
    const int esz = dtype == SL_F32 ? 4 : 2;
    SL_REQUIRE(sl::aligned16(d_q) && sl::aligned16(d_k) && sl::aligned16(d_v) && (kv->batch_stride * esz) % 16 == 0 &&
                   (kv->token_stride * esz) % 16 == 0 && (kv->head_stride * esz) % 16 == 0, SL_EALIGN,
               "sl_sparse_attn_decode: q/k/v and the cache strides must be 16-byte aligned");
    SL_REQUIRE(workspace_bytes >= sl_sparse_attn_workspace_bytes(B, KH, QH), SL_EWORKSPACE,
               "sl_sparse_attn_decode: workspace %zu < required %zu", workspace_bytes, sl_sparse_attn_workspace_bytes(B, KH, QH));
    SL_REQUIRE(sl::aligned16(d_workspace), SL_EALIGN, "sl_sparse_attn_decode: workspace not 16-byte aligned");
    AttnArgs a = {};
    a.q = d_q; a.k = d_k; a.v = d_v; a.kv_b = kv->batch_stride;
    a.tok_stride = kv->token_stride; a.head_stride = kv->head_stride; a.kv_div = kv->list_heads_per_kv_head;
    a.idx = d_idx; a.cap = idx_capacity; a.cnt = d_cnt;
    a.B = B; a.KH = KH; a.layout = gqa_layout;
    a.splits = pick_splits(B, KH, idx_capacity);
    a.out = d_out; a.lse = d_lse;
    a.part = static_cast<float*>(d_workspace);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    const int G = QH / KH;
    if (fill) {
        SL_REQUIRE(dtype == SL_BF16 && G <= 16, SL_ESHAPE, "sl_sparse_attn_decode_fill: bf16 and at most 16 query heads per list head");
        SL_REQUIRE(fill->d_tokens && fill->k_backing && fill->v_backing, SL_EINVAL, "sl_sparse_attn_decode_fill: null pointer");
        const sl_kv_layout& bk = fill->backing;
        SL_REQUIRE(bk.batch_stride >= 0 && bk.token_stride >= 128 && bk.head_stride >= 128 &&
                       bk.list_heads_per_kv_head == kv->list_heads_per_kv_head, SL_ESHAPE,
                   "sl_sparse_attn_decode_fill: backing-store strides must leave room for a 128-value row and group the list heads as the resident buffers do");
        SL_REQUIRE(sl::aligned16(fill->k_backing) && sl::aligned16(fill->v_backing) && (bk.batch_stride * 2) % 16 == 0 &&
                       (bk.token_stride * 2) % 16 == 0 && (bk.head_stride * 2) % 16 == 0, SL_EALIGN,
                   "sl_sparse_attn_decode_fill: the backing store and its strides must be 16-byte aligned");
        a.tok = fill->d_tokens; a.k_back = fill->k_backing; a.v_back = fill->v_backing;
        a.back_b = bk.batch_stride; a.back_tok = bk.token_stride; a.back_head = bk.head_stride;
        a.fill_write = fill->read_only ? 0 : 1;
    }
    if (dtype == SL_BF16 && G <= 16) {
        // read-only fill: the evictions of the same step run beside this launch, one CTA per (row, head): leave them their SMs
        a.splits = sl::attn_mma_splits(B, KH, idx_capacity, (fill && fill->read_only) ? std::min(B * KH, 32) : 0);
        return sl::launch_attn_mma(a, G, s);
    }
    switch (dtype) {
        case SL_BF16: return dispatch_g<__nv_bfloat16>(a, G, s);
        case SL_F16: return dispatch_g<__half>(a, G, s);
        default: return dispatch_g<float>(a, G, s);
    }
}

extern "C" int sl_sparse_attn_decode_ex(const void* d_q, const void* d_k, const void* d_v, int dtype, const sl_kv_layout* kv,
                                        const int32_t* d_idx, int idx_capacity, const int32_t* d_cnt, int B, int KH, int QH,
                                        int gqa_layout, void* d_out, float* d_lse, void* d_workspace, size_t workspace_bytes,
                                        void* stream) {
    return attn_decode(d_q, d_k, d_v, dtype, kv, d_idx, idx_capacity, d_cnt, B, KH, QH, gqa_layout, d_out, d_lse, d_workspace,
                       workspace_bytes, nullptr, stream);
}

extern "C" int sl_sparse_attn_decode_fill(const void* d_q, void* d_k_resident, void* d_v_resident, int dtype,
                                          const sl_kv_layout* resident, const int32_t* d_slots, int idx_capacity,
                                          const int32_t* d_cnt, int B, int KH, int QH, int gqa_layout, void* d_out, float* d_lse,
                                          void* d_workspace, size_t workspace_bytes, const sl_attn_fill* fill, void* stream) {
    SL_REQUIRE(fill, SL_EINVAL, "sl_sparse_attn_decode_fill: null fill description");
    return attn_decode(d_q, d_k_resident, d_v_resident, dtype, resident, d_slots, idx_capacity, d_cnt, B, KH, QH, gqa_layout,
                       d_out, d_lse, d_workspace, workspace_bytes, fill, stream);
}

extern "C" int sl_sparse_attn_decode(const void* d_q, const void* d_k, const void* d_v, int dtype,
                                     int64_t kv_batch_stride, const int32_t* d_idx, int idx_capacity,
                                     const int32_t* d_cnt, int B, int KH, int QH, int gqa_layout, void* d_out,
                                     float* d_lse, void* d_workspace, size_t workspace_bytes, void* stream) {
    const sl_kv_layout kv = {kv_batch_stride, (int64_t)KH * 128, 128, 1};
    return sl_sparse_attn_decode_ex(d_q, d_k, d_v, dtype, &kv, d_idx, idx_capacity, d_cnt, B, KH, QH, gqa_layout, d_out,
                                    d_lse, d_workspace, workspace_bytes, stream);
}

extern "C" int sl_merge_lse(const float* d_o, const float* d_lse, int R, int64_t rows, int dtype, void* d_out, void* stream) {
    SL_REQUIRE(d_o && d_lse && d_out, SL_EINVAL, "sl_merge_lse: null pointer");
    SL_REQUIRE(R > 0 && rows >= 0 && rows <= 0x7fffffffLL, SL_ESHAPE, "sl_merge_lse: bad shape");
    if (rows == 0) return SL_OK;
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    switch (dtype) {
        case SL_BF16: merge_lse_kernel<__nv_bfloat16><<<(unsigned)rows, 128, 0, s>>>(d_o, d_lse, R, rows, (__nv_bfloat16*)d_out); break;
        case SL_F16: merge_lse_kernel<__half><<<(unsigned)rows, 128, 0, s>>>(d_o, d_lse, R, rows, (__half*)d_out); break;
        case SL_F32: merge_lse_kernel<float><<<(unsigned)rows, 128, 0, s>>>(d_o, d_lse, R, rows, (float*)d_out); break;
        default: return sl::fail(SL_EINVAL, "sl_merge_lse: unsupported dtype %d", dtype);
    }
    SL_CUDA_OK(cudaGetLastError());
    return SL_OK;
}

extern "C" int sl_gather_rows(const void* d_cache, int64_t batch_stride, int elem_bytes, const int32_t* d_idx,
                              int idx_capacity, int B, int KH, int budget, void* d_out, void* stream) {
    SL_REQUIRE(d_cache && d_idx && d_out, SL_EINVAL, "sl_gather_rows: null pointer");
    SL_REQUIRE(B > 0 && B <= 65535 && KH > 0 && budget >= 0 && budget <= idx_capacity, SL_ESHAPE, "sl_gather_rows: bad shape");
    SL_REQUIRE(elem_bytes == 2 || elem_bytes == 4, SL_EINVAL, "sl_gather_rows: elem_bytes must be 2 or 4");
    SL_REQUIRE(sl::aligned16(d_cache) && sl::aligned16(d_out) && (batch_stride * elem_bytes) % 16 == 0, SL_EALIGN,
               "sl_gather_rows: buffers must be 16-byte aligned");
    if (budget == 0) return SL_OK;
    const int row_bytes = 128 * elem_bytes;
    const int rows_per_block = 256 / (row_bytes / 16);
    const long long rows = (long long)budget * KH;
    dim3 grid((unsigned)((rows + rows_per_block - 1) / rows_per_block), (unsigned)B);
    gather_rows_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
        static_cast<const unsigned char*>(d_cache), batch_stride * elem_bytes, row_bytes, d_idx, idx_capacity, KH, budget,
        static_cast<unsigned char*>(d_out));
    SL_CUDA_OK(cudaGetLastError());
    return SL_OK;
}

// ---- sparse attention without a caller workspace -------------------------------------------
// Some callers of this library are not allowed to allocate device memory at the point where they
// run attention: a serving engine that handed every free byte of HBM to its KV-cache pool at
// start-up, or a latency-critical decode loop in which cudaMalloc / cudaFree are banned because
// they can synchronise the whole device. For them the scratch of the split partials lives in
// this fixed array, which every GPU that loads the library keeps until the process exits.
// The name below is only a host-side handle: the device address is fetched once per device
// with cudaGetSymbolAddress (that device being current) and handed to the kernels.
static __device__ __align__(256) unsigned char g_attn_static_scratch[SL_ATTN_STATIC_SCRATCH_BYTES];

extern "C" int sl_sparse_attn_decode_static(const void* d_q, const void* d_k, const void* d_v, int dtype,
                                            int64_t kv_batch_stride, const int32_t* d_idx, int idx_capacity,
                                            const int32_t* d_cnt, int B, int KH, int QH, int gqa_layout, void* d_out,
                                            float* d_lse, void* stream) {
    SL_REQUIRE(B > 0 && KH > 0 && QH > 0, SL_ESHAPE, "sl_sparse_attn_decode_static: bad shape");
    const size_t need = sl_sparse_attn_workspace_bytes(B, KH, QH);
    SL_REQUIRE(need <= (size_t)SL_ATTN_STATIC_SCRATCH_BYTES, SL_EWORKSPACE,
               "sl_sparse_attn_decode_static: B*QH = %d needs %zu bytes of scratch but the built-in array holds %u; "
               "use sl_sparse_attn_decode with a caller-owned workspace",
               B * QH, need, (unsigned)SL_ATTN_STATIC_SCRATCH_BYTES);
    static void* scratch_of_device[64] = {nullptr};
    int dev = -1;
    SL_CUDA_OK(cudaGetDevice(&dev));
    SL_REQUIRE(dev >= 0 && dev < 64, SL_EINVAL, "sl_sparse_attn_decode_static: device ordinal %d out of range", dev);
    if (scratch_of_device[dev] == nullptr) {          // first call on this device: resolve the array's device address
        void* p = nullptr;
        SL_CUDA_OK(cudaGetSymbolAddress(&p, g_attn_static_scratch));
        SL_REQUIRE(p != nullptr, SL_ECUDA, "sl_sparse_attn_decode_static: no device address for the scratch array");
        scratch_of_device[dev] = p;
    }
    return sl_sparse_attn_decode(d_q, d_k, d_v, dtype, kv_batch_stride, d_idx, idx_capacity, d_cnt, B, KH, QH, gqa_layout,
                                 d_out, d_lse, scratch_of_device[dev], (size_t)SL_ATTN_STATIC_SCRATCH_BYTES, stream);
}
