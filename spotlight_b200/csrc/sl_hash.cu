// Hash stage: (optional RoPE) -> per-head MLP / linear projection -> sign -> 128-bit code,
// with the decode-step appends (code cache, K cache, V cache) fused into the same launch.
//
// One CTA owns one head and a tile of R rows (a row = one token of that head). The weight
// matrix of a layer is streamed once per CTA with 16-byte loads: thread (ks, cg) multiplies
// input rows ks, ks+KS, ... of W against columns [cg*CPT, cg*CPT+CPT), partial sums meet in
// shared memory. Rounding points follow the reference's torch operators in the run dtype:
// matmul (fp32 accumulate) -> round, + bias -> round, SiLU -> round, + residual -> round.
#include <cstdlib>

#include "sl_common.cuh"
#include "sl_mma.cuh"

namespace sl {
int launch_hash_encode_mma(const void* x, long long xs_b, long long xs_tok, long long xs_h, int B, long long T, int H, const sl_hash_params* hp,
                           uint32_t* codes, long long cs_b, cudaStream_t s);
int launch_hash_encode_tc(const void* x, long long xs_b, long long xs_tok, long long xs_h, int B, long long T, int H, const sl_hash_params* hp,
                          uint32_t* codes, long long cs_b, cudaStream_t s);
}

namespace {

constexpr int HT = 256;      // threads per CTA
constexpr int MAXD = 256;    // largest layer width

struct HashJob {
    const void* x; long long xs_b; long long T; int H; int B;
    long long xs_tok, xs_h;                          // elements between consecutive tokens / heads of x
    sl_hash_params hp;
    uint32_t* codes; long long cs_b;
    void* x_rot; long long xr_b;
    const void* cosr; const void* sinr;
    const void* v_src; void* v_dst; long long v_b;   // optional value-row append (decode)
    long long xr_h, v_h;                             // elements between consecutive heads of a row of x_rot / v_dst
    // position on the device (decode, optional): outputs move by *d_pos rows, cos/sin come from row *d_pos - tab_pos0
    const long long* d_pos;
    long long xr_tok, v_tok, code_tok;               // elements (code words) per position of x_rot / v_dst / codes
    long long tab_pos0;
    long long row_tiles;
};

struct HashArgs {
    HashJob job[2];
    int heads0;
    // Blocks with blockIdx.y >= heads do no hashing: they ask L2 for the code cache the scan of
    // this decode step is about to stream (rows 0..pos-1 of every batch element), so the fetch
    // from HBM overlaps this latency-bound kernel, which leaves most SMs idle.
    int heads;
    const unsigned char* pf_base; long long pf_bstride; long long pf_bytes; int pf_B;
    const long long* pf_pos; long long pf_row_bytes;      // position on the device: pf_bytes = *pf_pos * pf_row_bytes (capped)
};

constexpr int PF_PIECE = 2048;                     // bytes per bulk prefetch
constexpr long long PF_MAX_BYTES = 24ll << 20;     // what HBM delivers in the few us this kernel lasts

__device__ __forceinline__ void prefetch_codes(const HashArgs& args) {
    long long bytes = args.pf_bytes;
    if (args.pf_pos) {
        // Read before the wait on the preceding kernel, which may be the one that advances the position:
        // a stale value only makes the prefetch one row short.
        bytes = min(bytes, __ldcg(args.pf_pos) * args.pf_row_bytes);
        if (bytes <= 0) return;
    }
    const long long per_b = (bytes + PF_PIECE - 1) / PF_PIECE;
    const long long total = per_b * args.pf_B;
    const long long nthreads = (long long)(gridDim.y - args.heads) * gridDim.x * blockDim.x;
    long long p = ((long long)(blockIdx.y - args.heads) * gridDim.x + blockIdx.x) * blockDim.x + threadIdx.x;
    for (; p < total; p += nthreads) {
        const long long b = p / per_b, off = (p % per_b) * PF_PIECE;
        const unsigned size = (unsigned)min((long long)PF_PIECE, bytes - off);
        const unsigned char* ptr = args.pf_base + b * args.pf_bstride + off;
        asm volatile("cp.async.bulk.prefetch.L2.global [%0], %1;" ::"l"(ptr), "r"(size) : "memory");
    }
}

// Offsets of the R rows of a tile, computed once (integer divisions are kept out of the loops).
struct RowInfo {
    long long x, xrot, vsrc, vdst, code;
    long long trow;          // offset of the position's row in the cos / sin tables (0 without a device-side position)
    int valid;
};

template <typename T, int R>
__device__ __forceinline__ void stage_rows(const HashJob& J, int h, long long r0, RowInfo* rinfo, float* xa, float* xb) {
    const int tid = threadIdx.x;
    if (tid < R) {
        const long long rg = r0 + tid, rows = (long long)J.B * J.T;
        RowInfo ri = {};
        ri.valid = rg < rows;
        if (ri.valid) {
            long long b = rg, t = 0;
            if (J.T != 1) { b = rg / J.T; t = rg - b * J.T; }
            const long long th = t * J.H + h;
            const long long pos = J.d_pos ? __ldcg(J.d_pos) : 0;
            ri.trow = J.d_pos ? (pos - J.tab_pos0) * 128 : 0;
            ri.x = b * J.xs_b + t * J.xs_tok + h * J.xs_h;
            ri.xrot = b * J.xr_b + th * J.xr_h + pos * J.xr_tok;
            ri.vsrc = ((b * J.T + t) * J.H + h) * 128;
            ri.vdst = b * J.v_b + th * J.v_h + pos * J.v_tok;
            ri.code = b * J.cs_b + th * 4 + pos * J.code_tok;
        }
        rinfo[tid] = ri;
    }
    __syncthreads();
    // raw rows first, then the rotation (the rotated copy may overwrite the input in place); the cos / sin values
    // of an element are fetched together with it, so that the rotation does not wait for another trip to memory
    constexpr int EPT = (R * 128 + HT - 1) / HT;             // elements per thread
    float cs[EPT], sn[EPT];
#pragma unroll
    for (int i = 0; i < EPT; ++i) {
        const int e = tid + i * HT;
        cs[i] = 1.0f; sn[i] = 0.0f;
        if (e < R * 128) {
            const int r = e >> 7, j = e & 127;
            float val = 0.0f;
            if (rinfo[r].valid) {
                val = sl::VT<T>::to_f((reinterpret_cast<const T*>(J.x) + rinfo[r].x)[j]);
                if (J.v_dst) (reinterpret_cast<T*>(J.v_dst) + rinfo[r].vdst)[j] = (reinterpret_cast<const T*>(J.v_src) + rinfo[r].vsrc)[j];
            }
            if (J.cosr) {
                const long long trow = rinfo[r].trow;
                cs[i] = sl::VT<T>::to_f(reinterpret_cast<const T*>(J.cosr)[trow + j]);
                sn[i] = sl::VT<T>::to_f(reinterpret_cast<const T*>(J.sinr)[trow + j]);
            }
            xb[r * MAXD + j] = val;
        }
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < EPT; ++i) {
        const int e = tid + i * HT;
        if (e < R * 128) {
            const int r = e >> 7, j = e & 127;
            float val = xb[r * MAXD + j];
            if (J.cosr) {
                const float other = xb[r * MAXD + (j ^ 64)];
                const float rot = j < 64 ? -other : other;
                val = sl::VT<T>::round(__fadd_rn(sl::VT<T>::round(__fmul_rn(val, cs[i])), sl::VT<T>::round(__fmul_rn(rot, sn[i]))));
            }
            if (J.x_rot && rinfo[r].valid) (reinterpret_cast<T*>(J.x_rot) + rinfo[r].xrot)[j] = sl::VT<T>::from_f(val);
            xa[r * MAXD + j] = val;
        }
    }
    __syncthreads();
}

// Partial sums of the k-splits -> rounded layer output (bias, SiLU, residual at torch's rounding points).
template <typename T, int R>
__device__ __forceinline__ void finish_layer(const HashJob& J, int h, int layer, int dout, int KS, const float* red,
                                             const float* xin, float* xout, const T* bias_staged = nullptr) {
    const T* bias = J.hp.d_b[layer] ? (bias_staged ? bias_staged : reinterpret_cast<const T*>(J.hp.d_b[layer]) + (long long)h * dout) : nullptr;
    const bool act = layer < J.hp.n_layers - 1;
    for (int e = threadIdx.x; e < R * dout; e += HT) {
        const int r = e / dout, j = e - r * dout;
        float y0 = 0.0f, y1 = 0.0f;
        for (int s = 0; s < KS; s += 2) {
            y0 += red[(s * R + r) * dout + j];
            y1 += red[((s + 1) * R + r) * dout + j];
        }
        float y = sl::VT<T>::round(y0 + y1);
        if (bias) y = sl::VT<T>::round(y + sl::VT<T>::to_f(bias[j]));
        if (act) y = sl::VT<T>::round(y / (1.0f + expf(-y)));
        if (J.hp.residue) y = sl::VT<T>::round(y + xin[r * MAXD + j]);
        xout[r * MAXD + j] = y;
    }
    __syncthreads();
}

template <int R>
__device__ __forceinline__ void sign_pack(const HashJob& J, const RowInfo* rinfo, const float* x) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (warp < 4) {                // warp w builds word w of each row's code
#pragma unroll
        for (int r = 0; r < R; ++r) {
            const unsigned word = __ballot_sync(0xffffffffu, x[r * MAXD + warp * 32 + lane] > 0.0f);
            if (lane == 0 && rinfo[r].valid) J.codes[rinfo[r].code + warp] = word;
        }
    }
}

// One layer with compile-time widths. The head's weight matrix is copied into shared memory by
// 16-byte cp.async (issued before the kernel waits for its predecessor); thread (ks, cg) then owns
// columns [cg*CPT, +CPT) and the input rows ks, ks + KS, ... and walks them in a ROLLED loop: the
// kernel runs once per decode step with a cold instruction cache, so its cost is the number of
// distinct instructions it executes, and an unrolled multiply-accumulate over register-held
// weights cost more in instruction fetch than in arithmetic. The order of the additions is the
// same as before (k ascending per thread, then the k-splits pairwise in finish_layer).
template <typename T, int DIN, int DOUT>
struct Layer {
    static constexpr int CPT = 16 / sizeof(T), NCG = DOUT / CPT, KS = HT / NCG, NLOAD = DIN / KS;
    static constexpr int BYTES = DIN * DOUT * (int)sizeof(T);
    static __device__ __forceinline__ void fetch(const void* wbase, int h, unsigned char* wsm) {
        const unsigned char* W = reinterpret_cast<const unsigned char*>(wbase) + (size_t)h * BYTES;
        const unsigned dst = (unsigned)__cvta_generic_to_shared(wsm);
#pragma unroll 4
        for (int i = threadIdx.x * 16; i < BYTES; i += HT * 16) cp_async16(dst + i, W + i);
        cp_async_commit();
    }
    template <int R>
    static __device__ __forceinline__ void mac(const unsigned char* wsm, const float* xin, float* red) {
        const int cg = threadIdx.x % NCG, ks = threadIdx.x / NCG;
        float acc[R][CPT];
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
            for (int c = 0; c < CPT; ++c) acc[r][c] = 0.0f;
        const unsigned char* wp = wsm + ((size_t)ks * DOUT + cg * CPT) * sizeof(T);
#pragma unroll 2
        for (int j = 0; j < NLOAD; ++j) {
            const uint4 wq = *reinterpret_cast<const uint4*>(wp + (size_t)j * KS * DOUT * sizeof(T));
            const T* wv = reinterpret_cast<const T*>(&wq);
            float wf[CPT];
#pragma unroll
            for (int c = 0; c < CPT; ++c) wf[c] = sl::VT<T>::to_f(wv[c]);
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const float xv = xin[r * MAXD + ks + j * KS];
#pragma unroll
                for (int c = 0; c < CPT; ++c) acc[r][c] = fmaf(xv, wf[c], acc[r][c]);
            }
        }
#pragma unroll
        for (int r = 0; r < R; ++r) {
            float4* dst = reinterpret_cast<float4*>(red + (ks * R + r) * DOUT + cg * CPT);
#pragma unroll
            for (int c = 0; c < CPT; c += 4) dst[c / 4] = make_float4(acc[r][c], acc[r][c + 1], acc[r][c + 2], acc[r][c + 3]);
        }
        __syncthreads();
    }
};

// Fixed shapes 128 -> 128 (NL = 1) and 128 -> DH -> 128 (NL = 2) in 2-byte types: every weight
// copy of the whole MLP is in flight before the input rows are even staged.
template <typename T, int R, int NL, int DH>
__global__ void __launch_bounds__(HT) hash_kernel_fixed(const HashArgs args) {
    using L0 = Layer<T, 128, NL == 1 ? 128 : DH>;
    using L1 = Layer<T, NL == 1 ? 128 : DH, 128>;
    extern __shared__ __align__(16) unsigned char smem_raw[];
    float* xa = reinterpret_cast<float*>(smem_raw);            // [R][MAXD]
    float* xb = xa + R * MAXD;                                 // [R][MAXD]
    float* red = xb + R * MAXD;                                // [KS][R][dout]
    unsigned char* w0 = reinterpret_cast<unsigned char*>(red + HT * R * 8);
    unsigned char* w1 = w0 + L0::BYTES;
    __shared__ RowInfo rinfo[R];
    const int hy = blockIdx.y;
    const HashJob& J = hy < args.heads0 ? args.job[0] : args.job[1];
    const int h = hy < args.heads0 ? hy : hy - args.heads0;
    sl::pdl_trigger();
    if (hy >= args.heads) { prefetch_codes(args); sl::pdl_wait(); return; }
    if ((long long)blockIdx.x >= J.row_tiles) { sl::pdl_wait(); return; }
    // the biases travel with the first weight matrix (16-byte pieces; a bias that is not 16-byte aligned is read in place)
    __shared__ __align__(16) unsigned char sbias[2][MAXD * sizeof(T)];
    bool staged[2] = {false, false};
#pragma unroll
    for (int l = 0; l < NL; ++l) {
        const int dout = l == NL - 1 ? 128 : DH;
        const unsigned char* bsrc = reinterpret_cast<const unsigned char*>(J.hp.d_b[l]) + (size_t)h * dout * sizeof(T);
        staged[l] = J.hp.d_b[l] != nullptr && (reinterpret_cast<uintptr_t>(bsrc) & 15u) == 0;
        if (staged[l] && threadIdx.x * 16 < dout * (int)sizeof(T))
            cp_async16((unsigned)__cvta_generic_to_shared(sbias[l]) + threadIdx.x * 16, bsrc + threadIdx.x * 16);
    }
    L0::fetch(J.hp.d_w[0], h, w0);
    if (NL == 2) L1::fetch(J.hp.d_w[1], h, w1);
    sl::pdl_wait();                 // weights are nobody's output; everything below may be
    stage_rows<T, R>(J, h, (long long)blockIdx.x * R, rinfo, xa, xb);
    if (NL == 2) cp_async_wait<1>(); else cp_async_wait<0>();
    __syncthreads();
    L0::template mac<R>(w0, xa, red);
    finish_layer<T, R>(J, h, 0, NL == 1 ? 128 : DH, L0::KS, red, xa, xb, staged[0] ? reinterpret_cast<const T*>(sbias[0]) : nullptr);
    if (NL == 2) {
        cp_async_wait<0>();
        __syncthreads();
        L1::template mac<R>(w1, xb, red);
        finish_layer<T, R>(J, h, 1, 128, L1::KS, red, xb, xa, staged[1] ? reinterpret_cast<const T*>(sbias[1]) : nullptr);
    }
    sign_pack<R>(J, rinfo, NL == 2 ? xa : xb);
}

// Any supported shape (runtime widths, up to three layers): weights are loaded layer by layer.
template <typename T, int R>
__global__ void __launch_bounds__(HT) hash_kernel_generic(const HashArgs args) {
    constexpr int CPT = 16 / sizeof(T);
    extern __shared__ __align__(16) unsigned char smem_raw[];
    float* xa = reinterpret_cast<float*>(smem_raw);
    float* xb = xa + R * MAXD;
    float* red = xb + R * MAXD;
    __shared__ RowInfo rinfo[R];
    const int hy = blockIdx.y;
    const HashJob& J = hy < args.heads0 ? args.job[0] : args.job[1];
    const int h = hy < args.heads0 ? hy : hy - args.heads0;
    sl::pdl_trigger();
    if (hy >= args.heads) { prefetch_codes(args); sl::pdl_wait(); return; }
    sl::pdl_wait();
    if ((long long)blockIdx.x >= J.row_tiles) return;
    const int tid = threadIdx.x;
    stage_rows<T, R>(J, h, (long long)blockIdx.x * R, rinfo, xa, xb);
    float* xin = xa;
    float* xout = xb;
    for (int layer = 0; layer < J.hp.n_layers; ++layer) {
        const int din = J.hp.dims[layer], dout = J.hp.dims[layer + 1];
        const int ncg = dout / CPT, KS = HT / ncg;
        const int cg = tid % ncg, ks = tid / ncg;
        const T* W = reinterpret_cast<const T*>(J.hp.d_w[layer]) + (long long)h * din * dout;
        float acc[R][CPT];
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
            for (int c = 0; c < CPT; ++c) acc[r][c] = 0.0f;
#pragma unroll 8
        for (int i = ks; i < din; i += KS) {
            const uint4 raw = sl::ld_gather_v4(W + (long long)i * dout + cg * CPT);
            const T* wv = reinterpret_cast<const T*>(&raw);
#pragma unroll
            for (int r = 0; r < R; ++r) {
                const float xv = xin[r * MAXD + i];
#pragma unroll
                for (int c = 0; c < CPT; ++c) acc[r][c] = fmaf(xv, sl::VT<T>::to_f(wv[c]), acc[r][c]);
            }
        }
#pragma unroll
        for (int r = 0; r < R; ++r)
#pragma unroll
            for (int c = 0; c < CPT; ++c) red[(ks * R + r) * dout + cg * CPT + c] = acc[r][c];
        __syncthreads();
        finish_layer<T, R>(J, h, layer, dout, KS, red, xin, xout);
        float* t = xin; xin = xout; xout = t;
    }
    sign_pack<R>(J, rinfo, xin);
}

int check_params(const char* fn, const sl_hash_params* p, int dtype) {
    SL_REQUIRE(p != nullptr, SL_EINVAL, "%s: null hash params", fn);
    SL_REQUIRE(p->n_layers >= 1 && p->n_layers <= 3, SL_ESHAPE, "%s: n_layers=%d not in 1..3", fn, p->n_layers);
    SL_REQUIRE(p->dims[0] == 128 && p->dims[p->n_layers] == 128, SL_ESHAPE, "%s: first and last hash dims must be 128", fn);
    const int cpt = dtype == SL_F32 ? 4 : 8;
    for (int i = 0; i <= p->n_layers; ++i) {
        const int d = p->dims[i];
        SL_REQUIRE(d == 32 || d == 64 || d == 128 || d == 256, SL_ESHAPE, "%s: hash dim %d not in {32,64,128,256}", fn, d);
        SL_REQUIRE(HT % (d / cpt) == 0, SL_ESHAPE, "%s: hash dim %d unsupported", fn, d);
    }
    for (int i = 0; i < p->n_layers; ++i) {
        SL_REQUIRE(p->d_w[i] != nullptr, SL_EINVAL, "%s: null weight of layer %d", fn, i);
        SL_REQUIRE(sl::aligned16(p->d_w[i]), SL_EALIGN, "%s: weight of layer %d not 16-byte aligned", fn, i);
        if (p->residue) SL_REQUIRE(p->dims[i] == p->dims[i + 1], SL_ESHAPE, "%s: residue needs equal layer widths", fn);
    }
    return SL_OK;
}

size_t hash_smem(int R) {
    // red = KS*R*dout floats with KS*ncg = HT  =>  HT*R*CPT floats at most; CPT <= 8
    return (size_t)2 * R * MAXD * 4 + (size_t)HT * R * 8 * 4;
}

typedef void (*hash_kernel_t)(const HashArgs);

template <typename T, int R>
hash_kernel_t pick_kernel(const HashArgs& args, size_t* weight_smem) {
    *weight_smem = 0;
    // the fixed-shape kernels need both jobs to share one of the shapes below
    const sl_hash_params& p = args.job[0].hp;
    bool same = true;
    if (args.job[1].H > 0) {
        const sl_hash_params& q = args.job[1].hp;
        same = q.n_layers == p.n_layers;
        for (int i = 0; same && i <= p.n_layers; ++i) same = q.dims[i] == p.dims[i];
    }
    if (sizeof(T) == 2 && same) {      // the head's weights live in shared memory
        if (p.n_layers == 1) { *weight_smem = 128 * 128 * 2; return hash_kernel_fixed<T, R, 1, 128>; }
        if (p.n_layers == 2 && p.dims[1] == 128) { *weight_smem = 2 * 128 * 128 * 2; return hash_kernel_fixed<T, R, 2, 128>; }
        if (p.n_layers == 2 && p.dims[1] == 256) { *weight_smem = 2 * 128 * 256 * 2; return hash_kernel_fixed<T, R, 2, 256>; }
    }
    return hash_kernel_generic<T, R>;
}

template <typename T>
int launch_T(const HashArgs& args, int total_heads, long long max_tiles, int R, size_t smem, cudaStream_t s) {
    size_t wsm = 0;
    unsigned pf_rows = 0;
    if (args.pf_base != nullptr && args.pf_bytes > 0) {     // fill the SMs the hash leaves idle
        const long long busy = max_tiles * total_heads, sms = sl::sm_count();
        pf_rows = (unsigned)std::max<long long>(1, (sms - busy) / max_tiles);
    }
    dim3 grid((unsigned)max_tiles, (unsigned)total_heads + pf_rows);
    hash_kernel_t kern = nullptr;
    switch (R) {
        case 1: kern = pick_kernel<T, 1>(args, &wsm); break;
        case 2: kern = pick_kernel<T, 2>(args, &wsm); break;
        case 4: kern = pick_kernel<T, 4>(args, &wsm); break;
        default: kern = pick_kernel<T, 8>(args, &wsm); break;
    }
    smem += wsm;
    SL_CUDA_OK(sl::ensure_dyn_smem(reinterpret_cast<const void*>(kern), smem));
    SL_CUDA_OK(sl::launch_kernel(kern, grid, dim3(HT), smem, s, false, args));
    return SL_OK;
}

int launch(const HashArgs& args, int dtype, int total_heads, long long rows_max, cudaStream_t s) {
    const int R = rows_max >= 8 ? 8 : rows_max >= 4 ? 4 : rows_max >= 2 ? 2 : 1;
    HashArgs a = args;
    a.heads = total_heads;
    long long max_tiles = 0;
    for (int j = 0; j < 2; ++j) {
        const long long rows = (long long)a.job[j].B * a.job[j].T;
        a.job[j].row_tiles = a.job[j].H > 0 ? (rows + R - 1) / R : 0;
        max_tiles = std::max(max_tiles, a.job[j].row_tiles);
    }
    SL_REQUIRE(max_tiles <= 0x7fffffffLL && total_heads <= 65535, SL_ESHAPE, "hash: grid too large");
    if (max_tiles == 0) return SL_OK;
    const size_t smem = hash_smem(R);
    switch (dtype) {
        case SL_BF16: return launch_T<__nv_bfloat16>(a, total_heads, max_tiles, R, smem, s);
        case SL_F16: return launch_T<__half>(a, total_heads, max_tiles, R, smem, s);
        case SL_F32: return launch_T<float>(a, total_heads, max_tiles, R, smem, s);
        default: return sl::fail(SL_EINVAL, "hash: unsupported dtype %d", dtype);
    }
}

}  // namespace

extern "C" int sl_decode_prepare(const void* d_q, const void* d_k, const void* d_v, int dtype, int B, int QH, int KH,
                                 const void* d_cos, const void* d_sin, const sl_hash_params* hash_q,
                                 const sl_hash_params* hash_k, void* d_q_rot, uint32_t* d_q_codes,
                                 uint32_t* d_code_cache, int64_t code_batch_stride, void* d_k_cache, void* d_v_cache,
                                 int64_t kv_batch_stride, int64_t pos, void* stream) {
    const sl_kv_layout kv = {kv_batch_stride, (int64_t)KH * 128, 128, 1};
    return sl::decode_prepare_impl(d_q, d_k, d_v, dtype, B, QH, KH, d_cos, d_sin, hash_q, hash_k, d_q_rot, d_q_codes,
                                   d_code_cache, code_batch_stride, d_k_cache, d_v_cache, &kv, pos, nullptr, stream);
}

extern "C" int sl_decode_prepare_ex(const void* d_q, const void* d_k, const void* d_v, int dtype, int B, int QH, int KH,
                                    const void* d_cos, const void* d_sin, const sl_hash_params* hash_q,
                                    const sl_hash_params* hash_k, void* d_q_rot, uint32_t* d_q_codes,
                                    uint32_t* d_code_cache, int64_t code_batch_stride, void* d_k_cache, void* d_v_cache,
                                    const sl_kv_layout* kv, int64_t pos, void* stream) {
    SL_REQUIRE(kv != nullptr, SL_EINVAL, "sl_decode_prepare_ex: null cache layout");
    return sl::decode_prepare_impl(d_q, d_k, d_v, dtype, B, QH, KH, d_cos, d_sin, hash_q, hash_k, d_q_rot, d_q_codes,
                                   d_code_cache, code_batch_stride, d_k_cache, d_v_cache, kv, pos, nullptr, stream);
}

// dp == nullptr: the token sits at `pos`, d_cos / d_sin are its [128] rows. Otherwise the position is the
// device word *dp->d_pos, `pos` is the largest position the caches hold (bounds the prefetch) and the
// cos / sin rows are looked up in dp's tables.
int sl::decode_prepare_impl(const void* d_q, const void* d_k, const void* d_v, int dtype, int B, int QH, int KH,
                            const void* d_cos, const void* d_sin, const sl_hash_params* hash_q,
                            const sl_hash_params* hash_k, void* d_q_rot, uint32_t* d_q_codes, uint32_t* d_code_cache,
                            int64_t code_batch_stride, void* d_k_cache, void* d_v_cache, const sl_kv_layout* kv,
                            int64_t pos, const sl::DevPos* dp, void* stream) {
    SL_REQUIRE(d_q && d_q_codes, SL_EINVAL, "sl_decode_prepare: null query pointer");
    SL_REQUIRE(B > 0 && QH > 0 && KH >= 0 && pos >= 0, SL_ESHAPE, "sl_decode_prepare: bad shape");
    if (dp) { d_cos = dp->cos_tab; d_sin = dp->sin_tab; }
    SL_REQUIRE((d_cos == nullptr) == (d_sin == nullptr), SL_EINVAL, "sl_decode_prepare: cos and sin must come together");
    if (int rc = check_params("sl_decode_prepare", hash_q, dtype)) return rc;
    const bool with_k = d_k != nullptr && KH > 0;
    if (with_k) {
        if (int rc = check_params("sl_decode_prepare", hash_k, dtype)) return rc;
        SL_REQUIRE(d_code_cache != nullptr, SL_EINVAL, "sl_decode_prepare: key given without a code cache");
        SL_REQUIRE((d_v == nullptr) == (d_v_cache == nullptr), SL_EINVAL, "sl_decode_prepare: value and value cache must come together");
        SL_REQUIRE(kv->token_stride >= 128 && kv->head_stride >= 128, SL_ESHAPE, "sl_decode_prepare: cache strides must leave room for a 128-value row");
    }
    const long long pos_host = dp ? 0 : pos;               // rows are offset on the host, or by *d_pos in the kernel
    HashArgs args = {};
    HashJob& q = args.job[0];
    q.x = d_q; q.xs_b = (long long)QH * 128; q.xs_tok = (long long)QH * 128; q.xs_h = 128; q.T = 1; q.H = QH; q.B = B;
    q.hp = *hash_q;
    q.codes = d_q_codes; q.cs_b = (long long)QH * 4;
    q.x_rot = d_q_rot; q.xr_b = (long long)QH * 128; q.xr_h = 128; q.v_h = 128;
    q.cosr = d_cos; q.sinr = d_sin;
    if (dp) { q.d_pos = dp->d_pos; q.tab_pos0 = dp->tab_pos0; }
    args.heads0 = QH;
    int total = QH;
    if (with_k) {
        HashJob& k = args.job[1];
        const size_t esz = dtype == SL_F32 ? 4 : 2;
        k.x = d_k; k.xs_b = (long long)KH * 128; k.xs_tok = (long long)KH * 128; k.xs_h = 128; k.T = 1; k.H = KH; k.B = B;
        k.hp = *hash_k;
        k.codes = d_code_cache + pos_host * KH * 4; k.cs_b = code_batch_stride;
        k.xr_h = k.v_h = kv->head_stride;
        if (d_k_cache) {
            k.x_rot = static_cast<unsigned char*>(d_k_cache) + (size_t)pos_host * kv->token_stride * esz;
            k.xr_b = kv->batch_stride;
        }
        if (d_v_cache) {
            k.v_src = d_v;
            k.v_dst = static_cast<unsigned char*>(d_v_cache) + (size_t)pos_host * kv->token_stride * esz;
            k.v_b = kv->batch_stride;
        }
        k.cosr = d_cos; k.sinr = d_sin;
        if (dp) {
            k.d_pos = dp->d_pos; k.tab_pos0 = dp->tab_pos0;
            k.xr_tok = k.v_tok = kv->token_stride; k.code_tok = (long long)KH * 4;
        }
        total += KH;
    }
    if (d_code_cache != nullptr && KH > 0 && pos > 0 && sl::l2_prefetch_enabled() && sl::aligned16(d_code_cache) &&
        code_batch_stride % 4 == 0) {
        args.pf_base = reinterpret_cast<const unsigned char*>(d_code_cache);
        args.pf_bstride = code_batch_stride * 4;
        // a larger code cache would take longer to fetch than this kernel lasts and only delay it
        // (measured: 67 MB made the step 1.7 us slower, 16.8 MB made it 0.6 us faster)
        if ((long long)pos * KH * 16 * B <= PF_MAX_BYTES) {
            args.pf_bytes = (long long)pos * KH * 16;
            args.pf_B = B;
            if (dp) { args.pf_pos = dp->d_pos; args.pf_row_bytes = (long long)KH * 16; }
        } else {
            args.pf_base = nullptr;
        }
    }
    return launch(args, dtype, total, B, static_cast<cudaStream_t>(stream));
}

extern "C" int sl_hash_encode(const void* d_x, int64_t x_batch_stride, int dtype, int B, int64_t T, int H,
                              const sl_hash_params* hash, uint32_t* d_codes, int64_t code_batch_stride, void* stream) {
    return sl_hash_encode_ex(d_x, x_batch_stride, (int64_t)H * 128, 128, dtype, B, T, H, hash, d_codes, code_batch_stride,
                             stream);
}

extern "C" int sl_hash_encode_ex(const void* d_x, int64_t x_batch_stride, int64_t x_token_stride, int64_t x_head_stride,
                                 int dtype, int B, int64_t T, int H, const sl_hash_params* hash, uint32_t* d_codes,
                                 int64_t code_batch_stride, void* stream) {
    SL_REQUIRE(d_x && d_codes, SL_EINVAL, "sl_hash_encode: null pointer");
    SL_REQUIRE(B > 0 && T >= 0 && H > 0, SL_ESHAPE, "sl_hash_encode: bad shape");
    SL_REQUIRE(x_head_stride >= 128 && x_token_stride >= 128 && code_batch_stride >= T * H * 4, SL_ESHAPE,
               "sl_hash_encode: strides shorter than a row");
    if (int rc = check_params("sl_hash_encode", hash, dtype)) return rc;
    if (T == 0) return SL_OK;
    if (dtype == SL_BF16 && (long long)B * T >= 64 && sl::aligned16(d_x) && x_batch_stride % 8 == 0 &&
        x_token_stride % 8 == 0 && x_head_stride % 8 == 0) {
        // many rows: the tensor-core kernels (weights resident in shared memory); 1 = shape not covered
        const int rt = sl::launch_hash_encode_tc(d_x, x_batch_stride, x_token_stride, x_head_stride, B, T, H, hash, d_codes,
                                                 code_batch_stride, static_cast<cudaStream_t>(stream));
        if (rt <= 0) return rt;
        const int rc = sl::launch_hash_encode_mma(d_x, x_batch_stride, x_token_stride, x_head_stride, B, T, H, hash, d_codes,
                                                  code_batch_stride, static_cast<cudaStream_t>(stream));
        if (rc <= 0) return rc;
    }
    HashArgs args = {};
    HashJob& j = args.job[0];
    j.x = d_x; j.xs_b = x_batch_stride; j.xs_tok = x_token_stride; j.xs_h = x_head_stride; j.T = T; j.H = H; j.B = B;
    j.hp = *hash;
    j.codes = d_codes; j.cs_b = code_batch_stride; j.xr_h = j.v_h = 128;
    args.heads0 = H;
    return launch(args, dtype, H, (long long)B * T, static_cast<cudaStream_t>(stream));
}
