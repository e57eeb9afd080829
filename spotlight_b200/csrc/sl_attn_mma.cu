// Sparse GQA decode attention, bf16, on the warp-level tensor-core path (mma.sync m16n8k16).
//
// The kernel is bound by the random 256-byte row gathers, so it is organised around keeping many
// of them in flight: every warp owns 16-row tiles of the index list and runs its own cp.async
// ring (ST stages of 16 K rows + 16 V rows = 8 KB each) in shared memory -- no block-wide
// barrier in the main loop, a half-warp copies one whole 256-byte row with 16-byte cp.async.
// Rows are stored with their 16-byte chunks XOR-swizzled by the row number so that ldmatrix
// reads 8 rows x 16 bytes without bank conflicts.
//
//   S = Q K^T   M = query heads of the group (padded to 16), N = 8 keys, K = head dim;
//               B fragments by ldmatrix.x4 (two k-steps per instruction).
//   O += P V    A = P straight from the accumulator layout of S; B fragments by
//               ldmatrix.x4.trans (two 8-wide column tiles of V per instruction).
//
// Online softmax in fp32 (exp2 domain). Warps of a CTA merge through shared memory; the CTAs of
// a (batch row, kv head) leave partials that a small merge kernel combines (sl_attn.cu): its launch
// overlaps this kernel's tail (programmatic dependent launch). Letting the last CTA of a
// (row, head) combine the partials instead (a ticket per pair) measured 1.2 us SLOWER at the
// headline shape: the combining CTA's fence, ticket and two trips to L2 are a serial tail.
//
// Cache geometry is explicit (batch / token / head strides): K and V may be two caches
// [B, N, KH, 128] or one cache [B, N, KH, 2, 128] in which a key's K and V rows are adjacent, so
// that one gathered key is ONE 512-byte piece of DRAM instead of two 256-byte ones (measured on
// B200: no difference in time, 17.25 against 17.31 us at the headline shape).
#include <cooperative_groups.h>

#include "sl_attn.cuh"
#include "sl_mma.cuh"

namespace cg = cooperative_groups;

namespace {

using sl::AttnArgs;

constexpr int ST = 3;              // cp.async stages per warp
constexpr int STAGE_BYTES = 8192;  // 16 K rows + 16 V rows of 256 B
constexpr float LOG2E = 1.4426950408889634f;
constexpr float LN2 = 0.6931471805599453f;
constexpr float QK_SCALE = 0.08838834764831845f * LOG2E;   // 1/sqrt(128) in the exp2 domain

// byte offset of 16-byte chunk c (0..15) of row r (0..15) inside a swizzled 16 x 256 B tile
__device__ __forceinline__ unsigned swz(int r, int c) { return (unsigned)(r * 256 + (((c & 8) | ((c ^ r) & 7)) << 4)); }

// HI: the group has more than 8 query heads (rows 8..15 of the tile are used).
// MW warps per CTA: 8 (one CTA per SM) when there are at most as many (batch row, kv head) pairs as
// SMs -- fewer, fatter CTAs mean fewer partials to combine -- else 4 (two CTAs per SM).
// CL: the CTAs of a (batch row, kv head) are one thread-block cluster and combine their partials through
// distributed shared memory (no partials in global memory, no merge kernel).
// FILL: the caches are the resident buffers of an LRU table and the list holds slots; rows of entries -(slot + 1) come
// from the backing store and are written into their slot from shared memory once they have landed.
template <bool HI, int MW, bool CL, bool FILL>
__global__ void __launch_bounds__(MW * 32, 8 / MW) sparse_attn_mma_kernel(const AttnArgs a, const int G) {
    constexpr int MT = MW * 32;
    extern __shared__ __align__(128) unsigned char ring[];          // [MW][ST][K 4 KB | V 4 KB]; reused by the epilogue
    __shared__ float sm_m[MW][16], sm_l[MW][16];

    sl::pdl_trigger();
    sl::pdl_wait();                 // index list, counts, q and the new K/V row come from earlier kernels
    const int sp = blockIdx.x, h = blockIdx.y, b = blockIdx.z, KH = a.KH;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int grp = lane >> 2, tig = lane & 3;
    const int* list = a.idx + ((long long)b * KH + h) * a.cap;
    // The list length decides which tiles are this CTA's, and the list entries decide which rows to fetch: two dependent
    // trips to memory before the first gather. The lists of a decode step are (nearly) as long as their capacity, so the
    // first ST-1 tiles are read as if the length were the capacity, together with the length; they are used when the
    // split turns out the same (entries past the end are re-read clamped), else read again.
    int spec[ST - 1];
    const int cap_tiles = (a.cap + 15) >> 4;
    const int per_spec = (cap_tiles + a.splits - 1) / a.splits;
    {
        const int t_spec = min(cap_tiles, sp * per_spec) + warp;
#pragma unroll
        for (int s = 0; s < ST - 1; ++s) spec[s] = __ldg(list + min((t_spec + s * MW) * 16 + (lane & 15), a.cap - 1));
    }
    const int n = a.cnt[b * KH + h];
    const int ntiles = (n + 15) >> 4;
    const int per = (ntiles + a.splits - 1) / a.splits;
    const int tile_lo = min(ntiles, sp * per), tile_hi = min(ntiles, tile_lo + per);
    const bool spec_ok = per == per_spec;               // then tile_lo is the speculated one as well
    const long long row_stride = a.tok_stride;
    const long long hoff = (long long)b * a.kv_b + (long long)(h / a.kv_div) * a.head_stride;
    const __nv_bfloat16* kb = reinterpret_cast<const __nv_bfloat16*>(a.k) + hoff + (lane & 15) * 8;
    const __nv_bfloat16* vb = reinterpret_cast<const __nv_bfloat16*>(a.v) + hoff + (lane & 15) * 8;
    const unsigned wring = (unsigned)__cvta_generic_to_shared(ring) + warp * (ST * STAGE_BYTES);
    const int* toks = FILL ? a.tok + ((long long)b * KH + h) * a.cap : nullptr;
    const long long bhoff = FILL ? (long long)b * a.back_b + (long long)(h / a.kv_div) * a.back_head : 0;
    const __nv_bfloat16* kbb = FILL ? reinterpret_cast<const __nv_bfloat16*>(a.k_back) + bhoff + (lane & 15) * 8 : nullptr;
    const __nv_bfloat16* vbb = FILL ? reinterpret_cast<const __nv_bfloat16*>(a.v_back) + bhoff + (lane & 15) * 8 : nullptr;

    // one tile = list entries [16 t, 16 t + 16); lane l < 16 fetches entry l (clamped to the last one)
    auto entry = [&](int t) -> int { return list[min(t * 16 + (lane & 15), n - 1)]; };
    // a half-warp copies one 256-byte row per step: 8 steps for K, 8 for V
    // fill mode: the key of list entry 16 t + lane (read a tile ahead, like the entry itself)
    auto key_of = [&](int t) -> int { return FILL ? toks[min(t * 16 + (lane & 15), n - 1)] : 0; };
    auto issue = [&](int tok, int key, int stage) {
        const unsigned sbase = wring + stage * STAGE_BYTES;
        const int c = lane & 15;
#pragma unroll
        for (int it = 0; it < 8; ++it) {
            const int r = 2 * it + (lane >> 4);
            const int e = __shfl_sync(0xffffffffu, tok, r);
            const int kr = FILL ? __shfl_sync(0xffffffffu, key, r) : 0;      // both half-warps take part, whatever their rows are
            if (FILL && e < 0) {
                const long long off = (long long)kr * a.back_tok;
                cp_async16(sbase + swz(r, c), kbb + off);
                cp_async16(sbase + 4096 + swz(r, c), vbb + off);
            } else {
                const long long off = (long long)e * row_stride;
                cp_async16(sbase + swz(r, c), kb + off);
                cp_async16(sbase + 4096 + swz(r, c), vb + off);
            }
        }
    };
    // fill mode: the rows of this tile that came from the backing store go into their slots of the resident buffers
    auto write_through = [&](int e_own, int stage) {
        if (!__any_sync(0xffffffffu, e_own < 0)) return;
        const unsigned char* sb = ring + (size_t)warp * (ST * STAGE_BYTES) + stage * STAGE_BYTES;
        const int c = lane & 15;
        __nv_bfloat16* kw = const_cast<__nv_bfloat16*>(kb);
        __nv_bfloat16* vw = const_cast<__nv_bfloat16*>(vb);
#pragma unroll
        for (int it = 0; it < 8; ++it) {
            const int r = 2 * it + (lane >> 4);
            const int e = __shfl_sync(0xffffffffu, e_own, r);
            if (e < 0) {
                const long long off = (long long)(-e - 1) * row_stride;
                *reinterpret_cast<uint4*>(kw + off) = *reinterpret_cast<const uint4*>(sb + swz(r, c));
                *reinterpret_cast<uint4*>(vw + off) = *reinterpret_cast<const uint4*>(sb + 4096 + swz(r, c));
            }
        }
    };

    // ---- prologue: fill ST-1 stages
    int tile = tile_lo + warp;
    int tok_next = 0, key_next = 0;
    int inflight[ST - 1] = {};           // fill mode: the entries of the tiles on their way, oldest first
#pragma unroll
    for (int s = 0; s < ST - 1; ++s) {
        const int t = tile + s * MW;
        if (t < tile_hi) {
            inflight[s] = (spec_ok && t * 16 + 15 < n) ? spec[s] : entry(t);
            issue(inflight[s], key_of(t), s);
        }
        cp_async_commit();
    }
    if (tile + (ST - 1) * MW < tile_hi) { tok_next = entry(tile + (ST - 1) * MW); key_next = key_of(tile + (ST - 1) * MW); }

    // ---- Q fragments (A operand), natural order
    unsigned qa[8][HI ? 4 : 2];
    {
        const __nv_bfloat16* qbase = reinterpret_cast<const __nv_bfloat16*>(a.q) + (long long)b * KH * G * 128;   // KH * G query heads
#pragma unroll
        for (int half = 0; half < (HI ? 2 : 1); ++half) {
            const int g = grp + 8 * half;
            const int qh = a.layout == SL_GQA_INTERLEAVED ? g * KH + h : h * G + g;
            const unsigned* qrow = reinterpret_cast<const unsigned*>(qbase + (long long)qh * 128);
#pragma unroll
            for (int s = 0; s < 8; ++s) {
                const unsigned lo = g < G ? qrow[8 * s + tig] : 0u;          // k = 16 s + 2 tig, +1
                const unsigned hi = g < G ? qrow[8 * s + 4 + tig] : 0u;      // k = 16 s + 8 + 2 tig, +1
                if (half == 0) { qa[s][0] = lo; qa[s][HI ? 2 : 1] = hi; }
                else { qa[s][1] = lo; qa[s][3] = hi; }
            }
        }
    }

    float o[16][4];
#pragma unroll
    for (int t = 0; t < 16; ++t) { o[t][0] = o[t][1] = o[t][2] = o[t][3] = 0.0f; }
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.0f, l1 = 0.0f;   // rows grp and grp + 8

    int stage = 0;
    for (; tile < tile_hi; tile += MW) {
        // ---- keep the ring full: issue the tile ST-1 ahead, then wait for the current one
        {
            const int t = tile + (ST - 1) * MW;
            int st2 = stage + (ST - 1);
            if (st2 >= ST) st2 -= ST;
            if (t < tile_hi) issue(tok_next, key_next, st2);
            cp_async_commit();
            const int issued = tok_next;
            if (t + MW < tile_hi) { tok_next = entry(t + MW); key_next = key_of(t + MW); }
            cp_async_wait<ST - 1>();
            __syncwarp();
            if (FILL) {
                if (a.fill_write) write_through(inflight[0], stage);
#pragma unroll
                for (int i = 0; i + 1 < ST - 1; ++i) inflight[i] = inflight[i + 1];
                inflight[ST - 2] = issued;
            }
        }
        const unsigned kbase = wring + stage * STAGE_BYTES, vbase = kbase + 4096;
        const int valid = n - tile * 16;                    // list entries of this tile that exist

        // ---- S = Q K^T for keys 0..7 (s[0]) and 8..15 (s[1])
        float s[2][4];
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.0f;
#pragma unroll
            for (int p = 0; p < 4; ++p) {                  // k-steps 2p, 2p+1
                unsigned kf[4];
                ldsm_x4(kf, kbase + swz(8 * j + (lane & 7), 4 * p + (lane >> 3)));
                if (HI) {
                    mma_bf16(s[j], qa[2 * p][0], qa[2 * p][1], qa[2 * p][2], qa[2 * p][3], kf[0], kf[1]);
                    mma_bf16(s[j], qa[2 * p + 1][0], qa[2 * p + 1][1], qa[2 * p + 1][2], qa[2 * p + 1][3], kf[2], kf[3]);
                } else {
                    mma_bf16(s[j], qa[2 * p][0], 0u, qa[2 * p][1], 0u, kf[0], kf[1]);
                    mma_bf16(s[j], qa[2 * p + 1][0], 0u, qa[2 * p + 1][1], 0u, kf[2], kf[3]);
                }
            }
        }
        // ---- online softmax; lane holds keys {2tig, 2tig+1} of each n-tile for rows grp (, grp+8)
#pragma unroll
        for (int j = 0; j < 2; ++j) {
            const int c0 = 8 * j + 2 * tig;
            const bool v0 = c0 < valid, v1 = c0 + 1 < valid;
            s[j][0] = v0 ? s[j][0] * QK_SCALE : -INFINITY;
            s[j][1] = v1 ? s[j][1] * QK_SCALE : -INFINITY;
            s[j][2] = v0 ? s[j][2] * QK_SCALE : -INFINITY;
            s[j][3] = v1 ? s[j][3] * QK_SCALE : -INFINITY;
        }
        float t0 = fmaxf(fmaxf(s[0][0], s[0][1]), fmaxf(s[1][0], s[1][1]));
        t0 = fmaxf(t0, __shfl_xor_sync(0xffffffffu, t0, 1));
        t0 = fmaxf(t0, __shfl_xor_sync(0xffffffffu, t0, 2));
        const float mn0 = fmaxf(m0, t0);                   // finite: key 0 of a tile always exists
        const float corr0 = exp2f(m0 - mn0);
        m0 = mn0;
        float corr1 = 1.0f;
        if (HI) {
            float t1 = fmaxf(fmaxf(s[0][2], s[0][3]), fmaxf(s[1][2], s[1][3]));
            t1 = fmaxf(t1, __shfl_xor_sync(0xffffffffu, t1, 1));
            t1 = fmaxf(t1, __shfl_xor_sync(0xffffffffu, t1, 2));
            const float mn1 = fmaxf(m1, t1);
            corr1 = exp2f(m1 - mn1);
            m1 = mn1;
        }
        if (__any_sync(0xffffffffu, corr0 != 1.0f || corr1 != 1.0f)) {
            l0 *= corr0; l1 *= corr1;
#pragma unroll
            for (int t = 0; t < 16; ++t) {
                o[t][0] *= corr0; o[t][1] *= corr0;
                if (HI) { o[t][2] *= corr1; o[t][3] *= corr1; }
            }
        }
        unsigned pa[4];
        {
            const float p00 = exp2f(s[0][0] - m0), p01 = exp2f(s[0][1] - m0);
            const float p10 = exp2f(s[1][0] - m0), p11 = exp2f(s[1][1] - m0);
            l0 += (p00 + p01) + (p10 + p11);
            pa[0] = pack_bf16(p00, p01);                    // row grp, keys 2tig, 2tig+1
            pa[2] = pack_bf16(p10, p11);                    // row grp, keys 2tig+8, 2tig+9
            pa[1] = pa[3] = 0u;
            if (HI) {
                const float q00 = exp2f(s[0][2] - m1), q01 = exp2f(s[0][3] - m1);
                const float q10 = exp2f(s[1][2] - m1), q11 = exp2f(s[1][3] - m1);
                l1 += (q00 + q01) + (q10 + q11);
                pa[1] = pack_bf16(q00, q01);
                pa[3] = pack_bf16(q10, q11);
            }
        }
        // ---- O += P V, two 8-wide column tiles per ldmatrix.trans
#pragma unroll
        for (int t = 0; t < 16; t += 2) {
            unsigned vfr[4];
            ldsm_x4_trans(vfr, vbase + swz(((lane >> 3) & 1) * 8 + (lane & 7), t + (lane >> 4)));
            mma_bf16(o[t], pa[0], pa[1], pa[2], pa[3], vfr[0], vfr[1]);
            mma_bf16(o[t + 1], pa[0], pa[1], pa[2], pa[3], vfr[2], vfr[3]);
        }
        __syncwarp();                                      // the stage may be overwritten next round
        if (++stage == ST) stage = 0;
    }
    cp_async_wait<0>();
    __syncthreads();                                       // ring is reused for the merge below
    float (*sm_acc)[HI ? 16 : 8][128] = reinterpret_cast<float (*)[HI ? 16 : 8][128]>(ring);

    // ---- row sums across the four lanes of a group, then the warps of the CTA
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1);
    l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    if (HI) {
        l1 += __shfl_xor_sync(0xffffffffu, l1, 1);
        l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    }
#pragma unroll
    for (int t = 0; t < 16; ++t) {
        const int d0 = 8 * t + 2 * tig;
        sm_acc[warp][grp][d0] = o[t][0];
        sm_acc[warp][grp][d0 + 1] = o[t][1];
        if (HI) {
            sm_acc[warp][grp + 8][d0] = o[t][2];
            sm_acc[warp][grp + 8][d0 + 1] = o[t][3];
        }
    }
    if (tig == 0) {
        sm_m[warp][grp] = m0; sm_l[warp][grp] = l0;
        sm_m[warp][grp + 8] = HI ? m1 : -INFINITY; sm_l[warp][grp + 8] = HI ? l1 : 0.0f;
    }
    __syncthreads();

    const long long bh = (long long)b * KH + h;
    float* part = a.part + (bh * a.splits + sp) * G * 130;
    float* cpart = reinterpret_cast<float*>(ring + 65536);          // this CTA's partial [G][130], behind sm_acc (cluster mode)
    for (int e = tid; e < G * 128; e += MT) {
        const int g = e >> 7, col = e & 127;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < MW; ++w) M = fmaxf(M, sm_m[w][g]);
        float L = 0.0f, O = 0.0f;
        if (M != -INFINITY) {
#pragma unroll
            for (int w = 0; w < MW; ++w) {
                const float c = exp2f(sm_m[w][g] - M);
                L += sm_l[w][g] * c;
                O += sm_acc[w][g][col] * c;
            }
        }
        if (a.splits == 1) {
            const int qh = a.layout == SL_GQA_INTERLEAVED ? g * KH + h : h * G + g;
            const long long oo = ((long long)b * KH * G + qh) * 128 + col;
            reinterpret_cast<__nv_bfloat16*>(a.out)[oo] = __float2bfloat16_rn(L > 0.0f ? O / L : 0.0f);
            if (a.lse && col == 0) a.lse[(long long)b * KH * G + qh] = L > 0.0f ? (M + log2f(L)) * LN2 : -INFINITY;
        } else {
            float* dst = CL ? cpart : part;
            dst[g * 130 + col] = O;
            if (col == 0) { dst[g * 130 + 128] = M; dst[g * 130 + 129] = L; }
        }
    }
    if (CL) {
        // ---- every CTA of the cluster combines a slice of the (query head, column) pairs from all partials
        cg::cluster_group cluster = cg::this_cluster();
        cluster.sync();
        const int CS = a.splits;                                   // cluster size = splits <= 16, rank = sp
        const int total = G * 128, per = (total + CS - 1) / CS;
        const int lo = sp * per, hi = min(total, lo + per);
        for (int e = lo + tid; e < hi; e += MT) {
            const int g = e >> 7, col = e & 127;
            float ms[16], ls[16], os[16];
            float M = -INFINITY;
#pragma unroll
            for (int c = 0; c < 16; ++c) {
                ms[c] = -INFINITY; ls[c] = 0.0f; os[c] = 0.0f;
                if (c < CS) {
                    const float* r = cluster.map_shared_rank(cpart, c) + g * 130;
                    ms[c] = r[128]; ls[c] = r[129]; os[c] = r[col];
                }
                M = fmaxf(M, ms[c]);
            }
            float L = 0.0f, O = 0.0f;
            if (M != -INFINITY) {
#pragma unroll
                for (int c = 0; c < 16; ++c) {
                    const float w = exp2f(ms[c] - M);              // 0 for the ranks that do not exist
                    L += ls[c] * w;
                    O += os[c] * w;
                }
            }
            const int qh = a.layout == SL_GQA_INTERLEAVED ? g * KH + h : h * G + g;
            const long long oo = ((long long)b * KH * G + qh) * 128 + col;
            reinterpret_cast<__nv_bfloat16*>(a.out)[oo] = __float2bfloat16_rn(L > 0.0f ? O / L : 0.0f);
            if (a.lse && col == 0) a.lse[(long long)b * KH * G + qh] = L > 0.0f ? (M + log2f(L)) * LN2 : -INFINITY;
        }
        cluster.sync();                                            // nobody leaves while its partial is still being read
    }
}

}  // namespace

namespace sl {

static int g_attn_warps = 0;        // 0: by shape; 4 / 8: forced (sl_configure, for measurements)
static int g_attn_cluster = 1;      // 1: combine the splits inside a thread-block cluster where one fits; 0: always the merge kernel
void set_attn_warps(int v) { g_attn_warps = v; }
void set_attn_cluster(int v) { g_attn_cluster = v; }
static bool fat_ctas(int B, int KH) { return g_attn_warps ? g_attn_warps == 8 : B * KH <= sm_count(); }

template <bool HI, int MW, bool FILL>
static cudaError_t cluster_config(cudaLaunchConfig_t& cfg, cudaLaunchAttribute* attrs, int cs, int KH, int B, cudaStream_t s) {
    const size_t ring_bytes = (size_t)MW * ST * STAGE_BYTES;
    const void* fn = reinterpret_cast<const void*>(sparse_attn_mma_kernel<HI, MW, true, FILL>);
    cudaError_t e = ensure_dyn_smem(fn, ring_bytes);
    if (e != cudaSuccess) return e;
    static bool allowed = false;                       // per instantiation: clusters of more than 8 CTAs are an opt-in
    if (!allowed) {
        e = cudaFuncSetAttribute(fn, cudaFuncAttributeNonPortableClusterSizeAllowed, 1);
        if (e != cudaSuccess) return e;
        allowed = true;
    }
    cfg = {};
    cfg.gridDim = dim3((unsigned)cs, (unsigned)KH, (unsigned)B); cfg.blockDim = dim3(MW * 32); cfg.dynamicSmemBytes = ring_bytes; cfg.stream = s;
    unsigned n = 0;
    attrs[n].id = cudaLaunchAttributeClusterDimension;
    attrs[n].val.clusterDim.x = (unsigned)cs; attrs[n].val.clusterDim.y = 1; attrs[n].val.clusterDim.z = 1;
    ++n;
    if (pdl_enabled()) {
        attrs[n].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attrs[n].val.programmaticStreamSerializationAllowed = 1;
        ++n;
    }
    cfg.attrs = attrs; cfg.numAttrs = n;
    return cudaSuccess;
}

// How many clusters of cs CTAs of MW warps the device holds at once (0: none, or the query failed); cached.
template <int MW>
static int max_clusters(int cs) {
    static int cache[17] = {};                         // 0 = not asked yet, -1 = none
    if (cs < 2 || cs > 16) return 0;
    if (cache[cs] == 0) {
        cudaLaunchConfig_t cfg;
        cudaLaunchAttribute attrs[2];
        int n = 0;
        if (cluster_config<false, MW, false>(cfg, attrs, cs, 1, 1, nullptr) != cudaSuccess ||
            cudaOccupancyMaxActiveClusters(&n, reinterpret_cast<const void*>(sparse_attn_mma_kernel<false, MW, true, false>), &cfg) != cudaSuccess) {
            cudaGetLastError();
            n = 0;
        }
        cache[cs] = n > 0 ? n : -1;
    }
    return cache[cs] > 0 ? cache[cs] : 0;
}

// The splits of a (row, head) pair form one cluster when all the clusters of the launch fit on the device at once.
static bool use_cluster(int B, int KH, int splits) {
    if (!g_attn_cluster || splits < 2 || splits > 16) return false;
    const int have = fat_ctas(B, KH) ? max_clusters<8>(splits) : max_clusters<4>(splits);
    return have >= B * KH;
}

int attn_mma_splits(int B, int KH, int cap, int reserve_sms) {
    // never more CTAs than fit at once (one of eight warps per SM, or two of four); every warp
    // should get at least one 16-row tile
    const int ctas = B * KH;
    const int tiles = (cap + 15) / 16;
    const int mw = fat_ctas(B, KH) ? 8 : 4;
    int s = ((8 / mw) * std::max(1, sm_count() - reserve_sms)) / ctas;    // reserve_sms: left to a kernel that runs beside this one
    s = std::min(s, std::min(ATTN_MAX_SPLITS, std::max(1, tiles / mw)));
    s = std::max(s, 1);
    // a few more keys per CTA are cheaper than partials in global memory and a merge kernel
    if (s > 16 && s <= 24 && use_cluster(B, KH, 16)) s = 16;
    else if (s > 8 && tiles <= 12 * s) {
        // short lists (at most a tile or two per warp) are bound by latency, not by bandwidth: fewer, fatter CTAs in the
        // largest cluster whose copies all fit at once save the merge kernel (measured at 98 % pruning of 128K keys:
        // 10.2 -> 8.0 us; at 90 % the same move costs bandwidth: 34.0 -> 35.1 us for the step)
        for (int cs = std::min(s, 16); cs >= 8; --cs)
            if (use_cluster(B, KH, cs)) { s = cs; break; }
    }
    return s;
}

template <bool HI, int MW, bool FILL>
static int launch_one(const AttnArgs& a, int G, cudaStream_t s) {
    const size_t ring_bytes = (size_t)MW * ST * STAGE_BYTES;
    if (use_cluster(a.B, a.KH, a.splits)) {
        cudaLaunchConfig_t cfg;
        cudaLaunchAttribute attrs[2];
        SL_CUDA_OK((cluster_config<HI, MW, FILL>(cfg, attrs, a.splits, a.KH, a.B, s)));
        SL_CUDA_OK(cudaLaunchKernelEx(&cfg, sparse_attn_mma_kernel<HI, MW, true, FILL>, a, G));
        return SL_OK;
    }
    dim3 grid((unsigned)a.splits, (unsigned)a.KH, (unsigned)a.B);
    SL_CUDA_OK(ensure_dyn_smem(reinterpret_cast<const void*>(sparse_attn_mma_kernel<HI, MW, false, FILL>), ring_bytes));
    SL_CUDA_OK(launch_kernel(sparse_attn_mma_kernel<HI, MW, false, FILL>, grid, dim3(MW * 32), ring_bytes, s, false, a, G));
    if (a.splits > 1) return launch_attn_merge(a, G, SL_BF16, s);
    return SL_OK;
}

template <bool FILL>
static int launch_by_shape(const AttnArgs& a, int G, cudaStream_t s) {
    if (fat_ctas(a.B, a.KH)) return G > 8 ? launch_one<true, 8, FILL>(a, G, s) : launch_one<false, 8, FILL>(a, G, s);
    return G > 8 ? launch_one<true, 4, FILL>(a, G, s) : launch_one<false, 4, FILL>(a, G, s);
}

int attn_cluster_capacity(int warps, int cs) { return warps == 8 ? max_clusters<8>(cs) : max_clusters<4>(cs); }

int launch_attn_mma(const AttnArgs& a, int G, cudaStream_t s) {
    return a.tok ? launch_by_shape<true>(a, G, s) : launch_by_shape<false>(a, G, s);
}

}  // namespace sl
