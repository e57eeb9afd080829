// Fused Hamming scan + exact histogram top-k + sink/recent window (one cooperative launch),
// and its two halves for sequence-sharded contexts.
//
// Work split: the B*N keys are cut into contiguous chunks, `ctas_per_b` per batch row; one CTA
// of 1024 threads owns one chunk. The CTA streams its chunk of 128-bit codes once with
// 16-byte loads (4 in flight per thread), keeps the 16-bit scores ON CHIP in shared memory,
// and histograms them per kv head. Selection never sorts: the score domain is [0, 128*G], so
//   pass A  per-head histogram (shared-memory atomics, then one global add per non-empty bin)
//   -- grid barrier (bounded spin) --
//   pass B  every CTA derives the threshold tau and the number r of threshold ties to take,
//           counts its own {>tau, ==tau} keys per head and publishes the counts
//   -- grid barrier --
//   pass C  every CTA prefix-sums the counts of the chunks before it and writes its selected
//           keys at their final position: output is ascending, ties go to the lowest index.
// Algorithmic DRAM traffic is the code stream (16 B per key and kv head) plus the index list.
#include "sl_common.cuh"

namespace {

constexpr int NT = 1024;
constexpr int NW = NT / 32;
constexpr int U = 4;
constexpr int SMEM_BUDGET = 200 * 1024;
constexpr int MIN_CHUNK = 256;

enum { MODE_FUSED = 0, MODE_HIST_ONLY = 1, MODE_EMIT_ONLY = 2, MODE_FROM_SCORES = 3 };

struct ScanArgs {
    const uint4* q;            // [B,QH] codes
    const uint4* k;            // code stream
    long long k_bstride;       // batch stride in codes
    int B, KH, G, layout, N;   // N = keys of this batch row (local shard)
    int k_budget;
    int s_end, r_start;        // forced ranges in local key indices: [0,s_end) and [r_start,N)
    int* idx;
    int cap;
    int* cnt;
    short* scores_out;         // optional [B,N,KH]
    unsigned short* gscores;   // scores in global memory (spill, or the sharded halves), else null
    unsigned* hist;            // global histogram [R,B,KH,nbins]; this rank adds to / reads slice `rank`
    unsigned* seg;             // [B,ctas_per_b,KH,3]
    unsigned* sync;            // [B,2]
    int* status;
    int ctas_per_b, chunk, nbins, S, mode, R, rank;
};

struct Plan {
    int ctas_per_b, chunk, nbins, S;
    size_t smem;
    bool spill, cooperative;
};

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

inline size_t fixed_smem(int KH, int G, int nbins, int S) {
    return align_up((size_t)KH * G * 16, 16) + (size_t)KH * nbins * 4 + (size_t)KH * 2 * 4 +
           (size_t)KH * S * 3 * 4 + (size_t)KH * 4 * 4 + 64;
}

Plan make_plan(int B, long long N, int KH, int G, bool scores_in_global, int nbins = 0) {
    Plan p;
    const int max_ctas = sl::sm_count();
    p.nbins = nbins > 0 ? nbins : 128 * G + 1;
    p.S = std::max(1, NW / KH);
    if (B >= max_ctas) {
        p.ctas_per_b = 1;
    } else {
        long long want = (N + MIN_CHUNK - 1) / MIN_CHUNK;
        p.ctas_per_b = (int)std::max<long long>(1, std::min<long long>(max_ctas / B, want));
    }
    long long chunk = (N + p.ctas_per_b - 1) / p.ctas_per_b;
    p.chunk = (int)((chunk + 31) / 32 * 32);
    if (p.chunk < 32) p.chunk = 32;
    const size_t fixed = fixed_smem(KH, G, p.nbins, p.S);
    const size_t sc = (size_t)p.chunk * KH * 2;
    p.spill = scores_in_global || fixed + sc > (size_t)SMEM_BUDGET;
    p.smem = fixed + (p.spill ? 0 : sc);
    p.cooperative = p.ctas_per_b > 1;
    return p;
}

__device__ __forceinline__ int warp_sum(int v) {
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
    return v;
}

template <int GT>  // GT > 0: group size known at compile time (q codes in registers); 0: generic
__global__ void __launch_bounds__(NT, 1) scan_topk_kernel(const ScanArgs a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int KH = a.KH, G = GT > 0 ? GT : a.G, nbins = a.nbins, S = a.S, N = a.N;
    uint4* sq = reinterpret_cast<uint4*>(smem_raw);                                  // [KH][G]
    unsigned* shist = reinterpret_cast<unsigned*>(smem_raw + ((size_t)KH * G * 16));  // [KH][nbins]
    int* s_tau = reinterpret_cast<int*>(shist + (size_t)KH * nbins);                  // [KH]
    int* s_r = s_tau + KH;                                                            // [KH]
    unsigned* s_task = reinterpret_cast<unsigned*>(s_r + KH);                         // [KH][S][3]
    int* s_base = reinterpret_cast<int*>(s_task + (size_t)KH * S * 3);                // [KH][4]
    unsigned short* sscores = reinterpret_cast<unsigned short*>(
        smem_raw + (((size_t)((unsigned char*)(s_base + KH * 4) - smem_raw) + 15) & ~(size_t)15));

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int b = blockIdx.x / a.ctas_per_b, c = blockIdx.x % a.ctas_per_b;
    const int t0 = min(N, c * a.chunk), t1 = min(N, t0 + a.chunk);
    const int ncodes = (t1 - t0) * KH;
    unsigned short* sc = a.gscores ? a.gscores + ((long long)b * N + t0) * KH : sscores;
    unsigned* ghist = a.hist + ((long long)a.rank * a.B + b) * KH * nbins;           // this rank's slice
    unsigned* sync = a.sync ? a.sync + 2 * b : nullptr;
    const bool multi = a.ctas_per_b > 1;
    unsigned barriers = 0;

    // ---------------------------------------------------------------- pass A: scan + histogram
    if (a.mode == MODE_FROM_SCORES) {
        // scores are given (global memory): histogram them, then select as in the fused mode
        for (int i = tid; i < KH * nbins; i += NT) shist[i] = 0;
        __syncthreads();
        for (int i = tid; i < ncodes; i += NT) {
            const int s = min(max((int)(short)sc[i], 0), nbins - 1);
            atomicAdd(&shist[(i % KH) * nbins + s], 1u);
        }
        __syncthreads();
        if (multi) {
            for (int i = tid; i < KH * nbins; i += NT) {
                const unsigned v = shist[i];
                if (v) atomicAdd(&ghist[i], v);
            }
            sl::grid_barrier(&sync[0], ++barriers * (unsigned)a.ctas_per_b, a.status);
        }
    } else if (a.mode != MODE_EMIT_ONLY) {
        for (int i = tid; i < KH * G; i += NT) {
            const int h = i / G, g = i % G;
            const int qh = a.layout == SL_GQA_INTERLEAVED ? g * KH + h : h * G + g;
            sq[i] = a.q[(long long)b * KH * G + qh];
        }
        for (int i = tid; i < KH * nbins; i += NT) shist[i] = 0;
        __syncthreads();

        const bool headfixed = (32 % KH) == 0;
        uint4 qreg[GT > 0 ? GT : 1];
        if (GT > 0 && headfixed) {
#pragma unroll
            for (int g = 0; g < GT; ++g) qreg[g] = sq[(lane % KH) * GT + g];
        }
        const uint4* base = a.k + (long long)b * a.k_bstride + (long long)t0 * KH;
        short* so = a.scores_out ? a.scores_out + ((long long)b * N + t0) * KH : nullptr;
        const int full = 128 * G;
        for (int tile = warp; tile * (32 * U) < ncodes; tile += NW) {
            const int i0 = tile * (32 * U) + lane;
            uint4 cd[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int i = i0 + u * 32;
                if (i < ncodes) cd[u] = sl::ld_stream_v4(base + i);
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int i = i0 + u * 32;
                if (i < ncodes) {
                    const int h = headfixed ? (lane % KH) : (i % KH);
                    int diff = 0;
                    if (GT > 0 && headfixed) {
#pragma unroll
                        for (int g = 0; g < GT; ++g) diff += sl::popc4(sl::xor4(qreg[g], cd[u]));
                    } else {
                        const uint4* qh = sq + h * G;
                        for (int g = 0; g < G; ++g) diff += sl::popc4(sl::xor4(qh[g], cd[u]));
                    }
                    const int s = full - diff;
                    sc[i] = (unsigned short)s;
                    atomicAdd(&shist[h * nbins + s], 1u);
                    if (so) so[i] = (short)s;
                }
            }
        }
        __syncthreads();
        if (multi || a.mode == MODE_HIST_ONLY) {
            for (int i = tid; i < KH * nbins; i += NT) {
                const unsigned v = shist[i];
                if (v) atomicAdd(&ghist[i], v);
            }
        }
        if (a.mode == MODE_HIST_ONLY) return;
        if (multi) sl::grid_barrier(&sync[0], ++barriers * (unsigned)a.ctas_per_b, a.status);
    }

    // ---------------------------------------------------------------- pass B1: threshold per head
    // s_base[h][3] temporarily holds E_lower: threshold ties owned by lower ranks.
    {
        const int kk = min(a.k_budget, a.mode == MODE_EMIT_ONLY ? 0x7fffffff : N);
        const bool from_global = multi || a.mode == MODE_EMIT_ONLY;
        const long long rstride = (long long)a.B * KH * nbins;
        for (int h = warp; h < KH; h += NW) {
            int tau = nbins, r = 0, e_lower = 0;
            if (kk > 0) {
                const unsigned* H0 = a.hist + ((long long)b * KH + h) * nbins;   // rank 0 slice
                unsigned cum = 0;
                bool found = false;
                for (int top = nbins - 1; top >= 0 && !found; top -= 32) {
                    const int bin = top - lane;
                    unsigned v = 0;
                    if (bin >= 0) {
                        if (from_global) {
                            for (int rr = 0; rr < a.R; ++rr) v += __ldcg(H0 + rr * rstride + bin);
                        } else {
                            v = shist[h * nbins + bin];
                        }
                    }
                    unsigned inc = v;
#pragma unroll
                    for (int d = 1; d < 32; d <<= 1) {
                        const unsigned t = __shfl_up_sync(0xffffffffu, inc, d);
                        if (lane >= d) inc += t;
                    }
                    const unsigned ball = __ballot_sync(0xffffffffu, cum + inc >= (unsigned)kk);
                    if (ball) {
                        const int l = __ffs(ball) - 1;
                        const unsigned incl = __shfl_sync(0xffffffffu, inc, l);
                        const unsigned vl = __shfl_sync(0xffffffffu, v, l);
                        tau = top - l;
                        r = kk - (int)(cum + incl - vl);
                        found = true;
                    } else {
                        cum += __shfl_sync(0xffffffffu, inc, 31);
                    }
                }
                if (!found) {  // fewer than kk keys in total: everything is selected
                    tau = -1;
                    r = 0;
                } else if (a.mode == MODE_EMIT_ONLY) {
                    for (int rr = lane; rr < a.rank; rr += 32) e_lower += (int)__ldcg(H0 + rr * rstride + tau);
                    e_lower = warp_sum(e_lower);
                }
            }
            if (lane == 0) {
                s_tau[h] = tau;
                s_r[h] = r;
                s_base[h * 4 + 3] = e_lower;
            }
        }
    }
    __syncthreads();

    // ---------------------------------------------------------------- pass B2: own counts per task
    const int len = t1 - t0;
    const int sub = ((len + S - 1) / S + 31) / 32 * 32;
    const int ntasks = KH * S;
    for (int task = warp; task < ntasks; task += NW) {
        const int h = task % KH, s = task / KH;
        const int lo = t0 + min(len, s * sub), hi = t0 + min(len, (s + 1) * sub);
        const int tau = s_tau[h];
        int gtM = 0, eqM = 0, eqS = 0;
        for (int tb = lo; tb < hi; tb += 32) {
            const int t = tb + lane;
            const bool valid = t < hi;
            const int v = valid ? (int)sc[(t - t0) * KH + h] : -2;
            const bool mid = valid && t >= a.s_end && t < a.r_start;
            gtM += __popc(__ballot_sync(0xffffffffu, mid && v > tau));
            eqM += __popc(__ballot_sync(0xffffffffu, mid && v == tau));
            eqS += __popc(__ballot_sync(0xffffffffu, valid && t < a.s_end && v == tau));
        }
        if (lane == 0) {
            s_task[(h * S + s) * 3 + 0] = gtM;
            s_task[(h * S + s) * 3 + 1] = eqM;
            s_task[(h * S + s) * 3 + 2] = eqS;
        }
    }
    __syncthreads();
    if (multi) {
        for (int i = tid; i < KH * 3; i += NT) {
            const int h = i / 3, j = i % 3;
            unsigned v = 0;
            for (int s = 0; s < S; ++s) v += s_task[(h * S + s) * 3 + j];
            a.seg[(((long long)b * a.ctas_per_b + c) * KH + h) * 3 + j] = v;
        }
        sl::grid_barrier(&sync[0], ++barriers * (unsigned)a.ctas_per_b, a.status);
    }

    // ---------------------------------------------------------------- pass B3: prefix over chunks
    for (int h = warp; h < KH; h += NW) {
        int pre_gt = 0, pre_eq = 0, tot_gt = 0, tot_eq = 0, tot_eqS = 0;
        if (multi) {
            for (int cc = lane; cc < a.ctas_per_b; cc += 32) {
                const unsigned* p = a.seg + (((long long)b * a.ctas_per_b + cc) * KH + h) * 3;
                const int g = (int)__ldcg(p), e = (int)__ldcg(p + 1), es = (int)__ldcg(p + 2);
                tot_gt += g; tot_eq += e; tot_eqS += es;
                if (cc < c) { pre_gt += g; pre_eq += e; }
            }
            pre_gt = warp_sum(pre_gt); pre_eq = warp_sum(pre_eq);
            tot_gt = warp_sum(tot_gt); tot_eq = warp_sum(tot_eq); tot_eqS = warp_sum(tot_eqS);
        } else {
            for (int s = 0; s < S; ++s) {
                tot_gt += s_task[(h * S + s) * 3 + 0];
                tot_eq += s_task[(h * S + s) * 3 + 1];
                tot_eqS += s_task[(h * S + s) * 3 + 2];
            }
        }
        const int rM = max(s_r[h] - s_base[h * 4 + 3] - tot_eqS, 0);
        const int selM = tot_gt + min(tot_eq, rM);
        __syncwarp();
        if (lane == 0) {
            s_base[h * 4 + 0] = pre_gt;
            s_base[h * 4 + 1] = pre_eq;
            s_base[h * 4 + 2] = rM;
            s_base[h * 4 + 3] = selM;
            if (c == 0) a.cnt[b * KH + h] = a.s_end + selM + (N - a.r_start);
        }
    }
    __syncthreads();

    // ---------------------------------------------------------------- pass C: ordered emission
    for (int task = warp; task < ntasks; task += NW) {
        const int h = task % KH, s = task / KH;
        const int lo = t0 + min(len, s * sub), hi = t0 + min(len, (s + 1) * sub);
        const int tau = s_tau[h], rM = s_base[h * 4 + 2], selM = s_base[h * 4 + 3];
        int gt_before = s_base[h * 4 + 0], eq_before = s_base[h * 4 + 1];
        for (int s2 = 0; s2 < s; ++s2) {
            gt_before += s_task[(h * S + s2) * 3 + 0];
            eq_before += s_task[(h * S + s2) * 3 + 1];
        }
        int* oi = a.idx + ((long long)b * KH + h) * a.cap;
        const unsigned lt = (1u << lane) - 1u;
        for (int tb = lo; tb < hi; tb += 32) {
            const int t = tb + lane;
            const bool valid = t < hi;
            const int v = valid ? (int)sc[(t - t0) * KH + h] : -2;
            const bool mid = valid && t >= a.s_end && t < a.r_start;
            const bool isgt = mid && v > tau, iseq = mid && v == tau;
            const unsigned bgt = __ballot_sync(0xffffffffu, isgt);
            const unsigned beq = __ballot_sync(0xffffffffu, iseq);
            const bool taken = iseq && (eq_before + __popc(beq & lt)) < rM;
            const unsigned btk = __ballot_sync(0xffffffffu, taken);
            int pos = -1;
            if (isgt || taken) pos = a.s_end + gt_before + min(eq_before, rM) + __popc((bgt | btk) & lt);
            else if (valid && t < a.s_end) pos = t;
            else if (valid && t >= a.r_start) pos = a.s_end + selM + (t - a.r_start);
            if (pos >= 0) {
                if (pos < a.cap) oi[pos] = t;
                else if (a.status) atomicExch(a.status, 2);
            }
            gt_before += __popc(bgt);
            eq_before += __popc(beq);
        }
    }

    // ---------------------------------------------------------------- leave the workspace zeroed
    if (multi) {
        if (a.mode == MODE_FUSED || a.mode == MODE_FROM_SCORES) {
            const int total = KH * nbins;
            const int slice = (total + a.ctas_per_b - 1) / a.ctas_per_b;
            const int z0 = c * slice, z1 = min(total, z0 + slice);
            for (int i = z0 + tid; i < z1; i += NT) ghist[i] = 0;
        }
        __syncthreads();
        if (tid == 0) {
            __threadfence();
            const unsigned old = atomicAdd(&sync[1], 1u);
            if (old == (unsigned)a.ctas_per_b - 1u) {
                sync[0] = 0;
                sync[1] = 0;
                __threadfence();
            }
        }
    }
}

typedef void (*kernel_t)(const ScanArgs);

kernel_t pick_kernel(int G) {
    switch (G) {
        case 1: return scan_topk_kernel<1>;
        case 2: return scan_topk_kernel<2>;
        case 3: return scan_topk_kernel<3>;
        case 4: return scan_topk_kernel<4>;
        case 5: return scan_topk_kernel<5>;
        case 6: return scan_topk_kernel<6>;
        case 7: return scan_topk_kernel<7>;
        case 8: return scan_topk_kernel<8>;
        default: return scan_topk_kernel<0>;
    }
}

struct WsLayout {
    size_t sync_off, hist_off, seg_off, score_off, total;
};

WsLayout ws_layout(int B, long long N, int KH, int G, bool with_hist, bool spill, int nbins = 0) {
    WsLayout w;
    const int max_cpb = std::max(1, sl::sm_count() * 2);
    size_t off = 0;
    w.sync_off = off; off = align_up(off + (size_t)B * 2 * 4, 256);
    w.hist_off = off; if (with_hist) off = align_up(off + (size_t)B * KH * (nbins > 0 ? nbins : 128 * G + 1) * 4, 256);
    w.seg_off = off; off = align_up(off + (size_t)B * max_cpb * KH * 3 * 4, 256);
    w.score_off = off; if (spill) off = align_up(off + (size_t)B * N * KH * 2, 256);
    w.total = off;
    return w;
}

int check_common(const char* fn, int B, long long N, int KH, int QH) {
    SL_REQUIRE(B > 0 && N >= 0 && KH > 0 && QH > 0 && QH % KH == 0, SL_ESHAPE, "%s: bad shape B=%d N=%lld KH=%d QH=%d",
               fn, B, N, KH, QH);
    SL_REQUIRE(N <= 0x7fffffffLL / KH, SL_ESHAPE, "%s: N*KH exceeds 2^31", fn);
    const int G = QH / KH;
    SL_REQUIRE((size_t)KH * (128 * G + 1) * 4 <= 96 * 1024, SL_ESHAPE,
               "%s: KH*(128*G+1) histogram bins exceed the 96 KB shared-memory budget", fn);
    SL_REQUIRE((long long)B * sl::sm_count() * 2 < (1LL << 30), SL_ESHAPE, "%s: batch too large", fn);
    return SL_OK;
}

int launch(const ScanArgs& a, const Plan& p, cudaStream_t s) {
    kernel_t kern = pick_kernel(a.G);
    SL_CUDA_OK(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)p.smem));
    const unsigned grid = (unsigned)(a.B * p.ctas_per_b);
    if (p.cooperative) {
        void* params[] = {(void*)&a};
        SL_CUDA_OK(cudaLaunchCooperativeKernel((const void*)kern, dim3(grid), dim3(NT), params, p.smem, s));
    } else {
        kern<<<grid, NT, p.smem, s>>>(a);
        SL_CUDA_OK(cudaGetLastError());
    }
    return SL_OK;
}

}  // namespace

extern "C" size_t sl_scan_topk_workspace_bytes(int B, int64_t N, int KH, int QH) {
    if (B <= 0 || N < 0 || KH <= 0 || QH <= 0 || QH % KH) return 0;
    const int G = QH / KH;
    const Plan p = make_plan(B, N, KH, G, false);
    return ws_layout(B, N, KH, G, true, p.spill).total;
}

extern "C" int sl_scan_topk(const uint32_t* d_q_codes, const uint32_t* d_k_codes, int64_t k_batch_stride, int B,
                            int64_t N, int KH, int QH, int gqa_layout, int k, int sink, int recent, int32_t* d_idx,
                            int idx_capacity, int32_t* d_cnt, int16_t* d_scores_out, void* d_workspace,
                            size_t workspace_bytes, int32_t* d_status, void* stream) {
    SL_REQUIRE(d_q_codes && d_k_codes && d_idx && d_cnt && d_workspace, SL_EINVAL, "sl_scan_topk: null pointer");
    if (int rc = check_common("sl_scan_topk", B, N, KH, QH)) return rc;
    SL_REQUIRE(gqa_layout == SL_GQA_INTERLEAVED || gqa_layout == SL_GQA_BLOCKED, SL_EINVAL,
               "sl_scan_topk: unknown gqa_layout %d", gqa_layout);
    SL_REQUIRE(k >= 0 && sink >= 0 && recent >= 0, SL_EINVAL, "sl_scan_topk: negative k/sink/recent");
    SL_REQUIRE(sl::aligned16(d_q_codes) && sl::aligned16(d_k_codes) && k_batch_stride % 4 == 0, SL_EALIGN,
               "sl_scan_topk: codes must be 16-byte aligned");
    SL_REQUIRE(k_batch_stride >= N * KH * 4, SL_ESHAPE, "sl_scan_topk: batch stride shorter than a batch row");
    const int64_t need = std::min<int64_t>(N, (int64_t)k + sink + recent);
    SL_REQUIRE(idx_capacity >= need, SL_ESHAPE, "sl_scan_topk: idx_capacity %d < min(N, k+sink+recent) = %lld",
               idx_capacity, (long long)need);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (N == 0) {
        SL_CUDA_OK(cudaMemsetAsync(d_cnt, 0, (size_t)B * KH * 4, s));
        return SL_OK;
    }
    const int G = QH / KH;
    const Plan p = make_plan(B, N, KH, G, false);
    const WsLayout w = ws_layout(B, N, KH, G, true, p.spill);
    SL_REQUIRE(workspace_bytes >= w.total, SL_EWORKSPACE, "sl_scan_topk: workspace %zu < required %zu", workspace_bytes,
               w.total);
    SL_REQUIRE(sl::aligned16(d_workspace), SL_EALIGN, "sl_scan_topk: workspace not 16-byte aligned");
    unsigned char* ws = static_cast<unsigned char*>(d_workspace);
    ScanArgs a;
    a.q = reinterpret_cast<const uint4*>(d_q_codes);
    a.k = reinterpret_cast<const uint4*>(d_k_codes);
    a.k_bstride = k_batch_stride / 4;
    a.B = B; a.KH = KH; a.G = G; a.layout = gqa_layout; a.N = (int)N;
    a.k_budget = k;
    a.s_end = (int)std::min<int64_t>(sink, N);
    a.r_start = (int)std::max<int64_t>(a.s_end, N - recent);
    a.idx = d_idx; a.cap = idx_capacity; a.cnt = d_cnt;
    a.scores_out = d_scores_out;
    a.gscores = p.spill ? reinterpret_cast<unsigned short*>(ws + w.score_off) : nullptr;
    a.hist = reinterpret_cast<unsigned*>(ws + w.hist_off);
    a.seg = reinterpret_cast<unsigned*>(ws + w.seg_off);
    a.sync = reinterpret_cast<unsigned*>(ws + w.sync_off);
    a.status = d_status;
    a.ctas_per_b = p.ctas_per_b; a.chunk = p.chunk; a.nbins = p.nbins; a.S = p.S;
    a.mode = MODE_FUSED; a.R = 1; a.rank = 0;
    return launch(a, p, s);
}

extern "C" int sl_scan_hist(const uint32_t* d_q_codes, const uint32_t* d_k_codes, int64_t k_batch_stride, int B,
                            int64_t N_local, int KH, int QH, int gqa_layout, int16_t* d_scores, uint32_t* d_hist,
                            void* stream) {
    SL_REQUIRE(d_q_codes && d_k_codes && d_scores && d_hist, SL_EINVAL, "sl_scan_hist: null pointer");
    if (int rc = check_common("sl_scan_hist", B, N_local, KH, QH)) return rc;
    SL_REQUIRE(gqa_layout == SL_GQA_INTERLEAVED || gqa_layout == SL_GQA_BLOCKED, SL_EINVAL,
               "sl_scan_hist: unknown gqa_layout %d", gqa_layout);
    SL_REQUIRE(sl::aligned16(d_q_codes) && sl::aligned16(d_k_codes) && k_batch_stride % 4 == 0, SL_EALIGN,
               "sl_scan_hist: codes must be 16-byte aligned");
    SL_REQUIRE(k_batch_stride >= N_local * KH * 4, SL_ESHAPE, "sl_scan_hist: batch stride shorter than a batch row");
    if (N_local == 0) return SL_OK;
    const int G = QH / KH;
    Plan p = make_plan(B, N_local, KH, G, true);
    p.cooperative = false;
    ScanArgs a = {};
    a.q = reinterpret_cast<const uint4*>(d_q_codes);
    a.k = reinterpret_cast<const uint4*>(d_k_codes);
    a.k_bstride = k_batch_stride / 4;
    a.B = B; a.KH = KH; a.G = G; a.layout = gqa_layout; a.N = (int)N_local;
    a.gscores = reinterpret_cast<unsigned short*>(d_scores);
    a.hist = d_hist;
    a.ctas_per_b = p.ctas_per_b; a.chunk = p.chunk; a.nbins = p.nbins; a.S = p.S;
    a.mode = MODE_HIST_ONLY; a.R = 1; a.rank = 0;
    return launch(a, p, static_cast<cudaStream_t>(stream));
}

extern "C" size_t sl_select_emit_workspace_bytes(int B, int64_t N_local, int KH, int QH) {
    if (B <= 0 || N_local < 0 || KH <= 0 || QH <= 0 || QH % KH) return 0;
    return ws_layout(B, N_local, KH, QH / KH, false, false).total;
}

extern "C" int sl_select_emit(const int16_t* d_scores, const uint32_t* d_hist_all, int R, int rank, int B,
                              int64_t N_local, int64_t tok_offset, int64_t N_global, int KH, int QH, int k, int sink,
                              int recent, int32_t* d_idx, int idx_capacity, int32_t* d_cnt, void* d_workspace,
                              size_t workspace_bytes, int32_t* d_status, void* stream) {
    SL_REQUIRE(d_scores && d_hist_all && d_idx && d_cnt && d_workspace, SL_EINVAL, "sl_select_emit: null pointer");
    if (int rc = check_common("sl_select_emit", B, N_local, KH, QH)) return rc;
    SL_REQUIRE(R > 0 && rank >= 0 && rank < R, SL_EINVAL, "sl_select_emit: bad rank %d of %d", rank, R);
    SL_REQUIRE(tok_offset >= 0 && tok_offset + N_local <= N_global, SL_ESHAPE, "sl_select_emit: shard outside the context");
    SL_REQUIRE(k >= 0 && sink >= 0 && recent >= 0, SL_EINVAL, "sl_select_emit: negative k/sink/recent");
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (N_local == 0) {
        SL_CUDA_OK(cudaMemsetAsync(d_cnt, 0, (size_t)B * KH * 4, s));
        return SL_OK;
    }
    const int G = QH / KH;
    const Plan p = make_plan(B, N_local, KH, G, true);
    const WsLayout w = ws_layout(B, N_local, KH, G, false, false);
    SL_REQUIRE(workspace_bytes >= w.total, SL_EWORKSPACE, "sl_select_emit: workspace %zu < required %zu", workspace_bytes,
               w.total);
    // forced ranges of the GLOBAL context, clipped to this shard and made local
    const int64_t s_end_g = std::min<int64_t>(sink, N_global);
    const int64_t r_start_g = std::max<int64_t>(s_end_g, N_global - recent);
    const int64_t s_end = std::min<int64_t>(std::max<int64_t>(s_end_g - tok_offset, 0), N_local);
    const int64_t r_start = std::min<int64_t>(std::max<int64_t>(r_start_g - tok_offset, s_end), N_local);
    const int64_t need = std::min<int64_t>(N_local, (int64_t)k + s_end + (N_local - r_start));
    SL_REQUIRE(idx_capacity >= need, SL_ESHAPE, "sl_select_emit: idx_capacity %d < %lld", idx_capacity, (long long)need);
    unsigned char* ws = static_cast<unsigned char*>(d_workspace);
    ScanArgs a = {};
    a.B = B; a.KH = KH; a.G = G; a.N = (int)N_local;
    a.k_budget = k;
    a.s_end = (int)s_end; a.r_start = (int)r_start;
    a.idx = d_idx; a.cap = idx_capacity; a.cnt = d_cnt;
    a.gscores = reinterpret_cast<unsigned short*>(const_cast<int16_t*>(d_scores));
    a.hist = const_cast<unsigned*>(d_hist_all);
    a.seg = reinterpret_cast<unsigned*>(ws + w.seg_off);
    a.sync = reinterpret_cast<unsigned*>(ws + w.sync_off);
    a.status = d_status;
    a.ctas_per_b = p.ctas_per_b; a.chunk = p.chunk; a.nbins = p.nbins; a.S = p.S;
    a.mode = MODE_EMIT_ONLY; a.R = R; a.rank = rank;
    return launch(a, p, s);
}

extern "C" size_t sl_topk_from_scores_workspace_bytes(int B, int64_t N, int KH, int max_score) {
    if (B <= 0 || N < 0 || KH <= 0 || max_score < 0) return 0;
    return ws_layout(B, N, KH, 1, true, false, max_score + 1).total;
}

extern "C" int sl_topk_from_scores(const int16_t* d_scores, int B, int64_t N, int KH, int max_score, int k, int sink,
                                   int recent, int32_t* d_idx, int idx_capacity, int32_t* d_cnt, void* d_workspace,
                                   size_t workspace_bytes, int32_t* d_status, void* stream) {
    SL_REQUIRE(d_scores && d_idx && d_cnt && d_workspace, SL_EINVAL, "sl_topk_from_scores: null pointer");
    SL_REQUIRE(B > 0 && N >= 0 && KH > 0 && max_score >= 0, SL_ESHAPE, "sl_topk_from_scores: bad shape");
    SL_REQUIRE(N <= 0x7fffffffLL / KH, SL_ESHAPE, "sl_topk_from_scores: N*KH exceeds 2^31");
    SL_REQUIRE((size_t)KH * (max_score + 1) * 4 <= 96 * 1024, SL_ESHAPE,
               "sl_topk_from_scores: KH*(max_score+1) histogram bins exceed the 96 KB shared-memory budget");
    SL_REQUIRE(k >= 0 && sink >= 0 && recent >= 0, SL_EINVAL, "sl_topk_from_scores: negative k/sink/recent");
    const int64_t need = std::min<int64_t>(N, (int64_t)k + sink + recent);
    SL_REQUIRE(idx_capacity >= need, SL_ESHAPE, "sl_topk_from_scores: idx_capacity %d < %lld", idx_capacity, (long long)need);
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    if (N == 0) {
        SL_CUDA_OK(cudaMemsetAsync(d_cnt, 0, (size_t)B * KH * 4, s));
        return SL_OK;
    }
    const Plan p = make_plan(B, N, KH, 1, true, max_score + 1);
    const WsLayout w = ws_layout(B, N, KH, 1, true, false, max_score + 1);
    SL_REQUIRE(workspace_bytes >= w.total, SL_EWORKSPACE, "sl_topk_from_scores: workspace %zu < required %zu",
               workspace_bytes, w.total);
    unsigned char* ws = static_cast<unsigned char*>(d_workspace);
    ScanArgs a = {};
    a.B = B; a.KH = KH; a.G = 1; a.N = (int)N;
    a.k_budget = k;
    a.s_end = (int)std::min<int64_t>(sink, N);
    a.r_start = (int)std::max<int64_t>(a.s_end, N - recent);
    a.idx = d_idx; a.cap = idx_capacity; a.cnt = d_cnt;
    a.gscores = reinterpret_cast<unsigned short*>(const_cast<int16_t*>(d_scores));
    a.hist = reinterpret_cast<unsigned*>(ws + w.hist_off);
    a.seg = reinterpret_cast<unsigned*>(ws + w.seg_off);
    a.sync = reinterpret_cast<unsigned*>(ws + w.sync_off);
    a.status = d_status;
    a.ctas_per_b = p.ctas_per_b; a.chunk = p.chunk; a.nbins = p.nbins; a.S = p.S;
    a.mode = MODE_FROM_SCORES; a.R = 1; a.rank = 0;
    return launch(a, p, s);
}
