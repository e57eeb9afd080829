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
#include <cstdlib>

#include "sl_common.cuh"
#include "sl_scan.cuh"
#include "sl_sliced.cuh"

namespace {

#ifndef SL_SCAN_NT
#define SL_SCAN_NT 512
#endif
#ifndef SL_SCAN_U
#define SL_SCAN_U 8
#endif
constexpr int NT = SL_SCAN_NT;     // threads per CTA
constexpr int NW = NT / 32;
constexpr int U = SL_SCAN_U;       // 16-byte loads in flight per thread
constexpr int SMEM_BUDGET = 200 * 1024;
constexpr int MIN_CHUNK = 256;
constexpr int NCOPY = 4;           // copies of the global histogram in the workspace

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
    uint4* seg;                // [B,ctas_per_b,KH] {>tau, ==tau, ==tau inside the sink, -}
    unsigned* sync;            // [B,2]
    int* status;
    int ctas_per_b, chunk, nbins, S, mode, R, rank, ncopy;
    int stage;                 // copy this chunk's share of gscores into shared memory first
    unsigned long long* dbg;   // optional [grid][16] phase timestamps (ns)
};



struct Plan {
    int ctas_per_b, chunk, nbins, S;
    size_t smem;
    bool spill, cooperative;
    bool stage;     // scores are given in global memory and the chunk's share fits in shared memory: copy it in first
};

inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

inline size_t fixed_smem(int KH, int G, int nbins, int S) {
    return align_up((size_t)KH * G * 16, 16) + (size_t)KH * nbins * 4 + (size_t)KH * 2 * 4 +
           (size_t)KH * S * 3 * 4 + (size_t)KH * 4 * 4 + (size_t)KH * 32 * 4 + (size_t)KH * 4 * 4 + 64;
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
    const size_t sc = (size_t)(p.chunk + 64) * KH * 2;      // transposed rows, padded to 4 (mod 32) words
    p.spill = scores_in_global || fixed + sc > (size_t)SMEM_BUDGET;
    p.stage = false;
    p.smem = fixed + (p.spill ? 0 : sc);
    p.cooperative = p.ctas_per_b > 1;
    return p;
}

// The modes that are fed with scores (from-scores, emit-only) walk them twice; from shared memory
// that is several times faster than from global memory, so a chunk that fits is copied in first.
Plan make_plan_given_scores(int B, long long N, int KH, int G, int nbins = 0) {
    Plan p = make_plan(B, N, KH, G, true, nbins);
    const size_t sc = (size_t)(p.chunk + 64) * KH * 2;
    if (p.smem + sc <= (size_t)SMEM_BUDGET) {
        p.stage = true;
        p.smem += sc;
    }
    return p;
}

__device__ __forceinline__ int warp_sum(int v) {
#pragma unroll
    for (int d = 16; d > 0; d >>= 1) v += __shfl_xor_sync(0xffffffffu, v, d);
    return v;
}


__device__ __forceinline__ void touch(const void* p) {   // warms the TLB for a page used later
    unsigned v;
    asm volatile("ld.global.cg.u32 %0, [%1];" : "=r"(v) : "l"(p));
}

template <int PT>  // PT > 0: bit-sliced scoring with PT planes (needs 32 % KH == 0); 0: direct popcounts
__global__ void __launch_bounds__(NT, 1) scan_topk_kernel(const ScanArgs a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int KH = a.KH, G = a.G, nbins = a.nbins, S = a.S, N = a.N;
    uint4* sq = reinterpret_cast<uint4*>(smem_raw);                                  // [KH][G]
    unsigned* shist = reinterpret_cast<unsigned*>(smem_raw + ((size_t)KH * G * 16));  // [KH][nbins]
    int* s_tau = reinterpret_cast<int*>(shist + (size_t)KH * nbins);                  // [KH]
    int* s_r = s_tau + KH;                                                            // [KH]
    unsigned* s_task = reinterpret_cast<unsigned*>(s_r + KH);                         // [KH][S][3]
    int* s_base = reinterpret_cast<int*>(s_task + (size_t)KH * S * 3);                // [KH][4]
    uint32_t* s_planes = reinterpret_cast<uint32_t*>(                                 // [KH][2][P][4], 16-byte aligned
        smem_raw + (((size_t)((unsigned char*)(s_base + KH * 4) - smem_raw) + 15) & ~(size_t)15));
    int* s_pbase = reinterpret_cast<int*>(s_planes + KH * 32);                        // [KH][4]
    unsigned short* sscores = reinterpret_cast<unsigned short*>(s_pbase + KH * 4);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int b = blockIdx.x / a.ctas_per_b, c = blockIdx.x % a.ctas_per_b;
    const int t0 = min(N, c * a.chunk), t1 = min(N, t0 + a.chunk);
    const int ncodes = (t1 - t0) * KH;
    // Scores live either in shared memory, TRANSPOSED as [head][local key] with a row stride of
    // 4 (mod 32) words so that the interleaved writes of pass A spread over the banks, or in
    // global memory as [key][head] (spill of huge chunks, and the modes fed with scores).
    const bool fast = a.gscores == nullptr || a.stage;
    const int roww = (a.chunk >> 1) + ((4 - (a.chunk >> 1)) & 31);
    const int rowh = 2 * roww;
    unsigned short* sc = fast ? sscores : a.gscores + ((long long)b * N + t0) * KH;
    const long long hslice = (long long)a.B * KH * nbins;                            // one histogram copy / rank
    unsigned* hist_b = a.hist + (long long)b * KH * nbins;                            // slice 0 of this batch row
    unsigned* sync = a.sync ? a.sync + 2 * b : nullptr;
    const bool multi = a.ctas_per_b > 1;
    unsigned barriers = 0;
    SL_STAMP(0)
    sl::pdl_trigger();
    sl::pdl_wait();                 // codes, q codes and the workspace all come from earlier kernels

    if (a.mode == MODE_EMIT_ONLY && a.stage) {
        const unsigned short* gs = a.gscores + ((long long)b * N + t0) * KH;
        for (int i = tid; i < ncodes; i += NT) sscores[(i % KH) * rowh + i / KH] = gs[i];
        __syncthreads();
    }
    // ---------------------------------------------------------------- pass A: scan + histogram
    if (a.mode == MODE_FROM_SCORES) {
        // scores are given (global memory): histogram them, then select as in the fused mode
        for (int i = tid; i < KH * nbins; i += NT) shist[i] = 0;
        __syncthreads();
        const unsigned short* gs = a.gscores + ((long long)b * N + t0) * KH;
        for (int i = tid; i < ncodes; i += NT) {
            const int s = min(max((int)(short)gs[i], 0), nbins - 1);
            atomicAdd(&shist[(i % KH) * nbins + s], 1u);
            if (a.stage) sscores[(i % KH) * rowh + i / KH] = (unsigned short)s;
        }
        __syncthreads();
    } else if (a.mode != MODE_EMIT_ONLY) {
        // the first tile's loads are in flight while the query codes are staged
        const uint4* base = a.k + (long long)b * a.k_bstride + (long long)t0 * KH;
        const uint32_t* qb = reinterpret_cast<const uint32_t*>(a.q + (long long)b * KH * G);
        PlaneWords pw = {{0u, 0u}};
        if (PT > 0) pw = planes_issue(qb, KH, G, a.layout, warp, NW, lane);   // ahead of the stream's loads
        uint4 cd[U];
        int tile = warp;
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int i = tile * (32 * U) + u * 32 + lane;
            if (i < ncodes) cd[u] = sl::ld_stream_v4(base + i);
        }
        if (tid == NT - 32 && a.idx) {   // pages the later passes store to / load from
            touch(a.idx + ((long long)b * KH) * a.cap);
            touch(a.cnt + b * KH);
            if (a.seg) touch(a.seg + (long long)b * a.ctas_per_b * KH);
        }
        constexpr int PP = PT > 0 ? PT : 1;
        uint32_t M[PP][4], Mp[PP][4];
        int sbase = 0;
        const int ssh = sliced_shift(G);
        // Planes of the group's query codes (one warp per (head, word), straight from global
        // memory) while the other threads clear the histogram; one barrier, then every lane
        // copies the planes of its own head into registers.
        if (PT > 0) {
            planes_finish<PP>(pw, KH, G, s_planes, s_pbase, warp, NW, lane);
            stage_planes<PP>(qb, KH, G, a.layout, s_planes, s_pbase, warp, NW, lane, 1);     // KH > 8
        } else {
            for (int i = tid; i < KH * G; i += NT) {
                const int h = i / G, g = i % G;
                const int qh = a.layout == SL_GQA_INTERLEAVED ? g * KH + h : h * G + g;
                sq[i] = a.q[(long long)b * KH * G + qh];
            }
        }
        for (int i = tid; i < KH * nbins; i += NT) shist[i] = 0;
        __syncthreads();
        if (PT > 0) sbase = load_planes<PP>(s_planes, s_pbase, lane % KH, M, Mp);
        SL_STAMP(11)
        short* so = a.scores_out ? a.scores_out + ((long long)b * N + t0) * KH : nullptr;
        const int full = 128 * G;
        const int khs = 31 - __clz(KH);             // log2(KH) when KH is a power of two (PT > 0)
        while (tile * (32 * U) < ncodes) {
            const int i0 = tile * (32 * U) + lane;
            int sv[U];
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int i = i0 + u * 32;
                sv[u] = 0;
                if (i < ncodes) {
                    if (PT > 0) {
                        sv[u] = sbase + (sliced_score<PP>(cd[u], M, Mp) << ssh);
                    } else {
                        const uint4* qh = sq + (i % KH) * G;
                        int diff = 0;
                        for (int g = 0; g < G; ++g) diff += sl::popc4(sl::xor4(qh[g], cd[u]));
                        sv[u] = full - diff;
                    }
                }
            }
            if (tile == 0) { SL_STAMP(13) }
            tile += NW;
#pragma unroll
            for (int u = 0; u < U; ++u) {       // next tile's loads before the stores of this one
                const int i = tile * (32 * U) + u * 32 + lane;
                if (i < ncodes) cd[u] = sl::ld_stream_v4(base + i);
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int i = i0 + u * 32;
                if (i < ncodes) {
                    const int h = PT > 0 ? (lane % KH) : (i % KH);
                    const int tl = PT > 0 ? (i >> khs) : (i / KH);
                    if (fast) sscores[h * rowh + tl] = (unsigned short)sv[u];
                    else sc[i] = (unsigned short)sv[u];
                    atomicAdd(&shist[h * nbins + sv[u]], 1u);
                    if (so) so[i] = (short)sv[u];
                }
            }
        }
        __syncthreads();
    }
    SL_STAMP(7)
    if (a.mode != MODE_EMIT_ONLY && (multi || a.mode == MODE_HIST_ONLY)) {
        // one global add per non-empty bin; CTAs spread over the histogram copies and start at
        // different bins so that simultaneous adds rarely meet on one address
        unsigned* dst = hist_b + (long long)(c % a.ncopy) * hslice;
        const int total = KH * nbins;
        const int start = (int)(((long long)c * 977) % total);
        for (int j = tid; j < total; j += NT) {
            int i = j + start;
            if (i >= total) i -= total;
            const unsigned v = shist[i];
            if (v) atomicAdd(&dst[i], v);
        }
    }
    SL_STAMP(1)
    if (a.mode == MODE_HIST_ONLY) return;
    if (multi && a.mode != MODE_EMIT_ONLY) sl::grid_barrier(&sync[0], ++barriers * (unsigned)a.ctas_per_b, a.status);
    SL_STAMP(2)

    // ---------------------------------------------------------------- pass B1: threshold per head
    // The global histogram (sum of its copies, or of all ranks' histograms) is staged into
    // shared memory by all threads with every load in flight at once. Then one warp per head:
    // each lane sums a block of bins, a suffix scan over the lanes finds the block holding the
    // threshold, and that lane walks its block from the top.
    const int nslices = a.mode == MODE_EMIT_ONLY ? a.R : a.ncopy;
    if (multi || a.mode == MODE_EMIT_ONLY) {
        const int total = KH * nbins;
        for (int i0 = tid; i0 < total; i0 += NT * 4) {
            unsigned v[4] = {0u, 0u, 0u, 0u};
            for (int sl_ = 0; sl_ < nslices; ++sl_) {
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int i = i0 + j * NT;
                    if (i < total) v[j] += __ldcg(hist_b + sl_ * hslice + i);
                }
            }
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int i = i0 + j * NT;
                if (i < total) shist[i] = v[j];
            }
        }
        __syncthreads();
    }
    SL_STAMP(8)
    {
        const int kk = min(a.k_budget, a.mode == MODE_EMIT_ONLY ? 0x7fffffff : N);
        const int BW = (nbins + 31) >> 5;
        for (int h = warp; h < KH; h += NW) {
            int tau = nbins, r = 0, e_lower = 0;
            if (kk > 0) {
                const unsigned* H = shist + h * nbins;
                const int blo = lane * BW, bhi = min(nbins, blo + BW);
                unsigned bs = 0;
                for (int bin = blo; bin < bhi; ++bin) bs += H[bin];
                unsigned suf = bs;                                   // bins of this lane's block and above
#pragma unroll
                for (int d = 1; d < 32; d <<= 1) {
                    const unsigned t = __shfl_down_sync(0xffffffffu, suf, d);
                    if (lane + d < 32) suf += t;
                }
                const unsigned ball = __ballot_sync(0xffffffffu, suf >= (unsigned)kk);
                if (ball == 0) {        // fewer than kk keys in total: everything is selected
                    tau = -1;
                    r = 0;
                } else {
                    const int L = 31 - __clz(ball);                  // highest block whose suffix reaches kk
                    int tau_l = 0, gt_l = 0;
                    if (lane == L) {
                        unsigned cum = suf - bs;
                        for (int bin = bhi - 1; bin >= blo; --bin) {
                            const unsigned v = H[bin];
                            if (cum + v >= (unsigned)kk) { tau_l = bin; gt_l = (int)cum; break; }
                            cum += v;
                        }
                    }
                    tau = __shfl_sync(0xffffffffu, tau_l, L);
                    r = kk - __shfl_sync(0xffffffffu, gt_l, L);
                    if (a.mode == MODE_EMIT_ONLY) {                  // threshold ties owned by lower ranks
                        for (int rr = lane; rr < a.rank; rr += 32)
                            e_lower += (int)__ldcg(hist_b + rr * hslice + h * nbins + tau);
                        e_lower = warp_sum(e_lower);
                    }
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
    SL_STAMP(3)

    // ---------------------------------------------------------------- pass B2: own counts per task
    // A task is (head, sub-range of the chunk). In the shared-memory layout a lane tests four
    // consecutive keys of one head per 8-byte load: adding (0x7fff - tau) to a 16-bit score sets
    // bit 15 iff score > tau, adding (0x8000 - tau) iff score >= tau, two scores per 32-bit add.
    const int len = t1 - t0;
    const int sub = ((len + S - 1) / S + 127) / 128 * 128;
    const int ntasks = KH * S;
    for (int task = warp; task < ntasks; task += NW) {
        const int h = task % KH, s = task / KH;
        const int lo = t0 + min(len, s * sub), hi = t0 + min(len, (s + 1) * sub);
        const int tau = s_tau[h];
        int gtM = 0, eqM = 0, eqS = 0;
        if (fast) {
            const unsigned short* row = sscores + h * rowh;
            const int elo = max(lo, a.s_end) - t0, ehi = min(hi, a.r_start) - t0;
            const unsigned cgt = (unsigned)(0x7fff - tau) * 0x10001u, cge = (unsigned)(0x8000 - tau) * 0x10001u;
            for (int g0 = elo & ~3; g0 < ehi; g0 += 128) {
                const int tl = g0 + 4 * lane;
                uint2 x = make_uint2(0u, 0u);
                if (tl < ehi) x = *reinterpret_cast<const uint2*>(row + tl);
                unsigned vlo = 0x80008000u, vhi = 0x80008000u;
                if (tl < elo || tl + 3 >= ehi) {
                    vlo = ((tl >= elo && tl < ehi) ? 0x8000u : 0u) | ((tl + 1 >= elo && tl + 1 < ehi) ? 0x80000000u : 0u);
                    vhi = ((tl + 2 >= elo && tl + 2 < ehi) ? 0x8000u : 0u) | ((tl + 3 >= elo && tl + 3 < ehi) ? 0x80000000u : 0u);
                }
                const unsigned glo = (x.x + cgt) & vlo, ghi = (x.y + cgt) & vhi;
                const unsigned elo_ = (x.x + cge) & vlo & ~glo, ehi_ = (x.y + cge) & vhi & ~ghi;
                gtM += __popc(glo | (ghi >> 1));
                eqM += __popc(elo_ | (ehi_ >> 1));
            }
            gtM = __reduce_add_sync(0xffffffffu, gtM);
            eqM = __reduce_add_sync(0xffffffffu, eqM);
            if (s == 0) {       // threshold ties inside the sink part of this chunk
                for (int tb = t0; tb < min(t1, a.s_end); tb += 32) {
                    const int t = tb + lane;
                    const bool tie = t < min(t1, a.s_end) && (int)row[t - t0] == tau;
                    eqS += __popc(__ballot_sync(0xffffffffu, tie));
                }
            }
        } else {
            for (int tb = lo; tb < hi; tb += 32) {
                const int t = tb + lane;
                const bool valid = t < hi;
                const int v = valid ? (int)sc[(t - t0) * KH + h] : -2;
                const bool mid = valid && t >= a.s_end && t < a.r_start;
                gtM += __popc(__ballot_sync(0xffffffffu, mid && v > tau));
                eqM += __popc(__ballot_sync(0xffffffffu, mid && v == tau));
                eqS += __popc(__ballot_sync(0xffffffffu, valid && t < a.s_end && v == tau));
            }
        }
        if (lane == 0) {
            s_task[(h * S + s) * 3 + 0] = gtM;
            s_task[(h * S + s) * 3 + 1] = eqM;
            s_task[(h * S + s) * 3 + 2] = eqS;
        }
    }
    __syncthreads();
    SL_STAMP(10)
    if (multi) {
        for (int h = tid; h < KH; h += NT) {
            uint4 v = make_uint4(0, 0, 0, 0);
            for (int s = 0; s < S; ++s) {
                v.x += s_task[(h * S + s) * 3 + 0];
                v.y += s_task[(h * S + s) * 3 + 1];
                v.z += s_task[(h * S + s) * 3 + 2];
            }
            a.seg[((long long)b * KH + h) * a.ctas_per_b + c] = v;
        }
        sl::grid_barrier(&sync[0], ++barriers * (unsigned)a.ctas_per_b, a.status);
    }
    SL_STAMP(4)

    // ---------------------------------------------------------------- pass B3: prefix over chunks
    for (int h = warp; h < KH; h += NW) {
        int pre_gt = 0, pre_eq = 0, tot_gt = 0, tot_eq = 0, tot_eqS = 0;
        if (multi) {
            const uint4* segb = a.seg + ((long long)b * KH + h) * a.ctas_per_b;
            for (int cc0 = 0; cc0 < a.ctas_per_b; cc0 += 32 * 5) {
                uint4 v[5];
#pragma unroll
                for (int j = 0; j < 5; ++j) {            // all loads first: one round trip
                    const int cc = cc0 + j * 32 + lane;
                    v[j] = cc < a.ctas_per_b ? __ldcg(segb + cc) : make_uint4(0, 0, 0, 0);
                }
#pragma unroll
                for (int j = 0; j < 5; ++j) {
                    const int cc = cc0 + j * 32 + lane;
                    tot_gt += v[j].x; tot_eq += v[j].y; tot_eqS += v[j].z;
                    if (cc < c) { pre_gt += v[j].x; pre_eq += v[j].y; }
                }
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
    SL_STAMP(5)

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
        if (fast) {
            const unsigned short* row = sscores + h * rowh;
            const int elo = max(lo, a.s_end) - t0, ehi = min(hi, a.r_start) - t0;
            const unsigned cgt = (unsigned)(0x7fff - tau) * 0x10001u, cge = (unsigned)(0x8000 - tau) * 0x10001u;
            int out_base = a.s_end + gt_before + min(eq_before, rM);
            // Nearly every task takes either all of its threshold ties or none (the quota runs out
            // inside one task per head). Those go through a loop that handles 256 keys per trip:
            // two independent groups, their per-lane counts packed into one word and ranked by a
            // single warp scan.
            const int eq_task = (int)s_task[(h * S + s) * 3 + 1];
            const int mode = eq_before + eq_task <= rM ? 1 : (eq_before >= rM ? 0 : 2);
            const unsigned cth = mode == 1 ? cge : cgt;          // ties count as selected, or do not
            for (int g0 = elo & ~3; g0 < ehi && mode != 2; g0 += 256) {
                unsigned sb2[2];
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                    const int tl = g0 + 128 * u + 4 * lane;
                    uint2 x = make_uint2(0u, 0u);
                    if (tl < ehi) x = *reinterpret_cast<const uint2*>(row + tl);
                    unsigned vlo = 0x80008000u, vhi = 0x80008000u;
                    if (tl < elo || tl + 3 >= ehi) {
                        vlo = ((tl >= elo && tl < ehi) ? 0x8000u : 0u) | ((tl + 1 >= elo && tl + 1 < ehi) ? 0x80000000u : 0u);
                        vhi = ((tl + 2 >= elo && tl + 2 < ehi) ? 0x8000u : 0u) | ((tl + 3 >= elo && tl + 3 < ehi) ? 0x80000000u : 0u);
                    }
                    const unsigned slo = (x.x + cth) & vlo, shi = (x.y + cth) & vhi;
                    sb2[u] = ((slo >> 15) & 1u) | ((slo >> 30) & 2u) | ((shi >> 13) & 4u) | ((shi >> 28) & 8u);
                }
                const unsigned ns2 = (unsigned)__popc(sb2[0]) | ((unsigned)__popc(sb2[1]) << 16);
                unsigned inc = ns2;
#pragma unroll
                for (int d = 1; d < 32; d <<= 1) {
                    const unsigned t = __shfl_up_sync(0xffffffffu, inc, d);
                    if (lane >= d) inc += t;
                }
                const unsigned tot = __shfl_sync(0xffffffffu, inc, 31);
                const unsigned exc = inc - ns2;
                const int ex0 = out_base + (int)(exc & 0xffffu), ex1 = out_base + (int)(tot & 0xffffu) + (int)(exc >> 16);
#pragma unroll
                for (int u = 0; u < 2; ++u) {
                    const int tl = g0 + 128 * u + 4 * lane, ex = u ? ex1 : ex0;
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        if ((sb2[u] >> i) & 1u) {
                            const int pos = ex + __popc(sb2[u] & ((1u << i) - 1u));
                            if (pos < a.cap) oi[pos] = t0 + tl + i;
                            else if (a.status) atomicExch(a.status, 2);
                        }
                    }
                }
                out_base += (int)(tot & 0xffffu) + (int)(tot >> 16);
            }
            for (int g0 = elo & ~3; g0 < ehi && mode == 2; g0 += 128) {
                const int tl = g0 + 4 * lane;
                uint2 x = make_uint2(0u, 0u);
                if (tl < ehi) x = *reinterpret_cast<const uint2*>(row + tl);
                unsigned vlo = 0x80008000u, vhi = 0x80008000u;
                if (tl < elo || tl + 3 >= ehi) {
                    vlo = ((tl >= elo && tl < ehi) ? 0x8000u : 0u) | ((tl + 1 >= elo && tl + 1 < ehi) ? 0x80000000u : 0u);
                    vhi = ((tl + 2 >= elo && tl + 2 < ehi) ? 0x8000u : 0u) | ((tl + 3 >= elo && tl + 3 < ehi) ? 0x80000000u : 0u);
                }
                const unsigned glo = (x.x + cgt) & vlo, ghi = (x.y + cgt) & vhi;
                const unsigned elo_ = (x.x + cge) & vlo & ~glo, ehi_ = (x.y + cge) & vhi & ~ghi;
                // four flag bits per lane, bit i = key tl + i
                const unsigned gb = ((glo >> 15) & 1u) | ((glo >> 30) & 2u) | ((ghi >> 13) & 4u) | ((ghi >> 28) & 8u);
                const unsigned eb = ((elo_ >> 15) & 1u) | ((elo_ >> 30) & 2u) | ((ehi_ >> 13) & 4u) | ((ehi_ >> 28) & 8u);
                const int ne = __popc(eb);
                const int tot_e = __reduce_add_sync(0xffffffffu, ne);
                unsigned tb = 0;
                if (eq_before + tot_e <= rM) {
                    tb = eb;                                    // every tie of this group is inside the quota
                } else if (eq_before < rM) {                    // the quota runs out inside this group
                    int inc = ne;
#pragma unroll
                    for (int d = 1; d < 32; d <<= 1) {
                        const int t = __shfl_up_sync(0xffffffffu, inc, d);
                        if (lane >= d) inc += t;
                    }
                    const int ex = eq_before + inc - ne;
#pragma unroll
                    for (int i = 0; i < 4; ++i)
                        if (((eb >> i) & 1u) && ex + __popc(eb & ((1u << i) - 1u)) < rM) tb |= 1u << i;
                }
                const unsigned sb = gb | tb;
                const int ns = __popc(sb);
                int inc = ns;
#pragma unroll
                for (int d = 1; d < 32; d <<= 1) {
                    const int t = __shfl_up_sync(0xffffffffu, inc, d);
                    if (lane >= d) inc += t;
                }
                const int ex = out_base + inc - ns;
#pragma unroll
                for (int i = 0; i < 4; ++i) {
                    if ((sb >> i) & 1u) {
                        const int pos = ex + __popc(sb & ((1u << i) - 1u));
                        if (pos < a.cap) oi[pos] = t0 + tl + i;
                        else if (a.status) atomicExch(a.status, 2);
                    }
                }
                out_base += __shfl_sync(0xffffffffu, inc, 31);
                eq_before += tot_e;
            }
            if (task == 0) { SL_STAMP(9) }
            // always-kept keys of this sub-range: the sink at its own index, the recent window at the end
            for (int tb2 = lo; tb2 < min(hi, a.s_end); tb2 += 32)
                if (tb2 + lane < min(hi, a.s_end) && tb2 + lane < a.cap) oi[tb2 + lane] = tb2 + lane;
            for (int tb2 = max(lo, a.r_start); tb2 < hi; tb2 += 32) {
                const int t = tb2 + lane, pos = a.s_end + selM + (t - a.r_start);
                if (t < hi) {
                    if (pos < a.cap) oi[pos] = t;
                    else if (a.status) atomicExch(a.status, 2);
                }
            }
        } else {
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
    }
    SL_STAMP(6)

    // ---------------------------------------------------------------- leave the workspace zeroed
    if (multi) {
        if (a.mode == MODE_FUSED || a.mode == MODE_FROM_SCORES) {
            const int total = KH * nbins;
            const int slice = (total + a.ctas_per_b - 1) / a.ctas_per_b;
            const int z0 = c * slice, z1 = min(total, z0 + slice);
            for (int cp = 0; cp < a.ncopy; ++cp)
                for (int i = z0 + tid; i < z1; i += NT) hist_b[cp * hslice + i] = 0;
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

kernel_t pick_kernel(int G, int KH) {
    if (32 % KH != 0) return scan_topk_kernel<0>;      // lanes do not keep one head: direct popcounts
    switch (sliced_planes(G)) {
        case 1: return scan_topk_kernel<1>;
        case 2: return scan_topk_kernel<2>;
        case 3: return scan_topk_kernel<3>;
        case 4: return scan_topk_kernel<4>;
        default: return scan_topk_kernel<0>;
    }
}

// log2 of the coarse bin width of the lean fused kernel: at least 32 fine bins, at most 32 coarse bins
int coarse_shift(int nbins) {
    int s = 5;
    while (((nbins - 1) >> s) + 1 > 32) ++s;
    return s;
}

struct WsLayout {
    size_t sync_off, hist_off, chist_off, seg_off, score_off, total;
    size_t epoch_off, chist2_off, pub_off, puba_off, wsc_off;     // the one-barrier kernel's own areas
};

WsLayout ws_layout(int B, long long N, int KH, int G, bool with_hist, bool spill, int nbins = 0) {
    WsLayout w;
    const int max_cpb = std::max(1, sl::sm_count() * 2);
    size_t off = 0;
    w.sync_off = off; off = align_up(off + (size_t)B * 2 * 4, 256);
    w.hist_off = off; if (with_hist) off = align_up(off + (size_t)NCOPY * B * KH * (nbins > 0 ? nbins : 128 * G + 1) * 4, 256);
    w.chist_off = off; if (with_hist) off = align_up(off + (size_t)NCOPY * B * KH * 32 * 4, 256);
    w.seg_off = off; off = align_up(off + (size_t)B * max_cpb * KH * 16, 256);
    w.score_off = off; if (spill) off = align_up(off + (size_t)B * N * KH * 2, 256);
    w.epoch_off = w.chist2_off = w.pub_off = w.puba_off = w.wsc_off = off;
    if (with_hist && nbins <= 0) {
        const int nb = 128 * G + 1;
        w.epoch_off = off; off = align_up(off + (size_t)B * 4, 256);
        w.chist2_off = off; off = align_up(off + (size_t)2 * B * KH * slscan::lean_nc(nb) * 4, 256);
        w.pub_off = off; off = align_up(off + (size_t)std::max(B, sl::sm_count()) * KH * slscan::lean_nc(nb) * 16, 256);
        w.puba_off = off; off = align_up(off + (size_t)std::max(B, sl::sm_count()) * KH * slscan::lean_nc(nb) * 2, 256);
        w.wsc_off = off; off = align_up(off + (size_t)B * KH * slscan::LEAN_MAX_WIN * 2, 256);
    }
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

int launch(const ScanArgs& a_in, const Plan& p, cudaStream_t s) {
    ScanArgs a = a_in;
    a.dbg = SL_STAMP_BUF;
    kernel_t kern = pick_kernel(a.G, a.KH);
    SL_CUDA_OK(sl::ensure_dyn_smem(reinterpret_cast<const void*>(kern), p.smem));
    const unsigned grid = (unsigned)(a.B * p.ctas_per_b);
    SL_CUDA_OK(sl::launch_kernel(kern, dim3(grid), dim3(NT), p.smem, s, p.cooperative, a));
    return SL_OK;
}

}  // namespace

#ifdef SL_SCAN_TIMING
namespace slscan { unsigned long long* g_dbg_timing = nullptr; }
#endif
static int g_lean = 1;     // 1: one-barrier kernel where it applies (default); 2: the flagged-word kernel; 0: the general kernel

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
    return sl::scan_topk_impl(d_q_codes, d_k_codes, k_batch_stride, B, N, KH, QH, gqa_layout, k, sink, recent, d_idx,
                              idx_capacity, d_cnt, d_scores_out, d_workspace, workspace_bytes, d_status, nullptr, 0.0, 0,
                              stream);
}

// d_pos == nullptr: N keys, budget k. Otherwise N is the capacity the launch is planned for, the context
// is *d_pos + 1 keys and the budget follows the reference's rule from mask_out / min_remain on the device.
int sl::scan_topk_impl(const uint32_t* d_q_codes, const uint32_t* d_k_codes, int64_t k_batch_stride, int B, int64_t N,
                       int KH, int QH, int gqa_layout, int k, int sink, int recent, int32_t* d_idx, int idx_capacity,
                       int32_t* d_cnt, int16_t* d_scores_out, void* d_workspace, size_t workspace_bytes,
                       int32_t* d_status, const long long* d_pos, double mask_out, int min_remain, void* stream) {
    SL_REQUIRE(d_q_codes && d_k_codes && d_idx && d_cnt && d_workspace, SL_EINVAL, "sl_scan_topk: null pointer");
    if (d_pos) {
        SL_REQUIRE(N > 0 && mask_out >= 0.0 && mask_out <= 1.0 && min_remain >= 0, SL_EINVAL,
                   "sl_scan_topk: bad capacity / mask_out / min_remain for a device-side context length");
        k = (int)std::max<int64_t>(std::min<int64_t>(N, min_remain), N - (int64_t)((double)N * mask_out));
    }
    if (int rc = check_common("sl_scan_topk", B, N, KH, QH)) return rc;
    SL_REQUIRE(gqa_layout == SL_GQA_INTERLEAVED || gqa_layout == SL_GQA_BLOCKED, SL_EINVAL,
               "sl_scan_topk: unknown gqa_layout %d", gqa_layout);
    SL_REQUIRE(k >= 0 && sink >= 0 && recent >= 0, SL_EINVAL, "sl_scan_topk: negative k/sink/recent");
    SL_REQUIRE(sl::aligned16(d_q_codes) && sl::aligned16(d_k_codes) && k_batch_stride % 4 == 0, SL_EALIGN,
               "sl_scan_topk: codes must be 16-byte aligned");
    SL_REQUIRE(k_batch_stride == 0 || k_batch_stride >= N * KH * 4, SL_ESHAPE, "sl_scan_topk: batch stride shorter than a batch row");
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
    const int s_end0 = (int)std::min<int64_t>(sink, N);
    const int nwin0 = s_end0 + (int)(N - std::max<int64_t>(s_end0, N - recent));
    const bool lean_ok = p.cooperative && !p.spill && B * p.ctas_per_b <= sl::sm_count() &&
                         slscan::lean_covers(KH, G, p.ctas_per_b, p.chunk, d_pos ? sink + recent : nwin0);
    SL_REQUIRE(d_pos == nullptr || lean_ok, SL_ESHAPE,
               "sl_scan_topk: a device-side context length needs a shape the one-barrier kernel covers");
    if ((g_lean == 1 || d_pos) && lean_ok) {
        // the common decode shape: one barrier, everything the tail needs published before it
        slscan::LeanArgs f = {};
        f.q = reinterpret_cast<const uint4*>(d_q_codes);
        f.k = reinterpret_cast<const uint4*>(d_k_codes);
        f.k_bstride = k_batch_stride / 4;
        f.B = B; f.KH = KH; f.G = G; f.layout = gqa_layout; f.N = (int)N;
        f.k_budget = k;
        f.s_end = s_end0;
        f.r_start = (int)std::max<int64_t>(f.s_end, N - recent);
        f.idx = d_idx; f.cap = idx_capacity; f.cnt = d_cnt;
        f.scores_out = d_scores_out;
        f.sync = reinterpret_cast<unsigned*>(ws + w.sync_off);
        f.epoch = reinterpret_cast<unsigned*>(ws + w.epoch_off);
        f.chist = reinterpret_cast<unsigned*>(ws + w.chist2_off);
        f.pub = reinterpret_cast<uint4*>(ws + w.pub_off);
        f.puba = reinterpret_cast<unsigned short*>(ws + w.puba_off);
        f.wsc = reinterpret_cast<unsigned short*>(ws + w.wsc_off);
        f.status = d_status;
        f.ctas_per_b = p.ctas_per_b; f.chunk = p.chunk; f.nbins = p.nbins; f.S = p.S;
        f.d_pos = d_pos; f.sink = sink; f.recent = recent; f.min_remain = min_remain; f.mask_out = mask_out;
        f.NC = slscan::lean_nc(p.nbins);
        f.nc_magic = (unsigned)(((1ull << 32) + f.NC - 1) / f.NC);
        const int roww = (p.chunk >> 1) + ((4 - (p.chunk >> 1)) & 31);
        f.rowh = 2 * roww;
        const size_t smem = slscan::lean_plan_smem(f, KH, p.nbins, p.S, p.chunk);
        if (smem <= (size_t)SMEM_BUDGET + 24 * 1024) return slscan::launch_lean(f, smem, s);
    }
    if (g_lean && p.cooperative && !p.spill && slscan::fused_covers(KH, G) && p.chunk < (1 << 21) &&
        (long long)NCOPY * B * KH * p.nbins < (1ll << 30)) {
        // the two-phase kernel with flagged words (also the form the sequence shards use)
        slscan::FusedArgs f = {};
        f.q = reinterpret_cast<const uint4*>(d_q_codes);
        f.k = reinterpret_cast<const uint4*>(d_k_codes);
        f.k_bstride = k_batch_stride / 4;
        f.B = B; f.KH = KH; f.G = G; f.layout = gqa_layout; f.N = (int)N;
        f.k_budget = k;
        f.s_end = (int)std::min<int64_t>(sink, N);
        f.r_start = (int)std::max<int64_t>(f.s_end, N - recent);
        f.idx = d_idx; f.cap = idx_capacity; f.cnt = d_cnt;
        f.scores_out = d_scores_out;
        f.hist = reinterpret_cast<unsigned*>(ws + w.hist_off);
        f.chist = reinterpret_cast<unsigned*>(ws + w.chist_off);
        f.seg = reinterpret_cast<unsigned long long*>(ws + w.seg_off);
        f.sync = reinterpret_cast<unsigned*>(ws + w.sync_off);
        f.status = d_status;
        f.ctas_per_b = p.ctas_per_b; f.chunk = p.chunk; f.nbins = p.nbins; f.S = p.S;
        f.cws = coarse_shift(p.nbins);
        const int roww = (p.chunk >> 1) + ((4 - (p.chunk >> 1)) & 31);
        f.rowh = 2 * roww;
        const size_t smem = slscan::fused_plan_smem(f, KH, p.nbins, p.S, p.chunk);
        if (smem <= (size_t)SMEM_BUDGET + 24 * 1024) return slscan::launch_fused(f, smem, s);
    }
    ScanArgs a = {};
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
    a.seg = reinterpret_cast<uint4*>(ws + w.seg_off);
    a.sync = reinterpret_cast<unsigned*>(ws + w.sync_off);
    a.status = d_status;
    a.ctas_per_b = p.ctas_per_b; a.chunk = p.chunk; a.nbins = p.nbins; a.S = p.S;
    a.mode = MODE_FUSED; a.R = 1; a.rank = 0; a.ncopy = NCOPY;
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
    a.mode = MODE_HIST_ONLY; a.R = 1; a.rank = 0; a.ncopy = 1;
    return launch(a, p, static_cast<cudaStream_t>(stream));
}

extern "C" size_t sl_scan_topk_sharded_slot_bytes(int B, int KH, int QH) {
    if (B <= 0 || KH <= 0 || QH <= 0 || QH % KH) return 0;
    const int nbins = 128 * (QH / KH) + 1;
    // whichever of the two kernels serves the shape: the larger of their messages
    return std::max(slscan::shard_message_bytes(B, KH, nbins, coarse_shift(nbins)), slscan::lean_shard_message_bytes(B, KH, nbins));
}

extern "C" int sl_scan_topk_sharded(const uint32_t* d_q_codes, const uint32_t* d_k_codes, int64_t k_batch_stride, int B,
                                    int64_t N_local, int64_t tok_offset, int64_t N_global, int KH, int QH,
                                    int gqa_layout, int k, int sink, int recent, int32_t* d_idx, int idx_capacity,
                                    int32_t* d_cnt, void* d_workspace, size_t workspace_bytes, void* const* peer_bufs,
                                    int rank, int R, size_t slot_stride, int32_t* d_status, void* stream) {
    SL_REQUIRE(d_q_codes && d_k_codes && d_idx && d_cnt && d_workspace && peer_bufs, SL_EINVAL,
               "sl_scan_topk_sharded: null pointer");
    if (int rc = check_common("sl_scan_topk_sharded", B, N_local, KH, QH)) return rc;
    SL_REQUIRE(gqa_layout == SL_GQA_INTERLEAVED || gqa_layout == SL_GQA_BLOCKED, SL_EINVAL,
               "sl_scan_topk_sharded: unknown gqa_layout %d", gqa_layout);
    SL_REQUIRE(R >= 1 && R <= 8 && rank >= 0 && rank < R, SL_EINVAL, "sl_scan_topk_sharded: bad rank %d of %d", rank, R);
    SL_REQUIRE(R * B + B <= slscan::SHARD_EPOCH_WORD + 1, SL_ESHAPE, "sl_scan_topk_sharded: (R+1)*B exceeds the flag area");
    SL_REQUIRE(N_local > 0, SL_ESHAPE, "sl_scan_topk_sharded: an empty shard must use sl_scan_hist + sl_select_emit (every rank has to launch the exchange)");
    SL_REQUIRE(tok_offset >= 0 && tok_offset + N_local <= N_global, SL_ESHAPE, "sl_scan_topk_sharded: shard outside the context");
    SL_REQUIRE(k >= 0 && sink >= 0 && recent >= 0, SL_EINVAL, "sl_scan_topk_sharded: negative k/sink/recent");
    SL_REQUIRE(sl::aligned16(d_q_codes) && sl::aligned16(d_k_codes) && k_batch_stride % 4 == 0, SL_EALIGN,
               "sl_scan_topk_sharded: codes must be 16-byte aligned");
    SL_REQUIRE(k_batch_stride >= N_local * KH * 4, SL_ESHAPE, "sl_scan_topk_sharded: batch stride shorter than a batch row");
    const int G = QH / KH;
    const Plan p = make_plan(B, N_local, KH, G, false);
    // the fused form needs every rank to run the lean kernel; other shapes use sl_scan_hist + sl_select_emit
    SL_REQUIRE(p.cooperative && !p.spill && slscan::fused_covers(KH, G) && p.chunk < (1 << 21), SL_ESHAPE,
               "sl_scan_topk_sharded: shape not covered by the fused kernel");
    const WsLayout w = ws_layout(B, N_local, KH, G, true, false);
    SL_REQUIRE(workspace_bytes >= w.total, SL_EWORKSPACE, "sl_scan_topk_sharded: workspace %zu < required %zu",
               workspace_bytes, w.total);
    const size_t msg = slscan::shard_message_bytes(B, KH, p.nbins, coarse_shift(p.nbins));
    SL_REQUIRE(slot_stride >= msg && slot_stride % 16 == 0, SL_ESHAPE, "sl_scan_topk_sharded: slot of %zu bytes < message of %zu",
               slot_stride, msg);
    const int64_t s_end_g = std::min<int64_t>(sink, N_global);
    const int64_t r_start_g = std::max<int64_t>(s_end_g, N_global - recent);
    const int64_t s_end = std::min<int64_t>(std::max<int64_t>(s_end_g - tok_offset, 0), N_local);
    const int64_t r_start = std::min<int64_t>(std::max<int64_t>(r_start_g - tok_offset, s_end), N_local);
    const int64_t need = std::min<int64_t>(N_local, (int64_t)k + s_end + (N_local - r_start));
    SL_REQUIRE(idx_capacity >= need, SL_ESHAPE, "sl_scan_topk_sharded: idx_capacity %d < %lld", idx_capacity, (long long)need);
    unsigned char* ws = static_cast<unsigned char*>(d_workspace);
    for (int r = 0; r < R; ++r)
        SL_REQUIRE(peer_bufs[r] != nullptr && sl::aligned16(peer_bufs[r]), SL_EINVAL, "sl_scan_topk_sharded: bad buffer of rank %d", r);
    if (g_lean == 1 && B * p.ctas_per_b <= sl::sm_count() && 2 * B <= slscan::SHARD_EPOCH_WORD &&
        slscan::lean_covers(KH, G, p.ctas_per_b, p.chunk, sink + recent) &&
        slot_stride >= slscan::lean_shard_message_bytes(B, KH, p.nbins)) {
        // the one-barrier kernel: records of every chunk, the rank's counts sent by all CTAs at once
        slscan::LeanArgs f = {};
        f.q = reinterpret_cast<const uint4*>(d_q_codes);
        f.k = reinterpret_cast<const uint4*>(d_k_codes);
        f.k_bstride = k_batch_stride / 4;
        f.B = B; f.KH = KH; f.G = G; f.layout = gqa_layout; f.N = (int)N_local;
        f.k_budget = k;
        f.kk = (int)std::min<int64_t>(k, N_global);
        f.s_end = (int)s_end; f.r_start = (int)r_start;
        f.idx = d_idx; f.cap = idx_capacity; f.cnt = d_cnt;
        f.sync = reinterpret_cast<unsigned*>(ws + w.sync_off);
        f.epoch = reinterpret_cast<unsigned*>(ws + w.epoch_off);
        f.chist = reinterpret_cast<unsigned*>(ws + w.chist2_off);
        f.pub = reinterpret_cast<uint4*>(ws + w.pub_off);
        f.puba = reinterpret_cast<unsigned short*>(ws + w.puba_off);
        f.wsc = reinterpret_cast<unsigned short*>(ws + w.wsc_off);
        f.status = d_status;
        f.ctas_per_b = p.ctas_per_b; f.chunk = p.chunk; f.nbins = p.nbins; f.S = p.S;
        f.NC = slscan::lean_nc(p.nbins);
        f.nc_magic = (unsigned)(((1ull << 32) + f.NC - 1) / f.NC);
        const int roww = (p.chunk >> 1) + ((4 - (p.chunk >> 1)) & 31);
        f.rowh = 2 * roww;
        for (int r = 0; r < R; ++r) f.peer[r] = static_cast<unsigned char*>(peer_bufs[r]);
        f.R = R; f.rank = rank;
        f.slot_stride = slot_stride;
        f.pflags_off = (unsigned long long)R * slot_stride;
        const size_t smem = slscan::lean_plan_smem(f, KH, p.nbins, p.S, p.chunk);
        if (smem <= (size_t)SMEM_BUDGET + 24 * 1024) return slscan::launch_lean(f, smem, static_cast<cudaStream_t>(stream));
    }
    slscan::FusedArgs f = {};
    f.q = reinterpret_cast<const uint4*>(d_q_codes);
    f.k = reinterpret_cast<const uint4*>(d_k_codes);
    f.k_bstride = k_batch_stride / 4;
    f.B = B; f.KH = KH; f.G = G; f.layout = gqa_layout; f.N = (int)N_local;
    f.k_budget = k;
    f.kk = (int)std::min<int64_t>(k, N_global);
    f.s_end = (int)s_end; f.r_start = (int)r_start;
    f.idx = d_idx; f.cap = idx_capacity; f.cnt = d_cnt;
    f.hist = reinterpret_cast<unsigned*>(ws + w.hist_off);
    f.chist = reinterpret_cast<unsigned*>(ws + w.chist_off);
    f.seg = reinterpret_cast<unsigned long long*>(ws + w.seg_off);
    f.sync = reinterpret_cast<unsigned*>(ws + w.sync_off);
    f.status = d_status;
    f.ctas_per_b = p.ctas_per_b; f.chunk = p.chunk; f.nbins = p.nbins; f.S = p.S;
    f.cws = coarse_shift(p.nbins);
    const int roww = (p.chunk >> 1) + ((4 - (p.chunk >> 1)) & 31);
    f.rowh = 2 * roww;
    const size_t smem = slscan::fused_plan_smem(f, KH, p.nbins, p.S, p.chunk);
    SL_REQUIRE(smem <= (size_t)SMEM_BUDGET + 24 * 1024, SL_ESHAPE, "sl_scan_topk_sharded: chunk does not fit in shared memory");
    for (int r = 0; r < R; ++r) {
        SL_REQUIRE(peer_bufs[r] != nullptr && sl::aligned16(peer_bufs[r]), SL_EINVAL, "sl_scan_topk_sharded: bad buffer of rank %d", r);
        f.peer[r] = static_cast<unsigned char*>(peer_bufs[r]);
    }
    f.R = R; f.rank = rank;
    f.slot_stride = slot_stride;
    f.pflags_off = (unsigned long long)R * slot_stride;
    return slscan::launch_fused(f, smem, static_cast<cudaStream_t>(stream));
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
    const Plan p = make_plan_given_scores(B, N_local, KH, G);
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
    a.seg = reinterpret_cast<uint4*>(ws + w.seg_off);
    a.sync = reinterpret_cast<unsigned*>(ws + w.sync_off);
    a.status = d_status;
    a.ctas_per_b = p.ctas_per_b; a.chunk = p.chunk; a.nbins = p.nbins; a.S = p.S;
    a.mode = MODE_EMIT_ONLY; a.R = R; a.rank = rank; a.ncopy = 1; a.stage = p.stage ? 1 : 0;
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
    const Plan p = make_plan_given_scores(B, N, KH, 1, max_score + 1);
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
    a.seg = reinterpret_cast<uint4*>(ws + w.seg_off);
    a.sync = reinterpret_cast<unsigned*>(ws + w.sync_off);
    a.status = d_status;
    a.ctas_per_b = p.ctas_per_b; a.chunk = p.chunk; a.nbins = p.nbins; a.S = p.S;
    a.mode = MODE_FROM_SCORES; a.R = 1; a.rank = 0; a.ncopy = NCOPY; a.stage = p.stage ? 1 : 0;
    return launch(a, p, s);
}

namespace slscan { void set_scan_kernel(int v) { g_lean = v; } }

#ifdef SL_SCAN_TIMING
// Profiling builds only (not in the public header): thread 0 of every CTA of the scan kernels stores
// the SM cycle counter at its phase boundaries into d_buf [grid][16] uint64.
extern "C" void sl_profile_scan_timing(void* d_buf) { slscan::g_dbg_timing = static_cast<unsigned long long*>(d_buf); }
#endif
