// The decode step's fused Hamming scan + exact top-k + sink/recent window for the common shapes
// (several CTAs per batch row, a chunk's scores fit in shared memory, kv heads divide the warp, the
// bit-sliced scorer covers the group size). One cooperative launch with ONE grid-wide dependency:
// everything a CTA needs from the other chunks after the barrier is published before it, so the
// tail is two trips to L2 and one pass over the chunk's scores.
//
//   A  the chunk is cut into S contiguous sub-ranges, each streamed by its own group of warps
//      (8 x 16-byte loads in flight per thread); the bit-sliced scorer leaves the 16-bit scores in
//      shared memory ([head][key], bank-spread) and counts them in a histogram per (sub-range, head)
//   P  per (head, coarse bin of 8 scores): the chunk's 8 counts go to global memory as one 16-byte
//      record and the chunk's number of keys above the bin as a 16-bit word beside it, both laid out
//      [head][coarse bin][chunk] so that all chunks' entries for one bin are contiguous; the bins'
//      counts are added to a small global histogram; the scores of the chunk's sink / recent keys follow
//   -- the only grid barrier (bounded) --
//   T  one warp per head: the global coarse bins give the 8 scores that hold the threshold (trip 1);
//      all chunks' entries for that bin (trip 2: coalesced, one chunk per lane and round) give the
//      threshold itself, the tie quota, and -- from the same registers -- how many selected keys and
//      threshold ties lie in the chunks before this one
//   E  one pass over the chunk's scores: flags, one packed warp scan per 640 keys, the attended
//      keys written at their final positions (ascending, ties to the lowest index, sink and recent
//      window included).
// The coarse histogram is double-buffered by launch parity (a device-side launch counter in the
// workspace, advanced by the last CTA to finish): a launch adds into one buffer and clears the
// other, so nothing has to be cleared while others may still read it and no second grid-wide wait exists.
#include "sl_scan.cuh"
#include "sl_sliced.cuh"

namespace {

using namespace slscan;

__device__ __forceinline__ uint4 ldcg_v4(const void* p) {
    uint4 r;
    asm volatile("ld.global.cg.v4.u32 {%0,%1,%2,%3}, [%4];" : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w) : "l"(p));
    return r;
}
__device__ __forceinline__ unsigned ldcg_u32(const void* p) {
    unsigned r;
    asm volatile("ld.global.cg.u32 %0, [%1];" : "=r"(r) : "l"(p));
    return r;
}
__device__ __forceinline__ unsigned ldcg_u16(const void* p) {
    unsigned short r;
    asm volatile("ld.global.cg.u16 %0, [%1];" : "=h"(r) : "l"(p));
    return r;
}

// SHARD: this rank holds a contiguous part of a longer context (N, s_end, r_start and the indices written are
// local). After the local barrier the CTAs of a batch row add up the chunks' records, a few (head, coarse bin) pairs
// each, and store the rank's counts per score and per coarse bin straight into slot `rank` of EVERY rank's exchange
// buffer (peer stores over NVLink from all SMs at once); each CTA then fences at system scope and adds its share to
// an arrival counter in every buffer, and waits (bounded) until its own buffer's counter shows that all CTAs of all
// ranks have arrived. The threshold is then searched over the R slots, the ties that belong to lower ranks (lower
// key indices) come off this rank's tie quota, and the local prefix comes from the local records as before.
template <int PT, bool SHARD>
__global__ void __launch_bounds__(NT, 1) scan_lean_kernel(const LeanArgs a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int KH = a.KH, nbins = a.nbins, nb1 = (nbins + 4) & ~3, cpb = a.ctas_per_b, S = a.S;   // rows of nb1 words: 16-byte aligned, R[nbins..] = 0
    uint32_t* s_planes = reinterpret_cast<uint32_t*>(smem_raw);                 // [KH][2][PT][4]
    int* s_pbase = reinterpret_cast<int*>(s_planes + KH * 32);                    // [KH][4]
    int* s_tau = s_pbase + KH * 4;                                                // [KH]
    int* s_pre = s_tau + KH;                                                      // [KH][4] {> tau before, == tau before, rM, selM}
    unsigned short* s_win = reinterpret_cast<unsigned short*>(s_pre + KH * 4);    // [KH][LEAN_MAX_WIN]
    unsigned* s_coarse = reinterpret_cast<unsigned*>(s_win + KH * LEAN_MAX_WIN);  // [KH][NC]
    unsigned* shist = reinterpret_cast<unsigned*>(smem_raw + a.hist_off);         // [S][KH][nb1]
    unsigned short* sscores = reinterpret_cast<unsigned short*>(smem_raw + a.score_off);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int b = blockIdx.x / cpb, c = blockIdx.x - b * cpb;
    const int rowh = a.rowh;                                                      // row stride of sscores (halfwords)
    const int khs = 31 - __clz(KH);
    const int NC = a.NC, cslice = a.B * KH * NC;
    sl::pdl_trigger();
    sl::pdl_wait();
    SL_STAMP(0)
    // The context length is a launch argument, or -- so that one captured launch serves every token of
    // a decode loop -- the word *d_pos + 1 with the reference's budget rule evaluated here as Python
    // evaluates it (doubles): k = max(min(n, min_remain), n - int(n * mask_out)).
    int N = a.N, s_end = a.s_end, r_start = a.r_start, k_budget = a.k_budget;
    if (a.d_pos) {
        N = (int)min((long long)a.N, __ldcg(a.d_pos) + 1);
        s_end = min(a.sink, N);
        r_start = max(s_end, N - a.recent);
        k_budget = max(min(N, a.min_remain), N - (int)((double)N * a.mask_out));
    }
    const int t0 = min(N, c * a.chunk), t1 = min(N, t0 + a.chunk);
    const int len = t1 - t0, ncodes = len * KH;
    const int sub = ((len + S - 1) / S + 127) & ~127;                             // keys per sub-range
    const int nwin = s_end + (N - r_start);                                       // always-kept keys of the row
    const unsigned par = __ldcg(a.epoch + b) & 1u;                                // this launch's coarse buffer
    unsigned* chist_b = a.chist + (size_t)par * cslice + b * KH * NC;

    // ------------------------------------------------------------------ A: scan + histograms
    {
        const uint4* base0 = a.k + (size_t)b * a.k_bstride + (size_t)t0 * KH;
        const uint32_t* qb = reinterpret_cast<const uint32_t*>(a.q + (size_t)b * KH * a.G);
        const PlaneWords pw = planes_issue(qb, KH, a.G, a.layout, warp, NW, lane);   // ahead of the stream's loads
        // group g of warps streams sub-range g of the chunk
        const int wpg = NW / S, grp = warp / wpg, wig = warp - grp * wpg;
        const int gbeg = min(ncodes, grp * sub * KH), gend = min(ncodes, (grp + 1) * sub * KH);
        const uint4* base = base0 + gbeg;
        const int gcodes = gend - gbeg;
        uint4 cd[U];
        int tile = wig;
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int i = tile * (32 * U) + u * 32 + lane;
            if (i < gcodes) cd[u] = sl::ld_stream_v4(base + i);
        }
        if (tid == NT - 32) {            // pages the later phases store to
            touch(a.idx + (size_t)b * KH * a.cap);
            touch(a.cnt + b * KH);
            touch(a.pub + (size_t)b * KH * NC * cpb + c);
            touch(a.puba + (size_t)b * KH * NC * cpb + c);
        }
        for (int i = tid; i < S * KH * (nb1 >> 2); i += NT) reinterpret_cast<uint4*>(shist)[i] = make_uint4(0u, 0u, 0u, 0u);
        {   // last launch's coarse buffer: cleared here, added to by the next launch
            unsigned* other = a.chist + (size_t)(par ^ 1u) * cslice + b * KH * NC;
            for (int i = c * NT + tid; i < KH * NC; i += cpb * NT) other[i] = 0;
        }
        planes_finish<PT>(pw, KH, a.G, s_planes, s_pbase, warp, NW, lane);
        stage_planes<PT>(qb, KH, a.G, a.layout, s_planes, s_pbase, warp, NW, lane, 1);   // KH > 8
        __syncthreads();
        uint32_t M[PT][4], Mp[PT][4];
        const int hh = lane & (KH - 1);                       // this lane's head (KH is a power of two <= 32)
        const int sbase = load_planes<PT>(s_planes, s_pbase, hh, M, Mp);
        const int ssh = sliced_shift(a.G);
        unsigned short* srow = sscores + hh * rowh + (gbeg >> khs);
        unsigned* hrow = shist + (grp * KH + hh) * nb1;
        short* so = a.scores_out ? a.scores_out + ((size_t)b * N + t0) * KH + gbeg : nullptr;
        SL_STAMP(1)
#pragma unroll 1
        while (tile * (32 * U) < gcodes) {
            const int i0 = tile * (32 * U) + lane;
            int sv[U];
#pragma unroll
            for (int u = 0; u < U; ++u) sv[u] = sbase + (sliced_score<PT>(cd[u], M, Mp) << ssh);
            tile += wpg;
#pragma unroll
            for (int u = 0; u < U; ++u) {       // next tile's loads before the stores of this one
                const int i = tile * (32 * U) + u * 32 + lane;
                if (i < gcodes) cd[u] = sl::ld_stream_v4(base + i);
            }
#pragma unroll
            for (int u = 0; u < U; ++u) {
                const int i = i0 + u * 32;
                if (i < gcodes) {
                    srow[i >> khs] = (unsigned short)sv[u];
                    atomicAdd(hrow + sv[u], 1u);
                    if (so) so[i] = (short)sv[u];
                }
            }
        }
        __syncthreads();
    }
    SL_STAMP(2)

    // ------------------------------------------------------------------ P: suffix sums, publish
    {
        // scores of the always-kept keys this chunk owns (the other CTAs correct their counts with them)
        if (t0 < s_end || t1 > r_start) {
            if (tid < nwin) {
                const int t = tid < s_end ? tid : r_start + (tid - s_end);
                if (t >= t0 && t < t1)
                    for (int h = 0; h < KH; ++h) a.wsc[((size_t)b * KH + h) * LEAN_MAX_WIN + tid] = sscores[h * rowh + (t - t0)];
            }
        }
        // one thread per (head, coarse bin): the 8 counts (sub-ranges added up) as a record, their sum to shared memory
        const size_t pbase = (size_t)b * KH * NC * cpb + c;
#pragma unroll 1
        for (int i = tid; i < KH * NC; i += NT) {
            const int h = (int)__umulhi((unsigned)i, a.nc_magic), cb = i - h * NC;
            const uint4* R = reinterpret_cast<const uint4*>(shist + h * nb1 + (cb << LEAN_CWS));
            const bool two = (cb << LEAN_CWS) + 4 < nb1;
            unsigned v[8] = {0u, 0u, 0u, 0u, 0u, 0u, 0u, 0u};
#pragma unroll 2
            for (int s2 = 0; s2 < S; ++s2) {
                const uint4 x = R[s2 * KH * (nb1 >> 2)];
                v[0] += x.x; v[1] += x.y; v[2] += x.z; v[3] += x.w;
                if (two) {
                    const uint4 y = R[s2 * KH * (nb1 >> 2) + 1];
                    v[4] += y.x; v[5] += y.y; v[6] += y.z; v[7] += y.w;
                }
            }
            s_coarse[i] = ((v[0] + v[1]) + (v[2] + v[3])) + ((v[4] + v[5]) + (v[6] + v[7]));
            a.pub[pbase + (size_t)i * cpb] =
                make_uint4(v[0] | (v[1] << 16), v[2] | (v[3] << 16), v[4] | (v[5] << 16), v[6] | (v[7] << 16));
        }
        __syncthreads();
        SL_STAMP(7)
        // per head: keys of this chunk above each coarse bin; the bins' counts join the global ones
        const int CPL = (NC + 31) >> 5;
#pragma unroll 1
        for (int h = warp; h < KH; h += NW) {
            unsigned cv[LEAN_CPL_MAX], sum = 0;
#pragma unroll
            for (int i = 0; i < LEAN_CPL_MAX; ++i) {
                const int cb = lane * CPL + i;
                cv[i] = (i < CPL && cb < NC) ? s_coarse[h * NC + cb] : 0u;
                sum += cv[i];
            }
            unsigned above = suffix_sum(sum, lane) - sum;
            unsigned short* pa = a.puba + pbase + (size_t)(h * NC + lane * CPL) * cpb;
#pragma unroll
            for (int i = LEAN_CPL_MAX - 1; i >= 0; --i) {
                if (i < CPL && lane * CPL + i < NC) pa[(size_t)i * cpb] = (unsigned short)above;
                above += cv[i];
            }
            unsigned* dst = chist_b + h * NC + lane * CPL;
#pragma unroll
            for (int i = 0; i < LEAN_CPL_MAX; ++i)
                if (cv[i]) atomicAdd(dst + i, cv[i]);
        }
    }
    SL_STAMP(3)
    sl::grid_barrier(a.sync + 2 * b, (unsigned)cpb, a.status);
    SL_STAMP(4)
    const int npairs = KH * NC;                                   // (head, coarse bin) pairs of a batch row
    if (SHARD) {
        unsigned* own_words = reinterpret_cast<unsigned*>(a.peer[a.rank] + a.pflags_off);
        const unsigned ep = __ldcg(own_words + SHARD_EPOCH_WORD - b);        // launches completed on this buffer for the row
        const size_t fine_off = (size_t)a.B * npairs;                          // slot: coarse [B][KH][NC], fine [B][KH][NC][8]
#pragma unroll 1
        for (int p = c + warp * cpb; p < npairs; p += NW * cpb) {
            const size_t e0 = ((size_t)b * npairs + p) * cpb;
            unsigned pk[4] = {0u, 0u, 0u, 0u};
#pragma unroll
            for (int j = 0; j < LEAN_CPL_MAX; ++j) {
                const int cc = lane + 32 * j;
                if (cc < cpb) {
                    const uint4 x = __ldcg(a.pub + e0 + cc);
                    pk[0] += x.x; pk[1] += x.y; pk[2] += x.z; pk[3] += x.w;
                }
            }
            unsigned val = 0, coarse = 0;
#pragma unroll
            for (int i = 0; i < 8; ++i) {
                const unsigned v = (unsigned)__reduce_add_sync(0xffffffffu, (int)((i & 1) ? (pk[i >> 1] >> 16) : (pk[i >> 1] & 0xffffu)));
                coarse += v;
                val = lane == i ? v : val;
            }
            if (lane == 8) val = coarse;
            if (lane < 9) {
                const size_t w = lane < 8 ? fine_off + ((size_t)b * npairs + p) * 8 + lane : (size_t)b * npairs + p;
                for (int r = 0; r < a.R; ++r)
                    reinterpret_cast<unsigned*>(a.peer[r] + (unsigned long long)a.rank * a.slot_stride)[w] = val;
            }
        }
        __syncthreads();
        if (tid == 0) {
            // every CTA's share of a fixed per-rank total, so that ranks with differently cut rows still agree on the target
            const unsigned share = (unsigned)(((unsigned long long)(c + 1) << 16) / cpb - ((unsigned long long)c << 16) / cpb);
            __threadfence_system();              // the CTA's peer stores (ordered before this by the barrier) first
            for (int r = 0; r < a.R; ++r) {
                unsigned* pf = reinterpret_cast<unsigned*>(a.peer[r] + a.pflags_off) + b;
                asm volatile("red.relaxed.sys.global.add.u32 [%0], %1;" ::"l"(pf), "r"(share) : "memory");
            }
            const unsigned target = (ep + 1u) * (unsigned)a.R * 65536u;
            unsigned v = 0, it = 0;
            for (;;) {
                asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(own_words + b) : "memory");
                if ((int)(v - target) >= 0) break;
                if (++it > 400000u) {            // about a second: give up, tell the host, finish with what is there
                    if (a.status) atomicExch(a.status, 3);
                    break;
                }
                __nanosleep(64);
            }
        }
        __syncthreads();
    }

    // ------------------------------------------------------------------ T: threshold, quota, counts before this chunk
    {
        const int kk = SHARD ? a.kk : min(k_budget, N);
        const int CPL = (NC + 31) >> 5;                      // coarse bins per lane, consecutive
        const unsigned* own_slots = SHARD ? reinterpret_cast<const unsigned*>(a.peer[a.rank]) : nullptr;
        const size_t sstr = SHARD ? (size_t)(a.slot_stride >> 2) : 0;
#pragma unroll 1
        for (int h = warp; h < KH; h += NW) {
            unsigned wv[LEAN_MAX_WIN / 32];                      // scores of the row's always-kept keys
#pragma unroll
            for (int i = 0; i < LEAN_MAX_WIN / 32; ++i) wv[i] = 0xffffu;
            int tau = nbins, pre_gt = 0, pre_eq = 0, rM = 0, selM = 0;
            if (kk > 0) {
                // trip 1: the head's global coarse bins (and the always-kept keys' scores)
                unsigned cv[LEAN_CPL_MAX];
                unsigned csum = 0;
                {
                    const unsigned* src = SHARD ? own_slots + (size_t)(b * KH + h) * NC + lane * CPL : chist_b + h * NC + lane * CPL;
#pragma unroll
                    for (int i = 0; i < LEAN_CPL_MAX; ++i) {
                        cv[i] = 0u;
                        if (i < CPL && lane * CPL + i < NC) {
                            if (SHARD) {
                                for (int r = 0; r < a.R; ++r) cv[i] += __ldcg(src + r * sstr + i);     // the ranks' coarse bins
                            } else {
                                cv[i] = __ldcg(src + i);
                            }
                        }
                        csum += cv[i];
                    }
                }
#pragma unroll
                for (int i = 0; i < LEAN_MAX_WIN / 32; ++i) {
                    const int wj = lane + 32 * i;
                    if (wj < nwin) wv[i] = ldcg_u16(a.wsc + ((size_t)b * KH + h) * LEAN_MAX_WIN + wj);
                }
                const unsigned suf = suffix_sum(csum, lane);
                const unsigned ball = __ballot_sync(0xffffffffu, suf >= (unsigned)kk);   // not empty: the row holds N >= kk keys
                const int Ll = 31 - __clz(ball | 1u);
                int Lc_l = 0, A_l = 0;
                {
                    unsigned above = suf - csum;
#pragma unroll
                    for (int i = LEAN_CPL_MAX - 1; i >= 0; --i) {
                        if (above < (unsigned)kk && above + cv[i] >= (unsigned)kk) { Lc_l = lane * CPL + i; A_l = (int)above; }
                        above += cv[i];
                    }
                }
                const int Lc = __shfl_sync(0xffffffffu, Lc_l, Ll), Lb = Lc << LEAN_CWS;
                // all ranks' counts at the 8 scores of that bin: lane l holds rank l / 8 (and 4 + l / 8), score l % 8
                unsigned g0 = 0, g1 = 0;
                if (SHARD) {
                    const unsigned* fsrc = own_slots + (size_t)a.B * npairs + ((size_t)(b * KH + h) * NC + Lc) * 8 + (lane & 7);
                    if ((lane >> 3) < a.R) g0 = __ldcg(fsrc + (lane >> 3) * sstr);
                    if (4 + (lane >> 3) < a.R) g1 = __ldcg(fsrc + (4 + (lane >> 3)) * sstr);
                }
                SL_STAMP(8)
                // every chunk's record of coarse bin Lc and its count above the bin, chunk = lane + 32 j.
                // Sums of one lane stay below 2^16 per 16-bit field (chunk * LEAN_CPL_MAX < 65536): pairs are added packed.
                unsigned pk[4] = {0u, 0u, 0u, 0u}, pa = 0u;      // all of the lane's chunks
                unsigned qk[4] = {0u, 0u, 0u, 0u}, qa = 0u;      // those before this chunk
                {
                    const size_t e0 = ((size_t)(b * KH + h) * NC + Lc) * cpb;
                    uint4 x[LEAN_CPL_MAX];
                    unsigned y[LEAN_CPL_MAX];
#pragma unroll
                    for (int j = 0; j < LEAN_CPL_MAX; ++j) {
                        const int cc = lane + 32 * j;
                        x[j] = make_uint4(0u, 0u, 0u, 0u);
                        y[j] = 0u;
                        if (cc < cpb) { x[j] = __ldcg(a.pub + e0 + cc); y[j] = __ldcg(a.puba + e0 + cc); }
                    }
#pragma unroll
                    for (int j = 0; j < LEAN_CPL_MAX; ++j) {
                        pk[0] += x[j].x; pk[1] += x[j].y; pk[2] += x[j].z; pk[3] += x[j].w; pa += y[j];
                        if (lane + 32 * j < c) { qk[0] += x[j].x; qk[1] += x[j].y; qk[2] += x[j].z; qk[3] += x[j].w; qa += y[j]; }
                    }
                }
                SL_STAMP(9)
                int tot[9];                                   // the row's keys with score >= Lb + i, in every lane
                tot[8] = __reduce_add_sync(0xffffffffu, (int)pa);
#pragma unroll
                for (int i = 3; i >= 0; --i) {
                    tot[2 * i + 1] = tot[2 * i + 2] + __reduce_add_sync(0xffffffffu, (int)(pk[i] >> 16));
                    tot[2 * i] = tot[2 * i + 1] + __reduce_add_sync(0xffffffffu, (int)(pk[i] & 0xffffu));
                }
                SL_STAMP(10)
                int ls = 0, r = 0;                            // (all ranks') tot[0] >= kk > tot[8] by the choice of Lc
                if (SHARD) {
                    unsigned t = g0 + g1;
                    t += __shfl_xor_sync(0xffffffffu, t, 8);
                    t += __shfl_xor_sync(0xffffffffu, t, 16);         // lane l: all ranks' keys with score Lb + l % 8
                    int run = __shfl_sync(0xffffffffu, A_l, Ll), gt_all = 0;    // keys of all ranks above the bin
#pragma unroll
                    for (int i = 7; i >= 0; --i) {
                        const int above_i = run;
                        run += (int)__shfl_sync(0xffffffffu, t, i);
                        if (i >= 1 && run >= kk) ++ls;
                        if (run >= kk && above_i < kk) gt_all = above_i;       // i is the threshold's place in the bin
                    }
                    // threshold ties on lower ranks come first in key order
                    const int lower = ((lane & 7) == ls) ? (int)(((lane >> 3) < a.rank ? g0 : 0u) + ((4 + (lane >> 3)) < a.rank ? g1 : 0u)) : 0;
                    r = max(kk - gt_all - __reduce_add_sync(0xffffffffu, lower), 0);
                } else {
#pragma unroll
                    for (int i = 1; i < 8; ++i) ls += tot[i] >= kk ? 1 : 0;
                }
                tau = Lb + ls;
                int ge_tot = 0, gt_tot = 0;                   // this rank's keys at or above / above the threshold
#pragma unroll
                for (int i = 0; i < 8; ++i) {
                    ge_tot = i == ls ? tot[i] : ge_tot;
                    gt_tot = i == ls ? tot[i + 1] : gt_tot;
                }
                if (!SHARD) r = kk - gt_tot;
                // keys above / at the threshold in the chunks before this one, from the lane's packed sums
                {
                    int gt = (int)qa, eq = 0;
#pragma unroll
                    for (int i = 0; i < 8; ++i) {
                        const int v = (int)((i & 1) ? (qk[i >> 1] >> 16) : (qk[i >> 1] & 0xffffu));
                        gt += i > ls ? v : 0;
                        eq += i == ls ? v : 0;
                    }
                    pre_gt = __reduce_add_sync(0xffffffffu, gt);
                    pre_eq = __reduce_add_sync(0xffffffffu, eq);
                }
                // always-kept keys: threshold ties inside the sink come off the quota; all of them leave the totals
                int eq_sink = 0, gt_win = 0, eq_win = 0;
#pragma unroll
                for (int i = 0; i < LEAN_MAX_WIN / 32; ++i) {
                    const int wj = lane + 32 * i;
                    const bool in = wj < nwin;
                    const int v = (int)wv[i];
                    gt_win += __popc(__ballot_sync(0xffffffffu, in && v > tau));
                    eq_win += __popc(__ballot_sync(0xffffffffu, in && v == tau));
                    eq_sink += __popc(__ballot_sync(0xffffffffu, in && wj < s_end && v == tau));
                }
                rM = max(r - eq_sink, 0);
                selM = (gt_tot - gt_win) + min((ge_tot - gt_tot) - eq_win, rM);
            }
#pragma unroll
            for (int i = 0; i < LEAN_MAX_WIN / 32; ++i) s_win[h * LEAN_MAX_WIN + lane + 32 * i] = (unsigned short)wv[i];
            if (lane == 0) {
                s_tau[h] = tau;
                s_pre[h * 4 + 0] = pre_gt; s_pre[h * 4 + 1] = pre_eq; s_pre[h * 4 + 2] = rM; s_pre[h * 4 + 3] = selM;
                if (c == 0) a.cnt[b * KH + h] = s_end + selM + (N - r_start);
            }
        }
    }
    __syncthreads();
    SL_STAMP(5)

    // ------------------------------------------------------------------ E: flags, ranks, writes
    // A task is (head, sub-range). A lane walks RUN consecutive keys per trip (five 8-byte loads; the
    // odd number of 8-byte units between lanes keeps them free of bank conflicts) and keeps one flag
    // bit per key: adding (0x7fff - tau) to a 16-bit score sets bit 15 iff score > tau, adding
    // (0x8000 - tau) iff score >= tau, two scores per 32-bit add.
    {
        const int ntasks = KH * S;
        const int mlo = max(t0, s_end) - t0, mhi = min(t1, r_start) - t0;     // the chunk's keys outside both windows
        constexpr int RUN = 20;
#pragma unroll 1
        for (int task = warp; task < ntasks; task += NW) {
            const int h = task & (KH - 1), s = task >> khs;
            const int lo = min(len, s * sub), hi = min(len, (s + 1) * sub);
            const int elo = max(lo, mlo), ehi = min(hi, mhi);
            const int tau = s_tau[h];
            const int rM = s_pre[h * 4 + 2], selM = s_pre[h * 4 + 3];
            // selected keys / ties before this sub-range: earlier chunks, earlier sub-ranges of this chunk,
            // less the always-kept keys among them (they are written at their own positions)
            int gt_before = s_pre[h * 4 + 0], eq_before = s_pre[h * 4 + 1];
            {
                // earlier sub-ranges of this chunk: their keys above the threshold (summed from the counts) and at it
                const int v0 = (min(tau, nbins) + 4) & ~3;              // first 4-aligned score above the threshold ...
                for (int s2 = 0; s2 < s; ++s2) {
                    const unsigned* R = shist + (s2 * KH + h) * nb1;
                    unsigned part = 0;
                    for (int v = v0 + 4 * lane; v < nb1; v += 128) {
                        const uint4 x = *reinterpret_cast<const uint4*>(R + v);
                        part += (x.x + x.y) + (x.z + x.w);
                    }
                    if (lane == 0)                                       // ... and the up to three scores between
                        for (int v = min(tau, nbins) + 1; v < min(v0, nb1); ++v) part += R[v];
                    gt_before += (int)__reduce_add_sync(0xffffffffu, part);
                    eq_before += (int)R[min(tau, nbins)];
                }
                const int e0 = t0 + lo;
#pragma unroll
                for (int i = 0; i < LEAN_MAX_WIN / 32; ++i) {
                    const int wj = lane + 32 * i;
                    const int t = wj < s_end ? wj : r_start + (wj - s_end);
                    const bool in = wj < nwin && t < e0;
                    const int v = (int)s_win[h * LEAN_MAX_WIN + wj];
                    gt_before -= __popc(__ballot_sync(0xffffffffu, in && v > tau));
                    eq_before -= __popc(__ballot_sync(0xffffffffu, in && v == tau));
                }
            }
            int out_base = s_end + gt_before + min(eq_before, rM);
            int* oi = a.idx + ((size_t)b * KH + h) * a.cap;
            const unsigned short* row = sscores + h * rowh;
            const unsigned cgt = (unsigned)(0x7fff - tau) * 0x10001u, cge = (unsigned)(0x8000 - tau) * 0x10001u;
#pragma unroll 1
            for (int g0 = elo & ~3; g0 < ehi; g0 += 32 * RUN) {
                const int r0 = g0 + lane * RUN;
                unsigned Gf = 0, Ef = 0;                               // bit i: key r0 + i is > tau / == tau
#pragma unroll
                for (int j = 0; j < RUN / 4; ++j) {
                    const int tl = r0 + 4 * j;
                    uint2 x = make_uint2(0u, 0u);
                    if (tl < ehi) x = *reinterpret_cast<const uint2*>(row + tl);
                    Gf |= flags4(x.x + cgt, x.y + cgt) << (4 * j);
                    Ef |= flags4(x.x + cge, x.y + cge) << (4 * j);
                }
                {   // keys of the run inside [elo, ehi)
                    const int lc = min(max(elo - r0, 0), RUN), hc = min(max(ehi - r0, 0), RUN);
                    const unsigned vm = ((1u << hc) - 1u) & ~((1u << lc) - 1u);
                    Gf &= vm;
                    Ef &= vm & ~Gf;
                }
                const unsigned packed = (unsigned)__popc(Gf) | ((unsigned)__popc(Ef) << 16);
                const unsigned inc = (unsigned)prefix_sum((int)packed, lane);
                const unsigned tot = __shfl_sync(0xffffffffu, inc, 31);
                const unsigned exc = inc - packed;
                const int tot_e = (int)(tot >> 16);
                unsigned sel = Gf;
                int below = (int)(exc & 0xffffu), tot_sel = (int)(tot & 0xffffu);
                if (eq_before + tot_e <= rM) {                          // every tie of this trip is inside the quota
                    sel |= Ef;
                    below += (int)(exc >> 16);
                    tot_sel += tot_e;
                } else if (eq_before < rM) {                            // the quota runs out inside this trip
                    int rank = eq_before + (int)(exc >> 16);
                    unsigned e = Ef, tk = 0;
                    while (e && rank < rM) { const unsigned bit = e & (0u - e); tk |= bit; e ^= bit; ++rank; }
                    sel |= tk;
                    const int nt = __popc(tk), inc2 = prefix_sum(nt, lane);
                    below += inc2 - nt;
                    tot_sel += __shfl_sync(0xffffffffu, inc2, 31);
                }
                int pos = out_base + below;
                const int kbase = t0 + r0;
                while (sel) {
                    const int i = __ffs((int)sel) - 1;
                    sel &= sel - 1u;
                    if (pos < a.cap) oi[pos] = kbase + i;
                    ++pos;
                }
                out_base += tot_sel;
                eq_before += tot_e;
            }
            // always-kept keys of this sub-range: the sink at its own index, the recent window at the end
            for (int t = t0 + lo + lane; t < min(t0 + hi, s_end); t += 32)
                if (t < a.cap) oi[t] = t;
            for (int t = max(t0 + lo, r_start) + lane; t < t0 + hi; t += 32) {
                const int pos = s_end + selM + (t - r_start);
                if (pos < a.cap) oi[pos] = t;
            }
        }
    }
    SL_STAMP(6)

    // ------------------------------------------------------------------ the last CTA of the row advances the launch counter
    __syncthreads();
    if (tid == 0) {
        unsigned* sync = a.sync + 2 * b;
        __threadfence();
        const unsigned old = atomicAdd(&sync[1], 1u);
        if (old == (unsigned)cpb - 1u) {
            sync[0] = 0;
            sync[1] = 0;
            if (SHARD) {     // the row's last CTA: every CTA of the row has read the buffer's epoch word by now
                unsigned* epoch_w = reinterpret_cast<unsigned*>(a.peer[a.rank] + a.pflags_off) + SHARD_EPOCH_WORD - b;
                *epoch_w = __ldcg(epoch_w) + 1u;
            }
            a.epoch[b] = __ldcg(a.epoch + b) + 1u;           // the next launch takes the other coarse buffer
            __threadfence();
        }
    }
}

typedef void (*lean_kernel_t)(const LeanArgs);

template <bool SHARD>
lean_kernel_t pick(int P) {
    switch (P) {
        case 1: return scan_lean_kernel<1, SHARD>;
        case 2: return scan_lean_kernel<2, SHARD>;
        case 3: return scan_lean_kernel<3, SHARD>;
        default: return scan_lean_kernel<4, SHARD>;
    }
}

inline size_t up16(size_t v) { return (v + 15) / 16 * 16; }

}  // namespace

namespace slscan {

int lean_nc(int nbins) { return ((nbins - 1) >> LEAN_CWS) + 1; }

// What the one-barrier kernel covers beyond fused_covers(): at most LEAN_MAX_WIN always-kept keys,
// 16-bit sums per lane over its chunks, one trip for the chunks' records, at most LEAN_CPL_MAX coarse bins per lane.
bool lean_covers(int KH, int G, int ctas_per_b, int chunk, int nwin) {
    return fused_covers(KH, G) && ctas_per_b > 1 && ctas_per_b <= 32 * LEAN_CPL_MAX && chunk * LEAN_CPL_MAX < 65536 &&
           nwin <= LEAN_MAX_WIN && lean_nc(128 * G + 1) <= 32 * LEAN_CPL_MAX;
}

size_t lean_plan_smem(LeanArgs& f, int KH, int nbins, int S, int chunk) {
    size_t off = (size_t)KH * 32 * 4 + (size_t)KH * 4 * 4 + (size_t)KH * 4 + (size_t)KH * 4 * 4 +
                 (size_t)KH * LEAN_MAX_WIN * 2 + (size_t)KH * lean_nc(nbins) * 4;
    off = up16(off);
    f.hist_off = (int)off;
    off = up16(off + (size_t)S * KH * ((nbins + 4) & ~3) * 4);
    f.score_off = (int)off;
    off = up16(off + (size_t)(chunk + 64) * KH * 2);
    return off;
}

size_t lean_shard_message_bytes(int B, int KH, int nbins) {
    return ((size_t)B * KH * lean_nc(nbins) * 9 * 4 + 15) / 16 * 16;      // coarse [B][KH][NC] + fine [B][KH][NC][8], 32 bits each
}

int launch_lean(const LeanArgs& a_in, size_t smem, cudaStream_t s) {
    LeanArgs a = a_in;
    a.dbg = SL_STAMP_BUF;
    lean_kernel_t kern = a.R > 0 ? pick<true>(sliced_planes(a.G)) : pick<false>(sliced_planes(a.G));
    SL_CUDA_OK(sl::ensure_dyn_smem(reinterpret_cast<const void*>(kern), smem));
    SL_CUDA_OK(sl::launch_kernel(kern, dim3((unsigned)(a.B * a.ctas_per_b)), dim3(NT), smem, s, true, a));
    return SL_OK;
}

}  // namespace slscan
