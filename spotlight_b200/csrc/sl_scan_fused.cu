// The decode step's fused Hamming scan + exact top-k + sink/recent window: the lean kernel for
// the common case (several CTAs per batch row, scores of a chunk fit in shared memory, kv heads
// divide the warp, bit-sliced scorer covers the group size). Everything else goes through the
// general kernel in sl_scan_topk.cu; both produce identical results.
//
// One cooperative launch, one CTA of 512 threads per SM, each owning a contiguous chunk of keys:
//   A  stream the chunk's 128-bit codes (8 x 16-byte loads in flight per thread), score them with
//      the bit-sliced scorer, keep the 16-bit scores in shared memory ([head][key], bank-spread),
//      histogram per head in shared memory, then add the non-empty bins to a global fine
//      histogram and to a coarse one (<= 32 bins per head)
//   -- the only grid barrier (bounded) --
//   B  threshold per head: one warp reads the coarse bins (one per lane), then the fine bins of
//      the coarse bin that holds the threshold; flag, count and rank the own {> tau, == tau} keys
//      (kept in shared memory); publish the counts as one flagged 64-bit word per (head, chunk);
//      poll all chunks' words (bounded)
//   C  write the attended keys at their final positions: ascending, ties to the lowest index.
// The kernel is written for a small instruction footprint: its phases run once per launch, and
// code that is not in the instruction cache runs at a third of the resident rate.
#include "sl_scan.cuh"
#include "sl_sliced.cuh"

namespace {

using namespace slscan;

// SHARD: this rank holds a contiguous part of a longer context. After the grid barrier one CTA per
// batch row merges the copies of the row's local histograms and stores them into slot `rank` of
// every rank's exchange buffer (plain peer stores over NVLink), fences at system scope and writes
// this launch's epoch into the row's flag `rank` of every buffer; then the row's CTAs wait
// (bounded) until the R flags of the row in the own buffer carry the epoch. The threshold is then
// searched over the R slots, and the ties that belong to lower ranks (lower key indices) are taken
// off this rank's tie quota.
template <int PT, bool SHARD>
__global__ void __launch_bounds__(NT, 1) scan_fused_kernel(const FusedArgs a) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    const int KH = a.KH, nbins = a.nbins, N = a.N, cpb = a.ctas_per_b;
    uint32_t* s_planes = reinterpret_cast<uint32_t*>(smem_raw);                 // [KH][2][PT][4]
    int* s_pbase = reinterpret_cast<int*>(s_planes + KH * 32);                    // [KH][4]
    int* s_tau = s_pbase + KH * 4;                                                // [KH]
    int* s_r = s_tau + KH;                                                        // [KH]
    int* s_cnt = s_r + KH;                                                        // [KH*S][2] {> tau, == tau} per task
    int* s_pre = s_cnt + KH * a.S * 2;                                            // [KH][4] {gt before, eq before, rM, selM}
    unsigned* shist = reinterpret_cast<unsigned*>(s_pre + KH * 4);                // [KH][nbins]
    unsigned short* sscores = reinterpret_cast<unsigned short*>(smem_raw + a.score_off);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int b = blockIdx.x / cpb, c = blockIdx.x - b * cpb;
    const int t0 = min(N, c * a.chunk), t1 = min(N, t0 + a.chunk);
    const int len = t1 - t0, ncodes = len * KH;
    const int rowh = a.rowh;                                                      // row stride of sscores (halfwords)
    unsigned* hist_b = a.hist + b * KH * nbins;
    const int hslice = a.B * KH * nbins;
    const int NC = ((nbins - 1) >> a.cws) + 1, cslice = a.B * KH * NC;
    unsigned* chist_b = a.chist + b * KH * NC;
    unsigned long long* seg_b = a.seg + (size_t)b * KH * cpb;
    sl::pdl_trigger();
    sl::pdl_wait();
    SL_STAMP(0)

    // ------------------------------------------------------------------ A: scan + histogram
    {
        const uint4* base = a.k + (size_t)b * a.k_bstride + (size_t)t0 * KH;
        const uint32_t* qb = reinterpret_cast<const uint32_t*>(a.q + (size_t)b * KH * a.G);
        const PlaneWords pw = planes_issue(qb, KH, a.G, a.layout, warp, NW, lane);   // ahead of the stream's loads
        uint4 cd[U];
        int tile = warp;
#pragma unroll
        for (int u = 0; u < U; ++u) {
            const int i = tile * (32 * U) + u * 32 + lane;
            if (i < ncodes) cd[u] = sl::ld_stream_v4(base + i);
        }
        if (tid == NT - 32) {            // pages the later phases store to / poll
            touch(a.idx + (size_t)b * KH * a.cap);
            touch(a.cnt + b * KH);
            touch(seg_b);
        }
        for (int i = tid; i < KH * nbins; i += NT) shist[i] = 0;
        planes_finish<PT>(pw, KH, a.G, s_planes, s_pbase, warp, NW, lane);
        stage_planes<PT>(qb, KH, a.G, a.layout, s_planes, s_pbase, warp, NW, lane, 1);   // KH > 8
        __syncthreads();
        uint32_t M[PT][4], Mp[PT][4];
        const int hh = lane & (KH - 1);                       // this lane's head (KH is a power of two <= 32)
        const int sbase = load_planes<PT>(s_planes, s_pbase, hh, M, Mp);
        SL_STAMP(11)
        const int ssh = sliced_shift(a.G), khs = 31 - __clz(KH);
        unsigned short* srow = sscores + hh * rowh;
        unsigned* hrow = shist + hh * nbins;
        short* so = a.scores_out ? a.scores_out + ((size_t)b * N + t0) * KH : nullptr;
#pragma unroll 1
        while (tile * (32 * U) < ncodes) {
            const int i0 = tile * (32 * U) + lane;
            int sv[U];
#pragma unroll
            for (int u = 0; u < U; ++u) sv[u] = sbase + (sliced_score<PT>(cd[u], M, Mp) << ssh);
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
                    srow[i >> khs] = (unsigned short)sv[u];
                    atomicAdd(hrow + sv[u], 1u);
                    if (so) so[i] = (short)sv[u];
                }
            }
        }
        __syncthreads();
    }
    SL_STAMP(7)
    {
        // one global add per non-empty fine bin and per non-empty coarse bin; CTAs spread over the
        // histogram copies and start at different bins so that simultaneous adds rarely meet
        const int cp = c & (NCOPY - 1);
        unsigned* dstf = hist_b + cp * hslice;
        const int total = KH * nbins;
        const int start = (c * 977) % total;
#pragma unroll 4
        for (int j = tid; j < total; j += NT) {
            int i = j + start;
            if (i >= total) i -= total;
            const unsigned v = shist[i];
            if (v) atomicAdd(dstf + i, v);
        }
        const int CWm = (1 << a.cws) - 1;
#pragma unroll 1
        for (int t = tid; t < KH * NC; t += NT) {            // coarse bins: one thread each, skewed reads
            const int h = t / NC, cb = t - h * NC;
            const unsigned* F = shist + h * nbins + (cb << a.cws);
            const int nf = min(CWm + 1, nbins - (cb << a.cws));
            unsigned cs = 0;
#pragma unroll 8
            for (int k2 = 0; k2 <= CWm; ++k2) {
                const int f = (k2 + t) & CWm;
                if (f < nf) cs += F[f];
            }
            if (cs) atomicAdd(chist_b + cp * cslice + t, cs);
        }
        // last launch's flagged word of this chunk: cleared before the barrier, polled after it
        if (tid < KH) st_relaxed_u64(seg_b + tid * cpb + c, 0ull);
    }
    SL_STAMP(1)
    sl::grid_barrier(a.sync + 2 * b, (unsigned)cpb, a.status);
    SL_STAMP(2)
    const int W = KH * nbins + KH * NC;                          // words of one batch row's message
    if (SHARD) {
        // own buffer: [R slots][flags [R][B]] ... [epoch of row b at word SHARD_EPOCH_WORD - b of the flag area]
        unsigned* own_words = reinterpret_cast<unsigned*>(a.peer[a.rank] + a.pflags_off);
        const unsigned target = __ldcg(own_words + SHARD_EPOCH_WORD - b) + 1u;    // this launch's epoch of the row
        if (c == 0) {
            // One CTA per batch row carries the row's message (a few thousand words) to every rank and
            // then publishes the epoch in the row's flag on every rank. A system-scope fence costs
            // about 2.5 us on this machine, so exactly one is executed on the sending side.
            for (int i0 = tid; i0 < W; i0 += NT * 4) {
                unsigned v[4] = {0u, 0u, 0u, 0u};
#pragma unroll
                for (int j = 0; j < 4; ++j) {                // all loads of four rounds in flight together
                    const int i = i0 + j * NT;
                    if (i < KH * nbins) {
#pragma unroll
                        for (int cp = 0; cp < NCOPY; ++cp) v[j] += __ldcg(hist_b + cp * hslice + i);
                    } else if (i < W) {
#pragma unroll
                        for (int cp = 0; cp < NCOPY; ++cp) v[j] += __ldcg(chist_b + cp * cslice + (i - KH * nbins));
                    }
                }
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int i = i0 + j * NT;
                    if (i < W)
                        for (int r = 0; r < a.R; ++r)
                            reinterpret_cast<unsigned*>(a.peer[r] + (unsigned long long)a.rank * a.slot_stride)[b * W + i] = v[j];
                }
            }
            __syncthreads();
            if (tid == 0) {
                __threadfence_system();      // the CTA's peer stores (ordered before this by the barrier) first
                for (int r = 0; r < a.R; ++r) {
                    unsigned* pf = reinterpret_cast<unsigned*>(a.peer[r] + a.pflags_off) + a.rank * a.B + b;
                    asm volatile("st.relaxed.sys.global.u32 [%0], %1;" ::"l"(pf), "r"(target) : "memory");
                }
            }
        }
        if (tid < a.R) {
            const unsigned* lf = own_words + tid * a.B + b;
            unsigned v = 0, it = 0;
            for (;;) {
                asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(lf) : "memory");
                if ((int)(v - target) >= 0) break;
                if (++it > 400000u) {    // about a second: give up, tell the host, finish with what is there
                    if (a.status) atomicExch(a.status, 3);
                    break;
                }
                __nanosleep(64);
            }
        }
        __syncthreads();
    }
    // the histograms the threshold is searched in: the copies of the workspace, or the ranks' slots
    const int nsl = SHARD ? a.R : NCOPY;
    const unsigned* Fb = SHARD ? reinterpret_cast<const unsigned*>(a.peer[a.rank]) + b * W : hist_b;
    const unsigned* Cb = SHARD ? Fb + KH * nbins : chist_b;
    const long long fstr = SHARD ? (long long)(a.slot_stride >> 2) : (long long)hslice;
    const long long cstr = SHARD ? (long long)(a.slot_stride >> 2) : (long long)cslice;

    // ------------------------------------------------------------------ B: threshold per head
    {
        const int kk = SHARD ? a.kk : min(a.k_budget, N);
        const int FPL = 1 << (a.cws - 5);                    // fine bins per lane in the second step
#pragma unroll 1
        for (int h = warp; h < KH; h += NW) {
            int tau = nbins, r = 0;
            if (kk > 0) {
                unsigned cv = 0;
                if (lane < NC) {
#pragma unroll 4
                    for (int sl_ = 0; sl_ < nsl; ++sl_) cv += __ldcg(Cb + sl_ * cstr + h * NC + lane);
                }
                const unsigned suf = suffix_sum(cv, lane);
                const unsigned ball = __ballot_sync(0xffffffffu, suf >= (unsigned)kk);
                if (ball == 0) {        // fewer than kk keys in total: everything is selected
                    tau = -1;
                } else {
                    const int L = 31 - __clz(ball);
                    const unsigned above = __shfl_sync(0xffffffffu, suf - cv, L);    // keys in coarse bins above L
                    const unsigned* F = Fb + h * nbins;
                    const int f0 = (L << a.cws) + lane * FPL;
                    unsigned fv0 = 0, fv1 = 0, fs = 0;
                    if (FPL <= 2) {
#pragma unroll 4
                        for (int sl_ = 0; sl_ < nsl; ++sl_) {
                            if (f0 < nbins) fv0 += __ldcg(F + sl_ * fstr + f0);
                            if (FPL == 2 && f0 + 1 < nbins) fv1 += __ldcg(F + sl_ * fstr + f0 + 1);
                        }
                        fs = fv0 + fv1;
                    } else {
#pragma unroll 1
                        for (int t = 0; t < FPL; ++t)
                            for (int sl_ = 0; sl_ < nsl; ++sl_)
                                if (f0 + t < nbins) fs += __ldcg(F + sl_ * fstr + f0 + t);
                    }
                    const unsigned fsuf = suffix_sum(fs, lane);
                    const unsigned ball2 = __ballot_sync(0xffffffffu, above + fsuf >= (unsigned)kk);
                    const int L2 = 31 - __clz(ball2 | 1u);
                    int tau_l = 0, gt_l = 0;
                    if (lane == L2) {
                        unsigned cum = above + fsuf - fs;
#pragma unroll 1
                        for (int t = FPL - 1; t >= 0; --t) {
                            unsigned v = 0;
                            if (FPL <= 2) {
                                v = t ? fv1 : fv0;
                            } else if (f0 + t < nbins) {
#pragma unroll 1
                                for (int sl_ = 0; sl_ < nsl; ++sl_) v += __ldcg(F + sl_ * fstr + f0 + t);
                            }
                            if (cum + v >= (unsigned)kk) { tau_l = f0 + t; gt_l = (int)cum; break; }
                            cum += v;
                        }
                    }
                    tau = __shfl_sync(0xffffffffu, tau_l, L2);
                    r = kk - __shfl_sync(0xffffffffu, gt_l, L2);
                    if (SHARD) {        // threshold ties on lower ranks come first in key order
                        int e_lower = lane < a.rank ? (int)__ldcg(F + lane * fstr + tau) : 0;
                        e_lower = __reduce_add_sync(0xffffffffu, e_lower);
                        r = max(r - e_lower, 0);
                    }
                }
            }
            if (lane == 0) { s_tau[h] = tau; s_r[h] = r; }
        }
    }
    __syncthreads();
    SL_STAMP(3)

    // ------------------------------------------------------------------ B/C: count, publish, poll, emit
    // A task is (head, sub-range of the chunk). A lane walks RUN consecutive keys per trip (five
    // 8-byte loads; the odd number of 8-byte units between lanes keeps them free of bank conflicts)
    // and keeps one flag bit per key: adding (0x7fff - tau) to a 16-bit score sets bit 15 iff
    // score > tau, adding (0x8000 - tau) iff score >= tau, two scores per 32-bit add.
    // Everything that does not depend on the other chunks happens BEFORE their counts are polled:
    // flags, per-lane counts and one packed warp scan per trip are kept in shared memory, so that
    // after the poll only the tie decision and the writes remain.
    const int S = a.S, ntasks = KH * S;
    const int sub = ((len + S - 1) / S + 127) & ~127;
    const int mlo = max(t0, a.s_end) - t0, mhi = min(t1, a.r_start) - t0;     // the chunk's keys outside both windows
    constexpr int RUN = 20;
    uint4* s_trip = reinterpret_cast<uint4*>(smem_raw + a.trip_off) + warp * (a.trips_per_warp * 32) + lane;
    {
        int slot = 0;
#pragma unroll 1
        for (int task = warp; task < ntasks; task += NW) {
            const int h = task & (KH - 1), s = task >> (31 - __clz(KH));
            const int elo = max(min(len, s * sub), mlo), ehi = min(min(len, (s + 1) * sub), mhi);
            const int tau = s_tau[h];
            const unsigned short* row = sscores + h * rowh;
            const unsigned cgt = (unsigned)(0x7fff - tau) * 0x10001u, cge = (unsigned)(0x8000 - tau) * 0x10001u;
            unsigned task_tot = 0;                                     // > tau | == tau << 16 of the task
#pragma unroll 1
            for (int g0 = elo & ~3; g0 < ehi; g0 += 32 * RUN, ++slot) {
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
                s_trip[slot * 32] = make_uint4(Gf, Ef, inc - packed, tot);
                task_tot += tot;                                       // at most chunk < 65536 keys per field
            }
            if (lane == 0) { s_cnt[task * 2] = (int)(task_tot & 0xffffu); s_cnt[task * 2 + 1] = (int)(task_tot >> 16); }
        }
    }
    {
        __syncthreads();
        SL_STAMP(10)
        if (tid < KH) {
            // flag | > tau | == tau | == tau inside the sink, 21 bits each: one atomic 64-bit store
            unsigned long long gt = 0, eq = 0, eqs = 0;
#pragma unroll 1
            for (int s = 0; s < S; ++s) { gt += s_cnt[(s * KH + tid) * 2]; eq += s_cnt[(s * KH + tid) * 2 + 1]; }
            if (t0 < a.s_end) {
                const int tau = s_tau[tid];
#pragma unroll 1
                for (int t = t0; t < min(t1, a.s_end); ++t) eqs += (int)sscores[tid * rowh + (t - t0)] == tau;
            }
            st_relaxed_u64(seg_b + tid * cpb + c, (1ull << 63) | (gt << 42) | (eq << 21) | eqs);
        }
        __syncthreads();                 // nobody spins on memory while this CTA still has to publish
#pragma unroll 1
        for (int h = warp; h < KH; h += NW) {
            // Every chunk's word is polled until its flag shows (bounded): no second grid barrier, and
            // a CTA that gets past this knows that all CTAs have finished with the histograms.
            int pre_gt = 0, pre_eq = 0, tot_gt = 0, tot_eq = 0, tot_eqS = 0;
            const unsigned long long* sp = seg_b + h * cpb;
            bool ok = true;
#pragma unroll 1
            for (int cc0 = 0; cc0 < cpb; cc0 += 32 * 5) {
                unsigned long long w[5];
                unsigned it = 0;
                for (;;) {                               // all loads of a round in flight together
                    bool all = true;
#pragma unroll
                    for (int j = 0; j < 5; ++j) {
                        const int cc = cc0 + j * 32 + lane;
                        w[j] = cc < cpb ? ld_relaxed_u64(sp + cc) : (1ull << 63);
                    }
#pragma unroll
                    for (int j = 0; j < 5; ++j) all = all && (w[j] >> 63);
                    if (__all_sync(0xffffffffu, all)) break;
                    if (++it > 1000000u) { ok = false; break; }
                    __nanosleep(32);
                }
#pragma unroll
                for (int j = 0; j < 5; ++j) {
                    const int cc = cc0 + j * 32 + lane;
                    const int gt = (int)((w[j] >> 42) & 0x1fffffu), eq = (int)((w[j] >> 21) & 0x1fffffu);
                    tot_gt += gt; tot_eq += eq; tot_eqS += (int)(w[j] & 0x1fffffu);
                    if (cc < c) { pre_gt += gt; pre_eq += eq; }
                }
            }
            if (!ok && a.status) atomicExch(a.status, 1);
            pre_gt = __reduce_add_sync(0xffffffffu, pre_gt); pre_eq = __reduce_add_sync(0xffffffffu, pre_eq);
            tot_gt = __reduce_add_sync(0xffffffffu, tot_gt); tot_eq = __reduce_add_sync(0xffffffffu, tot_eq);
            tot_eqS = __reduce_add_sync(0xffffffffu, tot_eqS);
            const int rM = max(s_r[h] - tot_eqS, 0);
            const int selM = tot_gt + min(tot_eq, rM);
            if (lane == 0) {
                s_pre[h * 4 + 0] = pre_gt; s_pre[h * 4 + 1] = pre_eq; s_pre[h * 4 + 2] = rM; s_pre[h * 4 + 3] = selM;
                if (c == 0) a.cnt[b * KH + h] = a.s_end + selM + (N - a.r_start);
            }
        }
        __syncthreads();
        SL_STAMP(5)
    }
    {
        int slot = 0;
#pragma unroll 1
        for (int task = warp; task < ntasks; task += NW) {
            const int h = task & (KH - 1), s = task >> (31 - __clz(KH));
            const int lo = min(len, s * sub), hi = min(len, (s + 1) * sub);
            const int elo = max(lo, mlo), ehi = min(hi, mhi);
            const int rM = s_pre[h * 4 + 2], selM = s_pre[h * 4 + 3];
            int gt_before = s_pre[h * 4 + 0], eq_before = s_pre[h * 4 + 1];
#pragma unroll 1
            for (int s2 = 0; s2 < s; ++s2) { gt_before += s_cnt[(s2 * KH + h) * 2]; eq_before += s_cnt[(s2 * KH + h) * 2 + 1]; }
            int out_base = a.s_end + gt_before + min(eq_before, rM);
            int* oi = a.idx + ((size_t)b * KH + h) * a.cap;
#pragma unroll 1
            for (int g0 = elo & ~3; g0 < ehi; g0 += 32 * RUN, ++slot) {
                const uint4 st = s_trip[slot * 32];                    // {> tau flags, == tau flags, counts below, totals}
                const unsigned Ef = st.y, exc = st.z, tot = st.w;
                const int tot_e = (int)(tot >> 16);
                unsigned sel = st.x;
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
                const int kbase = t0 + g0 + lane * RUN;
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
            for (int t = t0 + lo + lane; t < min(t0 + hi, a.s_end); t += 32)
                if (t < a.cap) oi[t] = t;
            for (int t = max(t0 + lo, a.r_start) + lane; t < t0 + hi; t += 32) {
                const int pos = a.s_end + selM + (t - a.r_start);
                if (pos < a.cap) oi[pos] = t;
            }
        }
    }

    SL_STAMP(6)
    // ------------------------------------------------------------------ leave the workspace zeroed
    {
        const int total = KH * nbins, ctot = KH * NC;
#pragma unroll 1
        for (int i = c * NT + tid; i < NCOPY * total; i += cpb * NT) hist_b[(i / total) * hslice + i % total] = 0;
#pragma unroll 1
        for (int i = c * NT + tid; i < NCOPY * ctot; i += cpb * NT) chist_b[(i / ctot) * cslice + i % ctot] = 0;
        __syncthreads();
        if (tid == 0) {
            unsigned* sync = a.sync + 2 * b;
            __threadfence();
            const unsigned old = atomicAdd(&sync[1], 1u);
            if (old == (unsigned)cpb - 1u) {
                if (SHARD) {     // the row's last CTA: every CTA of the row has read the row's epoch word by now
                    unsigned* epoch_w = reinterpret_cast<unsigned*>(a.peer[a.rank] + a.pflags_off) + SHARD_EPOCH_WORD - b;
                    *epoch_w = __ldcg(epoch_w) + 1u;
                }
                sync[0] = 0;
                sync[1] = 0;
                __threadfence();
            }
        }
    }
}

typedef void (*fused_kernel_t)(const FusedArgs);

template <bool SHARD>
fused_kernel_t pick(int P) {
    switch (P) {
        case 1: return scan_fused_kernel<1, SHARD>;
        case 2: return scan_fused_kernel<2, SHARD>;
        case 3: return scan_fused_kernel<3, SHARD>;
        default: return scan_fused_kernel<4, SHARD>;
    }
}

}  // namespace

namespace slscan {

bool fused_covers(int KH, int G) { return KH <= 32 && (KH & (KH - 1)) == 0 && sliced_planes(G) > 0; }

size_t fused_fixed_smem(int KH, int nbins, int S) {
    return (size_t)KH * 32 * 4 + (size_t)KH * 4 * 4 + (size_t)KH * 2 * 4 + (size_t)KH * S * 2 * 4 + (size_t)KH * 4 * 4 +
           (size_t)KH * nbins * 4;
}

size_t fused_plan_smem(FusedArgs& f, int KH, int nbins, int S, int chunk) {
    size_t off = (fused_fixed_smem(KH, nbins, S) + 15) / 16 * 16;
    f.score_off = (int)off;
    off = (off + (size_t)(chunk + 64) * KH * 2 + 15) / 16 * 16;
    const int tasks_per_warp = (KH * S + NW - 1) / NW;
    const int sub = (((chunk + S - 1) / S) + 127) & ~127;              // the longest sub-range a task can get
    const int trips = (sub + 3 + 32 * 20 - 1) / (32 * 20) + 1;         // trips of 640 keys, one spare
    f.trips_per_warp = tasks_per_warp * trips;
    f.trip_off = (int)off;
    off += (size_t)NW * f.trips_per_warp * 32 * 16;
    return off;
}

size_t shard_message_bytes(int B, int KH, int nbins, int cws) {
    const int NC = ((nbins - 1) >> cws) + 1;
    return ((size_t)B * (KH * nbins + KH * NC) * 4 + 15) / 16 * 16;
}

int launch_fused(const FusedArgs& a_in, size_t smem, cudaStream_t s) {
    FusedArgs a = a_in;
    a.dbg = SL_STAMP_BUF;
    fused_kernel_t kern = a.R > 0 ? pick<true>(sliced_planes(a.G)) : pick<false>(sliced_planes(a.G));
    SL_CUDA_OK(sl::ensure_dyn_smem(reinterpret_cast<const void*>(kern), smem));
    SL_CUDA_OK(sl::launch_kernel(kern, dim3((unsigned)(a.B * a.ctas_per_b)), dim3(NT), smem, s, true, a));
    return SL_OK;
}

}  // namespace slscan
