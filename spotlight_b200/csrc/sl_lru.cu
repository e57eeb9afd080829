// LRU-resident KV buffer: stage (3) of the decode path.
//
// Per (batch row, kv head) a slot table of C slots keeps recently attended keys resident in a
// compact buffer [B, C, KH, 128] (slot-major, heads interleaved, i.e. the cache layout with
// "token" = slot, so the attention kernel reads it unchanged). One launch per decode step:
//   hits    attended keys already resident: their slot is stamped with the step number;
//   misses  take the least-recently-attended slots not used in this step (free slots first;
//           ages beyond 1023 steps are treated alike; ties go to the LOWEST slot index), in
//           attended-key order, and their K/V rows are copied from the backing store, which may
//           be device memory or mapped pinned host memory;
//   output  the slot of every attended key, in the order of the index list, so attention over
//           the resident buffer performs the same arithmetic as attention over the full cache.
// The reference has no such stage; the policy is specified here and restated in the CPU checker.
// With a workspace the update is spread over several CTAs per (b, kv head). Each probes a slice of the index list
// (list -> token-to-slot map, two dependent loads per entry, many in flight), stamps the hits, writes their slots and
// records the misses in a bitmap. Then either all of them work through the evictions, each on its range of the slots
// (lru_update_multi_kernel), or the last CTA of the pair to finish (a ticket, nobody waits) handles the misses alone
// (lru_update_kernel). Victim selection is a histogram select over ages (no sort), the ordered assignments use bitmaps
// and block scans.
#include "sl_common.cuh"

namespace {

constexpr int LT = 1024;
constexpr int LW = LT / 32;
constexpr int AGE_MAX = 1023;           // ages are clamped here; free slots count as AGE_MAX + 1
constexpr int NBIN = AGE_MAX + 2;

struct LruArgs {
    const int* idx; int cap; const int* cnt;
    int B, KH, C, step, row_bytes;
    const long long* d_step;               // optional: the step (clock of the table) in device memory
    const unsigned char* k_back; const unsigned char* v_back;
    long long back_bstride, back_tok, back_head;     // bytes: batch row, key, kv head of the backing store
    unsigned char* k_res; unsigned char* v_res;
    long long res_bstride, res_tok, res_head;        // bytes: batch row, slot, kv head of the resident buffers
    int* tok2slot; long long n_max; int* slot2tok; int* last_used;
    int* slots_out; int* stats; int* status;
    // several CTAs per (b, kv head): slices of the list, the miss bitmap and the counters in global memory
    int parts;                             // CTAs per (b, kv head); 1 = everything in one CTA
    unsigned* g_miss;                      // [B*KH][nw] bitmap of the list entries that missed
    unsigned* g_count;                     // [B*KH][2] hits of the step, finished CTAs (both left at zero)
    int2* g_pairs;                         // [B*KH][cap] {key, slot} of the misses, copied by lru_copy_kernel
    int* g_m;                              // [B*KH] number of misses of the step
    // the update spread over the CTAs of a (b, kv head) pair (lru_update_multi_kernel)
    unsigned* g_hist;                      // [B*KH][NBIN] ages of the pair's slots, all parts (left zeroed)
    int2* g_cnt;                           // [B*KH][parts] {older than tau, of age tau} in each part's slot range
    int* g_pm;                             // [B*KH][parts] misses in each part's slice of the list
    int* g_vict;                           // [B*KH][cap] slot taken by the r-th miss
    unsigned* g_bar;                       // [B*KH][8] barrier counters of the pair
    int deferred;                          // the rows of the misses are not copied here: their slots go out as -(slot + 1)
    // 0: the whole update in one launch. The decode step splits it so that the attention need not wait for the evictions:
    // 1: the probe only (hits stamped and their slots written, misses marked -1 and recorded in the bitmap, hits counted);
    // 2: the evictions only, one CTA per (b, kv head), from the bitmap and the count of a phase-1 launch; the slot list is
    //    not touched (the attention that runs beside it reads the misses from the backing store)
    int phase;
};

// exclusive prefix of one value per thread over the block (thread order) and the block total
__device__ __forceinline__ int block_exclusive_scan(int v, int* wsum, int& total) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    int inc = v;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, inc, d);
        if (lane >= d) inc += t;
    }
    if (lane == 31) wsum[warp] = inc;
    __syncthreads();
    int wv = wsum[lane];                      // LW == 32 warps: one value per lane
    int winc = wv;
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, winc, d);
        if (lane >= d) winc += t;
    }
    total = __shfl_sync(0xffffffffu, winc, 31);
    const int before = __shfl_sync(0xffffffffu, winc - wv, warp);
    __syncthreads();
    return before + inc - v;
}

// Ranks come from bitmaps, not from ordered loops: a flag per slot (or list entry) is packed into
// 32-bit words by warp ballots, one block scan over the words' popcounts gives every word its
// prefix, and every element finds its own rank with one more popcount. The kernel has a fixed,
// small number of block barriers whatever C and n are.
__global__ void __launch_bounds__(LT) lru_update_kernel(const LruArgs a) {
    extern __shared__ int smem_i[];
    const int cw = (a.C + 31) >> 5, nw = (a.cap + 31) >> 5;      // bitmap words over slots / list entries
    int* victims = smem_i;                 // [cap] slot taken by the r-th miss
    int* misstok = victims + a.cap;        // [cap] key of the r-th miss
    unsigned* m_gt = reinterpret_cast<unsigned*>(misstok + a.cap);   // [cw] slots older than tau
    unsigned* m_eq = m_gt + cw;            // [cw] slots of age tau
    int* p_gt = reinterpret_cast<int*>(m_eq + cw);                   // [cw] prefixes of the two bitmaps
    int* p_eq = p_gt + cw;
    unsigned* m_miss = reinterpret_cast<unsigned*>(p_eq + cw);       // [nw] list entries that missed
    int* p_miss = reinterpret_cast<int*>(m_miss + nw);               // [nw]
    unsigned short* age16 = reinterpret_cast<unsigned short*>(p_miss + nw);   // [C]
    __shared__ unsigned hist[NBIN];
    __shared__ int wsum[LW];
    __shared__ int s_hits, s_tau, s_r;

    const int h = blockIdx.x, b = blockIdx.y, part = blockIdx.z, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const long long bh = (long long)b * a.KH + h;
    sl::pdl_trigger();
    sl::pdl_wait();                        // the index list and the counts come from the scan before this launch
    const int n = min(a.cnt[bh], a.cap);
    const int* list = a.idx + bh * a.cap;
    int* out = a.slots_out + bh * a.cap;
    int* t2s = a.tok2slot + bh * a.n_max;
    int* s2t = a.slot2tok + bh * a.C;
    int* lu = a.last_used + bh * a.C;
    const int t = a.d_step ? (int)__ldg(a.d_step) : a.step;
    const unsigned lt = (1u << lane) - 1u;
    unsigned* gm = (a.parts > 1 || a.phase != 0) ? a.g_miss + bh * nw : nullptr;    // one CTA keeps its bitmap in shared memory

    if (tid == 0) s_hits = 0;
    for (int i = tid; i < NBIN; i += LT) hist[i] = 0;
    __syncthreads();
    if (n > a.C) {                          // the table cannot hold this step's attended set
        if (tid == 0 && part == 0) {
            if (a.status) atomicExch(a.status, 3);
            if (a.g_m) a.g_m[bh] = 0;
        }
        return;
    }

    // ---- hits: stamp their slots; misses go into a bitmap (eight entries per thread and round, so
    // that the two dependent loads of an entry cost one trip to memory per round, not per entry).
    // This CTA's slice of the list: whole bitmap words [w0, w1).
    const int wpp = (nw + a.parts - 1) / a.parts;
    const int w0 = min(nw, part * wpp), w1 = min(nw, w0 + wpp);
    int myhits = 0;
    for (int j0 = w0 * 32 + warp * 32; j0 < w1 * 32 && a.phase != 2; j0 += LT * 8) {
        int tok[8], sl_[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int j = j0 + u * LT + lane;
            tok[u] = (j < n && j < w1 * 32) ? __ldg(list + j) : -1;
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) sl_[u] = tok[u] >= 0 ? t2s[tok[u]] : -1;
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int j = j0 + u * LT + lane;
            if (tok[u] >= 0) {
                if (sl_[u] >= 0) { lu[sl_[u]] = t; ++myhits; }
                out[j] = sl_[u];
            }
            const unsigned mb = __ballot_sync(0xffffffffu, tok[u] >= 0 && sl_[u] < 0);
            if (lane == 0 && (j0 + u * LT) < w1 * 32) {
                if (gm) gm[(j0 + u * LT) >> 5] = mb;
                else m_miss[(j0 + u * LT) >> 5] = mb;
            }
        }
    }
    myhits = __reduce_add_sync(0xffffffffu, myhits);
    if (lane == 0 && myhits) atomicAdd(&s_hits, myhits);
    __syncthreads();
    if (a.phase == 1) {                      // the probe alone: leave the hits of this slice to the eviction launch
        if (tid == 0 && s_hits) atomicAdd(a.g_count + bh * 2, (unsigned)s_hits);
        return;
    }
    if (a.phase == 2) {                      // the evictions alone: everybody's hits and misses come from the probe launch
        if (tid == 0) s_hits = (int)atomicExch(a.g_count + bh * 2, 0u);
        for (int w = tid; w < nw; w += LT) m_miss[w] = __ldcg(gm + w);
        __syncthreads();
    } else if (a.parts > 1) {
        // ticket: the CTA that finds the other slices done goes on (with everybody's hits and misses)
        __shared__ int s_last;
        if (tid == 0) {
            unsigned* cnt2 = a.g_count + bh * 2;
            if (s_hits) atomicAdd(cnt2, (unsigned)s_hits);
            __threadfence();                                // this slice's stamps, slots and bitmap words first
            const unsigned old = atomicAdd(cnt2 + 1, 1u);
            s_last = old == (unsigned)a.parts - 1u;
            if (s_last) {
                __threadfence();
                s_hits = (int)atomicExch(cnt2, 0u);         // both counters are left at zero for the next step
                cnt2[1] = 0u;
            }
        }
        __syncthreads();
        if (!s_last) return;
        for (int w = tid; w < nw; w += LT) m_miss[w] = __ldcg(gm + w);
        __syncthreads();
    }
    const int m = n - s_hits;              // misses = victims needed
    if (m == 0) {                           // everything was resident: nothing to evict or copy
        if (tid == 0) {
            if (a.stats) { a.stats[bh * 2] = s_hits; a.stats[bh * 2 + 1] = 0; }
            if (a.g_m) a.g_m[bh] = 0;
        }
        return;
    }

    // ---- ages of the slots not used in this step: kept in shared memory, histogrammed
    for (int s0 = tid; s0 < a.C; s0 += LT * 16) {
        int l[16];
#pragma unroll
        for (int u = 0; u < 16; ++u) l[u] = s0 + u * LT < a.C ? __ldcg(lu + s0 + u * LT) : t;   // other slices stamped hits
#pragma unroll
        for (int u = 0; u < 16; ++u) {
            if (s0 + u * LT < a.C) {
                const int age = l[u] < 0 ? AGE_MAX + 1 : min(t - l[u], AGE_MAX);
                age16[s0 + u * LT] = (unsigned short)age;
                if (age > 0) atomicAdd(&hist[age], 1u);
            }
        }
    }
    __syncthreads();
    if (tid < 32) {                         // oldest first: largest age with a cumulative count >= m
        int tau = NBIN, r = 0;
        const int BW = (NBIN + 31) >> 5;
        const int blo = lane * BW, bhi = min(NBIN, blo + BW);
        unsigned bs = 0;
        for (int i = blo; i < bhi; ++i) bs += hist[i];
        unsigned suf = bs;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const unsigned v = __shfl_down_sync(0xffffffffu, suf, d);
            if (lane + d < 32) suf += v;
        }
        const unsigned ball = __ballot_sync(0xffffffffu, suf >= (unsigned)m);
        if (ball == 0u && lane == 0 && a.status) atomicExch(a.status, 4);   // table state is inconsistent
        const int L = ball ? 31 - __clz(ball) : 0;   // a consistent table always has n - hits evictable slots
        int tau_l = 0, gt_l = 0;
        if (lane == L) {
            unsigned cum = suf - bs;
            for (int i = bhi - 1; i >= blo; --i) {
                const unsigned v = hist[i];
                if (cum + v >= (unsigned)m) { tau_l = i; gt_l = (int)cum; break; }
                cum += v;
            }
        }
        tau = __shfl_sync(0xffffffffu, tau_l, L);
        r = m - __shfl_sync(0xffffffffu, gt_l, L);
        if (lane == 0) { s_tau = tau; s_r = r; }
    }
    __syncthreads();
    const int tau = s_tau, r = s_r;

    // ---- victim bitmaps: every slot older than tau, and the slots of age tau (the first r are taken)
#pragma unroll 4
    for (int w = warp; w < cw; w += LW) {
        const int s = w * 32 + lane;
        const int age = s < a.C ? (int)age16[s] : 0;
        const unsigned g = __ballot_sync(0xffffffffu, age > tau);
        const unsigned e = __ballot_sync(0xffffffffu, age == tau && age > 0);
        if (lane == 0) { m_gt[w] = g; m_eq[w] = e; }
    }
    __syncthreads();
    // prefixes of the word popcounts: thread i owns words [i*WPT, (i+1)*WPT)
    {
        const int WPT = (cw + LT - 1) / LT;
        int cg = 0, ce = 0;
        for (int k = 0; k < WPT; ++k) {
            const int w = tid * WPT + k;
            if (w < cw) { cg += __popc(m_gt[w]); ce += __popc(m_eq[w]); }
        }
        int tg, te;
        int pg = block_exclusive_scan(cg, wsum, tg);
        int pe = block_exclusive_scan(ce, wsum, te);
        for (int k = 0; k < WPT; ++k) {
            const int w = tid * WPT + k;
            if (w < cw) {
                p_gt[w] = pg; p_eq[w] = pe;
                pg += __popc(m_gt[w]); pe += __popc(m_eq[w]);
            }
        }
    }
    __syncthreads();
    // victims in slot order: a taken slot's position is (older slots before it) + (taken ties before it)
#pragma unroll 4
    for (int w = warp; w < cw; w += LW) {
        const unsigned g = m_gt[w], e = m_eq[w];
        const int gb = p_gt[w] + __popc(g & lt), eb = p_eq[w] + __popc(e & lt);
        const bool isg = (g >> lane) & 1u, ise = (e >> lane) & 1u;
        if (isg || (ise && eb < r)) victims[gb + min(eb, r)] = w * 32 + lane;
    }
    // ranks of the misses in list order
    {
        const int WPT = (nw + LT - 1) / LT;
        int cm = 0;
        for (int k = 0; k < WPT; ++k) {
            const int w = tid * WPT + k;
            if (w < nw) cm += __popc(m_miss[w]);
        }
        int tm;
        int pm = block_exclusive_scan(cm, wsum, tm);
        for (int k = 0; k < WPT; ++k) {
            const int w = tid * WPT + k;
            if (w < nw) { p_miss[w] = pm; pm += __popc(m_miss[w]); }
        }
    }
    __syncthreads();

    // ---- misses in list order take the victims in that order
    // (four list words per round: the loads of a round -- the key, the victim's old key -- are in flight together; the
    // stores cannot collide: victims are distinct slots, their old keys are resident and the misses are not)
    for (int w0 = warp; w0 < nw; w0 += 4 * LW) {
        int jv[4], vv[4], tokv[4], oldv[4], rankv[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int w = w0 + u * LW;
            const unsigned mm = w < nw ? m_miss[w] : 0u;
            jv[u] = -1;
            if ((mm >> lane) & 1u) {
                jv[u] = w * 32 + lane;
                rankv[u] = p_miss[w] + __popc(mm & lt);
                vv[u] = victims[rankv[u]];
                tokv[u] = __ldg(list + jv[u]);
                oldv[u] = s2t[vv[u]];
            }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            if (jv[u] >= 0) {
                if (oldv[u] >= 0) t2s[oldv[u]] = -1;
                t2s[tokv[u]] = vv[u];
                s2t[vv[u]] = tokv[u];
                lu[vv[u]] = t;
                if (a.phase != 2) out[jv[u]] = a.deferred ? -(vv[u] + 1) : vv[u];
                misstok[rankv[u]] = tokv[u];
            }
        }
    }
    __syncthreads();

    if (a.deferred) {
        // the attention launch that follows fetches these rows from the backing store and fills the slots on the way
        if (tid == 0 && a.g_m) a.g_m[bh] = m;
    } else if (a.g_pairs) {
        // the rows are copied by the launch that follows (many CTAs): leave it the {key, slot} pairs
        int2* pairs = a.g_pairs + bh * a.cap;
        for (int i = tid; i < m; i += LT) pairs[i] = make_int2(misstok[i], victims[i]);
        if (tid == 0) a.g_m[bh] = m;
    } else {
        // ---- copy the missing rows from the backing store into their slots (16-byte lanes, four rows in flight per group)
        const int lanes = a.row_bytes >> 4;                 // 16 (2-byte types) or 32 (4-byte types)
        const int groups = LT / lanes, grp = tid / lanes, c = tid % lanes;
        const unsigned char* kb = a.k_back + b * a.back_bstride + (long long)h * a.back_head + c * 16;
        const unsigned char* vb = a.v_back + b * a.back_bstride + (long long)h * a.back_head + c * 16;
        unsigned char* kr = a.k_res + b * a.res_bstride + (long long)h * a.res_head + c * 16;
        unsigned char* vr = a.v_res + b * a.res_bstride + (long long)h * a.res_head + c * 16;
        for (int i0 = grp; i0 < m; i0 += 4 * groups) {
            uint4 kv[4], vv[4];
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int i = i0 + u * groups;
                if (i < m) {
                    const long long src = (long long)misstok[i] * a.back_tok;
                    kv[u] = *reinterpret_cast<const uint4*>(kb + src);
                    vv[u] = *reinterpret_cast<const uint4*>(vb + src);
                }
            }
#pragma unroll
            for (int u = 0; u < 4; ++u) {
                const int i = i0 + u * groups;
                if (i < m) {
                    const long long dst = (long long)victims[i] * a.res_tok;
                    *reinterpret_cast<uint4*>(kr + dst) = kv[u];
                    *reinterpret_cast<uint4*>(vr + dst) = vv[u];
                }
            }
        }
    }
    if (tid == 0 && a.stats) { a.stats[bh * 2] = s_hits; a.stats[bh * 2 + 1] = m; }
}

// The same update with EVERY CTA of a (b, kv head) pair working all the way through: a CTA owns a slice of the index list
// and a range of the slots; what one CTA needs from the others crosses global memory behind four barriers of the pair
// (bounded spins; the launch is cooperative, so the CTAs of a pair are resident together):
//   probe own slice | B0 | ages of own slots -> shared histogram | B1 | threshold age (every CTA for itself), victim bitmaps of own
//   slots, their counts | B2 | victims of own slots at their global ranks | B3 | own slice's misses take their victims
// Same policy, same tables and slots afterwards as lru_update_kernel.
__global__ void __launch_bounds__(LT) lru_update_multi_kernel(const LruArgs a) {
    extern __shared__ int smem_i[];
    const int P = a.parts;
    const int cw = (a.C + 31) >> 5, nw = (a.cap + 31) >> 5;
    const int cwpp = (cw + P - 1) / P, wpp = (nw + P - 1) / P;
    unsigned* m_gt = reinterpret_cast<unsigned*>(smem_i);            // [cwpp] own slots older than tau
    unsigned* m_eq = m_gt + cwpp;                                    // [cwpp] own slots of age tau
    int* p_gt = reinterpret_cast<int*>(m_eq + cwpp);                 // [cwpp] prefixes inside the own range
    int* p_eq = p_gt + cwpp;
    unsigned* m_miss = reinterpret_cast<unsigned*>(p_eq + cwpp);     // [wpp] own list entries that missed
    int* p_miss = reinterpret_cast<int*>(m_miss + wpp);              // [wpp]
    unsigned short* age16 = reinterpret_cast<unsigned short*>(p_miss + wpp);   // [cwpp * 32]
    __shared__ unsigned hist[NBIN];
    __shared__ int wsum[LW];
    __shared__ int s_hits, s_tau, s_r, s_gb, s_eb, s_mb;

    const int h = blockIdx.x, b = blockIdx.y, part = blockIdx.z, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const long long bh = (long long)b * a.KH + h;
    sl::pdl_trigger();
    sl::pdl_wait();
    const int n = min(a.cnt[bh], a.cap);
    const int* list = a.idx + bh * a.cap;
    int* out = a.slots_out + bh * a.cap;
    int* t2s = a.tok2slot + bh * a.n_max;
    int* s2t = a.slot2tok + bh * a.C;
    int* lu = a.last_used + bh * a.C;
    const int t = a.d_step ? (int)__ldg(a.d_step) : a.step;
    const unsigned lt = (1u << lane) - 1u;
    unsigned* bar = a.g_bar + bh * 8;
    unsigned* cnt2 = a.g_count + bh * 2;

    if (tid == 0) s_hits = 0;
    for (int i = tid; i < NBIN; i += LT) hist[i] = 0;
    if (part == 0 && tid >= 1 && tid <= 3) bar[tid] = 0u;           // the counters of B1..B3: nobody is near them before B0
    __syncthreads();
    if (n > a.C) {                          // the table cannot hold this step's attended set (every CTA of the pair sees it)
        if (tid == 0 && part == 0) {
            if (a.status) atomicExch(a.status, 3);
            if (a.g_m) a.g_m[bh] = 0;
        }
        return;
    }

    // ---- probe of the own slice of the list: whole bitmap words [w0, w1)
    const int w0 = min(nw, part * wpp), w1 = min(nw, w0 + wpp);
    int myhits = 0;
    for (int j0 = w0 * 32 + warp * 32; j0 < w1 * 32; j0 += LT * 8) {
        int tok[8], sl_[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int j = j0 + u * LT + lane;
            tok[u] = (j < n && j < w1 * 32) ? __ldg(list + j) : -1;
        }
#pragma unroll
        for (int u = 0; u < 8; ++u) sl_[u] = tok[u] >= 0 ? t2s[tok[u]] : -1;
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            const int j = j0 + u * LT + lane;
            if (tok[u] >= 0) {
                if (sl_[u] >= 0) { lu[sl_[u]] = t; ++myhits; }
                out[j] = sl_[u];
            }
            const unsigned mb = __ballot_sync(0xffffffffu, tok[u] >= 0 && sl_[u] < 0);
            if (lane == 0 && (j0 + u * LT) < w1 * 32) m_miss[((j0 + u * LT) >> 5) - w0] = mb;
        }
    }
    myhits = __reduce_add_sync(0xffffffffu, myhits);
    if (lane == 0 && myhits) atomicAdd(&s_hits, myhits);
    __syncthreads();
    // ranks of the own misses inside the slice, and their number
    int my_misses;
    {
        const int WPT = (wpp + LT - 1) / LT;
        int cm = 0;
        for (int k = 0; k < WPT; ++k) {
            const int w = tid * WPT + k;
            if (w < w1 - w0) cm += __popc(m_miss[w]);
        }
        int pm = block_exclusive_scan(cm, wsum, my_misses);
        for (int k = 0; k < WPT; ++k) {
            const int w = tid * WPT + k;
            if (w < w1 - w0) { p_miss[w] = pm; pm += __popc(m_miss[w]); }
        }
    }
    if (tid == 0) {
        if (s_hits) atomicAdd(cnt2, (unsigned)s_hits);
        a.g_pm[bh * P + part] = my_misses;
    }
    sl::grid_barrier(bar + 0, (unsigned)P, a.status);               // B0: every slice is probed, every hit stamped
    const int total_hits = (int)__ldcg(cnt2);
    const int m = n - total_hits;              // misses = victims needed
    if (m == 0) {                               // everything was resident: nothing to evict
        // the last CTA of the pair to get here (a ticket, nobody waits) knows that everybody has read the count
        if (tid == 0 && atomicAdd(bar + 4, 1u) == (unsigned)P - 1u) {
            *cnt2 = 0u; bar[0] = 0u; bar[4] = 0u;
            if (a.stats) { a.stats[bh * 2] = total_hits; a.stats[bh * 2 + 1] = 0; }
            if (a.g_m) a.g_m[bh] = 0;
        }
        return;
    }

    // ---- ages of the own slots [32 cw0, 32 cw1) not used in this step, into the pair's histogram
    const int cw0 = min(cw, part * cwpp), cw1 = min(cw, cw0 + cwpp);
    const int s_lo = cw0 * 32, s_hi = min(a.C, cw1 * 32);
    for (int s0 = s_lo + tid; s0 < s_hi; s0 += LT * 8) {
        int l[8];
#pragma unroll
        for (int u = 0; u < 8; ++u) l[u] = s0 + u * LT < s_hi ? __ldcg(lu + s0 + u * LT) : t;
#pragma unroll
        for (int u = 0; u < 8; ++u) {
            if (s0 + u * LT < s_hi) {
                const int age = l[u] < 0 ? AGE_MAX + 1 : min(t - l[u], AGE_MAX);
                age16[s0 + u * LT - s_lo] = (unsigned short)age;
                if (age > 0) atomicAdd(&hist[age], 1u);
            }
        }
    }
    __syncthreads();
    unsigned* gh = a.g_hist + bh * NBIN;
    for (int i = tid; i < NBIN; i += LT)
        if (hist[i]) atomicAdd(gh + i, hist[i]);
    sl::grid_barrier(bar + 1, (unsigned)P, a.status);               // B1: the histogram is complete
    for (int i = tid; i < NBIN; i += LT) hist[i] = __ldcg(gh + i);
    __syncthreads();
    if (tid < 32) {                         // oldest first: largest age with a cumulative count >= m
        const int BW = (NBIN + 31) >> 5;
        const int blo = lane * BW, bhi = min(NBIN, blo + BW);
        unsigned bs = 0;
        for (int i = blo; i < bhi; ++i) bs += hist[i];
        unsigned suf = bs;
#pragma unroll
        for (int d = 1; d < 32; d <<= 1) {
            const unsigned v = __shfl_down_sync(0xffffffffu, suf, d);
            if (lane + d < 32) suf += v;
        }
        const unsigned ball = __ballot_sync(0xffffffffu, suf >= (unsigned)m);
        if (ball == 0u && lane == 0 && a.status) atomicExch(a.status, 4);   // table state is inconsistent
        const int L = ball ? 31 - __clz(ball) : 0;
        int tau_l = 0, gt_l = 0;
        if (lane == L) {
            unsigned cum = suf - bs;
            for (int i = bhi - 1; i >= blo; --i) {
                const unsigned v = hist[i];
                if (cum + v >= (unsigned)m) { tau_l = i; gt_l = (int)cum; break; }
                cum += v;
            }
        }
        const int tau = __shfl_sync(0xffffffffu, tau_l, L);
        const int r = m - __shfl_sync(0xffffffffu, gt_l, L);
        if (lane == 0) { s_tau = tau; s_r = r; }
    }
    __syncthreads();
    const int tau = s_tau, r = s_r;
    // ---- victim bitmaps of the own slots and their counts
#pragma unroll 4
    for (int w = cw0 + warp; w < cw1; w += LW) {
        const int s = w * 32 + lane;
        const int age = s < a.C ? (int)age16[s - s_lo] : 0;
        const unsigned g = __ballot_sync(0xffffffffu, age > tau);
        const unsigned e = __ballot_sync(0xffffffffu, age == tau && age > 0);
        if (lane == 0) { m_gt[w - cw0] = g; m_eq[w - cw0] = e; }
    }
    __syncthreads();
    {
        const int WPT = (cwpp + LT - 1) / LT;
        int cg = 0, ce = 0;
        for (int k = 0; k < WPT; ++k) {
            const int w = tid * WPT + k;
            if (w < cw1 - cw0) { cg += __popc(m_gt[w]); ce += __popc(m_eq[w]); }
        }
        int tg, te;
        int pg = block_exclusive_scan(cg, wsum, tg);
        int pe = block_exclusive_scan(ce, wsum, te);
        for (int k = 0; k < WPT; ++k) {
            const int w = tid * WPT + k;
            if (w < cw1 - cw0) {
                p_gt[w] = pg; p_eq[w] = pe;
                pg += __popc(m_gt[w]); pe += __popc(m_eq[w]);
            }
        }
        if (tid == 0) a.g_cnt[bh * P + part] = make_int2(tg, te);
    }
    sl::grid_barrier(bar + 2, (unsigned)P, a.status);               // B2: every range's counts are there
    if (tid == 0) {                          // the ranges before this one, the slices before this one
        int gb = 0, eb = 0, mb = 0;
        for (int q = 0; q < part; ++q) {
            const int2 c = __ldcg(a.g_cnt + bh * P + q);
            gb += c.x; eb += c.y;
            mb += __ldcg(a.g_pm + bh * P + q);
        }
        s_gb = gb; s_eb = eb; s_mb = mb;
    }
    // the pair's histogram is read by everybody by now: this CTA's share of it goes back to zero for the next call
    for (int i = part * LT + tid; i < NBIN; i += P * LT) gh[i] = 0u;
    __syncthreads();
    int* vict = a.g_vict + bh * a.cap;
#pragma unroll 4
    for (int w = warp; w < cw1 - cw0; w += LW) {
        const unsigned g = m_gt[w], e = m_eq[w];
        const int gb = s_gb + p_gt[w] + __popc(g & lt), eb = s_eb + p_eq[w] + __popc(e & lt);
        const bool isg = (g >> lane) & 1u, ise = (e >> lane) & 1u;
        if (isg || (ise && eb < r)) vict[gb + min(eb, r)] = (cw0 + w) * 32 + lane;
    }
    sl::grid_barrier(bar + 3, (unsigned)P, a.status);               // B3: the victims stand at their ranks
    // ---- the own slice's misses, in list order, take the victims in that order
    int2* pairs = (a.g_pairs && !a.deferred) ? a.g_pairs + bh * a.cap : nullptr;
    for (int wq = warp; wq < w1 - w0; wq += 4 * LW) {
        int jv[4], vv[4], tokv[4], oldv[4], rankv[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int w = wq + u * LW;
            const unsigned mm = w < w1 - w0 ? m_miss[w] : 0u;
            jv[u] = -1;
            if ((mm >> lane) & 1u) {
                jv[u] = (w0 + w) * 32 + lane;
                rankv[u] = s_mb + p_miss[w] + __popc(mm & lt);
                vv[u] = __ldcg(vict + rankv[u]);
                tokv[u] = __ldg(list + jv[u]);
                oldv[u] = s2t[vv[u]];
            }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            if (jv[u] >= 0) {
                if (oldv[u] >= 0) t2s[oldv[u]] = -1;
                t2s[tokv[u]] = vv[u];
                s2t[vv[u]] = tokv[u];
                lu[vv[u]] = t;
                out[jv[u]] = a.deferred ? -(vv[u] + 1) : vv[u];
                if (pairs) pairs[rankv[u]] = make_int2(tokv[u], vv[u]);
            }
        }
    }
    if (part == 0 && tid == 0) {
        *cnt2 = 0u; bar[0] = 0u;              // everybody is past B1 (and so past reading the count and leaving B0)
        if (a.g_m) a.g_m[bh] = m;
        if (a.stats) { a.stats[bh * 2] = total_hits; a.stats[bh * 2 + 1] = m; }
    }
}

// The rows of the step's misses, copied from the backing store into their slots by CP CTAs per (b, kv head):
// the {key, slot} pairs and their number come from lru_update_kernel; 16-byte lanes, four rows in flight per group.
constexpr int CT = 256;
__global__ void __launch_bounds__(CT) lru_copy_kernel(const LruArgs a) {
    sl::pdl_trigger();
    sl::pdl_wait();
    const int h = blockIdx.y, b = blockIdx.z, tid = threadIdx.x;
    const long long bh = (long long)b * a.KH + h;
    const int m = a.g_m[bh];
    if (m <= 0) return;
    const int2* pairs = a.g_pairs + bh * a.cap;
    const int lanes = a.row_bytes >> 4, groups = CT / lanes, grp = tid / lanes, c = tid % lanes;
    const unsigned char* kb = a.k_back + b * a.back_bstride + (long long)h * a.back_head + c * 16;
    const unsigned char* vb = a.v_back + b * a.back_bstride + (long long)h * a.back_head + c * 16;
    unsigned char* kr = a.k_res + b * a.res_bstride + (long long)h * a.res_head + c * 16;
    unsigned char* vr = a.v_res + b * a.res_bstride + (long long)h * a.res_head + c * 16;
    const int stride = gridDim.x * groups;
    for (int i0 = blockIdx.x * groups + grp; i0 < m; i0 += 4 * stride) {
        int2 p[4];
        uint4 kv[4], vv[4];
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            const int i = i0 + u * stride;
            p[u] = i < m ? __ldcg(pairs + i) : make_int2(0, 0);
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            if (i0 + u * stride < m) {
                const long long src = (long long)p[u].x * a.back_tok;
                kv[u] = *reinterpret_cast<const uint4*>(kb + src);
                vv[u] = *reinterpret_cast<const uint4*>(vb + src);
            }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
            if (i0 + u * stride < m) {
                const long long dst = (long long)p[u].y * a.res_tok;
                *reinterpret_cast<uint4*>(kr + dst) = kv[u];
                *reinterpret_cast<uint4*>(vr + dst) = vv[u];
            }
        }
    }
}

}  // namespace

namespace {

int g_lru_multi = 1;       // 1: every CTA of a (b, kv head) pair works through the whole update; 0: the last one alone handles the misses

int lru_parts(int B, int KH, int idx_capacity) {
    // enough CTAs to put every SM to work on the probe, at least 1024 list entries (one round of a CTA) each
    const int by_work = std::max(1, idx_capacity / 1024);
    const int by_sms = std::max(1, sl::sm_count() / std::max(1, B * KH));
    return std::max(1, std::min(std::min(by_work, by_sms), 64));
}

int lru_launch(const int32_t* d_idx, int idx_capacity, const int32_t* d_cnt, int B, int KH, const void* k_backing,
               const void* v_backing, const sl_kv_layout& back, int elem_bytes, void* d_k_resident, void* d_v_resident,
               const sl_kv_layout& res, int C, int32_t* d_tok2slot, int64_t n_max, int32_t* d_slot2tok,
               int32_t* d_last_used, int step, const int64_t* d_step, int32_t* d_slots_out, int32_t* d_stats,
               int32_t* d_status, void* d_workspace, size_t workspace_bytes, void* stream, bool deferred = false, int phase = 0) {
    SL_REQUIRE(d_idx && d_cnt && (deferred || phase == 1 || (k_backing && v_backing)) && d_k_resident && d_v_resident && d_tok2slot && d_slot2tok &&
                   d_last_used && d_slots_out,
               SL_EINVAL, "sl_lru_update: null pointer");
    SL_REQUIRE(B > 0 && B <= 65535 && KH > 0 && C > 0 && idx_capacity > 0 && n_max > 0 && step >= 0, SL_ESHAPE,
               "sl_lru_update: bad shape");
    SL_REQUIRE(elem_bytes == 2 || elem_bytes == 4, SL_EINVAL, "sl_lru_update: elem_bytes must be 2 or 4");
    SL_REQUIRE((deferred || phase == 1 || (sl::aligned16(k_backing) && sl::aligned16(v_backing))) && sl::aligned16(d_k_resident) &&
                   sl::aligned16(d_v_resident),
               SL_EALIGN, "sl_lru_update: K/V buffers must be 16-byte aligned");
    for (const sl_kv_layout* l : {&back, &res})
        SL_REQUIRE((l->batch_stride * elem_bytes) % 16 == 0 && (l->token_stride * elem_bytes) % 16 == 0 &&
                       (l->head_stride * elem_bytes) % 16 == 0 && l->token_stride >= 128 && l->head_stride >= 128,
                   SL_EALIGN, "sl_lru_update: cache strides must be multiples of 16 bytes and hold a 128-value row");
    const size_t cw = ((size_t)C + 31) / 32, nw = ((size_t)idx_capacity + 31) / 32;
    const size_t smem = (size_t)idx_capacity * 2 * sizeof(int) + cw * 16 + nw * 8 + (size_t)C * 2 + 16;
    SL_REQUIRE(smem <= 220 * 1024, SL_ESHAPE, "sl_lru_update: idx_capacity %d / %d slots too large for shared memory",
               idx_capacity, C);
    LruArgs a = {};
    a.idx = d_idx; a.cap = idx_capacity; a.cnt = d_cnt;
    a.B = B; a.KH = KH; a.C = C; a.step = step; a.row_bytes = 128 * elem_bytes;
    a.d_step = reinterpret_cast<const long long*>(d_step);
    a.k_back = static_cast<const unsigned char*>(k_backing); a.v_back = static_cast<const unsigned char*>(v_backing);
    a.back_bstride = back.batch_stride * elem_bytes; a.back_tok = back.token_stride * elem_bytes; a.back_head = back.head_stride * elem_bytes;
    a.k_res = static_cast<unsigned char*>(d_k_resident); a.v_res = static_cast<unsigned char*>(d_v_resident);
    a.res_bstride = res.batch_stride * elem_bytes; a.res_tok = res.token_stride * elem_bytes; a.res_head = res.head_stride * elem_bytes;
    a.tok2slot = d_tok2slot; a.n_max = n_max; a.slot2tok = d_slot2tok; a.last_used = d_last_used;
    a.slots_out = d_slots_out; a.stats = d_stats; a.status = d_status;
    a.parts = 1;
    a.deferred = deferred ? 1 : 0;
    a.phase = phase;
    SL_REQUIRE(phase == 0 || d_workspace, SL_EINVAL, "sl_lru_probe / sl_lru_evict: the workspace carries the misses from one launch to the other");
    if (d_workspace) {
        SL_REQUIRE(workspace_bytes >= sl_lru_workspace_bytes(B, KH, idx_capacity), SL_EWORKSPACE,
                   "sl_lru_update_ex: workspace %zu < required %zu", workspace_bytes, sl_lru_workspace_bytes(B, KH, idx_capacity));
        SL_REQUIRE(sl::aligned16(d_workspace), SL_EALIGN, "sl_lru_update_ex: workspace not 16-byte aligned");
        a.parts = lru_parts(B, KH, idx_capacity);
        a.g_count = static_cast<unsigned*>(d_workspace);
        a.g_m = reinterpret_cast<int*>(a.g_count + (((size_t)B * KH * 2 + 63) / 64) * 64);
        a.g_miss = reinterpret_cast<unsigned*>(a.g_m + (((size_t)B * KH + 63) / 64) * 64);
        a.g_pairs = reinterpret_cast<int2*>(a.g_miss + (((size_t)B * KH * nw + 3) / 4) * 4);
        // behind the pairs: what the CTAs of a pair exchange when all of them work through the update
        const size_t bh = (size_t)B * KH;
        a.g_hist = reinterpret_cast<unsigned*>(a.g_pairs + bh * idx_capacity);
        a.g_bar = a.g_hist + ((bh * NBIN + 3) / 4) * 4;
        a.g_cnt = reinterpret_cast<int2*>(a.g_bar + bh * 8);
        a.g_pm = reinterpret_cast<int*>(a.g_cnt + bh * 64);
        a.g_vict = a.g_pm + bh * 64;
    }
    if (g_lru_multi && phase == 0 && d_workspace && a.parts > 1 && B * KH * a.parts <= sl::sm_count()) {
        const size_t cwpp = (cw + a.parts - 1) / a.parts, wpp = (nw + a.parts - 1) / a.parts;
        const size_t smem_m = cwpp * 16 + wpp * 8 + cwpp * 64 + 16;
        SL_CUDA_OK(sl::ensure_dyn_smem(reinterpret_cast<const void*>(lru_update_multi_kernel), smem_m));
        SL_CUDA_OK(sl::launch_kernel(lru_update_multi_kernel, dim3((unsigned)KH, (unsigned)B, (unsigned)a.parts), dim3(LT), smem_m,
                                     static_cast<cudaStream_t>(stream), true, a));
        if (!deferred) {
            const int cp = std::max(1, std::min(32, sl::sm_count() / std::max(1, B * KH)));
            SL_CUDA_OK(sl::launch_kernel(lru_copy_kernel, dim3((unsigned)cp, (unsigned)KH, (unsigned)B), dim3(CT), 0,
                                         static_cast<cudaStream_t>(stream), false, a));
        }
        return SL_OK;
    }
    SL_CUDA_OK(sl::ensure_dyn_smem(reinterpret_cast<const void*>(lru_update_kernel), smem));
    if (phase == 2) a.parts = 1;
    dim3 grid((unsigned)KH, (unsigned)B, (unsigned)a.parts);
    SL_CUDA_OK(sl::launch_kernel(lru_update_kernel, grid, dim3(LT), smem, static_cast<cudaStream_t>(stream), false, a));
    if (a.g_pairs && !deferred && phase != 1) {
        const int cp = std::max(1, std::min(32, sl::sm_count() / std::max(1, B * KH)));
        SL_CUDA_OK(sl::launch_kernel(lru_copy_kernel, dim3((unsigned)cp, (unsigned)KH, (unsigned)B), dim3(CT), 0,
                                     static_cast<cudaStream_t>(stream), false, a));
    }
    return SL_OK;
}

}  // namespace

extern "C" size_t sl_lru_workspace_bytes(int B, int KH, int idx_capacity) {
    if (B <= 0 || KH <= 0 || idx_capacity <= 0) return 0;
    const size_t nw = ((size_t)idx_capacity + 31) / 32;
    // counters, misses per pair, miss bitmaps, {key, slot} pairs of the misses
    const size_t bh = (size_t)B * KH;
    return ((((size_t)B * KH * 2 + 63) / 64) * 64 + (((size_t)B * KH + 63) / 64) * 64 + (((size_t)B * KH * nw + 3) / 4) * 4) * 4 +
           (size_t)B * KH * idx_capacity * 8 +
           // histogram of ages, barrier counters, per-part counts ({older, ties}, misses; at most 64 parts), victims
           (((bh * NBIN + 3) / 4) * 4 + bh * 8) * 4 + bh * 64 * 8 + bh * 64 * 4 + bh * (size_t)idx_capacity * 4;
}

extern "C" int sl_lru_update(const int32_t* d_idx, int idx_capacity, const int32_t* d_cnt, int B, int KH,
                             const void* k_backing, const void* v_backing, int64_t backing_batch_stride, int elem_bytes,
                             void* d_k_resident, void* d_v_resident, int C, int32_t* d_tok2slot, int64_t n_max,
                             int32_t* d_slot2tok, int32_t* d_last_used, int step, int32_t* d_slots_out,
                             int32_t* d_stats, int32_t* d_status, void* stream) {
    const sl_kv_layout back = {backing_batch_stride, (int64_t)KH * 128, 128, 1};
    const sl_kv_layout res = {(int64_t)C * KH * 128, (int64_t)KH * 128, 128, 1};
    return lru_launch(d_idx, idx_capacity, d_cnt, B, KH, k_backing, v_backing, back, elem_bytes, d_k_resident, d_v_resident,
                      res, C, d_tok2slot, n_max, d_slot2tok, d_last_used, step, nullptr, d_slots_out, d_stats, d_status,
                      nullptr, 0, stream);
}

extern "C" int sl_lru_update_ex(const int32_t* d_idx, int idx_capacity, const int32_t* d_cnt, int B, int KH,
                                const void* k_backing, const void* v_backing, const sl_kv_layout* backing, int elem_bytes,
                                void* d_k_resident, void* d_v_resident, const sl_kv_layout* resident, int C,
                                int32_t* d_tok2slot, int64_t n_max, int32_t* d_slot2tok, int32_t* d_last_used, int step,
                                const int64_t* d_step, int32_t* d_slots_out, int32_t* d_stats, int32_t* d_status,
                                void* d_workspace, size_t workspace_bytes, void* stream) {
    SL_REQUIRE(backing && resident, SL_EINVAL, "sl_lru_update_ex: null cache layout");
    return lru_launch(d_idx, idx_capacity, d_cnt, B, KH, k_backing, v_backing, *backing, elem_bytes, d_k_resident,
                      d_v_resident, *resident, C, d_tok2slot, n_max, d_slot2tok, d_last_used, step, d_step, d_slots_out,
                      d_stats, d_status, d_workspace, workspace_bytes, stream);
}

extern "C" int sl_lru_update_deferred(const int32_t* d_idx, int idx_capacity, const int32_t* d_cnt, int B, int KH, int elem_bytes,
                                      void* d_k_resident, void* d_v_resident, const sl_kv_layout* resident, int C,
                                      int32_t* d_tok2slot, int64_t n_max, int32_t* d_slot2tok, int32_t* d_last_used, int step,
                                      const int64_t* d_step, int32_t* d_slots_out, int32_t* d_stats, int32_t* d_status,
                                      void* d_workspace, size_t workspace_bytes, void* stream) {
    SL_REQUIRE(resident, SL_EINVAL, "sl_lru_update_deferred: null cache layout");
    return lru_launch(d_idx, idx_capacity, d_cnt, B, KH, nullptr, nullptr, *resident, elem_bytes, d_k_resident, d_v_resident,
                      *resident, C, d_tok2slot, n_max, d_slot2tok, d_last_used, step, d_step, d_slots_out, d_stats, d_status,
                      d_workspace, workspace_bytes, stream, true);
}

extern "C" int sl_lru_probe(const int32_t* d_idx, int idx_capacity, const int32_t* d_cnt, int B, int KH, int elem_bytes,
                            void* d_k_resident, void* d_v_resident, const sl_kv_layout* resident, int C, int32_t* d_tok2slot,
                            int64_t n_max, int32_t* d_slot2tok, int32_t* d_last_used, int step, const int64_t* d_step,
                            int32_t* d_slots_out, int32_t* d_status, void* d_workspace, size_t workspace_bytes, void* stream) {
    SL_REQUIRE(resident, SL_EINVAL, "sl_lru_probe: null cache layout");
    return lru_launch(d_idx, idx_capacity, d_cnt, B, KH, nullptr, nullptr, *resident, elem_bytes, d_k_resident, d_v_resident,
                      *resident, C, d_tok2slot, n_max, d_slot2tok, d_last_used, step, d_step, d_slots_out, nullptr, d_status,
                      d_workspace, workspace_bytes, stream, false, 1);
}

extern "C" int sl_lru_evict(const int32_t* d_idx, int idx_capacity, const int32_t* d_cnt, int B, int KH, const void* k_backing,
                            const void* v_backing, const sl_kv_layout* backing, int elem_bytes, void* d_k_resident,
                            void* d_v_resident, const sl_kv_layout* resident, int C, int32_t* d_tok2slot, int64_t n_max,
                            int32_t* d_slot2tok, int32_t* d_last_used, int step, const int64_t* d_step, int32_t* d_slots_scratch,
                            int32_t* d_stats, int32_t* d_status, void* d_workspace, size_t workspace_bytes, void* stream) {
    SL_REQUIRE(backing && resident, SL_EINVAL, "sl_lru_evict: null cache layout");
    return lru_launch(d_idx, idx_capacity, d_cnt, B, KH, k_backing, v_backing, *backing, elem_bytes, d_k_resident, d_v_resident,
                      *resident, C, d_tok2slot, n_max, d_slot2tok, d_last_used, step, d_step, d_slots_scratch, d_stats, d_status,
                      d_workspace, workspace_bytes, stream, false, 2);
}

namespace sl { void set_lru_multi(int v) { g_lru_multi = v ? 1 : 0; } }
