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
// One CTA of 1024 threads per (b, kv head); victim selection is a histogram select over ages
// (no sort), ordered compaction by warp ballots.
#include "sl_common.cuh"

namespace {

constexpr int LT = 1024;
constexpr int LW = LT / 32;
constexpr int AGE_MAX = 1023;           // ages are clamped here; free slots count as AGE_MAX + 1
constexpr int NBIN = AGE_MAX + 2;

struct LruArgs {
    const int* idx; int cap; const int* cnt;
    int B, KH, C, step, row_bytes;
    const unsigned char* k_back; const unsigned char* v_back; long long back_bstride;   // bytes
    unsigned char* k_res; unsigned char* v_res;
    int* tok2slot; long long n_max; int* slot2tok; int* last_used;
    int* slots_out; int* stats; int* status;
};

// exclusive ranks of two flags over the block, in thread order; totals returned through tot0/tot1
__device__ __forceinline__ void block_rank2(bool f0, bool f1, int (*wt)[2], int& r0, int& r1, int& tot0, int& tot1) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const unsigned lt = (1u << lane) - 1u;
    const unsigned b0 = __ballot_sync(0xffffffffu, f0), b1 = __ballot_sync(0xffffffffu, f1);
    if (lane == 0) { wt[warp][0] = __popc(b0); wt[warp][1] = __popc(b1); }
    __syncthreads();
    int p0 = 0, p1 = 0, t0 = 0, t1 = 0;
    for (int w = 0; w < LW; ++w) {
        const int a0 = wt[w][0], a1 = wt[w][1];
        if (w < warp) { p0 += a0; p1 += a1; }
        t0 += a0; t1 += a1;
    }
    r0 = p0 + __popc(b0 & lt);
    r1 = p1 + __popc(b1 & lt);
    tot0 = t0; tot1 = t1;
    __syncthreads();
}

__global__ void __launch_bounds__(LT) lru_update_kernel(const LruArgs a) {
    extern __shared__ int smem_i[];
    int* victims = smem_i;                 // [cap] slot taken by the r-th miss
    int* misstok = smem_i + a.cap;         // [cap] key of the r-th miss
    __shared__ unsigned hist[NBIN];
    __shared__ int wt[LW][2];
    __shared__ int s_hits, s_tau, s_r;

    const int h = blockIdx.x, b = blockIdx.y, tid = threadIdx.x, lane = tid & 31;
    const long long bh = (long long)b * a.KH + h;
    const int n = min(a.cnt[bh], a.cap);
    const int* list = a.idx + bh * a.cap;
    int* out = a.slots_out + bh * a.cap;
    int* t2s = a.tok2slot + bh * a.n_max;
    int* s2t = a.slot2tok + bh * a.C;
    int* lu = a.last_used + bh * a.C;
    const int t = a.step;

    if (tid == 0) s_hits = 0;
    for (int i = tid; i < NBIN; i += LT) hist[i] = 0;
    __syncthreads();
    if (n > a.C) {                          // the table cannot hold this step's attended set
        if (tid == 0 && a.status) atomicExch(a.status, 3);
        return;
    }

    // ---- hits: stamp their slots
    int myhits = 0;
    for (int j = tid; j < n; j += LT) {
        const int s = t2s[list[j]];
        if (s >= 0) { lu[s] = t; ++myhits; }
        out[j] = s;
    }
    myhits = __reduce_add_sync(0xffffffffu, myhits);
    if (lane == 0 && myhits) atomicAdd(&s_hits, myhits);
    __syncthreads();
    const int m = n - s_hits;              // misses = victims needed

    // ---- age histogram of the slots not used in this step
    for (int s = tid; s < a.C; s += LT) {
        const int l = lu[s];
        const int age = l < 0 ? AGE_MAX + 1 : min(t - l, AGE_MAX);
        if (age > 0) atomicAdd(&hist[age], 1u);
    }
    __syncthreads();
    if (tid < 32) {                         // oldest first: largest age with a cumulative count >= m
        int tau = NBIN, r = 0;
        if (m > 0) {
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
        }
        if (lane == 0) { s_tau = tau; s_r = r; }
    }
    __syncthreads();
    const int tau = s_tau, r = s_r;

    // ---- victims in slot order: every slot older than tau, then the first r slots of age tau
    int gt_before = 0, eq_before = 0;
    for (int s0 = 0; s0 < a.C && m > 0; s0 += LT) {
        const int s = s0 + tid;
        int age = 0;
        if (s < a.C) {
            const int l = lu[s];
            age = l < 0 ? AGE_MAX + 1 : min(t - l, AGE_MAX);
        }
        const bool isgt = age > tau, iseq = age == tau && age > 0;
        int rg, re, tg, te;
        block_rank2(isgt, iseq, wt, rg, re, tg, te);
        const int eqr = eq_before + re;
        if (isgt || (iseq && eqr < r)) victims[gt_before + rg + min(eqr, r)] = s;
        gt_before += tg;
        eq_before += te;
    }
    __syncthreads();

    // ---- misses in list order take the victims in that order
    int miss_before = 0;
    for (int j0 = 0; j0 < n && m > 0; j0 += LT) {
        const int j = j0 + tid;
        const bool miss = j < n && out[j] < 0;
        int rm, dummy, tm, td;
        block_rank2(miss, false, wt, rm, dummy, tm, td);
        if (miss) {
            const int rank = miss_before + rm;
            const int v = victims[rank], tok = list[j];
            const int old = s2t[v];
            if (old >= 0) t2s[old] = -1;
            t2s[tok] = v;
            s2t[v] = tok;
            lu[v] = t;
            out[j] = v;
            misstok[rank] = tok;
        }
        miss_before += tm;
    }
    __syncthreads();

    // ---- copy the missing rows from the backing store into their slots (16-byte lanes)
    const int lanes = a.row_bytes >> 4;                 // 16 (2-byte types) or 32 (4-byte types)
    const int groups = LT / lanes, grp = tid / lanes, c = tid % lanes;
    const long long row_stride = (long long)a.KH * a.row_bytes;
    const unsigned char* kb = a.k_back + b * a.back_bstride + (long long)h * a.row_bytes + c * 16;
    const unsigned char* vb = a.v_back + b * a.back_bstride + (long long)h * a.row_bytes + c * 16;
    unsigned char* kr = a.k_res + ((long long)b * a.C * a.KH + h) * a.row_bytes + c * 16;
    unsigned char* vr = a.v_res + ((long long)b * a.C * a.KH + h) * a.row_bytes + c * 16;
    for (int i = grp; i < m; i += groups) {
        const long long src = (long long)misstok[i] * row_stride, dst = (long long)victims[i] * row_stride;
        const uint4 kv = *reinterpret_cast<const uint4*>(kb + src);
        const uint4 vv = *reinterpret_cast<const uint4*>(vb + src);
        *reinterpret_cast<uint4*>(kr + dst) = kv;
        *reinterpret_cast<uint4*>(vr + dst) = vv;
    }
    if (tid == 0 && a.stats) { a.stats[bh * 2] = s_hits; a.stats[bh * 2 + 1] = m; }
}

}  // namespace

extern "C" int sl_lru_update(const int32_t* d_idx, int idx_capacity, const int32_t* d_cnt, int B, int KH,
                             const void* k_backing, const void* v_backing, int64_t backing_batch_stride, int elem_bytes,
                             void* d_k_resident, void* d_v_resident, int C, int32_t* d_tok2slot, int64_t n_max,
                             int32_t* d_slot2tok, int32_t* d_last_used, int step, int32_t* d_slots_out,
                             int32_t* d_stats, int32_t* d_status, void* stream) {
    SL_REQUIRE(d_idx && d_cnt && k_backing && v_backing && d_k_resident && d_v_resident && d_tok2slot && d_slot2tok &&
                   d_last_used && d_slots_out,
               SL_EINVAL, "sl_lru_update: null pointer");
    SL_REQUIRE(B > 0 && B <= 65535 && KH > 0 && C > 0 && idx_capacity > 0 && n_max > 0 && step >= 0, SL_ESHAPE,
               "sl_lru_update: bad shape");
    SL_REQUIRE(elem_bytes == 2 || elem_bytes == 4, SL_EINVAL, "sl_lru_update: elem_bytes must be 2 or 4");
    SL_REQUIRE(sl::aligned16(k_backing) && sl::aligned16(v_backing) && sl::aligned16(d_k_resident) &&
                   sl::aligned16(d_v_resident) && (backing_batch_stride * elem_bytes) % 16 == 0,
               SL_EALIGN, "sl_lru_update: K/V buffers must be 16-byte aligned");
    const size_t smem = (size_t)idx_capacity * 2 * sizeof(int);
    SL_REQUIRE(smem <= 200 * 1024, SL_ESHAPE, "sl_lru_update: idx_capacity %d too large for the shared-memory victim list",
               idx_capacity);
    LruArgs a;
    a.idx = d_idx; a.cap = idx_capacity; a.cnt = d_cnt;
    a.B = B; a.KH = KH; a.C = C; a.step = step; a.row_bytes = 128 * elem_bytes;
    a.k_back = static_cast<const unsigned char*>(k_backing); a.v_back = static_cast<const unsigned char*>(v_backing);
    a.back_bstride = backing_batch_stride * elem_bytes;
    a.k_res = static_cast<unsigned char*>(d_k_resident); a.v_res = static_cast<unsigned char*>(d_v_resident);
    a.tok2slot = d_tok2slot; a.n_max = n_max; a.slot2tok = d_slot2tok; a.last_used = d_last_used;
    a.slots_out = d_slots_out; a.stats = d_stats; a.status = d_status;
    SL_CUDA_OK(cudaFuncSetAttribute(lru_update_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    dim3 grid((unsigned)KH, (unsigned)B);
    lru_update_kernel<<<grid, LT, smem, static_cast<cudaStream_t>(stream)>>>(a);
    SL_CUDA_OK(cudaGetLastError());
    return SL_OK;
}
