// Shared between the scan + top-k translation units (sl_scan_topk.cu: every mode and shape;
// sl_scan_lean.cu: the one-barrier kernel of the decode step; sl_scan_fused.cu: its predecessor).
#pragma once
#include "sl_common.cuh"

namespace slscan {

constexpr int NT = 512;            // threads per CTA
constexpr int NW = NT / 32;
constexpr int U = 8;               // 16-byte loads in flight per thread
constexpr int NCOPY = 4;           // copies of the global histograms in the workspace
constexpr int SHARD_EPOCH_WORD = 2040;   // the flag area of an exchange buffer is 8 KB: [R][B] flags, the epoch of batch row b at this word - b

struct FusedArgs {
    const uint4* q;            // [B,QH] codes
    const uint4* k;            // code stream
    long long k_bstride;       // batch stride in codes
    int B, KH, G, layout, N;
    int k_budget;
    int s_end, r_start;        // forced ranges: [0,s_end) and [r_start,N)
    int* idx;
    int cap;
    int* cnt;
    short* scores_out;         // optional [B,N,KH]
    unsigned* hist;            // fine global histogram [NCOPY,B,KH,nbins]
    unsigned* chist;           // coarse global histogram [NCOPY,B,KH,NC]
    unsigned long long* seg;   // [B,KH,ctas_per_b] flagged counts
    unsigned* sync;            // [B,2]
    int* status;
    int ctas_per_b, chunk, nbins, S;
    int cws;                   // log2 of the coarse bin width: NC = ((nbins - 1) >> cws) + 1 <= 32
    int rowh;                  // row stride of the score rows in shared memory (halfwords)
    int score_off;             // byte offset of the score rows in shared memory
    int trip_off, trips_per_warp;   // per-warp trip records ({flags, flags, counts below, totals} per lane): byte offset, records per warp
    unsigned long long* dbg;   // optional [grid][16] phase stamps (development aid)
    // sequence shards (R > 0): N, s_end, r_start, idx are local to this rank's keys; the merged local
    // histograms travel to every rank's exchange buffer and the threshold comes from all R of them
    unsigned char* peer[8];    // exchange buffer of every rank: [R slots][flags [R][B] ... epoch]
    int R, rank;
    unsigned long long slot_stride, pflags_off;
    int kk;                    // min(k, global number of keys)
};

// ---- the one-barrier kernel of the decode step (sl_scan_lean.cu) ----
constexpr int LEAN_CWS = 3;        // log2 of the coarse bin width: 8 scores
constexpr int LEAN_MAX_WIN = 96;   // always-kept keys (sink + recent) it handles, three per lane
constexpr int LEAN_CPL_MAX = 5;    // chunks per lane in the trip for the chunks' counts; coarse bins per lane

struct LeanArgs {
    const uint4* q;            // [B,QH] codes
    const uint4* k;            // code stream
    long long k_bstride;       // batch stride in codes
    int B, KH, G, layout, N;
    int k_budget;
    int s_end, r_start;        // forced ranges: [0,s_end) and [r_start,N)
    int* idx;
    int cap;
    int* cnt;
    short* scores_out;         // optional [B,N,KH]
    unsigned* sync;            // [B,2] barrier arrivals, finished CTAs
    unsigned* epoch;           // [B] launches completed on this workspace (parity picks the coarse buffer)
    unsigned* chist;           // [2][B][KH][NC] coarse histograms (one per launch parity)
    uint4* pub;                // [B][KH][NC][ctas_per_b] every chunk's counts of each coarse bin's 8 scores, 16 bits each
    unsigned short* puba;      // [B][KH][NC][ctas_per_b] every chunk's keys above each coarse bin
    unsigned nc_magic;         // ceil(2^32 / NC): i / NC == __umulhi(i, nc_magic) for i < 2^16
    unsigned short* wsc;       // [B][KH][LEAN_MAX_WIN] scores of the always-kept keys
    int* status;
    int ctas_per_b, chunk, nbins, S;
    int NC;                    // coarse bins per head
    int rowh;                  // row stride of the score rows in shared memory (halfwords)
    int hist_off, score_off;   // byte offsets of the histogram rows and of the score rows in shared memory
    // context length on the device (optional): N above is then the capacity the launch is planned for
    const long long* d_pos;    // position of the decode token: the context is *d_pos + 1 keys
    int sink, recent, min_remain;
    double mask_out;
    // sequence shards (R > 0): N, s_end, r_start and the indices written are local to this rank's keys; the rank's
    // counts travel to every rank's exchange buffer and the threshold comes from all R of them
    unsigned char* peer[8];    // exchange buffer of every rank: [R slots][arrival counter per row ... epoch per row]
    int R, rank;
    unsigned long long slot_stride, pflags_off;
    int kk;                    // min(k, global number of keys)
    unsigned long long* dbg;   // optional [grid][16] phase stamps (profiling builds only)
};

bool lean_covers(int KH, int G, int ctas_per_b, int chunk, int nwin);
int lean_nc(int nbins);
size_t lean_plan_smem(LeanArgs& f, int KH, int nbins, int S, int chunk);   // fills the offsets, returns the total
int launch_lean(const LeanArgs& a, size_t smem, cudaStream_t s);
size_t lean_shard_message_bytes(int B, int KH, int nbins);   // one rank's message to every rank, padded to 16 bytes

bool fused_covers(int KH, int G);
size_t fused_fixed_smem(int KH, int nbins, int S);
int launch_fused(const FusedArgs& a, size_t smem, cudaStream_t s);
size_t fused_plan_smem(FusedArgs& f, int KH, int nbins, int S, int chunk);   // fills the shared-memory offsets, returns the total
size_t shard_message_bytes(int B, int KH, int nbins, int cws);   // one rank's histogram message, padded to 16 bytes
// Phase stamps exist only in profiling builds (-DSL_SCAN_TIMING): thread 0 of every CTA stores the SM
// cycle counter at its phase boundaries into the buffer given to sl_profile_scan_timing.
#ifdef SL_SCAN_TIMING
extern unsigned long long* g_dbg_timing;
#define SL_STAMP(i) if (a.dbg && threadIdx.x == 0) a.dbg[blockIdx.x * 16 + (i)] = (unsigned long long)clock64();
#define SL_STAMP_BUF slscan::g_dbg_timing
#else
#define SL_STAMP(i)
#define SL_STAMP_BUF nullptr
#endif

__device__ __forceinline__ void touch(const void* p) {   // warms the TLB for a page used later
    unsigned v;
    asm volatile("ld.global.cg.u32 %0, [%1];" : "=r"(v) : "l"(p));
}
__device__ __forceinline__ void st_relaxed_u64(unsigned long long* p, unsigned long long v) {
    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(v) : "memory");
}
__device__ __forceinline__ unsigned long long ld_relaxed_u64(const unsigned long long* p) {
    unsigned long long v;
    asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(v) : "l"(p) : "memory");
    return v;
}
// sum over this lane and the lanes above it
__device__ __forceinline__ unsigned suffix_sum(unsigned v, int lane) {
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const unsigned t = __shfl_down_sync(0xffffffffu, v, d);
        if (lane + d < 32) v += t;
    }
    return v;
}
// sum over this lane and the lanes below it
__device__ __forceinline__ int prefix_sum(int v, int lane) {
#pragma unroll
    for (int d = 1; d < 32; d <<= 1) {
        const int t = __shfl_up_sync(0xffffffffu, v, d);
        if (lane >= d) v += t;
    }
    return v;
}
// bit 15 of each halfword of (vlo, vhi) says whether keys tl .. tl+3 lie inside [elo, ehi)
static __device__ __noinline__ void edge_masks(int tl, int elo, int ehi, unsigned& vlo, unsigned& vhi) {
    vlo = ((tl >= elo && tl < ehi) ? 0x8000u : 0u) | ((tl + 1 >= elo && tl + 1 < ehi) ? 0x80000000u : 0u);
    vhi = ((tl + 2 >= elo && tl + 2 < ehi) ? 0x8000u : 0u) | ((tl + 3 >= elo && tl + 3 < ehi) ? 0x80000000u : 0u);
}
// bits 15 / 31 of lo and hi -> bits 0..3
__device__ __forceinline__ unsigned flags4(unsigned lo, unsigned hi) {
    return ((lo >> 15) & 1u) | ((lo >> 30) & 2u) | ((hi >> 13) & 4u) | ((hi >> 28) & 8u);
}

}  // namespace slscan
