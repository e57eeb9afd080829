// Bit-sliced Hamming score of one 128-bit key code against the G query codes of a group.
#pragma once
#include "sl_common.cuh"

namespace {

// ---- bit-sliced group score -----------------------------------------------------------
// POPC issues at a quarter of the integer rate, and the direct score needs 4*G of them per
// key. Instead: per bit position b let cq_b = #{g : q_g has bit b set}. A key bit k_b = 1
// matches cq_b query heads, k_b = 0 matches G - cq_b. With M_j / M'_j the bit planes of cq and
// G - cq (P = bits(G) planes), X_{j,w} = select(k_w, M_{j,w}, M'_{j,w}) has weight 2^j and
//   score = sum_j 2^j sum_w popc(X_{j,w}).
// The 4*P words are added vertically with carry-save adders (LOP3 at full rate), leaving one
// word per power of two: P + 2 popcounts per key whatever G is.
#define SL_FA(a, b, c, s, cy) { const uint32_t t_ = (a) ^ (b); s = t_ ^ (c); cy = ((a) & (b)) | ((c) & t_); }
#define SL_HA(a, b, s, cy) { s = (a) ^ (b); cy = (a) & (b); }

template <int P>
__device__ __forceinline__ int sliced_score(const uint4 k, const uint32_t (&M)[P][4], const uint32_t (&Mp)[P][4]) {
    const uint32_t kw[4] = {k.x, k.y, k.z, k.w};
    uint32_t X[P][4];
#pragma unroll
    for (int j = 0; j < P; ++j)
#pragma unroll
        for (int w = 0; w < 4; ++w) X[j][w] = (kw[w] & M[j][w]) | (~kw[w] & Mp[j][w]);
    uint32_t s1, c1, c2, L0;
    SL_FA(X[0][0], X[0][1], X[0][2], s1, c1)
    SL_HA(s1, X[0][3], L0, c2)
    int score = __popc(L0);
    if constexpr (P == 1) {
        uint32_t L1, L2;
        SL_HA(c1, c2, L1, L2)
        score += 2 * __popc(L1) + 4 * __popc(L2);
    } else {
        uint32_t s, sp, d1, d2, d3, L1;
        SL_FA(X[1][0], X[1][1], X[1][2], s, d1)
        SL_FA(X[1][3], c1, c2, sp, d2)
        SL_HA(s, sp, L1, d3)
        score += 2 * __popc(L1);
        if constexpr (P == 2) {
            uint32_t L2, L3;
            SL_FA(d1, d2, d3, L2, L3)
            score += 4 * __popc(L2) + 8 * __popc(L3);
        } else {
            uint32_t e1, e2, e3, L2;
            SL_FA(X[2][0], X[2][1], X[2][2], s, e1)
            SL_FA(X[2][3], d1, d2, sp, e2)
            SL_FA(s, sp, d3, L2, e3)
            score += 4 * __popc(L2);
            if constexpr (P == 3) {
                uint32_t L3, L4;
                SL_FA(e1, e2, e3, L3, L4)
                score += 8 * __popc(L3) + 16 * __popc(L4);
            } else {
                uint32_t f1, f2, f3, L3, L4, L5;
                SL_FA(X[3][0], X[3][1], X[3][2], s, f1)
                SL_FA(X[3][3], e1, e2, sp, f2)
                SL_FA(s, sp, e3, L3, f3)
                SL_FA(f1, f2, f3, L4, L5)
                score += 8 * __popc(L3) + 16 * __popc(L4) + 32 * __popc(L5);
            }
        }
    }
    return score;
}


// Bit planes of cq (number of query heads with the bit set) and of G - cq for one (head, word):
// called by a whole warp, lane = bit position; m[j] / mp[j] are valid in every lane.
template <int P>
__device__ __forceinline__ void build_planes(int cq, int G, unsigned (&m)[P], unsigned (&mp)[P]) {
    const int cn = G - cq;
#pragma unroll
    for (int j = 0; j < P; ++j) {
        m[j] = __ballot_sync(0xffffffffu, (cq >> j) & 1);
        mp[j] = __ballot_sync(0xffffffffu, (cn >> j) & 1);
    }
}

}  // namespace
