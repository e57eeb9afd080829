// Bit-sliced Hamming score of one 128-bit key code against the G query codes of a group.
#pragma once
#include "sl_common.cuh"

namespace {

// ---- bit-sliced group score -----------------------------------------------------------
// POPC issues at a quarter of the integer rate, and the direct score needs 4*G of them per
// key. Instead: per bit position b let cq_b = #{g : q_g has bit b set}. A key bit k_b = 1
// matches a_b = cq_b query heads, k_b = 0 matches n_b = G - cq_b. The part both cases share,
// min(a_b, n_b), is summed once per head into a base; what is left is a_b - min or n_b - min,
// one of them zero, the other |2 cq_b - G| -- even when G is even, so it is halved then (sh = 1).
// With M_j / M'_j the bit planes of the two remainders (P = bits(G odd ? G : G/2) planes),
// X_{j,w} = select(k_w, M_{j,w}, M'_{j,w}) has weight 2^j and
//   score = base + (sum_j 2^j sum_w popc(X_{j,w})) << sh.
// The 4*P words are added vertically with carry-save adders (LOP3), leaving one word per power
// of two: P + 2 popcounts per key. G = 4 needs 2 planes, G = 7 three, G = 8 three.
// Every step below is ONE three-input logic instruction, written as lop3 so that the compiler
// cannot split it: select (k ? m : m'), the sum bit of a full adder (a ^ b ^ c) and its carry
// (majority). The truth tables are the values of the expression for a = 0xF0, b = 0xCC, c = 0xAA.
__device__ __forceinline__ uint32_t lop3_select(uint32_t k, uint32_t m, uint32_t mp) {
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0xCA;" : "=r"(r) : "r"(k), "r"(m), "r"(mp));
    return r;
}
__device__ __forceinline__ uint32_t lop3_xor3(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0x96;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
    return r;
}
__device__ __forceinline__ uint32_t lop3_maj(uint32_t a, uint32_t b, uint32_t c) {
    uint32_t r;
    asm("lop3.b32 %0, %1, %2, %3, 0xE8;" : "=r"(r) : "r"(a), "r"(b), "r"(c));
    return r;
}
#define SL_FA(a, b, c, s, cy) { s = lop3_xor3(a, b, c); cy = lop3_maj(a, b, c); }
#define SL_HA(a, b, s, cy) { s = (a) ^ (b); cy = (a) & (b); }

// sum_j 2^j sum_w popc(select(k_w, M_{j,w}, M'_{j,w})): the caller adds the base and shifts.
template <int P>
__device__ __forceinline__ int sliced_score(const uint4 k, const uint32_t (&M)[P][4], const uint32_t (&Mp)[P][4]) {
    const uint32_t kw[4] = {k.x, k.y, k.z, k.w};
    uint32_t X[P][4];
#pragma unroll
    for (int j = 0; j < P; ++j)
#pragma unroll
        for (int w = 0; w < 4; ++w) X[j][w] = lop3_select(kw[w], M[j][w], Mp[j][w]);
    uint32_t s1, c1, c2, L0;
    SL_FA(X[0][0], X[0][1], X[0][2], s1, c1)
    SL_HA(s1, X[0][3], L0, c2)
    const int p0 = __popc(L0);
    if constexpr (P == 1) {
        uint32_t L1, L2;
        SL_HA(c1, c2, L1, L2)
        return p0 + 2 * (__popc(L1) + 2 * __popc(L2));
    } else {
        uint32_t s, sp, d1, d2, d3, L1;
        SL_FA(X[1][0], X[1][1], X[1][2], s, d1)
        SL_FA(X[1][3], c1, c2, sp, d2)
        SL_HA(s, sp, L1, d3)
        const int p1 = __popc(L1);
        if constexpr (P == 2) {
            uint32_t L2, L3;
            SL_FA(d1, d2, d3, L2, L3)
            return p0 + 2 * (p1 + 2 * (__popc(L2) + 2 * __popc(L3)));
        } else {
            uint32_t e1, e2, e3, L2;
            SL_FA(X[2][0], X[2][1], X[2][2], s, e1)
            SL_FA(X[2][3], d1, d2, sp, e2)
            SL_FA(s, sp, d3, L2, e3)
            const int p2 = __popc(L2);
            if constexpr (P == 3) {
                uint32_t L3, L4;
                SL_FA(e1, e2, e3, L3, L4)
                return p0 + 2 * (p1 + 2 * (p2 + 2 * (__popc(L3) + 2 * __popc(L4))));
            } else {
                uint32_t f1, f2, f3, L3, L4, L5;
                SL_FA(X[3][0], X[3][1], X[3][2], s, f1)
                SL_FA(X[3][3], e1, e2, sp, f2)
                SL_FA(s, sp, e3, L3, f3)
                SL_FA(f1, f2, f3, L4, L5)
                return p0 + 2 * (p1 + 2 * (p2 + 2 * (__popc(L3) + 2 * (__popc(L4) + 2 * __popc(L5)))));
            }
        }
    }
}


// Planes needed for a group of G query heads; 0 = more than the scorer is instantiated for.
__host__ __device__ inline int sliced_planes(int G) {
    int v = (G & 1) ? G : (G >> 1), p = 0;
    while (v) { ++p; v >>= 1; }
    return p <= 4 ? p : 0;
}
__host__ __device__ inline int sliced_shift(int G) { return (G & 1) ? 0 : 1; }

// Planes of one (head, word), built by a whole warp with lane = bit position; cq = number of
// query heads of the group with that bit set. m[j] / mp[j] are valid in every lane, `base` is
// this word's share of the head's base score.
template <int P>
__device__ __forceinline__ void build_planes(int cq, int G, unsigned (&m)[P], unsigned (&mp)[P], int& base) {
    const int n = G - cq, mn = min(cq, n), sh = sliced_shift(G);
    const int va = (cq - mn) >> sh, vn = (n - mn) >> sh;
#pragma unroll
    for (int j = 0; j < P; ++j) {
        m[j] = __ballot_sync(0xffffffffu, (va >> j) & 1);
        mp[j] = __ballot_sync(0xffffffffu, (vn >> j) & 1);
    }
    base = __reduce_add_sync(0xffffffffu, mn);
}

// All planes of one batch row into shared memory: planes [KH][2][P][4], pbase [KH][4]; one
// warp per (head, word). Lane g loads the word of query head g (G <= 32), so a warp's loads for
// two tasks are all in flight together: one trip to memory per pair of tasks. Split in two so
// that a caller can put other loads between the issue and the use.
struct PlaneWords { uint32_t v[2]; };

__device__ __forceinline__ PlaneWords planes_issue(const uint32_t* __restrict__ qb, int KH, int G, int layout,
                                                   int hw0, int nwarps, int lane) {
    PlaneWords r = {{0u, 0u}};
#pragma unroll
    for (int t = 0; t < 2; ++t) {
        const int hw = hw0 + t * nwarps;
        if (hw < KH * 4 && lane < G) {
            const int h = hw >> 2;
            const int qh = layout == SL_GQA_INTERLEAVED ? lane * KH + h : h * G + lane;
            r.v[t] = __ldcg(qb + qh * 4 + (hw & 3));
        }
    }
    return r;
}

template <int P>
__device__ __forceinline__ void planes_finish(const PlaneWords& r, int KH, int G, uint32_t* planes, int* pbase,
                                              int hw0, int nwarps, int lane) {
#pragma unroll
    for (int t = 0; t < 2; ++t) {
        const int hw = hw0 + t * nwarps;
        if (hw >= KH * 4) break;                             // warp-uniform
        const int h = hw >> 2, w = hw & 3;
        int cq = 0;
        for (int g = 0; g < G; ++g) cq += (__shfl_sync(0xffffffffu, r.v[t], g) >> lane) & 1u;
        unsigned m[P], mp[P];
        int base;
        build_planes<P>(cq, G, m, mp, base);
        if (lane == 0) {
#pragma unroll
            for (int j = 0; j < P; ++j) {
                planes[((h * 2 + 0) * P + j) * 4 + w] = m[j];
                planes[((h * 2 + 1) * P + j) * 4 + w] = mp[j];
            }
            pbase[h * 4 + w] = base;
        }
    }
}

template <int P>
__device__ __forceinline__ void stage_planes(const uint32_t* __restrict__ qb, int KH, int G, int layout,
                                             uint32_t* planes, int* pbase, int warp, int nwarps, int lane,
                                             int first = 0) {
    for (int hw0 = warp + first * 2 * nwarps; hw0 < KH * 4; hw0 += 2 * nwarps) {
        const PlaneWords r = planes_issue(qb, KH, G, layout, hw0, nwarps, lane);
        planes_finish<P>(r, KH, G, planes, pbase, hw0, nwarps, lane);
    }
}

// The calling thread's copy of one head's planes and base (after a barrier behind stage_planes).
template <int P>
__device__ __forceinline__ int load_planes(const uint32_t* planes, const int* pbase, int h, uint32_t (&M)[P][4],
                                           uint32_t (&Mp)[P][4]) {
#pragma unroll
    for (int j = 0; j < P; ++j) {
        const uint4 a = *reinterpret_cast<const uint4*>(planes + ((h * 2 + 0) * P + j) * 4);
        const uint4 c = *reinterpret_cast<const uint4*>(planes + ((h * 2 + 1) * P + j) * 4);
        M[j][0] = a.x; M[j][1] = a.y; M[j][2] = a.z; M[j][3] = a.w;
        Mp[j][0] = c.x; Mp[j][1] = c.y; Mp[j][2] = c.z; Mp[j][3] = c.w;
    }
    const int4 pb = *reinterpret_cast<const int4*>(pbase + h * 4);
    return pb.x + pb.y + pb.z + pb.w;
}

}  // namespace
