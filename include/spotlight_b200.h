/*
 * spotlight_b200 -- C ABI of the B200 (sm_100a) decode-time retrieval path of Spotlight Attention.
 *
 * Conventions
 *  - Every pointer named d_* is a DEVICE pointer owned by the caller. The library never
 *    allocates or frees device memory (the one exception is documented at its declaration).
 *  - Every entry point returns SL_OK (0) or a negative sl_status; the message of the last
 *    failure on the calling thread is available from sl_last_error_string(). Nothing throws.
 *  - `stream` is a cudaStream_t passed as void*. All work is enqueued asynchronously on it;
 *    no entry point synchronises with the host.
 *  - Layouts follow the reference's caches (spotlight/modifiers/gpu_cache.py:28-36): token-major
 *    with heads interleaved. Keys/values: [B, N, KH, 128]; codes: [B, N, KH, 4] uint32
 *    (one 128-bit code = 16 contiguous bytes). A batch row may be a slice of a longer
 *    pre-allocated cache, hence the explicit batch strides; a batch stride of 0 on a READ-ONLY
 *    input (codes of sl_hamming_scores / sl_scan_topk, caches of sl_sparse_attn_decode_ex) makes
 *    every batch row read the same data (the reference's spotlight/modifiers/fake_cache.py).
 *  - gqa_layout says which query heads share kv head h (G = QH / KH):
 *      SL_GQA_INTERLEAVED: q heads { g*KH + h }   (the reference kernels,
 *                          spotlight/kernel/attn_k4_q28.cu:75, attn_dx_u32.py:110-113)
 *      SL_GQA_BLOCKED:     q heads { h*G + g }    (HF repeat_kv, spotlight_generation.py:128)
 */
#ifndef SPOTLIGHT_B200_H
#define SPOTLIGHT_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
    SL_OK = 0,
    SL_EINVAL = -1,     /* null pointer, negative size, unknown enum            */
    SL_ESHAPE = -2,     /* shape outside what the kernels are built for         */
    SL_EALIGN = -3,     /* pointer or stride not 16-byte aligned                */
    SL_EWORKSPACE = -4, /* workspace too small                                  */
    SL_ECUDA = -5,      /* a CUDA runtime call failed                           */
    SL_ETIMEOUT = -6    /* a bounded device-side wait ran out (status word set) */
} sl_status;

typedef enum { SL_BF16 = 0, SL_F32 = 1, SL_F16 = 2, SL_BOOL = 3 } sl_dtype;
typedef enum { SL_GQA_INTERLEAVED = 0, SL_GQA_BLOCKED = 1 } sl_gqa_layout;

int sl_version(void);
const char* sl_last_error_string(void);

/* Makes `device` current for the calling thread inside the library's CUDA runtime. Launches go
 * to the current device; callers that juggle several devices call this before the other entry
 * points (the reference sets a DeviceGuard per call, spotlight/kernel/attn_k4_q28.cu:116). */
int sl_set_device(int device);

/* Process-wide switches, for measurements and tests; the defaults are what the decode path is tuned
 * for. Takes effect for launches made after the call. No reference counterpart.
 *   SL_OPT_PDL          1 (default): decode-path kernels are launched with programmatic stream
 *                       serialisation, so a kernel's prologue overlaps its predecessor's tail; 0: plain launches
 *   SL_OPT_L2_PREFETCH  1 (default): sl_decode_prepare asks L2 for the code cache that the
 *                       sl_scan_topk of the same step streams next (caches of at most 24 MB); 0: off
 *   SL_OPT_SCAN_KERNEL  which kernel sl_scan_topk uses where several apply (results are identical):
 *                       1 (default) the one-barrier kernel, 2 the flagged-word kernel, 0 the general kernel
 *   SL_OPT_ATTN_WARPS   warps per CTA of the bf16 attention kernel: 0 (default) by shape, 4 or 8
 *   SL_OPT_PEER_SPIN_LIMIT  polls (100 ns apart) after which the peer-memory exchanges stop waiting for another
 *                       rank's message and set their status word to 3; default 400000, about a second
 *   SL_OPT_HASH_KERNEL  which kernel sl_hash_encode uses for bf16 rows of a 128 -> 256 -> 128 hash: 0 (default)
 *                       by size, 1 the warp-level tensor-core kernel, 2 the tcgen05 / TMEM kernel for every size
 *   SL_OPT_ATTN_CLUSTER 1 (default): the CTAs that share a (batch row, kv head) pair of the bf16 attention kernel form a
 *                       thread-block cluster and combine their partials through distributed shared memory where
 *                       all clusters of the launch fit on the device at once; 0: partials in the workspace and a merge kernel
 *   SL_OPT_LRU_FUSED_FILL  1 (default): sl_decode_step[_dev] with an LRU stage issue sl_lru_update_deferred +
 *                       sl_sparse_attn_decode_fill (bf16); 0: sl_lru_update_ex (which copies the missed rows) + sl_sparse_attn_decode_ex
 *   SL_OPT_LRU_MULTI_CTA  1 (default): with a workspace every CTA of a (batch row, kv head) pair works through the whole table
 *                       update (a cooperative launch, four barriers of the pair); 0: the last CTA of the pair handles the misses alone */
typedef enum { SL_OPT_PDL = 0, SL_OPT_L2_PREFETCH = 1, SL_OPT_SCAN_KERNEL = 2, SL_OPT_ATTN_WARPS = 3,
               SL_OPT_PEER_SPIN_LIMIT = 4, SL_OPT_HASH_KERNEL = 5, SL_OPT_ATTN_CLUSTER = 6, SL_OPT_LRU_FUSED_FILL = 7, SL_OPT_LRU_MULTI_CTA = 8 } sl_option;
int sl_configure(int option, int value);

/* How many thread-block clusters of `cluster_size` CTAs (2..16) of the bf16 attention kernel with `warps_per_cta`
 * (4 or 8) warps the current device holds at once; 0 when it holds none. The attention kernel combines the splits
 * of a (batch row, kv head) pair inside such a cluster when all clusters of a launch fit at once (SL_OPT_ATTN_CLUSTER).
 * No reference counterpart. */
int sl_attn_cluster_capacity(int warps_per_cta, int cluster_size);

/* Status of the prefill hash kernels since the last call: 0, or 3 after a bounded device-side wait (an mbarrier
 * of the tcgen05 kernel) ran out. Reading clears it. Synchronise the streams that ran sl_hash_encode first.
 * No reference counterpart. */
int sl_hash_status(void);

/* Sign-bit packing: bit j of output byte i  <=>  x[8*i + j] > 0 (LSB first). Read as uint32
 * words on a little-endian machine this is the 32-bit packing of the reference.
 * Replaces packbits (spotlight/kernel/packbits.cu:28-63), pack_dx_u32_func
 * (spotlight/kernel/pack_dx_u32.py:35-59) and pack_dx_u8_func (spotlight/kernel/pack_dx_u8.py:34-56).
 * d_x: n_elems contiguous values of `dtype` (n_elems % 8 == 0, 16-byte aligned);
 * d_out: n_elems/8 bytes. */
int sl_pack_signbits(const void* d_x, int dtype, int64_t n_elems, void* d_out, void* stream);

/* Hamming match count, 32-bit code words:
 *   out[b,n,h] = sum_g sum_w popc(~(q[b, qhead(g,h), w] ^ k[b,n,h,w]))     (int16)
 * Replaces attn_k4_q28 (spotlight/kernel/attn_k4_q28.cu:100-138) and attn_dx_u32_func
 * (spotlight/kernel/attn_dx_u32.py:131-162). d_q: [B,QH,W]; d_k: [B,N,KH,W] with batch stride
 * k_batch_stride (in uint32 words); d_out: [B,N,KH] contiguous. W in {1,2,4,8}. */
int sl_hamming_scores(const uint32_t* d_q, const uint32_t* d_k, int64_t k_batch_stride,
                      int16_t* d_out, int B, int64_t N, int KH, int QH, int W, int gqa_layout,
                      void* stream);

/* Hamming match count, 8-bit code words, one score per head (no group sum):
 *   out[r,n] = sum_d popc(~(q[r,d] ^ k[r,n,d])) mod 256, r = b*H + h.
 * Replaces attn_dx_u8_func (spotlight/kernel/attn_dx_u8.py:46-74).
 * d_q: [R,D] uint8; d_k: [R,N,D] uint8; d_out: [R,N] uint8. */
int sl_hamming_scores_u8(const uint8_t* d_q, const uint8_t* d_k, uint8_t* d_out, int64_t R,
                         int64_t N, int D, void* stream);

/* Workspace protocol for the fused scan + top-k. The workspace must be zero-filled once with
 * sl_workspace_init (or cudaMemset) before its first use; every successful call leaves it
 * ready for the next call WITH THE SAME (B, KH, QH): the internal layout depends on those
 * three, so a workspace is bound to one shape (N may change freely) and must be re-initialised
 * before it is used with another. After SL_ETIMEOUT / a non-zero status word it must be
 * re-initialised too. One workspace serves one call at a time (calls on one stream are fine). */
size_t sl_scan_topk_workspace_bytes(int B, int64_t N, int KH, int QH);
int sl_workspace_init(void* d_workspace, size_t bytes, void* stream);

/* Fused Hamming scan + exact top-k + sink/recent window for the decode query.
 * For each (b, kv head h): score every key 0..N-1 as in sl_hamming_scores (W = 4), keep the k
 * highest scores with ties broken by LOWEST index, then add keys [0, min(sink,N)) and
 * [N-recent, N). d_idx[b,h,0..cnt) receives the attended keys in ascending order,
 * d_cnt[b,h] their number (<= min(N, k+sink+recent) <= idx_capacity).
 * Replaces attn_cuda_func (spotlight/kernel/__init__.py:31-40) followed by the top-k of
 * topk_and_gather (spotlight/modifiers/gpu_cache.py:48-50) / aggregate_topk
 * (spotlight/modifiers/spotlight_generation.py:157-165) and the window of
 * spotlight/modifiers/spotlight_evaluation.py:341-346.
 * d_scores_out (optional, may be NULL): int16 [B,N,KH] copy of the scores.
 * d_status: one int32 the kernel sets non-zero if a bounded wait ran out (may be NULL). */
int sl_scan_topk(const uint32_t* d_q_codes, const uint32_t* d_k_codes, int64_t k_batch_stride,
                 int B, int64_t N, int KH, int QH, int gqa_layout, int k, int sink, int recent,
                 int32_t* d_idx, int idx_capacity, int32_t* d_cnt, int16_t* d_scores_out,
                 void* d_workspace, size_t workspace_bytes, int32_t* d_status, void* stream);

/* Exact top-k (lowest-index ties) + sink/recent window from scores that already exist:
 * d_scores int16 [B,N,KH] with values in [0, max_score]. Same output contract as sl_scan_topk.
 * Replaces the `attn.topk(budget, dim=1)` of topk_and_gather
 * (spotlight/modifiers/gpu_cache.py:48-50) when the caller holds attn_cuda_func's scores. */
size_t sl_topk_from_scores_workspace_bytes(int B, int64_t N, int KH, int max_score);
int sl_topk_from_scores(const int16_t* d_scores, int B, int64_t N, int KH, int max_score, int k,
                        int sink, int recent, int32_t* d_idx, int idx_capacity, int32_t* d_cnt,
                        void* d_workspace, size_t workspace_bytes, int32_t* d_status, void* stream);

/* Sequence-sharded selection, step 1: score the local shard (keys [0,N_local) of this rank),
 * write int16 scores [B,N_local,KH] and ADD the local histogram into d_hist [B,KH,nbins]
 * uint32 (nbins = 128*G + 1; the caller zeroes d_hist). No reference counterpart: the
 * reference has no sequence parallelism. */
int sl_scan_hist(const uint32_t* d_q_codes, const uint32_t* d_k_codes, int64_t k_batch_stride,
                 int B, int64_t N_local, int KH, int QH, int gqa_layout, int16_t* d_scores,
                 uint32_t* d_hist, void* stream);

/* Sequence-sharded selection, step 2: given the histograms of ALL ranks
 * d_hist_all [R,B,KH,nbins] (e.g. from an all-gather), derive the global threshold and this
 * rank's share of the threshold ties (lower ranks first = lowest global index first) and emit
 * the LOCAL indices (0-based within the shard) of the attended keys, ascending.
 * tok_offset = global index of local key 0; N_global = total context. The workspace follows
 * the same zero-once protocol as sl_scan_topk's. */
size_t sl_select_emit_workspace_bytes(int B, int64_t N_local, int KH, int QH);
int sl_select_emit(const int16_t* d_scores, const uint32_t* d_hist_all, int R, int rank, int B,
                   int64_t N_local, int64_t tok_offset, int64_t N_global, int KH, int QH, int k,
                   int sink, int recent, int32_t* d_idx, int idx_capacity, int32_t* d_cnt,
                   void* d_workspace, size_t workspace_bytes, int32_t* d_status, void* stream);

/* Geometry of a K or V cache, strides in ELEMENTS:
 *   row of key t, kv head g, batch row b  =  base + b*batch_stride + t*token_stride + g*head_stride.
 * See sl_sparse_attn_decode_ex for the layouts in use. */
typedef struct {
    int64_t batch_stride, token_stride, head_stride;
    int list_heads_per_kv_head;
} sl_kv_layout;

/* Hash parameters of one head set (query heads or key heads): an MLP of n_layers layers,
 * layer i: dx = act(x @ W_i + b_i), act = SiLU for i < n_layers-1 else identity,
 * x = dx + x when residue. n_layers = 1 with no bias is the linear hash.
 * Replaces MLPHashingFunction / MLPLayer (spotlight/modifiers/spotlight_generation.py:229-255)
 * and LinearHashingFunction (spotlight/modifiers/linearhashing_generation.py:224-231).
 * d_w[i]: [H, dims[i], dims[i+1]]; d_b[i]: [H, dims[i+1]] or NULL; all of `dtype`. */
typedef struct {
    int n_layers;          /* 1..3                                   */
    int dims[4];           /* dims[0] = 128, dims[n_layers] = 128    */
    int residue;
    const void* d_w[3];
    const void* d_b[3];
} sl_hash_params;

/* Stage 1 of a decode step, one launch: optional RoPE of q and the new key at the given
 * position, hash + sign + pack of both, append of the new key code / key / value rows to the
 * caches at token `pos`. Rounding follows the reference's operators in `dtype` (each matmul,
 * bias add, SiLU and residual rounds to `dtype`; fp32 accumulation inside a matmul).
 *   d_q [B,QH,128], d_k [B,KH,128], d_v [B,KH,128]  of `dtype` (the decode token)
 *   d_cos, d_sin: [128] of `dtype` for position pos, or NULL when q/k are already rotated
 *   d_q_rot [B,QH,128] (out, may alias d_q)         rotated query for the attention stage
 *   d_q_codes [B,QH,4] (out)
 *   d_code_cache [B,*,KH,4], d_k_cache / d_v_cache [B,*,KH,128] with batch strides in ELEMENTS
 *   (uint32 words resp. values); row `pos` of each is written. Caches may be NULL to skip.
 *   With a code cache of at most 24 MB (rows 0..pos-1 of all batch elements) the launch also asks
 *   L2 for those rows, which the sl_scan_topk of the same decode step streams next.
 * Replaces, for one decode token, check_and_apply_qk_rope (spotlight/modifiers/modify_llama.py:
 * 68-80) + hash_fn + sign (spotlight_generation.py:13-20) + pack_cuda_func
 * (spotlight/kernel/__init__.py:23-24) + KVHash.update / KVCache.update
 * (spotlight/modifiers/gpu_cache.py:38-45,108-118). */
int sl_decode_prepare(const void* d_q, const void* d_k, const void* d_v, int dtype, int B, int QH,
                      int KH, const void* d_cos, const void* d_sin,
                      const sl_hash_params* hash_q, const sl_hash_params* hash_k,
                      void* d_q_rot, uint32_t* d_q_codes, uint32_t* d_code_cache,
                      int64_t code_batch_stride, void* d_k_cache, void* d_v_cache,
                      int64_t kv_batch_stride, int64_t pos, void* stream);
/* The same with the cache geometry spelled out (d_k_cache and d_v_cache share it; list_heads_per_kv_head
 * is not used here): row `pos` of a fused cache [B,N,KH,2,128] is written with d_v_cache = d_k_cache + 128,
 * token_stride = KH*256, head_stride = 256. */
int sl_decode_prepare_ex(const void* d_q, const void* d_k, const void* d_v, int dtype, int B, int QH,
                         int KH, const void* d_cos, const void* d_sin,
                         const sl_hash_params* hash_q, const sl_hash_params* hash_k,
                         void* d_q_rot, uint32_t* d_q_codes, uint32_t* d_code_cache,
                         int64_t code_batch_stride, void* d_k_cache, void* d_v_cache,
                         const sl_kv_layout* kv, int64_t pos, void* stream);

/* Hash + sign + pack of many rows (code-cache build at prefill):
 * d_x [B,T,H,128] with batch stride x_batch_stride (elements) -> d_codes [B,T,H,4] with batch
 * stride code_batch_stride (words). Same rounding as sl_decode_prepare. */
int sl_hash_encode(const void* d_x, int64_t x_batch_stride, int dtype, int B, int64_t T, int H,
                   const sl_hash_params* hash, uint32_t* d_codes, int64_t code_batch_stride,
                   void* stream);
/* The same over rows with explicit token / head strides (elements), e.g. the K rows of a fused cache
 * [B,N,KH,2,128]: x_token_stride = KH*256, x_head_stride = 256. */
int sl_hash_encode_ex(const void* d_x, int64_t x_batch_stride, int64_t x_token_stride, int64_t x_head_stride,
                      int dtype, int B, int64_t T, int H, const sl_hash_params* hash, uint32_t* d_codes,
                      int64_t code_batch_stride, void* stream);

/* Sparse GQA decode attention over the attended keys only:
 *   out[b,qh,:] = softmax_j( q[b,qh] . K[b, idx[b,h,j], h] / sqrt(128) ) V[b, idx[b,h,j], h]
 * with fp32 online softmax; q heads of kv head h per gqa_layout. Rows are gathered straight
 * from the caches; no gathered copy is materialised.
 * Replaces the mask build + dense SDPA of the reference (spotlight/modifiers/
 * spotlight_generation.py:200-215, modify_llama.py:151-186) and the gather of
 * topk_and_gather (spotlight/modifiers/gpu_cache.py:51-54).
 *   d_q [B,QH,128], d_k/d_v caches of `dtype` (bf16 or f32) with batch stride in elements,
 *   d_idx [B,KH,idx_capacity] int32, d_cnt [B,KH] int32,
 *   d_out [B,QH,128] of `dtype`; d_lse (optional) [B,QH] float natural-log-sum-exp of the
 *   scaled logits, for merging partial results of sequence shards.
 * Workspace: sl_sparse_attn_workspace_bytes(B,KH,QH) bytes of scratch for the per-split
 * partials (no initial contents required, nothing is kept between calls). */
size_t sl_sparse_attn_workspace_bytes(int B, int KH, int QH);
int sl_sparse_attn_decode(const void* d_q, const void* d_k, const void* d_v, int dtype,
                          int64_t kv_batch_stride, const int32_t* d_idx, int idx_capacity,
                          const int32_t* d_cnt, int B, int KH, int QH, int gqa_layout,
                          void* d_out, float* d_lse, void* d_workspace, size_t workspace_bytes,
                          void* stream);

/* The same attention with the geometry of the caches spelled out (strides in ELEMENTS):
 * row of key t, kv head g, batch row b  =  base + b*batch_stride + t*token_stride + g*head_stride.
 *  - the reference's two caches [B,N,KH,128] (spotlight/modifiers/gpu_cache.py:28-36):
 *    token_stride = KH*128, head_stride = 128;
 *  - one fused cache [B,N,KH,2,128] with d_v = d_k + 128: token_stride = KH*256, head_stride = 256.
 *    A key's K and V rows are then one 512-byte piece of memory, which is what the gather wants;
 *  - batch_stride = 0 lets every batch row read the same cache (the batch aliasing of
 *    spotlight/modifiers/fake_cache.py:42-49,96-106).
 * list_heads_per_kv_head = 1 is the per-kv-head selection of the reference's kernels. With a value
 * m > 1 the KH index lists of a batch row are taken m at a time per kv head of the caches (list head
 * h reads kv head h / m): KH = QH and m = QH / kv heads gives every QUERY head its own list over
 * shared K/V, the per-query-head selection of the reference's modifier
 * (spotlight/modifiers/spotlight_generation.py:128-165) without repeating the caches. */
int sl_sparse_attn_decode_ex(const void* d_q, const void* d_k, const void* d_v, int dtype, const sl_kv_layout* kv,
                             const int32_t* d_idx, int idx_capacity, const int32_t* d_cnt, int B, int KH, int QH,
                             int gqa_layout, void* d_out, float* d_lse, void* d_workspace, size_t workspace_bytes,
                             void* stream);

/* sl_sparse_attn_decode for callers that may not allocate device memory where they run attention
 * (an engine whose memory pool took all of HBM at start-up; a decode loop in which cudaMalloc and
 * cudaFree are banned because they can stall the whole device). It has no counterpart in the
 * reference. Arguments and results are those of sl_sparse_attn_decode without the workspace:
 * the scratch for the per-split partials is a fixed array of SL_ATTN_STATIC_SCRATCH_BYTES inside
 * the library, resident on every GPU that loads it until the process ends. Shapes that need more
 * (B*QH > 252) are refused with SL_EWORKSPACE. The call allocates and frees nothing.
 * The first call on a device looks up the array's device address; make that call before any
 * stream capture begins. All calls share the one array and nothing in it has to be cleared
 * between them, but two calls whose kernels may run at the same time on one GPU (different
 * streams) race on it: serialise them or give the second a workspace of its own. */
#define SL_ATTN_STATIC_SCRATCH_BYTES (8u << 20)
int sl_sparse_attn_decode_static(const void* d_q, const void* d_k, const void* d_v, int dtype,
                                 int64_t kv_batch_stride, const int32_t* d_idx, int idx_capacity,
                                 const int32_t* d_cnt, int B, int KH, int QH, int gqa_layout,
                                 void* d_out, float* d_lse, void* stream);

/* Log-sum-exp merge of R partial attention results (sequence shards):
 * d_o [R,rows,128] float, d_lse [R,rows] float -> d_out [rows,128] of `dtype`. */
int sl_merge_lse(const float* d_o, const float* d_lse, int R, int64_t rows, int dtype, void* d_out,
                 void* stream);

/* LRU-resident KV buffer, stage (3) of the decode path; one launch per decode step and layer.
 * The reference has no counterpart (its nearest relatives are KVCache.gather,
 * spotlight/modifiers/gpu_cache.py:100-106, and the host-offloaded gather of
 * spotlight/modifiers/cpu_cache.py:105-113); the policy is this library's:
 *  - per (b, kv head) C slots; attended keys already resident are hits and get stamped with `step`;
 *  - each miss, in index-list order, takes the least recently attended slot not used in this
 *    step: never-used slots first, then by age in steps (ages above 1023 count as 1023), ties
 *    to the LOWEST slot index; its K and V rows are copied from the backing store
 *    [B, N, KH, 128] (device memory or mapped pinned host memory) into the resident buffers
 *    [B, C, KH, 128];
 *  - d_slots_out[b,h,j] = slot of d_idx[b,h,j]: sl_sparse_attn_decode over the resident buffers
 *    with d_slots_out as its index list performs exactly the arithmetic of the direct call.
 * State (caller-owned, initialised to -1): d_tok2slot [B,KH,n_max], d_slot2tok [B,KH,C],
 * d_last_used [B,KH,C], all int32. Requires cnt[b,h] <= C (else *d_status = 3).
 * d_stats (optional) [B,KH,2] receives hits and misses of the step. */
int sl_lru_update(const int32_t* d_idx, int idx_capacity, const int32_t* d_cnt, int B, int KH,
                  const void* k_backing, const void* v_backing, int64_t backing_batch_stride,
                  int elem_bytes, void* d_k_resident, void* d_v_resident, int C,
                  int32_t* d_tok2slot, int64_t n_max, int32_t* d_slot2tok, int32_t* d_last_used,
                  int step, int32_t* d_slots_out, int32_t* d_stats, int32_t* d_status, void* stream);

/* sl_lru_update with the cache geometries spelled out (backing store and resident buffers may be fused
 * K|V caches or host memory with any strides), an optional step in DEVICE memory (*d_step, e.g. the decode
 * position, so that a replayed CUDA graph advances the table's clock) and an optional workspace of
 * sl_lru_workspace_bytes(B, KH, idx_capacity) bytes, zero-filled once and left zeroed by every call: with it
 * the update is spread over several CTAs per (b, kv head), each owning a slice of the index list and a range of the
 * slots (a cooperative launch; what the CTAs of a pair need from one another crosses the workspace behind four bounded
 * barriers of the pair; SL_OPT_LRU_MULTI_CTA = 0: only the probe is spread and the last CTA to finish handles the
 * misses alone). Results are those of sl_lru_update. */
size_t sl_lru_workspace_bytes(int B, int KH, int idx_capacity);
int sl_lru_update_ex(const int32_t* d_idx, int idx_capacity, const int32_t* d_cnt, int B, int KH,
                     const void* k_backing, const void* v_backing, const sl_kv_layout* backing, int elem_bytes,
                     void* d_k_resident, void* d_v_resident, const sl_kv_layout* resident, int C,
                     int32_t* d_tok2slot, int64_t n_max, int32_t* d_slot2tok, int32_t* d_last_used, int step,
                     const int64_t* d_step, int32_t* d_slots_out, int32_t* d_stats, int32_t* d_status,
                     void* d_workspace, size_t workspace_bytes, void* stream);

/* Stage (3) without its own copy of the missed rows: the slot tables are updated exactly as by sl_lru_update_ex, but
 * the K/V rows of this step's misses are NOT copied; their entries of d_slots_out are -(slot + 1). The attention
 * call that follows, sl_sparse_attn_decode_fill, fetches those rows from the backing store, attends to them and
 * writes them into their slots of the resident buffers on the way, so a missed row crosses memory once instead of
 * three times and the step has one launch less. The pair must be issued together: after sl_lru_update_deferred the
 * resident buffers are complete only once sl_sparse_attn_decode_fill has run on the same lists. No reference counterpart. */
int sl_lru_update_deferred(const int32_t* d_idx, int idx_capacity, const int32_t* d_cnt, int B, int KH, int elem_bytes,
                           void* d_k_resident, void* d_v_resident, const sl_kv_layout* resident, int C,
                           int32_t* d_tok2slot, int64_t n_max, int32_t* d_slot2tok, int32_t* d_last_used, int step,
                           const int64_t* d_step, int32_t* d_slots_out, int32_t* d_stats, int32_t* d_status,
                           void* d_workspace, size_t workspace_bytes, void* stream);

/* Stage (3) in two launches, so that the attention need not wait for the evictions:
 *   sl_lru_probe   hits are stamped and their slots written to d_slots_out, misses get -1 there and are recorded in
 *                  the workspace;
 *   sl_lru_evict   the evictions of sl_lru_update_ex for those misses (same policy, same tables afterwards) and the copy
 *                  of their rows into the slots. It does not touch the slot list, so it may run on another stream beside
 *                  sl_sparse_attn_decode_fill with read_only = 1 on the probe's list (the slots it fills are not read by
 *                  that call: they belong to no key of this step's hits). Both must be over before the next probe of the
 *                  same table. The workspace (sl_lru_workspace_bytes) carries the misses from one launch to the other.
 * A building block for callers that schedule their own streams; sl_decode_step uses the deferred form above (measured
 * on B200 at the headline shape: running the evictions on a second stream beside the attention did not shorten the step,
 * the evictions and the row copy together outlast everything that could hide them). No reference counterpart. */
int sl_lru_probe(const int32_t* d_idx, int idx_capacity, const int32_t* d_cnt, int B, int KH, int elem_bytes,
                 void* d_k_resident, void* d_v_resident, const sl_kv_layout* resident, int C, int32_t* d_tok2slot,
                 int64_t n_max, int32_t* d_slot2tok, int32_t* d_last_used, int step, const int64_t* d_step,
                 int32_t* d_slots_out, int32_t* d_status, void* d_workspace, size_t workspace_bytes, void* stream);
int sl_lru_evict(const int32_t* d_idx, int idx_capacity, const int32_t* d_cnt, int B, int KH, const void* k_backing,
                 const void* v_backing, const sl_kv_layout* backing, int elem_bytes, void* d_k_resident,
                 void* d_v_resident, const sl_kv_layout* resident, int C, int32_t* d_tok2slot, int64_t n_max,
                 int32_t* d_slot2tok, int32_t* d_last_used, int step, const int64_t* d_step, int32_t* d_slots,
                 int32_t* d_stats, int32_t* d_status, void* d_workspace, size_t workspace_bytes, void* stream);

/* Where sl_sparse_attn_decode_fill finds the rows that are not resident yet: the keys of the list entries (the index
 * list the slots were made from, [B, KH, idx_capacity]) and the backing K/V store with its geometry (device memory or
 * mapped pinned host memory). */
typedef struct sl_attn_fill {
    const int32_t* d_tokens;
    const void* k_backing; const void* v_backing;
    sl_kv_layout backing;
    int read_only;      /* 1: the rows of negative entries are only read (any negative value marks a miss); the slots are
                           filled by somebody else, e.g. sl_lru_evict running beside this call */
} sl_attn_fill;

/* sl_sparse_attn_decode_ex over the resident buffers of an LRU table, with the slot list of sl_lru_update_deferred:
 * entries >= 0 are read from the resident buffers; an entry -(slot + 1) is read from the backing store at the key's
 * index and written into that slot. bf16, at most 16 query heads per list head. The arithmetic, and so the output, is
 * that of sl_sparse_attn_decode_ex over the full caches with the index list. */
int sl_sparse_attn_decode_fill(const void* d_q, void* d_k_resident, void* d_v_resident, int dtype,
                               const sl_kv_layout* resident, const int32_t* d_slots, int idx_capacity,
                               const int32_t* d_cnt, int B, int KH, int QH, int gqa_layout, void* d_out, float* d_lse,
                               void* d_workspace, size_t workspace_bytes, const sl_attn_fill* fill, void* stream);

/* Row gather for API parity with KVCache.gather (spotlight/modifiers/gpu_cache.py:100-106):
 * out[b,j,h,:] = cache[b, idx[b,h,j], h, :] for j < budget. */
int sl_gather_rows(const void* d_cache, int64_t batch_stride, int elem_bytes,
                   const int32_t* d_idx, int idx_capacity, int B, int KH, int budget,
                   void* d_out, void* stream);

/* One decode token through all layers, with the layer loop in native code: per layer
 * sl_decode_prepare (token `pos` appended) -> sl_scan_topk over keys 0..pos with the reference's
 * budget rule k = max(min(n, min_remain), n - int(n * mask_out)), n = pos + 1
 * (spotlight/modifiers/spotlight_generation.py:162-164) -> sl_sparse_attn_decode.
 * Replaces the per-layer Python of the attention hook for callers that own the layer loop
 * (spotlight/modifiers/spotlight_generation.py:109-226 runs once per layer and token).
 * With `lru` set the layer-step has four launches: ... -> sl_scan_topk -> sl_lru_update_deferred (the slot tables
 * are updated) -> sl_sparse_attn_decode_fill over the resident buffers, which fetches the rows of the step's misses
 * from the caches and fills their slots (bf16; other dtypes: sl_lru_update_ex, which copies the rows, and
 * sl_sparse_attn_decode_ex; SL_OPT_LRU_FUSED_FILL = 0 forces that form).
 * Pointer tables are HOST arrays of `layers` device pointers; d_k / d_v tables (or entries) may be
 * NULL when the token's key/value are already in the caches. The scratch buffers are shared by all
 * layers (the launches are in stream order); workspaces as for the single entry points. */
struct sl_lru_layer {
    void* d_k_resident; void* d_v_resident;
    int32_t* d_tok2slot; int32_t* d_slot2tok; int32_t* d_last_used;
    int32_t* d_stats;                                /* [B,KH,2] hits and misses of the last step, or NULL */
};
typedef struct {
    int B, QH, KH, layers, dtype, gqa_layout;
    int sink, recent, min_remain;
    double mask_out;
    int64_t code_batch_stride, kv_batch_stride;      /* uint32 words / elements, as in sl_decode_prepare */
    int64_t kv_token_stride, kv_head_stride;         /* elements; 0, 0 = the two-cache layout (KH*128, 128) */
    const void* const* d_q;                          /* [layers] -> [B,QH,128] */
    const void* const* d_k;                          /* [layers] -> [B,KH,128] */
    const void* const* d_v;
    const sl_hash_params* hash_q;                    /* [layers] */
    const sl_hash_params* hash_k;
    uint32_t* const* d_code_cache;                   /* [layers] -> [B,*,KH,4] */
    void* const* d_k_cache;                          /* [layers] -> [B,*,KH,128] */
    void* const* d_v_cache;
    void* const* d_out;                              /* [layers] -> [B,QH,128] */
    const void* d_cos; const void* d_sin;            /* [128] for position pos, or NULL */
    void* d_q_rot; uint32_t* d_q_codes;              /* scratch [B,QH,128], [B,QH,4] */
    int32_t* d_idx; int idx_capacity; int32_t* d_cnt;
    void* d_scan_workspace; size_t scan_workspace_bytes;
    void* d_attn_workspace; size_t attn_workspace_bytes;
    int32_t* d_status;
    /* stage (3), optional (lru == NULL: attention reads the caches directly): per layer the resident buffers
     * and slot tables of sl_lru_update_ex; the step of the tables is the token's position */
    const struct sl_lru_layer* lru;                  /* [layers] */
    int lru_slots; int64_t lru_n_max;
    int64_t lru_batch_stride, lru_token_stride, lru_head_stride;   /* geometry of the resident buffers, elements */
    int32_t* d_slots;                                /* scratch [B,KH,idx_capacity] */
    void* d_lru_workspace; size_t lru_workspace_bytes;
} sl_decode_step_args;
int sl_decode_step(const sl_decode_step_args* args, int64_t pos, void* stream);

/* sl_decode_step with the position in DEVICE memory, so that ONE captured sequence of launches (a CUDA
 * graph) serves every token of a decode loop: the token sits at *d_pos, the context is *d_pos + 1 keys,
 * the budget follows the same rule, evaluated on the device. Replaces the per-token Python of the
 * reference's generate loop (spotlight/modifiers/spotlight_generation.py:470-495), whose every
 * iteration rebuilds its launches and synchronises with `.item()`.
 *   d_pos            int64 word; 0 <= *d_pos < max_context. With advance != 0 the last launch adds 1 to it.
 *   max_context      what the launches are planned for (grid shapes, idx_capacity >= min(max_context,
 *                    k(max_context) + sink + recent)); the caches hold at least that many rows
 *   d_cos_table/d_sin_table  [table_rows,128] of args->dtype: row r holds position table_pos0 + r
 *                    (NULL, NULL: q/k arrive rotated); args->d_cos / d_sin are ignored
 * Shapes the one-barrier scan kernel does not cover return SL_ESHAPE: use sl_decode_step per position then. */
typedef struct {
    int64_t* d_pos;
    int64_t max_context;
    const void* d_cos_table; const void* d_sin_table;
    int64_t table_pos0, table_rows;
    int advance;
} sl_decode_dev;
int sl_decode_step_dev(const sl_decode_step_args* args, const sl_decode_dev* dev, void* stream);

/* ---- exchange between the GPUs of one node over peer memory (sequence-sharded contexts) ----
 * No reference counterpart: the reference has no sequence parallelism (its only collectives are
 * in training, train.py:250-260). A sequence-sharded decode step all-gathers two KB-sized
 * messages per layer (score histograms, attention partials); these entry points do that with one
 * kernel per exchange over CUDA-IPC peer mappings instead of a collective library.
 *   sl_peer_buffer_bytes  size of one rank's exchange buffer for R ranks and a slot of slot_stride bytes
 *   sl_peer_alloc / sl_peer_free     the buffer (cudaMalloc, zero-filled); one per rank and exchange
 *   sl_peer_export                   64-byte IPC handle of a buffer, to be sent to the other ranks
 *   sl_peer_open / sl_peer_close     map / unmap another rank's buffer from its handle
 *   sl_peer_allgather                this rank's message (bytes % 16 == 0, <= slot_stride) -> slot `rank`
 *                                    of every buffer in peer_bufs[0..R) (host array, own buffer at index
 *                                    `rank`); returns in stream order once all R slots of the OWN buffer
 *                                    hold this round's messages. Every rank must call it for every round,
 *                                    in the same order; a buffer may be used again only after another
 *                                    exchange (or any other synchronisation of all ranks) has completed.
 *                                    The wait is bounded (about a second): *d_status = 3 when it ran out. */
size_t sl_peer_buffer_bytes(int R, size_t slot_stride);
int sl_peer_alloc(size_t bytes, void** d_ptr);
int sl_peer_free(void* d_ptr);
int sl_peer_export(const void* d_ptr, unsigned char* handle64);
int sl_peer_open(const unsigned char* handle64, void** d_ptr);
int sl_peer_close(void* d_ptr);
int sl_peer_allgather(const void* d_src, size_t bytes, void* const* peer_bufs, int rank, int R,
                      size_t slot_stride, int32_t* d_status, void* stream);
/* The exchange of attention partials and their merge in one launch: this rank's partial output
 * d_o [rows,128] (`dtype`) and d_lse [rows] go to every rank as [rows][129] floats, and d_out
 * [rows,128] receives the log-sum-exp merge of all R partials (the arithmetic of sl_merge_lse).
 * slot_stride >= rows*129*4; the same calling rules as sl_peer_allgather. Several CTAs send and merge a few
 * rows each and count their arrivals in the buffers' flag area, which they lay out in their own way: a buffer
 * given to this entry point is used for nothing else. */
int sl_peer_merge_lse(const void* d_o, const float* d_lse, int dtype, int64_t rows, void* const* peer_bufs,
                      int rank, int R, size_t slot_stride, void* d_out, int32_t* d_status, void* stream);

/* Fused form of sl_scan_hist + histogram all-gather + sl_select_emit for a sequence shard: one
 * cooperative launch per rank that scans the local codes, stores the merged local histograms into
 * every rank's exchange buffer (peer stores), waits (bounded, *d_status = 3 when it ran out) for
 * the other ranks' histograms and writes this rank's share of the global selection: the k highest
 * scores of the WHOLE context with ties to the lowest GLOBAL index, plus the parts of the sink and
 * of the recent window that fall into [tok_offset, tok_offset + N_local). d_idx holds LOCAL indices.
 * peer_bufs[0..R): exchange buffers of sl_peer_buffer_bytes(R, slot_stride) bytes each (own one at
 * index `rank`), slot_stride >= sl_scan_topk_sharded_slot_bytes(B, KH, QH), used for nothing else.
 * All R ranks must call it for every step with grids of the same shape, and must all pass another
 * exchange (e.g. the attention partials) before the next call. Shapes the fused kernel does not
 * cover return SL_ESHAPE: use sl_scan_hist + sl_select_emit then. No reference counterpart. */
size_t sl_scan_topk_sharded_slot_bytes(int B, int KH, int QH);
int sl_scan_topk_sharded(const uint32_t* d_q_codes, const uint32_t* d_k_codes, int64_t k_batch_stride, int B,
                         int64_t N_local, int64_t tok_offset, int64_t N_global, int KH, int QH,
                         int gqa_layout, int k, int sink, int recent, int32_t* d_idx, int idx_capacity,
                         int32_t* d_cnt, void* d_workspace, size_t workspace_bytes, void* const* peer_bufs,
                         int rank, int R, size_t slot_stride, int32_t* d_status, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* SPOTLIGHT_B200_H */
