// Arguments shared by the sparse decode-attention kernels.
#pragma once
#include "sl_common.cuh"

namespace sl {

constexpr int ATTN_MAX_SPLITS = 64;

struct AttnArgs {
    const void* q; const void* k; const void* v;
    long long kv_b;                // batch stride in elements
    long long tok_stride;          // elements between the rows of consecutive keys (KH * 128 for [B,N,KH,128])
    long long head_stride;         // elements between the rows of consecutive kv heads of one key (128)
    int kv_div;                    // list heads (entries of idx/cnt per batch row) per kv head of the caches (1)
    const int* idx; int cap; const int* cnt;
    int B, KH, layout, splits;
    void* out; float* lse;
    float* part;                   // [B*KH][splits][G][130]: o[128], m, l
    // fill mode (bf16 tensor-core kernel only): k / v are the resident buffers of an LRU table and idx holds SLOTS; a
    // negative entry -(slot + 1) is a key whose rows are not resident yet: they are fetched from the backing store at
    // the key's index (tok) and written into the slot on the way
    const int* tok;                // [B*KH][cap] keys of the list entries, or null: no fill mode
    const void* k_back; const void* v_back;
    long long back_b, back_tok, back_head;   // elements
    int fill_write;                // 1: write the fetched rows into their slots; 0: only read them (somebody else fills the slots)
};


// Merge of the per-split partials [B*KH][splits][G][130] into the output (one CTA per query head).
int launch_attn_merge(const AttnArgs& a, int G, int dtype, cudaStream_t s);

// bf16 tensor-core path (sl_attn_mma.cu); G = QH / KH <= 16.
int launch_attn_mma(const AttnArgs& a, int G, cudaStream_t s);
int attn_mma_splits(int B, int KH, int cap, int reserve_sms = 0);

}  // namespace sl
