// One decode token through the retrieval path of all layers, launched from native code: the
// layer loop (hash + append -> scan + top-k -> sparse attention, three entry points per layer) runs
// here instead of in the host language, so that a decode loop at advancing positions pays a few
// microseconds of launch work per kernel instead of an interpreter round trip.
#include "sl_common.cuh"

extern "C" int sl_decode_step(const sl_decode_step_args* a, int64_t pos, void* stream) {
    SL_REQUIRE(a != nullptr, SL_EINVAL, "sl_decode_step: null argument block");
    SL_REQUIRE(a->layers > 0 && a->d_q && a->d_out && a->hash_q && a->d_code_cache && a->d_k_cache && a->d_v_cache,
               SL_EINVAL, "sl_decode_step: null pointer table");
    SL_REQUIRE(pos >= 0, SL_ESHAPE, "sl_decode_step: negative position");
    const int64_t n = pos + 1;
    // the reference's budget rule, evaluated in doubles as Python does
    // (spotlight/modifiers/spotlight_generation.py:162-164)
    const int64_t remain = n - (int64_t)((double)n * a->mask_out);
    const int k = (int)std::max<int64_t>(std::min<int64_t>(n, a->min_remain), remain);
    for (int l = 0; l < a->layers; ++l) {
        const bool with_k = a->d_k != nullptr && a->d_k[l] != nullptr;
        int rc = sl_decode_prepare(a->d_q[l], with_k ? a->d_k[l] : nullptr, with_k && a->d_v ? a->d_v[l] : nullptr, a->dtype,
                                   a->B, a->QH, a->KH, a->d_cos, a->d_sin, &a->hash_q[l],
                                   with_k ? &a->hash_k[l] : nullptr, a->d_q_rot, a->d_q_codes, a->d_code_cache[l],
                                   a->code_batch_stride, a->d_k_cache[l], a->d_v_cache[l], a->kv_batch_stride, pos,
                                   stream);
        if (rc) return rc;
        rc = sl_scan_topk(a->d_q_codes, a->d_code_cache[l], a->code_batch_stride, a->B, n, a->KH, a->QH, a->gqa_layout, k,
                          a->sink, a->recent, a->d_idx, a->idx_capacity, a->d_cnt, nullptr, a->d_scan_workspace,
                          a->scan_workspace_bytes, a->d_status, stream);
        if (rc) return rc;
        rc = sl_sparse_attn_decode(a->d_q_rot, a->d_k_cache[l], a->d_v_cache[l], a->dtype, a->kv_batch_stride, a->d_idx,
                                   a->idx_capacity, a->d_cnt, a->B, a->KH, a->QH, a->gqa_layout, a->d_out[l], nullptr,
                                   a->d_attn_workspace, a->attn_workspace_bytes, stream);
        if (rc) return rc;
    }
    return SL_OK;
}
