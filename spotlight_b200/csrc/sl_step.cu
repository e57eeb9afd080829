// One decode token through the retrieval path of all layers, launched from native code: the
// layer loop (hash + append -> scan + top-k -> sparse attention, three entry points per layer) runs
// here instead of in the host language, so that a decode loop at advancing positions pays a few
// microseconds of launch work per kernel instead of an interpreter round trip.
#include "sl_common.cuh"

namespace {

__global__ void advance_pos_kernel(long long* pos) {
    sl::pdl_trigger();
    sl::pdl_wait();
    *pos += 1;
}

int run_layers(const sl_decode_step_args* a, int64_t pos, const sl_decode_dev* dev, void* stream) {
    SL_REQUIRE(a != nullptr, SL_EINVAL, "sl_decode_step: null argument block");
    SL_REQUIRE(a->layers > 0 && a->d_q && a->d_out && a->hash_q && a->d_code_cache && a->d_k_cache && a->d_v_cache,
               SL_EINVAL, "sl_decode_step: null pointer table");
    SL_REQUIRE(pos >= 0, SL_ESHAPE, "sl_decode_step: negative position");
    SL_REQUIRE(a->lru == nullptr || (a->d_slots && a->lru_slots > 0 && a->lru_n_max > 0 && a->lru_token_stride >= 128 &&
                                     a->lru_head_stride >= 128),
               SL_EINVAL, "sl_decode_step: incomplete description of the LRU-resident buffers");
    SL_REQUIRE((a->kv_token_stride == 0) == (a->kv_head_stride == 0), SL_EINVAL,
               "sl_decode_step: kv_token_stride and kv_head_stride must be given together");
    const sl_kv_layout kv = {a->kv_batch_stride, a->kv_token_stride ? a->kv_token_stride : (int64_t)a->KH * 128,
                             a->kv_head_stride ? a->kv_head_stride : 128, 1};
    const int64_t n = pos + 1;       // the context, or with a device-side position the capacity planned for
    // the reference's budget rule, evaluated in doubles as Python does
    // (spotlight/modifiers/spotlight_generation.py:162-164)
    const int64_t remain = n - (int64_t)((double)n * a->mask_out);
    const int k = (int)std::max<int64_t>(std::min<int64_t>(n, a->min_remain), remain);
    sl::DevPos dp = {};
    if (dev) {
        SL_REQUIRE(dev->d_pos != nullptr && dev->max_context > 0, SL_EINVAL, "sl_decode_step_dev: null position word");
        SL_REQUIRE((dev->d_cos_table == nullptr) == (dev->d_sin_table == nullptr), SL_EINVAL,
                   "sl_decode_step_dev: cos and sin tables must come together");
        SL_REQUIRE(dev->d_cos_table == nullptr || (dev->table_pos0 >= 0 && dev->table_pos0 + dev->table_rows >= dev->max_context),
                   SL_ESHAPE, "sl_decode_step_dev: cos/sin tables end before max_context");
        dp.d_pos = reinterpret_cast<const long long*>(dev->d_pos);
        dp.cos_tab = dev->d_cos_table; dp.sin_tab = dev->d_sin_table; dp.tab_pos0 = dev->table_pos0;
    }
    for (int l = 0; l < a->layers; ++l) {
        const bool with_k = a->d_k != nullptr && a->d_k[l] != nullptr;
        int rc = sl::decode_prepare_impl(a->d_q[l], with_k ? a->d_k[l] : nullptr, with_k && a->d_v ? a->d_v[l] : nullptr,
                                         a->dtype, a->B, a->QH, a->KH, a->d_cos, a->d_sin, &a->hash_q[l],
                                         with_k ? &a->hash_k[l] : nullptr, a->d_q_rot, a->d_q_codes, a->d_code_cache[l],
                                         a->code_batch_stride, a->d_k_cache[l], a->d_v_cache[l], &kv, pos, dev ? &dp : nullptr,
                                         stream);
        if (rc) return rc;
        rc = sl::scan_topk_impl(a->d_q_codes, a->d_code_cache[l], a->code_batch_stride, a->B, n, a->KH, a->QH, a->gqa_layout,
                                k, a->sink, a->recent, a->d_idx, a->idx_capacity, a->d_cnt, nullptr, a->d_scan_workspace,
                                a->scan_workspace_bytes, a->d_status, dev ? dp.d_pos : nullptr, a->mask_out, a->min_remain,
                                stream);
        if (rc) return rc;
        if (a->lru) {
            const sl_lru_layer& t = a->lru[l];
            const sl_kv_layout res = {a->lru_batch_stride, a->lru_token_stride, a->lru_head_stride, 1};
            const int64_t* d_step = dev ? reinterpret_cast<const int64_t*>(dp.d_pos) : nullptr;
            if (sl::lru_fused_fill() && a->dtype == SL_BF16 && a->QH / a->KH <= 16) {
                // the attention launch fetches the rows of the misses itself and fills their slots on the way
                rc = sl_lru_update_deferred(a->d_idx, a->idx_capacity, a->d_cnt, a->B, a->KH, 2, t.d_k_resident, t.d_v_resident,
                                            &res, a->lru_slots, t.d_tok2slot, a->lru_n_max, t.d_slot2tok, t.d_last_used, (int)pos,
                                            d_step, a->d_slots, t.d_stats, a->d_status, a->d_lru_workspace,
                                            a->lru_workspace_bytes, stream);
                if (rc) return rc;
                const sl_attn_fill fill = {a->d_idx, a->d_k_cache[l], a->d_v_cache[l], kv};
                rc = sl_sparse_attn_decode_fill(a->d_q_rot, t.d_k_resident, t.d_v_resident, a->dtype, &res, a->d_slots,
                                                a->idx_capacity, a->d_cnt, a->B, a->KH, a->QH, a->gqa_layout, a->d_out[l], nullptr,
                                                a->d_attn_workspace, a->attn_workspace_bytes, &fill, stream);
            } else {
                rc = sl_lru_update_ex(a->d_idx, a->idx_capacity, a->d_cnt, a->B, a->KH, a->d_k_cache[l], a->d_v_cache[l], &kv,
                                      a->dtype == SL_F32 ? 4 : 2, t.d_k_resident, t.d_v_resident, &res, a->lru_slots, t.d_tok2slot,
                                      a->lru_n_max, t.d_slot2tok, t.d_last_used, (int)pos, d_step, a->d_slots, t.d_stats,
                                      a->d_status, a->d_lru_workspace, a->lru_workspace_bytes, stream);
                if (rc) return rc;
                rc = sl_sparse_attn_decode_ex(a->d_q_rot, t.d_k_resident, t.d_v_resident, a->dtype, &res, a->d_slots,
                                              a->idx_capacity, a->d_cnt, a->B, a->KH, a->QH, a->gqa_layout, a->d_out[l], nullptr,
                                              a->d_attn_workspace, a->attn_workspace_bytes, stream);
            }
        } else {
            rc = sl_sparse_attn_decode_ex(a->d_q_rot, a->d_k_cache[l], a->d_v_cache[l], a->dtype, &kv, a->d_idx,
                                          a->idx_capacity, a->d_cnt, a->B, a->KH, a->QH, a->gqa_layout, a->d_out[l], nullptr,
                                          a->d_attn_workspace, a->attn_workspace_bytes, stream);
        }
        if (rc) return rc;
    }
    if (dev && dev->advance)
        SL_CUDA_OK(sl::launch_kernel(advance_pos_kernel, dim3(1), dim3(1), 0, static_cast<cudaStream_t>(stream), false,
                                     reinterpret_cast<long long*>(dev->d_pos)));
    return SL_OK;
}

}  // namespace

extern "C" int sl_decode_step(const sl_decode_step_args* a, int64_t pos, void* stream) {
    return run_layers(a, pos, nullptr, stream);
}

extern "C" int sl_decode_step_dev(const sl_decode_step_args* a, const sl_decode_dev* dev, void* stream) {
    SL_REQUIRE(dev != nullptr, SL_EINVAL, "sl_decode_step_dev: null device-position block");
    return run_layers(a, dev->max_context - 1, dev, stream);
}
