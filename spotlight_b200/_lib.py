"""ctypes binding of libspotlight_b200.so (the C ABI declared in include/spotlight_b200.h).

There is no fallback: if the library has not been built, importing this module raises
ImportError, as the reference does when its compiled kernels are missing
(spotlight/kernel/__init__.py:7-11)."""
from __future__ import annotations

import ctypes as C
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "lib", "libspotlight_b200.so")

SL_OK, SL_EINVAL, SL_ESHAPE, SL_EALIGN, SL_EWORKSPACE, SL_ECUDA, SL_ETIMEOUT = 0, -1, -2, -3, -4, -5, -6
SL_BF16, SL_F32, SL_F16, SL_BOOL = 0, 1, 2, 3
GQA_INTERLEAVED, GQA_BLOCKED = 0, 1
SL_OPT_PDL, SL_OPT_L2_PREFETCH, SL_OPT_SCAN_KERNEL, SL_OPT_ATTN_WARPS, SL_OPT_PEER_SPIN_LIMIT, SL_OPT_HASH_KERNEL, SL_OPT_ATTN_CLUSTER, SL_OPT_LRU_FUSED_FILL, SL_OPT_LRU_MULTI_CTA = 0, 1, 2, 3, 4, 5, 6, 7, 8


class HashParamsStruct(C.Structure):
    _fields_ = [("n_layers", C.c_int), ("dims", C.c_int * 4), ("residue", C.c_int),
                ("d_w", C.c_void_p * 3), ("d_b", C.c_void_p * 3)]


_P, _I, _L, _Z = C.c_void_p, C.c_int, C.c_int64, C.c_size_t
_HP = C.POINTER(HashParamsStruct)
_PP = C.POINTER(C.c_void_p)


class LruLayer(C.Structure):
    """sl_lru_layer of include/spotlight_b200.h."""
    _fields_ = [("d_k_resident", _P), ("d_v_resident", _P), ("d_tok2slot", _P), ("d_slot2tok", _P),
                ("d_last_used", _P), ("d_stats", _P)]


class DecodeStepArgs(C.Structure):
    """sl_decode_step_args of include/spotlight_b200.h."""
    _fields_ = [("B", _I), ("QH", _I), ("KH", _I), ("layers", _I), ("dtype", _I), ("gqa_layout", _I),
                ("sink", _I), ("recent", _I), ("min_remain", _I), ("mask_out", C.c_double),
                ("code_batch_stride", _L), ("kv_batch_stride", _L), ("kv_token_stride", _L), ("kv_head_stride", _L),
                ("d_q", _PP), ("d_k", _PP), ("d_v", _PP), ("hash_q", _HP), ("hash_k", _HP),
                ("d_code_cache", _PP), ("d_k_cache", _PP), ("d_v_cache", _PP), ("d_out", _PP),
                ("d_cos", _P), ("d_sin", _P), ("d_q_rot", _P), ("d_q_codes", _P),
                ("d_idx", _P), ("idx_capacity", _I), ("d_cnt", _P),
                ("d_scan_workspace", _P), ("scan_workspace_bytes", _Z),
                ("d_attn_workspace", _P), ("attn_workspace_bytes", _Z), ("d_status", _P),
                ("lru", C.POINTER(LruLayer)), ("lru_slots", _I), ("lru_n_max", _L),
                ("lru_batch_stride", _L), ("lru_token_stride", _L), ("lru_head_stride", _L),
                ("d_slots", _P), ("d_lru_workspace", _P), ("lru_workspace_bytes", _Z)]

class KvLayout(C.Structure):
    """sl_kv_layout of include/spotlight_b200.h (strides in elements)."""
    _fields_ = [("batch_stride", _L), ("token_stride", _L), ("head_stride", _L), ("list_heads_per_kv_head", _I)]


class DecodeDev(C.Structure):
    """sl_decode_dev of include/spotlight_b200.h."""
    _fields_ = [("d_pos", _P), ("max_context", _L), ("d_cos_table", _P), ("d_sin_table", _P),
                ("table_pos0", _L), ("table_rows", _L), ("advance", _I)]


class AttnFill(C.Structure):
    """sl_attn_fill of include/spotlight_b200.h."""
    _fields_ = [("d_tokens", _P), ("k_backing", _P), ("v_backing", _P), ("backing", KvLayout), ("read_only", _I)]


_KV = C.POINTER(KvLayout)

# name -> (restype, argtypes); must list every symbol of include/spotlight_b200.h
SIGNATURES = {
    "sl_version": (_I, []),
    "sl_last_error_string": (C.c_char_p, []),
    "sl_set_device": (_I, [_I]),
    "sl_configure": (_I, [_I, _I]),
    "sl_hash_status": (_I, []),
    "sl_attn_cluster_capacity": (_I, [_I, _I]),
    "sl_pack_signbits": (_I, [_P, _I, _L, _P, _P]),
    "sl_hamming_scores": (_I, [_P, _P, _L, _P, _I, _L, _I, _I, _I, _I, _P]),
    "sl_hamming_scores_u8": (_I, [_P, _P, _P, _L, _L, _I, _P]),
    "sl_scan_topk_workspace_bytes": (_Z, [_I, _L, _I, _I]),
    "sl_workspace_init": (_I, [_P, _Z, _P]),
    "sl_scan_topk": (_I, [_P, _P, _L, _I, _L, _I, _I, _I, _I, _I, _I, _P, _I, _P, _P, _P, _Z, _P, _P]),
    "sl_topk_from_scores_workspace_bytes": (_Z, [_I, _L, _I, _I]),
    "sl_topk_from_scores": (_I, [_P, _I, _L, _I, _I, _I, _I, _I, _P, _I, _P, _P, _Z, _P, _P]),
    "sl_scan_hist": (_I, [_P, _P, _L, _I, _L, _I, _I, _I, _P, _P, _P]),
    "sl_select_emit_workspace_bytes": (_Z, [_I, _L, _I, _I]),
    "sl_select_emit": (_I, [_P, _P, _I, _I, _I, _L, _L, _L, _I, _I, _I, _I, _I, _P, _I, _P, _P, _Z, _P, _P]),
    "sl_decode_prepare": (_I, [_P, _P, _P, _I, _I, _I, _I, _P, _P, _HP, _HP, _P, _P, _P, _L, _P, _P, _L, _L, _P]),
    "sl_decode_prepare_ex": (_I, [_P, _P, _P, _I, _I, _I, _I, _P, _P, _HP, _HP, _P, _P, _P, _L, _P, _P, _KV, _L, _P]),
    "sl_hash_encode": (_I, [_P, _L, _I, _I, _L, _I, _HP, _P, _L, _P]),
    "sl_hash_encode_ex": (_I, [_P, _L, _L, _L, _I, _I, _L, _I, _HP, _P, _L, _P]),
    "sl_sparse_attn_workspace_bytes": (_Z, [_I, _I, _I]),
    "sl_sparse_attn_decode": (_I, [_P, _P, _P, _I, _L, _P, _I, _P, _I, _I, _I, _I, _P, _P, _P, _Z, _P]),
    "sl_sparse_attn_decode_ex": (_I, [_P, _P, _P, _I, _KV, _P, _I, _P, _I, _I, _I, _I, _P, _P, _P, _Z, _P]),
    "sl_sparse_attn_decode_fill": (_I, [_P, _P, _P, _I, _KV, _P, _I, _P, _I, _I, _I, _I, _P, _P, _P, _Z, C.POINTER(AttnFill), _P]),
    "sl_lru_probe": (_I, [_P, _I, _P, _I, _I, _I, _P, _P, _KV, _I, _P, _L, _P, _P, _I, _P, _P, _P, _P, _Z, _P]),
    "sl_lru_evict": (_I, [_P, _I, _P, _I, _I, _P, _P, _KV, _I, _P, _P, _KV, _I, _P, _L, _P, _P, _I, _P, _P, _P, _P, _P, _Z, _P]),
    "sl_lru_update_deferred": (_I, [_P, _I, _P, _I, _I, _I, _P, _P, _KV, _I, _P, _L, _P, _P, _I, _P, _P, _P, _P, _P, _Z, _P]),
    "sl_sparse_attn_decode_static": (_I, [_P, _P, _P, _I, _L, _P, _I, _P, _I, _I, _I, _I, _P, _P, _P]),
    "sl_merge_lse": (_I, [_P, _P, _I, _L, _I, _P, _P]),
    "sl_lru_update": (_I, [_P, _I, _P, _I, _I, _P, _P, _L, _I, _P, _P, _I, _P, _L, _P, _P, _I, _P, _P, _P, _P]),
    "sl_lru_workspace_bytes": (_Z, [_I, _I, _I]),
    "sl_lru_update_ex": (_I, [_P, _I, _P, _I, _I, _P, _P, _KV, _I, _P, _P, _KV, _I, _P, _L, _P, _P, _I, _P, _P, _P, _P, _P, _Z, _P]),
    "sl_gather_rows": (_I, [_P, _L, _I, _P, _I, _I, _I, _I, _P, _P]),
    "sl_decode_step": (_I, [C.POINTER(DecodeStepArgs), _L, _P]),
    "sl_decode_step_dev": (_I, [C.POINTER(DecodeStepArgs), C.POINTER(DecodeDev), _P]),
    "sl_scan_topk_sharded_slot_bytes": (_Z, [_I, _I, _I]),
    "sl_scan_topk_sharded": (_I, [_P, _P, _L, _I, _L, _L, _L, _I, _I, _I, _I, _I, _I, _P, _I, _P, _P, _Z, C.POINTER(_P),
                                  _I, _I, _Z, _P, _P]),
    "sl_peer_buffer_bytes": (_Z, [_I, _Z]),
    "sl_peer_alloc": (_I, [_Z, C.POINTER(_P)]),
    "sl_peer_free": (_I, [_P]),
    "sl_peer_export": (_I, [_P, C.c_char_p]),
    "sl_peer_open": (_I, [C.c_char_p, C.POINTER(_P)]),
    "sl_peer_close": (_I, [_P]),
    "sl_peer_allgather": (_I, [_P, _Z, C.POINTER(_P), _I, _I, _Z, _P, _P]),
    "sl_peer_merge_lse": (_I, [_P, _P, _I, _L, C.POINTER(_P), _I, _I, _Z, _P, _P, _P]),
}


def _load():
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build the CUDA library first with `python -m spotlight_b200.build` "
            "(there is no CPU or PyTorch fallback)")
    lib = C.CDLL(LIB_PATH)
    for name, (res, args) in SIGNATURES.items():
        fn = getattr(lib, name)
        fn.restype = res
        fn.argtypes = args
    return lib


lib = _load()

_ERRORS = {SL_EINVAL: ValueError, SL_ESHAPE: ValueError, SL_EALIGN: ValueError, SL_EWORKSPACE: ValueError,
           SL_ECUDA: RuntimeError, SL_ETIMEOUT: RuntimeError}


def check(rc: int) -> None:
    """Map a negative status to an exception carrying the library's message."""
    if rc != SL_OK:
        msg = lib.sl_last_error_string().decode("utf-8", "replace")
        raise _ERRORS.get(rc, RuntimeError)(f"spotlight_b200 [{rc}]: {msg}")
