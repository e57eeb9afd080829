"""Drop-in for the reference's ``spotlight.kernel`` package (spotlight/kernel/__init__.py:1-40):
the same eight entry points, all served by the one CUDA library (no Triton, no dispatch).

Importing this package raises ImportError when the library has not been built, exactly as the
reference does when its compiled kernels are missing (spotlight/kernel/__init__.py:7-11).

Differences, all supersets: ``attn_cuda_func`` accepts any (k_head, q_head) with
q_head % k_head == 0 (the reference's table holds only (4, 28), :14-16); ``pack_cuda_func``
accepts fp32/fp16/bool besides bf16 (packbits.cu:30 checks bf16)."""
from .. import ops as _ops
from .._lib import GQA_INTERLEAVED as _INTERLEAVED


def pack_dx_u32_func(x):
    """[..., 32m] -> uint32 [..., m]; bit j of word i <=> x[32i+j] > 0
    (spotlight/kernel/pack_dx_u32.py:35-59)."""
    assert x.shape[-1] % 32 == 0, "suppose `last_dim % 8 == 0`"
    assert x.is_contiguous()
    return _ops.pack_signbits(x, 32)


def pack_dx_u8_func(x):
    """[..., 8m] -> uint8 [..., m] (spotlight/kernel/pack_dx_u8.py:34-56)."""
    assert x.shape[-1] % 8 == 0, "suppose `last_dim % 8 == 0`"
    return _ops.pack_signbits(x, 8)


def attn_dx_u32_func(q_hash, k_hash):
    """uint32 [B,1,QH,D] x uint32 [B,KN,KH,D] -> int16 [B,KN,KH], kv head h scored against
    q heads {g*KH + h} (spotlight/kernel/attn_dx_u32.py:131-162)."""
    B, QN, QH, D = q_hash.shape
    _, KN, KH, _ = k_hash.shape
    assert QN == 1, "only support single query"
    assert QH % KH == 0, "query head must be multiple of key head"
    assert q_hash.is_contiguous()
    assert k_hash.is_contiguous()
    return _ops.hamming_scores(q_hash, k_hash, _INTERLEAVED)


def attn_dx_u8_func(q_hash, k_hash):
    """uint8 [B,H,1,D] x uint8 [B,H,KN,D] -> uint8 [B,H,KN] (spotlight/kernel/attn_dx_u8.py:46-74)."""
    return _ops.hamming_scores_u8(q_hash, k_hash)


def pack_triton_func(x):
    return pack_dx_u32_func(x)


def pack_cuda_func(x):
    """spotlight/kernel/__init__.py:23-24 -> packbits.cu:28-63 (which makes its input contiguous)."""
    assert x.shape[-1] % 32 == 0, "Last dimension must be divisible by 32"
    return _ops.pack_signbits(x.contiguous(), 32)


def attn_triton_func(q_hash, k_hash):
    return attn_dx_u32_func(q_hash, k_hash)


def attn_cuda_func(q_hash, k_hash):
    """spotlight/kernel/__init__.py:31-40 -> attn_k4_q28.cu:100-138."""
    _, _, q_head, head_dim = q_hash.shape
    _, _, k_head, _ = k_hash.shape
    assert head_dim == 4, "only support head dim = 4 now"
    assert q_head % k_head == 0, f"(k_head, q_head) of {k_head}, {q_head} is not supported"
    return _ops.hamming_scores(q_hash, k_hash, _INTERLEAVED)
