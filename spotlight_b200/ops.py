"""Torch-facing wrappers over the C ABI: tensors in, tensors out. PyTorch is used only for
device memory and streams; every computation is a kernel of libspotlight_b200.so.

All tensors must live on a CUDA device. There is no CPU path."""
from __future__ import annotations

import ctypes as C
from typing import List, Optional, Sequence, Tuple

import torch

from . import _lib
from ._lib import GQA_BLOCKED, GQA_INTERLEAVED, check, lib

_DTYPES = {torch.bfloat16: _lib.SL_BF16, torch.float32: _lib.SL_F32, torch.float16: _lib.SL_F16,
           torch.bool: _lib.SL_BOOL}

launch_count = 0     # kernels launched through this module (bench accounting)


def _count(n: int = 1) -> None:
    global launch_count
    launch_count += n


def _dt(t: torch.Tensor) -> int:
    try:
        return _DTYPES[t.dtype]
    except KeyError:
        raise TypeError(f"unsupported dtype {t.dtype}") from None


def _cuda(*tensors: torch.Tensor) -> torch.device:
    dev = tensors[0].device
    for t in tensors:
        if t is None:
            continue
        if not t.is_cuda:
            raise RuntimeError("spotlight_b200 kernels need CUDA tensors (there is no CPU path)")
        if t.device != dev:
            raise RuntimeError("all tensors must be on the same device")
    check(lib.sl_set_device(dev.index if dev.index is not None else torch.cuda.current_device()))
    return dev


def _stream() -> int:
    return torch.cuda.current_stream().cuda_stream


def _ptr(t: Optional[torch.Tensor]) -> Optional[int]:
    return None if t is None else t.data_ptr()


def _rows_view(t: torch.Tensor, inner: int) -> int:
    """Batch stride (in elements) of a [B, N, H, inner] tensor whose batch rows are contiguous
    [N,H,inner] blocks (a `cache[:, :end]` view qualifies)."""
    B, N, H, D = t.shape
    assert D == inner
    if N * H * D and t.stride()[1:] != (H * D, D, 1):
        raise ValueError("expected token-major rows [N, H, D] contiguous inside each batch row")
    return t.stride(0) if B > 1 else max(t.stride(0), N * H * D)


def _kv_layout(t: torch.Tensor, list_heads_per_kv_head: int = 1) -> "_lib.KvLayout":
    """Geometry of a cache view [B, N, H, 128]: any batch / token / head strides with unit stride inside
    a row (two caches [B,N,H,128], the K or V half of a fused cache [B,N,H,2,128], an aliased batch
    made with ``expand``)."""
    B, N, H, D = t.shape
    sb, st, sh, sd = t.stride()
    if D != 128 or (sd != 1 and D > 1):
        raise ValueError("expected rows of 128 contiguous values")
    if N <= 1:
        st = max(st, H * D)
    if H <= 1:
        sh = max(sh, D)
    return _lib.KvLayout(sb if B > 1 else max(sb, 0), st, sh, list_heads_per_kv_head)


# ----------------------------------------------------------------------------- workspaces
class _Workspaces:
    """Zero-initialised scratch buffers, one per (kind, device, shape); the kernels leave
    them zeroed, so they are allocated once and reused. A status word rides along."""

    def __init__(self):
        self._bufs = {}

    def get(self, kind: str, device: torch.device, nbytes: int, shape=()) -> Tuple[torch.Tensor, torch.Tensor]:
        """`shape` = (B, KH, QH): the library lays a workspace out per shape and only guarantees
        to leave it zeroed for that shape, so every shape gets its own buffer."""
        key = (kind, device, tuple(shape))
        cur = self._bufs.get(key)
        if cur is None or cur[0].numel() < nbytes:
            buf = torch.zeros(max(nbytes, 256), dtype=torch.uint8, device=device)
            status = torch.zeros(1, dtype=torch.int32, device=device)
            cur = (buf, status)
            self._bufs[key] = cur
        return cur

    def reset(self):
        self._bufs.clear()


workspaces = _Workspaces()


def configure(option: int, value: int) -> None:
    """Process-wide switch of the library (`_lib.SL_OPT_*`): measurement and test aid; every default is
    the fast path."""
    _lib.check(_lib.lib.sl_configure(int(option), int(value)))


def check_status(device=None) -> None:
    """Host-side read of every status word (synchronises). Raises if a bounded device-side wait
    ran out; the affected workspace is dropped so the next call starts from a clean one."""
    bad = []
    for key, (buf, status) in list(workspaces._bufs.items()):
        if device is not None and key[1] != torch.device(device):
            continue
        if int(status.item()) != 0:
            bad.append((key, int(status.item())))
            del workspaces._bufs[key]
    hs = int(_lib.lib.sl_hash_status())
    if hs != 0:
        bad.append((("hash_encode",), hs))
    if bad:
        raise RuntimeError(f"spotlight_b200 [{_lib.SL_ETIMEOUT}]: device-side status set: {bad}")


# ----------------------------------------------------------------------------- hash params
class HashParams:
    """Device-resident hash parameters of one head set. ``weights[i]``: [H, in_i, out_i];
    ``biases[i]``: [H, out_i] or None. One layer without bias is the linear hash."""

    def __init__(self, weights: Sequence[torch.Tensor], biases: Optional[Sequence[Optional[torch.Tensor]]] = None,
                 residue: bool = False):
        assert 1 <= len(weights) <= 3
        biases = list(biases) if biases is not None else [None] * len(weights)
        self.weights = [w.contiguous() for w in weights]
        self.biases = [None if b is None else b.contiguous() for b in biases]
        self.residue = bool(residue)
        self.heads = self.weights[0].shape[0]
        self.dtype = self.weights[0].dtype
        s = _lib.HashParamsStruct()
        s.n_layers = len(self.weights)
        dims = [self.weights[0].shape[1]] + [w.shape[2] for w in self.weights]
        for i, w in enumerate(self.weights):
            assert w.dim() == 3 and w.shape[0] == self.heads and w.shape[1] == dims[i] and w.dtype == self.dtype
            s.d_w[i] = w.data_ptr()
            b = self.biases[i]
            if b is not None:
                assert b.shape == (self.heads, dims[i + 1]) and b.dtype == self.dtype
                s.d_b[i] = b.data_ptr()
        for i, d in enumerate(dims):
            s.dims[i] = d
        s.residue = int(self.residue)
        self.struct = s

    @classmethod
    def from_dict(cls, params: dict, device, residue: bool = False) -> "HashParams":
        """From workloads.make_hash_params output."""
        ws = [w.to(device) for w in params["w"]]
        bs = [None if b is None else b.to(device) for b in params["b"]]
        return cls(ws, bs, residue if params["kind"] == "mlp" else False)

    def ref(self):
        return C.byref(self.struct)


# ----------------------------------------------------------------------------- pack / scores
def pack_signbits(x: torch.Tensor, word_bits: int = 32) -> torch.Tensor:
    """[..., 32m] (bf16/fp16/fp32/bool) -> uint32 [..., m] (or uint8 [..., 4m] for word_bits=8)."""
    assert word_bits in (8, 32)
    last = x.shape[-1]
    assert last % word_bits == 0, f"suppose `last_dim % {word_bits} == 0`"
    _cuda(x)
    x = x.contiguous()
    out_dtype = torch.uint32 if word_bits == 32 else torch.uint8
    out = torch.empty((*x.shape[:-1], last // word_bits), dtype=out_dtype, device=x.device)
    check(lib.sl_pack_signbits(x.data_ptr(), _dt(x), x.numel(), out.data_ptr(), _stream()))
    _count()
    return out


def hamming_scores(q_hash: torch.Tensor, k_hash: torch.Tensor, layout: int = GQA_INTERLEAVED) -> torch.Tensor:
    """uint32 [B,1,QH,W] x uint32 [B,N,KH,W] -> int16 [B,N,KH] match counts."""
    B, QN, QH, W = q_hash.shape
    B2, N, KH, W2 = k_hash.shape
    assert QN == 1, "only support single query"
    assert QH % KH == 0, "query head must be multiple of key head"
    assert B == B2 and W == W2
    assert q_hash.dtype == torch.uint32 and k_hash.dtype == torch.uint32, "Inputs must be uint32"
    _cuda(q_hash, k_hash)
    q_hash = q_hash.contiguous()
    kb = _rows_view(k_hash, W)
    out = torch.empty((B, N, KH), dtype=torch.int16, device=q_hash.device)
    check(lib.sl_hamming_scores(q_hash.data_ptr(), k_hash.data_ptr(), kb, out.data_ptr(), B, N, KH, QH, W,
                                layout, _stream()))
    _count()
    return out


def hamming_scores_u8(q_hash: torch.Tensor, k_hash: torch.Tensor) -> torch.Tensor:
    """uint8 [B,H,1,D] x uint8 [B,H,N,D] -> uint8 [B,H,N] per-head match counts."""
    B, H, q_len, D = q_hash.shape
    _, _, N, _ = k_hash.shape
    assert q_len == 1, "only support single query"
    assert q_hash.dtype == torch.uint8 and k_hash.dtype == torch.uint8
    _cuda(q_hash, k_hash)
    q = q_hash.reshape(-1, D).contiguous()
    k = k_hash.reshape(-1, N, D).contiguous()
    out = torch.empty((B * H, N), dtype=torch.uint8, device=q.device)
    check(lib.sl_hamming_scores_u8(q.data_ptr(), k.data_ptr(), out.data_ptr(), B * H, N, D, _stream()))
    _count()
    return out.view(B, H, N)


# ----------------------------------------------------------------------------- scan + top-k
def scan_topk(q_codes: torch.Tensor, k_codes: torch.Tensor, k: int, sink: int = 4, recent: int = 64,
              layout: int = GQA_BLOCKED, idx: Optional[torch.Tensor] = None, cnt: Optional[torch.Tensor] = None,
              return_scores: bool = False):
    """Fused Hamming scan + exact top-k (lowest-index ties) + sink/recent window.
    q_codes uint32 [B,QH,4] (or [B,1,QH,4]); k_codes uint32 [B,N,KH,4] (a cache view is fine).
    Returns (idx int32 [B,KH,cap] ascending, cnt int32 [B,KH]) [+ scores int16 [B,N,KH]]."""
    if q_codes.dim() == 4:
        q_codes = q_codes[:, 0]
    B, QH, W = q_codes.shape
    B2, N, KH, W2 = k_codes.shape
    assert W == 4 and W2 == 4 and B == B2, "only support head dim = 4 now"
    dev = _cuda(q_codes, k_codes)
    q_codes = q_codes.contiguous()
    kb = _rows_view(k_codes, 4)
    cap = max(1, min(N, k + sink + recent))
    if idx is None:
        idx = torch.empty((B, KH, cap), dtype=torch.int32, device=dev)
    if cnt is None:
        cnt = torch.empty((B, KH), dtype=torch.int32, device=dev)
    assert idx.shape[0] == B and idx.shape[1] == KH and idx.is_contiguous() and idx.dtype == torch.int32
    scores = torch.empty((B, N, KH), dtype=torch.int16, device=dev) if return_scores else None
    need = lib.sl_scan_topk_workspace_bytes(B, N, KH, QH)
    ws, status = workspaces.get("scan", dev, need, (B, KH, QH))
    check(lib.sl_scan_topk(q_codes.data_ptr(), k_codes.data_ptr(), kb, B, N, KH, QH, layout, k, sink, recent,
                           idx.data_ptr(), idx.shape[2], cnt.data_ptr(), _ptr(scores), ws.data_ptr(), ws.numel(),
                           status.data_ptr(), _stream()))
    _count()
    return (idx, cnt, scores) if return_scores else (idx, cnt)


def scan_topk_sharded(q_codes: torch.Tensor, k_codes: torch.Tensor, peer, tok_offset: int, n_global: int, k: int,
                      sink: int = 4, recent: int = 64, layout: int = GQA_BLOCKED):
    """One rank's share of the global selection in ONE launch (see sl_scan_topk_sharded): local scan,
    histogram exchange through the peer buffer `peer` (sharded.PeerBuffer sized with
    scan_sharded_slot_bytes), emission of LOCAL indices. Raises ValueError when the fused kernel does
    not cover the shape."""
    if q_codes.dim() == 4:
        q_codes = q_codes[:, 0]
    B, QH, _ = q_codes.shape
    _, N, KH, _ = k_codes.shape
    dev = _cuda(q_codes, k_codes)
    q_codes = q_codes.contiguous()
    kb = _rows_view(k_codes, 4)
    s_end = min(sink, n_global)
    r_start = max(s_end, n_global - recent)
    forced = max(0, min(s_end - tok_offset, N)) + max(0, tok_offset + N - max(r_start, tok_offset))
    cap = max(1, min(N, k + forced))
    idx = torch.empty((B, KH, cap), dtype=torch.int32, device=dev)
    cnt = torch.empty((B, KH), dtype=torch.int32, device=dev)
    need = lib.sl_scan_topk_workspace_bytes(B, N, KH, QH)
    ws, status = workspaces.get("scan", dev, need, (B, KH, QH))
    check(lib.sl_scan_topk_sharded(q_codes.data_ptr(), k_codes.data_ptr(), kb, B, N, tok_offset, n_global, KH, QH, layout,
                                   k, sink, recent, idx.data_ptr(), cap, cnt.data_ptr(), ws.data_ptr(), ws.numel(),
                                   peer.bufs, peer.rank, peer.world, peer.nbytes, status.data_ptr(), _stream()))
    _count()
    return idx, cnt


def scan_sharded_slot_bytes(B: int, KH: int, QH: int) -> int:
    return int(lib.sl_scan_topk_sharded_slot_bytes(B, KH, QH))


def topk_from_scores(scores: torch.Tensor, k: int, max_score: int, sink: int = 0, recent: int = 0):
    """scores int16 [B,N,KH] in [0,max_score] -> (idx int32 [B,KH,cap] ascending, cnt int32 [B,KH])."""
    B, N, KH = scores.shape
    assert scores.dtype == torch.int16
    dev = _cuda(scores)
    scores = scores.contiguous()
    cap = max(1, min(N, k + sink + recent))
    idx = torch.empty((B, KH, cap), dtype=torch.int32, device=dev)
    cnt = torch.empty((B, KH), dtype=torch.int32, device=dev)
    need = lib.sl_topk_from_scores_workspace_bytes(B, N, KH, max_score)
    ws, status = workspaces.get("topk", dev, need, (B, KH, max_score))
    check(lib.sl_topk_from_scores(scores.data_ptr(), B, N, KH, max_score, k, sink, recent, idx.data_ptr(), cap,
                                  cnt.data_ptr(), ws.data_ptr(), ws.numel(), status.data_ptr(), _stream()))
    _count()
    return idx, cnt


def scan_hist(q_codes: torch.Tensor, k_codes: torch.Tensor, layout: int = GQA_BLOCKED):
    """Sequence-shard step 1: local scores int16 [B,N,KH] and local histogram uint32 [B,KH,nbins]."""
    if q_codes.dim() == 4:
        q_codes = q_codes[:, 0]
    B, QH, _ = q_codes.shape
    _, N, KH, _ = k_codes.shape
    dev = _cuda(q_codes, k_codes)
    q_codes = q_codes.contiguous()
    kb = _rows_view(k_codes, 4)
    nbins = 128 * (QH // KH) + 1
    scores = torch.empty((B, N, KH), dtype=torch.int16, device=dev)
    hist = torch.zeros((B, KH, nbins), dtype=torch.int32, device=dev)
    check(lib.sl_scan_hist(q_codes.data_ptr(), k_codes.data_ptr(), kb, B, N, KH, QH, layout, scores.data_ptr(),
                           hist.data_ptr(), _stream()))
    _count()
    return scores, hist


def select_emit(scores: torch.Tensor, hist_all: torch.Tensor, rank: int, tok_offset: int, n_global: int, QH: int,
                k: int, sink: int = 4, recent: int = 64):
    """Sequence-shard step 2: local attended indices from the all-gathered histograms
    hist_all [R,B,KH,nbins]."""
    B, N, KH = scores.shape
    R = hist_all.shape[0]
    dev = _cuda(scores, hist_all)
    hist_all = hist_all.contiguous()
    s_end = min(sink, n_global)
    r_start = max(s_end, n_global - recent)
    forced = max(0, min(s_end - tok_offset, N)) + max(0, tok_offset + N - max(r_start, tok_offset))
    cap = max(1, min(N, k + forced))
    idx = torch.empty((B, KH, cap), dtype=torch.int32, device=dev)
    cnt = torch.empty((B, KH), dtype=torch.int32, device=dev)
    need = lib.sl_select_emit_workspace_bytes(B, N, KH, QH)
    ws, status = workspaces.get("emit", dev, need, (B, KH, QH))
    check(lib.sl_select_emit(scores.data_ptr(), hist_all.data_ptr(), R, rank, B, N, tok_offset, n_global, KH, QH, k,
                             sink, recent, idx.data_ptr(), cap, cnt.data_ptr(), ws.data_ptr(), ws.numel(),
                             status.data_ptr(), _stream()))
    _count()
    return idx, cnt


# ----------------------------------------------------------------------------- hash stage
def decode_prepare(q: torch.Tensor, k: Optional[torch.Tensor], v: Optional[torch.Tensor], hash_q: HashParams,
                   hash_k: Optional[HashParams], pos: int, code_cache: Optional[torch.Tensor] = None,
                   k_cache: Optional[torch.Tensor] = None, v_cache: Optional[torch.Tensor] = None,
                   cos: Optional[torch.Tensor] = None, sin: Optional[torch.Tensor] = None,
                   q_rot: Optional[torch.Tensor] = None, q_codes: Optional[torch.Tensor] = None):
    """Stage 1 of a decode step in one launch (see sl_decode_prepare). q [B,QH,128], k/v [B,KH,128];
    caches are full pre-allocated tensors [B,Nmax,KH,*]; row `pos` of each is written.
    Returns (q_rot [B,QH,128], q_codes uint32 [B,QH,4])."""
    B, QH, D = q.shape
    assert D == 128
    dev = _cuda(q)
    q = q.contiguous()
    KH = 0 if k is None else k.shape[1]
    if q_rot is None:
        q_rot = torch.empty_like(q)
    if q_codes is None:
        q_codes = torch.empty((B, QH, 4), dtype=torch.uint32, device=dev)
    code_b = 0
    kv = _lib.KvLayout(0, max(KH, 1) * 128, 128, 1)
    if k is not None:
        k = k.contiguous()
        v = None if v is None else v.contiguous()
        assert code_cache is not None and code_cache.shape[0] == B and code_cache.shape[2:] == (KH, 4)
        assert pos < code_cache.shape[1], "code cache is full"
        code_b = _rows_view(code_cache, 4)
        if k_cache is not None:
            assert pos < k_cache.shape[1], "kv cache is full"
            kv = _kv_layout(k_cache)
            if v_cache is not None:
                kv2 = _kv_layout(v_cache)
                assert (kv2.batch_stride, kv2.token_stride, kv2.head_stride) == (kv.batch_stride, kv.token_stride, kv.head_stride)
    check(lib.sl_decode_prepare_ex(q.data_ptr(), _ptr(k), _ptr(v), _dt(q), B, QH, KH, _ptr(cos), _ptr(sin),
                                   hash_q.ref(), hash_k.ref() if hash_k is not None else None, q_rot.data_ptr(),
                                   q_codes.data_ptr(), _ptr(code_cache), code_b, _ptr(k_cache), _ptr(v_cache), C.byref(kv),
                                   pos, _stream()))
    _count()
    return q_rot, q_codes


def hash_encode(x: torch.Tensor, params: HashParams, out: Optional[torch.Tensor] = None) -> torch.Tensor:
    """x [B,T,H,128] -> codes uint32 [B,T,H,4] (hash + sign + pack)."""
    B, T, H, D = x.shape
    assert D == 128 and H == params.heads
    dev = _cuda(x)
    xl = _kv_layout(x)
    if out is None:
        out = torch.empty((B, T, H, 4), dtype=torch.uint32, device=dev)
    ob = _rows_view(out, 4)
    check(lib.sl_hash_encode_ex(x.data_ptr(), xl.batch_stride, xl.token_stride, xl.head_stride, _dt(x), B, T, H,
                                params.ref(), out.data_ptr(), ob, _stream()))
    _count()
    return out


# ----------------------------------------------------------------------------- attention
def sparse_attn_decode(q: torch.Tensor, k_cache: torch.Tensor, v_cache: torch.Tensor, idx: torch.Tensor,
                       cnt: torch.Tensor, layout: int = GQA_BLOCKED, out: Optional[torch.Tensor] = None,
                       return_lse: bool = False):
    """q [B,QH,128]; k_cache/v_cache [B,N,KVH,128] views with any batch / token / head strides (two
    caches, the halves of a fused [B,N,KVH,2,128] cache, an ``expand``-ed batch);
    idx int32 [B,LH,cap], cnt int32 [B,LH] -> out [B,QH,128] (+ lse float [B,QH]).
    LH = KVH is the per-kv-head selection; LH = QH (a multiple of KVH) gives every query head its own
    list over the shared K/V (query head j reads kv head j // (QH / KVH))."""
    B, QH, D = q.shape
    KVH = k_cache.shape[2]
    LH = idx.shape[1]
    assert D == 128 and k_cache.dtype == q.dtype and v_cache.dtype == q.dtype
    assert LH % KVH == 0 and QH % LH == 0, "index lists must be per kv head or per query head"
    dev = _cuda(q, k_cache, v_cache, idx, cnt)
    q = q.contiguous()
    kv = _kv_layout(k_cache, LH // KVH)
    kv2 = _kv_layout(v_cache)
    assert (kv2.batch_stride, kv2.token_stride, kv2.head_stride) == (kv.batch_stride, kv.token_stride, kv.head_stride)
    assert idx.is_contiguous() and cnt.is_contiguous() and idx.dtype == torch.int32 and cnt.dtype == torch.int32
    if out is None:
        out = torch.empty_like(q)
    lse = torch.empty((B, QH), dtype=torch.float32, device=dev) if return_lse else None
    need = lib.sl_sparse_attn_workspace_bytes(B, LH, QH)
    ws, _ = workspaces.get("attn", dev, need, (B, LH, QH))
    check(lib.sl_sparse_attn_decode_ex(q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(), _dt(q), C.byref(kv),
                                       idx.data_ptr(), idx.shape[2], cnt.data_ptr(), B, LH, QH, layout,
                                       out.data_ptr(), _ptr(lse), ws.data_ptr(), ws.numel(), _stream()))
    _count()
    return (out, lse) if return_lse else out


def sparse_attn_decode_fill(q: torch.Tensor, table: "LruTable", slots: torch.Tensor, idx: torch.Tensor, cnt: torch.Tensor,
                            k_backing: Optional[torch.Tensor], v_backing: Optional[torch.Tensor], layout: int = GQA_BLOCKED,
                            out: Optional[torch.Tensor] = None, return_lse: bool = False, backing_ptrs=None,
                            read_only: bool = False):
    """Attention over the resident buffers of an LRU table with the slot list of lru_update(..., defer_copy=True):
    the rows of the entries -(slot + 1) are fetched from the backing store (k_backing / v_backing [B,N,KH,128] views,
    or backing_ptrs=(k_ptr, v_ptr, batch_stride_elems) for mapped pinned host memory) at the keys idx names, and
    written into their slots on the way. bf16. Same arithmetic as sparse_attn_decode over the full caches.
    read_only: the slot list comes from lru_probe (misses are -1); their rows are only read, lru_evict fills the slots."""
    B, QH, D = q.shape
    KH = table.KH
    assert D == 128 and q.dtype == torch.bfloat16 and table.k.dtype == q.dtype
    dev = _cuda(q, table.k, slots, idx, cnt)
    q = q.contiguous()
    assert slots.is_contiguous() and idx.is_contiguous() and cnt.is_contiguous() and slots.shape == idx.shape
    res = _kv_layout(table.k)
    if backing_ptrs is None:
        back = _kv_layout(k_backing)
        b2 = _kv_layout(v_backing)
        assert (b2.batch_stride, b2.token_stride, b2.head_stride) == (back.batch_stride, back.token_stride, back.head_stride)
        kp, vp = k_backing.data_ptr(), v_backing.data_ptr()
    else:
        kp, vp, kb = backing_ptrs
        back = _lib.KvLayout(kb, KH * 128, 128, 1)
    fill = _lib.AttnFill(idx.data_ptr(), kp, vp, back, 1 if read_only else 0)
    if out is None:
        out = torch.empty_like(q)
    lse = torch.empty((B, QH), dtype=torch.float32, device=dev) if return_lse else None
    need = lib.sl_sparse_attn_workspace_bytes(B, KH, QH)
    ws, _ = workspaces.get("attn", dev, need, (B, KH, QH))
    check(lib.sl_sparse_attn_decode_fill(q.data_ptr(), table.k.data_ptr(), table.v.data_ptr(), _dt(q), C.byref(res),
                                         slots.data_ptr(), slots.shape[2], cnt.data_ptr(), B, KH, QH, layout, out.data_ptr(),
                                         _ptr(lse), ws.data_ptr(), ws.numel(), C.byref(fill), _stream()))
    _count()
    return (out, lse) if return_lse else out


def _lru_ws(table: "LruTable", B, KH, cap, dev):
    need = lib.sl_lru_workspace_bytes(B, KH, cap)
    if table.ws is None or table.ws.numel() < need:
        table.ws = torch.zeros(need, dtype=torch.uint8, device=dev)
    return table.ws


def lru_probe(table: "LruTable", idx: torch.Tensor, cnt: torch.Tensor, slots_out: Optional[torch.Tensor] = None,
              step_dev: Optional[torch.Tensor] = None) -> torch.Tensor:
    """First half of stage 3: hits are stamped and their slots returned, misses come back as -1 and are left in the
    table's workspace for lru_evict (which must follow before the table's next probe)."""
    B, KH, cap = idx.shape
    dev = _cuda(idx, cnt, table.k)
    if slots_out is None:
        slots_out = torch.empty_like(idx)
    res = _kv_layout(table.k)
    ws = _lru_ws(table, B, KH, cap, dev)
    check(lib.sl_lru_probe(idx.data_ptr(), cap, cnt.data_ptr(), B, KH, table.k.element_size(), table.k.data_ptr(),
                           table.v.data_ptr(), C.byref(res), table.C, table.tok2slot.data_ptr(), table.n_max,
                           table.slot2tok.data_ptr(), table.last_used.data_ptr(), table.step, _ptr(step_dev),
                           slots_out.data_ptr(), table.status.data_ptr(), ws.data_ptr(), ws.numel(), _stream()))
    _count()
    return slots_out


def lru_evict(table: "LruTable", idx: torch.Tensor, cnt: torch.Tensor, k_backing: torch.Tensor, v_backing: torch.Tensor,
              slots: torch.Tensor, step_dev: Optional[torch.Tensor] = None) -> None:
    """Second half of stage 3: victims for the misses lru_probe recorded, table update, copy of the missed rows into
    their slots. Does not touch `slots`; may run on another stream beside sparse_attn_decode_fill(read_only=True)."""
    B, KH, cap = idx.shape
    dev = _cuda(idx, cnt, table.k)
    back, res = _kv_layout(k_backing), _kv_layout(table.k)
    ws = _lru_ws(table, B, KH, cap, dev)
    check(lib.sl_lru_evict(idx.data_ptr(), cap, cnt.data_ptr(), B, KH, k_backing.data_ptr(), v_backing.data_ptr(), C.byref(back),
                           table.k.element_size(), table.k.data_ptr(), table.v.data_ptr(), C.byref(res), table.C,
                           table.tok2slot.data_ptr(), table.n_max, table.slot2tok.data_ptr(), table.last_used.data_ptr(),
                           table.step, _ptr(step_dev), slots.data_ptr(), table.stats.data_ptr(), table.status.data_ptr(),
                           ws.data_ptr(), ws.numel(), _stream()))
    if step_dev is None:
        table.step += 1
    _count(2)


class LruTable:
    """Resident K/V buffers and the slot tables of one layer (see sl_lru_update). The buffers are
    [B,C,KH,128] each, or -- fused=True -- the halves of one [B,C,KH,2,128] buffer, in which a slot's K and
    V rows are adjacent like the rows of a fused cache."""

    def __init__(self, batch: int, kv_heads: int, n_max: int, slots: int, dtype: torch.dtype, device, fused: bool = False):
        self.B, self.KH, self.n_max, self.C = batch, kv_heads, n_max, slots
        if fused:
            self.kv = torch.zeros((batch, slots, kv_heads, 2, 128), dtype=dtype, device=device)
            self.k, self.v = self.kv[:, :, :, 0], self.kv[:, :, :, 1]
        else:
            self.k = torch.zeros((batch, slots, kv_heads, 128), dtype=dtype, device=device)
            self.v = torch.zeros((batch, slots, kv_heads, 128), dtype=dtype, device=device)
        self.tok2slot = torch.full((batch, kv_heads, n_max), -1, dtype=torch.int32, device=device)
        self.slot2tok = torch.full((batch, kv_heads, slots), -1, dtype=torch.int32, device=device)
        self.last_used = torch.full((batch, kv_heads, slots), -1, dtype=torch.int32, device=device)
        self.stats = torch.zeros((batch, kv_heads, 2), dtype=torch.int32, device=device)
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        self.ws = None              # workspace of the multi-CTA probe, sized at the first update
        self.step = 0


def lru_update(table: LruTable, idx: torch.Tensor, cnt: torch.Tensor, k_backing: torch.Tensor,
               v_backing: torch.Tensor, slots_out: Optional[torch.Tensor] = None, backing_ptrs=None,
               step_dev: Optional[torch.Tensor] = None, defer_copy: bool = False) -> torch.Tensor:
    """Make this step's attended keys resident; returns their slots int32 [B,KH,cap] in list order.
    defer_copy: only the tables are updated; the slots of the misses come back as -(slot + 1) and the
    sparse_attn_decode_fill call that must follow fetches those rows and fills the slots on the way.
    k_backing / v_backing: [B,N,KH,128] device tensors (views of a larger or fused cache are fine), or pass
    backing_ptrs=(k_ptr, v_ptr, batch_stride_elems) for mapped pinned host memory in the two-cache layout.
    step_dev: int64 device tensor holding the step (the table's clock), e.g. the decode position, so that
    a replayed CUDA graph advances it; else the table's host-side counter is used and incremented."""
    B, KH, cap = idx.shape
    dev = _cuda(idx, cnt, table.k)
    assert idx.is_contiguous() and cnt.is_contiguous() and (B, KH) == (table.B, table.KH)
    if slots_out is None:
        slots_out = torch.empty_like(idx)
    if defer_copy:
        kp = vp = back = None
    elif backing_ptrs is None:
        back = _kv_layout(k_backing)
        b2 = _kv_layout(v_backing)
        assert (b2.batch_stride, b2.token_stride, b2.head_stride) == (back.batch_stride, back.token_stride, back.head_stride)
        assert k_backing.dtype == table.k.dtype
        kp, vp = k_backing.data_ptr(), v_backing.data_ptr()
    else:
        kp, vp, kb = backing_ptrs
        back = _lib.KvLayout(kb, KH * 128, 128, 1)
    res = _kv_layout(table.k)
    need = lib.sl_lru_workspace_bytes(B, KH, cap)
    if table.ws is None or table.ws.numel() < need:
        table.ws = torch.zeros(need, dtype=torch.uint8, device=dev)
    if defer_copy:
        check(lib.sl_lru_update_deferred(idx.data_ptr(), cap, cnt.data_ptr(), B, KH, table.k.element_size(),
                                         table.k.data_ptr(), table.v.data_ptr(), C.byref(res), table.C,
                                         table.tok2slot.data_ptr(), table.n_max, table.slot2tok.data_ptr(),
                                         table.last_used.data_ptr(), table.step, _ptr(step_dev), slots_out.data_ptr(),
                                         table.stats.data_ptr(), table.status.data_ptr(), table.ws.data_ptr(),
                                         table.ws.numel(), _stream()))
        if step_dev is None:
            table.step += 1
        _count()
        return slots_out
    check(lib.sl_lru_update_ex(idx.data_ptr(), cap, cnt.data_ptr(), B, KH, kp, vp, C.byref(back), table.k.element_size(),
                               table.k.data_ptr(), table.v.data_ptr(), C.byref(res), table.C, table.tok2slot.data_ptr(),
                               table.n_max, table.slot2tok.data_ptr(), table.last_used.data_ptr(), table.step,
                               _ptr(step_dev), slots_out.data_ptr(), table.stats.data_ptr(), table.status.data_ptr(),
                               table.ws.data_ptr(), table.ws.numel(), _stream()))
    if step_dev is None:
        table.step += 1
    _count(2)        # the update and the row copy
    return slots_out


def merge_lse(o_parts: torch.Tensor, lse_parts: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """o_parts float [R,...,128], lse_parts float [R,...] -> merged [...,128] of `dtype`."""
    R = o_parts.shape[0]
    dev = _cuda(o_parts, lse_parts)
    o_parts = o_parts.contiguous().float()
    lse_parts = lse_parts.contiguous().float()
    rows = lse_parts[0].numel()
    out = torch.empty(o_parts.shape[1:], dtype=dtype, device=dev)
    check(lib.sl_merge_lse(o_parts.data_ptr(), lse_parts.data_ptr(), R, rows, _DTYPES[dtype], out.data_ptr(), _stream()))
    _count()
    return out


def gather_rows(cache: torch.Tensor, idx: torch.Tensor, budget: int, device=None) -> torch.Tensor:
    """cache [B,N,KH,128], idx int32 [B,KH,cap] -> [B,budget,KH,128] with
    out[b,j,h] = cache[b, idx[b,h,j], h]. The cache may be PINNED host memory (the kernel then pulls
    the selected rows across PCIe); the result is on the device of idx."""
    B, N, KH, D = cache.shape
    assert D == 128
    if cache.is_cuda:
        dev = _cuda(cache, idx)
    else:
        if not cache.is_pinned():
            raise RuntimeError("a host-resident cache must be pinned memory so that the GPU can address it")
        dev = _cuda(idx)
    cb = _rows_view(cache, 128)
    out = torch.empty((B, budget, KH, D), dtype=cache.dtype, device=dev)
    check(lib.sl_gather_rows(cache.data_ptr(), cb, cache.element_size(), idx.data_ptr(), idx.shape[2], B, KH, budget,
                             out.data_ptr(), _stream()))
    _count()
    return out
