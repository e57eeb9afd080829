"""Sequence-sharded decode attention (million-token contexts): every rank owns a contiguous
range of keys of every (batch row, kv head) and the ranks exchange two small messages per
layer-step:

  1. local Hamming scan + score histogram          -> all-gather of histograms  [R, B, KH, 128*G+1]
     every rank derives the SAME global threshold and takes its share of the threshold ties in
     rank order (lower rank = lower key index), which reproduces the single-device rule
     "k highest scores, ties to the lowest index" exactly;
  2. local sparse attention with log-sum-exp       -> all-gather of (o, lse)     [R, B, QH, 129]
     merged by log-sum-exp.

The sink keys live on the first rank(s), the recent window on the last; the kernels clip both
to the local range. The reference has no sequence parallelism (its only collectives are in
training, train.py:250-260); this module is new design on top of torch.distributed (NCCL on
GPUs). `backend` is the set of compute kernels: the CUDA ops by default; host-side tests swap in
a CPU implementation to exercise the collective logic with gloo."""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.distributed as dist


def shard_bounds(n_global: int, world: int, rank: int) -> Tuple[int, int]:
    """Contiguous key range [lo, hi) of a rank (sizes differ by at most one)."""
    return n_global * rank // world, n_global * (rank + 1) // world


def _all_gather(t: torch.Tensor, group) -> torch.Tensor:
    world = dist.get_world_size(group)
    out = torch.empty((world, *t.shape), dtype=t.dtype, device=t.device)
    dist.all_gather_into_tensor(out.view(-1), t.contiguous().view(-1), group=group)
    return out


class PeerBuffer:
    """One rank's exchange buffer ([world slots of nbytes][flags][epoch]) mapped into every rank of
    the group through CUDA IPC; the handles travel once, here, through torch.distributed. The ranks
    must be GPUs of one node. `bufs[r]` is rank r's buffer as seen from this process."""

    def __init__(self, nbytes: int, device: torch.device, group=None):
        import ctypes as C
        from ._lib import check, lib
        self._C, self._lib, self._check = C, lib, check
        self.rank, self.world = dist.get_rank(group), dist.get_world_size(group)
        self.nbytes = int(nbytes)
        assert self.nbytes % 16 == 0, "messages are sent in 16-byte units"
        self.device = device
        total = lib.sl_peer_buffer_bytes(self.world, self.nbytes)
        own = C.c_void_p()
        check(lib.sl_peer_alloc(total, C.byref(own)))
        self._own = own.value
        handle = C.create_string_buffer(64)
        check(lib.sl_peer_export(self._own, handle))
        handles = [None] * self.world
        dist.all_gather_object(handles, bytes(handle.raw), group=group)
        self.bufs = (C.c_void_p * self.world)()
        self._opened = []
        for r in range(self.world):
            if r == self.rank:
                self.bufs[r] = self._own
            else:
                ptr = C.c_void_p()
                check(lib.sl_peer_open(C.create_string_buffer(handles[r], 64), C.byref(ptr)))
                self.bufs[r] = ptr.value
                self._opened.append(ptr.value)
        self.status = torch.zeros(1, dtype=torch.int32, device=device)
        dist.barrier(group)                      # every buffer is mapped everywhere before the first store

    def check_status(self):
        code = int(self.status.item())
        if code:
            raise RuntimeError(f"peer exchange gave up waiting for another rank (status {code})")

    def close(self):
        for p in self._opened:
            self._lib.sl_peer_close(p)
        self._opened = []
        if self._own:
            self._lib.sl_peer_free(self._own)
            self._own = None


class PeerExchange(PeerBuffer):
    """All-gather of one fixed-size message per rank over peer memory (sl_peer_allgather): one
    kernel per exchange stores the message into every rank's buffer and waits (bounded) for the
    others. Same result as `_all_gather`, without a collective library on the critical path."""

    def _slots(self, dtype: torch.dtype, shape) -> torch.Tensor:
        """The own buffer's slots as a tensor [world, *shape] (no copy)."""
        class _Raw:
            pass
        raw = _Raw()
        raw.__cuda_array_interface__ = {"shape": (self.world * self.nbytes,), "typestr": "|u1",
                                        "data": (self._own, False), "version": 3}
        flat = torch.as_tensor(raw, device=self.device)
        return flat.view(dtype).view(self.world, *shape)

    def all_gather(self, t: torch.Tensor) -> torch.Tensor:
        t = t.contiguous()
        assert t.numel() * t.element_size() == self.nbytes, "message size is fixed at construction"
        stream = torch.cuda.current_stream(self.device).cuda_stream
        self._check(self._lib.sl_peer_allgather(t.data_ptr(), self.nbytes, self.bufs, self.rank, self.world,
                                                self.nbytes, self.status.data_ptr(), stream))
        return self._slots(t.dtype, t.shape)


    def merge_lse(self, o: torch.Tensor, lse: torch.Tensor) -> torch.Tensor:
        """This rank's partial (o [...,128], lse [...]) -> the merge of all ranks' partials, one launch
        (pack, exchange, log-sum-exp merge: sl_peer_merge_lse)."""
        from .ops import _dt
        o, lse = o.contiguous(), lse.contiguous()
        assert lse.dtype == torch.float32
        rows = o.numel() // 128
        assert rows * 129 * 4 <= self.nbytes, "partials do not fit the slot"
        out = torch.empty_like(o)
        stream = torch.cuda.current_stream(self.device).cuda_stream
        self._check(self._lib.sl_peer_merge_lse(o.data_ptr(), lse.data_ptr(), _dt(o), rows, self.bufs, self.rank,
                                                self.world, self.nbytes, out.data_ptr(), self.status.data_ptr(), stream))
        return out


def make_peer_exchange(B: int, KH: int, QH: int, device: torch.device, group=None, fused_scan: bool = True):
    """The peer buffers of a sequence-sharded step: (histograms, partials[, fused-scan buffer])."""
    from . import ops
    G = QH // KH
    ex = [PeerExchange(B * KH * (128 * G + 1) * 4, device, group), PeerExchange(B * QH * 129 * 4, device, group)]
    if fused_scan:
        ex.append(PeerBuffer(ops.scan_sharded_slot_bytes(B, KH, QH), device, group))
    return tuple(ex)


def sharded_decode_attention(q_rot: torch.Tensor, q_codes: torch.Tensor, codes_local: torch.Tensor,
                             k_local: torch.Tensor, v_local: torch.Tensor, tok_offset: int, n_global: int,
                             k_budget: int, sink: int = 4, recent: int = 64, layout: int = 1, group=None,
                             backend=None, return_selection: bool = False, exchange=None):
    """One layer-step on this rank. q_rot [B,QH,128], q_codes uint32 [B,QH,4] (identical on all
    ranks); codes_local [B,n_local,KH,4], k_local / v_local [B,n_local,KH,128]: this rank's keys
    [tok_offset, tok_offset + n_local). Returns the merged output [B,QH,128] (identical on all
    ranks) and, on request, this rank's attended LOCAL indices and counts. `exchange`: the tuple of
    make_peer_exchange (histograms, partials[, fused-scan buffer]) to use peer memory instead of the
    group's all-gathers; with the third buffer the scan, the histogram exchange and the emission are
    one launch (sl_scan_topk_sharded)."""
    if backend is None:
        from . import ops as backend
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    QH = q_rot.shape[1]
    if exchange and len(exchange) > 2:
        # one launch: local scan, histograms to the peers, wait for theirs, emit
        idx, cnt = backend.scan_topk_sharded(q_codes, codes_local, exchange[2], tok_offset, n_global, k_budget,
                                             sink, recent, layout)
    else:
        scores, hist = backend.scan_hist(q_codes, codes_local, layout)
        hist_all = exchange[0].all_gather(hist) if exchange else _all_gather(hist, group)
        idx, cnt = backend.select_emit(scores, hist_all, rank, tok_offset, n_global, QH, k_budget, sink, recent)
    o, lse = backend.sparse_attn_decode(q_rot, k_local, v_local, idx, cnt, layout, return_lse=True)
    if exchange:
        out = exchange[1].merge_lse(o, lse)                          # pack + exchange + merge in one launch
    else:
        packed = torch.cat([o.float(), lse[..., None]], dim=-1)      # one message: [B,QH,129]
        parts = _all_gather(packed, group)
        out = backend.merge_lse(parts[..., :128].contiguous(), parts[..., 128].contiguous(), q_rot.dtype)
    return (out, idx, cnt) if return_selection else out
