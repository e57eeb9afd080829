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


def sharded_decode_attention(q_rot: torch.Tensor, q_codes: torch.Tensor, codes_local: torch.Tensor,
                             k_local: torch.Tensor, v_local: torch.Tensor, tok_offset: int, n_global: int,
                             k_budget: int, sink: int = 4, recent: int = 64, layout: int = 1, group=None,
                             backend=None, return_selection: bool = False):
    """One layer-step on this rank. q_rot [B,QH,128], q_codes uint32 [B,QH,4] (identical on all
    ranks); codes_local [B,n_local,KH,4], k_local / v_local [B,n_local,KH,128]: this rank's keys
    [tok_offset, tok_offset + n_local). Returns the merged output [B,QH,128] (identical on all
    ranks) and, on request, this rank's attended LOCAL indices and counts."""
    if backend is None:
        from . import ops as backend
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    QH = q_rot.shape[1]
    scores, hist = backend.scan_hist(q_codes, codes_local, layout)
    hist_all = _all_gather(hist, group)
    idx, cnt = backend.select_emit(scores, hist_all, rank, tok_offset, n_global, QH, k_budget, sink, recent)
    o, lse = backend.sparse_attn_decode(q_rot, k_local, v_local, idx, cnt, layout, return_lse=True)
    packed = torch.cat([o.float(), lse[..., None]], dim=-1)          # one message: [B,QH,129]
    parts = _all_gather(packed, group)
    out = backend.merge_lse(parts[..., :128].contiguous(), parts[..., 128].contiguous(), q_rot.dtype)
    return (out, idx, cnt) if return_selection else out
