"""Drop-in for the reference's oracle-selection baseline (spotlight/modifiers/upperbound_generation.py):
the same hook and driver as the hashing modifiers, but the index source of a pruned layer is the
EXACT top-k of the attention logits ``q . K^T`` (:12-15, 140-150) instead of the Hamming top-k of hash
codes. It bounds from above what any hash can achieve, and gives an in-library quality figure: the
overlap (IoU) of the hashed selection with this one (``selection_iou``).

The logits are a plain batched matmul over the cached, already rotated keys (torch; the reference
uses ``query @ key.transpose``, :14): this modifier is a measuring stick, not a fast path. The
selected rows then go through the same sparse attention kernel as every other index source.
With ``gqa_mode = "query_head"`` every query head takes its own top-k, as the reference does after
``repeat_kv`` (:120-121); the default sums the logits over the query heads of a group and selects
per KV head, the counterpart of the hashing path's per-KV-head selection."""
from __future__ import annotations

import types

import torch

from ..workloads import budget
from .spotlight_generation import Spotlight


def exact_topk_indices(q_rot: torch.Tensor, keys: torch.Tensor, keep: int, sink: int, recent: int, per_query_head: bool):
    """q_rot [B,QH,128], keys [B,n,KH,128] (rotated) -> (idx int32 [B,LH,cap] ascending, cnt int32 [B,LH]):
    the `keep` largest logits per list head (per KV head: summed over the group), plus keys [0,sink) and
    [n-recent, n)."""
    B, QH, _ = q_rot.shape
    n, KH = keys.shape[1], keys.shape[2]
    G = QH // KH
    qg = q_rot.float().view(B, KH, G, 128)
    logits = torch.einsum("bhgd,bnhd->bhgn", qg, keys.float())                 # [B,KH,G,n]
    logits = logits.reshape(B, QH, n) if per_query_head else logits.sum(dim=2)
    LH = logits.shape[1]
    keep = min(keep, n)
    sel = torch.zeros((B, LH, n), dtype=torch.bool, device=q_rot.device)
    if keep > 0:
        sel.scatter_(2, logits.topk(keep, dim=-1).indices, True)
    sel[..., : min(sink, n)] = True
    sel[..., max(0, n - recent):] = True
    cnt = sel.sum(-1).to(torch.int32)
    cap = int(min(n, keep + sink + recent))
    # ascending indices of the selected keys, padded: a stable sort of "not selected" keeps the key order
    order = torch.sort((~sel).to(torch.int8), dim=-1, stable=True).indices[..., :cap]
    return order.to(torch.int32).contiguous(), cnt.contiguous()


def _select_indices(self, q_rot, st, n):
    kw = self.draft_kwargs
    keep = budget(n, kw["mask_out"], kw.get("min_remain", 20))
    per_q = kw.get("gqa_mode", "kv_head") == "query_head"
    return exact_topk_indices(q_rot, st.k[:, :n], keep, int(kw.get("sink", 4)), int(kw.get("recent", 64)), per_q)


class UpperBound(Spotlight):
    def __init__(self, model, save_ckp=None, load_ckp=None, config=None):
        super().__init__(model, save_ckp, load_ckp, config, hash_kind="exact")
        for layer in self.model.layers:
            layer.self_attn.select_indices = types.MethodType(_select_indices, layer.self_attn)


def selection_iou(idx_a: torch.Tensor, cnt_a: torch.Tensor, idx_b: torch.Tensor, cnt_b: torch.Tensor, n: int) -> torch.Tensor:
    """Intersection over union of two attended sets per (batch row, list head) -> float [B,LH]; the
    figure the reference's ``bench_mark`` mode reports per head (spotlight_evaluation.py:303-316)."""
    def mask(idx, cnt):
        B, H, cap = idx.shape
        m = torch.zeros((B, H, n + 1), dtype=torch.bool, device=idx.device)
        valid = torch.arange(cap, device=idx.device)[None, None, :] < cnt[..., None]
        m.scatter_(2, torch.where(valid, idx.long(), torch.full_like(idx, n, dtype=torch.long)), True)
        return m[..., :n]
    a, b = mask(idx_a, cnt_a), mask(idx_b, cnt_b)
    return (a & b).sum(-1).float() / (a | b).sum(-1).clamp(min=1).float()
