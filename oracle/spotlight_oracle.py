"""CPU restatement of the reference's decode-time retrieval path.  TEST INFRASTRUCTURE ONLY.

This module is the checker the CUDA path is compared against. Only the test-suite, the smoke
check and the benchmark's CPU-baseline / reference arm may import it; the product package
(``spotlight_b200``) never does and fails loudly when its CUDA library is missing.

Parity status: PINNED. ``tests/golden/*.npz`` were produced by running the reference's own
functions (``get_attn_score_using_angle_lsh``, ``MLPHashingFunction``, ``LinearHashingFunction``,
``do_sdpa_attn``, ``check_and_apply_qk_rope``) imported from the reference tree on seeded
inputs (``tests/golden/make_golden.py``); ``tests/test_oracle_golden.py`` checks every function
here against them. The only known-answer check inside the reference itself, the shift/add
formula of spotlight/kernel/pack_dx_u8.py:62-67, is restated in ``pack_signbits_u8``.

Each function cites the reference file:line it follows. Integer work is numpy; floating-point
work is torch on the CPU so that rounding follows the reference's own operators.
"""
from __future__ import annotations

import math
from typing import List, Optional, Sequence, Tuple

import numpy as np
import torch

INTERLEAVED = 0   # kv head h is scored against q heads {g*KH + h}   (reference kernels)
BLOCKED = 1       # kv head h is scored against q heads {h*G + g}    (HF repeat_kv / flash-attn)


# --------------------------------------------------------------------------------------
# budget rule
# --------------------------------------------------------------------------------------
def budget(n: int, mask_out: float, min_remain: int = 20) -> int:
    """spotlight/modifiers/spotlight_generation.py:162-164 (Python double arithmetic)."""
    num_remain = n - int(n * mask_out)
    return max(min(n, min_remain), num_remain)


# --------------------------------------------------------------------------------------
# sign-bit packing
# --------------------------------------------------------------------------------------
def pack_signbits(x) -> np.ndarray:
    """bit j of word i  <=>  x[..., 32*i + j] > 0, LSB first.
    spotlight/kernel/packbits.cu:19-25, spotlight/kernel/pack_dx_u32.py:27-28."""
    if isinstance(x, torch.Tensor):
        x = x.detach().to(torch.float32).cpu().numpy() if x.dtype != torch.bool else x.cpu().numpy()
    x = np.asarray(x)
    assert x.shape[-1] % 32 == 0
    bits = (x > 0).reshape(*x.shape[:-1], x.shape[-1] // 32, 32).astype(np.uint64)
    weights = (np.uint64(1) << np.arange(32, dtype=np.uint64))
    return (bits * weights).sum(-1).astype(np.uint32)


def pack_signbits_u8(x) -> np.ndarray:
    """8-bit variant: the shift/add known-answer formula of spotlight/kernel/pack_dx_u8.py:62-67."""
    if isinstance(x, torch.Tensor):
        x = x.detach().to(torch.float32).cpu().numpy() if x.dtype != torch.bool else x.cpu().numpy()
    x = np.asarray(x)
    assert x.shape[-1] % 8 == 0
    b = (x > 0).reshape(*x.shape[:-1], x.shape[-1] // 8, 8)
    ref = np.zeros(b.shape[:-1], dtype=np.uint8)
    for i in range(8):
        ref += (b[..., i].astype(np.uint8) << i).astype(np.uint8)
    return ref


# --------------------------------------------------------------------------------------
# Hamming match count
# --------------------------------------------------------------------------------------
def q_head_of(g: int, h: int, kv_heads: int, group: int, layout: int) -> int:
    return g * kv_heads + h if layout == INTERLEAVED else h * group + g


def match_count(q_codes: np.ndarray, k_codes: np.ndarray, layout: int = INTERLEAVED) -> np.ndarray:
    """out[b,n,h] = sum_g sum_w popc(~(q[b,0,qh(g,h),w] ^ k[b,n,h,w])), int16.
    spotlight/kernel/attn_k4_q28.cu:72-94 (interleaved grouping, ``q_base = (g*KH + h)*D``),
    spotlight/kernel/attn_dx_u32.py:110-128."""
    q_codes = np.asarray(q_codes, dtype=np.uint32)
    k_codes = np.asarray(k_codes, dtype=np.uint32)
    B, QN, QH, W = q_codes.shape
    _, N, KH, _ = k_codes.shape
    assert QN == 1 and QH % KH == 0
    G = QH // KH
    out = np.zeros((B, N, KH), dtype=np.int32)
    for g in range(G):
        qh = [q_head_of(g, h, KH, G, layout) for h in range(KH)]
        qg = q_codes[:, 0, qh, :]                                   # [B,KH,W]
        x = ~(qg[:, None, :, :] ^ k_codes)                          # [B,N,KH,W]
        out += np.bitwise_count(x).astype(np.int32).sum(-1)
    return out.astype(np.int16)


def match_count_u8(q_codes: np.ndarray, k_codes: np.ndarray) -> np.ndarray:
    """Per-head (no group sum) 8-bit variant: q [B,H,1,D] u8, k [B,H,N,D] u8 -> u8 [B,H,N].
    spotlight/kernel/attn_dx_u8.py:33-43 (and the commented torch twin at :77-88)."""
    q = np.asarray(q_codes, dtype=np.uint8)
    k = np.asarray(k_codes, dtype=np.uint8)
    x = ~(q ^ k)                                                     # broadcast over N
    return np.bitwise_count(x).astype(np.int32).sum(-1).astype(np.uint8)


def sign_sim(hq: torch.Tensor, hk: torch.Tensor) -> torch.Tensor:
    """Modifier-path score ``sign(hq) @ sign(hk)^T``; spotlight_generation.py:19-22."""
    return torch.sign(hq) @ torch.sign(hk).transpose(-1, -2)


# --------------------------------------------------------------------------------------
# selection
# --------------------------------------------------------------------------------------
def canonical_topk(scores: np.ndarray, k: int) -> np.ndarray:
    """Indices of the k largest scores of a 1-D array, ties broken by lowest index, returned
    ascending. The reference calls ``torch.topk`` (spotlight_generation.py:157-165,
    gpu_cache.py:50) whose tie order is unspecified; this is the canonical choice."""
    scores = np.asarray(scores)
    k = min(int(k), scores.shape[0])
    order = np.argsort(-scores.astype(np.int64), kind="stable")[:k]
    return np.sort(order).astype(np.int32)


def forced_ranges(n: int, sink: int, recent: int) -> Tuple[int, int]:
    """Always-kept ranges for the decode query at position n-1: keys [0, s_end) and
    [r_start, n); spotlight/modifiers/spotlight_evaluation.py:341-346 with q_idx = n-1."""
    s_end = min(sink, n)
    r_start = max(s_end, n - recent)
    return s_end, r_start


def attended_set(scores: np.ndarray, k: int, sink: int = 4, recent: int = 64) -> np.ndarray:
    """top-k over ALL keys, then OR-in the sink and recent ranges; ascending, no duplicates."""
    n = scores.shape[0]
    s_end, r_start = forced_ranges(n, sink, recent)
    top = canonical_topk(scores, k)
    forced = np.concatenate([np.arange(0, s_end), np.arange(r_start, n)]).astype(np.int32)
    return np.union1d(top, forced).astype(np.int32)


def select(scores: np.ndarray, k: int, sink: int = 4, recent: int = 64):
    """scores int16 [B,N,KH] -> (idx int32 [B,KH,cap] padded with -1, cnt int32 [B,KH]),
    cap = min(N, k+sink+recent)."""
    B, N, KH = scores.shape
    cap = min(N, k + sink + recent)
    idx = np.full((B, KH, cap), -1, dtype=np.int32)
    cnt = np.zeros((B, KH), dtype=np.int32)
    for b in range(B):
        for h in range(KH):
            s = attended_set(scores[b, :, h], k, sink, recent)
            idx[b, h, : len(s)] = s
            cnt[b, h] = len(s)
    return idx, cnt


def exact_logits(q_rot: torch.Tensor, k_rot: torch.Tensor, per_query_head: bool) -> np.ndarray:
    """The oracle-selection baseline's scores (spotlight/modifiers/upperbound_generation.py:12-15:
    ``query @ key.transpose(-1,-2)`` on rotated q and k, keys repeated to the query heads): fp64 logits
    [B,QH,N] for q_rot [B,QH,D], k_rot [B,N,KH,D]; with per_query_head False the logits of the query
    heads of a group are added up, [B,KH,N] (the per-kv-head counterpart used by this library)."""
    B, QH, D = q_rot.shape
    KH = k_rot.shape[2]
    G = QH // KH
    qg = q_rot.to(torch.float64).view(B, KH, G, D)
    lg = torch.einsum("bhgd,bnhd->bhgn", qg, k_rot.to(torch.float64))
    lg = lg.reshape(B, QH, -1) if per_query_head else lg.sum(dim=2)
    return lg.numpy()


def select_by_logits(logits: np.ndarray, k: int, sink: int = 4, recent: int = 64):
    """Exact top-k of real-valued scores [B,H,N] (ties, should there be any, to the lowest index) plus the
    sink / recent ranges -> (idx int32 [B,H,cap] padded with -1, cnt int32 [B,H]); the selection of
    spotlight/modifiers/upperbound_generation.py:140-150 with the window of
    spotlight_evaluation.py:341-346."""
    B, H, N = logits.shape
    cap = min(N, k + sink + recent)
    idx = np.full((B, H, cap), -1, dtype=np.int32)
    cnt = np.zeros((B, H), dtype=np.int32)
    s_end, r_start = forced_ranges(N, sink, recent)
    forced = np.concatenate([np.arange(0, s_end), np.arange(r_start, N)]).astype(np.int32)
    for b in range(B):
        for h in range(H):
            top = np.sort(np.argsort(-logits[b, h], kind="stable")[: min(k, N)])
            s = np.union1d(top, forced).astype(np.int32)
            idx[b, h, : len(s)] = s
            cnt[b, h] = len(s)
    return idx, cnt


def iou(a: np.ndarray, b: np.ndarray) -> float:
    """Intersection over union of two index sets (the per-head figure of the reference's bench_mark
    mode, spotlight/modifiers/spotlight_evaluation.py:303-316)."""
    a, b = set(np.asarray(a).tolist()), set(np.asarray(b).tolist())
    return len(a & b) / max(1, len(a | b))


def histogram(scores: np.ndarray, nbins: int) -> np.ndarray:
    """Per-(b,h) histogram of match counts, int64 [B,KH,nbins]."""
    B, N, KH = scores.shape
    out = np.zeros((B, KH, nbins), dtype=np.int64)
    for b in range(B):
        for h in range(KH):
            out[b, h] = np.bincount(scores[b, :, h].astype(np.int64), minlength=nbins)
    return out


def threshold_from_hist(hist: np.ndarray, k: int) -> Tuple[int, int]:
    """(tau, r): tau = largest s with #(score >= s) >= k; r = k - #(score > tau) ties to take."""
    n = int(hist.sum())
    k = min(k, n)
    if k <= 0:
        return len(hist), 0
    suffix = np.cumsum(hist[::-1])[::-1]                # suffix[s] = #(score >= s)
    tau = int(np.nonzero(suffix >= k)[0].max())
    gt = int(suffix[tau + 1]) if tau + 1 < len(hist) else 0
    return tau, k - gt


def sharded_select(score_shards: Sequence[np.ndarray], k: int, sink: int = 4, recent: int = 64):
    """Sequence-sharded exact selection: shard r holds scores of the contiguous token range r.
    Every shard histograms locally; the summed histogram gives the global threshold; ties are
    granted to shards in rank order (lower rank = lower indices), which reproduces the
    lowest-index tie rule of ``attended_set``. Returns per-shard lists of GLOBAL indices for one
    (b,h) column given 1-D shards."""
    sizes = [len(s) for s in score_shards]
    n = sum(sizes)
    nb = int(max(int(s.max()) if len(s) else 0 for s in score_shards)) + 1
    hists = [np.bincount(s.astype(np.int64), minlength=nb) for s in score_shards]
    tau, r = threshold_from_hist(np.sum(hists, axis=0), k)
    s_end, r_start = forced_ranges(n, sink, recent)
    out, off, ties_before = [], 0, 0
    for s, h in zip(score_shards, hists):
        gidx = np.arange(off, off + len(s))
        eq = (s == tau) if tau < nb else np.zeros(len(s), bool)
        rank = ties_before + np.cumsum(eq) - 1
        sel = (s > tau) | (eq & (rank < r)) | (gidx < s_end) | (gidx >= r_start)
        out.append(gidx[sel].astype(np.int32))
        ties_before += int(eq.sum())
        off += len(s)
    return out


# --------------------------------------------------------------------------------------
# RoPE and hash modules (floating point: torch on CPU)
# --------------------------------------------------------------------------------------
def rope_tables(n: int, theta: float, dim: int = 128):
    inv_freq = 1.0 / (theta ** (torch.arange(0, dim, 2, dtype=torch.float32) / dim))
    freqs = torch.arange(n, dtype=torch.float32)[:, None] * inv_freq[None, :]
    emb = torch.cat([freqs, freqs], dim=-1)
    return emb.cos(), emb.sin()


def rotate_half(x: torch.Tensor) -> torch.Tensor:
    h = x.shape[-1] // 2
    return torch.cat([-x[..., h:], x[..., :h]], dim=-1)


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, positions) -> torch.Tensor:
    """x [B,H,n,128]; ``x*cos[pos] + rotate_half(x)*sin[pos]``; modify_llama.py:54-59."""
    c = cos[positions].to(x.dtype)[None, None]
    s = sin[positions].to(x.dtype)[None, None]
    return x * c + rotate_half(x) * s


def hash_forward(x: torch.Tensor, params: dict, residue: bool = True) -> torch.Tensor:
    """x [B,H,n,in] in the run dtype; params from workloads.make_hash_params ([H,in,out], [H,out]).
    linear: ``x @ W``  (linearhashing_generation.py:230-231).
    mlp: per layer ``dx = act(x @ W + b)``, SiLU on all but the last layer, ``dx + x`` when
    residue  (spotlight_generation.py:238-240, 252-255)."""
    if params["kind"] == "linear":
        return x @ params["w"][0][None]
    L = len(params["w"])
    for i, (w, b) in enumerate(zip(params["w"], params["b"])):
        dx = x @ w[None] + b[None, :, None, :]
        if i < L - 1:
            dx = torch.nn.functional.silu(dx)
        x = dx + x if residue else dx
    return x


def hash_codes(x: torch.Tensor, params: dict, residue: bool = True):
    """(codes u32 [B,H,n,4], pre-sign activations) for x [B,H,n,128]."""
    y = hash_forward(x, params, residue)
    return pack_signbits(y), y


# --------------------------------------------------------------------------------------
# attention
# --------------------------------------------------------------------------------------
def sparse_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, idx: np.ndarray,
                     cnt: np.ndarray, layout: int = BLOCKED, return_lse: bool = False):
    """softmax(q.K_sel^T / sqrt(d)) V_sel over the selected rows only, accumulated in fp64.
    q [B,QH,D], k/v [B,N,KH,D], idx [B,KH,cap], cnt [B,KH] -> fp32 [B,QH,D].
    Equals the reference's additive ``finfo.min`` mask + dense SDPA (spotlight_generation.py:
    200-215, modify_llama.py:172-180): masked keys contribute exp(-inf)=0."""
    B, QH, D = q.shape
    KH = k.shape[2]
    G = QH // KH
    out = torch.zeros((B, QH, D), dtype=torch.float64)
    lse = torch.zeros((B, QH), dtype=torch.float64)
    scale = 1.0 / math.sqrt(D)
    for b in range(B):
        for h in range(KH):
            sel = torch.from_numpy(idx[b, h, : cnt[b, h]].astype(np.int64))
            ks = k[b, sel, h].to(torch.float64)
            vs = v[b, sel, h].to(torch.float64)
            for g in range(G):
                qh = q_head_of(g, h, KH, G, layout)
                logits = (ks @ q[b, qh].to(torch.float64)) * scale
                m = logits.max()
                p = torch.exp(logits - m)
                out[b, qh] = (p[:, None] * vs).sum(0) / p.sum()
                lse[b, qh] = m + torch.log(p.sum())
    if return_lse:
        return out.to(torch.float32), lse.to(torch.float32)
    return out.to(torch.float32)


def dense_masked_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, idx: np.ndarray,
                           cnt: np.ndarray, layout: int = BLOCKED) -> torch.Tensor:
    """The reference's literal formulation: a [*,N] additive mask filled with ``finfo.min``,
    zeroed at the attended indices, then torch SDPA over all N keys
    (spotlight_generation.py:200-205, modify_llama.py:172-180). q,k already rotated."""
    B, QH, D = q.shape
    N, KH = k.shape[1], k.shape[2]
    G = QH // KH
    qf = q.to(torch.float32)[:, :, None, :]                                   # [B,QH,1,D]
    kv_of = [0] * QH
    for h in range(KH):
        for g in range(G):
            kv_of[q_head_of(g, h, KH, G, layout)] = h
    kf = k.to(torch.float32).permute(0, 2, 1, 3)[:, kv_of]                    # [B,QH,N,D]
    vf = v.to(torch.float32).permute(0, 2, 1, 3)[:, kv_of]
    mask = torch.full((B, QH, 1, N), torch.finfo(torch.float32).min)
    for b in range(B):
        for qh in range(QH):
            h = kv_of[qh]
            mask[b, qh, 0, torch.from_numpy(idx[b, h, : cnt[b, h]].astype(np.int64))] = 0
    o = torch.nn.functional.scaled_dot_product_attention(qf, kf, vf, attn_mask=mask, is_causal=False)
    return o[:, :, 0, :]


def merge_partials(o: torch.Tensor, m: torch.Tensor, l: torch.Tensor) -> torch.Tensor:
    """Log-sum-exp merge of split attention partials: o [S,...,D] un-normalised accumulators
    (sum of exp(logit - m) * v), m [S,...] running maxima, l [S,...] sums of exp(logit - m)."""
    mg = m.max(dim=0).values
    w = torch.exp(m - mg[None])
    w = torch.where(torch.isfinite(m), w, torch.zeros_like(w))
    num = (o * w[..., None]).sum(0)
    den = (l * w).sum(0)
    return num / den[..., None]


# --------------------------------------------------------------------------------------
# whole path, kernel semantics (per-KV-head codes, group-summed score, per-KV-head top-k)
# --------------------------------------------------------------------------------------
def decode_path(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, hash_q: dict, hash_k: dict,
                mask_out: float, min_remain: int = 20, sink: int = 4, recent: int = 64,
                residue: bool = True, layout: int = BLOCKED, k_codes: Optional[np.ndarray] = None):
    """hash -> pack -> match count -> budget -> canonical top-k U sink U recent -> sparse
    attention. q [B,QH,D] and k,v [B,N,KH,D] are post-RoPE. Returns a dict of every stage."""
    B, N, KH, D = k.shape
    qc, q_pre = hash_codes(q[:, :, None, :], hash_q, residue)                 # [B,QH,1,4]
    if k_codes is None:
        kc, _ = hash_codes(k.permute(0, 2, 1, 3), hash_k, residue)            # [B,KH,N,4]
        k_codes = np.ascontiguousarray(kc.transpose(0, 2, 1, 3))              # [B,N,KH,4]
    q_codes = np.ascontiguousarray(qc.transpose(0, 2, 1, 3))                  # [B,1,QH,4]
    scores = match_count(q_codes, k_codes, layout)
    kk = budget(N, mask_out, min_remain)
    idx, cnt = select(scores, kk, sink, recent)
    out = sparse_attention(q, k, v, idx, cnt, layout)
    return {"q_codes": q_codes, "k_codes": k_codes, "scores": scores, "k": kk,
            "idx": idx, "cnt": cnt, "out": out, "q_pre": q_pre}


# --------------------------------------------------------------------------------------
# whole path, the reference modifier's own operator sequence (dense; used as the CPU baseline)
# --------------------------------------------------------------------------------------
def modifier_path_dense(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, hash_params: dict,
                        mask_out: float, min_remain: int = 20, sink: int = 4, recent: int = 64,
                        residue: bool = True, theta: float = 10000.0) -> torch.Tensor:
    """One decode layer-step exactly as the reference modifier spends its time
    (spotlight_generation.py:128-215): repeat_kv'd un-rotated K [1,H,N,D] -> RoPE of all keys ->
    hash of all keys -> sign -> [1,H,1,128]@[1,H,128,N] -> torch.topk -> mask fill + scatter ->
    RoPE again -> additive-mask dense SDPA. Inputs are PRE-RoPE: q [1,H,1,D], k,v [1,H,N,D]."""
    _, H, N, D = k.shape
    cos, sin = rope_tables(N, theta, D)
    cos, sin = cos.to(q.dtype), sin.to(q.dtype)
    pos = torch.arange(N)
    Q = apply_rope(q, cos, sin, pos[-1:])
    K = apply_rope(k, cos, sin, pos)
    sim = sign_sim(hash_forward(Q, hash_params, residue), hash_forward(K, hash_params, residue))
    kk = budget(N, mask_out, min_remain)
    top = sim.topk(k=kk, dim=-1).indices
    mask = torch.full((1, H, 1, N), torch.finfo(sim.dtype).min, dtype=sim.dtype)
    mask.scatter_(dim=-1, index=top, value=0)
    mask[..., : min(sink, N)] = 0
    mask[..., max(0, N - recent):] = 0
    Q = apply_rope(q, cos, sin, pos[-1:])
    K = apply_rope(k, cos, sin, pos)
    o = torch.nn.functional.scaled_dot_product_attention(Q, K, v, attn_mask=mask, is_causal=False)
    return o.transpose(1, 2).flatten(2)


# --------------------------------------------------------------------------------------
# LRU-resident KV buffer (no reference counterpart; the policy of sl_lru_update restated)
# --------------------------------------------------------------------------------------
class LruModel:
    """Slot table of ONE (batch row, kv head): hits are stamped, misses (in list order) take the
    least recently attended slot not used in this step -- never-used slots first, then by age in
    steps with ages above `age_max` counted as `age_max`, ties to the lowest slot index."""

    def __init__(self, n_max: int, slots: int, age_max: int = 1023):
        self.tok2slot = np.full(n_max, -1, np.int32)
        self.slot2tok = np.full(slots, -1, np.int32)
        self.last_used = np.full(slots, -1, np.int32)
        self.age_max = age_max
        self.step = 0

    def update(self, tokens: np.ndarray):
        t = self.step
        slots = self.tok2slot[tokens].copy()
        hit = slots >= 0
        self.last_used[slots[hit]] = t
        lu = self.last_used
        age = np.where(lu < 0, self.age_max + 1, np.minimum(t - lu, self.age_max))
        cand = np.nonzero(age > 0)[0]
        order = cand[np.argsort(-age[cand], kind="stable")]          # oldest first, lowest slot on ties
        m = int((~hit).sum())
        assert m <= len(order), "table too small for this step"
        victims = np.sort(order[:m])                                    # misses take victims in slot order
        for tok, v in zip(tokens[~hit], victims):
            old = self.slot2tok[v]
            if old >= 0:
                self.tok2slot[old] = -1
            self.tok2slot[tok] = v
            self.slot2tok[v] = tok
            self.last_used[v] = t
        slots[~hit] = victims
        self.step += 1
        return slots.astype(np.int32), int(hit.sum()), m
