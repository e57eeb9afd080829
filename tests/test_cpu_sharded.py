"""world_size-2 (and 3) gloo runs of the sequence-sharded driver on the CPU. The compute kernels
are replaced by the CPU checker so that what is exercised is the host logic: shard bounds, the
two all-gathers, the tie quota across ranks and the log-sum-exp merge. The merged result must
equal the unsharded checker bit-for-bit in its index sets and within 1e-5 in its output."""
import os
import socket

import numpy as np
import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import spotlight_oracle as O


class CpuBackend:
    """The four ops the sharded driver calls, served by the checker."""

    @staticmethod
    def scan_hist(q_codes, codes_local, layout):
        qc = q_codes.view(torch.int32).numpy().view(np.uint32)[:, None]
        kc = codes_local.view(torch.int32).numpy().view(np.uint32)
        scores = O.match_count(qc, kc, layout)
        G = q_codes.shape[1] // codes_local.shape[2]
        hist = O.histogram(scores, 128 * G + 1).astype(np.int32)
        return torch.from_numpy(scores), torch.from_numpy(hist)

    @staticmethod
    def select_emit(scores, hist_all, rank, tok_offset, n_global, QH, k, sink, recent):
        s, H = scores.numpy(), hist_all.numpy().astype(np.int64)
        B, n, KH = s.shape
        s_end, r_start = O.forced_ranges(n_global, sink, recent)
        lists = [[None] * KH for _ in range(B)]
        for b in range(B):
            for h in range(KH):
                tau, r = O.threshold_from_hist(H[:, b, h].sum(0), k)
                ties_before = int(H[:rank, b, h, tau].sum()) if tau < H.shape[-1] else 0
                col = s[:, :, h][b]
                g = np.arange(tok_offset, tok_offset + n)
                eq = col == tau
                rank_of = ties_before + np.cumsum(eq) - 1
                sel = (col > tau) | (eq & (rank_of < r)) | (g < s_end) | (g >= r_start)
                lists[b][h] = np.nonzero(sel)[0].astype(np.int32)
        cap = max(1, max(len(x) for row in lists for x in row))
        idx = np.zeros((B, KH, cap), np.int32)
        cnt = np.zeros((B, KH), np.int32)
        for b in range(B):
            for h in range(KH):
                idx[b, h, : len(lists[b][h])] = lists[b][h]
                cnt[b, h] = len(lists[b][h])
        return torch.from_numpy(idx), torch.from_numpy(cnt)

    @staticmethod
    def sparse_attn_decode(q, k, v, idx, cnt, layout, return_lse=True):
        B, QH, _ = q.shape
        out, lse = O.sparse_attention(q, k, v, idx.numpy(), cnt.numpy(), layout, return_lse=True)
        empty = (cnt.numpy() == 0)
        if empty.any():                                      # a shard may hold no attended key of a head
            KH = k.shape[2]
            G = QH // KH
            for b in range(B):
                for h in range(KH):
                    if empty[b, h]:
                        for g in range(G):
                            qh = O.q_head_of(g, h, KH, G, layout)
                            out[b, qh] = 0.0
                            lse[b, qh] = -float("inf")
        return out, lse

    @staticmethod
    def merge_lse(o_parts, lse_parts, dtype):
        m = lse_parts.max(0).values
        w = torch.exp(lse_parts - m[None])
        w = torch.where(torch.isfinite(lse_parts), w, torch.zeros_like(w))
        return ((o_parts * w[..., None]).sum(0) / w.sum(0)[..., None]).to(dtype)


class CpuExchange:
    """The surface of sharded.PeerExchange / PeerBuffer served by gloo, so that the driver's
    peer-memory branches (one-launch scan, one-launch partial merge) run on the CPU."""

    def all_gather(self, t):
        from spotlight_b200.sharded import _all_gather
        return _all_gather(t, None)

    def merge_lse(self, o, lse):
        parts = self.all_gather(torch.cat([o.float(), lse[..., None].float()], dim=-1))
        return CpuBackend.merge_lse(parts[..., :128].contiguous(), parts[..., 128].contiguous(), o.dtype)


def _scan_topk_sharded(q_codes, codes_local, peer, tok_offset, n_global, k, sink, recent, layout):
    scores, hist = CpuBackend.scan_hist(q_codes, codes_local, layout)
    hist_all = peer.all_gather(hist)
    return CpuBackend.select_emit(scores, hist_all, dist.get_rank(), tok_offset, n_global, q_codes.shape[1], k, sink, recent)


CpuBackend.scan_topk_sharded = staticmethod(_scan_topk_sharded)


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _make(n, B, KH, QH, seed, low_entropy):
    g = torch.Generator().manual_seed(seed)
    if low_entropy:                                          # few distinct codes: ties in the hundreds
        protos = torch.randint(0, 2 ** 31, (3, 4), generator=g)
        codes = protos[torch.randint(0, 3, (B, n, KH), generator=g)]
        codes = codes ^ ((torch.rand((B, n, KH, 4), generator=g) < 0.2).long() << torch.randint(0, 31, (B, n, KH, 4), generator=g))
    else:
        codes = torch.randint(0, 2 ** 31, (B, n, KH, 4), generator=g)
    q_codes = torch.randint(0, 2 ** 31, (B, QH, 4), generator=g)
    k = torch.randn((B, n, KH, 128), generator=g)
    v = torch.randn((B, n, KH, 128), generator=g)
    q = torch.randn((B, QH, 128), generator=g)
    return q, q_codes.to(torch.int32).view(torch.uint32), codes.to(torch.int32).view(torch.uint32), k, v


def _worker(rank, world, port, n, keep, low_entropy, ret, peer_branches=False):
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        from spotlight_b200.sharded import shard_bounds, sharded_decode_attention
        B, KH, QH = 2, 2, 6
        q, q_codes, codes, k, v = _make(n, B, KH, QH, 5, low_entropy)   # every rank builds the same global tensors
        lo, hi = shard_bounds(n, world, rank)
        out, idx, cnt = sharded_decode_attention(q, q_codes, codes[:, lo:hi], k[:, lo:hi], v[:, lo:hi], lo, n, keep,
                                                 4, 64, O.BLOCKED, backend=CpuBackend, return_selection=True,
                                                 exchange=(CpuExchange(), CpuExchange(), CpuExchange()) if peer_branches else None)
        ret[rank] = (out.numpy(), idx.numpy() + lo, cnt.numpy())
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,n,keep,low,peer_branches",
                         [(2, 700, 60, True, False), (2, 90, 20, False, False), (3, 1000, 100, True, False),
                          (2, 70, 5, True, False), (2, 700, 60, True, True), (3, 500, 40, False, True)])
def test_sequence_sharded_driver_equals_unsharded(world, n, keep, low, peer_branches):
    mgr = mp.Manager()
    ret = mgr.dict()
    mp.spawn(_worker, args=(world, _free_port(), n, keep, low, ret, peer_branches), nprocs=world, join=True)
    B, KH, QH = 2, 2, 6
    q, q_codes, codes, k, v = _make(n, B, KH, QH, 5, low)
    scores = O.match_count(q_codes.view(torch.int32).numpy().view(np.uint32)[:, None],
                           codes.view(torch.int32).numpy().view(np.uint32), O.BLOCKED)
    ref_idx, ref_cnt = O.select(scores, keep, 4, 64)
    ref_out = O.sparse_attention(q, k, v, ref_idx, ref_cnt, O.BLOCKED).numpy()
    for b in range(B):
        for h in range(KH):
            got = np.concatenate([ret[r][1][b, h, : ret[r][2][b, h]] for r in range(world)])
            np.testing.assert_array_equal(got, ref_idx[b, h, : ref_cnt[b, h]])
    for r in range(world):
        assert np.abs(ret[r][0] - ref_out).max() < 1e-5
        np.testing.assert_array_equal(ret[r][0], ret[0][0])          # every rank holds the same merged output


def test_shard_bounds_cover_the_sequence():
    from spotlight_b200.sharded import shard_bounds
    for n, w in ((1048576, 8), (1000, 3), (5, 8)):
        edges = [shard_bounds(n, w, r) for r in range(w)]
        assert edges[0][0] == 0 and edges[-1][1] == n
        assert all(edges[i][1] == edges[i + 1][0] for i in range(w - 1))


def test_block_seeded_generation_is_rank_independent():
    import dataclasses
    from spotlight_b200.workloads import CONFIGS, make_block
    cfg = dataclasses.replace(CONFIGS["cfg4"], batch=1)
    a0, _ = make_block(cfg, 0, tokens=64)
    a1, _ = make_block(cfg, 1, tokens=64)
    b1, _ = make_block(cfg, 1, tokens=64)
    assert torch.equal(a1, b1) and not torch.equal(a0[:, :64], a1[:, :64])
    assert a0.shape == (1, 64, 8, 128) and a0.dtype == torch.bfloat16
