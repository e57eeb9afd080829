"""Sequence-sharded decode attention on real devices over NCCL (needs >= 2 GPUs; skipped on a
single-GPU machine). Every rank builds the same seeded global tensors, keeps its shard, and the
merged output / the union of the index sets must equal the single-device kernels' and the CPU
checker's."""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from oracle import spotlight_oracle as O  # noqa: E402


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _inputs(n, B, KH, QH):
    g = torch.Generator().manual_seed(77)
    codes = torch.randint(0, 2 ** 31, (B, n, KH, 4), generator=g).to(torch.int32).view(torch.uint32)
    q_codes = torch.randint(0, 2 ** 31, (B, QH, 4), generator=g).to(torch.int32).view(torch.uint32)
    k = torch.randn((B, n, KH, 128), generator=g).to(torch.bfloat16)
    v = torch.randn((B, n, KH, 128), generator=g).to(torch.bfloat16)
    q = torch.randn((B, QH, 128), generator=g).to(torch.bfloat16)
    return q, q_codes, codes, k, v


def _worker(rank, world, port, n, keep, ret, peer=False):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from spotlight_b200 import ops
        from spotlight_b200.sharded import shard_bounds, sharded_decode_attention
        q, q_codes, codes, k, v = _inputs(n, 1, 8, 40)
        lo, hi = shard_bounds(n, world, rank)
        exchange = None
        if peer:            # the exchanges over peer memory instead of NCCL; "fused": scan + exchange + emit in one launch
            from spotlight_b200.sharded import make_peer_exchange
            exchange = make_peer_exchange(1, 8, 40, dev, fused_scan=(peer == "fused"))
        args = (q.to(dev), q_codes.to(dev), codes[:, lo:hi].contiguous().to(dev), k[:, lo:hi].contiguous().to(dev),
                v[:, lo:hi].contiguous().to(dev), lo, n, keep, 4, 64, O.BLOCKED)
        for _ in range(3 if peer else 1):            # several rounds: the exchange buffers are reused
            out, idx, cnt = sharded_decode_attention(*args, return_selection=True, exchange=exchange)
        torch.cuda.synchronize(dev)
        ops.check_status(dev)
        if exchange:
            for e in exchange:
                e.check_status()
            dist.barrier()
            for e in exchange:
                e.close()
        ret[rank] = (out.float().cpu().numpy(), idx.cpu().numpy() + lo, cnt.cpu().numpy())
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least two GPUs")
@pytest.mark.parametrize("peer", [False, True, "fused"], ids=["nccl", "peer-memory", "peer-memory-fused-scan"])
def test_sequence_sharded_attention_over_nccl(peer):
    import torch.multiprocessing as mp
    world = min(torch.cuda.device_count(), 4)
    n, keep = 200000, 4000
    ret = mp.Manager().dict()
    mp.spawn(_worker, args=(world, _free_port(), n, keep, ret, peer), nprocs=world, join=True)
    q, q_codes, codes, k, v = _inputs(n, 1, 8, 40)
    scores = O.match_count(q_codes.view(torch.int32).numpy().view(np.uint32)[:, None],
                           codes.view(torch.int32).numpy().view(np.uint32), O.BLOCKED)
    ref_idx, ref_cnt = O.select(scores, keep, 4, 64)
    for h in range(8):
        got = np.concatenate([ret[r][1][0, h, : ret[r][2][0, h]] for r in range(world)])
        np.testing.assert_array_equal(got, ref_idx[0, h, : ref_cnt[0, h]])
    ref_out = O.sparse_attention(q, k, v, ref_idx, ref_cnt, O.BLOCKED).numpy()
    for r in range(world):
        assert np.abs(ret[r][0] - ref_out).max() <= 2e-2           # bf16 tolerance
        np.testing.assert_array_equal(ret[r][0], ret[0][0])


def _cfg4_worker(rank, world, port, ret, peer):
    import torch.distributed as dist
    os.environ["MASTER_ADDR"] = "127.0.0.1"
    os.environ["MASTER_PORT"] = str(port)
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=dev)
    try:
        from spotlight_b200 import ops
        from spotlight_b200.sharded import shard_bounds, sharded_decode_attention
        from spotlight_b200.workloads import BLOCK_TOKENS, CONFIGS, budget, make_block, make_inputs
        cfg = CONFIGS["cfg4"]
        n = cfg.context
        lo, hi = shard_bounds(n, world, rank)
        assert lo % BLOCK_TOKENS == 0 and hi % BLOCK_TOKENS == 0
        blocks = [make_block(cfg, j) for j in range(lo // BLOCK_TOKENS, hi // BLOCK_TOKENS)]   # only the blocks this rank owns
        k = torch.cat([b[0] for b in blocks], 1).to(dev)
        v = torch.cat([b[1] for b in blocks], 1).to(dev)
        inp = make_inputs(cfg, context=64)                                                    # q and hash parameters of the config
        codes = ops.hash_encode(k, ops.HashParams.from_dict(inp.hash_k, dev))
        q_rot, q_codes = ops.decode_prepare(inp.q.to(dev), None, None, ops.HashParams.from_dict(inp.hash_q, dev), None, n - 1)
        exchange = None
        if peer:
            from spotlight_b200.sharded import make_peer_exchange
            exchange = make_peer_exchange(cfg.batch, cfg.kv_heads, cfg.q_heads, dev, fused_scan=True)
        keep = budget(n, cfg.mask_out, cfg.min_remain)
        for _ in range(2):
            out, idx, cnt = sharded_decode_attention(q_rot, q_codes, codes, k, v, lo, n, keep, cfg.sink, cfg.recent, O.BLOCKED,
                                                     return_selection=True, exchange=exchange)
        torch.cuda.synchronize(dev)
        ops.check_status(dev)
        if exchange:
            for e in exchange:
                e.check_status()
            dist.barrier()
            for e in exchange:
                e.close()
        ret[rank] = (out.float().cpu().numpy(), [idx[0, h, : int(cnt[0, h])].cpu().numpy() + lo for h in range(cfg.kv_heads)])
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs at least two GPUs")
@pytest.mark.parametrize("peer", [False, True], ids=["nccl", "peer-memory-fused-scan"])
def test_config4_full_size_sequence_shards(peer):
    """Config 4 at full size -- Qwen2.5-14B shape (40/8 heads), ONE MILLION keys, 98 % pruned -- over all
    the GPUs of the machine (2, 4 or 8): block-seeded inputs, every rank materialises only its own blocks.
    The union of the ranks' index sets and every rank's merged output must equal the single-device kernels'
    on the whole context (which other tests pin to the CPU checker at this size and smaller)."""
    import torch.multiprocessing as mp
    from spotlight_b200 import ops
    from spotlight_b200.workloads import BLOCK_TOKENS, CONFIGS, budget, make_block, make_inputs
    world = max(w for w in (2, 4, 8) if w <= torch.cuda.device_count())
    ret = mp.Manager().dict()
    mp.spawn(_cfg4_worker, args=(world, _free_port(), ret, peer), nprocs=world, join=True)
    cfg = CONFIGS["cfg4"]
    n = cfg.context
    dev = torch.device("cuda", 0)
    blocks = [make_block(cfg, j) for j in range(n // BLOCK_TOKENS)]
    k = torch.cat([b[0] for b in blocks], 1).to(dev)
    v = torch.cat([b[1] for b in blocks], 1).to(dev)
    del blocks
    inp = make_inputs(cfg, context=64)
    codes = ops.hash_encode(k, ops.HashParams.from_dict(inp.hash_k, dev))
    q_rot, q_codes = ops.decode_prepare(inp.q.to(dev), None, None, ops.HashParams.from_dict(inp.hash_q, dev), None, n - 1)
    keep = budget(n, cfg.mask_out, cfg.min_remain)
    idx, cnt = ops.scan_topk(q_codes, codes, keep, cfg.sink, cfg.recent, O.BLOCKED)
    whole = ops.sparse_attn_decode(q_rot, k, v, idx, cnt).float().cpu().numpy()
    for h in range(cfg.kv_heads):
        got = np.concatenate([ret[r][1][h] for r in range(world)])
        np.testing.assert_array_equal(got, idx[0, h, : int(cnt[0, h])].cpu().numpy())
    for r in range(world):
        assert np.abs(ret[r][0] - whole).max() <= 2e-2               # bf16 tolerance: partials merged in another order
        np.testing.assert_array_equal(ret[r][0], ret[0][0])          # every rank holds the same bits
    ops.check_status(dev)
