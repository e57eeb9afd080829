"""DecodeSession (the layer loop a caller owns) on the GPU: the Python loop, the native loop
(sl_decode_step) and a replayed CUDA graph must agree bit for bit over consecutive tokens, and a
layer-step must equal the single ops applied by hand."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = torch.device("cuda", 0) if torch.cuda.is_available() else None


def _session(seed=3, layers=3, B=2, QH=8, KH=4, n=2500, extra=8, mask_out=0.9):
    from spotlight_b200 import ops
    from spotlight_b200.session import DecodeSession, SessionConfig
    from spotlight_b200.workloads import make_hash_params
    g = torch.Generator().manual_seed(seed)
    dt = torch.bfloat16
    hq = [ops.HashParams.from_dict(make_hash_params("mlp", QH, (128, 256, 128), g, dt, mlp_scale=0.05), DEV) for _ in range(layers)]
    hk = [ops.HashParams.from_dict(make_hash_params("mlp", KH, (128, 256, 128), g, dt, mlp_scale=0.05), DEV) for _ in range(layers)]
    s = DecodeSession(SessionConfig(B, QH, KH, layers, n + extra, dt, mask_out), hq, hk, DEV)
    for layer in range(layers):
        k = torch.randn((B, n, KH, 128), generator=g).to(dt).to(DEV)
        v = torch.randn((B, n, KH, 128), generator=g).to(dt).to(DEV)
        s.load_context(layer, k, v)
    return s, g, n


def _token(s, g):
    for t in (s.q_in, s.k_in, s.v_in):
        t.copy_(torch.randn(t.shape, generator=g).to(t.dtype))


def test_native_loop_and_graph_equal_the_python_loop():
    from spotlight_b200 import ops
    a, ga, n = _session()
    b, gb, _ = _session()
    for step in range(4):                      # consecutive tokens: every one is appended, the scan grows
        pos = n + step
        _token(a, ga)
        _token(b, gb)
        a.set_position(pos, 500000.0)
        b.set_position(pos, 500000.0)
        a.step(pos)
        b.step_native(pos)
        torch.cuda.synchronize()
        assert torch.equal(a.out, b.out), f"token {step}: native loop differs from the Python loop"
        for layer in range(a.cfg.layers):
            assert torch.equal(a.codes[layer][:, : pos + 1], b.codes[layer][:, : pos + 1])
            assert torch.equal(a.k_cache[layer][:, pos], b.k_cache[layer][:, pos])
    ref = a.out.clone()
    graph = a.capture(n + 3)                   # same position again: appends rewrite the same row
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(a.out, ref)
    ops.check_status()


def test_layer_step_equals_the_single_ops():
    from spotlight_b200 import ops
    from spotlight_b200.workloads import budget
    s, g, n = _session(seed=5, layers=1)
    _token(s, g)
    s.set_position(n, 500000.0)
    q, k, v = s.q_in[0].clone(), s.k_in[0].clone(), s.v_in[0].clone()
    s.step(n)
    codes, kc, vc = s.codes[0].clone(), s.k_cache[0].clone(), s.v_cache[0].clone()   # token n already appended
    q_rot, q_codes = ops.decode_prepare(q, k, v, s.hash_q[0], s.hash_k[0], n, codes, kc, vc, s.cos, s.sin)
    idx, cnt = ops.scan_topk(q_codes, codes[:, : n + 1], budget(n + 1, s.cfg.mask_out), 4, 64)
    out = ops.sparse_attn_decode(q_rot, kc[:, : n + 1], vc[:, : n + 1], idx, cnt)
    torch.cuda.synchronize()
    assert torch.equal(out, s.out[0])
    assert np.array_equal(cnt.cpu().numpy(), s.cnt.cpu().numpy())
    ops.check_status()


def test_one_graph_serves_every_token():
    """The position lives in device memory: ONE captured step (sl_decode_step_dev) replayed for
    consecutive tokens must produce what the per-position launches produce -- outputs, appended codes
    and K/V rows, attended counts -- bit for bit."""
    from spotlight_b200 import ops
    a, ga, n = _session(seed=9, extra=12)
    b, gb, _ = _session(seed=9, extra=12)
    b.set_position_table(n, 12, 500000.0)
    b.pos_dev.fill_(n)
    graph = b.capture_dev()
    b.pos_dev.fill_(n)
    for step in range(6):
        pos = n + step
        _token(a, ga)
        _token(b, gb)
        a.set_position(pos, 500000.0)
        a.step(pos)
        graph.replay()
        torch.cuda.synchronize()
        assert int(b.pos_dev.item()) == pos + 1
        assert torch.equal(a.out, b.out), f"token {step}"
        assert torch.equal(a.cnt, b.cnt)
        for layer in range(a.cfg.layers):
            assert torch.equal(a.codes[layer][:, : pos + 1], b.codes[layer][:, : pos + 1])
            assert torch.equal(a.k_cache[layer][:, pos], b.k_cache[layer][:, pos])
            assert torch.equal(a.v_cache[layer][:, pos], b.v_cache[layer][:, pos])
    ops.check_status()


def test_fused_and_separate_caches_agree():
    from spotlight_b200 import ops
    import dataclasses
    a, ga, n = _session(seed=11)
    b, gb, _ = _session(seed=11)
    assert a.kv_cache is not None                       # the default: one fused cache per layer
    from spotlight_b200.session import DecodeSession
    c = DecodeSession(dataclasses.replace(b.cfg, fused_kv=False), b.hash_q, b.hash_k, DEV)
    for layer in range(b.cfg.layers):
        c.load_context(layer, b.k_cache[layer][:, :n].contiguous(), b.v_cache[layer][:, :n].contiguous())
    for step in range(2):
        pos = n + step
        _token(a, ga)
        c.q_in.copy_(a.q_in); c.k_in.copy_(a.k_in); c.v_in.copy_(a.v_in)
        a.set_position(pos, 500000.0)
        c.set_position(pos, 500000.0)
        a.step(pos)
        c.step_native(pos)
        torch.cuda.synchronize()
        assert torch.equal(a.out, c.out)
    ops.check_status()


def test_four_stage_step_with_a_device_side_clock():
    """hash -> scan + top-k -> LRU update -> attention over the resident buffers, as ONE replayed graph with
    the position (and with it the LRU clock) in device memory: outputs must equal the three-stage step's bit
    for bit (the stage is results-invisible), and the tables must register hits once the selections overlap."""
    import dataclasses
    from spotlight_b200 import ops
    from spotlight_b200.session import DecodeSession
    from spotlight_b200.workloads import budget
    a, ga, n = _session(seed=13, extra=12)
    b0, gb, _ = _session(seed=13, extra=12)
    slots = 2 * (budget(n + 12, a.cfg.mask_out, a.cfg.min_remain) + 68)
    b = DecodeSession(dataclasses.replace(b0.cfg, lru_slots=slots), b0.hash_q, b0.hash_k, DEV)
    for layer in range(b.cfg.layers):
        b.load_context(layer, b0.k_cache[layer][:, :n].contiguous(), b0.v_cache[layer][:, :n].contiguous())
    b.set_position_table(n, 12, 500000.0)
    b.pos_dev.fill_(n)
    graph = b.capture_dev()
    for t in b.lru:                                    # the warm-up token of the capture touched the tables: start clean
        t.tok2slot.fill_(-1); t.slot2tok.fill_(-1); t.last_used.fill_(-1)
    b.pos_dev.fill_(n)
    base_q = torch.randn(a.q_in.shape, generator=ga).to(a.q_in.dtype)
    hits = []
    for step in range(5):
        pos = n + step
        q = (base_q + 0.2 * torch.randn(a.q_in.shape, generator=ga).to(a.q_in.dtype))       # drifting query: overlapping selections
        kk = torch.randn(a.k_in.shape, generator=ga).to(a.k_in.dtype)
        vv = torch.randn(a.v_in.shape, generator=ga).to(a.v_in.dtype)
        for s_ in (a, b):
            s_.q_in.copy_(q); s_.k_in.copy_(kk); s_.v_in.copy_(vv)
        a.set_position(pos, 500000.0)
        a.step(pos)
        graph.replay()
        torch.cuda.synchronize()
        assert torch.equal(a.out, b.out), f"token {step}"
        st = b.lru[-1].stats.sum((0, 1)).cpu().numpy()
        assert st[0] + st[1] == int(b.cnt.sum())
        hits.append(int(st[0]))
        assert int(b.lru[-1].status.item()) == 0
    assert hits[0] == 0 and min(hits[1:]) > 0
    ops.check_status()
