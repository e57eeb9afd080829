"""Parity of every CUDA kernel against the CPU checker (oracle/), through the C ABI.
Integer work is bit-exact; attention is within the tolerance written at each assert."""
import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from oracle import spotlight_oracle as O  # noqa: E402


@pytest.fixture(scope="module")
def ops():
    from spotlight_b200 import ops as _ops
    return _ops


DEV = "cuda"


def rand_codes(gen, shape, low_entropy=False):
    """uint32 codes; low_entropy draws every code from 3 prototypes with a few flipped bits so
    that scores collide massively (threshold ties in the hundreds)."""
    if not low_entropy:
        return torch.randint(0, 2 ** 32, shape, generator=gen, dtype=torch.int64).to(torch.uint32)
    protos = torch.randint(0, 2 ** 32, (3, shape[-1]), generator=gen, dtype=torch.int64)
    pick = torch.randint(0, 3, shape[:-1], generator=gen)
    x = protos[pick]
    flip = (torch.rand(shape, generator=gen) < 0.3).to(torch.int64) << torch.randint(0, 32, shape, generator=gen)
    return (x ^ flip).to(torch.uint32)


def np_u32(t):
    return t.cpu().view(torch.int32).numpy().view(np.uint32)


def check_selection(idx, cnt, ref_idx, ref_cnt):
    idx, cnt = idx.cpu().numpy(), cnt.cpu().numpy()
    np.testing.assert_array_equal(cnt, ref_cnt)
    B, KH = cnt.shape
    for b in range(B):
        for h in range(KH):
            np.testing.assert_array_equal(idx[b, h, : cnt[b, h]], ref_idx[b, h, : ref_cnt[b, h]])


# ------------------------------------------------------------------------------------------ pack
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32, torch.float16, torch.bool])
def test_pack_signbits(ops, dtype):
    g = torch.Generator().manual_seed(1)
    x = torch.randn((3, 77, 128), generator=g)
    x[0, 0, :5] = 0.0                                   # exact zeros pack as 0 bits
    x = (x > 0.3) if dtype == torch.bool else x.to(dtype)
    got32 = ops.pack_signbits(x.to(DEV), 32)
    got8 = ops.pack_signbits(x.to(DEV), 8)
    assert got32.dtype == torch.uint32 and got32.shape == (3, 77, 4)
    np.testing.assert_array_equal(np_u32(got32), O.pack_signbits(x))
    np.testing.assert_array_equal(got8.cpu().numpy(), O.pack_signbits_u8(x))


# ------------------------------------------------------------------------------------------ scores
@pytest.mark.parametrize("B,N,KH,QH,W", [(1, 100, 4, 28, 4), (2, 1000, 8, 32, 4), (3, 65, 3, 6, 4),
                                         (1, 257, 2, 2, 2), (2, 129, 4, 8, 8), (1, 64, 1, 5, 1)])
@pytest.mark.parametrize("layout", [O.INTERLEAVED, O.BLOCKED])
def test_hamming_scores(ops, B, N, KH, QH, W, layout):
    g = torch.Generator().manual_seed(N)
    q = rand_codes(g, (B, 1, QH, W))
    cache = rand_codes(g, (B, N + 37, KH, W))             # scores over a view of a longer cache
    got = ops.hamming_scores(q.to(DEV), cache.to(DEV)[:, :N], layout)
    ref = O.match_count(np_u32(q), np_u32(cache)[:, :N], layout)
    np.testing.assert_array_equal(got.cpu().numpy(), ref)


def test_hamming_scores_u8(ops):
    g = torch.Generator().manual_seed(5)
    q = torch.randint(0, 256, (2, 5, 1, 16), generator=g, dtype=torch.int64).to(torch.uint8)
    k = torch.randint(0, 256, (2, 5, 333, 16), generator=g, dtype=torch.int64).to(torch.uint8)
    got = ops.hamming_scores_u8(q.to(DEV), k.to(DEV))
    np.testing.assert_array_equal(got.cpu().numpy(), O.match_count_u8(q.numpy(), k.numpy()))


# ------------------------------------------------------------------------------------------ scan + top-k
SCAN_CASES = [
    # B, N, KH, QH, k, sink, recent, low_entropy
    (1, 1, 8, 8, 1, 4, 64, False),
    (1, 3, 4, 28, 2, 4, 64, False),
    (2, 63, 8, 32, 20, 4, 64, False),
    (1, 64, 8, 8, 20, 4, 64, True),
    (1, 65, 8, 8, 20, 4, 64, True),
    (1, 68, 2, 2, 20, 4, 64, False),
    (1, 69, 2, 4, 20, 4, 64, True),
    (1, 100, 4, 28, 20, 4, 64, True),
    (1, 4096, 8, 8, 410, 4, 64, False),
    (1, 4096, 8, 8, 410, 4, 64, True),
    (3, 5000, 3, 6, 77, 4, 64, True),          # kv heads not a power of two
    (2, 3000, 32, 32, 60, 4, 64, True),
    (1, 2000, 64, 64, 40, 4, 64, False),       # more heads than warps
    (8, 16384, 32, 32, 328, 4, 64, False),     # config 2 shape
    (1, 131072, 8, 32, 2622, 4, 64, False),    # headline shape
    (1, 131072, 8, 32, 13108, 4, 64, True),
    (2, 40000, 4, 28, 800, 0, 0, True),        # pure top-k
    (2, 40000, 4, 28, 0, 4, 64, False),        # window only
    (1, 300, 4, 4, 1000, 4, 64, False),        # k >= N
    (1, 9000, 8, 40, 180, 100, 300, True),     # wide windows, G = 5
    (1, 2048, 2, 24, 64, 4, 64, False),        # G = 12: three bit planes (even group: halved)
    (1, 1500, 2, 40, 64, 4, 64, True),         # G = 20: four bit planes
    (1, 1500, 2, 18, 64, 4, 64, True),         # G = 9: four bit planes (odd group)
    (1, 1500, 2, 34, 64, 4, 64, True),         # G = 17: direct popcount path
    (2, 2500, 4, 64, 64, 4, 64, False),        # G = 16
    (160, 700, 4, 8, 30, 4, 64, True),         # more batch rows than SMs: one CTA per row, no grid barrier
    (150, 20000, 8, 8, 100, 4, 64, False),     # the same with scores spilled to global memory
]


@pytest.mark.parametrize("B,N,KH,QH,k,sink,recent,low", SCAN_CASES)
@pytest.mark.parametrize("layout", [O.BLOCKED, O.INTERLEAVED])
def test_scan_topk_bit_exact(ops, B, N, KH, QH, k, sink, recent, low, layout):
    if layout == O.INTERLEAVED and B * N * KH > 600000:
        pytest.skip("large shapes run once")
    g = torch.Generator().manual_seed(B * 131 + N)
    q = rand_codes(g, (B, QH, 4), low)
    cache = rand_codes(g, (B, N + 5, KH, 4), low)
    qd, cd = q.to(DEV), cache.to(DEV)
    scores_ref = O.match_count(np_u32(q)[:, None], np_u32(cache)[:, :N], layout)
    ref_idx, ref_cnt = O.select(scores_ref, k, sink, recent)
    for _ in range(3):                                   # later calls reuse the workspace the kernel left behind
        idx, cnt, scores = ops.scan_topk(qd, cd[:, :N], k, sink, recent, layout, return_scores=True)
        np.testing.assert_array_equal(scores.cpu().numpy(), scores_ref)
        check_selection(idx, cnt, ref_idx, ref_cnt)
    ops.check_status()


GENERAL_CASES = [c for c in SCAN_CASES if c[0] < 100 and c[0] * c[1] * c[2] <= 1100000][::2]


@pytest.mark.parametrize("B,N,KH,QH,k,sink,recent,low", GENERAL_CASES)
def test_scan_topk_general_kernel(ops, B, N, KH, QH, k, sink, recent, low):
    """sl_scan_topk sends the common decode shapes to its one-barrier kernel; the general kernel (other
    shapes, the spill path, the sharded halves) and the flagged-word kernel (the sequence shards' fused
    form) must give the same answer on them, also when they take turns on one workspace."""
    from spotlight_b200 import _lib

    def setter(mode):
        _lib.check(_lib.lib.sl_configure(_lib.SL_OPT_SCAN_KERNEL, mode))
    g = torch.Generator().manual_seed(B * 977 + N)
    q = rand_codes(g, (B, QH, 4), low)
    cache = rand_codes(g, (B, N, KH, 4), low)
    scores_ref = O.match_count(np_u32(q)[:, None], np_u32(cache), O.BLOCKED)
    ref_idx, ref_cnt = O.select(scores_ref, k, sink, recent)
    try:
        for mode in (0, 2, 1, 0, 1, 2, 1):               # 0 general, 2 flagged words, 1 one barrier (default)
            setter(mode)
            for _ in range(2):
                idx, cnt, scores = ops.scan_topk(q.to(DEV), cache.to(DEV), k, sink, recent, O.BLOCKED, return_scores=True)
                np.testing.assert_array_equal(scores.cpu().numpy(), scores_ref)
                check_selection(idx, cnt, ref_idx, ref_cnt)
    finally:
        setter(1)
    ops.check_status()


@pytest.mark.parametrize("B,KH,QH,N0,sink,recent", [(1, 8, 32, 40000, 4, 64), (2, 4, 28, 9000, 4, 64), (1, 8, 8, 520, 4, 64),
                                                   (1, 2, 2, 3000, 1, 95), (4, 1, 4, 20000, 7, 30), (1, 16, 32, 30000, 0, 5),
                                                   (1, 8, 64, 12000, 4, 64), (3, 32, 32, 5000, 4, 64)])
def test_scan_topk_growing_context(ops, B, KH, QH, N0, sink, recent):
    """A decode loop: the context grows by one key per call on ONE workspace (the chunking, and with it
    the kernel that serves the call, changes along the way), low-entropy codes so that the threshold
    bin is crowded with ties, some of them inside the sink and the recent window."""
    g = torch.Generator().manual_seed(N0 + KH)
    q = rand_codes(g, (B, QH, 4), True)
    cache = rand_codes(g, (B, N0 + 40, KH, 4), True)
    qd, cd = q.to(DEV), cache.to(DEV)
    for step, N in enumerate(list(range(N0, N0 + 6)) + [N0 // 2, N0 + 33, 300, N0 + 40]):
        k = max(min(N, 20), N - int(N * 0.9))
        scores_ref = O.match_count(np_u32(q)[:, None], np_u32(cache)[:, :N], O.BLOCKED)
        ref_idx, ref_cnt = O.select(scores_ref, k, sink, recent)
        idx, cnt = ops.scan_topk(qd, cd[:, :N], k, sink, recent, O.BLOCKED)
        check_selection(idx, cnt, ref_idx, ref_cnt)
    ops.check_status()


def test_scan_topk_full_size_config3(ops):
    """Qwen2.5-7B shape of the reference CUDA kernel at full size (B 8, 28/4 heads, 128K keys)."""
    B, N, KH, QH, k = 8, 131072, 4, 28, 2622
    g = torch.Generator().manual_seed(1003)
    q = rand_codes(g, (B, QH, 4))
    cache = rand_codes(g, (B, N, KH, 4))
    idx, cnt = ops.scan_topk(q.to(DEV), cache.to(DEV), k, 4, 64, O.INTERLEAVED)
    scores_ref = O.match_count(np_u32(q)[:, None], np_u32(cache), O.INTERLEAVED)
    ref_idx, ref_cnt = O.select(scores_ref, k, 4, 64)
    check_selection(idx, cnt, ref_idx, ref_cnt)
    ops.check_status()


def test_scan_topk_million_keys(ops):
    """Config 4 size on one device (1M keys, 40/8 heads): scores spill past shared memory; checked
    through properties that hold at any size plus a full comparison of two heads."""
    B, N, KH, QH, k = 1, 1048576, 8, 40, 20972
    g = torch.Generator().manual_seed(1004)
    q = rand_codes(g, (B, QH, 4))
    cache = rand_codes(g, (B, N, KH, 4))
    idx, cnt, scores = ops.scan_topk(q.to(DEV), cache.to(DEV), k, 4, 64, O.BLOCKED, return_scores=True)
    idx, cnt, scores = idx.cpu().numpy(), cnt.cpu().numpy(), scores.cpu().numpy()
    for h in range(KH):
        sel = idx[0, h, : cnt[0, h]]
        assert np.all(np.diff(sel) > 0)                                     # ascending, unique
        assert set(range(4)) <= set(sel[:4].tolist()) and sel[-1] == N - 1   # sink + newest key
        s = scores[0, :, h]
        top = np.setdiff1d(sel, np.concatenate([np.arange(4), np.arange(N - 64, N)]))
        tau = np.sort(s)[::-1][k - 1]
        assert s[top].min() >= tau                                          # nothing below threshold
    sub = O.match_count(np_u32(q)[:, None], np_u32(cache), O.BLOCKED)
    np.testing.assert_array_equal(scores, sub)
    for h in (0, 5):
        np.testing.assert_array_equal(idx[0, h, : cnt[0, h]], O.attended_set(sub[0, :, h], k, 4, 64))
    ops.check_status()


def test_topk_from_scores(ops):
    g = torch.Generator().manual_seed(9)
    s = torch.randint(0, 897, (2, 7000, 4), generator=g, dtype=torch.int64).to(torch.int16)
    s[:, 100:4000] = 500                                                    # a plateau of ties
    idx, cnt = ops.topk_from_scores(s.to(DEV), 1234, 896, sink=0, recent=0)
    ref_idx, ref_cnt = O.select(s.numpy(), 1234, 0, 0)
    check_selection(idx, cnt, ref_idx, ref_cnt)


@pytest.mark.parametrize("R", [2, 4, 8])
@pytest.mark.parametrize("N,k,low", [(9000, 333, True), (70, 20, False), (4096, 410, True), (40, 5, True)])
def test_sharded_selection_equals_single_device(ops, R, N, k, low):
    """Sequence shards emulated on one device: per-shard scan+histogram, stacked histograms,
    per-shard emission; the union must be the single-device selection, bit for bit."""
    B, KH, QH = 2, 4, 20
    g = torch.Generator().manual_seed(N + R)
    q = rand_codes(g, (B, QH, 4), low)
    cache = rand_codes(g, (B, N, KH, 4), low)
    qd, cd = q.to(DEV), cache.to(DEV)
    bounds = [N * r // R for r in range(R + 1)]
    parts = [ops.scan_hist(qd, cd[:, bounds[r]:bounds[r + 1]].contiguous(), O.BLOCKED) for r in range(R)]
    hist_all = torch.stack([p[1] for p in parts])
    got = [[[] for _ in range(KH)] for _ in range(B)]
    for r in range(R):
        idx, cnt = ops.select_emit(parts[r][0], hist_all, r, bounds[r], N, QH, k, 4, 64)
        idx, cnt = idx.cpu().numpy(), cnt.cpu().numpy()
        for b in range(B):
            for h in range(KH):
                got[b][h].append(idx[b, h, : cnt[b, h]] + bounds[r])
    scores_ref = O.match_count(np_u32(q)[:, None], np_u32(cache), O.BLOCKED)
    for b in range(B):
        for h in range(KH):
            np.testing.assert_array_equal(np.concatenate(got[b][h]), O.attended_set(scores_ref[b, :, h], k, 4, 64))
    ops.check_status()


# ------------------------------------------------------------------------------------------ hash
def _hash_case(kind, dtype, heads, dims, residue, seed, scale):
    from spotlight_b200.workloads import make_hash_params
    g = torch.Generator().manual_seed(seed)
    p = make_hash_params(kind, heads, dims, g, dtype, mlp_scale=scale)
    if kind == "mlp":
        p["b"] = [(torch.randn(b.shape, generator=g) * scale).to(dtype) for b in p["b"]]
    return p


def _assert_codes_match(got_u32, ref_pre, tol_rel=2e-2):
    """Bit-exact except where the pre-sign value is within rounding noise of zero."""
    ref_bits = (ref_pre > 0).numpy()
    got_bits = np.unpackbits(got_u32.view(np.uint8), axis=-1, bitorder="little").astype(bool)
    got_bits = got_bits.reshape(ref_bits.shape)
    bad = got_bits != ref_bits
    if bad.any():
        mag = ref_pre.float().abs().numpy()
        scale = np.median(mag)
        assert (mag[bad] <= tol_rel * scale).all(), f"{bad.sum()} sign mismatches away from zero"
        assert bad.mean() < 5e-3


@pytest.mark.parametrize("kind,dtype,dims,residue,scale", [
    ("linear", torch.float32, (128, 128), False, None),
    ("linear", torch.bfloat16, (128, 128), False, None),
    ("mlp", torch.bfloat16, (128, 256, 128), False, 0.05),
    ("mlp", torch.bfloat16, (128, 128, 128), True, 0.05),
    ("mlp", torch.float32, (128, 256, 128), False, 0.05),
    ("mlp", torch.float16, (128, 64, 128), False, 0.05),
])
@pytest.mark.parametrize("B", [1, 8])
def test_decode_prepare(ops, kind, dtype, dims, residue, scale, B):
    QH, KH, NMAX, pos, theta = 8, 2, 50, 17, 500000.0
    hq = _hash_case(kind, dtype, QH, dims, residue, 21, scale)
    hk = _hash_case(kind, dtype, KH, dims, residue, 22, scale)
    g = torch.Generator().manual_seed(B)
    q = torch.randn((B, QH, 128), generator=g).to(dtype)
    k = torch.randn((B, KH, 128), generator=g).to(dtype)
    v = torch.randn((B, KH, 128), generator=g).to(dtype)
    cos, sin = O.rope_tables(NMAX, theta)
    cos, sin = cos.to(dtype), sin.to(dtype)
    code_cache = torch.zeros((B, NMAX, KH, 4), dtype=torch.uint32, device=DEV)
    k_cache = torch.zeros((B, NMAX, KH, 128), dtype=dtype, device=DEV)
    v_cache = torch.zeros_like(k_cache)
    q_rot, q_codes = ops.decode_prepare(
        q.to(DEV), k.to(DEV), v.to(DEV), ops.HashParams.from_dict(hq, DEV, residue),
        ops.HashParams.from_dict(hk, DEV, residue), pos, code_cache, k_cache, v_cache,
        cos[pos].contiguous().to(DEV), sin[pos].contiguous().to(DEV))
    # rotation follows the reference's operator order and rounding exactly
    q_ref = O.apply_rope(q[:, :, None], cos, sin, torch.tensor([pos]))[:, :, 0]
    k_ref = O.apply_rope(k[:, :, None], cos, sin, torch.tensor([pos]))[:, :, 0]
    assert torch.equal(q_rot.cpu(), q_ref)
    assert torch.equal(k_cache[:, pos].cpu(), k_ref)
    assert torch.equal(v_cache[:, pos].cpu(), v)
    assert int(k_cache[:, :pos].abs().sum()) == 0 and int(k_cache[:, pos + 1:].abs().sum()) == 0
    _, q_pre = O.hash_codes(q_ref[:, :, None], hq, residue)
    _, k_pre = O.hash_codes(k_ref[:, :, None], hk, residue)
    _assert_codes_match(np_u32(q_codes), q_pre[:, :, 0])
    _assert_codes_match(np_u32(code_cache[:, pos]), k_pre[:, :, 0])
    assert int(code_cache[:, :pos].view(torch.int32).abs().sum()) == 0


@pytest.mark.parametrize("kind,dtype,dims,residue", [("linear", torch.bfloat16, (128, 128), False),
                                                     ("mlp", torch.bfloat16, (128, 256, 128), False),
                                                     ("mlp", torch.float32, (128, 128, 128), True)])
def test_hash_encode_rows(ops, kind, dtype, dims, residue):
    B, T, H = 2, 203, 4
    hp = _hash_case(kind, dtype, H, dims, residue, 31, 0.05)
    g = torch.Generator().manual_seed(3)
    x = torch.randn((B, T + 9, H, 128), generator=g).to(dtype)
    codes = ops.hash_encode(x.to(DEV)[:, :T], ops.HashParams.from_dict(hp, DEV, residue))
    _, pre = O.hash_codes(x[:, :T].permute(0, 2, 1, 3), hp, residue)          # [B,H,T,128]
    _assert_codes_match(np_u32(codes), pre.permute(0, 2, 1, 3))


@pytest.mark.parametrize("kind,dims,residue", [("mlp", (128, 256, 128), False), ("mlp", (128, 128, 128), False),
                                               ("mlp", (128, 128, 128), True), ("linear", (128, 128), False)])
@pytest.mark.parametrize("B,T,H,fused", [(2, 203, 4, False), (1, 1000, 3, True), (3, 128, 2, False), (1, 5, 1, False), (1, 1500, 2, False)])
def test_hash_encode_tcgen05_kernel(ops, B, T, H, fused, kind, dims, residue):
    """The tcgen05 / TMEM kernels (forced for every size) against the checker: ragged tiles, several batch rows,
    rows taken from the K half of a fused K|V cache; the MLP hash and the linear hash."""
    from spotlight_b200 import _lib
    hp = _hash_case(kind, torch.bfloat16, H, dims, residue, 41, 0.05)
    g = torch.Generator().manual_seed(5)
    x = torch.randn((B, T + 9, H, 128), generator=g).to(torch.bfloat16)
    if fused:
        cache = torch.zeros((B, T + 9, H, 2, 128), dtype=torch.bfloat16, device=DEV)
        cache[:, :, :, 0] = x.to(DEV)
        xd = cache[:, :T, :, 0]
    else:
        xd = x.to(DEV)[:, :T]
    params = ops.HashParams.from_dict(hp, DEV, residue)
    try:
        ops.configure(_lib.SL_OPT_HASH_KERNEL, 2)
        codes = ops.hash_encode(xd, params)
        torch.cuda.synchronize()
        ops.check_status(DEV)
        ops.configure(_lib.SL_OPT_HASH_KERNEL, 1)
        codes_warp = ops.hash_encode(xd, params)
    finally:
        ops.configure(_lib.SL_OPT_HASH_KERNEL, 0)
    _, pre = O.hash_codes(x[:, :T].permute(0, 2, 1, 3), hp, residue)            # [B,H,T,128]
    _assert_codes_match(np_u32(codes), pre.permute(0, 2, 1, 3))
    flips = np.bitwise_count(np_u32(codes) ^ np_u32(codes_warp)).sum() / (codes.numel() * 32.0)
    assert flips <= 1e-4, f"{flips:.2e} of the bits differ between the two tensor-core kernels"


@pytest.mark.parametrize("kind,dims,residue", [("mlp", (128, 256, 128), False), ("mlp", (128, 128, 128), True), ("linear", (128, 128), False)])
def test_hash_encode_tcgen05_many_tiles(ops, parity_report, kind, dims, residue):
    """Many tiles per CTA (barrier phases wrapping many times): the two tensor-core kernels agree except where
    a pre-sign value is within rounding of zero, and the kernel is deterministic."""
    from spotlight_b200 import _lib
    B, T, H = 1, 70001, 8
    hp = _hash_case(kind, torch.bfloat16, H, dims, residue, 43, 0.05)
    g = torch.Generator(device=DEV).manual_seed(7)
    x = torch.randn((B, T, H, 128), generator=g, device=DEV).to(torch.bfloat16)
    params = ops.HashParams.from_dict(hp, DEV, residue)
    try:
        ops.configure(_lib.SL_OPT_HASH_KERNEL, 2)
        a = ops.hash_encode(x, params)
        b = ops.hash_encode(x, params)
        torch.cuda.synchronize()
        ops.check_status(DEV)
        ops.configure(_lib.SL_OPT_HASH_KERNEL, 1)
        c = ops.hash_encode(x, params)
    finally:
        ops.configure(_lib.SL_OPT_HASH_KERNEL, 0)
    assert torch.equal(a.view(torch.int32), b.view(torch.int32))
    flips = np.bitwise_count(np_u32(a) ^ np_u32(c)).sum() / (a.numel() * 32.0)
    parity_report(f"tcgen05 hash kernel vs warp-level kernel (70 001 x 8 rows, bf16, {kind} {dims}{' residual' if residue else ''})", bit_flip_rate=f"{flips:.2e}")
    assert flips <= 1e-4


# ------------------------------------------------------------------------------------------ attention
def _attn_inputs(B, N, KH, QH, dtype, seed):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn((B, QH, 128), generator=g).to(dtype)
    k = torch.randn((B, N, KH, 128), generator=g)
    k[:, 0] *= 4.0
    v = torch.randn((B, N, KH, 128), generator=g)
    return q, k.to(dtype), v.to(dtype), g


@pytest.mark.parametrize("B,N,KH,QH,keep", [(1, 4096, 8, 8, 478), (2, 3000, 8, 32, 300), (1, 9000, 4, 28, 2000),
                                            (3, 500, 2, 10, 1), (1, 70, 1, 1, 70), (2, 20000, 8, 40, 5000)])
@pytest.mark.parametrize("dtype,tol", [(torch.bfloat16, 2e-2), (torch.float32, 2e-5)])
@pytest.mark.parametrize("layout", [O.BLOCKED, O.INTERLEAVED])
def test_sparse_attention(ops, B, N, KH, QH, keep, dtype, tol, layout):
    q, k, v, g = _attn_inputs(B, N, KH, QH, dtype, N + QH)
    cap = keep + 3
    idx = np.full((B, KH, cap), -1, np.int32)
    cnt = np.zeros((B, KH), np.int32)
    for b in range(B):
        for h in range(KH):
            n = max(1, keep - (b + h) % 3)                                    # ragged list lengths
            idx[b, h, :n] = np.sort(torch.randperm(N, generator=g)[:n].numpy())
            cnt[b, h] = n
    kc = torch.zeros((B, N + 11, KH, 128), dtype=dtype, device=DEV)           # rows of a longer cache
    vc = torch.zeros_like(kc)
    kc[:, :N], vc[:, :N] = k.to(DEV), v.to(DEV)
    out, lse = ops.sparse_attn_decode(q.to(DEV), kc[:, :N], vc[:, :N], torch.from_numpy(idx).to(DEV),
                                      torch.from_numpy(cnt).to(DEV), layout, return_lse=True)
    ref, ref_lse = O.sparse_attention(q, k, v, idx, cnt, layout, return_lse=True)
    assert (out.float().cpu() - ref).abs().max().item() <= tol               # bf16 tolerance 2e-2
    assert (lse.cpu() - ref_lse).abs().max().item() <= (2e-2 if dtype == torch.bfloat16 else 1e-4)
    out2 = ops.sparse_attn_decode(q.to(DEV), kc[:, :N], vc[:, :N], torch.from_numpy(idx).to(DEV),
                                  torch.from_numpy(cnt).to(DEV), layout)
    assert torch.equal(out, out2)                                             # deterministic, workspace self-cleans


@pytest.mark.parametrize("B,N,KH,QH,keep", [(1, 131072, 8, 32, 13176), (1, 131072, 8, 32, 2690), (1, 40000, 8, 32, 900), (8, 20000, 4, 28, 470),
                                            (2, 9000, 2, 24, 3000)])
def test_sparse_attention_cluster_merge(ops, B, N, KH, QH, keep):
    """The splits of a (row, head) pair combined inside a thread-block cluster (distributed shared memory) against
    the same launch with partials in the workspace and the merge kernel, and both against the checker."""
    from spotlight_b200 import _lib
    q, k, v, g = _attn_inputs(B, N, KH, QH, torch.bfloat16, 5)
    idx = torch.stack([torch.stack([torch.sort(torch.randperm(N, generator=g)[:keep]).values for _ in range(KH)])
                       for _ in range(B)]).to(torch.int32)
    cnt = torch.full((B, KH), keep, dtype=torch.int32)
    qd, kd, vd, idd, cd = q.to(DEV), k.to(DEV), v.to(DEV), idx.to(DEV), cnt.to(DEV)
    try:
        ops.configure(_lib.SL_OPT_ATTN_CLUSTER, 1)
        out_c, lse_c = ops.sparse_attn_decode(qd, kd, vd, idd, cd, return_lse=True)
        ops.configure(_lib.SL_OPT_ATTN_CLUSTER, 0)
        out_m, lse_m = ops.sparse_attn_decode(qd, kd, vd, idd, cd, return_lse=True)
    finally:
        ops.configure(_lib.SL_OPT_ATTN_CLUSTER, 1)
    assert (out_c.float() - out_m.float()).abs().max().item() <= 2e-3
    assert (lse_c - lse_m).abs().max().item() <= 1e-4
    if N <= 40000:
        ref, ref_lse = O.sparse_attention(q, k, v, idx.numpy(), cnt.numpy(), O.BLOCKED, return_lse=True)
        assert (out_c.float().cpu() - ref).abs().max().item() <= 2e-2
        assert (lse_c.cpu() - torch.as_tensor(ref_lse)).abs().max().item() <= 2e-2



@pytest.mark.parametrize("B,N,KH,QH,keep", [(1, 30000, 8, 32, 3000), (2, 5000, 4, 28, 600), (9, 3000, 32, 32, 200)])
def test_sparse_attention_cache_geometries(ops, B, N, KH, QH, keep):
    """The same attention over two caches [B,N,KH,128], over the halves of one fused cache
    [B,N,KH,2,128] (a key's K and V rows adjacent) and over a batch aliased with expand (every row reads
    batch row 0, spotlight/modifiers/fake_cache.py:42-49,96-106): identical bits, and the checker's values."""
    q, k, v, g = _attn_inputs(B, N, KH, QH, torch.bfloat16, N + B)
    idx = np.zeros((B, KH, keep), np.int32)
    for b in range(B):
        for h in range(KH):
            idx[b, h] = np.sort(torch.randperm(N, generator=g)[:keep].numpy())
    cnt = np.full((B, KH), keep, np.int32)
    qd, idx_d, cnt_d = q.to(DEV), torch.from_numpy(idx).to(DEV), torch.from_numpy(cnt).to(DEV)
    kd, vd = k.to(DEV), v.to(DEV)
    two = ops.sparse_attn_decode(qd, kd, vd, idx_d, cnt_d)
    fused = torch.empty((B, N + 3, KH, 2, 128), dtype=torch.bfloat16, device=DEV)
    fused[:, :N, :, 0], fused[:, :N, :, 1] = kd, vd
    one = ops.sparse_attn_decode(qd, fused[:, :N, :, 0], fused[:, :N, :, 1], idx_d, cnt_d)
    assert torch.equal(one, two)
    ref = O.sparse_attention(q, k, v, idx, cnt, O.BLOCKED)
    assert (one.float().cpu() - ref).abs().max().item() <= 2e-2
    # aliased batch: all rows read row 0's cache
    alias = ops.sparse_attn_decode(qd, kd[:1].expand(B, -1, -1, -1), vd[:1].expand(B, -1, -1, -1), idx_d, cnt_d)
    ref_alias = O.sparse_attention(q, k[:1].expand(B, -1, -1, -1), v[:1].expand(B, -1, -1, -1), idx, cnt, O.BLOCKED)
    assert (alias.float().cpu() - ref_alias).abs().max().item() <= 2e-2


@pytest.mark.parametrize("B,N,KH,QH,keep", [(1, 6000, 2, 8, 500), (2, 3000, 4, 28, 100)])
def test_sparse_attention_per_query_head_lists(ops, B, N, KH, QH, keep):
    """Every query head with its own index list over the shared K/V caches (the per-query-head
    selection of the reference's modifier, spotlight_generation.py:128-165): equals attention with
    the caches repeated per query head as repeat_kv does."""
    q, k, v, g = _attn_inputs(B, N, KH, QH, torch.bfloat16, N + QH)
    G = QH // KH
    idx = np.zeros((B, QH, keep), np.int32)
    for b in range(B):
        for h in range(QH):
            idx[b, h] = np.sort(torch.randperm(N, generator=g)[:keep].numpy())
    cnt = np.full((B, QH), keep, np.int32)
    out = ops.sparse_attn_decode(q.to(DEV), k.to(DEV), v.to(DEV), torch.from_numpy(idx).to(DEV), torch.from_numpy(cnt).to(DEV))
    k_rep, v_rep = k.repeat_interleave(G, dim=2), v.repeat_interleave(G, dim=2)      # [B,N,QH,128], head j <- kv head j // G
    ref = O.sparse_attention(q, k_rep, v_rep, idx, cnt, O.BLOCKED)
    assert (out.float().cpu() - ref).abs().max().item() <= 2e-2


def test_merge_lse_equals_unsplit(ops):
    """Attention over 4 sequence shards merged by log-sum-exp equals attention over the whole list."""
    B, N, KH, QH, R = 2, 8000, 4, 20, 4
    q, k, v, g = _attn_inputs(B, N, KH, QH, torch.bfloat16, 77)
    sel = np.sort(torch.randperm(N, generator=g)[:1500].numpy()).astype(np.int32)
    idx = np.broadcast_to(sel, (B, KH, len(sel))).copy()
    cnt = np.full((B, KH), len(sel), np.int32)
    qd, kd, vd = q.to(DEV), k.to(DEV), v.to(DEV)
    whole = ops.sparse_attn_decode(qd, kd, vd, torch.from_numpy(idx).to(DEV), torch.from_numpy(cnt).to(DEV))
    os_, ls_ = [], []
    for r in range(R):
        lo, hi = N * r // R, N * (r + 1) // R
        loc = sel[(sel >= lo) & (sel < hi)] - lo
        if r == 2:
            loc = loc[:0]                                                     # an empty shard must not poison the merge
        li = np.broadcast_to(loc, (B, KH, len(loc))).copy() if len(loc) else np.zeros((B, KH, 1), np.int32)
        lc = np.full((B, KH), len(loc), np.int32)
        o, l = ops.sparse_attn_decode(qd, kd[:, lo:hi].contiguous(), vd[:, lo:hi].contiguous(),
                                      torch.from_numpy(li).to(DEV), torch.from_numpy(lc).to(DEV), return_lse=True)
        os_.append(o.float())
        ls_.append(l)
    merged = ops.merge_lse(torch.stack(os_), torch.stack(ls_), torch.bfloat16)
    keep = sel[~((sel >= N * 2 // R) & (sel < N * 3 // R))]
    idx2 = np.broadcast_to(keep, (B, KH, len(keep))).copy()
    ref = O.sparse_attention(q, k, v, idx2, np.full((B, KH), len(keep), np.int32))
    assert (merged.float().cpu() - ref).abs().max().item() <= 2e-2
    assert (whole.float().cpu() - O.sparse_attention(q, k, v, idx, cnt)).abs().max().item() <= 2e-2


def test_gather_rows(ops):
    g = torch.Generator().manual_seed(2)
    cache = torch.randn((2, 500, 4, 128), generator=g).to(torch.bfloat16)
    idx = torch.stack([torch.stack([torch.randperm(500, generator=g)[:60] for _ in range(4)]) for _ in range(2)])
    out = ops.gather_rows(cache.to(DEV), idx.to(torch.int32).to(DEV), 50)
    ref = torch.gather(cache, 1, idx[:, :, :50].permute(0, 2, 1)[..., None].expand(-1, -1, -1, 128))
    assert torch.equal(out.cpu(), ref)


# ------------------------------------------------------------------------------------------ errors
def test_errors_are_exceptions_not_crashes(ops):
    q = torch.zeros((1, 8, 4), dtype=torch.uint32, device=DEV)
    k = torch.zeros((1, 100, 8, 4), dtype=torch.uint32, device=DEV)
    with pytest.raises(RuntimeError):
        ops.scan_topk(q.cpu(), k.cpu(), 10)                                   # no CPU path
    with pytest.raises(ValueError):
        ops.scan_topk(q, k, 50, idx=torch.empty((1, 8, 10), dtype=torch.int32, device=DEV))  # idx too small
    with pytest.raises(ValueError):
        ops.hamming_scores(q[:, None], k.transpose(1, 2).contiguous().transpose(1, 2))  # not token-major
    with pytest.raises(AssertionError):
        ops.pack_signbits(torch.zeros((4, 100), device=DEV))                  # last dim % 32


# ------------------------------------------------------------------------------------------ LRU
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
@pytest.mark.parametrize("B,KH,N,C,keep", [(2, 4, 3000, 400, 300), (1, 8, 5000, 1500, 1400), (3, 2, 200, 64, 64),
                                           (1, 4, 60000, 9000, 4200), (2, 2, 40000, 14000, 6500)])
@pytest.mark.parametrize("multi", [1, 0])
def test_lru_resident_buffer_is_results_invisible(ops, dtype, B, KH, N, C, keep, multi):
    """A dozen decode steps with drifting attended sets: slot tables bit-exact against the CPU
    model of the policy, resident rows equal to the backing rows, and attention over the resident
    buffer bit-identical to attention over the full cache. The long lists are probed by several CTAs
    per (row, kv head): all of them work through the whole update (multi = 1, four barriers of the pair), or the
    last of them handles the misses alone (multi = 0). Fused K|V buffers on both sides in the bf16 runs of the long lists."""
    from spotlight_b200 import _lib
    ops.configure(_lib.SL_OPT_LRU_MULTI_CTA, multi)
    try:
        _lru_steps(ops, dtype, B, KH, N, C, keep)
    finally:
        ops.configure(_lib.SL_OPT_LRU_MULTI_CTA, 1)


def _lru_steps(ops, dtype, B, KH, N, C, keep):
    QH = KH * 2
    g = torch.Generator().manual_seed(B * 100 + C)
    k = torch.randn((B, N, KH, 128), generator=g).to(dtype)
    v = torch.randn((B, N, KH, 128), generator=g).to(dtype)
    kd, vd = k.to(DEV), v.to(DEV)
    fused = keep > 4000 and dtype == torch.bfloat16
    if fused:
        kvd = torch.stack([kd, vd], dim=3)                           # [B,N,KH,2,128]
        kd, vd = kvd[:, :, :, 0], kvd[:, :, :, 1]
    table = ops.LruTable(B, KH, N, C, dtype, DEV, fused=fused)
    models = [[O.LruModel(N, C) for _ in range(KH)] for _ in range(B)]
    pool = [[torch.randperm(N, generator=g)[: 2 * keep] for _ in range(KH)] for _ in range(B)]   # working set
    for step in range(12):
        idx = np.zeros((B, KH, keep), np.int32)
        cnt = np.zeros((B, KH), np.int32)
        for b in range(B):
            for h in range(KH):
                n = keep - (step + b + h) % 5
                if step % 4 == 3:                                   # now and then the working set moves
                    pool[b][h] = torch.cat([pool[b][h][keep // 2:], torch.randperm(N, generator=g)[: keep // 2]])
                pick = pool[b][h][torch.randperm(len(pool[b][h]), generator=g)].unique()[:n]
                n = len(pick)
                idx[b, h, :n] = np.sort(pick.numpy())
                cnt[b, h] = n
        idx_d, cnt_d = torch.from_numpy(idx).to(DEV), torch.from_numpy(cnt).to(DEV)
        slots = ops.lru_update(table, idx_d, cnt_d, kd, vd)
        assert int(table.status.item()) == 0
        stats = table.stats.cpu().numpy()
        for b in range(B):
            for h in range(KH):
                n = cnt[b, h]
                ref_slots, hits, misses = models[b][h].update(idx[b, h, :n])
                np.testing.assert_array_equal(slots[b, h, :n].cpu().numpy(), ref_slots)
                assert (stats[b, h, 0], stats[b, h, 1]) == (hits, misses)
                np.testing.assert_array_equal(table.tok2slot[b, h].cpu().numpy(), models[b][h].tok2slot)
                np.testing.assert_array_equal(table.slot2tok[b, h].cpu().numpy(), models[b][h].slot2tok)
                np.testing.assert_array_equal(table.last_used[b, h].cpu().numpy(), models[b][h].last_used)
                res = models[b][h].slot2tok
                live = np.nonzero(res >= 0)[0]
                assert torch.equal(table.k[b, live, h].cpu(), k[b, res[live], h])
                assert torch.equal(table.v[b, live, h].cpu(), v[b, res[live], h])
        if step >= 1:
            assert stats[..., 0].sum() > 0                           # overlapping sets do hit
        q = torch.randn((B, QH, 128), generator=g).to(dtype).to(DEV)
        direct = ops.sparse_attn_decode(q, kd, vd, idx_d, cnt_d)
        resident = ops.sparse_attn_decode(q, table.k, table.v, slots, cnt_d)
        assert torch.equal(direct, resident)


def test_lru_refuses_a_table_smaller_than_the_attended_set(ops):
    table = ops.LruTable(1, 2, 100, 8, torch.bfloat16, DEV)
    kv = torch.zeros((1, 100, 2, 128), dtype=torch.bfloat16, device=DEV)
    idx = torch.arange(20, dtype=torch.int32, device=DEV).expand(1, 2, 20).contiguous()
    cnt = torch.full((1, 2), 20, dtype=torch.int32, device=DEV)
    ops.lru_update(table, idx, cnt, kv, kv)
    assert int(table.status.item()) == 3
    assert int((table.slot2tok >= 0).sum()) == 0                      # nothing was touched


@pytest.mark.parametrize("fused,host,shape", [(False, False, (2, 4, 16, 6000, 900, 700, 6)), (True, False, (2, 4, 16, 6000, 900, 700, 6)),
                                              (False, True, (2, 4, 16, 6000, 900, 700, 6)),
                                              (True, False, (1, 8, 32, 131072, 26352, 13176, 3))])   # the headline's lists: 18 splits, no cluster
def test_lru_deferred_fill(ops, fused, host, shape):
    """lru_update(defer_copy=True) + sparse_attn_decode_fill against the table that copies the missed rows itself: the
    same slots, the same resident rows after every step, and attention bit-identical to attention over the full caches."""
    B, KH, QH, N, C, keep, steps = shape
    g = torch.Generator().manual_seed(21)
    if fused:
        kv = torch.randn((B, N, KH, 2, 128), generator=g).to(torch.bfloat16).to(DEV)
        kd, vd = kv[:, :, :, 0], kv[:, :, :, 1]
    else:
        kd = torch.randn((B, N, KH, 128), generator=g).to(torch.bfloat16).to(DEV)
        vd = torch.randn((B, N, KH, 128), generator=g).to(torch.bfloat16).to(DEV)
    ptrs = None
    if host:
        k_host, v_host = kd.cpu().pin_memory(), vd.cpu().pin_memory()
        ptrs = (k_host.data_ptr(), v_host.data_ptr(), k_host.stride(0))
    ta = ops.LruTable(B, KH, N, C, torch.bfloat16, DEV, fused=fused)
    tb = ops.LruTable(B, KH, N, C, torch.bfloat16, DEV, fused=fused)
    tc = ops.LruTable(B, KH, N, C, torch.bfloat16, DEV, fused=fused)      # probe / evict in two launches
    side = torch.cuda.Stream(device=DEV)
    cur = torch.stack([torch.randperm(N, generator=g)[:keep] for _ in range(B * KH)]).view(B, KH, keep)
    misses = 0
    for step in range(steps):
        idx = torch.sort(cur, dim=-1).values.to(torch.int32).to(DEV)
        cnt = torch.full((B, KH), keep - (step % 3), dtype=torch.int32, device=DEV)      # ragged: the last entries are unused
        q = torch.randn((B, QH, 128), generator=g).to(torch.bfloat16).to(DEV)
        slots_a = ops.lru_update(ta, idx, cnt, kd, vd)
        slots_b = ops.lru_update(tb, idx, cnt, None, None, defer_copy=True)
        out_b = ops.sparse_attn_decode_fill(q, tb, slots_b, idx, cnt, kd, vd, backing_ptrs=ptrs)
        n = int(cnt[0, 0])
        sa, sb = slots_a[..., :n], slots_b[..., :n]
        assert torch.equal(torch.where(sb < 0, -sb - 1, sb), sa)
        misses += int((sb < 0).sum())
        # the two-launch form: the evictions run on a second stream beside the attention that only reads the misses
        slots_c = ops.lru_probe(tc, idx, cnt)
        side.wait_stream(torch.cuda.current_stream())
        with torch.cuda.stream(side):
            ops.lru_evict(tc, idx, cnt, kd, vd, slots_c)
        out_c = ops.sparse_attn_decode_fill(q, tc, slots_c, idx, cnt, kd, vd, backing_ptrs=ptrs, read_only=True)
        torch.cuda.current_stream().wait_stream(side)
        # (the read-only form leaves SMs to the evictions: with long lists it may split them differently, and the order
        # of the fp32 additions with it)
        assert (out_c.float() - out_b.float()).abs().max().item() <= 2e-3
        assert torch.equal(torch.where(slots_c[..., :n] < 0, sa, slots_c[..., :n]), sa) and torch.equal(slots_c[..., :n] < 0, sb < 0)
        assert torch.equal(tc.slot2tok, ta.slot2tok) and torch.equal(tc.tok2slot, ta.tok2slot) and torch.equal(tc.last_used, ta.last_used)
        assert torch.equal(tc.k.permute(0, 2, 1, 3)[ta.slot2tok >= 0], ta.k.permute(0, 2, 1, 3)[ta.slot2tok >= 0])
        assert torch.equal(tc.v.permute(0, 2, 1, 3)[ta.slot2tok >= 0], ta.v.permute(0, 2, 1, 3)[ta.slot2tok >= 0])
        assert torch.equal(tc.stats, ta.stats) and int(tc.status.item()) == 0
        assert torch.equal(out_b, ops.sparse_attn_decode(q, kd, vd, idx, cnt))
        assert torch.equal(out_b, ops.sparse_attn_decode(q, ta.k, ta.v, slots_a, cnt))
        used = ta.slot2tok >= 0                                                            # [B,KH,C]
        assert torch.equal(ta.slot2tok, tb.slot2tok) and torch.equal(ta.tok2slot, tb.tok2slot)
        ka, kb_ = ta.k.permute(0, 2, 1, 3)[used], tb.k.permute(0, 2, 1, 3)[used]
        assert torch.equal(ka, kb_) and torch.equal(ta.v.permute(0, 2, 1, 3)[used], tb.v.permute(0, 2, 1, 3)[used])
        assert int(ta.status.item()) == 0 and int(tb.status.item()) == 0
        # drift: a fifth of every list is replaced by keys that are not in it
        for r in range(B * KH):
            flat = cur.view(B * KH, keep)
            absent = torch.ones(N, dtype=torch.bool)
            absent[flat[r]] = False
            pool = absent.nonzero().flatten()
            fresh = pool[torch.randperm(pool.numel(), generator=g)[:keep // 5]]
            flat[r, torch.randperm(keep, generator=g)[:keep // 5]] = fresh
    assert misses > B * KH * keep            # the first step and the drift both missed


def test_lru_with_host_backing_store(ops):
    """The backing K/V store lives in pinned HOST memory (the offloaded variant of the reference,
    spotlight/modifiers/cpu_cache.py:60-130): the kernel reads the missed rows straight from
    it, and attention over the resident buffer equals attention over a device copy of the store."""
    B, KH, QH, N, C, keep = 1, 4, 8, 4000, 600, 500
    g = torch.Generator().manual_seed(8)
    k_host = torch.randn((B, N, KH, 128), generator=g).to(torch.bfloat16).pin_memory()
    v_host = torch.randn((B, N, KH, 128), generator=g).to(torch.bfloat16).pin_memory()
    table = ops.LruTable(B, KH, N, C, torch.bfloat16, DEV)
    kd, vd = k_host.to(DEV), v_host.to(DEV)
    for step in range(3):
        idx = torch.stack([torch.stack([torch.sort(torch.randperm(N, generator=g)[:keep]).values for _ in range(KH)])
                           for _ in range(B)]).to(torch.int32).to(DEV)
        if step == 2:
            idx = prev                                                   # same set again: all hits, no host reads
        prev = idx
        cnt = torch.full((B, KH), keep, dtype=torch.int32, device=DEV)
        slots = ops.lru_update(table, idx, cnt, None, None,
                               backing_ptrs=(k_host.data_ptr(), v_host.data_ptr(), k_host.stride(0)))
        q = torch.randn((B, QH, 128), generator=g).to(torch.bfloat16).to(DEV)
        assert torch.equal(ops.sparse_attn_decode(q, kd, vd, idx, cnt), ops.sparse_attn_decode(q, table.k, table.v, slots, cnt))
        assert int(table.status.item()) == 0
    assert table.stats[..., 1].sum().item() == 0 and table.stats[..., 0].sum().item() == B * KH * keep


def test_peer_allgather_single_rank(ops):
    """The peer-memory all-gather with one rank: the message lands in the own slot, the epoch
    advances, nothing waits. (Two and more ranks: tests/test_gpu_multi.py.)"""
    import ctypes as C
    from spotlight_b200._lib import check, lib
    nbytes = 4096
    buf = C.c_void_p()
    check(lib.sl_peer_alloc(lib.sl_peer_buffer_bytes(1, nbytes), C.byref(buf)))
    try:
        bufs = (C.c_void_p * 1)(buf.value)
        status = torch.zeros(1, dtype=torch.int32, device=DEV)
        stream = torch.cuda.current_stream().cuda_stream
        for rnd in range(3):
            msg = torch.arange(nbytes // 4, dtype=torch.int32, device=DEV) + rnd
            check(lib.sl_peer_allgather(msg.data_ptr(), nbytes, bufs, 0, 1, nbytes, status.data_ptr(), stream))
            torch.cuda.synchronize()

            class Raw:
                pass
            raw = Raw()
            raw.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (buf.value, False), "version": 3}
            got = torch.as_tensor(raw, device=DEV).view(torch.int32).clone()
            torch.testing.assert_close(got, msg, rtol=0, atol=0)
        assert int(status.item()) == 0
        with pytest.raises(ValueError):
            check(lib.sl_peer_allgather(msg.data_ptr(), 24, bufs, 0, 1, nbytes, status.data_ptr(), stream))
    finally:
        check(lib.sl_peer_free(buf))


def test_peer_wait_runs_out_and_the_context_stays_usable(ops):
    """A rank that never shows up: two exchange buffers on ONE GPU, the second never written by anybody.
    The kernel's bounded wait on that rank's flag must run out (the limit is shortened for the test),
    return normally with the status word set to 3, and the next exchange on fresh buffers must work."""
    import ctypes as C
    from spotlight_b200 import _lib
    from spotlight_b200._lib import check, lib
    nbytes = 1024
    bufs = []
    for _ in range(3):
        p = C.c_void_p()
        check(lib.sl_peer_alloc(lib.sl_peer_buffer_bytes(2, nbytes), C.byref(p)))
        bufs.append(p)
    status = torch.zeros(1, dtype=torch.int32, device=DEV)
    stream = torch.cuda.current_stream().cuda_stream
    msg = torch.arange(nbytes // 4, dtype=torch.int32, device=DEV)
    check(lib.sl_configure(_lib.SL_OPT_PEER_SPIN_LIMIT, 20000))               # ~2 ms instead of a second
    try:
        pair = (C.c_void_p * 2)(bufs[0].value, bufs[1].value)
        check(lib.sl_peer_allgather(msg.data_ptr(), nbytes, pair, 0, 2, nbytes, status.data_ptr(), stream))
        torch.cuda.synchronize()                                               # the kernel came back by itself
        assert int(status.item()) == 3
        with pytest.raises(RuntimeError):
            _lib.check(_lib.SL_ETIMEOUT if int(status.item()) == 3 else 0)
        status.zero_()
        one = (C.c_void_p * 1)(bufs[2].value)
        check(lib.sl_peer_allgather(msg.data_ptr(), nbytes, one, 0, 1, nbytes, status.data_ptr(), stream))
        torch.cuda.synchronize()
        assert int(status.item()) == 0
        assert int((msg * 2).sum().item()) == int(msg.sum().item()) * 2        # the context still computes
    finally:
        check(lib.sl_configure(_lib.SL_OPT_PEER_SPIN_LIMIT, 400000))
        for p in bufs:
            lib.sl_peer_free(p)


@pytest.mark.parametrize("kernel", [1, 2], ids=["one-barrier", "flagged-words"])
@pytest.mark.parametrize("B,N,KH,QH,k", [(1, 131072, 8, 32, 13108), (2, 60000, 4, 28, 1200), (1, 40000, 8, 40, 800), (3, 9000, 2, 2, 50)])
def test_scan_topk_sharded_single_rank(ops, B, N, KH, QH, k, kernel):
    """The one-launch sharded scan with a world of one rank (the rank's counts go through its own exchange
    buffer) must reproduce sl_scan_topk, with either of the two kernels that serve it; run three times: epochs
    advance, buffers are reused. (A buffer stays with one kernel: the two lay its flag area out differently.)"""
    import ctypes as C
    from spotlight_b200 import _lib
    from spotlight_b200._lib import check, lib

    class Peer:
        pass
    peer = Peer()
    peer.rank, peer.world = 0, 1
    peer.nbytes = ops.scan_sharded_slot_bytes(B, KH, QH)
    own = C.c_void_p()
    check(lib.sl_peer_alloc(lib.sl_peer_buffer_bytes(1, peer.nbytes), C.byref(own)))
    peer.bufs = (C.c_void_p * 1)(own.value)
    try:
        g = torch.Generator().manual_seed(N + KH)
        q = rand_codes(g, (B, QH, 4), True).to(DEV)
        cache = rand_codes(g, (B, N, KH, 4), True).to(DEV)
        ref_idx, ref_cnt = ops.scan_topk(q, cache, k, 4, 64, O.BLOCKED)
        check(lib.sl_configure(_lib.SL_OPT_SCAN_KERNEL, kernel))
        for _ in range(3):
            idx, cnt = ops.scan_topk_sharded(q, cache, peer, 0, N, k, 4, 64, O.BLOCKED)
            torch.testing.assert_close(cnt, ref_cnt, rtol=0, atol=0)
            for b in range(B):
                for h in range(KH):
                    c = int(cnt[b, h])
                    torch.testing.assert_close(idx[b, h, :c], ref_idx[b, h, :c], rtol=0, atol=0)
        ops.check_status()
    finally:
        check(lib.sl_configure(_lib.SL_OPT_SCAN_KERNEL, 1))
        torch.cuda.synchronize()
        check(lib.sl_peer_free(own))
