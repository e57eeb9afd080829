"""Pins the CPU checker (oracle/) against fixtures produced by the reference's own functions
(tests/golden/make_golden.py). CPU only."""
import hashlib

import numpy as np
import pytest
import torch

from cases import CASES, build_case
from oracle import spotlight_oracle as O


def _digest(t):
    return hashlib.sha256(t.detach().contiguous().view(torch.uint8).numpy().tobytes()).hexdigest()


def _load(name):
    return np.load(f"{__file__.rsplit('/', 1)[0]}/golden/ref_{name}.npz")


def _rotated(c):
    cos, sin = O.rope_tables(c["n"], c["theta"])
    cos, sin = cos.to(c["dtype"]), sin.to(c["dtype"])
    pos = torch.arange(c["n"])
    return O.apply_rope(c["q"], cos, sin, pos[-1:]), O.apply_rope(c["k"], cos, sin, pos)


@pytest.mark.parametrize("name", list(CASES))
def test_inputs_regenerate(name):
    c, f = build_case(name), _load(name)
    assert _digest(c["q"]) == str(f["dig_q"])
    assert _digest(c["k"]) == str(f["dig_k"])
    assert _digest(c["v"]) == str(f["dig_v"])
    assert _digest(torch.cat([w.flatten().float() for w in c["params"]["w"]])) == str(f["dig_w"])


@pytest.mark.parametrize("name", list(CASES))
def test_rope_and_hash_match_reference(name):
    c, f = build_case(name), _load(name)
    Q, K = _rotated(c)
    np.testing.assert_array_equal(Q[0, :, 0].float().numpy(), f["q_rot"])
    hq = O.hash_forward(Q, c["params"], c["residue"])
    np.testing.assert_array_equal(hq[0, :, 0].float().numpy(), f["hq_pre"])
    if f["hk_bits"].size:
        hk = O.hash_forward(K, c["params"], c["residue"])
        codes = O.pack_signbits(hk[0])                               # [H,N,4] u32
        ref = np.ascontiguousarray(f["hk_bits"]).view(np.uint32)     # little-endian bit order
        np.testing.assert_array_equal(codes, ref.reshape(codes.shape))


@pytest.mark.parametrize("name", list(CASES))
def test_scores_match_reference(name):
    c, f = build_case(name), _load(name)
    Q, K = _rotated(c)
    hq = O.hash_forward(Q, c["params"], c["residue"])
    hk = O.hash_forward(K, c["params"], c["residue"])
    sim = O.sign_sim(hq, hk)[0, :, 0].float().numpy()
    np.testing.assert_array_equal(sim.astype(np.int16), f["sim"])
    # kernel-path integers: sim = 2*match - 128 for MHA wherever no pre-sign value is exactly 0
    qc = O.pack_signbits(hq).transpose(0, 2, 1, 3)                    # [1,1,H,4]
    kc = np.ascontiguousarray(O.pack_signbits(hk).transpose(0, 2, 1, 3))  # [1,N,H,4]
    match = O.match_count(qc, kc, O.INTERLEAVED)[0].T.astype(np.int32)     # [H,N]
    clean = ((hk[0] != 0).all(-1) & (hq[0] != 0).all(-1)).numpy()     # [H,N]
    assert clean.mean() > 0.5
    np.testing.assert_array_equal((2 * match - 128)[clean], f["sim"].astype(np.int32)[clean])
    # blocked and interleaved coincide when every q head has its own kv head
    np.testing.assert_array_equal(O.match_count(qc, kc, O.BLOCKED)[0].T, match)


@pytest.mark.parametrize("name", list(CASES))
def test_selection_consistent_with_reference_topk(name):
    c, f = build_case(name), _load(name)
    k = int(f["k"])
    assert k == O.budget(c["n"], c["mask_out"], 20)
    s_end, r_start = O.forced_ranges(c["n"], 4, 64)
    for h in range(c["heads"]):
        s = f["sim"][h]
        mine = O.canonical_topk(s, k)
        ref = f["topk"][h]
        assert len(mine) == len(ref) == k == len(set(ref.tolist()))
        tau = np.sort(s)[::-1][k - 1]
        above = set(np.nonzero(s > tau)[0].tolist())
        assert above <= set(mine.tolist()) and above <= set(ref.tolist())
        np.testing.assert_array_equal(np.sort(s[mine]), np.sort(s[ref]))
        ties = np.nonzero(s == tau)[0]
        np.testing.assert_array_equal(np.setdiff1d(mine, list(above)), ties[: k - len(above)])
        # sink + recent window exactly as the reference mask has them
        ref_att = np.nonzero(f["attended"][h])[0]
        forced = np.concatenate([np.arange(s_end), np.arange(r_start, c["n"])])
        np.testing.assert_array_equal(ref_att, np.union1d(ref, forced))
        np.testing.assert_array_equal(O.attended_set(s, k), np.union1d(mine, forced))


@pytest.mark.parametrize("name", list(CASES))
def test_attention_matches_reference_on_its_index_set(name):
    c, f = build_case(name), _load(name)
    Q, K = _rotated(c)
    H, N = c["heads"], c["n"]
    att = f["attended"]
    cap = int(att.sum(1).max())
    idx = np.full((1, H, cap), -1, np.int32)
    cnt = np.zeros((1, H), np.int32)
    for h in range(H):
        a = np.nonzero(att[h])[0]
        idx[0, h, : len(a)] = a
        cnt[0, h] = len(a)
    q = Q[:, :, 0]                                                    # [1,H,128]
    k = K.permute(0, 2, 1, 3).contiguous()                            # [1,N,H,128]
    v = c["v"].permute(0, 2, 1, 3).contiguous()
    tol = 2e-2 if c["dtype"] == torch.bfloat16 else 2e-5
    ref = f["out"].reshape(H, 128)
    out = O.sparse_attention(q, k, v, idx, cnt)[0].numpy()
    assert np.abs(out - ref).max() <= tol
    dense = O.dense_masked_attention(q, k, v, idx, cnt)[0].numpy()
    assert np.abs(dense - ref).max() <= tol


def test_pack_u8_known_answer():
    g = torch.Generator().manual_seed(3)
    x = torch.randn((64, 128), generator=g)
    u8 = O.pack_signbits_u8(x)
    u32 = O.pack_signbits(x)
    np.testing.assert_array_equal(u8.view(np.uint32).reshape(u32.shape), u32)
    assert u8[0, 0] == sum(int(x[0, i] > 0) << i for i in range(8))
