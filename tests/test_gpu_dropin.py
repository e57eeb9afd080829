"""The reference-facing surface on a GPU: the ``spotlight.kernel`` entry points, the caches, the
attention hook, and the whole path against the fixtures produced by the reference itself."""
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from cases import CASES, build_case  # noqa: E402
from oracle import spotlight_oracle as O  # noqa: E402

DEV = "cuda"
GOLD = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def np_u32(t):
    return t.cpu().view(torch.int32).numpy().view(np.uint32)


def test_kernel_entry_points_match_reference_contracts():
    import spotlight_b200.kernel as K
    g = torch.Generator().manual_seed(0)
    x = torch.randn((4096, 128), generator=g)
    # the reference's own known-answer check (spotlight/kernel/pack_dx_u8.py:59-73)
    xb = (x > 0).unflatten(-1, (-1, 8))
    ref = torch.zeros(xb.shape[:2], dtype=torch.uint8)
    for i in range(8):
        ref += (xb[..., i] << i).to(torch.uint8)
    ans = K.pack_dx_u8_func(x.to(DEV))
    assert torch.equal(ans.cpu(), ref)
    xb16 = x.to(torch.bfloat16).to(DEV)
    for fn in (K.pack_cuda_func, K.pack_triton_func, K.pack_dx_u32_func):
        got = fn(xb16)
        assert got.dtype == torch.uint32 and got.shape == (4096, 4)
        np.testing.assert_array_equal(np_u32(got), O.pack_signbits(x.to(torch.bfloat16)))
    # attn: u32 [B,1,QH,4] x [B,N,KH,4] -> int16 [B,N,KH], interleaved grouping
    q = torch.randint(0, 2 ** 32, (2, 1, 28, 4), generator=g, dtype=torch.int64).to(torch.uint32)
    k = torch.randint(0, 2 ** 32, (2, 1000, 4, 4), generator=g, dtype=torch.int64).to(torch.uint32)
    ref_s = O.match_count(np_u32(q), np_u32(k), O.INTERLEAVED)
    for fn in (K.attn_cuda_func, K.attn_triton_func, K.attn_dx_u32_func):
        got = fn(q.to(DEV), k.to(DEV))
        assert got.dtype == torch.int16 and got.shape == (2, 1000, 4)
        np.testing.assert_array_equal(got.cpu().numpy(), ref_s)
    with pytest.raises(AssertionError):
        K.attn_cuda_func(q.to(DEV)[..., :2], k.to(DEV)[..., :2])              # head dim must be 4
    q8 = torch.randint(0, 256, (2, 3, 1, 16), generator=g, dtype=torch.int64).to(torch.uint8)
    k8 = torch.randint(0, 256, (2, 3, 50, 16), generator=g, dtype=torch.int64).to(torch.uint8)
    np.testing.assert_array_equal(K.attn_dx_u8_func(q8.to(DEV), k8.to(DEV)).cpu().numpy(),
                                  O.match_count_u8(q8.numpy(), k8.numpy()))


def test_caches_update_and_gather():
    from spotlight_b200.modifiers import gpu_cache as GC
    GC.KVHash.init_seq_length = GC.KVCache.init_seq_length = 4096
    try:
        B, KH, L = 2, 4, 2
        hc = GC.KVHash(B, KH, 4, L, dtype=torch.uint32, device=[DEV] * L)
        kv = GC.KVCache(B, KH, 128, L, dtype=torch.bfloat16, device=[DEV] * L)
        g = torch.Generator().manual_seed(4)
        ks = torch.randn((B, 700, KH, 128), generator=g).to(torch.bfloat16)
        vs = torch.randn((B, 700, KH, 128), generator=g).to(torch.bfloat16)
        codes = torch.randint(0, 2 ** 32, (B, 700, KH, 4), generator=g, dtype=torch.int64).to(torch.uint32)
        for lo, hi in ((0, 650), (650, 651), (651, 700)):                     # prefill, then appends
            kview, vview = kv.update(1, ks[:, lo:hi].to(DEV), vs[:, lo:hi].to(DEV))
            cview = hc.update(1, codes[:, lo:hi].to(DEV))
        assert kv.length == [0, 700] and hc.length == [0, 700]
        assert kview.shape == (B, 700, KH, 128) and torch.equal(kview.cpu(), ks) and torch.equal(vview.cpu(), vs)
        assert torch.equal(cview.cpu().view(torch.int32), codes.view(torch.int32))
        attn = torch.randint(0, 897, (B, 700, KH), generator=g, dtype=torch.int64).to(torch.int16)
        kt, vt = kv.gather(1, attn.to(DEV), 70)
        assert kt.shape == (B, 70, KH, 128)
        for b in range(B):
            for h in range(KH):
                sel = torch.from_numpy(O.canonical_topk(attn[b, :, h].numpy(), 70).astype(np.int64))
                assert torch.equal(kt[b, :, h].cpu(), ks[b, sel, h]) and torch.equal(vt[b, :, h].cpu(), vs[b, sel, h])
    finally:
        GC.KVHash.init_seq_length = GC.KVCache.init_seq_length = GC.INIT_SEQ_LEN


@pytest.mark.parametrize("name", list(CASES))
def test_path_against_reference_fixtures(name):
    """Same seeded inputs as the reference run that produced the fixture. Scores: ours are
    match counts, the reference's are sign products, related by sim = 2*match - 128 (exactly
    wherever no pre-sign value is zero or within float rounding of zero). Attention: ours on the
    REFERENCE's own attended set must reproduce its output."""
    from spotlight_b200 import ops
    c = build_case(name)
    f = np.load(os.path.join(GOLD, f"ref_{name}.npz"))
    H, N, dtype = c["heads"], c["n"], c["dtype"]
    cos, sin = O.rope_tables(N, c["theta"])
    cos, sin = cos.to(dtype), sin.to(dtype)
    K = O.apply_rope(c["k"], cos, sin, torch.arange(N))                        # [1,H,N,128], reference rounding
    k_tok = K.permute(0, 2, 1, 3).contiguous().to(DEV)                         # [1,N,H,128]
    v_tok = c["v"].permute(0, 2, 1, 3).contiguous().to(DEV)
    hp = ops.HashParams.from_dict(c["params"], DEV, c["residue"])
    k_codes = ops.hash_encode(k_tok, hp)
    q_rot, q_codes = ops.decode_prepare(c["q"][:, :, 0].to(DEV), None, None, hp, None, N - 1,
                                        cos=cos[N - 1].contiguous().to(DEV), sin=sin[N - 1].contiguous().to(DEV))
    np.testing.assert_array_equal(q_rot.float().cpu().numpy()[0], f["q_rot"])
    k_keep = O.budget(N, c["mask_out"], 20)
    assert k_keep == int(f["k"])
    idx, cnt, scores = ops.scan_topk(q_codes, k_codes, k_keep, 4, 64, O.BLOCKED, return_scores=True)
    # the kernel's integers are exactly the match counts of the codes it was given
    ours = O.match_count(np_u32(q_codes)[:, None], np_u32(k_codes), O.BLOCKED)
    np.testing.assert_array_equal(scores.cpu().numpy(), ours)
    ref_idx, ref_cnt = O.select(ours, k_keep, 4, 64)
    np.testing.assert_array_equal(cnt.cpu().numpy(), ref_cnt)
    for h in range(H):
        np.testing.assert_array_equal(idx[0, h, : ref_cnt[0, h]].cpu().numpy(), ref_idx[0, h, : ref_cnt[0, h]])
    # codes against the reference's own sign bits (differences only where a pre-sign value is
    # within rounding of zero), then the score relation sim = 2*match - 128
    q_bits_ref = O.pack_signbits(f["hq_pre"])                                  # [H,4]
    assert (np_u32(q_codes)[0] != q_bits_ref).sum() <= 1
    if f["hk_bits"].size:
        k_ref = np.ascontiguousarray(f["hk_bits"]).view(np.uint32).reshape(H, N, 4).transpose(1, 0, 2)
        diff_bits = np.bitwise_count(np_u32(k_codes)[0] ^ k_ref).sum()
        assert diff_bits <= 2e-3 * k_ref.size * 32, f"{diff_bits} key code bits differ from the reference's"
    if (np_u32(q_codes)[0] == q_bits_ref).all():
        sim = 2 * ours[0].T.astype(np.int32) - 128                             # [H,N]
        mismatch = sim != f["sim"].astype(np.int32)                            # zeros (sign 0) and near-zero flips
        assert mismatch.mean() < (0.2 if dtype == torch.bfloat16 else 2e-3)
        if not mismatch.any():
            for h in range(H):
                np.testing.assert_array_equal(idx[0, h, : cnt[0, h]].cpu().numpy(), O.attended_set(f["sim"][h], k_keep))
    # attention on the reference's attended set
    att = f["attended"]
    cap = int(att.sum(1).max())
    ridx = np.full((1, H, cap), 0, np.int32)
    rcnt = np.zeros((1, H), np.int32)
    for h in range(H):
        a = np.nonzero(att[h])[0]
        ridx[0, h, : len(a)] = a
        rcnt[0, h] = len(a)
    out = ops.sparse_attn_decode(q_rot, k_tok, v_tok, torch.from_numpy(ridx).to(DEV), torch.from_numpy(rcnt).to(DEV))
    tol = 2e-2 if dtype == torch.bfloat16 else 2e-5
    assert np.abs(out.float().cpu().numpy()[0] - f["out"].reshape(H, 128)).max() <= tol
    ops.check_status()


def _tiny_llama(layers=3, heads=4, kv_heads=2, dtype=torch.bfloat16):
    from transformers import LlamaConfig, LlamaForCausalLM
    cfg = LlamaConfig(vocab_size=512, hidden_size=heads * 128, intermediate_size=256, num_hidden_layers=layers,
                      num_attention_heads=heads, num_key_value_heads=kv_heads, max_position_embeddings=4096,
                      rope_theta=500000.0, attention_bias=False, tie_word_embeddings=False)
    torch.manual_seed(0)
    return LlamaForCausalLM(cfg).to(dtype).to(DEV).eval(), cfg


def test_hook_decode_equals_dense_attention_when_nothing_is_pruned():
    """With mask_out = 0 every key is attended, so the patched model must reproduce the stock HF
    model's greedy continuation and last-position logits."""
    from spotlight_b200.modifiers.spotlight_generation import Spotlight
    model, cfg = _tiny_llama()
    ids = torch.randint(0, 512, (1, 200), generator=torch.Generator().manual_seed(1)).to(DEV)
    with torch.no_grad():
        ref_logits = model(ids).logits[:, -1].float()
        ref_next = model(torch.cat([ids, ref_logits.argmax(-1, keepdim=True)], -1)).logits[:, -1].float()
    conf = {"draft_kwargs": {"enable": True, "fix_layers": [0], "mask_out": 0.0, "min_remain": 20,
                             "num_mlp_layers": 2, "mlp_dims": "[128,128,128]", "mlp_residue": True}}
    sp = Spotlight(model, config=conf)
    with torch.no_grad():
        out = sp.model(input_ids=ids)
        assert (out.logits[:, -1] - ref_logits).abs().max().item() < 0.08
        tok = out.logits[:, -1:].argmax(-1)
        out2 = sp.model(input_ids=tok, kv_cache=out.past_key_values)          # one decode step through the kernels
        assert (out2.logits[:, -1] - ref_next).abs().max().item() < 0.08
        st = out2.past_key_values[1]
        assert st.length == 201 and int(st.last_cnt.min()) == 201


def test_hook_pruned_layer_matches_checker():
    """One pruned decode step of one layer: indices bit-exact and output within bf16 tolerance of
    the checker run on the tensors the hook actually cached."""
    from spotlight_b200.modifiers.spotlight_generation import Spotlight
    model, cfg = _tiny_llama(layers=2, heads=8, kv_heads=2)
    conf = {"draft_kwargs": {"enable": True, "fix_layers": [], "mask_out": 0.9, "min_remain": 20,
                             "num_mlp_layers": 2, "mlp_dims": "[128,256,128]", "mlp_residue": False}}
    sp = Spotlight(model, config=conf)
    for layer in sp.model.layers:                                             # make the hash non-trivial
        for p in layer.self_attn.hash_fn.parameters():
            p.data = (torch.randn(p.shape, generator=torch.Generator().manual_seed(3)) * 0.05).to(p.dtype).to(DEV)
    ids = torch.randint(0, 512, (2, 1500), generator=torch.Generator().manual_seed(2)).to(DEV)
    with torch.no_grad():
        out = sp.model(input_ids=ids)
        tok = out.logits[:, -1:].argmax(-1).view(2, 1)
        attn = sp.model.layers[0].self_attn
        captured = {}
        orig_o = attn.o_proj.forward

        def spy(x):
            captured["o"] = x.detach().clone()
            return orig_o(x)
        attn.o_proj.forward = spy
        out2 = sp.model(input_ids=tok, kv_cache=out.past_key_values)
    st = out2.past_key_values[0]
    n = st.length
    assert n == 1501
    keep = O.budget(n, 0.9, 20)
    codes = np_u32(st.codes[:, :n])
    # recompute the query codes the hook used: run prepare again on the captured projections
    hs = model.model.layers[0].input_layernorm(model.model.embed_tokens(tok))
    from spotlight_b200 import ops
    from spotlight_b200.modifiers.spotlight_generation import _rope_rows
    q = attn.q_proj(hs).view(2, 8, 128)
    cos, sin = _rope_rows(torch.tensor([n - 1], device=DEV), 500000.0, q.dtype)
    q_rot, q_codes = ops.decode_prepare(q, None, None, attn._hash_q_params(), None, n - 1,
                                        cos=cos[0].contiguous(), sin=sin[0].contiguous())
    scores = O.match_count(np_u32(q_codes)[:, None], codes, O.BLOCKED)
    ref_idx, ref_cnt = O.select(scores, keep, 4, 64)
    np.testing.assert_array_equal(st.last_cnt.cpu().numpy(), ref_cnt)
    for b in range(2):
        for h in range(2):
            np.testing.assert_array_equal(st.last_idx[b, h, : ref_cnt[b, h]].cpu().numpy(), ref_idx[b, h, : ref_cnt[b, h]])
    ref = O.sparse_attention(q_rot.cpu(), st.k[:, :n].cpu(), st.v[:, :n].cpu(), ref_idx, ref_cnt, O.BLOCKED)
    got = captured["o"].view(2, 8, 128).float().cpu()
    assert (got - ref).abs().max().item() <= 2e-2
