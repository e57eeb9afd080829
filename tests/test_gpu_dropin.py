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


# Bounds on how far the CUDA path's codes may sit from the reference's: ten times the rates measured on a
# B200 (they are printed at the end of every run), zero where none was measured. A pre-sign value within
# rounding of zero may land on either side; nothing else may differ.
# Measured: no key or query code bit differs on any fixture that stores the reference's key bits; scores differ on
# 6.1e-5 of cfg0_linear's entries (fp32 sums within rounding of zero, one head's set then differs in one key) and on
# 0.103 of the bf16 fixture's entries, where EVERY difference is an exact 0.0 before the sign (torch.sign(0) = 0 in
# the reference's product, bit 0 in a packed code) and no attended set differs.
MAX_KEY_BIT_FLIP_RATE = {"tiny_linear": 0.0, "cfg0_linear": 0.0, "small_mlp": 0.0, "small_mlp_res_bf16": 0.0, "gqa_mlp": 0.0}
MAX_SIM_DIFF_SHARE = {"tiny_linear": 0.0, "cfg0_linear": 6.1e-4, "small_mlp": 0.0, "small_mlp_res_bf16": 0.2, "gqa_mlp": 0.0}
MIN_SET_IOU = {"tiny_linear": 1.0, "cfg0_linear": 0.99, "small_mlp": 1.0, "small_mlp_res_bf16": 1.0, "gqa_mlp": 1.0}


@pytest.mark.parametrize("name", list(CASES))
def test_path_against_reference_fixtures(name, parity_report):
    """Same seeded inputs as the reference run that produced the fixture. Scores: ours are
    match counts, the reference's are sign products, related by sim = 2*match - 128 (exactly
    wherever no pre-sign value is zero or within float rounding of zero). The attended set of the CUDA
    path is compared with the reference's own (top-k of its sim plus its window lines) on EVERY fixture:
    identical where no code bit differs, else by overlap. Attention: ours on the REFERENCE's own
    attended set must reproduce its output. (The grouped-query fixture runs here as the reference
    modifier sees it: keys repeated to the query heads, one hash per query head.)"""
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
    # ---- codes against the reference's own sign bits
    q_bits_ref = O.pack_signbits(f["hq_pre"])                                  # [H,4]
    q_flips = int(np.bitwise_count(np_u32(q_codes)[0] ^ q_bits_ref).sum())
    key_flip_rate = None
    if f["hk_bits"].size:
        k_ref = np.ascontiguousarray(f["hk_bits"]).view(np.uint32).reshape(H, N, 4).transpose(1, 0, 2)
        key_flip_rate = float(np.bitwise_count(np_u32(k_codes)[0] ^ k_ref).sum()) / (k_ref.size * 32)
        assert key_flip_rate <= MAX_KEY_BIT_FLIP_RATE[name], f"{key_flip_rate:.3g} of the key code bits differ from the reference's"
    assert q_flips <= (1 if dtype == torch.bfloat16 else 0), f"{q_flips} query code bits differ from the reference's"
    # ---- scores: sim = 2*match - 128 except where the reference's sign() saw an exact zero or a bit flipped
    sim = 2 * ours[0].T.astype(np.int32) - 128                                 # [H,N]
    sim_diff = float((sim != f["sim"].astype(np.int32)).mean())
    assert sim_diff <= MAX_SIM_DIFF_SHARE[name], f"{sim_diff:.3g} of the scores differ from the reference's"
    # ---- the attended set against the reference's own, on every fixture
    ious = [O.iou(idx[0, h, : cnt[0, h]].cpu().numpy(), O.attended_set(f["sim"][h], k_keep)) for h in range(H)]
    exact = sum(np.array_equal(idx[0, h, : cnt[0, h]].cpu().numpy(), O.attended_set(f["sim"][h], k_keep)) for h in range(H))
    assert min(ious) >= MIN_SET_IOU[name], f"attended-set IoU with the reference's set: {min(ious):.4f}"
    if sim_diff == 0.0:
        assert exact == H, "no score differs, so the attended sets must be the reference's"
    if dtype == torch.bfloat16:     # the scores differ although no code bit does: exact zeros before the sign, nothing else
        assert q_flips == 0 and key_flip_rate == 0.0
    parity_report(f"fixture {name} ({str(dtype).split('.')[-1]}, {H} heads, {N} keys)", query_bit_flips=q_flips,
                  key_bit_flip_rate=("n/a" if key_flip_rate is None else f"{key_flip_rate:.2e}"), score_diff_share=f"{sim_diff:.2e}",
                  heads_with_identical_set=f"{exact}/{H}", min_set_iou=f"{min(ious):.4f}")
    # ---- attention on the reference's attended set
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


def test_grouped_query_semantics_against_the_reference(parity_report):
    """8 query / 2 kv heads, fixture produced by the reference's modifier (per-query-head hash, scores and
    top-k over repeated keys, spotlight_generation.py:128-165).
      query_head mode: per-query-head codes of the shared keys, per-query-head lists over the UNREPEATED
                       K/V caches -> the reference's attended sets and its output;
      kv_head mode:    the reference kernels' semantics (one code per kv head from the group's first query
                       head's parameters, group-summed score, one list per kv head): a different
                       selection by design; its overlap with the reference modifier's sets and the
                       distance of its output are measured and printed."""
    from spotlight_b200 import ops
    c = build_case("gqa_mlp")
    f = np.load(os.path.join(GOLD, "ref_gqa_mlp.npz"))
    QH, KH, N, dtype = c["heads"], c["kv_heads"], c["n"], c["dtype"]
    G = QH // KH
    cos, sin = O.rope_tables(N, c["theta"])
    K = O.apply_rope(c["k_kv"], cos, sin, torch.arange(N))                     # [1,KH,N,128]
    k_tok = K.permute(0, 2, 1, 3).contiguous().to(DEV)                         # [1,N,KH,128]
    v_tok = c["v_kv"].permute(0, 2, 1, 3).contiguous().to(DEV)
    hp = ops.HashParams.from_dict(c["params"], DEV, c["residue"])
    q_rot, q_codes = ops.decode_prepare(c["q"][:, :, 0].to(DEV), None, None, hp, None, N - 1,
                                        cos=cos[N - 1].contiguous().to(DEV), sin=sin[N - 1].contiguous().to(DEV))
    keep = int(f["k"])
    ref_sets = [O.attended_set(f["sim"][j], keep) for j in range(QH)]
    # ---- query_head mode
    codes_q = ops.hash_encode(k_tok.repeat_interleave(G, dim=2), hp)           # [1,N,QH,4]
    idx, cnt = ops.scan_topk(q_codes, codes_q, keep, 4, 64, O.BLOCKED)         # KH := QH, one list per query head
    same = sum(np.array_equal(idx[0, j, : cnt[0, j]].cpu().numpy(), ref_sets[j]) for j in range(QH))
    iou_q = [O.iou(idx[0, j, : cnt[0, j]].cpu().numpy(), ref_sets[j]) for j in range(QH)]
    assert min(iou_q) >= 0.99
    att = [np.nonzero(f["attended"][j])[0] for j in range(QH)]                  # the reference's own sets (its tie choices)
    cap = max(len(s_) for s_ in att)
    ridx = np.zeros((1, QH, cap), np.int32)
    rcnt = np.zeros((1, QH), np.int32)
    for j, s_ in enumerate(att):
        ridx[0, j, : len(s_)], rcnt[0, j] = s_, len(s_)
    out_q = ops.sparse_attn_decode(q_rot, k_tok, v_tok, torch.from_numpy(ridx).to(DEV), torch.from_numpy(rcnt).to(DEV))
    err_q = float(np.abs(out_q.float().cpu().numpy()[0] - f["out"].reshape(QH, 128)).max())
    assert err_q <= 2e-5                                                        # fp32 tolerance of the suite
    # ---- kv_head mode
    lead = {"kind": "mlp", "w": [w[::G] for w in c["params"]["w"]], "b": [b_[::G] for b_ in c["params"]["b"]]}
    codes_kv = ops.hash_encode(k_tok, ops.HashParams.from_dict(lead, DEV, c["residue"]))
    idx_kv, cnt_kv = ops.scan_topk(q_codes, codes_kv, keep, 4, 64, O.BLOCKED)  # [1,KH,cap]
    iou_kv = [O.iou(idx_kv[0, j // G, : cnt_kv[0, j // G]].cpu().numpy(), ref_sets[j]) for j in range(QH)]
    out_kv = ops.sparse_attn_decode(q_rot, k_tok, v_tok, idx_kv, cnt_kv)
    err_kv = float(np.abs(out_kv.float().cpu().numpy()[0] - f["out"].reshape(QH, 128)).max())
    parity_report("grouped-query fixture gqa_mlp (8/2 heads, random-init MLP hash)",
                  query_head_mode_identical_sets=f"{same}/{QH}", query_head_mode_min_iou=f"{min(iou_q):.4f}",
                  query_head_mode_out_err=f"{err_q:.2e}", kv_head_mode_mean_iou=f"{np.mean(iou_kv):.3f}",
                  kv_head_mode_min_iou=f"{min(iou_kv):.3f}", kv_head_mode_out_err=f"{err_kv:.3f}")
    assert np.isfinite(err_kv)
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


def _conf(**kw):
    d = {"enable": True, "fix_layers": [], "mask_out": 0.9, "min_remain": 20, "num_mlp_layers": 2,
         "mlp_dims": "[128,128,128]", "mlp_residue": True}
    d.update(kw)
    return {"draft_kwargs": d}


def _randomize_hash(sp, seed=3, scale=0.05):
    g = torch.Generator().manual_seed(seed)
    for p in sp.ft_params():
        p.data = (torch.randn(p.shape, generator=g) * scale).to(p.dtype).to(p.device)
    sp.reset()


def test_generate_equals_greedy_decoding_when_nothing_is_pruned():
    """`generate` (prefill, then one kernel-path step per token) with mask_out = 0 must reproduce the
    stock HF model's greedy continuation token for token."""
    from spotlight_b200.modifiers import get_modifier
    model, cfg = _tiny_llama()
    ids = torch.randint(0, 512, (1, 150), generator=torch.Generator().manual_seed(5)).to(DEV)
    with torch.no_grad():
        ref = model.generate(ids, max_new_tokens=16, do_sample=False, eos_token_id=None, pad_token_id=0)
    _, cls = get_modifier("spotlight-generation")
    sp = cls(model, None, None, _conf(fix_layers=[0], mask_out=0.0))
    got = sp.generate(ids, max_new_tokens=16, eos_token_id=())
    assert got.shape == ref.shape and torch.equal(got, ref)


def test_checkpoint_round_trip_in_the_reference_format():
    """save_checkpoint writes the reference's flat list (per layer: proj, bias of every MLP layer,
    spotlight/modifier.py:62-76, spotlight_generation.py:363-369); a fresh model that loads it produces
    the same codes bit for bit. The linear-hash modifier keeps one tensor per pruned layer."""
    import tempfile
    from spotlight_b200 import ops
    from spotlight_b200.modifiers import get_modifier
    _, cls = get_modifier("spotlight-generation")
    model, cfg = _tiny_llama(layers=2, heads=4, kv_heads=4)
    a = cls(model, None, None, _conf(mlp_dims="[128,256,128]", mlp_residue=False, fix_layers=[0]))
    _randomize_hash(a)
    x = torch.randn((1, 300, 4, 128), generator=torch.Generator().manual_seed(1)).to(torch.bfloat16).to(DEV)
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "hash.pth")
        a.save_checkpoint(path)
        flat = torch.load(path, map_location="cpu")
        assert [tuple(t.shape) for t in flat] == [(1, 4, 128, 256), (1, 4, 1, 256), (1, 4, 256, 128), (1, 4, 1, 128)] * 2
        model2, _ = _tiny_llama(layers=2, heads=4, kv_heads=4)
        b = cls(model2, None, path, _conf(mlp_dims="[128,256,128]", mlp_residue=False, fix_layers=[0]))
    for la, lb in zip(a.model.layers, b.model.layers):
        assert torch.equal(la.self_attn.hash_fn.codes(x), lb.self_attn.hash_fn.codes(x))
        assert torch.equal(ops.hash_encode(x, la.self_attn._hash_k_params()), ops.hash_encode(x, lb.self_attn._hash_k_params()))
    _, lin = get_modifier("linearhashing-generation")
    model3, _ = _tiny_llama(layers=3, heads=4, kv_heads=4)
    c = lin(model3, None, None, _conf(fix_layers=[0, 1]))
    assert [tuple(p.shape) for p in c.ft_params()] == [(1, 4, 128, 128)]       # the one pruned layer
    with pytest.raises(NotImplementedError):
        get_modifier("spotlight-train")


def test_hook_query_head_mode_matches_the_reference_math(parity_report):
    """gqa_mode = "query_head", no window: the hook's attended sets against the reference modifier's math
    (hash_fn of q and of the repeated keys, sign product, top-k per query head,
    spotlight_generation.py:13-23,157-165) restated by the checker on the tensors the hook cached."""
    from spotlight_b200 import ops
    from spotlight_b200.modifiers.spotlight_generation import Spotlight
    model, cfg = _tiny_llama(layers=2, heads=8, kv_heads=2)
    sp = Spotlight(model, config=_conf(gqa_mode="query_head", sink=0, recent=0))
    _randomize_hash(sp)
    ids = torch.randint(0, 512, (1, 900), generator=torch.Generator().manual_seed(4)).to(DEV)
    with torch.no_grad():
        out = sp.model(input_ids=ids)
        tok = out.logits[:, -1:].argmax(-1).view(1, 1)
        attn = sp.model.layers[1].self_attn
        captured = {}
        orig_q = attn.q_proj.forward
        attn.q_proj.forward = lambda x: captured.setdefault("q", orig_q(x))
        out2 = sp.model(input_ids=tok, kv_cache=out.past_key_values)
    st = out2.past_key_values[1]
    n = st.length
    assert st.codes.shape[2] == 8 and st.last_idx.shape[1] == 8 and st.kv.shape[2] == 2
    keep = O.budget(n, 0.9, 20)
    from spotlight_b200.modifiers.spotlight_generation import _rope_rows
    cos, sin = _rope_rows(torch.tensor([n - 1], device=DEV), 500000.0, torch.bfloat16)
    q_rot, q_codes = ops.decode_prepare(captured["q"].view(1, 8, 128), None, None, attn._hash_q_params(), None, n - 1,
                                        cos=cos[0].contiguous(), sin=sin[0].contiguous())
    # kernels against the checker, given the device's codes
    scores = O.match_count(np_u32(q_codes)[:, None], np_u32(st.codes[:, :n]), O.BLOCKED)
    ref_idx, ref_cnt = O.select(scores, keep, 0, 0)
    np.testing.assert_array_equal(st.last_cnt.cpu().numpy(), ref_cnt)
    for j in range(8):
        np.testing.assert_array_equal(st.last_idx[0, j, : ref_cnt[0, j]].cpu().numpy(), ref_idx[0, j, : ref_cnt[0, j]])
    # the reference's math on the cached tensors (bf16 operators on the CPU)
    params = {"kind": "mlp", "w": [l.proj.data[0].cpu() for l in attn.hash_fn.mlp], "b": [l.bias.data[0, :, 0].cpu() for l in attn.hash_fn.mlp]}
    k_rep = st.k[:, :n].repeat_interleave(4, dim=2).permute(0, 2, 1, 3).cpu()   # [1,8,n,128], already rotated
    hq = O.hash_forward(q_rot.cpu()[:, :, None], params, True)
    hk = O.hash_forward(k_rep, params, True)
    sim = O.sign_sim(hq, hk)[0, :, 0].float().numpy()
    ious = [O.iou(st.last_idx[0, j, : ref_cnt[0, j]].cpu().numpy(), O.attended_set(sim[j], keep, 0, 0)) for j in range(8)]
    parity_report("hook, query_head mode, tiny Llama 8/2 heads, bf16", min_set_iou_vs_reference_math=f"{min(ious):.4f}")
    assert min(ious) >= 0.9


def test_upper_bound_modifier_and_hash_quality(parity_report):
    """The oracle-selection baseline (spotlight/modifiers/upperbound_generation.py): its attended sets
    equal the checker's exact top-k of q.K^T on the cached tensors (up to logits within rounding of the
    threshold), and the overlap of the hashed selection with it is reported as the quality figure."""
    from spotlight_b200.modifiers import get_modifier
    from spotlight_b200.modifiers.upperbound_generation import selection_iou
    _, UB = get_modifier("upperbound-generation")
    _, SP = get_modifier("spotlight-generation")
    ids = torch.randint(0, 512, (2, 700), generator=torch.Generator().manual_seed(6)).to(DEV)
    results = {}
    for mode in ("kv_head", "query_head"):
        model, cfg = _tiny_llama(layers=2, heads=8, kv_heads=2)
        ub = UB(model, None, None, _conf(gqa_mode=mode))
        with torch.no_grad():
            out = ub.model(input_ids=ids)
            tok = out.logits[:, -1:].argmax(-1).view(2, 1)
            attn = ub.model.layers[0].self_attn
            captured = {}
            orig_o = attn.o_proj.forward

            def spy(x):
                captured["o"] = x.detach().clone()
                return orig_o(x)
            attn.o_proj.forward = spy
            orig_q = attn.q_proj.forward
            attn.q_proj.forward = lambda x: captured.setdefault("q", orig_q(x))
            out2 = ub.model(input_ids=tok, kv_cache=out.past_key_values)
        st = out2.past_key_values[0]
        n = st.length
        keep = O.budget(n, 0.9, 20)
        from spotlight_b200 import ops
        from spotlight_b200.modifiers.spotlight_generation import _rope_rows
        cos, sin = _rope_rows(torch.tensor([n - 1], device=DEV), 500000.0, torch.bfloat16)
        from spotlight_b200.modifiers.spotlight_generation import _IDENTITY_HASH
        q_rot, _ = ops.decode_prepare(captured["q"].view(2, 8, 128), None, None, _IDENTITY_HASH.get(8, captured["q"]), None, n - 1,
                                      cos=cos[0].contiguous(), sin=sin[0].contiguous())
        logits = O.exact_logits(q_rot.cpu(), st.k[:, :n].cpu(), mode == "query_head")
        ref_idx, ref_cnt = O.select_by_logits(logits, keep, 4, 64)
        LH = 8 if mode == "query_head" else 2
        assert st.last_idx.shape[1] == LH
        np.testing.assert_array_equal(st.last_cnt.cpu().numpy(), ref_cnt)
        worst = min(O.iou(st.last_idx[b, h, : ref_cnt[b, h]].cpu().numpy(), ref_idx[b, h, : ref_cnt[b, h]])
                    for b in range(2) for h in range(LH))
        assert worst >= 0.98                                # fp32 on the device against fp64: ties at the threshold only
        if LH == 2:                                         # the layer's output over exactly these sets
            ref_out = O.sparse_attention(q_rot.cpu(), st.k[:, :n].cpu(), st.v[:, :n].cpu(), st.last_idx.cpu().numpy(),
                                         st.last_cnt.cpu().numpy(), O.BLOCKED)
            assert (captured["o"].view(2, 8, 128).float().cpu() - ref_out).abs().max().item() <= 2e-2
        # the hashed selection of a random-init hash on the same model and prompt, against the exact one
        model_h, _ = _tiny_llama(layers=2, heads=8, kv_heads=2)
        sp = SP(model_h, None, None, _conf(gqa_mode=mode))
        _randomize_hash(sp)
        with torch.no_grad():
            o1 = sp.model(input_ids=ids)
            o2 = sp.model(input_ids=tok, kv_cache=o1.past_key_values)
        sh = o2.past_key_values[0]
        results[mode] = float(selection_iou(sh.last_idx, sh.last_cnt, st.last_idx, st.last_cnt, n).mean())
    parity_report("hash-vs-exact selection overlap (tiny Llama, random-init hash, 90 % pruned)",
                  **{f"{m}_mean_iou": f"{v:.3f}" for m, v in results.items()})


def test_offloaded_and_aliased_caches():
    """cpu_cache: K/V of the non-frozen layers in pinned host memory, gather pulls the selected rows across
    PCIe (spotlight/modifiers/cpu_cache.py:60-130). fake_cache: batch row 0 stored once and read by every
    batch row (spotlight/modifiers/fake_cache.py:42-49,96-106)."""
    from spotlight_b200 import ops
    from spotlight_b200.modifiers import cpu_cache as CC, fake_cache as FC
    g = torch.Generator().manual_seed(2)
    B, KH, L, N = 2, 4, 3, 600
    ks = torch.randn((B, N, KH, 128), generator=g).to(torch.bfloat16)
    vs = torch.randn((B, N, KH, 128), generator=g).to(torch.bfloat16)
    kv = CC.KVCache(B, KH, 128, L, dtype=torch.bfloat16, freeze=[0], device=[DEV] * L)
    kv.max_score = 128 * 7
    assert kv.key_cache[0].is_cuda and not kv.key_cache[1].is_cuda and kv.key_cache[1].is_pinned()
    attn = torch.randint(0, 897, (B, N, KH), generator=g, dtype=torch.int64).to(torch.int16)
    for layer in (0, 1):
        for lo, hi in ((0, 590), (590, 600)):
            kv.update(layer, ks[:, lo:hi].to(DEV), vs[:, lo:hi].to(DEV))
        kt, vt = kv.gather(layer, attn.to(DEV), 50)
        assert kt.is_cuda and kt.shape == (B, 50, KH, 128)
        for b in range(B):
            for h in range(KH):
                sel = torch.from_numpy(O.canonical_topk(attn[b, :, h].numpy(), 50).astype(np.int64))
                assert torch.equal(kt[b, :, h].cpu(), ks[b, sel, h]) and torch.equal(vt[b, :, h].cpu(), vs[b, sel, h])
    # aliased batch: 16 rows of batch over one stored row
    hc = FC.KVHash(16, KH, 4, 1, dtype=torch.uint32, device=[DEV])
    fk = FC.KVCache(16, KH, 128, 1, dtype=torch.bfloat16, device=[DEV])
    FC.KVHash.init_seq_length = FC.KVCache.init_seq_length = 4096
    try:
        hc = FC.KVHash(16, KH, 4, 1, dtype=torch.uint32, device=[DEV])
        fk = FC.KVCache(16, KH, 128, 1, dtype=torch.bfloat16, device=[DEV])
        codes = torch.randint(0, 2 ** 32, (16, N, KH, 4), generator=g, dtype=torch.int64).to(torch.uint32)
        cview = hc.update(0, codes.to(DEV))
        kview, vview = fk.update(0, ks[:1].expand(16, -1, -1, -1).to(DEV), vs[:1].expand(16, -1, -1, -1).to(DEV))
        assert cview.shape == (16, N, KH, 4) and cview.stride(0) == 0 and kview.stride(0) == 0
        q_codes = torch.randint(0, 2 ** 32, (16, 28, 4), generator=g, dtype=torch.int64).to(torch.uint32)
        idx, cnt = ops.scan_topk(q_codes.to(DEV), cview, 40, 4, 64)
        ref_scores = O.match_count(np_u32(q_codes)[:, None], np.broadcast_to(np_u32(codes[:1]), (16, N, KH, 4)), O.BLOCKED)
        ref_idx, ref_cnt = O.select(ref_scores, 40, 4, 64)
        np.testing.assert_array_equal(cnt.cpu().numpy(), ref_cnt)
        for b in range(16):
            for h in range(KH):
                np.testing.assert_array_equal(idx[b, h, : ref_cnt[b, h]].cpu().numpy(), ref_idx[b, h, : ref_cnt[b, h]])
        q = torch.randn((16, 28, 128), generator=g).to(torch.bfloat16)
        out = ops.sparse_attn_decode(q.to(DEV), kview, vview, idx, cnt)
        ref = O.sparse_attention(q, ks[:1].expand(16, -1, -1, -1), vs[:1].expand(16, -1, -1, -1), ref_idx, ref_cnt, O.BLOCKED)
        assert (out.float().cpu() - ref).abs().max().item() <= 2e-2
    finally:
        FC.KVHash.init_seq_length = FC.KVCache.init_seq_length = FC.INIT_SEQ_LEN
    ops.check_status()
