"""Decode-time attention hook: drop-in for the reference's generation modifier
(spotlight/modifiers/spotlight_generation.py:109-226, 298-330, 470-495).

``self_attn_forward(self, hidden_states, kv_cache=None) -> (attn_output, kv_cache)`` keeps the
reference's signature and is bound onto every HF ``LlamaAttention`` with ``types.MethodType`` by
``Decoder``. ``kv_cache`` is an opaque per-layer ``LayerState`` (code cache + post-RoPE K cache +
V cache) instead of the reference's concatenated tensors.

Per decode token the hook runs three launches of the CUDA library:
  decode_prepare  RoPE(q, k_new) + hash + sign + pack + append code / K / V rows
  scan_topk       Hamming scan of the code cache + exact top-k + sink/recent window
  sparse_attn     gather-attention over the attended keys only
The q/k/v/o projections stay torch ``nn.Linear`` calls: they are not part of the retrieval path.

Semantics fixed where the reference is silent (all explicit, none hidden):
  * ``draft_kwargs['gqa_mode']`` chooses between the reference's two GQA semantics:
      "kv_head" (default)  keys are hashed per KV head (with the hash parameters of the group's first
                   query head, or of ``hash_fn_k`` when the layer has one), scores are summed over the
                   query heads of a group and one top-k is taken per KV head, as in the reference's
                   kernels (spotlight/kernel/attn_k4_q28.cu:72-92, spotlight/modifiers/gpu_cache.py:48-54);
      "query_head" every query head hashes the (shared) keys with its OWN parameters and takes its own
                   top-k, as in the reference's modifier (spotlight_generation.py:128-165); the code
                   cache holds one code per query head (G times the bytes to scan), K/V stay per KV head.
    With QH == KH the two are the same computation;
  * query head j belongs to kv head j // G (HF ``repeat_kv``, spotlight_generation.py:128-129);
  * the sink (4) and recent (64) windows of spotlight/modifiers/spotlight_evaluation.py:341-346
    are applied at decode; ``draft_kwargs['sink'] / ['recent']`` override them (0 / 0 is the reference's
    generation modifier, which has no window);
  * keys are cached AFTER RoPE (their position never changes), q is rotated at its position;
    the reference re-rotates the whole cache every step (modify_llama.py:98-108) with the same
    result; positions beyond the reference's 8192-row table (spotlight_generation.py:139) work;
  * any batch size (the reference asserts batch 1, :138).
"""
from __future__ import annotations

import json
import types
from typing import List, Optional

import torch

from .. import ops
from .._lib import GQA_BLOCKED
from ..workloads import budget


# ------------------------------------------------------------------------------- hash modules
class MLPLayer(torch.nn.Module):
    """Parameter layout of spotlight_generation.py:229-236: proj [1,H,in,out], bias [1,H,1,out]."""

    def __init__(self, info, num_heads, in_features, out_features, silu=False, residue=True):
        super().__init__()
        self.proj = torch.nn.Parameter(torch.randn((1, num_heads, in_features, out_features), **info) * 0.001)
        self.bias = torch.nn.Parameter(torch.zeros((1, num_heads, 1, out_features), **info))
        self.has_silu = silu
        self.resi = residue


class MLPHashingFunction(torch.nn.Module):
    """spotlight_generation.py:243-255. ``codes`` runs hash + sign + pack on the device; the
    activations themselves are never materialised."""

    def __init__(self, info, num_heads, num_mlp_layers, mlp_dims, mlp_residue):
        super().__init__()
        self.mlp = torch.nn.ModuleList(
            MLPLayer(info, num_heads, mlp_dims[i], mlp_dims[i + 1], i < num_mlp_layers - 1, mlp_residue)
            for i in range(num_mlp_layers))
        self.residue = mlp_residue

    def hash_params(self, heads: Optional[torch.Tensor] = None) -> ops.HashParams:
        ws = [l.proj.data[0] if heads is None else l.proj.data[0, heads] for l in self.mlp]
        bs = [l.bias.data[0, :, 0] if heads is None else l.bias.data[0, heads, 0] for l in self.mlp]
        return ops.HashParams(ws, bs, self.residue)

    def codes(self, x: torch.Tensor) -> torch.Tensor:
        """x [B,T,H,128] -> uint32 [B,T,H,4]."""
        return ops.hash_encode(x, self.hash_params())


class LinearHashingFunction(torch.nn.Module):
    """linearhashing_generation.py:224-231: one [1,H,128,128] projection."""

    def __init__(self, info, num_heads=32):
        super().__init__()
        self.linear = torch.nn.Parameter(torch.randn((1, num_heads, 128, 128), **info))

    def hash_params(self, heads: Optional[torch.Tensor] = None) -> ops.HashParams:
        w = self.linear.data[0] if heads is None else self.linear.data[0, heads]
        return ops.HashParams([w], [None], False)

    def codes(self, x: torch.Tensor) -> torch.Tensor:
        return ops.hash_encode(x, self.hash_params())


# ------------------------------------------------------------------------------- per-layer state
class LayerState:
    """What the hook keeps per layer between steps (the reference keeps two concatenated
    tensors, spotlight_generation.py:131-136): one fused K|V cache [B, cap, KH, 2, 128] (a key's K and
    V rows adjacent), keys stored AFTER RoPE, and the code cache [B, cap, LH, 4] with LH = KH
    ("kv_head" mode) or QH ("query_head" mode)."""

    def __init__(self, batch, kv_heads, capacity, dtype, device, list_heads=None):
        self.kv = torch.empty((batch, capacity, kv_heads, 2, 128), dtype=dtype, device=device)
        self.codes = torch.empty((batch, capacity, list_heads or kv_heads, 4), dtype=torch.uint32, device=device)
        self.length = 0
        self.last_idx = None
        self.last_cnt = None

    @property
    def k(self):
        return self.kv[:, :, :, 0]

    @property
    def v(self):
        return self.kv[:, :, :, 1]

    @property
    def capacity(self):
        return self.kv.shape[1]

    def reserve(self, n):
        """Grow (doubling) when a caller outruns the capacity it announced with
        ``draft_kwargs['max_seq_len']``; a correctly sized state never takes this path."""
        if n <= self.capacity:
            return
        cap = max(n, 2 * self.capacity)
        for name in ("kv", "codes"):
            old = getattr(self, name)
            new = torch.empty((old.shape[0], cap, *old.shape[2:]), dtype=old.dtype, device=old.device)
            new[:, : self.length] = old[:, : self.length]
            setattr(self, name, new)


def _rope_theta(config) -> float:
    rp = getattr(config, "rope_parameters", None)
    if isinstance(rp, dict) and "rope_theta" in rp:
        return float(rp["rope_theta"])
    return float(getattr(config, "rope_theta", 10000.0))


def _rope_rows(positions: torch.Tensor, theta: float, dtype: torch.dtype):
    inv = 1.0 / (theta ** (torch.arange(0, 128, 2, dtype=torch.float32, device=positions.device) / 128))
    f = positions.to(torch.float32)[:, None] * inv[None, :]
    emb = torch.cat([f, f], dim=-1)
    return emb.cos().to(dtype), emb.sin().to(dtype)


_ROPE_TABLES = {}


def _rope_table(n: int, theta: float, dtype: torch.dtype, device):
    """cos / sin rows of positions [0, n) on `device`, computed once and grown by doubling: the decode
    hook reads row `pos` as a view, so a token costs no host-to-device copy and no table kernels."""
    key = (torch.device(device), dtype, float(theta))
    cur = _ROPE_TABLES.get(key)
    if cur is None or cur[0].shape[0] < n:
        rows = max(n, 4096, 0 if cur is None else 2 * cur[0].shape[0])
        cur = _rope_rows(torch.arange(rows, device=device), theta, dtype)
        _ROPE_TABLES[key] = cur
    return cur


def _rotate(x, cos, sin):
    half = x.shape[-1] // 2
    return x * cos + torch.cat([-x[..., half:], x[..., :half]], dim=-1) * sin


# ------------------------------------------------------------------------------- the hook
def _select(self, q_rot, q_codes, st, n, lh):
    """Index source of the pruned layers: Hamming scan + exact top-k + window over the code cache.
    Returns (idx int32 [B,LH,cap] ascending, cnt int32 [B,LH])."""
    kw = self.draft_kwargs
    keep = budget(n, kw["mask_out"], kw.get("min_remain", 20))
    return ops.scan_topk(q_codes, st.codes[:, :n], keep, int(kw.get("sink", 4)), int(kw.get("recent", 64)), GQA_BLOCKED)


def self_attn_forward(self, hidden_states: torch.Tensor, kv_cache: Optional[LayerState] = None):
    cfg = self.config
    num_heads, num_kv_heads = cfg.num_attention_heads, cfg.num_key_value_heads
    head_dim = cfg.hidden_size // num_heads
    assert head_dim == 128, "the retrieval kernels are built for head_dim 128"
    B, T, _ = hidden_states.shape
    kw = self.draft_kwargs
    G = num_heads // num_kv_heads
    per_q = kw.get("gqa_mode", "kv_head") == "query_head" and G > 1
    pruned = bool(kw.get("enable", True)) and not self.is_fix_layer
    hashed = pruned and getattr(self, "index_source", "hash") == "hash"
    lh = num_heads if (per_q and hashed) else num_kv_heads     # heads of the code cache: per kv head or per query head

    q = self.q_proj(hidden_states).view(B, T, num_heads, head_dim)
    k = self.k_proj(hidden_states).view(B, T, num_kv_heads, head_dim)
    v = self.v_proj(hidden_states).view(B, T, num_kv_heads, head_dim)
    theta = _rope_theta(cfg)

    if kv_cache is None:
        cap = int(kw.get("max_seq_len", 0)) or (T + 4096)
        kv_cache = LayerState(B, num_kv_heads, max(cap, T), q.dtype, q.device, lh)
    st = kv_cache

    if T > 1:
        # prefill (or a multi-token append): dense causal attention, as the reference does
        # (spotlight_generation.py:145-147, 217-224); then build the code cache of the new keys.
        st.reserve(st.length + T)
        lo, hi = st.length, st.length + T
        cos, sin = _rope_table(hi, theta, q.dtype, q.device)
        cos, sin = cos[lo:hi], sin[lo:hi]
        qr = _rotate(q, cos[None, :, None, :], sin[None, :, None, :])
        st.k[:, lo:hi] = _rotate(k, cos[None, :, None, :], sin[None, :, None, :])
        st.v[:, lo:hi] = v
        if hashed:
            if per_q:   # every query head's own code of the shared key (repeat_kv, then hash_fn, spotlight_generation.py:128,17)
                ops.hash_encode(st.k[:, lo:hi].repeat_interleave(G, dim=2), self._hash_q_params(), out=st.codes[:, lo:hi])
            else:
                ops.hash_encode(st.k[:, lo:hi], self._hash_k_params(), out=st.codes[:, lo:hi])
        st.length = hi
        kk = st.k[:, :hi].permute(0, 2, 1, 3)
        vv = st.v[:, :hi].permute(0, 2, 1, 3)
        mask = torch.ones((T, hi), dtype=torch.bool, device=q.device).tril(diagonal=hi - T)
        o = torch.nn.functional.scaled_dot_product_attention(
            qr.permute(0, 2, 1, 3), kk, vv, attn_mask=mask, enable_gqa=num_heads != num_kv_heads)
        o = o.permute(0, 2, 1, 3).reshape(B, T, num_heads * head_dim)
        return self.o_proj(o), st

    # ---- one decode token
    st.reserve(st.length + 1)
    pos = st.length
    cos, sin = _rope_table(pos + 1, theta, q.dtype, q.device)
    cos, sin = cos[pos], sin[pos]
    if hashed and per_q:
        # codes of the new key under every query head's parameters; its K/V rows are appended per KV head
        q_rot, q_codes = ops.decode_prepare(q[:, 0], k[:, 0].repeat_interleave(G, dim=1), None, self._hash_q_params(),
                                            self._hash_q_params(), pos, code_cache=st.codes, cos=cos, sin=sin)
        st.k[:, pos] = _rotate(k[:, 0], cos, sin)
        st.v[:, pos] = v[:, 0]
    else:
        q_rot, q_codes = ops.decode_prepare(
            q[:, 0], k[:, 0], v[:, 0], self._hash_q_params() if hashed else _IDENTITY_HASH.get(num_heads, q),
            self._hash_k_params() if hashed else _IDENTITY_HASH.get(num_kv_heads, q), pos,
            code_cache=st.codes, k_cache=st.k, v_cache=st.v, cos=cos, sin=sin)
    st.length = n = pos + 1
    if hashed:
        idx, cnt = _select(self, q_rot, q_codes, st, n, lh)
    elif pruned:
        idx, cnt = self.select_indices(q_rot, st, n)          # another index source (e.g. the exact top-k)
    else:
        idx = torch.arange(n, dtype=torch.int32, device=q.device).expand(B, num_kv_heads, n).contiguous()
        cnt = torch.full((B, num_kv_heads), n, dtype=torch.int32, device=q.device)
    st.last_idx, st.last_cnt = idx, cnt
    o = ops.sparse_attn_decode(q_rot, st.k[:, :n], st.v[:, :n], idx, cnt, GQA_BLOCKED)
    return self.o_proj(o.view(B, 1, num_heads * head_dim)), st


class _IdentityHash:
    """Layers that do not hash (dense layers, other index sources) still go through decode_prepare for
    RoPE and the cache appends; it needs SOME hash parameters, so they get a 128x128 linear one per
    (heads, dtype, device), built once. The codes it produces are never read."""

    def __init__(self):
        self._cache = {}

    def get(self, heads, like):
        key = (heads, like.dtype, like.device)
        if key not in self._cache:
            w = torch.zeros((heads, 128, 128), dtype=like.dtype, device=like.device)
            self._cache[key] = ops.HashParams([w], [None], False)
        return self._cache[key]


_IDENTITY_HASH = _IdentityHash()


def _hash_q_params(self):
    if getattr(self, "_hq", None) is None:
        self._hq = self.hash_fn.hash_params()
    return self._hq


def _hash_k_params(self):
    """Key-side parameters: the module's own when QH == KH; for GQA the parameters of the first
    query head of each group (a reference checkpoint stores one set per query head)."""
    if getattr(self, "_hk", None) is None:
        cfg = self.config
        qh, kh = cfg.num_attention_heads, cfg.num_key_value_heads
        fn = getattr(self, "hash_fn_k", None)
        if fn is not None:
            self._hk = fn.hash_params()
        elif qh == kh:
            self._hk = self._hash_q_params()
        else:
            lead = torch.arange(kh, device=self.q_proj.weight.device) * (qh // kh)
            self._hk = self.hash_fn.hash_params(lead)
    return self._hk


# ------------------------------------------------------------------------------- model plumbing
def layer_forward(self, hidden_states, kv_cache=None):
    """spotlight_generation.py:82-106."""
    dev = self.self_attn.q_proj.weight.device
    if hidden_states.device != dev:
        hidden_states = hidden_states.to(dev)
    h, kv_cache = self.self_attn(self.input_layernorm(hidden_states), kv_cache)
    hidden_states = hidden_states + h
    hidden_states = hidden_states + self.mlp(self.post_attention_layernorm(hidden_states))
    return hidden_states, kv_cache


def model_model_forward(self, input_ids=None, kv_cache=None):
    """spotlight_generation.py:58-79."""
    hidden_states = self.embed_tokens(input_ids)
    if kv_cache is None:
        kv_cache = [None] * len(self.layers)
    for i, layer in enumerate(self.layers):
        hidden_states, kv_cache[i] = layer(hidden_states, kv_cache[i])
    return self.norm(hidden_states), kv_cache


def model_forward(self, input_ids, labels=None, kv_cache=None, **kwargs):
    """spotlight_generation.py:26-55: logits of the last position only."""
    from transformers.modeling_outputs import CausalLMOutputWithPast
    hidden_states, kv_cache = self.model(input_ids=input_ids, kv_cache=kv_cache)
    logits = self.lm_head(hidden_states[..., -1:, :]).float()
    return CausalLMOutputWithPast(loss=None, logits=logits, past_key_values=kv_cache)


class Decoder(torch.nn.Module):
    """Binds the hook onto every layer of an HF Llama-family causal LM
    (spotlight_generation.py:298-330) and owns the hash modules."""

    def __init__(self, decoder, draft_kwargs, hash_kind: str = "mlp"):
        super().__init__()
        self.decoder = decoder
        self.draft_kwargs = draft_kwargs
        self.hash_kind = hash_kind
        fix_layers = draft_kwargs.get("fix_layers", [])
        num_mlp_layers = draft_kwargs.get("num_mlp_layers", 2)
        mlp_dims = draft_kwargs.get("mlp_dims", "[128,128,128]")
        mlp_dims = json.loads(mlp_dims) if isinstance(mlp_dims, str) else list(mlp_dims)
        mlp_residue = draft_kwargs.get("mlp_residue", True)
        model = self.model
        model.forward = types.MethodType(model_forward, model)
        model.model.forward = types.MethodType(model_model_forward, model.model)
        heads = model.config.num_attention_heads
        for i, layer in enumerate(self.layers):
            attn = layer.self_attn
            w = attn.q_proj.weight.data
            info = {"device": w.device, "dtype": w.dtype}
            attn.is_fix_layer = i in fix_layers
            attn.draft_kwargs = draft_kwargs
            attn.config = model.config
            layer.forward = types.MethodType(layer_forward, layer)
            attn.forward = types.MethodType(self_attn_forward, attn)
            attn._hash_q_params = types.MethodType(_hash_q_params, attn)
            attn._hash_k_params = types.MethodType(_hash_k_params, attn)
            attn._hq = attn._hk = None
            if hash_kind == "linear":
                # as the reference, which gives only the pruned layers a hash (linearhashing_generation.py:330-331)
                if not attn.is_fix_layer:
                    attn.hash_fn = LinearHashingFunction(info, heads)
            elif hash_kind == "mlp":
                attn.hash_fn = MLPHashingFunction(info, heads, num_mlp_layers, mlp_dims, mlp_residue)
            else:
                attn.index_source = hash_kind            # no hash at all: the layer brings its own select_indices

    @property
    def layers(self):
        return self.decoder.model.layers

    @property
    def model(self):
        return self.decoder

    def reset(self):
        for layer in self.layers:
            layer.self_attn._hq = layer.self_attn._hk = None

    def layer_ft_params(self, layer):
        """spotlight_generation.py:357-360."""
        attn = self.layers[layer].self_attn
        if attn.is_fix_layer or not hasattr(attn, "hash_fn"):
            return []
        return list(attn.hash_fn.parameters())

    def ft_params(self, layer=None):
        """The reference's order: layer by layer, per layer ``proj, bias`` of every MLP layer
        (spotlight_generation.py:363-369); every layer for the MLP hash, the pruned layers only for the
        linear hash (linearhashing_generation.py:375-382)."""
        params = []
        for l in self.layers:
            if hasattr(l.self_attn, "hash_fn"):
                params += l.self_attn.hash_fn.parameters()
        return list(params)

    def forward(self, input_ids, labels=None, kv_cache=None):
        return self.decoder(input_ids=input_ids, labels=labels, kv_cache=kv_cache)


class Spotlight(torch.nn.Module):
    """spotlight_generation.py:453-495 + the checkpoint format of spotlight/modifier.py:62-76
    (a flat list of tensors in ``ft_params()`` order)."""

    def __init__(self, model, save_ckp=None, load_ckp=None, config=None, hash_kind: str = "mlp"):
        super().__init__()
        if isinstance(config, str):
            with open(config) as f:
                config = json.load(f)
        self.conf = config
        self.model = Decoder(model, draft_kwargs=config["draft_kwargs"], hash_kind=hash_kind)
        self.save_ckp, self.load_ckp = save_ckp, load_ckp
        if load_ckp is not None:
            self.load_checkpoint()

    def ft_params(self):
        return self.model.ft_params()

    def reset(self):
        self.model.reset()

    def forward(self, *args, **kwargs):
        return self.model(*args, **kwargs)

    def load_checkpoint(self, ckp: Optional[str] = None):
        tensors = torch.load(ckp or self.load_ckp, map_location="cpu")
        params = self.ft_params()
        assert len(tensors) == len(params), "number of parameters in checkpoint and model are different"
        for p, t in zip(params, tensors):
            p.data = t.data.to(device=p.data.device, dtype=p.data.dtype)
        self.reset()

    def save_checkpoint(self, ckp: Optional[str] = None):
        torch.save([p.detach().cpu().clone() for p in self.ft_params()], ckp or self.save_ckp)

    @torch.no_grad()
    def generate(self, input_ids, max_new_tokens=128, eos_token_id=(2,)):
        """Greedy decoding (spotlight_generation.py:470-495). The new tokens stay on the device until the
        end -- the reference synchronises with ``.item()`` per token (:485-487) -- so an EOS is honoured
        by truncation afterwards; the caches are sized once for prompt + new tokens; the forward pass
        after the last token, whose logits nobody reads, is not run. One host read of the kernels'
        status words at the end turns a device-side wait that ran out into an exception."""
        if input_ids.ndim == 3:
            input_ids = input_ids.flatten(0, 1)
        device = next(iter(self.model.parameters())).device
        input_ids = input_ids.to(device)
        kw = self.model.draft_kwargs
        hint, had = kw.get("max_seq_len"), "max_seq_len" in kw
        if not hint:
            kw["max_seq_len"] = input_ids.shape[1] + max_new_tokens + 1
        try:
            out = self.model(input_ids=input_ids)
            kv_cache = out.past_key_values
            tok = out.logits[:, -1:].argmax(dim=-1)
            new = [tok]
            for _ in range(max_new_tokens - 1):
                out = self.model(input_ids=tok, kv_cache=kv_cache)
                kv_cache = out.past_key_values
                tok = out.logits.argmax(dim=-1).view(-1, 1)
                new.append(tok)
        finally:
            if had:
                kw["max_seq_len"] = hint
            else:
                kw.pop("max_seq_len", None)
        new = torch.cat(new[:max_new_tokens], dim=-1) if max_new_tokens > 0 else input_ids[:, :0]
        if new.shape[0] == 1 and eos_token_id:
            hit = torch.isin(new[0], torch.tensor(list(eos_token_id), device=device)).nonzero()
            if hit.numel():
                new = new[:, : int(hit[0])]
        ops.check_status(device)
        self.model.reset()
        return torch.cat([input_ids, new.to(input_ids.dtype)], dim=-1)
