"""Seeded synthetic inputs for the decode-time retrieval path.

Every benchmark configuration of this project is synthetic: keys/values/queries are drawn
from a seeded CPU generator so that the CPU checker and the device path see identical bits.
No public dataset item is used.

Shapes follow the reference's cache layout (spotlight/modifiers/gpu_cache.py:28-36):
token-major with heads interleaved, i.e. K/V are ``[B, N, KH, 128]`` and codes ``[B, N, KH, 4]``.
"""
from __future__ import annotations

import math
from dataclasses import dataclass, field
from typing import Optional, Tuple

import torch

HEAD_DIM = 128


@dataclass(frozen=True)
class PathConfig:
    """One decode-attention workload (names follow the reference's ``draft_kwargs``,
    config/llama3-8b-spotlight-generation.json:2-12, plus the sink/recent window of
    spotlight/modifiers/spotlight_evaluation.py:341-346)."""
    name: str
    batch: int
    q_heads: int
    kv_heads: int
    context: int
    dtype: str = "bf16"            # "bf16" | "fp32" (dtype of q/K/V and hash weights)
    hash: str = "linear"           # "linear" | "mlp"
    mlp_dims: Tuple[int, ...] = (128, 128, 128)
    mlp_residue: bool = True
    mask_out: float = 0.98
    min_remain: int = 20
    sink: int = 4
    recent: int = 64
    rope_theta: float = 10000.0
    layers: int = 1
    seed: int = 1000

    @property
    def group(self) -> int:
        return self.q_heads // self.kv_heads


def budget(n: int, mask_out: float, min_remain: int = 20) -> int:
    """Number of keys kept by top-k; the reference's rule evaluated in Python doubles
    (spotlight/modifiers/spotlight_generation.py:162-164)."""
    num_remain = n - int(n * mask_out)
    return max(min(n, min_remain), num_remain)


# The five benchmark configurations plus the headline shape.
CONFIGS = {
    "cfg0": PathConfig("cfg0", 1, 8, 8, 4096, "fp32", "linear", mask_out=0.9, seed=1000),
    "cfg1": PathConfig("cfg1", 1, 32, 8, 32768, "bf16", "mlp", (128, 256, 128), False, 0.9,
                       rope_theta=500000.0, layers=32, seed=1001),
    "cfg2": PathConfig("cfg2", 8, 32, 32, 16384, "bf16", "linear", mask_out=0.98, seed=1002),
    "cfg3": PathConfig("cfg3", 8, 28, 4, 131072, "bf16", "linear", mask_out=0.98,
                       rope_theta=1000000.0, seed=1003),
    "cfg4": PathConfig("cfg4", 1, 40, 8, 1048576, "bf16", "linear", mask_out=0.98,
                       rope_theta=1000000.0, seed=1004),
    "headline": PathConfig("headline", 1, 32, 8, 131072, "bf16", "mlp", (128, 256, 128), False,
                           0.9, rope_theta=500000.0, layers=32, seed=1001),
}


def torch_dtype(name: str) -> torch.dtype:
    return {"bf16": torch.bfloat16, "fp32": torch.float32, "fp16": torch.float16}[name]


def rope_tables(positions: torch.Tensor, theta: float, dim: int = HEAD_DIM):
    """cos/sin rows for the given positions, HF-Llama convention (frequencies repeated over the
    two halves, matching ``rotate_half`` used by spotlight/modifiers/modify_llama.py:54-59)."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, dim, 2, dtype=torch.float32) / dim))
    freqs = positions.to(torch.float32)[:, None] * inv_freq[None, :]
    emb = torch.cat([freqs, freqs], dim=-1)
    return emb.cos(), emb.sin()


def apply_rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """``x*cos + rotate_half(x)*sin`` over the last dim; cos/sin broadcast against x."""
    half = x.shape[-1] // 2
    rot = torch.cat([-x[..., half:], x[..., :half]], dim=-1)
    return x * cos + rot * sin


@dataclass
class PathInputs:
    q: torch.Tensor            # [B, QH, 128]  post-RoPE query of the decode token
    k: torch.Tensor            # [B, N, KH, 128] post-RoPE keys (cache content)
    v: torch.Tensor            # [B, N, KH, 128]
    hash_q: dict = field(default_factory=dict)   # hash parameters for query heads
    hash_k: dict = field(default_factory=dict)   # hash parameters for key heads
    outlier_channels: Optional[torch.Tensor] = None


def make_hash_params(kind: str, heads: int, dims, gen: torch.Generator, dtype: torch.dtype,
                     mlp_scale: float = 1e-3) -> dict:
    """Random-init hash parameters. ``linear``: W ~ N(0, 1/128) of shape [H,128,128]
    (shape of spotlight/modifiers/linearhashing_generation.py:227). ``mlp``: per layer
    proj ~ N(0,1)*1e-3 [H,in,out] and zero bias [H,out]
    (spotlight/modifiers/spotlight_generation.py:232-234)."""
    if kind == "linear":
        w = torch.randn((heads, HEAD_DIM, HEAD_DIM), generator=gen) / math.sqrt(HEAD_DIM)
        return {"kind": "linear", "w": [w.to(dtype)], "b": [None]}
    ws, bs = [], []
    for i in range(len(dims) - 1):
        ws.append((torch.randn((heads, dims[i], dims[i + 1]), generator=gen) * mlp_scale).to(dtype))
        bs.append(torch.zeros((heads, dims[i + 1]), dtype=dtype))
    return {"kind": "mlp", "w": ws, "b": bs}


def make_inputs(cfg: PathConfig, context: Optional[int] = None, batch: Optional[int] = None,
                seed: Optional[int] = None, mlp_scale: float = 1e-3) -> PathInputs:
    """Draw one layer-step's inputs on the CPU in fp32, then cast to the run dtype.

    K, V ~ N(0,1); four key channels (a seeded permutation's first four) are scaled x8 to mimic
    RoPE outliers; key token 0 is scaled x4 as an attention sink; q ~ N(0,1). RoPE with the
    config's theta is applied to q (position N-1) and K (positions 0..N-1)."""
    n = context if context is not None else cfg.context
    b = batch if batch is not None else cfg.batch
    gen = torch.Generator().manual_seed(cfg.seed if seed is None else seed)
    dt = torch_dtype(cfg.dtype)
    k = torch.randn((b, n, cfg.kv_heads, HEAD_DIM), generator=gen)
    v = torch.randn((b, n, cfg.kv_heads, HEAD_DIM), generator=gen)
    q = torch.randn((b, cfg.q_heads, HEAD_DIM), generator=gen)
    ch = torch.randperm(HEAD_DIM, generator=gen)[:4]
    k[..., ch] *= 8.0
    k[:, 0] *= 4.0
    cos, sin = rope_tables(torch.arange(n), cfg.rope_theta)
    k = apply_rope(k, cos[None, :, None, :], sin[None, :, None, :])
    q = apply_rope(q, cos[n - 1][None, None, :], sin[n - 1][None, None, :])
    hq = make_hash_params(cfg.hash, cfg.q_heads, cfg.mlp_dims, gen, dt, mlp_scale)
    if cfg.q_heads == cfg.kv_heads:
        hk = hq            # MHA: one parameter set, as in the reference modifier
    else:
        hk = make_hash_params(cfg.hash, cfg.kv_heads, cfg.mlp_dims, gen, dt, mlp_scale)
    return PathInputs(q.to(dt), k.to(dt), v.to(dt), hq, hk, ch)


BLOCK_TOKENS = 131072


def make_block(cfg: PathConfig, block: int, tokens: int = BLOCK_TOKENS):
    """Keys/values of one fixed-size block of a long context (config 4): block j is seeded
    ``cfg.seed * 1000 + j`` -- never by rank -- so any number of ranks, and the CPU checker, see
    the same global tensor; a rank materialises only the blocks it owns. Returns post-RoPE
    (k, v) of shape [B, tokens, KH, 128] in the run dtype."""
    gen = torch.Generator().manual_seed(cfg.seed * 1000 + block)
    k = torch.randn((cfg.batch, tokens, cfg.kv_heads, HEAD_DIM), generator=gen)
    v = torch.randn((cfg.batch, tokens, cfg.kv_heads, HEAD_DIM), generator=gen)
    ch = torch.randperm(HEAD_DIM, generator=torch.Generator().manual_seed(cfg.seed))[:4]
    k[..., ch] *= 8.0
    if block == 0:
        k[:, 0] *= 4.0
    pos = torch.arange(block * tokens, (block + 1) * tokens)
    cos, sin = rope_tables(pos, cfg.rope_theta)
    k = apply_rope(k, cos[None, :, None, :], sin[None, :, None, :])
    dt = torch_dtype(cfg.dtype)
    return k.to(dt), v.to(dt)


def ar1_step(k_prev: torch.Tensor, gen: torch.Generator, rho: float = 0.95) -> torch.Tensor:
    """Seeded AR(1) drift of the keys, ``K_t = rho*K_{t-1} + sqrt(1-rho^2)*eps`` (config 2)."""
    eps = torch.randn(k_prev.shape, generator=gen)
    return (rho * k_prev.float() + math.sqrt(1.0 - rho * rho) * eps).to(k_prev.dtype)


def algorithmic_bytes(batch: int, n: int, kv_heads: int, q_heads: int, nsel_total: int) -> dict:
    """Bytes credited to one layer-step: the code stream the scan must read and the K/V rows the
    attention must gather (``nsel_total`` = sum over (b, kv head) of attended-set sizes)."""
    scan = batch * n * kv_heads * 16 + batch * q_heads * 16
    attn = nsel_total * HEAD_DIM * 2 * 2 + batch * q_heads * HEAD_DIM * 2
    return {"scan": scan, "attn": attn}
