"""Drop-in for the reference's ``spotlight.modifiers.gpu_cache`` (gpu_cache.py:6-118): per-layer
pre-allocated code cache (``KVHash``) and K/V cache (``KVCache``) with append and top-k gather.

Constructor arguments, attribute names (``key_cache``, ``val_cache``, ``length``) and method
contracts are the reference's. ``gather`` selects with the exact histogram top-k (lowest index
wins a tie; rows come back in ascending key order, the reference's ``topk(sorted=False)`` order
being unspecified) and copies rows with a gather kernel. The decode hot path does not call
``gather``: it hands the index list straight to the sparse attention kernel."""
import torch

from .. import ops

INIT_SEQ_LEN = 1024 * 2048 + 128     # gpu_cache.py:3


class _LayerBuffers:
    """Token-major [B, capacity, KH, D] buffers, one per layer and per name, filled by appends."""

    init_seq_length = INIT_SEQ_LEN

    def _allocate(self, names, batch_size, num_kv_heads, head_dim, num_layers, dtype, device):
        self.num_kv_heads = num_kv_heads
        self.num_layers = num_layers
        self.max_length = self.init_seq_length
        self.length = [0] * num_layers
        self.device = list(device) if device is not None else ["cuda"] * num_layers
        shape = (batch_size, self.max_length, num_kv_heads, head_dim)
        for name in names:
            setattr(self, name, [torch.zeros(shape, dtype=dtype, device=d) for d in self.device])

    def _append(self, layer_idx, **rows):
        first = next(iter(rows.values()))
        lo = self.length[layer_idx]
        hi = lo + first.shape[1]
        if hi > self.max_length:
            raise RuntimeError(f"cache of layer {layer_idx} is full ({hi} > {self.max_length})")
        views = []
        for name, value in rows.items():
            buf = getattr(self, name)[layer_idx]
            buf[:, lo:hi] = value
            views.append(buf[:, :hi])
        self.length[layer_idx] = hi
        return views


class KVHash(_LayerBuffers):
    def __init__(self, batch_size, num_kv_heads, head_dim, num_layers, dtype=torch.bfloat16, device=None):
        self._allocate(("key_cache",), batch_size, num_kv_heads, head_dim, num_layers, dtype, device)

    def update(self, layer_idx, key):
        return self._append(layer_idx, key_cache=key)[0]


def topk_and_gather(attn, keys, vals, budget, max_score=None):
    """int16 scores [B,N,KH] + caches [B,>=N,KH,128] -> two [B,budget,KH,128] tensors
    (gpu_cache.py:48-54). `max_score` = 128 * (query heads per kv head) bounds the scores; given, the
    call enqueues its kernels and returns without a host read. Left out (the reference's signature has
    no such argument), it costs one device-to-host read of the largest score."""
    n = attn.shape[1]
    budget = min(int(budget), n)
    if max_score is None:
        max_score = int(attn.max().item()) if n else 0
    idx, _ = ops.topk_from_scores(attn, budget, int(max_score), sink=0, recent=0)
    return ops.gather_rows(keys[:, :n], idx, budget), ops.gather_rows(vals[:, :n], idx, budget)


class KVCache(_LayerBuffers):
    def __init__(self, batch_size, num_kv_heads, head_dim, num_layers, dtype=torch.bfloat16, device=None, **kwargs):
        self._allocate(("key_cache", "val_cache"), batch_size, num_kv_heads, head_dim, num_layers, dtype, device)

    def update(self, layer_idx, key, val):
        k, v = self._append(layer_idx, key_cache=key, val_cache=val)
        return k, v

    max_score = None     # set to 128 * (query heads per kv head) to keep gather() free of host reads

    def gather(self, layer_idx, attn, budget):
        return topk_and_gather(attn, self.key_cache[layer_idx], self.val_cache[layer_idx], budget, self.max_score)
