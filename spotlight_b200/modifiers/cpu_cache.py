"""Drop-in for the reference's ``spotlight.modifiers.cpu_cache`` (cpu_cache.py:6-130): the K/V caches of
the layers not listed in ``freeze`` live in HOST memory, the code cache and the frozen layers stay on
the GPU.

The reference copies the scores to the host, runs top-k and the row gather there and sends the
gathered rows back (cpu_cache.py:50-57,105-113: a host sync and a CPU gather per layer and token).
Here the host store is PINNED memory that the GPU addresses directly: the scores never leave the
device, the exact top-k runs there, and the gather kernel pulls only the selected 256-byte rows across
PCIe -- no host sync, nothing for the CPU to do. ``update`` writes new rows into the pinned store with
an asynchronous device-to-host copy on the current stream (stream order keeps a later gather behind
it). Wrapping the store in an LRU-resident device buffer (ops.LruTable / sl_lru_update with
``backing_ptrs``) removes the PCIe traffic of rows that were attended recently."""
import torch

from .. import ops
from .gpu_cache import KVHash as _GpuKVHash

INIT_SEQ_LEN = 1024 * 32 + 128       # cpu_cache.py:4


class KVHash(_GpuKVHash):
    init_seq_length = INIT_SEQ_LEN


class KVCache:
    init_seq_length = INIT_SEQ_LEN
    max_score = None     # set to 128 * (query heads per kv head) to keep gather() free of host reads

    def __init__(self, batch_size, num_kv_heads, head_dim, num_layers, dtype=torch.bfloat16, freeze=(0, 1), device=None):
        assert head_dim == 128, "the gather kernel copies 128-value rows"
        self.freeze = list(freeze)
        self.num_kv_heads = num_kv_heads
        self.num_layers = num_layers
        self.max_length = self.init_seq_length
        self.length = [0] * num_layers
        self.device = list(device) if device is not None else ["cuda"] * num_layers
        shape = (batch_size, self.max_length, num_kv_heads, head_dim)

        def alloc(i, dev):
            if i in self.freeze:
                return torch.zeros(shape, dtype=dtype, device=dev)
            return torch.zeros(shape, dtype=dtype).pin_memory()          # host store the GPU can address
        self.key_cache = [alloc(i, d) for i, d in enumerate(self.device)]
        self.val_cache = [alloc(i, d) for i, d in enumerate(self.device)]

    def update(self, layer_idx, key, val):
        lo = self.length[layer_idx]
        hi = lo + key.shape[1]
        if hi > self.max_length:
            raise RuntimeError(f"cache of layer {layer_idx} is full ({hi} > {self.max_length})")
        self.key_cache[layer_idx][:, lo:hi].copy_(key, non_blocking=True)
        self.val_cache[layer_idx][:, lo:hi].copy_(val, non_blocking=True)
        self.length[layer_idx] = hi
        return self.key_cache[layer_idx][:, :hi], self.val_cache[layer_idx][:, :hi]

    def gather(self, layer_idx, attn, budget):
        """int16 scores [B,N,KH] on the device -> two device tensors [B,budget,KH,128] holding the rows of
        the `budget` highest scores (lowest index wins a tie, rows in ascending key order)."""
        n = attn.shape[1]
        budget = min(int(budget), n)
        top = self.max_score if self.max_score is not None else (int(attn.max().item()) if n else 0)
        idx, _ = ops.topk_from_scores(attn, budget, int(top), sink=0, recent=0)
        k, v = self.key_cache[layer_idx], self.val_cache[layer_idx]
        dev = attn.device
        return ops.gather_rows(k[:, :n], idx, budget, device=dev), ops.gather_rows(v[:, :n], idx, budget, device=dev)
