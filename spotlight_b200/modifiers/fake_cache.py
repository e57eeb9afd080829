"""Drop-in for the reference's ``spotlight.modifiers.fake_cache`` (fake_cache.py:7-106): the batch-aliasing
backend with which large-batch latency is measured without large-batch memory. Codes and K/V of
batch row 0 are stored once; ``update`` returns views expanded to ``batch_size`` rows (batch stride 0),
which the scan and attention kernels read as they are -- every batch row streams the same cache, so
the timing is that of a real batch whose rows happen to hold equal data (the cache traffic then comes
from L2 after the first row, which is what the reference's version measures too)."""
import torch

from .gpu_cache import INIT_SEQ_LEN, _LayerBuffers

BOUND_SEQ_LEN = INIT_SEQ_LEN


class _Aliased(_LayerBuffers):
    bound_seq_length = BOUND_SEQ_LEN

    def _allocate_aliased(self, names, batch_size, num_kv_heads, head_dim, num_layers, dtype, device):
        self.batch_size = batch_size
        self._allocate(names, 1, num_kv_heads, head_dim, num_layers, dtype, device)

    def _append_aliased(self, layer_idx, **rows):
        views = self._append(layer_idx, **{name: value[:1] for name, value in rows.items()})
        return [v.expand(self.batch_size, -1, -1, -1) for v in views]


class KVHash(_Aliased):
    def __init__(self, batch_size, num_kv_heads, head_dim, num_layers, dtype=torch.bfloat16, device=None):
        self._allocate_aliased(("key_cache",), batch_size, num_kv_heads, head_dim, num_layers, dtype, device)

    def update(self, layer_idx, key):
        return self._append_aliased(layer_idx, key_cache=key)[0]


class KVCache(_Aliased):
    def __init__(self, batch_size, num_kv_heads, head_dim, num_layers, dtype=torch.bfloat16, device=None):
        self._allocate_aliased(("key_cache", "val_cache"), batch_size, num_kv_heads, head_dim, num_layers, dtype, device)

    def update(self, layer_idx, key, val):
        k, v = self._append_aliased(layer_idx, key_cache=key, val_cache=val)
        return k, v
