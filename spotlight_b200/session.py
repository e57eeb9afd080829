"""A decode session over the retrieval path for models whose attention layers share one shape:
per-layer code / K / V caches, per-layer hash parameters, and the three-launch layer step

    decode_prepare -> scan_topk -> sparse_attn_decode

for all layers of one decode token, eagerly or as a replayed CUDA graph, with device-resident
inputs or with pinned host buffers (host->device copy of the token's q/k/v and device->host
copy of the attention outputs inside the step).

This is the host-side counterpart of the reference's per-layer loop
(spotlight/modifiers/spotlight_generation.py:58-79 calling :109-226) with its caches
(spotlight/modifiers/gpu_cache.py) for callers that drive the attention path themselves."""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional

import torch

from . import ops
from ._lib import GQA_BLOCKED
from .workloads import budget


@dataclass
class SessionConfig:
    batch: int
    q_heads: int
    kv_heads: int
    layers: int
    capacity: int                      # tokens per cache row
    dtype: torch.dtype = torch.bfloat16
    mask_out: float = 0.98
    min_remain: int = 20
    sink: int = 4
    recent: int = 64
    layout: int = GQA_BLOCKED
    fix_layers: tuple = ()             # layers that attend to every key
    lru_slots: int = 0                 # > 0: attend over an LRU-resident K/V buffer of this many slots per (row, kv head)
    fused_kv: bool = True              # one cache [B,C,KH,2,128] per layer (a key's K and V rows adjacent) instead of two


class DecodeSession:
    def __init__(self, cfg: SessionConfig, hash_q: List[ops.HashParams], hash_k: List[ops.HashParams],
                 device="cuda"):
        assert len(hash_q) == cfg.layers and len(hash_k) == cfg.layers
        self.cfg, self.device = cfg, torch.device(device)
        B, QH, KH, L, C = cfg.batch, cfg.q_heads, cfg.kv_heads, cfg.layers, cfg.capacity
        dev, dt = self.device, cfg.dtype
        self.hash_q, self.hash_k = hash_q, hash_k
        if cfg.fused_kv:
            # a gathered key is then ONE 512-byte piece of memory: k_cache / v_cache are strided views
            self.kv_cache = [torch.empty((B, C, KH, 2, 128), dtype=dt, device=dev) for _ in range(L)]
            self.k_cache = [kv[:, :, :, 0] for kv in self.kv_cache]
            self.v_cache = [kv[:, :, :, 1] for kv in self.kv_cache]
        else:
            self.kv_cache = None
            self.k_cache = [torch.empty((B, C, KH, 128), dtype=dt, device=dev) for _ in range(L)]
            self.v_cache = [torch.empty((B, C, KH, 128), dtype=dt, device=dev) for _ in range(L)]
        self.codes = [torch.empty((B, C, KH, 4), dtype=torch.uint32, device=dev) for _ in range(L)]
        self.length = 0
        # one token's inputs and outputs for all layers
        self.q_in = torch.zeros((L, B, QH, 128), dtype=dt, device=dev)
        self.k_in = torch.zeros((L, B, KH, 128), dtype=dt, device=dev)
        self.v_in = torch.zeros((L, B, KH, 128), dtype=dt, device=dev)
        self.out = torch.zeros((L, B, QH, 128), dtype=dt, device=dev)
        self.cos = torch.zeros((128,), dtype=dt, device=dev)
        self.sin = torch.zeros((128,), dtype=dt, device=dev)
        self.q_rot = torch.empty((B, QH, 128), dtype=dt, device=dev)
        self.q_codes = torch.empty((B, QH, 4), dtype=torch.uint32, device=dev)
        cap = min(C, budget(C, cfg.mask_out, cfg.min_remain) + cfg.sink + cfg.recent + 1)
        self.idx = torch.empty((B, KH, cap), dtype=torch.int32, device=dev)
        self.cnt = torch.zeros((B, KH), dtype=torch.int32, device=dev)
        # stage 3 (optional): the attended keys are made resident in a per-layer LRU buffer and the
        # attention reads that buffer through the slots the update returns
        self.lru = None
        if cfg.lru_slots > 0:
            self.lru = [ops.LruTable(B, KH, C, cfg.lru_slots, dt, dev, fused=cfg.fused_kv) for _ in range(L)]
            self.slots = torch.empty_like(self.idx)
        self.use_lru = self.lru is not None      # stage 3 can be switched off to time the three-stage step on the same caches
        self._graphs = {}
        self._host = None
        # device-side position: one captured step serves every token (see step_dev)
        self.pos_dev = torch.zeros((1,), dtype=torch.int64, device=dev)
        self.cos_tab = self.sin_tab = None
        self.tab_pos0 = 0

    # ------------------------------------------------------------------ cache filling
    def load_context(self, layer: int, k: torch.Tensor, v: torch.Tensor, start: int = 0, codes: bool = True):
        """Copy post-RoPE keys / values [B,T,KH,128] into the caches at [start, start+T) and build
        their codes with the layer's key hash."""
        T = k.shape[1]
        self.k_cache[layer][:, start:start + T] = k
        self.v_cache[layer][:, start:start + T] = v
        if codes:
            ops.hash_encode(self.k_cache[layer][:, start:start + T], self.hash_k[layer],
                            out=self.codes[layer][:, start:start + T])

    def set_position(self, pos: int, theta: float):
        """RoPE row of the decode position (host-computed, as the reference's tables are)."""
        inv = 1.0 / (theta ** (torch.arange(0, 128, 2, dtype=torch.float32) / 128))
        f = float(pos) * inv
        emb = torch.cat([f, f])
        self.cos.copy_(emb.cos().to(self.cfg.dtype))
        self.sin.copy_(emb.sin().to(self.cfg.dtype))

    def set_position_table(self, pos0: int, count: int, theta: float):
        """RoPE rows of positions [pos0, pos0 + count) on the device, computed as set_position computes
        one row, for decode loops whose position lives in device memory (step_dev)."""
        inv = 1.0 / (theta ** (torch.arange(0, 128, 2, dtype=torch.float32) / 128))
        f = torch.arange(pos0, pos0 + count, dtype=torch.float32)[:, None] * inv[None, :]
        emb = torch.cat([f, f], dim=-1)
        self.cos_tab = emb.cos().to(self.cfg.dtype).to(self.device)
        self.sin_tab = emb.sin().to(self.cfg.dtype).to(self.device)
        self.tab_pos0 = pos0

    # ------------------------------------------------------------------ one token
    def layer_step(self, layer: int, pos: int, stage: Optional[str] = None):
        """The three launches of one layer for the token at position `pos` (its key/value are
        appended at row `pos`; keys 0..pos are scanned). `stage` restricts to one launch."""
        c = self.cfg
        n = pos + 1
        if stage in (None, "prepare"):
            ops.decode_prepare(self.q_in[layer], self.k_in[layer], self.v_in[layer], self.hash_q[layer],
                               self.hash_k[layer], pos, self.codes[layer], self.k_cache[layer], self.v_cache[layer],
                               self.cos, self.sin, q_rot=self.q_rot, q_codes=self.q_codes)
        if stage in (None, "scan"):
            if layer in c.fix_layers:
                raise NotImplementedError("dense layers are served by the attention hook, not the session")
            ops.scan_topk(self.q_codes, self.codes[layer][:, :n], budget(n, c.mask_out, c.min_remain), c.sink,
                          c.recent, c.layout, idx=self.idx, cnt=self.cnt)
        # bf16: the attention launch fetches the rows of the LRU misses itself and fills their slots on the way
        fill = c.dtype == torch.bfloat16 and c.q_heads // c.kv_heads <= 16
        if self.lru is not None and self.use_lru and stage in (None, "lru"):
            ops.lru_update(self.lru[layer], self.idx, self.cnt, self.k_cache[layer][:, :n], self.v_cache[layer][:, :n],
                           slots_out=self.slots, defer_copy=fill)
        if stage in (None, "attn"):
            if self.lru is not None and self.use_lru and fill:
                ops.sparse_attn_decode_fill(self.q_rot, self.lru[layer], self.slots, self.idx, self.cnt,
                                            self.k_cache[layer][:, :n], self.v_cache[layer][:, :n], c.layout, out=self.out[layer])
            elif self.lru is not None and self.use_lru:
                ops.sparse_attn_decode(self.q_rot, self.lru[layer].k, self.lru[layer].v, self.slots, self.cnt, c.layout,
                                       out=self.out[layer])
            else:
                ops.sparse_attn_decode(self.q_rot, self.k_cache[layer][:, :n], self.v_cache[layer][:, :n], self.idx,
                                       self.cnt, c.layout, out=self.out[layer])

    def step(self, pos: int, stage: Optional[str] = None):
        for layer in range(self.cfg.layers):
            self.layer_step(layer, pos, stage)

    def _native_args(self):
        import ctypes as C
        from . import _lib
        c = self.cfg
        assert not c.fix_layers
        if getattr(self, "_native", None) is None:
            self._native = {}
        if self.use_lru not in self._native:
            L = c.layers
            arr = lambda ts: (C.c_void_p * L)(*[t.data_ptr() for t in ts])
            a = _lib.DecodeStepArgs()
            a.B, a.QH, a.KH, a.layers = c.batch, c.q_heads, c.kv_heads, L
            a.dtype, a.gqa_layout = ops._dt(self.q_in), c.layout
            a.sink, a.recent, a.min_remain, a.mask_out = c.sink, c.recent, c.min_remain, c.mask_out
            a.code_batch_stride = self.codes[0].stride(0)
            kv = ops._kv_layout(self.k_cache[0])
            a.kv_batch_stride, a.kv_token_stride, a.kv_head_stride = kv.batch_stride, kv.token_stride, kv.head_stride
            keep = {"q": arr([self.q_in[l] for l in range(L)]), "k": arr([self.k_in[l] for l in range(L)]),
                    "v": arr([self.v_in[l] for l in range(L)]), "codes": arr(self.codes), "kc": arr(self.k_cache),
                    "vc": arr(self.v_cache), "out": arr([self.out[l] for l in range(L)]),
                    "hq": (_lib.HashParamsStruct * L)(*[h.struct for h in self.hash_q]),
                    "hk": (_lib.HashParamsStruct * L)(*[h.struct for h in self.hash_k])}
            a.d_q, a.d_k, a.d_v = keep["q"], keep["k"], keep["v"]
            a.hash_q, a.hash_k = keep["hq"], keep["hk"]
            a.d_code_cache, a.d_k_cache, a.d_v_cache, a.d_out = keep["codes"], keep["kc"], keep["vc"], keep["out"]
            a.d_cos, a.d_sin = self.cos.data_ptr(), self.sin.data_ptr()
            a.d_q_rot, a.d_q_codes = self.q_rot.data_ptr(), self.q_codes.data_ptr()
            a.d_idx, a.idx_capacity, a.d_cnt = self.idx.data_ptr(), self.idx.shape[2], self.cnt.data_ptr()
            shape = (c.batch, c.kv_heads, c.q_heads)
            sw, status = ops.workspaces.get("scan", self.device, _lib.lib.sl_scan_topk_workspace_bytes(
                c.batch, c.capacity, c.kv_heads, c.q_heads), shape)
            aw, _ = ops.workspaces.get("attn", self.device, _lib.lib.sl_sparse_attn_workspace_bytes(
                c.batch, c.kv_heads, c.q_heads), shape)
            a.d_scan_workspace, a.scan_workspace_bytes = sw.data_ptr(), sw.numel()
            a.d_attn_workspace, a.attn_workspace_bytes = aw.data_ptr(), aw.numel()
            a.d_status = status.data_ptr()
            if self.lru is not None and self.use_lru:   # stage 3: the attended keys are made resident, attention reads the resident buffers
                keep["lru"] = (_lib.LruLayer * L)()
                for l, t in enumerate(self.lru):
                    keep["lru"][l].d_k_resident, keep["lru"][l].d_v_resident = t.k.data_ptr(), t.v.data_ptr()
                    keep["lru"][l].d_tok2slot, keep["lru"][l].d_slot2tok = t.tok2slot.data_ptr(), t.slot2tok.data_ptr()
                    keep["lru"][l].d_last_used, keep["lru"][l].d_stats = t.last_used.data_ptr(), t.stats.data_ptr()
                a.lru = keep["lru"]
                a.lru_slots, a.lru_n_max = c.lru_slots, c.capacity
                res = ops._kv_layout(self.lru[0].k)
                a.lru_batch_stride, a.lru_token_stride, a.lru_head_stride = res.batch_stride, res.token_stride, res.head_stride
                a.d_slots = self.slots.data_ptr()
                need = _lib.lib.sl_lru_workspace_bytes(c.batch, c.kv_heads, self.idx.shape[2])
                keep["lru_ws"] = torch.zeros(need, dtype=torch.uint8, device=self.device)
                a.d_lru_workspace, a.lru_workspace_bytes = keep["lru_ws"].data_ptr(), need
            self._native[self.use_lru] = (a, keep, sw, aw, status)
        return self._native[self.use_lru][0]

    def step_native(self, pos: int):
        """`step(pos)` with the layer loop in the library (sl_decode_step): one call per token instead
        of three per layer."""
        import ctypes as C
        from . import _lib
        _lib.check(_lib.lib.sl_decode_step(C.byref(self._native_args()), pos,
                                           torch.cuda.current_stream(self.device).cuda_stream))
        ops.launch_count += (6 if self.use_lru else 4) * self.cfg.layers

    def step_dev(self, max_context: Optional[int] = None, advance: bool = True):
        """One token at the position held in `self.pos_dev` (device memory): the launches depend on no
        host-side position, so a captured graph of this call serves every token of a decode loop
        (capture_dev). Needs set_position_table to cover the positions that will be visited."""
        import ctypes as C
        from . import _lib
        assert self.cos_tab is not None, "call set_position_table first"
        d = _lib.DecodeDev()
        d.d_pos = self.pos_dev.data_ptr()
        d.max_context = int(max_context or self.cfg.capacity)
        d.d_cos_table, d.d_sin_table = self.cos_tab.data_ptr(), self.sin_tab.data_ptr()
        d.table_pos0, d.table_rows = self.tab_pos0, self.cos_tab.shape[0]
        d.advance = int(advance)
        _lib.check(_lib.lib.sl_decode_step_dev(C.byref(self._native_args()), C.byref(d),
                                               torch.cuda.current_stream(self.device).cuda_stream))
        ops.launch_count += (6 if self.use_lru else 4) * self.cfg.layers + int(advance)

    def capture_dev(self, host_io: bool = False, max_context: Optional[int] = None) -> torch.cuda.CUDAGraph:
        """One CUDA graph for every token: step_dev (which advances the device-side position at its end),
        optionally with the pinned-host copies of the token's inputs and outputs around it. The warm-up
        run outside the capture executes one token: set `pos_dev` afterwards."""
        key = ("dev", host_io, max_context, self.use_lru)
        if key in self._graphs:
            return self._graphs[key]
        if host_io:
            self._ensure_host()

        def run():
            if host_io:
                self.q_in.copy_(self._host["q"], non_blocking=True)
                self.k_in.copy_(self._host["k"], non_blocking=True)
                self.v_in.copy_(self._host["v"], non_blocking=True)
            self.step_dev(max_context)
            if host_io:
                self._host["out"].copy_(self.out, non_blocking=True)
                self._host["status"].copy_(self._scan_status(), non_blocking=True)

        saved = self.pos_dev.clone()
        s = torch.cuda.Stream(device=self.device)
        s.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(s):
            run()
        torch.cuda.current_stream(self.device).wait_stream(s)
        torch.cuda.synchronize(self.device)
        self.pos_dev.copy_(saved)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            run()
        self._graphs[key] = g
        return g

    # ------------------------------------------------------------------ graphs
    def capture(self, pos: int, stage: Optional[str] = None, host_io: bool = False) -> torch.cuda.CUDAGraph:
        """Capture `step(pos)` (optionally one stage only, optionally with the pinned-host copies)
        into a CUDA graph; replays reuse the same position and buffers."""
        key = (pos, stage, host_io, self.use_lru)
        if key in self._graphs:
            return self._graphs[key]
        if host_io:
            self._ensure_host()
        s = torch.cuda.Stream(device=self.device)
        s.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(s):
            self._run(pos, stage, host_io)            # warm-up outside capture (workspaces allocate here)
        torch.cuda.current_stream(self.device).wait_stream(s)
        torch.cuda.synchronize(self.device)
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self._run(pos, stage, host_io)
        self._graphs[key] = g
        return g

    def _run(self, pos, stage, host_io):
        if host_io:
            self.q_in.copy_(self._host["q"], non_blocking=True)
            self.k_in.copy_(self._host["k"], non_blocking=True)
            self.v_in.copy_(self._host["v"], non_blocking=True)
        self.step(pos, stage)
        if host_io:
            self._host["out"].copy_(self.out, non_blocking=True)
            self._host["status"].copy_(self._scan_status(), non_blocking=True)   # rides along with the outputs

    def _scan_status(self) -> torch.Tensor:
        """The status word of the scan workspace this session's steps use (set by a bounded wait that ran out)."""
        from . import _lib
        c = self.cfg
        need = _lib.lib.sl_scan_topk_workspace_bytes(c.batch, c.capacity, c.kv_heads, c.q_heads)
        return ops.workspaces.get("scan", self.device, need, (c.batch, c.kv_heads, c.q_heads))[1]

    # ------------------------------------------------------------------ host buffers
    def _ensure_host(self):
        if self._host is None:
            self._host = {
                "q": torch.zeros(self.q_in.shape, dtype=self.cfg.dtype).pin_memory(),
                "k": torch.zeros(self.k_in.shape, dtype=self.cfg.dtype).pin_memory(),
                "v": torch.zeros(self.v_in.shape, dtype=self.cfg.dtype).pin_memory(),
                "out": torch.zeros(self.out.shape, dtype=self.cfg.dtype).pin_memory(),
                "status": torch.zeros((1,), dtype=torch.int32).pin_memory(),
            }
        return self._host

    def step_host(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, pos: int, graph: bool = True) -> torch.Tensor:
        """One token with HOST inputs q [L,B,QH,128], k/v [L,B,KH,128]: stage them in pinned memory,
        copy to the device, run every layer, copy the outputs [L,B,QH,128] back and wait for them."""
        h = self._ensure_host()
        if q is not h["q"]:               # callers that fill host_inputs() in place skip the staging copy
            h["q"].copy_(q)
        if k is not h["k"]:
            h["k"].copy_(k)
        if v is not h["v"]:
            h["v"].copy_(v)
        if graph:
            self.capture(pos, None, True).replay()
        else:
            self._run(pos, None, True)
        torch.cuda.current_stream(self.device).synchronize()
        if int(h["status"][0]) != 0:      # a device-side wait ran out: the step's results are not to be trusted
            ops.check_status(self.device)
        return h["out"]

    def host_inputs(self):
        """The pinned host buffers q [L,B,QH,128], k, v [L,B,KH,128] that step_host copies to the device: a caller
        that writes a token's inputs straight into them and passes them to step_host saves the staging copy."""
        h = self._ensure_host()
        return h["q"], h["k"], h["v"]

    @property
    def host_bytes_per_step(self):
        e = self.q_in.element_size()
        return (self.q_in.numel() + self.k_in.numel() + self.v_in.numel()) * e, self.out.numel() * e + 4   # + the status word
