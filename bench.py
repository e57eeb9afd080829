#!/usr/bin/env python
"""Benchmark of the decode-time retrieval path (hash -> Hamming scan + top-k -> sparse attention).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload NAME]

Metric: decode-attention microseconds per layer at a 128K-token context, Llama-3-8B shape
(32 layers, 32 query / 8 KV heads, head_dim 128, bf16, batch 1, MLP hash 128->256->128, 90 % of
the keys pruned per head, + sink 4 and recent 64). One "step" is one decode token through the
retrieval path of all 32 layers. Data is synthetic and seeded (K,V ~ N(0,1), four outlier key
channels x8, key 0 x4, RoPE theta 5e5), generated on the device; the 17.7 GB of caches exceed
the L2 by two orders of magnitude, so no flush is needed between steps.

One JSON line is printed by rank 0:
  value       device-resident inputs, CUDA-graph replay of the step, CUDA events, max over ranks
  e2e         the same step through DecodeSession.step_host: pinned HOST q/k/v in, outputs back
  roofline    the dominant kernel: algorithmic bytes / its mean launch time / measured HBM peak
  cpu_baseline  the reference modifier's operator sequence (CPU restatement) on the host cores
With --impl reference the CPU restatement itself is the timed arm (rank 0 only)."""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import tempfile
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from spotlight_b200.workloads import CONFIGS, HEAD_DIM, budget, make_hash_params  # noqa: E402

METRIC = "decode_attn_us_per_layer_128k_llama3_8b_shape"
UNIT = "us/layer"
def measured_traffic(cfg, kernel):
    """DRAM bytes per launch (read + written) of `kernel` as one ncu capture measured them, from the small
    tracked table beside the capture summaries; None when no capture covers this workload."""
    path = os.path.join(ROOT, "profiles", "dram_traffic.json")
    try:
        with open(path) as f:
            table = json.load(f)
    except (OSError, ValueError):
        return None
    key = f"{cfg.name}:B{cfg.batch}:N{cfg.context}:{cfg.q_heads}/{cfg.kv_heads}:mask_out={cfg.mask_out}"
    entry = table.get(key, {}).get(kernel)
    return None if entry is None else float(entry["dram_bytes_per_launch"])


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        with open(p) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


class ClockSampler:
    Q = ("index,clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.active,"
         "clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, gpu_index: int):
        self.idx = gpu_index
        self.f = tempfile.NamedTemporaryFile("w+", suffix=".csv", delete=False)
        self.p = None

    def __enter__(self):
        try:
            self.p = subprocess.Popen(["nvidia-smi", f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                       "-lms", "20", "-i", str(self.idx)], stdout=self.f, stderr=subprocess.DEVNULL)
        except OSError:
            self.p = None
        # nvidia-smi needs a few hundred ms to start: wait for its first line so that the samples
        # that follow fall inside the timed region
        t_end = time.time() + 3.0
        while self.p is not None and time.time() < t_end and os.path.getsize(self.f.name) == 0:
            time.sleep(0.02)
        return self

    def __exit__(self, *a):
        if self.p is not None:
            self.p.terminate()
            try:
                self.p.wait(timeout=5)
            except subprocess.TimeoutExpired:
                self.p.kill()

    def summary(self):
        self.f.flush()
        self.f.seek(0)
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for line in self.f.read().splitlines():
            parts = [x.strip() for x in line.split(",")]
            if len(parts) < 9:
                continue
            try:
                sm.append(float(parts[1]))
                mx.append(float(parts[2]))
            except ValueError:
                continue
            for n, v in zip(names, parts[5:9]):
                if v.lower().startswith("active"):
                    reasons.add(n)
        os.unlink(self.f.name)
        if not sm:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": [], "samples": 0}
        return {"sm_mhz": statistics.median(sm), "sm_max_mhz": max(mx), "reasons": sorted(reasons), "samples": len(sm)}


# ------------------------------------------------------------------------------------------
# CPU arm: the reference modifier's operator sequence on the host cores
# ------------------------------------------------------------------------------------------
def cpu_layer_step_factory(cfg, heads: int, n: int, threads: int):
    """Returns f() running ONE layer-step of the reference modifier path
    (oracle.modifier_path_dense) on `heads` of the q heads at context n, fp32."""
    from oracle import spotlight_oracle as O
    torch.set_num_threads(threads)
    g = torch.Generator().manual_seed(cfg.seed)
    k = torch.randn((1, heads, n, HEAD_DIM), generator=g)
    v = torch.randn((1, heads, n, HEAD_DIM), generator=g)
    q = torch.randn((1, heads, 1, HEAD_DIM), generator=g)
    ch = torch.randperm(HEAD_DIM, generator=g)[:4]
    k[..., ch] *= 8.0
    k[:, :, 0] *= 4.0
    params = make_hash_params(cfg.hash, heads, cfg.mlp_dims, g, torch.float32)

    def f():
        with torch.no_grad():
            return O.modifier_path_dense(q, k, v, params, cfg.mask_out, cfg.min_remain, cfg.sink, cfg.recent,
                                         cfg.mlp_residue, cfg.rope_theta)
    return f


def time_cpu(cfg, n: int, steps: int, warmup: int, budget_s: float):
    """(us_per_layer, heads_used, threads, per-step seconds): per-head cost is uniform, so a
    bounded sample runs a subset of the q heads and scales by q_heads / heads."""
    threads = os.cpu_count() or 1
    probe = cpu_layer_step_factory(cfg, 1, n, threads)
    probe()
    t0 = time.perf_counter()
    probe()
    t1 = time.perf_counter() - t0
    total = max(1, steps + warmup)
    heads = int(max(1, min(cfg.q_heads, budget_s / total / max(t1, 1e-6))))
    f = cpu_layer_step_factory(cfg, heads, n, threads)
    for _ in range(warmup):
        f()
    ts = []
    for _ in range(steps):
        t0 = time.perf_counter()
        f()
        ts.append(time.perf_counter() - t0)
    med = statistics.median(ts)
    return med * 1e6 * cfg.q_heads / heads, heads, threads, med


def run_reference(args, cfg):
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    us, heads, threads, sec = time_cpu(cfg, cfg.context, args.steps, args.warmup, budget_s=150.0)
    sample = (f"one layer-step of the reference modifier path (RoPE all keys, hash all keys, sign matmul, topk, "
              f"mask, dense SDPA) at N={cfg.context}, fp32, {heads} of {cfg.q_heads} q heads per step, "
              f"scaled x{cfg.q_heads / heads:g}")
    # One timed step = one call of the restated operator sequence on `heads` query heads (the sample);
    # `value` scales it to all query heads of one layer; a whole token (all layers) is extrapolated apart.
    line = {
        "impl": "reference", "metric": METRIC, "value": us, "unit": UNIT, "n_gpus": args.gpus, "steps": args.steps,
        "warmup": args.warmup, "ms_per_step": sec * 1e3, "higher_is_better": False, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(cfg),
        "cpu_baseline": {"value": us, "unit": UNIT, "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": us, "unit": UNIT, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "extrapolated_ms_per_token_all_layers": us * cfg.layers / 1e3,
        "gpu_launches": 0,
    }
    print(json.dumps(line), flush=True)


def workload_config(cfg):
    shape = "Llama-3-8B-shaped " if (cfg.q_heads, cfg.kv_heads) == (32, 8) else ""
    return {"workload": f"{cfg.name}: {shape}decode attention, batch {cfg.batch}, {cfg.layers} layers, "
                        f"{cfg.q_heads}/{cfg.kv_heads} heads, context {cfg.context}, {cfg.hash} hash {list(cfg.mlp_dims)}, "
                        f"mask_out {cfg.mask_out}, sink {cfg.sink}, recent {cfg.recent}",
            "context": cfg.context, "batch_per_gpu": cfg.batch, "layers": cfg.layers, "mask_out": cfg.mask_out,
            "l2": "inputs larger than L2 (per-layer caches rotate; working set >> 126 MB)"}


# ------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------
PREFILL_CODE_BUILD = None


def build_session(cfg, device, lru=False, extra_capacity=0, fused_kv=True):
    from spotlight_b200 import ops
    from spotlight_b200.session import DecodeSession, SessionConfig
    from spotlight_b200.workloads import apply_rope, rope_tables, torch_dtype
    dt = torch_dtype(cfg.dtype)
    n = cfg.context
    gen = torch.Generator().manual_seed(cfg.seed)
    hq, hk = [], []
    for layer in range(cfg.layers):
        pq = make_hash_params(cfg.hash, cfg.q_heads, cfg.mlp_dims, gen, dt)
        pk = pq if cfg.q_heads == cfg.kv_heads else make_hash_params(cfg.hash, cfg.kv_heads, cfg.mlp_dims, gen, dt)
        hq.append(ops.HashParams.from_dict(pq, device, cfg.mlp_residue))
        hk.append(ops.HashParams.from_dict(pk, device, cfg.mlp_residue))
    lru_slots = 2 * (budget(n, cfg.mask_out, cfg.min_remain) + cfg.sink + cfg.recent) if lru else 0
    scfg = SessionConfig(cfg.batch, cfg.q_heads, cfg.kv_heads, cfg.layers, n + extra_capacity, dt, cfg.mask_out,
                         cfg.min_remain, cfg.sink, cfg.recent, lru_slots=lru_slots, fused_kv=fused_kv)
    s = DecodeSession(scfg, hq, hk, device)
    dgen = torch.Generator(device=device).manual_seed(cfg.seed)
    ch = torch.randperm(HEAD_DIM, generator=gen)[:4].to(device)
    chunk = 16384
    t_codes = 0.0
    t_layers = []
    for layer in range(cfg.layers):
        for lo in range(0, n, chunk):
            hi = min(n, lo + chunk)
            k = torch.randn((cfg.batch, hi - lo, cfg.kv_heads, HEAD_DIM), generator=dgen, device=device)
            v = torch.randn((cfg.batch, hi - lo, cfg.kv_heads, HEAD_DIM), generator=dgen, device=device)
            k[..., ch] *= 8.0
            if lo == 0:
                k[:, 0] *= 4.0
            cos, sin = rope_tables(torch.arange(lo, hi), cfg.rope_theta)
            k = apply_rope(k, cos.to(device)[None, :, None, :], sin.to(device)[None, :, None, :])
            s.load_context(layer, k.to(dt), v.to(dt), lo, codes=False)
        torch.cuda.synchronize(device)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        ops.hash_encode(s.k_cache[layer][:, :n], s.hash_k[layer], out=s.codes[layer][:, :n])
        e1.record()
        torch.cuda.synchronize(device)
        t_codes += e0.elapsed_time(e1)
        t_layers.append(e0.elapsed_time(e1))
    s.q_in.copy_(torch.randn(s.q_in.shape, generator=dgen, device=device).to(dt))
    s.k_in.copy_(torch.randn(s.k_in.shape, generator=dgen, device=device).to(dt))
    s.v_in.copy_(torch.randn(s.v_in.shape, generator=dgen, device=device).to(dt))
    s.set_position(n - 1, cfg.rope_theta)
    # the prefill contraction: all keys of a layer through the key-side hash (the first layer also pays one-time set-up)
    warm = t_layers[1:] if len(t_layers) > 1 else t_layers
    dims = cfg.mlp_dims if cfg.hash == "mlp" else (HEAD_DIM, HEAD_DIM)
    rows = cfg.batch * n * cfg.kv_heads
    flop = rows * sum(2.0 * a * b for a, b in zip(dims[:-1], dims[1:]))
    ms = sum(warm) / len(warm)
    global PREFILL_CODE_BUILD
    PREFILL_CODE_BUILD = {"ms_per_layer": ms, "rows_per_layer": rows, "tflops": flop / ms / 1e9,
                          "gbs": rows * (HEAD_DIM * s.k_cache[0].element_size() + 16) / ms / 1e6,
                          "kernel": "tcgen05 (TMEM accumulators, TMA input tiles)" if (tuple(dims) in ((128, 256, 128), (128, 128)) and rows >= 32768
                                     and dt == torch.bfloat16 and not (cfg.hash == "mlp" and cfg.mlp_residue)) else "warp-level mma / scalar"}
    return s, t_codes / cfg.layers


def time_four_stage(args, cfg, s, device, dist, tokens, drift=0.25, with_lru=True):
    """The four-stage layer-step (hash -> scan + top-k -> LRU update -> attention over the resident buffers) as ONE
    graph replayed for consecutive tokens: the position, and with it the clock of the LRU tables, lives in device
    memory and advances with every replay; the query drifts from token to token (a fixed query plus fresh noise), so
    the selections overlap partially and the update sees hits AND misses. Returns us per layer (max over ranks) and
    what the tables saw at the last token."""
    was = s.use_lru
    s.use_lru = with_lru
    n, L = cfg.context, cfg.layers
    s.set_position_table(n - 1, s.cfg.capacity - (n - 1), cfg.rope_theta)
    s.pos_dev.fill_(n - 1)
    graph = s.capture_dev()
    for t in s.lru:
        t.tok2slot.fill_(-1); t.slot2tok.fill_(-1); t.last_used.fill_(-1)
    s.pos_dev.fill_(n - 1)
    g = torch.Generator(device=device).manual_seed(cfg.seed + 11)
    base = s.q_in.clone().float()
    qsets = [(base + drift * torch.randn(base.shape, generator=g, device=device)).to(s.cfg.dtype) for _ in range(8)]

    def token(i):
        s.q_in.copy_(qsets[i % len(qsets)], non_blocking=True)
        graph.replay()

    for i in range(args.warmup):
        token(i)
    torch.cuda.synchronize(device)
    if dist is not None:
        dist.barrier()
        torch.cuda.synchronize(device)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(args.steps):
        token(args.warmup + i)
    e1.record()
    torch.cuda.synchronize(device)
    ms = e0.elapsed_time(e1) / args.steps
    if dist is not None:
        t = torch.tensor([ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
    stats = torch.stack([t.stats.sum((0, 1)) for t in s.lru]).double().mean(0).tolist()     # last token, mean over layers
    bad = sum(int(t.status.item()) != 0 for t in s.lru)
    s.use_lru = was
    hits, misses = stats
    if not with_lru:        # the same graph (device-side position, drifting query) without stage 3: what the stage adds is the difference
        return {"value_without_lru_same_graph": ms * 1e3 / L, "unit": UNIT, "tokens_timed": args.steps, "query_drift": drift}
    return {"value_with_lru": ms * 1e3 / L, "unit": UNIT, "tokens_timed": args.steps, "query_drift": drift,
            "hit_rate_last_token": hits / max(1.0, hits + misses), "missed_rows_per_layer": misses,
            "miss_bytes_per_layer": misses * HEAD_DIM * 2 * 2, "lru_slots_per_head": s.cfg.lru_slots,
            "status_words_ok": bad == 0,
            "note": "one CUDA graph for every token (device-side position and LRU clock); the query drifts, so the tables see hits and misses"}


def _leave_together(device, dist):
    """Meet the other ranks once more and exit without the group's teardown; a rank that cannot be met (it fell out
    of an exchange measurement) is not waited for longer than a few seconds: the numbers are out by now."""
    import threading
    threading.Timer(20.0, lambda: os._exit(0)).start()
    try:
        torch.cuda.synchronize(device)
        dist.barrier()
    except Exception:
        pass
    os._exit(0)


def time_graph(g, steps, warmup, device, dist=None):
    for _ in range(warmup):
        g.replay()
    torch.cuda.synchronize(device)
    if dist is not None:
        dist.barrier()
        torch.cuda.synchronize(device)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for _ in range(steps):
        g.replay()
    e1.record()
    torch.cuda.synchronize(device)
    if dist is not None:
        dist.barrier()
    return e0.elapsed_time(e1) / steps          # ms per replay


def run_ours(args, cfg):
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the retrieval path has no CPU fallback")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    dist = None
    if world > 1:
        import torch.distributed as dist_
        dist_.init_process_group("nccl", device_id=device)
        dist = dist_
    from spotlight_b200 import ops

    if args.attn_warps:
        from spotlight_b200 import _lib
        _lib.check(_lib.lib.sl_configure(_lib.SL_OPT_ATTN_WARPS, args.attn_warps))
    if args.no_attn_cluster:
        from spotlight_b200 import _lib
        ops.configure(_lib.SL_OPT_ATTN_CLUSTER, 0)
    with_lru = not args.no_lru and cfg.name in ("headline", "cfg1", "cfg2")
    lru_tokens = args.warmup + args.steps + 8
    s, code_build_ms = build_session(cfg, device, lru=with_lru, fused_kv=not args.separate_kv,
                                     extra_capacity=lru_tokens + 8 if with_lru else 0)
    s.use_lru = bool(args.lru) and with_lru
    n, L = cfg.context, cfg.layers
    pos = n - 1

    # one eager pass: attended-set sizes per layer (for the algorithmic byte count)
    nsel = []
    for layer in range(L):
        s.layer_step(layer, pos)
        nsel.append(int(s.cnt.sum().item()))
    ops.check_status(device)
    mean_nsel = sum(nsel) / L

    use_graph = not args.no_graph
    launches0 = ops.launch_count
    try:
        g_all = s.capture(pos) if use_graph else None
    except RuntimeError as e:                    # capture unsupported: fall back to eager launches
        print(f"# graph capture failed ({e}); timing eager launches", file=sys.stderr)
        use_graph, g_all = False, None

    class Eager:
        def __init__(self, stage=None, host=False):
            self.stage, self.host = stage, host

        def replay(self):
            s._run(pos, self.stage, self.host)

    with ClockSampler(local) as clocks:
        ms_step = time_graph(g_all if use_graph else Eager(), args.steps, args.warmup, device, dist)
        stage_ms = {}
        for stage in ("prepare", "scan", "attn") + (("lru",) if s.use_lru else ()):
            g = s.capture(pos, stage) if use_graph else Eager(stage)
            stage_ms[stage] = time_graph(g, max(3, args.steps // 2), 3, device) / L
        # end to end: pinned host inputs in, outputs back, one host sync per token
        hq, hk, hv = s.host_inputs()                 # the token's inputs are produced straight in pinned host memory
        hq.copy_(torch.randn(s.q_in.shape).to(s.cfg.dtype))
        hk.copy_(torch.randn(s.k_in.shape).to(s.cfg.dtype))
        hv.copy_(torch.randn(s.v_in.shape).to(s.cfg.dtype))
        for _ in range(max(3, args.warmup)):
            s.step_host(hq, hk, hv, pos, graph=use_graph)
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize(device)
        t0 = time.perf_counter()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for _ in range(args.steps):
            out_host = s.step_host(hq, hk, hv, pos, graph=use_graph)
        e1.record()
        torch.cuda.synchronize(device)
        ms_e2e = e0.elapsed_time(e1) / args.steps
        wall_e2e = (time.perf_counter() - t0) * 1e3 / args.steps
        lru_info = None
        if with_lru:
            # two regimes: a slowly and a quickly drifting query (noise of 0.05 / 0.25 of a unit-variance query per token)
            lru_info = [time_four_stage(args, cfg, s, device, dist, lru_tokens, drift) for drift in (0.05, 0.25)]
            lru_info.append(time_four_stage(args, cfg, s, device, dist, lru_tokens, 0.25, with_lru=False))
    ops.check_status(device)
    clk = clocks.summary()
    hash_weight_bytes = sum(w.numel() * w.element_size() for w in s.hash_q[0].weights + s.hash_k[0].weights)
    host_bytes = s.host_bytes_per_step
    lru_slots = s.cfg.lru_slots

    if dist is not None:
        t = torch.tensor([ms_step, ms_e2e, wall_e2e], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_step, ms_e2e, wall_e2e = t.tolist()
    checksum = float(out_host.float().abs().sum())
    us_layer = ms_step * 1e3 / L
    peak, peak_kind = peaks()
    by_scan = cfg.batch * n * cfg.kv_heads * 16 + cfg.batch * cfg.q_heads * 16
    by_attn = mean_nsel * HEAD_DIM * 2 * 2 + cfg.batch * cfg.q_heads * HEAD_DIM * 2
    wbytes = hash_weight_bytes
    kern = {
        "scan_topk": {"bytes": by_scan, "us": stage_ms["scan"] * 1e3},
        "sparse_attn": {"bytes": by_attn, "us": stage_ms["attn"] * 1e3},
        "decode_prepare": {"bytes": wbytes, "us": stage_ms["prepare"] * 1e3},
    }
    if "lru" in stage_ms:     # stage 3 replayed at one position: every attended key is resident, only the tables are walked
        kern["lru_update"] = {"bytes": cfg.batch * cfg.kv_heads * lru_slots * 8, "us": stage_ms["lru"] * 1e3}
    for k_, d in kern.items():
        d["gbs"] = d["bytes"] / (d["us"] * 1e-6) / 1e9
        d["frac"] = d["gbs"] / peak
    dom = max(("scan_topk", "sparse_attn"), key=lambda k_: kern[k_]["us"])
    path_gbs = (by_scan + by_attn) / (us_layer * 1e-6) / 1e9
    line = {
        "metric": METRIC, "value": us_layer, "unit": UNIT, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": ms_step, "higher_is_better": False, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic", "config": workload_config(cfg),
        "tokens_per_s": world * cfg.batch / (ms_step * 1e-3),
        "e2e": {"value": max(ms_e2e, wall_e2e) * 1e3 / L, "unit": UNIT,
                "h2d_bytes_per_step": host_bytes[0], "d2h_bytes_per_step": host_bytes[1],
                "device_ms_per_step": ms_e2e, "wall_ms_per_step": wall_e2e},
        # per layer: decode_prepare, scan, attention, its merge kernel (+ the LRU table update when stage 3 runs; the
        # attention launch then fetches and fills the missed rows itself)
        "gpu_launches": (5 if args.lru and with_lru else 4) * L * args.steps,
        "lru_stage": bool(args.lru and with_lru),
        "cuda_graph": use_graph,
        "roofline": {"bound": "hbm", "kernel": dom, "achieved": kern[dom]["gbs"], "peak": peak, "unit": "GB/s",
                     "frac": kern[dom]["frac"], "traffic": measured_traffic(cfg, dom), "peak_kind": peak_kind,
                     "algorithmic_bytes_per_launch": kern[dom]["bytes"], "us_per_launch": kern[dom]["us"],
                     "frac_of_nominal_8TBs": kern[dom]["gbs"] / 8000.0},
        "kernels": kern,
        "path": {"algorithmic_bytes_per_layer": by_scan + by_attn, "gbs": path_gbs, "frac": path_gbs / peak,
                 "attended_keys_per_head": mean_nsel / (cfg.batch * cfg.kv_heads), "budget_k": budget(n, cfg.mask_out, cfg.min_remain)},
        "code_build_ms_per_layer": code_build_ms,
        "prefill_code_build": PREFILL_CODE_BUILD,
        "clocks": clk,
        "checksum": checksum,
    }
    if lru_info is not None:
        line["four_stage"] = lru_info
    # With several ranks the measurements that exchange data between them come last, under a watchdog: if they stall
    # (a rank that fell out, an exchange that waits), every rank gives up on them and rank 0 still prints the line.
    if dist is not None and cfg.name == "headline" and not args.no_extras:
        import threading
        done = threading.Event()
        limit = float(os.environ.get("SL_BENCH_EXTRAS_TIMEOUT_S", "360"))

        def watchdog():
            if done.wait(limit):
                return
            if rank == 0:
                line["multi_rank_extras_error"] = f"gave up after {limit:.0f} s"
                print(json.dumps(line), flush=True)
            os._exit(0)

        threading.Thread(target=watchdog, daemon=True).start()
        g_all = g = None
        del s
        torch.cuda.empty_cache()
        try:
            extras = multi_rank_extras(args, device, dist, world, rank)
        except Exception as e:
            extras = {"multi_rank_extras_error": str(e)[:300]}
        done.set()
        s = None
        line.update(extras)
    if rank != 0:
        if dist is not None:
            _leave_together(device, dist)
        return
    if world == 1 and not args.no_reference_kernels and cfg.name == "headline":
        try:
            line["row_gather"] = row_gather(cfg, s, device)
        except Exception as e:                       # a measurement beside the headline, never a reason to lose the line
            line["row_gather"] = {"error": str(e)[:200]}
        g_all = g = None
        del s
        torch.cuda.empty_cache()
        line["reference_gpu_kernels"] = reference_gpu_kernels(device)
        try:
            line["host_backing_store"] = host_backing_store(cfg, device)
        except Exception as e:
            line["host_backing_store"] = {"error": str(e)[:200]}
    if world == 1 and not args.no_cpu_baseline:
        us, heads, threads, sec = time_cpu(cfg, n, steps=2, warmup=1, budget_s=25.0)
        line["cpu_baseline"] = {
            "value": us, "unit": UNIT, "cores": threads, "kind": "port",
            "sample": f"one layer-step of the reference modifier path at N={n}, fp32, {heads} of {cfg.q_heads} q heads, "
                      f"scaled x{cfg.q_heads / heads:g}; median of 2 after 1 warm-up ({sec:.2f} s each)"}
    print(json.dumps(line), flush=True)
    if dist is not None:      # captured graphs may hold communicator work: leave without the group's teardown
        sys.stdout.flush()
        _leave_together(device, dist)


def run_decode_loop(args, cfg):
    """Config 1 as the reference runs it: a prefilled context, then `--decode-steps` consecutive decode
    tokens, each appended at the next position (the scan grows by one key per token). Launches are
    issued eagerly, one position after the other (positions are host arguments of the C ABI, so
    every token needs its own launches); the time is the device time of the whole loop."""
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the retrieval path has no CPU fallback")
    device = torch.device("cuda", int(os.environ.get("LOCAL_RANK", "0")))
    torch.cuda.set_device(device)
    from spotlight_b200 import ops
    T = args.decode_steps
    s, code_build_ms = build_session(cfg, device, extra_capacity=T + 1)
    n0, L = cfg.context, cfg.layers
    dt = s.cfg.dtype
    g = torch.Generator(device=device).manual_seed(cfg.seed + 7)
    for t in range(3):                                  # warm-up tokens (they stay in the cache)
        s.set_position(n0 + t, cfg.rope_theta)
        s.step(n0 + t)
    torch.cuda.synchronize(device)
    launches0 = ops.launch_count
    with ClockSampler(device.index or 0) as clocks:
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t_wall = time.perf_counter()
        e0.record()
        for t in range(3, T):
            pos = n0 + t
            s.q_in.copy_(torch.randn(s.q_in.shape, generator=g, device=device).to(dt))   # this token's q/k/v
            s.k_in.copy_(torch.randn(s.k_in.shape, generator=g, device=device).to(dt))
            s.v_in.copy_(torch.randn(s.v_in.shape, generator=g, device=device).to(dt))
            s.set_position(pos, cfg.rope_theta)
            if args.python_loop:
                s.step(pos)
            else:
                s.step_native(pos)
        e1.record()
        torch.cuda.synchronize(device)
        wall_ms = (time.perf_counter() - t_wall) * 1e3
    ops.check_status(device)
    ms = e0.elapsed_time(e1)
    tokens = T - 3
    line = {
        "metric": "decode_loop_us_per_layer", "value": ms * 1e3 / tokens / L, "unit": UNIT, "n_gpus": 1,
        "steps": tokens, "warmup": 3, "ms_per_step": ms / tokens, "higher_is_better": False, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": dict(workload_config(cfg), decode_steps=tokens, first_position=n0 + 3,
                       launches="eager, one position per token, layer loop in " + ("Python" if args.python_loop else "the library (sl_decode_step)")),
        "tokens_per_s": cfg.batch * tokens / (ms * 1e-3), "wall_ms_per_step": wall_ms / tokens,
        "gpu_launches": ops.launch_count - launches0, "cuda_graph": False,
        "code_build_ms_per_layer": code_build_ms, "clocks": clocks.summary(),
        "checksum": float(s.out.float().abs().sum()),
    }
    print(json.dumps(line), flush=True)


def sharded_setup(cfg, device, world, rank, L):
    """Per-rank inputs of the sequence-sharded layer-step: this rank's contiguous share of the keys of L
    rotating layers (working set >> L2) and the query, which is the same on every rank."""
    from spotlight_b200.sharded import shard_bounds
    from spotlight_b200.workloads import torch_dtype
    dt = torch_dtype(cfg.dtype)
    n, B, QH, KH = cfg.context, cfg.batch, cfg.q_heads, cfg.kv_heads
    lo, hi = shard_bounds(n, world, rank)
    nl = hi - lo
    g = torch.Generator(device=device).manual_seed(cfg.seed + rank)
    codes, ks, vs = [], [], []
    for _ in range(L):
        codes.append(torch.randint(0, 2 ** 31, (B, nl, KH, 4), generator=g, device=device, dtype=torch.int64).to(torch.uint32))
        ks.append(torch.randn((B, nl, KH, HEAD_DIM), generator=g, device=device).to(dt))
        vs.append(torch.randn((B, nl, KH, HEAD_DIM), generator=g, device=device).to(dt))
    gq = torch.Generator().manual_seed(cfg.seed)
    q_rot = torch.randn((B, QH, HEAD_DIM), generator=gq).to(dt).to(device)
    q_codes = torch.randint(0, 2 ** 31, (B, QH, 4), generator=gq, dtype=torch.int64).to(torch.uint32).to(device)
    return dict(codes=codes, ks=ks, vs=vs, q_rot=q_rot, q_codes=q_codes, lo=lo, nl=nl, L=L)


def sharded_time(args, cfg, data, device, dist, world, exchange, steps, warmup):
    """us per layer of the sharded layer-step (one CUDA graph over the L rotating layers), max over ranks.
    `exchange`: None = NCCL all-gathers, else the peer-memory exchange objects."""
    from spotlight_b200 import ops
    from spotlight_b200.sharded import sharded_decode_attention
    n = cfg.context
    kb = budget(n, cfg.mask_out, cfg.min_remain)
    L = data["L"]

    def layer_step(layer):
        if world > 1:
            return sharded_decode_attention(data["q_rot"], data["q_codes"], data["codes"][layer], data["ks"][layer],
                                            data["vs"][layer], data["lo"], n, kb, cfg.sink, cfg.recent, ops.GQA_BLOCKED,
                                            exchange=exchange)
        idx, cnt = ops.scan_topk(data["q_codes"], data["codes"][layer], kb, cfg.sink, cfg.recent, ops.GQA_BLOCKED)
        return ops.sparse_attn_decode(data["q_rot"], data["ks"][layer], data["vs"][layer], idx, cnt, ops.GQA_BLOCKED)

    def step():
        out = None
        for layer in range(L):
            out = layer_step(layer)
        return out

    use_graph = not args.no_graph
    graph = None
    for _ in range(2):
        step()
    torch.cuda.synchronize(device)
    if use_graph:
        try:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                step()
        except RuntimeError as e:
            print(f"# graph capture failed ({e}); timing eager launches", file=sys.stderr)
            graph, use_graph = None, False
            torch.cuda.synchronize(device)

    class Runner:
        def replay(self):
            if graph is not None:
                graph.replay()
            else:
                step()

    ms_step = time_graph(Runner(), steps, warmup, device, dist if world > 1 else None)
    ops.check_status(device)
    status_ok = True
    if exchange:
        for e in exchange:
            try:
                e.check_status()
            except RuntimeError:
                status_ok = False
    if world > 1:
        t = torch.tensor([ms_step, 0.0 if status_ok else 1.0], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms_step, bad = t.tolist()
        status_ok = bad == 0.0
    del graph
    torch.cuda.synchronize(device)
    return ms_step * 1e3 / L, use_graph, status_ok


def run_sharded(args, cfg):
    """Sequence-sharded layer-step (config 4: 1M-token context): every rank owns n/world keys of
    `layers` rotating layers, a step is one layer-step through sharded_decode_attention (local scan +
    histogram, all-gather, emission, local attention, all-gather of (o, lse), merge). Launched under
    torchrun; with one rank it times the unsharded kernels on the same global shape."""
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the retrieval path has no CPU fallback")
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    import torch.distributed as dist
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    n, B, QH, KH = cfg.context, cfg.batch, cfg.q_heads, cfg.kv_heads
    L = max(2, min(args.layers or 4, 8))                       # rotating layers: working set >> L2
    data = sharded_setup(cfg, device, world, rank, L)
    kb = budget(n, cfg.mask_out, cfg.min_remain)
    exchange = None
    if world > 1 and args.peer:
        from spotlight_b200.sharded import make_peer_exchange
        exchange = make_peer_exchange(B, KH, QH, device, fused_scan=not args.no_fused_scan)
    with ClockSampler(local) as clocks:
        us_layer, use_graph, status_ok = sharded_time(args, cfg, data, device, dist, world, exchange, args.steps, args.warmup)
    clk = clocks.summary()
    if rank == 0:
        peak, peak_kind = peaks()
        by = B * n * KH * 16 + kb * B * KH * HEAD_DIM * 2 * 2            # codes + attended K/V rows, whole job
        line = {
            "metric": "decode_attn_us_per_layer_seq_sharded", "value": us_layer, "unit": UNIT, "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": us_layer * L / 1e3, "higher_is_better": False,
            "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": f"{cfg.name}: sequence-sharded decode attention, batch {B}, {QH}/{KH} heads, context {n} "
                                   f"over {world} rank(s), mask_out {cfg.mask_out}, sink {cfg.sink}, recent {cfg.recent}",
                       "context": n, "keys_per_rank": data["nl"], "rotating_layers": L,
                       "exchange": ("peer memory, fused scan" if exchange and len(exchange) > 2 else "peer memory") if exchange
                       else ("nccl" if world > 1 else "none"),
                       "l2": "inputs larger than L2 (layers rotate)"},
            "tokens_per_s": B / (us_layer * 1e-6 * 48) if cfg.name == "cfg4" else None,
            "cuda_graph": use_graph, "status_words_ok": status_ok,
            "path": {"algorithmic_bytes_per_layer": by, "gbs": by / (us_layer * 1e-6) / 1e9,
                     "frac_of_aggregate_peak": by / (us_layer * 1e-6) / 1e9 / (peak * world), "peak_kind": peak_kind},
            "clocks": clk,
        }
        print(json.dumps(line), flush=True)
    # A captured graph holds NCCL work: leave without the group's teardown (a hang there would only cost
    # time, the numbers are out).
    torch.cuda.synchronize(device)
    if world > 1:
        dist.barrier()
        torch.cuda.synchronize(device)
        sys.stdout.flush()
        os._exit(0)


def multi_rank_extras(args, device, dist, world, rank):
    """What the ranks of one node measure beyond the replicated headline step (rank 0 prints them inside the
    one JSON line): config 4's sequence-sharded layer-step in both forms of the exchange (strong scaling of a
    1M-token context: the path's only step that communicates), and config 3's batch of 8 split over the ranks
    (strong scaling without communication)."""
    import dataclasses
    from spotlight_b200.sharded import make_peer_exchange
    peak, _ = peaks()
    out = {}
    # ---- config 4, sequence shards
    cfg4 = CONFIGS["cfg4"]
    L = 4
    data = sharded_setup(cfg4, device, world, rank, L)
    kb = budget(cfg4.context, cfg4.mask_out, cfg4.min_remain)
    by = cfg4.batch * cfg4.context * cfg4.kv_heads * 16 + kb * cfg4.batch * cfg4.kv_heads * HEAD_DIM * 2 * 2
    seq = {"workload": f"cfg4: batch 1, {cfg4.q_heads}/{cfg4.kv_heads} heads, context {cfg4.context} over {world} ranks, "
                       f"mask_out {cfg4.mask_out}", "ranks": world, "keys_per_rank": data["nl"], "rotating_layers": L,
           "algorithmic_bytes_per_layer": by}
    us, graph, ok = sharded_time(args, cfg4, data, device, dist, world, None, 20, 5)
    seq["nccl"] = {"us_per_layer": us, "frac_of_aggregate_peak": by / (us * 1e-6) / 1e9 / (peak * world), "cuda_graph": graph}
    try:
        ex = make_peer_exchange(cfg4.batch, cfg4.kv_heads, cfg4.q_heads, device, fused_scan=True)
        us, graph, ok = sharded_time(args, cfg4, data, device, dist, world, ex, 20, 5)
        seq["peer_memory_fused_scan"] = {"us_per_layer": us, "frac_of_aggregate_peak": by / (us * 1e-6) / 1e9 / (peak * world),
                                         "cuda_graph": graph, "status_words_ok": ok}
    except Exception as e:        # peer mappings need the GPUs of one node with peer access
        seq["peer_memory_fused_scan"] = {"unavailable": str(e)[:200]}
    out["seq_sharded"] = seq
    del data
    torch.cuda.empty_cache()
    # ---- config 3, batch split (strong scaling, no exchange)
    cfg3 = CONFIGS["cfg3"]
    if cfg3.batch % world == 0:
        c3 = dataclasses.replace(cfg3, batch=cfg3.batch // world, layers=4)
        s3, _ = build_session(c3, device)
        g3 = s3.capture(c3.context - 1)
        ms = time_graph(g3, 20, 5, device, dist)
        t = torch.tensor([ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        out["cfg3_batch_split"] = {"workload": f"cfg3: batch {cfg3.batch} split over {world} ranks ({c3.batch} rows each), "
                                               f"{cfg3.q_heads}/{cfg3.kv_heads} heads, context {cfg3.context}, mask_out {cfg3.mask_out}",
                                   "us_per_layer": float(t.item()) * 1e3 / c3.layers, "scaling": "strong", "collectives": 0}
        del s3, g3
        torch.cuda.empty_cache()
    return out


def row_gather(cfg, s, device, steps=10):
    """The reference's gather step on the attended keys' index lists: sl_gather_rows (KVCache.gather of
    spotlight/modifiers/gpu_cache.py:51-54) copies the selected 256-byte rows of ONE dense [B, N, KH, 128] cache into a
    packed buffer; three caches of the layer's size rotate, so the rows come from HBM. The sparse attention kernel
    reads the same rows of K and of V without writing them anywhere: twice the gathered bytes in about the same time."""
    from spotlight_b200 import ops
    n = cfg.context
    caches = [torch.randn((cfg.batch, n, cfg.kv_heads, HEAD_DIM), device=device).to(s.cfg.dtype) for _ in range(3)]
    nsel = int(s.cnt.min().item())
    rows = cfg.batch * cfg.kv_heads * nsel
    for c in caches:
        ops.gather_rows(c, s.idx, nsel)
    torch.cuda.synchronize(device)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    for i in range(steps * 3):
        ops.gather_rows(caches[i % 3], s.idx, nsel)
    e1.record()
    torch.cuda.synchronize(device)
    us = e0.elapsed_time(e1) * 1e3 / (steps * 3)
    row_bytes = HEAD_DIM * caches[0].element_size()
    return {"kernel": "sl_gather_rows", "rows_per_launch": rows, "us_per_launch": us,
            "read_gbs": rows * row_bytes / us / 1e3, "read_plus_write_gbs": 2 * rows * row_bytes / us / 1e3}


def host_backing_store(cfg, device, steps=8, churn=0.1):
    """Stage 3 with the backing K/V store in pinned HOST memory (the offloaded variant of the reference,
    spotlight/modifiers/cpu_cache.py:60-130): one layer of the workload's shape; every step a tenth of each head's
    attended keys is replaced by new ones, which sl_lru_update pulls across PCIe into the resident buffer. Reports
    the time of the update and the rate of the missed rows (K and V, 512 bytes per miss)."""
    from spotlight_b200 import ops
    from spotlight_b200.workloads import torch_dtype
    dt = torch_dtype(cfg.dtype)
    B, KH, n = cfg.batch, cfg.kv_heads, cfg.context
    nsel = budget(n, cfg.mask_out, cfg.min_remain) + cfg.sink + cfg.recent
    k_host = torch.empty((B, n, KH, HEAD_DIM), dtype=dt).pin_memory()
    v_host = torch.empty((B, n, KH, HEAD_DIM), dtype=dt).pin_memory()
    k_host.normal_(); v_host.normal_()
    table = ops.LruTable(B, KH, n, 2 * nsel, dt, device)
    g = torch.Generator(device=device).manual_seed(cfg.seed + 11)
    cur = torch.stack([torch.randperm(n, generator=g, device=device)[:nsel] for _ in range(B * KH)]).view(B, KH, nsel)
    cnt = torch.full((B, KH), nsel, dtype=torch.int32, device=device)
    ptrs = (k_host.data_ptr(), v_host.data_ptr(), k_host.stride(0))
    times, missed = [], []
    for step in range(steps + 2):
        idx = torch.sort(cur, dim=-1).values.to(torch.int32).contiguous()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        ops.lru_update(table, idx, cnt, None, None, backing_ptrs=ptrs)
        e1.record()
        torch.cuda.synchronize(device)
        if step >= 2:                                    # step 0 fills the table, step 1 warms up
            times.append(e0.elapsed_time(e1) * 1e3)
            missed.append(table.stats[..., 1].sum().item())      # the table's counters are per update: [hits, misses]
        nswap = max(1, int(churn * nsel))
        flat = cur.view(B * KH, nsel)
        for r in range(B * KH):                          # replace nswap entries of every list by tokens that are not in it
            absent = torch.ones(n, dtype=torch.bool, device=device)
            absent[flat[r]] = False
            pool = absent.nonzero().flatten()
            fresh = pool[torch.randperm(pool.numel(), generator=g, device=device)[:nswap]]
            where = torch.randperm(nsel, generator=g, device=device)[:nswap]
            flat[r, where] = fresh
    ok = int(table.status.item()) == 0
    us = sum(times) / len(times)
    rows = sum(missed) / len(missed)
    return {"workload": f"one layer, B{B} x {n} keys x {KH} kv heads, {nsel} attended keys per head, {churn:.0%} replaced per step",
            "us_per_update": us, "missed_rows_per_update": rows, "pcie_gbs": rows * 2 * HEAD_DIM * k_host.element_size() / us / 1e3,
            "status_words_ok": ok}


def reference_gpu_kernels(device):
    """The reference's own CUDA scorer beside this library's kernels, on the one shape it supports
    ((KH, QH) = (4, 28), spotlight/kernel/__init__.py:14-16): B 8 x 128K keys, three rotating code buffers.
    attn_k4_q28 is the reference's attn_k4_q28.cu compiled UNCHANGED for sm_100a into the checker's directory
    (oracle/build_ref.py); its top-k + gather is the operator sequence of spotlight/modifiers/gpu_cache.py:48-54
    (attn.topk(sorted=False), two torch.gather) run eagerly. The reference's Triton scorer is a source file of the
    reference and is not available where this runs."""
    import importlib.util
    path = os.path.join(ROOT, "oracle", "_ref", "attn_k4_q28.so")
    if not os.path.exists(path):
        return {"unavailable": "oracle/_ref/attn_k4_q28.so not built (oracle/build_ref.py needs a checkout of the reference)"}
    try:
        spec = importlib.util.spec_from_file_location("attn_k4_q28", path)
        ref = importlib.util.module_from_spec(spec)
        spec.loader.exec_module(ref)
    except Exception as e:
        return {"unavailable": f"could not load the reference kernel: {str(e)[:160]}"}
    import spotlight_b200.kernel as K
    from spotlight_b200 import ops
    g = torch.Generator(device=device).manual_seed(3)
    B, N, KH, QH, keep = 8, 131072, 4, 28, 2622
    q = torch.randint(0, 2 ** 31, (B, 1, QH, 4), generator=g, device=device).to(torch.int32).view(torch.uint32)
    ks = [torch.randint(0, 2 ** 31, (B, N, KH, 4), generator=g, device=device).to(torch.int32).view(torch.uint32) for _ in range(3)]
    kc = torch.randn((B, N, KH, HEAD_DIM), generator=g, device=device).to(torch.bfloat16)
    vc = torch.randn((B, N, KH, HEAD_DIM), generator=g, device=device).to(torch.bfloat16)

    def timed(fn, iters=30):
        for i in range(5):
            fn(ks[i % 3])
        torch.cuda.synchronize(device)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(iters):
            fn(ks[i % 3])
        e1.record()
        torch.cuda.synchronize(device)
        return e0.elapsed_time(e1) / iters * 1e3

    def ref_topk_and_gather(k):
        attn = ref.attn_k4_q28(q, k)
        ind = attn.topk(k=keep, dim=1, sorted=False).indices.unsqueeze(-1).expand(-1, -1, -1, HEAD_DIM)
        return torch.gather(kc, 1, ind), torch.gather(vc, 1, ind)

    qr = torch.randn((B, QH, HEAD_DIM), generator=g, device=device).to(torch.bfloat16)

    def ours_scan_and_attention(k):
        idx, cnt = ops.scan_topk(q, k, keep, 4, 64, 0)
        return ops.sparse_attn_decode(qr, kc, vc, idx, cnt, 0)

    res = {
        "shape": f"B{B} x {N} keys x ({KH},{QH}) heads, {B * N * KH * 16 / 1e6:.1f} MB of codes, top {keep}",
        "reference_attn_k4_q28_us": timed(lambda k: ref.attn_k4_q28(q, k)),
        "reference_attn_k4_q28_plus_torch_topk_us": timed(lambda k: ref.attn_k4_q28(q, k).topk(k=keep, dim=1, sorted=False)),
        "reference_scores_topk_and_gather_us": timed(ref_topk_and_gather),
        "ours_scores_only_us": timed(lambda k: K.attn_cuda_func(q, k)),
        "ours_fused_scan_topk_window_us": timed(lambda k: ops.scan_topk(q, k, keep, 4, 64, 0)),
        "ours_scan_topk_plus_sparse_attention_us": timed(ours_scan_and_attention),
        "triton_scorer": "not run: spotlight/kernel/attn_dx_u32.py is a source file of the reference, absent here",
    }
    del ks, kc, vc
    torch.cuda.empty_cache()
    return res


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=20)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="headline", choices=sorted(CONFIGS))
    ap.add_argument("--context", type=int, default=None)
    ap.add_argument("--layers", type=int, default=None)
    ap.add_argument("--batch", type=int, default=None)
    ap.add_argument("--mask-out", type=float, default=None)
    ap.add_argument("--no-graph", action="store_true")
    ap.add_argument("--separate-kv", action="store_true", help="two K/V caches per layer instead of one fused cache")
    ap.add_argument("--attn-warps", type=int, default=0, choices=[0, 4, 8], help="warps per CTA of the attention kernel (0: by shape)")
    ap.add_argument("--no-attn-cluster", action="store_true", help="combine the attention splits with the merge kernel even where a thread-block cluster fits")
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-reference-kernels", action="store_true", help="skip timing the reference's CUDA scorer beside ours (1 GPU)")
    ap.add_argument("--no-extras", action="store_true", help="with several ranks: skip the sharded / batch-split measurements")
    ap.add_argument("--decode-steps", type=int, default=0,
                    help="run this many consecutive decode tokens at advancing positions (config 1: 256) instead of "
                         "replaying one position")
    ap.add_argument("--python-loop", action="store_true",
                    help="with --decode-steps: keep the layer loop in Python (three calls per layer) instead of sl_decode_step")
    ap.add_argument("--lru", action="store_true",
                    help="make the four-stage step (with the LRU update) the timed `value` instead of reporting it beside the three-stage one")
    ap.add_argument("--no-lru", action="store_true", help="skip the four-stage measurement (stage 3: LRU-resident K/V buffer)")
    ap.add_argument("--peer", action="store_true",
                    help="with --sharded: exchange over peer memory (sl_peer_allgather) instead of NCCL all-gathers")
    ap.add_argument("--no-fused-scan", action="store_true",
                    help="with --peer: keep sl_scan_hist + exchange + sl_select_emit instead of the one-launch form")
    ap.add_argument("--sharded", action="store_true",
                    help="sequence-sharded layer-step across the ranks of a torchrun launch (config 4)")
    args = ap.parse_args()
    if args.impl == "ours":
        args.warmup = max(args.warmup, 3)
    cfg = CONFIGS[args.workload]
    over = {k: v for k, v in (("context", args.context), ("layers", args.layers), ("batch", args.batch),
                              ("mask_out", args.mask_out)) if v is not None}
    if over:
        import dataclasses
        cfg = dataclasses.replace(cfg, **over)
    if args.impl == "reference":
        run_reference(args, cfg)
    elif args.decode_steps:
        run_decode_loop(args, cfg)
    elif args.sharded:
        run_sharded(args, cfg)
    else:
        run_ours(args, cfg)


if __name__ == "__main__":
    main()
