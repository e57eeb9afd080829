"""Phase timing of the fused scan + top-k kernel (development aid).

    python -m spotlight_b200.profile_scan [B N KH QH [mask_out]]

The library's debug hook `sl_debug_scan_timing` makes thread 0 of every CTA record the SM cycle
counter at the kernel's phase boundaries (slot 15: the global timer at entry). This script runs
one stamped launch after a few warm-up launches and prints, per phase boundary, the minimum /
median / maximum over the CTAs of the time since the CTA's own start."""
from __future__ import annotations

import ctypes
import sys

import numpy as np
import torch

from . import _lib, ops
from .workloads import budget

PHASES = [(11, "planes ready, first loads back"), (7, "chunk scored"), (1, "histograms flushed"), (2, "grid barrier"),
          (3, "thresholds known"), (10, "own counts done"), (5, "all chunks' counts polled"), (6, "attended keys written")]


def main(argv):
    B, N, KH, QH = [int(x) for x in argv[:4]] if len(argv) >= 4 else (1, 131072, 8, 32)
    mask_out = float(argv[4]) if len(argv) > 4 else 0.9
    dev = torch.device("cuda")
    g = torch.Generator(device=dev).manual_seed(0)
    codes = [torch.randint(0, 2 ** 31, (B, N, KH, 4), generator=g, device=dev, dtype=torch.int64).to(torch.uint32)
             for _ in range(4)]
    q = torch.randint(0, 2 ** 31, (B, QH, 4), generator=g, device=dev, dtype=torch.int64).to(torch.uint32)
    k = budget(N, mask_out)
    buf = torch.zeros((4096, 16), dtype=torch.int64, device=dev)
    hook = _lib.lib.sl_debug_scan_timing
    hook.argtypes, hook.restype = [ctypes.c_void_p], None
    for i in range(5):
        ops.scan_topk(q, codes[i % 4], k, 4, 64)
    hook(buf.data_ptr())
    ops.scan_topk(q, codes[1], k, 4, 64)
    torch.cuda.synchronize()
    hook(None)
    ops.check_status()
    t = buf.cpu().numpy()
    t = t[t[:, 15] > 0]
    try:
        ghz = torch.cuda.clock_rate() / 1e3          # SM clock in MHz, sampled right after the launch
    except Exception:
        ghz = 1.965
    print(f"B={B} N={N} KH={KH} QH={QH} k={k}: {t.shape[0]} CTAs, start skew {(t[:, 15].max() - t[:, 15].min()) / 1e3:.2f} us, "
          f"SM clock {ghz:.3f} GHz")
    for col, name in PHASES:
        ok = t[:, col] > 0
        if not ok.any():
            continue
        rel = (t[ok, col] - t[ok, 0]) / ghz / 1e3
        print(f"  {name:32s} min {rel.min():6.2f}  median {np.median(rel):6.2f}  max {rel.max():6.2f} us")


if __name__ == "__main__":
    main(sys.argv[1:])
