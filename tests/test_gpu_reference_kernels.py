"""The reference's own CUDA kernels (built from a checkout into oracle/_ref by oracle/build_ref.py)
run on the GPU beside ours: bit-exact agreement on the shape they support, (KH, QH) = (4, 28).
Skipped when the modules were not built."""
import importlib.util
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

REF = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "oracle", "_ref")


def _load(name):
    path = os.path.join(REF, name + ".so")
    if not os.path.exists(path):
        pytest.skip(f"{path} not built")
    spec = importlib.util.spec_from_file_location(name, path)
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    return mod


@pytest.mark.parametrize("B,N", [(1, 1000), (8, 131072), (3, 4097)])
def test_attn_k4_q28_bit_exact(B, N):
    import spotlight_b200.kernel as K
    from spotlight_b200 import ops
    ref = _load("attn_k4_q28")
    g = torch.Generator(device="cuda").manual_seed(N)
    q = torch.randint(0, 2 ** 31, (B, 1, 28, 4), generator=g, device="cuda").to(torch.int32).view(torch.uint32)
    k = torch.randint(0, 2 ** 31, (B, N, 4, 4), generator=g, device="cuda").to(torch.int32).view(torch.uint32)
    want = ref.attn_k4_q28(q, k)
    torch.cuda.synchronize()
    got = K.attn_cuda_func(q, k)
    assert got.dtype == want.dtype and got.shape == want.shape
    assert torch.equal(got, want)
    _, _, fused = ops.scan_topk(q, k, 20, 4, 64, 0, return_scores=True)      # the fused scorer, interleaved grouping
    assert torch.equal(fused, want)


def test_packbits_bit_exact():
    import spotlight_b200.kernel as K
    ref = _load("packbits")
    g = torch.Generator(device="cuda").manual_seed(1)
    x = torch.randn((7, 333, 128), generator=g, device="cuda").to(torch.bfloat16)
    x[0, 0, :9] = 0
    want = ref.packbits(x)
    torch.cuda.synchronize()
    got = K.pack_cuda_func(x)
    assert got.shape == want.shape and torch.equal(got.view(torch.int32), want.view(torch.int32))


def test_timing_beside_the_reference_kernel(capsys):
    """Not a pass/fail speed gate: times the reference's attn_k4_q28 beside this library's
    score-only shim and the fused scan + top-k on the reference kernel's native shape
    (B 8, 28/4 heads, 128K keys = 67 MB of codes, three rotating buffers so nothing stays in L2)
    and prints the figures; the only assertion is that the fused kernel is not slower than the
    reference's scoring pass alone plus a second of slack."""
    import spotlight_b200.kernel as K
    from spotlight_b200 import ops
    ref = _load("attn_k4_q28")
    g = torch.Generator(device="cuda").manual_seed(3)
    B, N = 8, 131072
    q = torch.randint(0, 2 ** 31, (B, 1, 28, 4), generator=g, device="cuda").to(torch.int32).view(torch.uint32)
    ks = [torch.randint(0, 2 ** 31, (B, N, 4, 4), generator=g, device="cuda").to(torch.int32).view(torch.uint32) for _ in range(3)]

    def timed(fn, iters=30):
        for i in range(5):
            fn(ks[i % 3])
        torch.cuda.synchronize()
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        e0.record()
        for i in range(iters):
            fn(ks[i % 3])
        e1.record()
        torch.cuda.synchronize()
        return e0.elapsed_time(e1) / iters * 1e3

    t_ref = timed(lambda k: ref.attn_k4_q28(q, k))
    t_topk = timed(lambda k: ref.attn_k4_q28(q, k).topk(k=2622, dim=1, sorted=False))
    t_shim = timed(lambda k: K.attn_cuda_func(q, k))
    t_fused = timed(lambda k: ops.scan_topk(q, k, 2622, 4, 64, 0))
    with capsys.disabled():
        print(f"\n[reference kernel timing, B8 x 128K x (4,28), 67.1 MB of codes] "
              f"reference attn_k4_q28 {t_ref:.1f} us | reference attn_k4_q28 + torch.topk {t_topk:.1f} us | "
              f"this library: scores only {t_shim:.1f} us, fused scan + exact top-k + window {t_fused:.1f} us")
    assert t_fused < t_ref + 1e6
