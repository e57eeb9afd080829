"""The workspace-free attention entry point, called straight through the C ABI.

`sl_sparse_attn_decode_static` exists for callers that cannot allocate device memory at the
point where they run attention (an engine whose pool already owns all of HBM, a decode loop that
bans cudaMalloc/cudaFree because they can stall the device): its scratch is a fixed array inside
the library. The test runs it twice in a row with different inputs -- the array keeps the
previous call's partials -- and requires both results to equal the caller-workspace entry
point's. This file sorts last so that a `-x` run has finished every other test before it."""
import ctypes

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _call(lib, fn, q, k, v, idx, cnt, out, lse, extra):
    B, QH, _ = q.shape
    KH = k.shape[2]
    args = [q.data_ptr(), k.data_ptr(), v.data_ptr(), 0, k.stride(0), idx.data_ptr(), idx.shape[2], cnt.data_ptr(),
            B, KH, QH, 1, out.data_ptr(), lse.data_ptr(), *extra, torch.cuda.current_stream().cuda_stream]
    return fn(*args)


def test_static_scratch_entry_point_matches_workspace_entry_point():
    from spotlight_b200 import _lib
    lib = _lib.lib
    dev = torch.device("cuda", 0)
    _lib.check(lib.sl_set_device(0))
    g = torch.Generator().manual_seed(123)
    B, N, KH, QH = 2, 6000, 4, 16
    k = torch.randn((B, N, KH, 128), generator=g).to(torch.bfloat16).to(dev)
    v = torch.randn((B, N, KH, 128), generator=g).to(torch.bfloat16).to(dev)
    need = lib.sl_sparse_attn_workspace_bytes(B, KH, QH)
    ws = torch.empty(need, dtype=torch.uint8, device=dev)
    for call, keep in enumerate((1500, 700)):                  # second call: shorter lists over stale partials
        q = torch.randn((B, QH, 128), generator=g).to(torch.bfloat16).to(dev)
        idx = torch.stack([torch.stack([torch.sort(torch.randperm(N, generator=g)[:keep]).values for _ in range(KH)])
                           for _ in range(B)]).to(torch.int32).to(dev)
        cnt = torch.full((B, KH), keep, dtype=torch.int32, device=dev)
        ref, ref_lse = torch.empty_like(q), torch.empty((B, QH), dtype=torch.float32, device=dev)
        got, got_lse = torch.empty_like(q), torch.empty((B, QH), dtype=torch.float32, device=dev)
        _lib.check(_call(lib, lib.sl_sparse_attn_decode, q, k, v, idx, cnt, ref, ref_lse, [ws.data_ptr(), ws.numel()]))
        _lib.check(_call(lib, lib.sl_sparse_attn_decode_static, q, k, v, idx, cnt, got, got_lse, []))
        torch.cuda.synchronize()
        assert torch.isfinite(got.float()).all()
        assert (got.float() - ref.float()).abs().max().item() <= 2e-2, f"call {call}"   # the suite's bf16 tolerance
        assert torch.equal(got, ref), f"call {call}: same kernels, same inputs -> same bits"
        assert torch.equal(got_lse, ref_lse)


def test_static_scratch_entry_point_refuses_shapes_beyond_its_array():
    from spotlight_b200 import _lib
    lib = _lib.lib
    _lib.check(lib.sl_set_device(0))
    B, KH, QH = 16, 8, 32                                          # B*QH = 512 > 252
    assert lib.sl_sparse_attn_workspace_bytes(B, KH, QH) > (8 << 20)
    t = torch.zeros(16, device="cuda")
    rc = lib.sl_sparse_attn_decode_static(t.data_ptr(), t.data_ptr(), t.data_ptr(), 0, 1024, t.data_ptr(), 1,
                                          t.data_ptr(), B, KH, QH, 1, t.data_ptr(), None, None)
    assert rc == _lib.SL_EWORKSPACE
    assert b"built-in array" in lib.sl_last_error_string()
