"""CPU-side checks of the boundary: the library builds/loads, exports every symbol the header
declares, rejects bad arguments with status codes (no compute without a GPU), and the host
logic (budget rule, workload generators, sharded-selection arithmetic) is right."""
import os
import re

import numpy as np
import pytest
import torch

from oracle import spotlight_oracle as O

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    from spotlight_b200 import build
    build.build()
    from spotlight_b200 import _lib
    return _lib


def test_library_exports_every_declared_symbol(lib):
    header = open(os.path.join(ROOT, "include", "spotlight_b200.h")).read()
    declared = set(re.findall(r"\b(sl_[a-z0-9_]+)\s*\(", header))
    declared -= {"sl_status", "sl_dtype", "sl_gqa_layout", "sl_hash_params"}
    assert declared, "no declarations found"
    assert declared == set(lib.SIGNATURES), declared ^ set(lib.SIGNATURES)
    for name in declared:
        assert hasattr(lib.lib, name), name
    assert lib.lib.sl_version() >= 100


def test_bad_arguments_return_status_codes(lib):
    L = lib.lib
    assert L.sl_pack_signbits(None, 0, 8, None, None) == lib.SL_EINVAL
    assert b"null" in L.sl_last_error_string()
    assert L.sl_pack_signbits(16, 0, 7, 16, None) == lib.SL_ESHAPE
    assert L.sl_pack_signbits(8, 0, 8, 16, None) == lib.SL_EALIGN
    assert L.sl_hamming_scores(16, 16, 0, 16, 1, 10, 4, 28, 3, 0, None) == lib.SL_ESHAPE       # W = 3
    assert L.sl_hamming_scores(16, 16, 0, 16, 1, 10, 4, 30, 4, 0, None) == lib.SL_ESHAPE       # QH % KH
    assert L.sl_scan_topk(16, 16, 4000, 1, 100, 8, 8, 7, 10, 4, 64, 16, 100, 16, None, 256, 1 << 20, None, None) \
        == lib.SL_EINVAL                                                                          # layout 7
    assert L.sl_scan_topk(16, 16, 4000, 1, 100, 8, 8, 1, 10, 4, 64, 16, 5, 16, None, 256, 1 << 20, None, None) \
        == lib.SL_ESHAPE                                                                          # idx too small
    assert L.sl_scan_topk(16, 16, 4000, 1, 100, 8, 8, 1, 10, 4, 64, 16, 100, 16, None, 256, 8, None, None) \
        == lib.SL_EWORKSPACE
    with pytest.raises(ValueError):
        lib.check(lib.SL_ESHAPE)
    with pytest.raises(RuntimeError):
        lib.check(lib.SL_ETIMEOUT)
    assert L.sl_scan_topk_workspace_bytes(1, 131072, 8, 32) > 0
    assert L.sl_scan_topk_workspace_bytes(1, 131072, 8, 30) == 0


def test_ops_refuse_cpu_tensors(lib):
    from spotlight_b200 import ops
    with pytest.raises(RuntimeError, match="no CPU path"):
        ops.pack_signbits(torch.zeros((4, 128)))


def test_budget_rule_matches_reference_arithmetic():
    from spotlight_b200.workloads import budget
    table = {(4096, 0.9): 410, (32769, 0.9): 3277, (16384, 0.98): 328, (131072, 0.9): 13108,
             (131072, 0.98): 2622, (1048576, 0.98): 20972, (10, 0.98): 10, (100, 0.98): 20}
    for (n, m), k in table.items():
        assert budget(n, m, 20) == k == O.budget(n, m, 20)


def test_workload_generator_is_seeded_and_shaped():
    import dataclasses
    from spotlight_b200.workloads import CONFIGS, make_inputs
    cfg = dataclasses.replace(CONFIGS["cfg3"], context=300, batch=2)
    a, b = make_inputs(cfg), make_inputs(cfg)
    assert a.k.shape == (2, 300, 4, 128) and a.q.shape == (2, 28, 128) and a.k.dtype == torch.bfloat16
    assert torch.equal(a.k, b.k) and torch.equal(a.q, b.q) and torch.equal(a.hash_k["w"][0], b.hash_k["w"][0])
    assert a.hash_q["w"][0].shape == (28, 128, 128) and a.hash_k["w"][0].shape == (4, 128, 128)
    c = make_inputs(CONFIGS["cfg0"], context=64)
    assert c.hash_q is c.hash_k and c.k.dtype == torch.float32


@pytest.mark.parametrize("n,k,R", [(9000, 333, 4), (70, 20, 8), (40, 5, 8), (4096, 410, 2), (5, 20, 3)])
def test_sharded_selection_arithmetic(n, k, R):
    """The histogram/tie-quota rule used across sequence shards reproduces the single-shard
    selection (lowest index wins ties) for any cut of the sequence."""
    rng = np.random.default_rng(n)
    s = rng.integers(60, 70, size=n).astype(np.int16)                  # few distinct values: many ties
    bounds = [n * r // R for r in range(R + 1)]
    shards = [s[bounds[r]:bounds[r + 1]] for r in range(R)]
    got = np.concatenate(O.sharded_select(shards, k, 4, 64))
    np.testing.assert_array_equal(got, O.attended_set(s, k, 4, 64))


def test_selection_oracle_edge_cases():
    s = np.array([5, 9, 9, 1, 9, 9, 2], dtype=np.int16)
    np.testing.assert_array_equal(O.canonical_topk(s, 3), [1, 2, 4])          # ties -> lowest index
    np.testing.assert_array_equal(O.canonical_topk(s, 100), np.arange(7))     # k >= N
    np.testing.assert_array_equal(O.attended_set(s, 1, sink=1, recent=2), [0, 1, 5, 6])
    assert O.forced_ranges(3, 4, 64) == (3, 3)
    assert O.forced_ranges(1000, 4, 64) == (4, 936)
    assert O.threshold_from_hist(np.bincount(s, minlength=10), 3) == (9, 3)


def test_merge_partials_identity():
    g = torch.Generator().manual_seed(0)
    logits = torch.randn((6, 50), generator=g, dtype=torch.float64)
    v = torch.randn((50, 8), generator=g, dtype=torch.float64)
    whole = torch.softmax(logits, -1) @ v
    parts_o, parts_m, parts_l = [], [], []
    for lo, hi in ((0, 20), (20, 20), (20, 50)):                               # one empty part
        sl = logits[:, lo:hi]
        m = sl.max(-1).values if hi > lo else torch.full((6,), -float("inf"), dtype=torch.float64)
        p = torch.exp(sl - m[:, None]) if hi > lo else torch.zeros((6, 0), dtype=torch.float64)
        parts_o.append(p @ v[lo:hi]); parts_m.append(m); parts_l.append(p.sum(-1))
    got = O.merge_partials(torch.stack(parts_o), torch.stack(parts_m), torch.stack(parts_l))
    assert torch.allclose(got, whole, atol=1e-12)


def test_lru_model_policy():
    m = O.LruModel(n_max=50, slots=4)
    s, hits, misses = m.update(np.array([3, 9, 20]))
    assert (hits, misses) == (0, 3) and s.tolist() == [0, 1, 2]          # free slots, lowest index first
    s, hits, misses = m.update(np.array([9, 30]))
    assert (hits, misses) == (1, 1) and s.tolist() == [1, 3]             # the never-used slot goes before used ones
    s, hits, misses = m.update(np.array([9, 40, 41]))
    assert (hits, misses) == (1, 2) and s.tolist() == [1, 0, 2]          # oldest stamps (step 0) evicted, slot order
    assert m.tok2slot[3] == -1 and m.tok2slot[20] == -1 and m.tok2slot[30] == 3
