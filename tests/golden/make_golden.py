"""Regenerates tests/golden/*.npz by running the REFERENCE's own functions on seeded inputs.

Run in a container that has the reference checkout (the fixtures, not the checkout, are what the tests read):

    python tests/golden/make_golden.py /path/to/reference [case ...]

The reference is imported unmodified; three import shims are needed with the installed
library versions: stub modules ``peft`` and ``profiler`` (imported but unused by
spotlight/modifiers/spotlight_generation.py:6,10) and the name ``CrossEntropyLoss`` that newer
transformers no longer re-export from modeling_llama (:4). cos/sin tables are supplied here
because the reference hard-codes a CUDA device and 8192 positions when it builds them (:139).

One ref_<case>.npz per case of cases.py, holding outputs of reference callables only:
  sim, topk      get_attn_score_using_angle_lsh -> sim [H,N]; torch.topk indices (the budget rule)
  attended, out  do_sdpa_attn with the reference mask (scatter of its top-k, then the
                 sink/recent lines of spotlight_evaluation.py:341-346 for the decode query)
  hq_pre, hk_bits, q_rot   LinearHashingFunction / MLPHashingFunction forward on the
                 check_and_apply_qk_rope outputs
Each file also stores SHA-256 digests of the seeded inputs so generator drift is detected, and
the tiny cases store the inputs themselves.
"""
import hashlib
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(os.path.dirname(HERE)))
sys.path.insert(0, HERE)


def import_reference(root):
    peft = types.ModuleType("peft")
    peft.get_peft_model = peft.LoraConfig = peft.TaskType = None
    sys.modules["peft"] = peft
    prof = types.ModuleType("profiler")
    prof.WallTime = object
    sys.modules["profiler"] = prof
    import transformers.models.llama.modeling_llama as ml
    if not hasattr(ml, "CrossEntropyLoss"):
        ml.CrossEntropyLoss = torch.nn.CrossEntropyLoss
    sys.path.insert(0, root)
    import spotlight.modifiers.spotlight_generation as sg
    import spotlight.modifiers.linearhashing_generation as lg
    import spotlight.modifiers.modify_llama as mll
    return sg, lg, mll


def digest(t: torch.Tensor) -> str:
    return hashlib.sha256(t.detach().contiguous().view(torch.uint8).numpy().tobytes()).hexdigest()


def main(root, only=()):
    sg, lg, mll = import_reference(root)
    from spotlight_b200.workloads import budget, rope_tables

    from cases import CASES, build_case
    for name in CASES:
        if only and name not in only:
            continue
        c = build_case(name)
        q, dtype, H, N = c["q"], c["dtype"], c["heads"], c["n"]
        G = H // c["kv_heads"]
        if G > 1:      # keys / values per kv head, repeated to the query heads by the reference's own import
            from transformers.models.llama.modeling_llama import repeat_kv
            k, v = repeat_kv(c["k_kv"], G), repeat_kv(c["v_kv"], G)
            assert torch.equal(k, c["k"]) and torch.equal(v, c["v"])
        else:
            k, v = c["k"], c["v"]
        mask_out, residue, theta, kind = c["mask_out"], c["residue"], c["theta"], c["params"]["kind"]
        seed = CASES[name][0]
        info = {"device": "cpu", "dtype": dtype}
        if kind == "linear":
            fn = lg.LinearHashingFunction(info)
            fn.linear = torch.nn.Parameter(c["params"]["w"][0][None], requires_grad=False)
        else:
            dims = list(CASES[name][6])
            fn = sg.MLPHashingFunction(info, H, len(dims) - 1, dims, residue)
            for layer, w, b in zip(fn.mlp, c["params"]["w"], c["params"]["b"]):
                assert layer.proj.shape == w[None].shape and layer.bias.shape == b[None, :, None].shape
                layer.proj = torch.nn.Parameter(w[None], requires_grad=False)
                layer.bias = torch.nn.Parameter(b[None, :, None], requires_grad=False)
        cos, sin = rope_tables(torch.arange(N), theta)
        cos, sin = cos.to(dtype), sin.to(dtype)
        with torch.no_grad():
            sim = sg.get_attn_score_using_angle_lsh(q, k, fn, cos, sin)        # [1,H,1,N]
            kk = budget(N, mask_out, 20)
            top = sim.topk(k=kk, dim=-1).indices                              # as aggregate_topk
            mask = torch.full((1, H, 1, N), torch.finfo(sim.dtype).min, dtype=sim.dtype)
            mask = mask.scatter_(dim=-1, index=top, value=0)
            bound = N                                                         # q_idx + 1, decode
            mask[..., 0, :min(4, bound)] = 0
            mask[..., 0, max(0, bound - 64):bound] = 0
            out = mll.do_sdpa_attn(q, k, v, cos, sin, mask=mask)               # [1,1,H*128]
            Qr, Kr = mll.check_and_apply_qk_rope(q, k, cos, sin)
            hq = fn(Qr)
            hk = fn(Kr)
        store = dict(
            seed=seed, heads=H, n=N, mask_out=mask_out, k=kk, kind=kind, theta=theta,
            dtype=str(dtype), residue=residue,
            sim=sim[0, :, 0].float().numpy().astype(np.int16),
            topk=top[0, :, 0].numpy().astype(np.int32),
            attended=(mask[0, :, 0] == 0).numpy(),
            out=out[0, 0].float().numpy(),
            hq_pre=hq[0, :, 0].float().numpy(),
            hk_bits=np.packbits((hk[0] > 0).numpy(), axis=-1, bitorder="little") if N <= 1024 else np.zeros(0, np.uint8),
            hk_absmin=np.float32(hk.float().abs().min().item()),
            q_rot=Qr[0, :, 0].float().numpy(),
            dig_q=digest(q), dig_k=digest(k), dig_v=digest(v),
            dig_w=digest(torch.cat([w.flatten().float() for w in c["params"]["w"]])),
        )
        if N <= 128:
            store.update(q=q.float().numpy(), k_in=k.float().numpy(), v_in=v.float().numpy(),
                         k_rot=Kr.float().numpy())
        np.savez_compressed(os.path.join(HERE, f"ref_{name}.npz"), **store)
        print(name, "k", kk, "sim range", int(sim.min()), int(sim.max()),
              "distinct", sim.unique().numel())


if __name__ == "__main__":
    if len(sys.argv) < 2:
        sys.exit("usage: make_golden.py <reference checkout> [case ...]")
    main(sys.argv[1], tuple(sys.argv[2:]))
