"""Seeded inputs shared by the fixture generator (make_golden.py) and the tests that read the
fixtures. Inputs are in the reference modifier's layout and PRE-RoPE: q [1,H,1,128],
k,v [1,H,N,128]; hash parameters are [H,in,out] / [H,out]."""
import torch

# name: (seed, heads, N, mask_out, hash kind, dtype, mlp_dims, residue, param scale, rope theta)
CASES = {
    "tiny_linear": (7, 2, 96, 0.5, "linear", torch.float32, None, True, None, 10000.0),
    "cfg0_linear": (1000, 8, 4096, 0.9, "linear", torch.float32, None, True, None, 10000.0),
    "small_mlp": (11, 4, 777, 0.9, "mlp", torch.float32, (128, 256, 128), False, 0.05, 500000.0),
    "small_mlp_res_bf16": (12, 4, 640, 0.98, "mlp", torch.bfloat16, (128, 128, 128), True, 0.05, 10000.0),
    # grouped-query attention, 8 query / 2 kv heads (last field): k, v are drawn per kv head and repeated to the
    # query heads as the reference modifier does (repeat_kv, spotlight_generation.py:128-129); the hash has
    # one parameter set per QUERY head, applied to the queries and to the repeated keys
    "gqa_mlp": (13, 8, 640, 0.9, "mlp", torch.float32, (128, 128, 128), True, 0.05, 500000.0, 2),
}


def build_case(name):
    seed, H, N, mask_out, kind, dtype, dims, residue, scale, theta, *rest = CASES[name]
    KH = rest[0] if rest else H
    g = torch.Generator().manual_seed(seed)
    k = torch.randn((1, KH, N, 128), generator=g)
    v = torch.randn((1, KH, N, 128), generator=g)
    q = torch.randn((1, H, 1, 128), generator=g)
    ch = torch.randperm(128, generator=g)[:4]
    k[..., ch] *= 8.0
    k[:, :, 0] *= 4.0
    if kind == "linear":
        ws = [(torch.randn((H, 128, 128), generator=g) / 128 ** 0.5).to(dtype)]
        bs = [None]
    else:
        ws, bs = [], []
        for i in range(len(dims) - 1):
            ws.append((torch.randn((H, dims[i], dims[i + 1]), generator=g) * scale).to(dtype))
            bs.append((torch.randn((H, dims[i + 1]), generator=g) * scale).to(dtype))
    params = {"kind": kind, "w": ws, "b": bs}
    k, v = k.to(dtype), v.to(dtype)
    G = H // KH
    return dict(q=q.to(dtype), k=k.repeat_interleave(G, dim=1), v=v.repeat_interleave(G, dim=1), params=params, heads=H, n=N,
                mask_out=mask_out, dtype=dtype, residue=residue, theta=theta, kv_heads=KH, k_kv=k, v_kv=v)
