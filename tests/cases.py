"""Seeded synthetic inputs shared by the golden-fixture generator and the tests.

Shapes follow the reference's Llama-3.1-8B attention layer (H = 4*KVH, D = 128);
values are i.i.d. N(0,1) (K optionally scaled), optionally with planted heavy
hitters: 1% of key positions per (batch, kv-head) are replaced by
4*q/||q|| + 0.1*N(0,1) for one head of the group, so attention mass is skewed.
Everything is drawn on the CPU from one torch.Generator so that the same call
gives the same bits on any machine."""
from __future__ import annotations

import math

import numpy as np
import torch

# name -> (kind, B, L_valid, L_storage, KVH, dtype, S, seed, block_n, kscale, heavy)
FLASH_CASES = {
    "cfg0_L4096_S32": dict(B=1, L=4096, Ls=4096, KVH=8, dtype="bf16", S=32, seed=1690, block_n=0,
                           kscale=1.0 / math.sqrt(128.0), heavy=False, gen_seed=1690),
    "bn32_L700_f16": dict(B=2, L=700, Ls=768, KVH=2, dtype="f16", S=64, seed=11, block_n=0, kscale=1.0,
                          heavy=True, gen_seed=3),
    "bn64_L2500": dict(B=1, L=2500, Ls=2500, KVH=4, dtype="bf16", S=300, seed=5, block_n=0, kscale=1.0,
                       heavy=True, gen_seed=4),
    "bn256_L1000_ragged": dict(B=2, L=1000, Ls=1100, KVH=2, dtype="bf16", S=2048, seed=42, block_n=256,
                               kscale=0.5, heavy=False, gen_seed=5),
}

PROP_CASES = {
    "vec_L4096_S256": dict(L=4096, KVH=8, GH=4, dtype="bf16", S=256, seed=1690, block_n=0, kscale=1.0, heavy=True,
                           gen_seed=6),
    "vec_L3300_S64_f16": dict(L=3300, KVH=2, GH=4, dtype="f16", S=64, seed=7, block_n=0, kscale=1.0, heavy=True,
                              gen_seed=7),
    "mma_L600_S48": dict(L=600, KVH=2, GH=4, dtype="bf16", S=48, seed=9, block_n=0, kscale=1.0, heavy=False,
                         gen_seed=8),
    "mma_L2000_bn64": dict(L=2000, KVH=4, GH=4, dtype="bf16", S=100, seed=10, block_n=0, kscale=1.0, heavy=True,
                           gen_seed=9),
}


def torch_dtype(name: str):
    return torch.bfloat16 if name == "bf16" else torch.float16


def make_qkv(B, Ls, KVH, dtype, gen_seed, kscale=1.0, heavy=False, GH=4, D=128):
    """Returns CPU tensors q [B,H,D], K,V [B,Ls,KVH,D] in the storage dtype."""
    g = torch.Generator().manual_seed(gen_seed)
    H = GH * KVH
    q = torch.randn(B, H, D, generator=g)
    K = torch.randn(B, Ls, KVH, D, generator=g) * kscale
    V = torch.randn(B, Ls, KVH, D, generator=g)
    if heavy:
        nh = max(1, Ls // 100)
        for b in range(B):
            for kv in range(KVH):
                idx = torch.randperm(Ls, generator=g)[:nh]
                qq = q[b, GH * kv + (idx % GH)]
                K[b, idx, kv] = 4.0 * qq / qq.norm(dim=-1, keepdim=True) + 0.1 * torch.randn(nh, D, generator=g)
    dt = torch_dtype(dtype)
    return q.to(dt), K.to(dt).contiguous(), V.to(dt).contiguous()


def bits(t: torch.Tensor) -> np.ndarray:
    """uint16 bit patterns of a bf16/f16 tensor (CPU or CUDA)."""
    return t.detach().cpu().contiguous().view(torch.int16).numpy().view(np.uint16)


# ---- the step in front of the attention call (RoPE of q/k, cache append, packed q) ------------
ROPE_CASES = {
    "bf16_B3_pos517": dict(B=3, H=32, KVH=8, L=640, pos=517, dtype="bf16", gen_seed=21),
    "f16_B2_pos0": dict(B=2, H=8, KVH=2, L=64, pos=0, dtype="f16", gen_seed=22),
    "bf16_B1_pos40000": dict(B=1, H=32, KVH=8, L=40001, pos=40000, dtype="bf16", gen_seed=23),
}


def make_rope_inputs(c):
    """Seeded projections of one new token per sequence and caches filled with a marker value."""
    dt = torch_dtype(c["dtype"])
    g = torch.Generator().manual_seed(c["gen_seed"])
    B, H, KVH, D, L = c["B"], c["H"], c["KVH"], 128, c["L"]
    q_proj = (2.0 * torch.randn(B, H * D, generator=g)).to(dt)
    k_proj = (2.0 * torch.randn(B, KVH * D, generator=g)).to(dt)
    v_proj = torch.randn(B, KVH * D, generator=g).to(dt)
    kc = torch.full((B, L, KVH, D), 0.5, dtype=dt)
    vc = torch.full((B, L, KVH, D), -0.25, dtype=dt)
    return q_proj, k_proj, v_proj, kc, vc
