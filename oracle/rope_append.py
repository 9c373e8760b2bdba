"""CPU restatement of the reference runtime's step in front of the attention call -- TEST
INFRASTRUCTURE ONLY (imported by tests/ and tests/golden/make_golden_rope.py, never by the product).

Follows tutorial_code/runtime_common.py of the reference:
  :165-168  rotate_half(x) = cat(-x[..., D/2:], x[..., :D/2])
  :174-185  apply_rotary_pos_emb: x_embed = (x * cos) + (rotate_half(x) * sin), every elementwise op on
            16-bit tensors computing in fp32 and rounding its result to the tensor dtype
  :544-546  q/k/v projections viewed as [B,1,heads,D] and transposed to [B,heads,1,D]
  :551-556  kc[:, pos].copy_(k[:, :, 0, :]); vc[:, pos].copy_(v[:, :, 0, :]); q_bhd = q[:, :, 0, :]

The roundings are written out one by one here (product, product, sum) instead of relying on
torch's 16-bit operators; tests/golden/rope_*.npz, produced by the reference's own function,
pin this restatement.  Pinned: yes (tests/test_oracle_cpu.py::test_rope_oracle_matches_reference_golden).
"""
from __future__ import annotations

import torch


def rope_tables(positions: torch.Tensor, D: int, dtype: torch.dtype, theta: float = 500000.0):
    """cos/sin [B,D] of integer positions [B], computed in fp32 and cast (the default rotary of a
    Llama-style model; the tables are inputs of the step, any values would do)."""
    inv_freq = 1.0 / (theta ** (torch.arange(0, D, 2, dtype=torch.float32) / D))
    freqs = positions.to(torch.float32)[:, None] * inv_freq[None, :]
    emb = torch.cat((freqs, freqs), dim=-1)
    return emb.cos().to(dtype), emb.sin().to(dtype)


def _rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x [B,heads,D], cos/sin [B,D], all of one 16-bit dtype."""
    dt = x.dtype
    half = x.shape[-1] // 2
    rot = torch.cat((-x[..., half:], x[..., :half]), dim=-1)            # exact (sign flip)
    c, s = cos[:, None, :].float(), sin[:, None, :].float()
    a = (x.float() * c).to(dt)                                          # rounding 1
    r = (rot.float() * s).to(dt)                                        # rounding 2
    return (a.float() + r.float()).to(dt)                               # rounding 3


def rope_append_step(q_proj, k_proj, v_proj, cos, sin, k_cache, v_cache, pos):
    """One decode step's tensor work between the projections and the attention call.
    q_proj [B,H*D], k_proj/v_proj [B,KVH*D], cos/sin [B,D]; caches [B,L,KVH,D] are updated in place
    at ``pos`` (an int, or a list/tensor of per-sequence positions).  Returns q [B,H,D]."""
    B, _, KVH, D = k_cache.shape
    q = _rope(q_proj.reshape(B, -1, D), cos.reshape(B, D), sin.reshape(B, D))
    k = _rope(k_proj.reshape(B, KVH, D), cos.reshape(B, D), sin.reshape(B, D))
    v = v_proj.reshape(B, KVH, D)
    positions = [int(pos)] * B if not hasattr(pos, "__len__") else [int(x) for x in pos]
    for b, pb in enumerate(positions):
        k_cache[b, pb].copy_(k[b])
        v_cache[b, pb].copy_(v[b])
    return q.contiguous()
