"""Dense (exact) decode attention on the host CPU -- the reference's `sdpa` backend.

TEST INFRASTRUCTURE / BASELINE ONLY: used by the benchmark's CPU-baseline leg and its reference
arm, and by tests.  Restates SDPABackend.decode (tutorial_code/attention_backends.py:76-89): the
arithmetic itself is torch's scaled_dot_product_attention with grouped-query broadcasting.
"""
from __future__ import annotations

import torch
import torch.nn.functional as F


def sdpa_decode(q_bhd: torch.Tensor, k_nhd: torch.Tensor, v_nhd: torch.Tensor, valid_len: int) -> torch.Tensor:
    """q_bhd [B,H,D], k_nhd/v_nhd [B,T,KVH,D] -> [B,H,D] (any device, any float dtype)."""
    q = q_bhd.unsqueeze(2)
    k = k_nhd[:, :valid_len].permute(0, 2, 1, 3)
    v = v_nhd[:, :valid_len].permute(0, 2, 1, 3)
    out = F.scaled_dot_product_attention(q, k, v, attn_mask=None, dropout_p=0.0, is_causal=False,
                                         enable_gqa=(q.shape[1] != k.shape[1]))
    return out[:, :, 0, :].contiguous()
