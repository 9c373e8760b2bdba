"""Decode-attention backend objects with the interface of the reference's adapter layer
(tutorial_code/attention_backends.py): ``backend.decode(q_bhd, k_nhd, v_nhd, valid_len) -> out_bhd``
on ``q [B,H,D]`` and NHD caches ``[B,T,KVH,D]``, plus ``name``, ``exact_attention``, ``actual_mode``
and ``info()``.  Code written against the reference's ``SantaFlashBackend`` / ``SantaPropBackend`` /
``SDPABackend`` (:76-89, :418-520) can take these instead.

Differences, all in the direction of fewer launches:
  * ``SantaPropBackend`` decodes the whole batch with one ragged call
    (``santa_prop_batch_cuda.decode_systematic_ragged``, ``actual_mode == "batch_ragged"``) where the
    reference loops over the sequences (``"single_loop_fallback"``, :491-500); every sequence still uses
    the head index ``h`` in the random stream, as in that loop.  The ragged call always works on
    256-row tiles, so it is only taken when the reference's tile-size rule
    (santa_fused_proportional_tile_budgets/santa_cuda.cpp:61-77) gives 256 for the call: an integer
    ``valid_len`` above 3072 with no explicit ``block_n``, or ``block_n == 256``.  Shorter contexts
    and other tile sizes go through the per-sequence loop and sample exactly what the reference
    adapter samples.  ``loop=True`` forces the loop.  With per-sequence lengths on the device (see
    below) the host cannot apply the rule: the ragged call is used and sequences of at most 3072
    tokens are sampled on 256-row tiles instead of the rule's 32 / 64 rows.
  * ``valid_len`` may be an int (the reference's contract) or an int32 device tensor ``[B]`` of
    per-sequence lengths; the tensor form never touches the host and is what a captured CUDA graph needs.
"""
from __future__ import annotations

from typing import Any, Dict, Optional, Union

import torch
import torch.nn.functional as F


class BackendError(RuntimeError):
    pass


class DecodeAttentionBackend:
    name = "base"
    exact_attention = False

    def decode(self, q_bhd: torch.Tensor, k_nhd: torch.Tensor, v_nhd: torch.Tensor,
               valid_len: Union[int, torch.Tensor]) -> torch.Tensor:
        raise NotImplementedError

    def info(self) -> Dict[str, Any]:
        return {"name": self.name, "exact_attention": self.exact_attention}

    def smoke_test(self, *, device, dtype, num_heads: int, num_kv_heads: int, head_dim: int,
                   valid_len: int = 16) -> Dict[str, Any]:
        """Two random sequences of ``valid_len`` cached tokens through ``decode``; the output must have
        the query's shape and be finite (the reference's start-up check of a backend,
        attention_backends.py:41-67, which looks at the shape only)."""
        B = 2
        q = torch.randn(B, num_heads, head_dim, device=device, dtype=dtype)
        k = torch.randn(B, valid_len, num_kv_heads, head_dim, device=device, dtype=dtype)
        v = torch.randn(B, valid_len, num_kv_heads, head_dim, device=device, dtype=dtype)
        out = self.decode(q, k, v, valid_len)
        if tuple(out.shape) != (B, num_heads, head_dim):
            raise BackendError(f"Smoke test returned wrong shape for {self.name}: got {tuple(out.shape)}, "
                               f"expected {(B, num_heads, head_dim)}")
        if not bool(torch.isfinite(out.float()).all()):
            raise BackendError(f"Smoke test of {self.name} produced non-finite values")
        return {"backend": self.name, "batch_size": B, "valid_len": int(valid_len),
                "output_shape": list(out.shape), **self.info()}


class SDPABackend(DecodeAttentionBackend):
    """Dense, exact attention over the valid prefix (the reference's CPU-runnable backend)."""
    name = "sdpa"
    exact_attention = True

    def decode(self, q_bhd, k_nhd, v_nhd, valid_len):
        L = int(valid_len)
        k = k_nhd[:, :L].permute(0, 2, 1, 3)
        v = v_nhd[:, :L].permute(0, 2, 1, 3)
        return F.scaled_dot_product_attention(q_bhd[:, :, None, :], k, v, enable_gqa=True)[:, :, 0, :].contiguous()


class _SantaBackend(DecodeAttentionBackend):
    module_name = ""

    def __init__(self, *, S: int, seed: int, block_n: Optional[int] = None, score_mode: int = 0) -> None:
        import santa_b200
        santa_b200.enable_dropin()
        import importlib
        try:
            self.module = importlib.import_module(self.module_name)
        except Exception as exc:  # noqa: BLE001
            raise BackendError(f"Could not import the {self.name} extension module {self.module_name}: {exc}")
        self.S, self.seed = int(S), int(seed)
        self.block_n = None if block_n is None else int(block_n)
        # 0: the reference's score arithmetic (sampled rows equal the reference's); 1: the opt-in
        # tensor-core scores.  Passed on only when set, so the default call is the reference adapter's.
        self._mode_kw = {"score_mode": int(score_mode)} if int(score_mode) != 0 else {}
        self.actual_mode = "unknown"
        self.supports_true_batch_decode = hasattr(self.module, "decode_systematic_batched")

    def info(self) -> Dict[str, Any]:
        return {**super().info(), "module": self.module_name, "requested_S": self.S, "seed": self.seed,
                "block_n": self.block_n, "actual_mode": self.actual_mode,
                "score_mode": self._mode_kw.get("score_mode", 0)}

    @staticmethod
    def _lengths(valid_len, B, device):
        if isinstance(valid_len, torch.Tensor):
            return valid_len
        return torch.full((B,), int(valid_len), dtype=torch.int32, device=device)


class SantaFlashBackend(_SantaBackend):
    name = "santa_flash"
    module_name = "santa_flash_batch_cuda"

    def decode(self, q_bhd, k_nhd, v_nhd, valid_len):
        bn = 0 if self.block_n is None else self.block_n
        if isinstance(valid_len, torch.Tensor):   # per-sequence lengths on the device
            self.actual_mode = "batch_ragged"
            return self.module.decode_systematic_ragged(q_bhd, k_nhd, v_nhd, valid_len, self.S, seed=self.seed,
                                                        block_n=bn, want_vrows=False, **self._mode_kw)[0]
        self.actual_mode = "batch"
        return self.module.decode_systematic_batched(q_bhd, k_nhd, v_nhd, self.S, seed=self.seed, block_n=bn,
                                                     want_vrows=False, valid_len=int(valid_len), **self._mode_kw)[0]


class SantaPropBackend(_SantaBackend):
    name = "santa_prop"
    module_name = "santa_prop_batch_cuda"

    def __init__(self, *, S: int, seed: int, block_n: Optional[int] = None, loop: bool = False,
                 score_mode: int = 0) -> None:
        super().__init__(S=S, seed=seed, block_n=block_n, score_mode=score_mode)
        self.loop = bool(loop)

    def decode(self, q_bhd, k_nhd, v_nhd, valid_len):
        B = int(q_bhd.shape[0])
        if isinstance(valid_len, torch.Tensor):
            ragged_ok = self.block_n in (None, 0, 256) and not self.loop
        else:  # the ragged call's 256-row tiles must be what the reference's rule picks for this length
            from . import capi
            bn = capi.block_n_rule(int(valid_len), 0 if self.block_n is None else self.block_n)
            ragged_ok = bn == 256 and not self.loop
        if ragged_ok:
            self.actual_mode = "batch_ragged"
            lens = self._lengths(valid_len, B, q_bhd.device)
            return self.module.decode_systematic_ragged(q_bhd, k_nhd, v_nhd, lens, self.S, seed=self.seed,
                                                        want_vrows=False, **self._mode_kw)[0]
        # the reference adapter's per-sequence loop over contiguous prefixes
        self.actual_mode = "single_loop_fallback"
        lens = [int(n) for n in valid_len.tolist()] if isinstance(valid_len, torch.Tensor) else [int(valid_len)] * B
        kw = dict(self._mode_kw) if self.block_n is None else {"block_n": self.block_n, **self._mode_kw}
        outs = [self.module.decode_systematic_scalar(q_bhd[b].contiguous(), k_nhd[b, :lens[b]].contiguous(),
                                                     v_nhd[b, :lens[b]].contiguous(), self.S, seed=self.seed,
                                                     want_vrows=False, **kw)[0] for b in range(B)]
        return torch.stack(outs, dim=0).contiguous()


def make_backend(name: str, *, santa_s: int = 256, santa_seed: int = 1690,
                 santa_block_n: Optional[int] = None, score_mode: int = 0) -> DecodeAttentionBackend:
    """Backend by the reference's names: "sdpa", "santa_flash", "santa_prop"."""
    if name == "sdpa":
        return SDPABackend()
    if name == "santa_flash":
        return SantaFlashBackend(S=santa_s, seed=santa_seed, block_n=santa_block_n, score_mode=score_mode)
    if name == "santa_prop":
        return SantaPropBackend(S=santa_s, seed=santa_seed, block_n=santa_block_n, score_mode=score_mode)
    raise BackendError(f"unknown backend {name!r} (this package provides sdpa, santa_flash, santa_prop)")
