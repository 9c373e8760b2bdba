"""A minimal batched decode runtime around the attention operator: preallocated NHD KV caches,
chunked prefill that writes straight into them, and a lock-step greedy decode loop whose whole
per-token step (all layers) is captured once in a CUDA graph and replayed.

It stands where the reference's tutorial runtime stands (tutorial_code/runtime_common.py):
  * cache layout contract  k_nhd / v_nhd ``[B, total_len, KVH, D]``        (:375-379)
  * chunked prefill        ``prefill_in_chunks`` + ``alloc_nhd_caches_from_prefill`` (:274-397) --
    here K/V are written into the preallocated cache directly, there is no second
    ``[B,KVH,L,D]`` copy and no ``torch.cat`` growth;
  * one decode step        ``forward_one_token_manual_batched``            (:501-573);
  * lock-step greedy loop  ``generate_lockstep_batch``                     (:575-676): argmax of the
    current logits, finished sequences keep emitting the stop token, the forward pass runs
    ``max_new_tokens - 1`` times, the returned dictionary has the same timing keys.

The transformer itself (projections, norms, MLP, sampling) is plain PyTorch: those are callers of the
attention path, not the path.  The path's own pieces are this package's kernels: the fused
RoPE + cache append + q pack launch (``ops.rope_append``) and the decode attention with lengths read
from device memory (``santa_flash_batch_cuda.decode_systematic_ragged``), which is what makes the
step graph-capturable while the cache grows.
"""
from __future__ import annotations

import time
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import torch
import torch.nn.functional as F

from . import ops


@dataclass
class LlamaShape:
    """Architecture numbers of a Llama-style decoder (defaults: Llama-3.1-8B)."""
    hidden: int = 4096
    layers: int = 32
    heads: int = 32
    kv_heads: int = 8
    head_dim: int = 128
    intermediate: int = 14336
    vocab: int = 128256
    rms_eps: float = 1e-5
    rope_theta: float = 500000.0


class DecodeRuntime:
    """Random-initialised (or externally loaded) Llama-style model with NHD caches.

    attention: "santa_flash" / "santa_prop" (S samples per head, this package's kernels; fixed per-tile
    budget / budget proportional to the tiles' softmax mass, 256-row tiles) or "sdpa" (dense
    ``scaled_dot_product_attention`` over the cache, the reference's SDPABackend,
    tutorial_code/attention_backends.py:76-89).
    """

    def __init__(self, shape: LlamaShape, batch: int, total_len: int, device, *, dtype=torch.bfloat16,
                 weight_seed: int = 0, attention: str = "santa_flash", S: int = 256, attn_seed: int = 1690,
                 block_n: int = 0, init_std: float = 0.02, score_mode: int = 0):
        if shape.head_dim != 128 or shape.heads != 4 * shape.kv_heads:
            raise RuntimeError("This build supports only D=128 and GH=4 (H/KVH)")
        if attention not in ("santa_flash", "santa_prop", "sdpa"):
            raise ValueError(f"unknown attention backend {attention!r}")
        self.shape, self.B, self.T = shape, int(batch), int(total_len)
        self.dev, self.dtype = torch.device(device), dtype
        self.attention, self.S, self.attn_seed, self.block_n = attention, int(S), int(attn_seed), int(block_n)
        self.score_mode = int(score_mode)  # 0: the reference's score arithmetic; 1: opt-in tensor-core scores
        s, g = shape, torch.Generator(device=self.dev).manual_seed(weight_seed)

        def w(*size):
            return (torch.randn(*size, generator=g, device=self.dev, dtype=torch.float32) * init_std).to(dtype)

        qkv_out = (s.heads + 2 * s.kv_heads) * s.head_dim
        self.embed = w(s.vocab, s.hidden)
        self.lm_head = w(s.vocab, s.hidden)
        self.final_norm = torch.ones(s.hidden, device=self.dev, dtype=dtype)
        self.layers: List[Dict[str, torch.Tensor]] = []
        for _ in range(s.layers):
            self.layers.append(dict(
                wqkv=w(qkv_out, s.hidden), wo=w(s.hidden, s.heads * s.head_dim),
                w_gate_up=w(2 * s.intermediate, s.hidden), w_down=w(s.hidden, s.intermediate),
                norm1=torch.ones(s.hidden, device=self.dev, dtype=dtype),
                norm2=torch.ones(s.hidden, device=self.dev, dtype=dtype)))
        self.inv_freq = 1.0 / (s.rope_theta ** (torch.arange(0, s.head_dim, 2, device=self.dev,
                                                             dtype=torch.float32) / s.head_dim))
        # caches, layout contract of the reference: [B, total_len, KVH, D]
        self.k_cache = [torch.zeros(self.B, self.T, s.kv_heads, s.head_dim, device=self.dev, dtype=dtype)
                        for _ in range(s.layers)]
        self.v_cache = [torch.zeros(self.B, self.T, s.kv_heads, s.head_dim, device=self.dev, dtype=dtype)
                        for _ in range(s.layers)]
        # device-side step state (what a captured step reads and advances)
        self.pos = torch.zeros(self.B, dtype=torch.int32, device=self.dev)        # next write position
        self.seq_lens = torch.zeros(self.B, dtype=torch.int32, device=self.dev)   # pos + 1 during a step
        self.status = torch.zeros(1, dtype=torch.int32, device=self.dev)
        self.tok = torch.zeros(self.B, dtype=torch.long, device=self.dev)
        self.logits = torch.zeros(self.B, s.vocab, device=self.dev, dtype=torch.float32)
        self._graph: Optional[torch.cuda.CUDAGraph] = None
        self._graph_max_len = 0
        self._graph_stream: Optional[torch.cuda.Stream] = None
        self.attn_events: Optional[list] = None   # filled by eager steps when profiling is on
        if attention in ("santa_flash", "santa_prop"):
            import santa_b200
            santa_b200.enable_dropin()
            import santa_flash_batch_cuda
            import santa_prop_batch_cuda
            self._flash, self._prop = santa_flash_batch_cuda, santa_prop_batch_cuda
        self._bn = 0  # tile size the captured graph was planned for

    # ------------------------------------------------------------------ helpers
    def _tables(self, positions: torch.Tensor):
        """cos/sin [B,D] of int positions [B]: fp32 angles, cast to the storage type."""
        freqs = positions.to(torch.float32)[:, None] * self.inv_freq[None, :]
        emb = torch.cat((freqs, freqs), dim=-1)
        return emb.cos().to(self.dtype), emb.sin().to(self.dtype)

    def _norm(self, x, weight):
        return F.rms_norm(x, (self.shape.hidden,), weight, self.shape.rms_eps)

    def _mlp(self, x, lw):
        gu = F.linear(x, lw["w_gate_up"])
        gate, up = gu[..., : self.shape.intermediate], gu[..., self.shape.intermediate:]
        return F.linear(F.silu(gate) * up, lw["w_down"])

    def load_hf_state_dict(self, sd: Dict[str, torch.Tensor]) -> None:
        """Copy the weights of a Hugging Face Llama checkpoint/state dict (parity tests)."""
        def get(name):
            return sd[name].to(device=self.dev, dtype=self.dtype)
        self.embed.copy_(get("model.embed_tokens.weight"))
        self.lm_head.copy_(get("lm_head.weight") if "lm_head.weight" in sd else get("model.embed_tokens.weight"))
        self.final_norm.copy_(get("model.norm.weight"))
        for i, lw in enumerate(self.layers):
            p = f"model.layers.{i}."
            lw["wqkv"].copy_(torch.cat([get(p + "self_attn.q_proj.weight"), get(p + "self_attn.k_proj.weight"),
                                        get(p + "self_attn.v_proj.weight")], dim=0))
            lw["wo"].copy_(get(p + "self_attn.o_proj.weight"))
            lw["w_gate_up"].copy_(torch.cat([get(p + "mlp.gate_proj.weight"), get(p + "mlp.up_proj.weight")], dim=0))
            lw["w_down"].copy_(get(p + "mlp.down_proj.weight"))
            lw["norm1"].copy_(get(p + "input_layernorm.weight"))
            lw["norm2"].copy_(get(p + "post_attention_layernorm.weight"))

    # ------------------------------------------------------------------ prefill
    @torch.inference_mode()
    def prefill(self, input_ids: torch.Tensor, chunk: int = 512, seqs_per_pass: int = 4) -> torch.Tensor:
        """Chunked dense prefill of ``input_ids [B,L]``; K (rotated) and V of every chunk go straight
        into the caches.  ``seqs_per_pass`` sequences are run at a time, so that the dense attention
        of a chunk against a long prefix stays a few GB whatever the batch size.  Returns the last
        position's logits ``[B,V]`` (fp32)."""
        if chunk <= 0:
            raise ValueError(f"prefill_chunk_size must be > 0, got {chunk}")
        s, B = self.shape, self.B
        L = int(input_ids.shape[1])
        if input_ids.shape[0] != B or L > self.T:
            raise RuntimeError("prompt does not fit the runtime's batch / cache length")
        H, KVH, D = s.heads, s.kv_heads, s.head_dim
        last = torch.empty(B, s.vocab, device=self.dev, dtype=torch.float32)
        step_b = max(1, int(seqs_per_pass))
        for b0 in range(0, B, step_b):
            b1 = min(B, b0 + step_b)
            nb = b1 - b0
            for start in range(0, L, chunk):
                end = min(L, start + chunk)
                n = end - start
                x = self.embed[input_ids[b0:b1, start:end].to(self.dev)]                   # [nb,n,hidden]
                positions = torch.arange(start, end, device=self.dev)
                cos, sin = self._tables(positions)                                          # [n,D]
                cos, sin = cos[None, :, None, :], sin[None, :, None, :]
                mask = None
                if start > 0:  # keys [0,end) against queries [start,end): causal inside the chunk only
                    kidx = torch.arange(end, device=self.dev)[None, :]
                    mask = kidx <= positions[:, None]
                for li, lw in enumerate(self.layers):
                    h = self._norm(x, lw["norm1"])
                    qkv = F.linear(h, lw["wqkv"]).view(nb, n, H + 2 * KVH, D)
                    q, k, v = qkv[:, :, :H], qkv[:, :, H:H + KVH], qkv[:, :, H + KVH:]
                    q = _rope_seq(q, cos, sin)
                    k = _rope_seq(k, cos, sin)
                    self.k_cache[li][b0:b1, start:end].copy_(k)
                    self.v_cache[li][b0:b1, start:end].copy_(v)
                    kk = self.k_cache[li][b0:b1, :end].permute(0, 2, 1, 3)                 # [nb,KVH,end,D] view
                    vv = self.v_cache[li][b0:b1, :end].permute(0, 2, 1, 3)
                    a = F.scaled_dot_product_attention(q.permute(0, 2, 1, 3), kk, vv, attn_mask=mask,
                                                       is_causal=(mask is None), enable_gqa=True)
                    a = a.permute(0, 2, 1, 3).reshape(nb, n, H * D)
                    x = x + F.linear(a, lw["wo"])
                    x = x + self._mlp(self._norm(x, lw["norm2"]), lw)
                if end == L:
                    last[b0:b1] = F.linear(self._norm(x[:, -1], self.final_norm), self.lm_head).float()
        self.pos.fill_(L)
        return last

    def fill_cache_synthetic(self, prompt_len: int, seed: int = 0) -> None:
        """Fill rows [0, prompt_len) of every cache with seeded N(0,1) values (stands in for a prefill
        when only the decode phase is measured) and set the positions."""
        g = torch.Generator(device=self.dev).manual_seed(seed)
        for kc, vc in zip(self.k_cache, self.v_cache):
            kc[:, :prompt_len].normal_(generator=g)
            vc[:, :prompt_len].normal_(generator=g)
        self.pos.fill_(prompt_len)

    # ------------------------------------------------------------------ one decode step
    def _attend(self, q_bhd, li, max_len):
        if self.attention == "santa_flash":
            return self._flash.decode_systematic_ragged(q_bhd, self.k_cache[li], self.v_cache[li], self.seq_lens,
                                                        self.S, seed=self.attn_seed, block_n=self._bn,
                                                        want_vrows=False, max_len=max_len,
                                                        score_mode=self.score_mode)[0]
        if self.attention == "santa_prop":
            return self._prop.decode_systematic_ragged(q_bhd, self.k_cache[li], self.v_cache[li], self.seq_lens,
                                                       self.S, seed=self.attn_seed, want_vrows=False,
                                                       max_len=max_len, score_mode=self.score_mode)[0]
        # dense reference backend over the valid prefix (host-known bound; eager only)
        L = int(max_len)
        kk = self.k_cache[li][:, :L].permute(0, 2, 1, 3)
        vv = self.v_cache[li][:, :L].permute(0, 2, 1, 3)
        return F.scaled_dot_product_attention(q_bhd[:, :, None, :], kk, vv, enable_gqa=True)[:, :, 0, :]

    def _step(self, max_len: int) -> None:
        """Forward of ``self.tok`` at ``self.pos`` -> ``self.logits``; advances ``self.pos``.  Every
        length-dependent quantity is read from device memory."""
        s, B = self.shape, self.B
        H, KVH, D = s.heads, s.kv_heads, s.head_dim
        x = self.embed[self.tok]                                                        # [B,hidden]
        cos, sin = self._tables(self.pos)
        for li, lw in enumerate(self.layers):
            h = self._norm(x, lw["norm1"])
            qkv = F.linear(h, lw["wqkv"])                                               # [B,(H+2KVH)*D]
            q_bhd = ops.rope_append(qkv[:, : H * D], qkv[:, H * D: (H + KVH) * D], qkv[:, (H + KVH) * D:],
                                    cos, sin, self.k_cache[li], self.v_cache[li], self.pos,
                                    seq_lens_out=self.seq_lens, status=self.status)
            if self.attn_events is not None:
                e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                e0.record()
            a = self._attend(q_bhd, li, max_len)
            if self.attn_events is not None:
                e1.record()
                self.attn_events.append((e0, e1))
            x = x + F.linear(a.reshape(B, H * D), lw["wo"])
            x = x + self._mlp(self._norm(x, lw["norm2"]), lw)
        self.logits.copy_(F.linear(self._norm(x, self.final_norm), self.lm_head))
        self.pos.add_(1)

    def _plan_tile(self, max_len: int) -> int:
        from . import capi
        return capi.block_n_rule(max_len, self.block_n)

    @torch.inference_mode()
    def capture(self, max_len: int) -> None:
        """Capture the step for caches up to ``max_len`` rows long (the tile size is fixed per capture:
        the reference's rule applied to ``max_len``)."""
        if self.attention == "sdpa":
            raise RuntimeError("only the sampled-attention steps are graph-capturable (their lengths live on the device)")
        max_len = min(int(max_len), self.T)         # the lengths can never exceed the cache
        self._bn = self._plan_tile(max_len)
        saved = (self.pos.clone(), self.tok.clone())
        stream = torch.cuda.Stream(device=self.dev)
        stream.wait_stream(torch.cuda.current_stream(self.dev))
        with torch.cuda.stream(stream):
            for _ in range(2):                      # warm-up: workspaces, cuBLAS handles, kernel attributes
                self.pos.copy_(saved[0])
                self._step(max_len)
            self.pos.copy_(saved[0])
        torch.cuda.current_stream(self.dev).wait_stream(stream)
        torch.cuda.synchronize(self.dev)
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph, stream=stream):
            self._step(max_len)
        self._graph, self._graph_stream, self._graph_max_len = graph, stream, int(max_len)
        self.pos.copy_(saved[0])                    # capture does not run the step
        self.tok.copy_(saved[1])

    @torch.inference_mode()
    def step(self, max_len: int) -> None:
        if self._graph is not None and max_len <= self._graph_max_len:
            self._graph.replay()
        else:
            self._bn = self._plan_tile(max_len)
            self._step(max_len)

    # ------------------------------------------------------------------ generation loop
    @torch.inference_mode()
    def generate(self, prefill_logits_last: torch.Tensor, prompt_len: int, max_new_tokens: int,
                 stop_token_ids: Sequence[int] = (), lockstep_stop_mode: str = "max_tokens",
                 use_graph: bool = True) -> Dict[str, object]:
        """Lock-step greedy decoding (semantics of the reference's generate_lockstep_batch)."""
        B, dev = self.B, self.dev
        if prompt_len + max_new_tokens > self.T + 1:
            raise RuntimeError("cache too short for prompt_len + max_new_tokens")
        stop = torch.tensor(sorted({int(x) for x in stop_token_ids}), dtype=torch.long, device=dev)
        stop_fill = int(stop[0].item()) if stop.numel() else 0
        finished = torch.zeros(B, dtype=torch.bool, device=dev)
        out_tokens = torch.zeros(B, max_new_tokens, dtype=torch.long, device=dev)
        cur_logits = prefill_logits_last.to(dev).float().contiguous()
        self.pos.fill_(prompt_len)
        max_len = prompt_len + max_new_tokens
        if use_graph and self.attention != "sdpa" and (self._graph is None or max_len > self._graph_max_len):
            self.capture(max_len)
        torch.cuda.synchronize(dev)
        t0 = time.perf_counter()
        steps_sampled = 0
        for step in range(int(max_new_tokens)):
            next_ids = torch.argmax(cur_logits, dim=-1)
            next_ids = torch.where(finished, torch.full_like(next_ids, stop_fill), next_ids)
            out_tokens[:, step] = next_ids
            if stop.numel():
                finished |= torch.isin(next_ids, stop)
            steps_sampled = step + 1
            if step == int(max_new_tokens) - 1:
                break
            if lockstep_stop_mode == "all_finished" and bool(finished.all().item()):
                break
            self.tok.copy_(next_ids)
            if use_graph and self.attention != "sdpa":
                self.step(max_len)
            else:
                self._bn = self._plan_tile(prompt_len + step + 1)
                self._step(prompt_len + step + 1)
            cur_logits = self.logits
        torch.cuda.synchronize(dev)
        t1 = time.perf_counter()
        return {
            "decode_time_s": float(t1 - t0),
            "steps_sampled": int(steps_sampled),
            "timed_generated_tokens": int(B * steps_sampled),
            "generated_token_ids_all": out_tokens[:, :steps_sampled].cpu(),
            "device_status_word": int(self.status.item()),
        }


def _rope_seq(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """apply_rotary_pos_emb of the reference runtime (runtime_common.py:174-185) on [B,n,heads,D]."""
    half = x.shape[-1] // 2
    rot = torch.cat((-x[..., half:], x[..., :half]), dim=-1)
    return (x * cos) + (rot * sin)
