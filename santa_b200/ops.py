"""Python host mirror of the reference operator surface, over the C ABI.

``flash_decode`` / ``prop_decode`` take the same positional and keyword
arguments, tensor layouts and seed semantics as the reference's
``santa_flash_batch_cuda.decode_systematic_{batched,scalar}`` and
``santa_prop_batch_cuda.decode_systematic_scalar`` (santa_cuda.cpp:174-359 of
flash_style_fused_santa_fixed_tile_budgets, santa_cuda.cpp:270-359 of
santa_fused_proportional_tile_budgets), raise ``RuntimeError`` with the same
messages on bad input, and return ``(out, m_star, vrows)``.  Extra keyword-only
arguments expose what the sharded runs and the parity tests need.  PyTorch only
supplies device memory and the current stream.
"""
from __future__ import annotations

import ctypes as C
import os
from dataclasses import dataclass
from typing import Dict, Tuple

import torch

from . import capi

_workspaces: Dict[Tuple[str, int, int], torch.Tensor] = {}


def _check(cond: bool, msg: str) -> None:
    if not cond:
        raise RuntimeError(msg)


def _workspace(kind: str, device: torch.device, nbytes: int) -> torch.Tensor:
    """Zero-initialised scratch, one per (kind, device, stream); grown on demand.

    Calls on one stream are ordered, so they can share the scratch; the kernels
    leave it zeroed where it has to be."""
    stream = torch.cuda.current_stream(device).cuda_stream
    key = (kind, device.index if device.index is not None else torch.cuda.current_device(), stream)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.zeros(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def _dtype_code(t: torch.Tensor) -> int:
    return capi.SANTA_DTYPE_BF16 if t.dtype == torch.bfloat16 else capi.SANTA_DTYPE_F16


@dataclass
class FlashTrace:
    """Per-tile and per-row intermediates of one Flash call (parity tests)."""
    block_n: int
    T_c: int
    S_per_tile: int
    m_tiles: torch.Tensor    # [B,H,T_c] fp32
    ell_tiles: torch.Tensor  # [B,H,T_c] fp32
    u16: torch.Tensor        # [B,H,L] int16 view of storage bits
    counts: torch.Tensor     # [B,H,L] int16
    rowmask: torch.Tensor    # [B,KVH,L] int32
    invdel: torch.Tensor     # [B,H,T_c] fp32


def _check_flash_inputs(q_h, K_g, V_g):
    # messages follow flash_style_fused_santa_fixed_tile_budgets/santa_cuda.cpp:123-171
    _check(q_h.is_cuda, "q_h must be CUDA")
    _check(K_g.is_cuda and V_g.is_cuda, "K_g and V_g must be CUDA")
    _check(q_h.dtype in (torch.bfloat16, torch.float16), "q_h must be bf16 or f16")
    _check(K_g.dtype in (torch.bfloat16, torch.float16), "K_g must be bf16 or f16")
    _check(K_g.dtype == V_g.dtype, "K_g and V_g must have the same dtype")
    _check(q_h.dtype == K_g.dtype, "q_h dtype must match K_g/V_g dtype")
    _check(q_h.device == K_g.device and q_h.device == V_g.device, "device mismatch")
    _check(K_g.is_contiguous() and V_g.is_contiguous(),
           "K_g/V_g must be contiguous. Expected [L,KVH,D] for single or [B,L,KVH,D] for batch.")
    if q_h.dim() == 2:
        _check(K_g.dim() == 3 and V_g.dim() == 3, "Single-request path expects q_h [H,D], K_g/V_g [L,KVH,D]")
        _check(K_g.shape == V_g.shape, "K_g and V_g must have the same shape")
        _check(q_h.size(1) == K_g.size(2), "D mismatch (q_h.size(1) vs K_g.size(2))")
        return False, 1, q_h.size(0), q_h.size(1), K_g.size(0), K_g.size(1)
    _check(q_h.dim() == 3 and K_g.dim() == 4 and V_g.dim() == 4,
           "Batched path expects q_h [B,H,D], K_g/V_g [B,L,KVH,D]")
    _check(K_g.shape == V_g.shape, "K_g and V_g must have the same shape")
    _check(q_h.size(0) == K_g.size(0), "Batch mismatch between q_h and K_g/V_g")
    _check(q_h.size(2) == K_g.size(3), "D mismatch (q_h.size(2) vs K_g.size(3))")
    return True, q_h.size(0), q_h.size(1), q_h.size(2), K_g.size(1), K_g.size(2)


def flash_decode(q_h, K_g, V_g, S, seed=42, block_n=0, want_vrows=False, valid_len=-1, *,
                 batch_offset=0, tile_offset=0, s_per_tile=None, partial=False, trace=False, out=None,
                 score_mode=0):
    """S2ANTA-Flash decode.  Returns ``(out, m_star, vrows)``; with ``partial=True``
    the first element is the unnormalised partial ``[B,H,130]`` fp32 instead of
    ``out``; with ``trace=True`` a ``FlashTrace`` is appended.  ``out`` may name the result buffer: a
    contiguous tensor of q's shape and dtype on q's device, or in PINNED HOST memory -- the merge kernel
    then stores the result straight into the caller's host buffer (no separate device-to-host copy).
    ``score_mode=1`` forms the scores on the tensor cores (opt-in; sampled counts then differ from the
    reference's on rare rows), 0 is the reference's fp32 order."""
    batched, B, H, D, L_storage, KVH = _check_flash_inputs(q_h, K_g, V_g)
    if seed < 0:
        raise TypeError("seed must be a non-negative 64-bit integer")
    q = q_h.contiguous()
    L = int(valid_len) if valid_len > 0 else L_storage
    _check(L > 0, f"valid_len must be > 0; got {L}")
    _check(L <= L_storage, f"valid_len exceeds storage length: valid_len={L} storage={L_storage}")
    _check(D == 128, f"This build supports only D=128. Got D={D}")
    _check(H % KVH == 0, f"H must be divisible by KVH. Got H={H} KVH={KVH}")
    _check(H // KVH == 4, f"This build supports only GH=4 (H/KVH). Got GH={H // KVH} (H={H} KVH={KVH})")
    bn = capi.block_n_rule(L, int(block_n))
    _check(bn in (32, 64, 256), f"block_n must be 0 (auto) or one of {{32,64,256}}. Got block_n={bn}")
    T_c, spt = capi.flash_budget(L, bn, int(S))
    if s_per_tile is not None:
        spt = int(s_per_tile)

    dev = q.device
    with torch.cuda.device(dev):
        lib = capi.lib()
        nbytes = lib.santa_flash_workspace_bytes(B, KVH, L, bn)
        ws = _workspace("flash", dev, nbytes)
        fopt = dict(device=dev, dtype=torch.float32)
        if out is not None:
            _check(not partial, "out= and partial=True exclude each other")
            _check(out.dtype == q.dtype and tuple(out.shape) == ((B, H, D) if batched else (H, D))
                   and out.is_contiguous(), "out must be a contiguous tensor of q's shape and dtype")
            _check((out.is_cuda and out.device == dev) or (not out.is_cuda and out.is_pinned()),
                   "out must live on q's device or in pinned host memory")
        elif not partial:
            out = torch.empty((B, H, D) if batched else (H, D), device=dev, dtype=q.dtype)
        m_star = torch.empty((B, H) if batched else (H,), **fopt)
        vrows = torch.empty((B, KVH) if (want_vrows and batched) else ((KVH,) if want_vrows else (0,)),
                            device=dev, dtype=torch.int32)
        ext = capi.FlashExt(batch_offset=int(batch_offset), tile_offset=int(tile_offset),
                            s_per_tile_override=-1 if s_per_tile is None else int(s_per_tile),
                            score_mode=int(score_mode))
        part = None
        if partial:
            part = torch.empty((B, H, D + 2), **fopt)
            ext.partial_out = part.data_ptr()
        tr = None
        if trace:
            tr = FlashTrace(bn, T_c, spt,
                            torch.empty((B, H, T_c), **fopt), torch.empty((B, H, T_c), **fopt),
                            torch.zeros((B, H, L), device=dev, dtype=torch.int16),
                            torch.zeros((B, H, L), device=dev, dtype=torch.int16),
                            torch.zeros((B, KVH, L), device=dev, dtype=torch.int32),
                            torch.empty((B, H, T_c), **fopt))
            ext.invdel = tr.invdel.data_ptr()
            ext.m_tiles, ext.ell_tiles = tr.m_tiles.data_ptr(), tr.ell_tiles.data_ptr()
            if trace != "tiles":  # trace="tiles": per-tile statistics only, no per-row tables
                ext.u16, ext.counts, ext.rowmask = tr.u16.data_ptr(), tr.counts.data_ptr(), tr.rowmask.data_ptr()
        rc = lib.santa_flash_decode(
            q.data_ptr(), K_g.data_ptr(), V_g.data_ptr(), _dtype_code(q), B, H, KVH, D, L, L_storage,
            int(S), int(seed) & (2**64 - 1), bn,
            None if out is None else out.data_ptr(), m_star.data_ptr(),
            vrows.data_ptr() if want_vrows else None,
            ws.data_ptr(), ws.numel(), C.byref(ext), torch.cuda.current_stream(dev).cuda_stream)
        capi.check(rc)
    res = (part if partial else out, m_star, vrows)
    return res + (tr,) if trace else res


def flash_decode_ragged(q_bh, K_g, V_g, seq_lens, S, seed=42, block_n=0, want_vrows=False, *, max_len=None,
                        batch_offset=0, trace=False, score_mode=0):
    """S2ANTA-Flash decode with per-sequence lengths read from device memory: ``q_bh [B,H,D]``,
    ``K_g/V_g [B,L_storage,KVH,D]``, ``seq_lens`` int32 ``[B]`` (a CPU tensor or list is copied over).
    Sequence ``b`` gets the result of ``flash_decode`` on it alone with ``valid_len=len_b``, the same
    ``block_n`` and ``batch_offset + b``.  ``block_n <= 0`` applies the tile-size rule to ``max_len``
    (default: the storage length).  Returns ``(out, m_star, vrows)`` (+ ``FlashTrace`` with arrays laid
    out for ``max_len``)."""
    batched, B, H, D, L_storage, KVH = _check_flash_inputs(q_bh, K_g, V_g)
    _check(batched, "Ragged path expects q_h [B,H,D], K_g/V_g [B,L,KVH,D]")
    if seed < 0:
        raise TypeError("seed must be a non-negative 64-bit integer")
    q = q_bh.contiguous()
    _check(D == 128, f"This build supports only D=128. Got D={D}")
    _check(H % KVH == 0 and H // KVH == 4, f"This build supports only GH=4 (H/KVH). Got H={H} KVH={KVH}")
    dev = q.device
    if not isinstance(seq_lens, torch.Tensor):
        seq_lens = torch.tensor(list(seq_lens), dtype=torch.int32)
    _check(seq_lens.numel() == B, "seq_lens must hold one length per sequence")
    lens = seq_lens.to(device=dev, dtype=torch.int32).contiguous()
    mlen = L_storage if max_len is None else int(max_len)
    _check(0 < mlen <= L_storage, f"max_len must be in (0, storage length]; got {mlen} (storage {L_storage})")
    bn = capi.block_n_rule(mlen, int(block_n))
    _check(bn in (32, 64, 256), f"block_n must be 0 (auto) or one of {{32,64,256}}. Got block_n={bn}")
    T_max = (mlen + bn - 1) // bn
    with torch.cuda.device(dev):
        lib = capi.lib()
        nbytes = lib.santa_flash_ragged_workspace_bytes(B, KVH, mlen, bn)
        _check(nbytes > 0, "santa_b200: unsupported ragged problem (B must be 1..1024)")
        ws = _workspace("flash_ragged", dev, nbytes)
        fopt = dict(device=dev, dtype=torch.float32)
        out = torch.empty((B, H, D), device=dev, dtype=q.dtype)
        m_star = torch.empty((B, H), **fopt)
        vrows = torch.empty((B, KVH) if want_vrows else (0,), device=dev, dtype=torch.int32)
        ext = capi.FlashExt(batch_offset=int(batch_offset), tile_offset=0, s_per_tile_override=-1,
                            score_mode=int(score_mode))
        tr = None
        if trace:
            tr = FlashTrace(bn, T_max, -1,
                            torch.zeros((B, H, T_max), **fopt), torch.zeros((B, H, T_max), **fopt),
                            torch.zeros((B, H, mlen), device=dev, dtype=torch.int16),
                            torch.zeros((B, H, mlen), device=dev, dtype=torch.int16),
                            torch.zeros((B, KVH, mlen), device=dev, dtype=torch.int32),
                            torch.zeros((B, H, T_max), **fopt))
            ext.invdel = tr.invdel.data_ptr()
            ext.m_tiles, ext.ell_tiles = tr.m_tiles.data_ptr(), tr.ell_tiles.data_ptr()
            ext.u16, ext.counts, ext.rowmask = tr.u16.data_ptr(), tr.counts.data_ptr(), tr.rowmask.data_ptr()
        rc = lib.santa_flash_decode_ragged(
            q.data_ptr(), K_g.data_ptr(), V_g.data_ptr(), _dtype_code(q), B, H, KVH, D, L_storage,
            lens.data_ptr(), mlen, int(S), int(seed) & (2**64 - 1), bn, out.data_ptr(), m_star.data_ptr(),
            vrows.data_ptr() if want_vrows else None, ws.data_ptr(), ws.numel(), C.byref(ext),
            torch.cuda.current_stream(dev).cuda_stream)
        capi.check(rc)
    res = (out, m_star, vrows)
    return res + (tr,) if trace else res


def rope_append(q_proj, k_proj, v_proj, cos, sin, k_cache, v_cache, pos, *, seq_lens_out=None, status=None,
                q_out=None):
    """Rotary embedding of one new token's q/k, append of k/v to the NHD caches at ``pos`` and the packed
    ``q [B,H,D]`` -- one launch for runtime_common.py:540-556 of the reference.  ``q_proj`` is
    ``[B,H*D]``/``[B,1,H*D]``/``[B,H,D]``, ``k_proj``/``v_proj`` likewise with KVH heads, ``cos``/``sin``
    ``[B,D]`` or ``[B,1,D]``; ``pos`` is an int or an int32 device tensor ``[B]``.  The three projections
    may also be pinned host tensors: the kernel then reads them over PCIe, which saves the separate
    host-to-device copy of a step's inputs.  Returns the rotated q."""
    B, L_storage, KVH, D = k_cache.shape
    _check(D == 128, f"This build supports only D=128. Got D={D}")
    _check(k_cache.shape == v_cache.shape and k_cache.is_contiguous() and v_cache.is_contiguous(),
           "k_cache/v_cache must be contiguous [B,L,KVH,D] tensors of one shape")
    dev = k_cache.device
    _check(k_cache.is_cuda and q_proj.dtype in (torch.bfloat16, torch.float16), "the caches must be CUDA tensors, q_proj bf16/f16")
    for t in (q_proj, k_proj, v_proj):  # the new token's projections: on the caches' device, or in pinned host memory
        _check(t.dtype == q_proj.dtype and (t.device == dev or (t.device.type == "cpu" and t.is_pinned())),
               "q_proj/k_proj/v_proj must share one dtype and live on the caches' device or in pinned host memory")
    for t in (cos, sin, k_cache, v_cache):
        _check(t.dtype == q_proj.dtype and t.device == dev, "cos/sin and the caches must share q_proj's dtype and one device")
    _check(q_proj.size(0) == B and q_proj.numel() % (B * D) == 0, "q_proj must hold [B, H*D] elements")
    H = q_proj.numel() // (B * D)
    _check(k_proj.numel() == B * KVH * D and v_proj.numel() == B * KVH * D, "k_proj/v_proj must hold [B, KVH*D] elements")
    _check(cos.numel() == B * D and sin.numel() == B * D, "cos/sin must hold [B, D] elements")
    def rows(t):
        # [B, n] with unit inner stride is taken as is (a slice of a fused projection), else packed
        if t.dim() == 2 and t.stride(1) == 1 and t.stride(0) % 4 == 0 and t.data_ptr() % 8 == 0:
            return t, t.stride(0)
        t = t.contiguous()
        return t, t.numel() // B
    (q_proj, qs), (k_proj, ks), (v_proj, vs) = rows(q_proj), rows(k_proj), rows(v_proj)
    cos, sin = cos.contiguous(), sin.contiguous()
    pos_dev = None
    if isinstance(pos, torch.Tensor):
        _check(pos.dtype == torch.int32 and pos.device == dev and pos.numel() == B and pos.is_contiguous(),
               "pos must be an int or a contiguous int32 tensor [B] on the same device")
        pos_dev, pos_host = pos, 0
    else:
        pos_host = int(pos)
        _check(0 <= pos_host < L_storage, f"pos out of range: {pos_host} (storage {L_storage})")
    with torch.cuda.device(dev):
        if q_out is None:
            q_out = torch.empty((B, H, D), device=dev, dtype=q_proj.dtype)
        rc = capi.lib().santa_rope_append(
            q_proj.data_ptr(), k_proj.data_ptr(), v_proj.data_ptr(), qs, ks, vs, cos.data_ptr(), sin.data_ptr(),
            _dtype_code(q_proj), B, H, KVH, D, k_cache.data_ptr(), v_cache.data_ptr(), L_storage, pos_host,
            None if pos_dev is None else pos_dev.data_ptr(), q_out.data_ptr(),
            None if seq_lens_out is None else seq_lens_out.data_ptr(),
            None if status is None else status.data_ptr(), torch.cuda.current_stream(dev).cuda_stream)
        capi.check(rc)
    return q_out


def workspace_status(kind: str, device: torch.device) -> int:
    """Synchronise and read the status word of the scratch used on the current stream."""
    stream = torch.cuda.current_stream(device).cuda_stream
    key = (kind, device.index if device.index is not None else torch.cuda.current_device(), stream)
    ws = _workspaces.get(key)
    if ws is None:
        return 0
    torch.cuda.synchronize(device)
    return int(ws[:4].view(torch.int32).item())


@dataclass
class PropTrace:
    """Intermediates of one Prop call (parity tests)."""
    block_n: int
    T_c: int
    m_tiles: torch.Tensor    # [H,T_c] fp32
    ell_tiles: torch.Tensor  # [H,T_c] fp32
    u16: torch.Tensor        # [H,L] int16 view of storage bits
    counts: torch.Tensor     # [H,L] int16
    rowmask: torch.Tensor    # [KVH,L] int32
    S_tiles: torch.Tensor    # [H,T_c] int32
    invdelta: torch.Tensor   # [H,T_c] fp32
    a0: torch.Tensor         # [H,T_c] fp32


_PASS1_MODES = {"auto": 0, "gqa": 1, "perhead": 1, "vec": 2, "gqa_vec": 2}


def _pass1_mode_from_env() -> int:
    # santa_fused_proportional_tile_budgets/santa_cuda.cpp:39-51
    return _PASS1_MODES.get(os.environ.get("SANTA_PASS1", "").lower(), 0)


def prop_decode(q_h, K_g, V_g, S, seed=42, block_n=0, want_vrows=False, *, trace=False, flags=None,
                pass1_mode=None, score_mode=0):
    """S2ANTA-Prop decode of one sequence: ``q_h [H,D]``, ``K_g/V_g [L,KVH,D]``.
    Returns ``(out [H,D], m_star [H], vrows [KVH] or empty)`` (+ ``PropTrace``)."""
    # messages follow santa_fused_proportional_tile_budgets/santa_cuda.cpp:141-167
    _check(q_h.is_cuda, "q_h must be CUDA")
    _check(K_g.is_cuda and V_g.is_cuda, "K_g and V_g must be CUDA")
    _check(q_h.dtype in (torch.bfloat16, torch.float16), "q_h must be bf16 or f16")
    _check(K_g.dtype in (torch.bfloat16, torch.float16) and K_g.dtype == V_g.dtype,
           "K_g/V_g must be bf16 or f16 and match")
    _check(q_h.dtype == K_g.dtype, "q_h dtype must match K_g/V_g")
    _check(q_h.dim() == 2 and K_g.dim() == 3 and V_g.dim() == 3, "bad ranks")
    _check(q_h.device == K_g.device and q_h.device == V_g.device, "device mismatch")
    _check(K_g.shape == V_g.shape, "K_g and V_g must have the same shape")
    _check(q_h.size(1) == K_g.size(2), "D mismatch (q_h.size(1) vs K_g.size(2))")
    _check(q_h.size(0) % K_g.size(1) == 0, "H must be divisible by KVH (expected KVH == K_g.size(1) for NHD)")
    _check(K_g.is_contiguous() and V_g.is_contiguous(), "K_g/V_g must be contiguous with layout [L, KVH, D] (NHD)")
    if seed < 0:
        raise TypeError("seed must be a non-negative 64-bit integer")
    q = q_h.contiguous()
    H, D = q.shape
    L, KVH = K_g.size(0), K_g.size(1)
    mode = _pass1_mode_from_env() if pass1_mode is None else int(pass1_mode)
    # any GH and D % 16 == 0 like the reference (santa_cuda.cpp:212-247); its second pass launches
    # 128 x GH threads per block (santa_cuda_kernel.cu:924-927), which bounds GH by 8
    _check(H // KVH <= 8, f"This build supports up to 8 query heads per kv-head. Got GH={H // KVH}")
    _check(D <= 256, f"This build supports head dimensions up to 256. Got D={D}")
    bn = int(block_n)
    if bn <= 0:
        bn = 256 if mode == 2 else capi.block_n_rule(L, 0)
    _check(mode != 2 or (bn == 256 and H // KVH == 4 and D == 128),
           f"SANTA_PASS1=vec requires GH=4, D=128, block_n=256. Got GH={H // KVH} D={D} block_n={bn}")
    _check(D % 16 == 0 and bn % 16 == 0,
           f"Pass-1 WMMA-GQA requires D % 16 == 0 and block_n % 16 == 0. Got D={D} block_n={bn}")
    _check(bn <= 256, f"This build supports block_n up to 256. Got block_n={bn}")
    T_c = (L + bn - 1) // bn
    dev = q.device
    with torch.cuda.device(dev):
        lib = capi.lib()
        nbytes = lib.santa_prop_workspace_bytes(H, KVH, D, L, bn)
        ws = _workspace("prop", dev, nbytes)
        out = torch.empty((H, D), device=dev, dtype=q.dtype)
        m_star = torch.empty((H,), device=dev, dtype=torch.float32)
        vrows = torch.empty((KVH,) if want_vrows else (0,), device=dev, dtype=torch.int32)
        ext = capi.PropExt(pass1_mode=mode, flags=3 if flags is None else int(flags), score_mode=int(score_mode))
        tr = None
        if trace:
            f32 = dict(device=dev, dtype=torch.float32)
            tr = PropTrace(bn, T_c, torch.empty((H, T_c), **f32), torch.empty((H, T_c), **f32),
                           torch.zeros((H, L), device=dev, dtype=torch.int16),
                           torch.zeros((H, L), device=dev, dtype=torch.int16),
                           torch.zeros((KVH, L), device=dev, dtype=torch.int32),
                           torch.empty((H, T_c), device=dev, dtype=torch.int32),
                           torch.empty((H, T_c), **f32), torch.empty((H, T_c), **f32))
            ext.m_tiles, ext.ell_tiles, ext.u16 = tr.m_tiles.data_ptr(), tr.ell_tiles.data_ptr(), tr.u16.data_ptr()
            ext.counts, ext.rowmask = tr.counts.data_ptr(), tr.rowmask.data_ptr()
            ext.S_tiles, ext.invdelta, ext.a0 = tr.S_tiles.data_ptr(), tr.invdelta.data_ptr(), tr.a0.data_ptr()
        rc = lib.santa_prop_decode(
            q.data_ptr(), K_g.data_ptr(), V_g.data_ptr(), _dtype_code(q), H, KVH, D, L, int(S),
            int(seed) & (2**64 - 1), bn, out.data_ptr(), m_star.data_ptr(),
            vrows.data_ptr() if want_vrows else None, ws.data_ptr(), ws.numel(), C.byref(ext),
            torch.cuda.current_stream(dev).cuda_stream)
        capi.check(rc)
    res = (out, m_star, vrows)
    return res + (tr,) if trace else res


def prop_decode_ragged(q_bh, K_g, V_g, seq_lens, S, seed=42, want_vrows=False, *, max_len=None, trace=False,
                       flags=None, score_mode=0):
    """S2ANTA-Prop decode of a ragged batch in one launch sequence: ``q_bh [B,H,D]``,
    ``K_g/V_g [B,L_storage,KVH,D]``, ``seq_lens`` int32 ``[B]`` on the device (a CPU tensor or a
    list is copied there).  Sequence ``b`` gets the result of
    ``prop_decode(q_bh[b], K_g[b, :len_b], V_g[b, :len_b], S, seed, block_n=256)``.
    ``max_len`` bounds the lengths (default: the storage length) and sizes the scratch.
    Returns ``(out [B,H,D], m_star [B,H], vrows [B,KVH] or empty)`` (+ ``PropTrace`` with batched
    arrays ``[B,H,T_max]`` / ``[B,H,max_len]``)."""
    _check(q_bh.is_cuda and K_g.is_cuda and V_g.is_cuda, "q_bh, K_g and V_g must be CUDA")
    _check(q_bh.dtype in (torch.bfloat16, torch.float16), "q_bh must be bf16 or f16")
    _check(K_g.dtype == q_bh.dtype and V_g.dtype == q_bh.dtype, "q_bh dtype must match K_g/V_g")
    _check(q_bh.dim() == 3 and K_g.dim() == 4 and V_g.dim() == 4,
           "Ragged path expects q_bh [B,H,D], K_g/V_g [B,L,KVH,D]")
    _check(q_bh.device == K_g.device and q_bh.device == V_g.device, "device mismatch")
    _check(K_g.shape == V_g.shape, "K_g and V_g must have the same shape")
    _check(q_bh.size(0) == K_g.size(0), "Batch mismatch between q_bh and K_g/V_g")
    _check(q_bh.size(2) == K_g.size(3), "D mismatch (q_bh.size(2) vs K_g.size(3))")
    _check(K_g.is_contiguous() and V_g.is_contiguous(), "K_g/V_g must be contiguous with layout [B, L, KVH, D]")
    if seed < 0:
        raise TypeError("seed must be a non-negative 64-bit integer")
    q = q_bh.contiguous()
    B, H, D = q.shape
    L_storage, KVH = K_g.size(1), K_g.size(2)
    _check(D == 128 and H == 4 * KVH, f"This build supports only D=128 and GH=4 (H/KVH). Got D={D} H={H} KVH={KVH}")
    dev = q.device
    if not isinstance(seq_lens, torch.Tensor):
        seq_lens = torch.tensor(list(seq_lens), dtype=torch.int32)
    _check(seq_lens.numel() == B, "seq_lens must hold one length per sequence")
    lens = seq_lens.to(device=dev, dtype=torch.int32).contiguous()
    mlen = L_storage if max_len is None else int(max_len)
    _check(0 < mlen <= L_storage, f"max_len must be in (0, storage length]; got {mlen} (storage {L_storage})")
    T_max = (mlen + 255) // 256
    with torch.cuda.device(dev):
        lib = capi.lib()
        nbytes = lib.santa_prop_ragged_workspace_bytes(B, H, KVH, D, mlen)
        _check(nbytes > 0, "santa_b200: unsupported ragged problem (B must be 1..1024)")
        ws = _workspace("prop_ragged", dev, nbytes)
        out = torch.empty((B, H, D), device=dev, dtype=q.dtype)
        m_star = torch.empty((B, H), device=dev, dtype=torch.float32)
        vrows = torch.empty((B, KVH) if want_vrows else (0,), device=dev, dtype=torch.int32)
        ext = capi.PropExt(pass1_mode=0, flags=3 if flags is None else int(flags), score_mode=int(score_mode))
        tr = None
        if trace:
            f32 = dict(device=dev, dtype=torch.float32)
            tr = PropTrace(256, T_max, torch.zeros((B, H, T_max), **f32), torch.zeros((B, H, T_max), **f32),
                           torch.zeros((B, H, mlen), device=dev, dtype=torch.int16),
                           torch.zeros((B, H, mlen), device=dev, dtype=torch.int16),
                           torch.zeros((B, KVH, mlen), device=dev, dtype=torch.int32),
                           torch.zeros((B, H, T_max), device=dev, dtype=torch.int32),
                           torch.zeros((B, H, T_max), **f32), torch.zeros((B, H, T_max), **f32))
            ext.m_tiles, ext.ell_tiles, ext.u16 = tr.m_tiles.data_ptr(), tr.ell_tiles.data_ptr(), tr.u16.data_ptr()
            ext.counts, ext.rowmask = tr.counts.data_ptr(), tr.rowmask.data_ptr()
            ext.S_tiles, ext.invdelta, ext.a0 = tr.S_tiles.data_ptr(), tr.invdelta.data_ptr(), tr.a0.data_ptr()
        rc = lib.santa_prop_decode_ragged(
            q.data_ptr(), K_g.data_ptr(), V_g.data_ptr(), _dtype_code(q), B, H, KVH, D, L_storage,
            lens.data_ptr(), mlen, int(S), int(seed) & (2**64 - 1), out.data_ptr(), m_star.data_ptr(),
            vrows.data_ptr() if want_vrows else None, ws.data_ptr(), ws.numel(), C.byref(ext),
            torch.cuda.current_stream(dev).cuda_stream)
        capi.check(rc)
    res = (out, m_star, vrows)
    return res + (tr,) if trace else res


def lse_combine(partials: torch.Tensor, S_per_tile: int, dtype: torch.dtype):
    """Combine ``partials [G,B,H,130]`` (or ``[G,BH,130]``) fp32 into ``(out [B,H,128], m_star [B,H])``."""
    _check(partials.is_cuda and partials.dtype == torch.float32 and partials.is_contiguous(),
           "partials must be a contiguous CUDA fp32 tensor")
    G = partials.size(0)
    lead = tuple(partials.shape[1:-1])
    BH = 1
    for d in lead:
        BH *= d
    dev = partials.device
    with torch.cuda.device(dev):
        out = torch.empty(lead + (128,), device=dev, dtype=dtype)
        m_star = torch.empty(lead, device=dev, dtype=torch.float32)
        rc = capi.lib().santa_lse_combine(partials.data_ptr(), G, BH, 128, int(S_per_tile),
                                          capi.SANTA_DTYPE_BF16 if dtype == torch.bfloat16 else capi.SANTA_DTYPE_F16,
                                          out.data_ptr(), m_star.data_ptr(),
                                          torch.cuda.current_stream(dev).cuda_stream)
        capi.check(rc)
    return out, m_star
