"""Drive the REFERENCE's own CUDA kernels (compiled unmodified into
``oracle/_ref/*.so`` by ``make -C oracle ref``) through their ``extern "C"``
launchers, in the order the reference's host glue launches them.

TEST INFRASTRUCTURE ONLY.  Used by the GPU parity tests (bit-exact sampled
counts against the reference binary), by the script that generates the golden
fixtures, and by the benchmark's reference arm.  The product never imports it.

The launch sequences restate
  flash_style_fused_santa_fixed_tile_budgets/santa_cuda.cpp:174-343  (Flash)
  santa_fused_proportional_tile_budgets/santa_cuda.cpp:170-352        (Prop)
and, unlike the reference's Python entry points, hand back the workspace
tensors (m_tiles, ell_tiles, out_tiles, rowmask, u_stash, S_tiles, ...) that
the reference keeps internal.
"""
from __future__ import annotations

import ctypes as C
import math
import os
from types import SimpleNamespace

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
FLASH_SO = os.path.join(_HERE, "_ref", "libsanta_ref_flash.so")
PROP_SO = os.path.join(_HERE, "_ref", "libsanta_ref_prop.so")

_flash = None
_prop = None


def available() -> bool:
    return os.path.exists(FLASH_SO) and os.path.exists(PROP_SO)


def _vp(t):
    return C.c_void_p(t.data_ptr()) if t is not None else C.c_void_p(0)


def flash_lib():
    global _flash
    if _flash is None:
        _flash = C.CDLL(FLASH_SO, mode=os.RTLD_LOCAL)
    return _flash


def prop_lib():
    global _prop
    if _prop is None:
        _prop = C.CDLL(PROP_SO, mode=os.RTLD_LOCAL)
    return _prop


def _block_n(L, block_n):
    if block_n > 0:
        return block_n
    return 32 if L <= 1536 else (64 if L <= 3072 else 256)


def flash_decode(q, K, V, S, seed=42, block_n=0, want_vrows=False, valid_len=-1):
    """q:[B,H,128] K,V:[B,L_storage,KVH,128] (bf16/f16, CUDA).  Returns a namespace
    with out, m_star, vrows and the reference's workspaces."""
    lib = flash_lib()
    B, H, D = q.shape
    L_storage, KVH = K.shape[1], K.shape[2]
    L = valid_len if valid_len > 0 else L_storage
    bn = _block_n(L, block_n)
    T_c = (L + bn - 1) // bn
    spt = max(1, S // T_c) if S > 0 else 0
    dev = q.device
    f32 = dict(device=dev, dtype=torch.float32)
    m_tiles = torch.empty(B, H, T_c, **f32)
    ell_tiles = torch.empty(B, H, T_c, **f32)
    out_tiles = torch.empty(B, H, T_c, D, **f32)
    rowmask = torch.zeros(B, KVH, L, device=dev, dtype=torch.int32) if want_vrows else None
    sfx = "bf16" if q.dtype == torch.bfloat16 else "f16"
    stream = C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    q_scale = 1.0 / math.sqrt(float(D))
    fused = getattr(lib, f"launch_fused_tiles_vec_gqa_gh4_d128_bn{bn}_{sfx}")
    fused(_vp(q), _vp(K), _vp(V), C.c_int(B), C.c_int(H), C.c_int(KVH), C.c_int(L), C.c_int(L_storage),
          C.c_int(T_c), C.c_float(q_scale), C.c_int(spt), C.c_uint64(seed), _vp(m_tiles), _vp(ell_tiles),
          _vp(out_tiles), _vp(rowmask), stream)
    out = torch.empty(B, H, D, device=dev, dtype=q.dtype)
    m_star = torch.empty(B, H, **f32)
    fin = getattr(lib, f"launch_finalize_weighted_{sfx}")
    fin(_vp(m_tiles), _vp(ell_tiles), _vp(out_tiles), C.c_int(B), C.c_int(H), C.c_int(T_c), C.c_int(D),
        C.c_int(spt), _vp(out), _vp(m_star), stream)
    vrows = torch.empty(0, device=dev, dtype=torch.int32)
    if want_vrows:
        vrows = torch.empty(B, KVH, device=dev, dtype=torch.int32)
        lib.launch_reduce_vrows(_vp(rowmask), C.c_int(B), C.c_int(KVH), C.c_int(L), _vp(vrows), stream)
    return SimpleNamespace(out=out, m_star=m_star, vrows=vrows, m_tiles=m_tiles, ell_tiles=ell_tiles,
                           out_tiles=out_tiles, rowmask=rowmask, block_n=bn, T_c=T_c, S_per_tile=spt)


def probe_values(L, KVH, dtype, device, block_n):
    """A V tensor [1,L,KVH,128] that makes out_tiles spell out the sampled counts:
    row r of a tile contributes weight 1 (r%256 < 128) or 1024 (r%256 >= 128) on
    dim r%128, so out_tiles[..., d] = c[d] + 1024*c[d+128] exactly in fp32 for
    counts below 1024 (for block_n <= 128 only the weight-1 half is used)."""
    n = torch.arange(L, device=device)
    r = n % block_n
    V = torch.zeros(L, 128, device=device, dtype=torch.float32)
    V[n, r % 128] = torch.where((r % 256) < 128, 1.0, 1024.0).to(torch.float32)
    return V[None, :, None, :].expand(1, L, KVH, 128).to(dtype).contiguous()


def flash_counts(q, K, S, seed=42, block_n=0, valid_len=-1):
    """Sampled row counts [B,H,L] (int32) of the reference Flash kernel, recovered
    from out_tiles with the probe V above (no change to the reference code)."""
    B, H, D = q.shape
    L_storage, KVH = K.shape[1], K.shape[2]
    L = valid_len if valid_len > 0 else L_storage
    bn = _block_n(L, block_n)
    Vp = probe_values(L_storage, KVH, q.dtype, q.device, bn).expand(B, -1, -1, -1).contiguous()
    r = flash_decode(q, K, Vp, S, seed=seed, block_n=block_n, want_vrows=True, valid_len=valid_len)
    ot = r.out_tiles.round().to(torch.int64)  # [B,H,T_c,128]
    T_c = r.T_c
    if bn == 256:
        lo, hi = ot % 1024, ot // 1024
        counts = torch.cat([lo, hi], dim=-1).reshape(B, H, T_c * 256)[:, :, :L]
    else:
        counts = ot[..., :bn].reshape(B, H, T_c * bn)[:, :, :L]
    return counts.to(torch.int32), r


def prop_decode(q, K, V, S, seed=42, block_n=0, want_vrows=False, pass1_mode="auto"):
    """q:[H,D] K,V:[L,KVH,D].  Returns a namespace with out, m_star, vrows and the
    reference's workspaces (m_tiles, ell_tiles, u_stash, S_tiles, invdelta, a0, out_fp32)."""
    lib = prop_lib()
    H, D = q.shape
    L, KVH = K.shape[0], K.shape[1]
    GH = H // KVH
    if block_n <= 0 and pass1_mode == "vec":
        bn = 256
    else:
        bn = _block_n(L, block_n)
    T_c = (L + bn - 1) // bn
    dev = q.device
    f32 = dict(device=dev, dtype=torch.float32)
    sfx = "bf16" if q.dtype == torch.bfloat16 else "f16"
    stream = C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    m_tiles = torch.empty(H, T_c, **f32)
    ell_tiles = torch.empty(H, T_c, **f32)
    m_star = torch.empty(H, **f32)
    u_stash = torch.zeros(L, H, device=dev, dtype=q.dtype)
    can_vec = GH == 4 and D == 128 and bn == 256
    use_vec = (pass1_mode == "auto" and can_vec) or pass1_mode == "vec"
    scale = 1.0 / math.sqrt(float(D))
    p1 = getattr(lib, f"launch_pass1_tiles_{'vec' if use_vec else 'wmma'}_gqa_{sfx}")
    p1(_vp(q), _vp(K), C.c_int(H), C.c_int(KVH), C.c_int(L), C.c_int(D), C.c_int(bn), C.c_int(T_c),
       C.c_float(scale), _vp(m_tiles), _vp(ell_tiles), _vp(u_stash), stream)
    S_tiles = torch.empty(H, T_c, device=dev, dtype=torch.int32)
    invdelta = torch.empty(H, T_c, **f32)
    a0 = torch.empty(H, T_c, **f32)
    lib.launch_tile_budgets(_vp(m_tiles), _vp(ell_tiles), _vp(m_star), C.c_int(H), C.c_int(T_c), C.c_int(int(S)),
                            C.c_uint64(seed), _vp(S_tiles), _vp(invdelta), _vp(a0), stream)
    out_fp32 = torch.zeros(H, D, **f32)
    rowmask = torch.zeros(KVH, L, device=dev, dtype=torch.int32) if want_vrows else None
    p2 = getattr(lib, f"launch_pass2_grouped_fused_atomic_{sfx}")
    p2(_vp(V), _vp(u_stash), C.c_int(H), C.c_int(KVH), C.c_int(L), C.c_int(D), C.c_int(bn), C.c_int(T_c),
       _vp(invdelta), _vp(a0), _vp(S_tiles), _vp(out_fp32), _vp(rowmask), stream)
    out = torch.empty(H, D, device=dev, dtype=q.dtype)
    scale_out = (1.0 / float(S)) if S > 0 else 0.0
    getattr(lib, f"launch_cast_scale_out_{sfx}")(_vp(out_fp32), _vp(out), C.c_int(H), C.c_int(D),
                                                  C.c_float(scale_out), stream)
    vrows = torch.empty(0, device=dev, dtype=torch.int32)
    if want_vrows:
        vrows = torch.empty(KVH, device=dev, dtype=torch.int32)
        lib.launch_reduce_vrows(_vp(rowmask), C.c_int(KVH), C.c_int(L), _vp(vrows), stream)
    return SimpleNamespace(out=out, m_star=m_star, vrows=vrows, m_tiles=m_tiles, ell_tiles=ell_tiles,
                           u_stash=u_stash, S_tiles=S_tiles, invdelta=invdelta, a0=a0, out_fp32=out_fp32,
                           rowmask=rowmask, block_n=bn, T_c=T_c)


def prop_counts(q, K, S, seed=42, block_n=0):
    """Sampled row counts [H,L] of the reference Prop pipeline, one pass-2 launch
    per tile with a probe V that is non-zero only inside that tile."""
    H, D = q.shape
    L, KVH = K.shape[0], K.shape[1]
    base = prop_decode(q, K, torch.zeros_like(K), S, seed=seed, block_n=block_n, want_vrows=True)
    bn, T_c = base.block_n, base.T_c
    lib = prop_lib()
    sfx = "bf16" if q.dtype == torch.bfloat16 else "f16"
    stream = C.c_void_p(torch.cuda.current_stream(q.device).cuda_stream)
    counts = torch.zeros(H, L, device=q.device, dtype=torch.int32)
    p2 = getattr(lib, f"launch_pass2_grouped_fused_atomic_{sfx}")
    for t in range(T_c):
        n0, n1 = t * bn, min(L, (t + 1) * bn)
        for half in range((n1 - n0 + D - 1) // D):          # D rows at a time: one output dim per row
            a, b = n0 + D * half, min(n1, n0 + D * (half + 1))
            Vp = torch.zeros(L, KVH, D, device=q.device, dtype=q.dtype)
            idx = torch.arange(a, b, device=q.device)
            Vp[idx, :, idx - a] = 1.0
            out_fp32 = torch.zeros(H, D, device=q.device, dtype=torch.float32)
            p2(_vp(Vp), _vp(base.u_stash), C.c_int(H), C.c_int(KVH), C.c_int(L), C.c_int(D), C.c_int(bn),
               C.c_int(T_c), _vp(base.invdelta), _vp(base.a0), _vp(base.S_tiles), _vp(out_fp32), _vp(None),
               stream)
            counts[:, a:b] = out_fp32[:, : b - a].round().to(torch.int32)
    return counts, base
