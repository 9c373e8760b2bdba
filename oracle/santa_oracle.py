"""numpy front-end of the CPU oracle (``santa_oracle.c``).

TEST INFRASTRUCTURE ONLY: imported by ``tests/``, by the smoke test and by the
CPU-baseline leg of the benchmark.  The product path never imports it.

Arrays of 16-bit floats travel as ``uint16`` bit patterns so that bf16 and
fp16 share one code path; ``to16`` / ``from16`` convert.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from dataclasses import dataclass
from typing import Optional

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libsanta_oracle.so")


def build(force: bool = False) -> str:
    """Compile the C restatement with the Makefile beside it."""
    src = os.path.join(_HERE, "santa_oracle.c")
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(src):
        subprocess.check_call(["make", "-C", _HERE, "libsanta_oracle.so"], stdout=subprocess.DEVNULL)
    return _LIB_PATH


_lib = None


def lib() -> C.CDLL:
    global _lib
    if _lib is None:
        build()
        _lib = C.CDLL(_LIB_PATH)
        _lib.santa_or_u01.restype = C.c_float
        _lib.santa_or_u01.argtypes = [C.c_uint64, C.c_int, C.c_int]
        _lib.santa_or_block_n.restype = C.c_int
    return _lib


def _p(a: Optional[np.ndarray]):
    if a is None:
        return None
    assert a.flags["C_CONTIGUOUS"]
    return a.ctypes.data_as(C.c_void_p)


# ---------------------------------------------------------------- 16-bit helpers
def to16(x: np.ndarray, is_bf16: bool = True) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.float32)
    out = np.empty(x.shape, dtype=np.uint16)
    lib().santa_or_f32_to_16(_p(x), _p(out), C.c_long(x.size), C.c_int(int(is_bf16)))
    return out


def from16(x: np.ndarray, is_bf16: bool = True) -> np.ndarray:
    x = np.ascontiguousarray(x, dtype=np.uint16)
    out = np.empty(x.shape, dtype=np.float32)
    lib().santa_or_16_to_f32(_p(x), _p(out), C.c_long(x.size), C.c_int(int(is_bf16)))
    return out


# ---------------------------------------------------------------- host rules
def block_n_rule(L: int, block_n: int = 0) -> int:
    return int(lib().santa_or_block_n(C.c_int(L), C.c_int(block_n)))


def flash_budget(L: int, block_n: int, S: int):
    tc, spt = C.c_int(), C.c_int()
    lib().santa_or_flash_budget(C.c_int(L), C.c_int(block_n), C.c_long(S), C.byref(tc), C.byref(spt))
    return tc.value, spt.value


def u01(seed: int, h: int, t: int) -> np.float32:
    return np.float32(lib().santa_or_u01(C.c_uint64(seed & (2**64 - 1)), C.c_int(h), C.c_int(t)))


def q_scale(D: int) -> np.float32:
    return np.float32(1.0) / np.sqrt(np.float32(D))


# ---------------------------------------------------------------- stages
def scores_vec(q16, K16, is_bf16, L):
    """q16:[H,128] K16:[L_storage,KVH,128] -> scores [H,L] fp32 (vec order)."""
    H, D = q16.shape
    KVH = K16.shape[1]
    assert D == 128
    out = np.empty((H, L), dtype=np.float32)
    lib().santa_or_scores_vec(_p(q16), _p(K16), C.c_int(int(is_bf16)), C.c_int(H), C.c_int(KVH),
                              C.c_int(L), C.c_float(q_scale(D)), _p(out))
    return out


def scores_mma(q16, K16, is_bf16, L):
    H, D = q16.shape
    KVH = K16.shape[1]
    out = np.empty((H, L), dtype=np.float32)
    lib().santa_or_scores_mma(_p(q16), _p(K16), C.c_int(int(is_bf16)), C.c_int(H), C.c_int(KVH),
                              C.c_int(L), C.c_int(D), C.c_float(q_scale(D)), _p(out))
    return out


def tile_stats(scores, block_n, is_bf16, mma=False):
    H, L = scores.shape
    T_c = (L + block_n - 1) // block_n
    m = np.empty((H, T_c), np.float32)
    ell = np.empty((H, T_c), np.float32)
    u16 = np.zeros((H, L), np.uint16)
    fn = lib().santa_or_tile_stats_mma if mma else lib().santa_or_tile_stats_vec
    fn(_p(np.ascontiguousarray(scores)), C.c_int(H), C.c_int(L), C.c_int(block_n), C.c_int(int(is_bf16)),
       _p(m), _p(ell), _p(u16))
    return m, ell, u16


def flash_counts(u16, ell, is_bf16, block_n, S_per_tile, seed, rng_head0=0, tile0=0, invdel=None):
    H, L = u16.shape
    T_c = (L + block_n - 1) // block_n
    counts = np.zeros((H, L), np.int16)
    a0 = np.empty((H, T_c), np.float32)
    inv = np.empty((H, T_c), np.float32)
    lib().santa_or_flash_counts(_p(np.ascontiguousarray(u16)), _p(np.ascontiguousarray(ell, np.float32)),
                                C.c_int(int(is_bf16)), C.c_int(H), C.c_int(L), C.c_int(block_n),
                                C.c_int(S_per_tile), C.c_uint64(seed), C.c_int(rng_head0), C.c_int(tile0),
                                _p(None if invdel is None else np.ascontiguousarray(invdel, np.float32)),
                                _p(counts), _p(a0), _p(inv))
    return counts, a0, inv


def prop_counts(u16, is_bf16, block_n, invdelta, a0):
    H, L = u16.shape
    counts = np.zeros((H, L), np.int16)
    lib().santa_or_prop_counts(_p(np.ascontiguousarray(u16)), C.c_int(int(is_bf16)), C.c_int(H), C.c_int(L),
                               C.c_int(block_n), _p(np.ascontiguousarray(invdelta, np.float32)),
                               _p(np.ascontiguousarray(a0, np.float32)), _p(counts))
    return counts


def rowflags(counts, KVH):
    H, L = counts.shape
    flags = np.empty((KVH, L), np.uint8)
    vrows = np.empty((KVH,), np.int32)
    lib().santa_or_rowflags(_p(np.ascontiguousarray(counts)), C.c_int(H), C.c_int(KVH), C.c_int(L),
                            _p(flags), _p(vrows))
    return flags, vrows


def flash_estimate(counts, V16, is_bf16, block_n, S_per_tile, m_tiles, ell_tiles):
    H, L = counts.shape
    KVH = V16.shape[1]
    out = np.empty((H, 128), np.float32)
    out16 = np.empty((H, 128), np.uint16)
    m_star = np.empty((H,), np.float32)
    lib().santa_or_flash_estimate(_p(np.ascontiguousarray(counts)), _p(V16), C.c_int(int(is_bf16)),
                                  C.c_int(H), C.c_int(KVH), C.c_int(L), C.c_int(block_n),
                                  C.c_int(S_per_tile), _p(np.ascontiguousarray(m_tiles, np.float32)),
                                  _p(np.ascontiguousarray(ell_tiles, np.float32)), _p(out), _p(out16),
                                  _p(m_star))
    return out, out16, m_star


def prop_estimate(counts, V16, is_bf16, block_n, S):
    H, L = counts.shape
    KVH, D = V16.shape[1], V16.shape[2]
    out = np.empty((H, D), np.float32)
    out16 = np.empty((H, D), np.uint16)
    lib().santa_or_prop_estimate(_p(np.ascontiguousarray(counts)), _p(V16), C.c_int(int(is_bf16)),
                                 C.c_int(H), C.c_int(KVH), C.c_int(L), C.c_int(D), C.c_int(block_n),
                                 C.c_long(S), _p(out), _p(out16))
    return out, out16


def prop_budgets(m_tiles, ell_tiles, S, seed, flags=0, W=None):
    H, T_c = m_tiles.shape
    m_star = np.empty((H,), np.float32)
    S_tiles = np.empty((H, T_c), np.int32)
    invdelta = np.empty((H, T_c), np.float32)
    a0 = np.empty((H, T_c), np.float32)
    W_out = np.empty((H, T_c), np.float32)
    lib().santa_or_prop_budgets(_p(np.ascontiguousarray(m_tiles, np.float32)),
                                _p(np.ascontiguousarray(ell_tiles, np.float32)), C.c_int(H), C.c_int(T_c),
                                C.c_long(S), C.c_uint64(seed), C.c_int(flags),
                                _p(None if W is None else np.ascontiguousarray(W, np.float32)),
                                _p(m_star), _p(S_tiles), _p(invdelta), _p(a0), _p(W_out))
    return m_star, S_tiles, invdelta, a0, W_out


def merge_partials(part, S_per_tile):
    G, H, W = part.shape
    D = W - 2
    out = np.empty((H, D), np.float32)
    m_star = np.empty((H,), np.float32)
    lib().santa_or_merge_partials(_p(np.ascontiguousarray(part, np.float32)), C.c_int(G), C.c_int(H),
                                  C.c_int(D), C.c_int(S_per_tile), _p(out), _p(m_star))
    return out, m_star


# ---------------------------------------------------------------- whole decodes
@dataclass
class FlashResult:
    block_n: int
    T_c: int
    S_per_tile: int
    scores: np.ndarray     # [B,H,L]
    m_tiles: np.ndarray    # [B,H,T_c]
    ell_tiles: np.ndarray  # [B,H,T_c]
    u16: np.ndarray        # [B,H,L]
    counts: np.ndarray     # [B,H,L] int16
    vrows: np.ndarray      # [B,KVH]
    out: np.ndarray        # [B,H,128] fp32
    out16: np.ndarray      # [B,H,128] storage bits
    m_star: np.ndarray     # [B,H]


def flash_decode(q16, K16, V16, S, seed=42, block_n=0, valid_len=-1, is_bf16=True,
                 batch_offset=0, tile_offset=0, S_per_tile=None,
                 inject_u16=None, inject_ell=None, inject_invdel=None, inject_m=None) -> FlashResult:
    """Whole Flash decode, F.cpp:174-343 over the stages above.

    q16:[B,H,128]  K16,V16:[B,L_storage,KVH,128] (uint16 bit patterns).
    ``inject_*`` ([B,H,L] / [B,H,T_c]) replace the modelled hardware-approximate
    intermediates with values dumped by a GPU run.
    """
    B, H, D = q16.shape
    L_storage, KVH = K16.shape[1], K16.shape[2]
    L = valid_len if valid_len > 0 else L_storage
    assert 0 < L <= L_storage
    bn = block_n_rule(L, block_n)
    T_c, spt = flash_budget(L, bn, S)
    if S_per_tile is not None:
        spt = S_per_tile
    R = dict(scores=[], m=[], ell=[], u16=[], counts=[], vrows=[], out=[], out16=[], m_star=[])
    for b in range(B):
        sc = scores_vec(q16[b], K16[b], is_bf16, L)
        m, ell, u = tile_stats(sc, bn, is_bf16)
        if inject_m is not None:
            m = np.ascontiguousarray(inject_m[b])
        if inject_u16 is not None:
            u = np.ascontiguousarray(inject_u16[b])
        if inject_ell is not None:
            ell = np.ascontiguousarray(inject_ell[b])
        cnt, _, _ = flash_counts(u, ell, is_bf16, bn, spt, seed, rng_head0=(batch_offset + b) * H,
                                 tile0=tile_offset,
                                 invdel=None if inject_invdel is None else inject_invdel[b])
        _, vr = rowflags(cnt, KVH)
        out, out16, ms = flash_estimate(cnt, V16[b], is_bf16, bn, spt, m, ell)
        for k, v in zip(R.keys(), (sc, m, ell, u, cnt, vr, out, out16, ms)):
            R[k].append(v)
    S_ = {k: np.stack(v) for k, v in R.items()}
    return FlashResult(bn, T_c, spt, S_["scores"], S_["m"], S_["ell"], S_["u16"], S_["counts"],
                       S_["vrows"], S_["out"], S_["out16"], S_["m_star"])


@dataclass
class PropResult:
    block_n: int
    T_c: int
    scores: np.ndarray
    m_tiles: np.ndarray
    ell_tiles: np.ndarray
    u16: np.ndarray
    m_star: np.ndarray
    S_tiles: np.ndarray
    invdelta: np.ndarray
    a0: np.ndarray
    counts: np.ndarray
    vrows: np.ndarray
    out: np.ndarray
    out16: np.ndarray


def prop_uses_vec(H, KVH, D, bn):
    """P.cpp:212-229: the vec score path applies iff GH==4, D==128, block_n==256."""
    return (H // KVH == 4) and D == 128 and bn == 256


def prop_decode(q16, K16, V16, S, seed=42, block_n=0, is_bf16=True, flags=0,
                inject_u16=None, inject_ell=None, inject_m=None) -> PropResult:
    """Whole Prop decode for one sequence, P.cpp:270-352.

    q16:[H,D]  K16,V16:[L,KVH,D]."""
    H, D = q16.shape
    L, KVH = K16.shape[0], K16.shape[1]
    bn = block_n_rule(L, block_n)
    T_c = (L + bn - 1) // bn
    vec = prop_uses_vec(H, KVH, D, bn)
    sc = scores_vec(q16, K16, is_bf16, L) if vec else scores_mma(q16, K16, is_bf16, L)
    m, ell, u = tile_stats(sc, bn, is_bf16, mma=not vec)
    if inject_m is not None:
        m = np.ascontiguousarray(inject_m)
    if inject_u16 is not None:
        u = np.ascontiguousarray(inject_u16)
    if inject_ell is not None:
        ell = np.ascontiguousarray(inject_ell)
    m_star, S_tiles, invdelta, a0, _ = prop_budgets(m, ell, S, seed, flags)
    cnt = prop_counts(u, is_bf16, bn, invdelta, a0)
    _, vr = rowflags(cnt, KVH)
    out, out16 = prop_estimate(cnt, V16, is_bf16, bn, S)
    return PropResult(bn, T_c, sc, m, ell, u, m_star, S_tiles, invdelta, a0, cnt, vr, out, out16)


# ---------------------------------------------------------------- fp32 evaluations over given counts
def flash_eval_over_counts(counts, V_f32, m_tiles, ell_tiles, block_n, S_per_tile):
    """fp64 evaluation of the Flash estimator identity over a given count table:
    out[h] = sum_t w_t (sum_r c[h,r] V[r]) / (Z * S_per_tile), w_t = exp(m_t-m*) ell_t.
    counts:[H,L]  V_f32:[L,KVH,D]  -> [H,D] float64."""
    H, L = counts.shape
    KVH, D = V_f32.shape[1], V_f32.shape[2]
    GH = H // KVH
    T_c = m_tiles.shape[1]
    out = np.zeros((H, D), np.float64)
    for h in range(H):
        ms = m_tiles[h].max()
        w = np.exp(m_tiles[h].astype(np.float64) - float(ms)) * ell_tiles[h].astype(np.float64)
        Z = w.sum()
        wrow = np.repeat(w, block_n)[:L]
        c = counts[h].astype(np.float64) * wrow
        nz = np.nonzero(c)[0]
        if S_per_tile > 0 and Z > 0 and nz.size:
            out[h] = (c[nz, None] * V_f32[nz, h // GH, :].astype(np.float64)).sum(0) / (Z * S_per_tile)
    return out


def prop_eval_over_counts(counts, V_f32, S):
    H, L = counts.shape
    KVH, D = V_f32.shape[1], V_f32.shape[2]
    GH = H // KVH
    out = np.zeros((H, D), np.float64)
    if S <= 0:
        return out
    for h in range(H):
        nz = np.nonzero(counts[h])[0]
        if nz.size:
            out[h] = (counts[h, nz, None].astype(np.float64) * V_f32[nz, h // GH, :].astype(np.float64)).sum(0) / S
    return out
