"""ctypes view of ``libsanta_b200.so`` (the C ABI declared in ``include/santa_b200.h``).

The library is the only compute path: importing this module fails loudly when
the shared object is missing, and nothing here falls back to PyTorch or CPU
arithmetic.
"""
from __future__ import annotations

import ctypes as C
import os

_PKG = os.path.dirname(os.path.abspath(__file__))
# SANTA_B200_LIB selects another build of the same library, e.g. the bounds-checked one
# (`python -m santa_b200._build --checks` -> lib/libsanta_b200_checks.so)
LIB_PATH = os.environ.get("SANTA_B200_LIB") or os.path.join(_PKG, "lib", "libsanta_b200.so")

SANTA_DTYPE_BF16 = 0
SANTA_DTYPE_F16 = 1
SANTA_PEER_COMBINE = 1
SANTA_SCORE_EXACT = 0
SANTA_SCORE_TENSOR = 1


class SantaError(RuntimeError):
    """A C-ABI call returned a negative status."""

    def __init__(self, code: int, text: str) -> None:
        super().__init__(f"santa_b200: {text} (code {code})")
        self.code = code


class PeerExchange(C.Structure):
    """``santa_peer_exchange`` of include/santa_b200.h."""

    _fields_ = [
        ("world", C.c_int),
        ("rank", C.c_int),
        ("epoch", C.c_uint32),
        ("flags", C.c_uint32),
        ("peer_buffer", C.c_void_p * 16),
    ]


class FlashExt(C.Structure):
    """``santa_flash_ext`` of include/santa_b200.h."""

    _fields_ = [
        ("batch_offset", C.c_int),
        ("tile_offset", C.c_int),
        ("s_per_tile_override", C.c_int),
        ("score_mode", C.c_int),
        ("partial_out", C.c_void_p),
        ("m_tiles", C.c_void_p),
        ("ell_tiles", C.c_void_p),
        ("u16", C.c_void_p),
        ("counts", C.c_void_p),
        ("rowmask", C.c_void_p),
        ("invdel", C.c_void_p),
        ("peer", C.POINTER(PeerExchange)),
    ]


class PropExt(C.Structure):
    """``santa_prop_ext`` of include/santa_b200.h."""

    _fields_ = [
        ("pass1_mode", C.c_int),
        ("flags", C.c_int),
        ("m_tiles", C.c_void_p),
        ("ell_tiles", C.c_void_p),
        ("u16", C.c_void_p),
        ("counts", C.c_void_p),
        ("rowmask", C.c_void_p),
        ("S_tiles", C.c_void_p),
        ("invdelta", C.c_void_p),
        ("a0", C.c_void_p),
        ("score_mode", C.c_int),
        ("reserved", C.c_int),
    ]


_lib = None

# every symbol include/santa_b200.h declares
EXPORTS = (
    "santa_strerror",
    "santa_last_cuda_error",
    "santa_abi_version",
    "santa_block_n_rule",
    "santa_flash_budget",
    "santa_u01",
    "santa_flash_workspace_bytes",
    "santa_flash_decode",
    "santa_workspace_status",
    "santa_prop_workspace_bytes",
    "santa_prop_decode",
    "santa_lse_combine",
    "santa_flash_decode_noalloc",
    "santa_noalloc_status",
    "santa_peer_exchange_status",
    "santa_prop_ragged_workspace_bytes",
    "santa_prop_decode_ragged",
    "santa_flash_ragged_workspace_bytes",
    "santa_flash_decode_ragged",
    "santa_rope_append",
    "santa_peer_exchange_bytes",
    "santa_lse_combine_wait",
)


def lib() -> C.CDLL:
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} is missing: build it with `python -m santa_b200._build` "
            "(there is no fallback implementation)"
        )
    L = C.CDLL(LIB_PATH)
    L.santa_strerror.restype = C.c_char_p
    L.santa_strerror.argtypes = [C.c_int]
    L.santa_block_n_rule.restype = C.c_int
    L.santa_block_n_rule.argtypes = [C.c_int, C.c_int]
    L.santa_flash_budget.restype = None
    L.santa_flash_budget.argtypes = [C.c_int, C.c_int, C.c_int64, C.POINTER(C.c_int), C.POINTER(C.c_int)]
    L.santa_u01.restype = C.c_float
    L.santa_u01.argtypes = [C.c_uint64, C.c_int, C.c_int]
    L.santa_flash_workspace_bytes.restype = C.c_size_t
    L.santa_flash_workspace_bytes.argtypes = [C.c_int] * 4
    L.santa_flash_decode.restype = C.c_int
    L.santa_flash_decode.argtypes = [
        C.c_void_p, C.c_void_p, C.c_void_p, C.c_int,  # q K V dtype
        C.c_int, C.c_int, C.c_int, C.c_int,  # B H KVH D
        C.c_int, C.c_int, C.c_int64, C.c_uint64, C.c_int,  # L_valid L_storage S seed block_n
        C.c_void_p, C.c_void_p, C.c_void_p,  # out m_star vrows
        C.c_void_p, C.c_size_t, C.POINTER(FlashExt), C.c_void_p,  # workspace bytes ext stream
    ]
    L.santa_workspace_status.restype = C.c_void_p
    L.santa_workspace_status.argtypes = [C.c_void_p]
    if hasattr(L, "santa_prop_decode"):
        L.santa_prop_workspace_bytes.restype = C.c_size_t
        L.santa_prop_workspace_bytes.argtypes = [C.c_int] * 5
        L.santa_prop_decode.restype = C.c_int
        L.santa_prop_decode.argtypes = [
            C.c_void_p, C.c_void_p, C.c_void_p, C.c_int,  # q K V dtype
            C.c_int, C.c_int, C.c_int, C.c_int,  # H KVH D L
            C.c_int64, C.c_uint64, C.c_int,  # S seed block_n
            C.c_void_p, C.c_void_p, C.c_void_p,  # out m_star vrows
            C.c_void_p, C.c_size_t, C.POINTER(PropExt), C.c_void_p,
        ]
    if hasattr(L, "santa_lse_combine_wait"):
        L.santa_peer_exchange_bytes.restype = C.c_size_t
        L.santa_peer_exchange_bytes.argtypes = [C.c_int, C.c_int]
        L.santa_lse_combine_wait.restype = C.c_int
        L.santa_lse_combine_wait.argtypes = [
            C.POINTER(PeerExchange), C.c_int, C.c_int, C.c_int, C.c_int,  # px BH D S_per_tile dtype
            C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,  # out m_star status stream
        ]
    if hasattr(L, "santa_rope_append"):
        L.santa_rope_append.restype = C.c_int
        L.santa_rope_append.argtypes = [
            C.c_void_p, C.c_void_p, C.c_void_p, C.c_int64, C.c_int64, C.c_int64,  # q k v and their strides
            C.c_void_p, C.c_void_p, C.c_int,  # cos sin dtype
            C.c_int, C.c_int, C.c_int, C.c_int,  # B H KVH D
            C.c_void_p, C.c_void_p, C.c_int, C.c_int, C.c_void_p,  # k_cache v_cache L_storage pos pos_dev
            C.c_void_p, C.c_void_p, C.c_void_p, C.c_void_p,  # q_out seq_lens_out status stream
        ]
    if hasattr(L, "santa_flash_decode_ragged"):
        L.santa_flash_ragged_workspace_bytes.restype = C.c_size_t
        L.santa_flash_ragged_workspace_bytes.argtypes = [C.c_int] * 4
        L.santa_flash_decode_ragged.restype = C.c_int
        L.santa_flash_decode_ragged.argtypes = [
            C.c_void_p, C.c_void_p, C.c_void_p, C.c_int,  # q K V dtype
            C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,  # B H KVH D L_storage
            C.c_void_p, C.c_int, C.c_int64, C.c_uint64, C.c_int,  # seq_lens max_len S seed block_n
            C.c_void_p, C.c_void_p, C.c_void_p,  # out m_star vrows
            C.c_void_p, C.c_size_t, C.POINTER(FlashExt), C.c_void_p,
        ]
    if hasattr(L, "santa_prop_decode_ragged"):
        L.santa_prop_ragged_workspace_bytes.restype = C.c_size_t
        L.santa_prop_ragged_workspace_bytes.argtypes = [C.c_int] * 5
        L.santa_prop_decode_ragged.restype = C.c_int
        L.santa_prop_decode_ragged.argtypes = [
            C.c_void_p, C.c_void_p, C.c_void_p, C.c_int,  # q K V dtype
            C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,  # B H KVH D L_storage
            C.c_void_p, C.c_int, C.c_int64, C.c_uint64,  # seq_lens max_len S seed
            C.c_void_p, C.c_void_p, C.c_void_p,  # out m_star vrows
            C.c_void_p, C.c_size_t, C.POINTER(PropExt), C.c_void_p,
        ]
    if hasattr(L, "santa_flash_decode_noalloc"):
        L.santa_flash_decode_noalloc.restype = C.c_int
        L.santa_flash_decode_noalloc.argtypes = L.santa_flash_decode.argtypes[:16] + [C.POINTER(FlashExt), C.c_void_p]
    if hasattr(L, "santa_noalloc_status"):
        L.santa_noalloc_status.restype = C.c_void_p
        L.santa_noalloc_status.argtypes = []
    if hasattr(L, "santa_peer_exchange_status"):
        L.santa_peer_exchange_status.restype = C.c_void_p
        L.santa_peer_exchange_status.argtypes = [C.c_void_p]
    if hasattr(L, "santa_lse_combine"):
        L.santa_lse_combine.restype = C.c_int
        L.santa_lse_combine.argtypes = [
            C.c_void_p, C.c_int, C.c_int, C.c_int, C.c_int, C.c_int,  # partials G BH D S_per_tile dtype
            C.c_void_p, C.c_void_p, C.c_void_p,  # out m_star stream
        ]
    _lib = L
    return L


def check(code: int) -> None:
    if code != 0:
        raise SantaError(code, lib().santa_strerror(code).decode())


def block_n_rule(L: int, block_n: int = 0) -> int:
    return int(lib().santa_block_n_rule(L, block_n))


def flash_budget(L: int, block_n: int, S: int):
    tc, spt = C.c_int(), C.c_int()
    lib().santa_flash_budget(L, block_n, S, C.byref(tc), C.byref(spt))
    return tc.value, spt.value


def u01(seed: int, h: int, t: int) -> float:
    return float(lib().santa_u01(seed & (2**64 - 1), h, t))
