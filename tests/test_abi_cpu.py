"""The C-ABI library loads without a GPU and exports every symbol include/santa_b200.h declares;
its host-side rules agree with the oracle; the host mirrors reject bad input like the reference."""
import ctypes
import os
import re

import numpy as np
import pytest
import torch

from oracle import santa_oracle as so
from santa_b200 import capi, ops

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, "include", "santa_b200.h")).read()
    return sorted(set(re.findall(r"SANTA_API[^;(]*?\b(santa_\w+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = ctypes.CDLL(capi.LIB_PATH)
    syms = declared_symbols()
    assert len(syms) >= 9
    for s in syms:
        assert hasattr(lib, s), f"{s} is declared in santa_b200.h but not exported"
    assert sorted(capi.EXPORTS) == syms


def test_host_rules_match_oracle():
    for L in (1, 16, 1536, 1537, 3072, 3073, 4096, 32768, 32769, 524288):
        for bn in (0, 32, 64, 256):
            assert capi.block_n_rule(L, bn) == so.block_n_rule(L, bn)
        bn = capi.block_n_rule(L)
        for S in (0, 1, 32, 256, 2048):
            assert capi.flash_budget(L, bn, S) == so.flash_budget(L, bn, S)
    rng = np.random.default_rng(2)
    for _ in range(100):
        seed, h, t = int(rng.integers(0, 2**62)), int(rng.integers(0, 1024)), int(rng.integers(0, 1 << 16))
        assert np.float32(capi.u01(seed, h, t)) == so.u01(seed, h, t)


def test_strerror_and_version():
    lib = capi.lib()
    assert lib.santa_abi_version() >= 1
    assert b"block_n" in lib.santa_strerror(-4)
    assert lib.santa_strerror(0) == b"ok"


def test_argument_validation_needs_no_gpu():
    """Bad arguments are rejected before any CUDA call."""
    lib = capi.lib()
    rc = lib.santa_flash_decode(None, None, None, 0, 1, 32, 8, 128, 16, 16, 4, 1, 0, None, None, None, None, 0, None, None)
    assert rc == -8
    rc = lib.santa_flash_decode(256, 256, 256, 7, 1, 32, 8, 128, 16, 16, 4, 1, 0, 256, 256, None, None, 0, None, None)
    assert rc == -1
    rc = lib.santa_flash_decode(256, 256, 256, 0, 1, 32, 8, 64, 16, 16, 4, 1, 0, 256, 256, None, None, 0, None, None)
    assert rc == -2
    rc = lib.santa_flash_decode(256, 256, 256, 0, 1, 32, 8, 128, 17, 16, 4, 1, 0, 256, 256, None, None, 0, None, None)
    assert rc == -3


def test_host_mirror_rejects_like_the_reference():
    q = torch.zeros(2, 32, 128, dtype=torch.bfloat16)
    K = torch.zeros(2, 16, 8, 128, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="q_h must be CUDA"):
        ops.flash_decode(q, K, K, 4)
    with pytest.raises(RuntimeError, match="q_h must be CUDA"):
        ops.prop_decode(q[0], K[0], K[0], 4)


def test_argument_validation_of_the_entries_around_the_path():
    """The ragged decode entries and the RoPE/append entry reject bad arguments before any CUDA call."""
    lib = capi.lib()
    P = 256  # a non-null, aligned stand-in pointer; never dereferenced on these paths
    # santa_flash_decode_ragged: null lengths, bad dtype, bad shape, bound above the storage, sharding ext
    fr = lib.santa_flash_decode_ragged
    assert fr(P, P, P, 0, 2, 32, 8, 128, 64, None, 64, 4, 1, 0, P, P, None, None, 0, None, None) == -8
    assert fr(P, P, P, 5, 2, 32, 8, 128, 64, P, 64, 4, 1, 0, P, P, None, None, 0, None, None) == -1
    assert fr(P, P, P, 0, 2, 32, 9, 128, 64, P, 64, 4, 1, 0, P, P, None, None, 0, None, None) == -2
    assert fr(P, P, P, 0, 2, 32, 8, 128, 64, P, 65, 4, 1, 0, P, P, None, None, 0, None, None) == -3
    ext = capi.FlashExt(batch_offset=0, tile_offset=3, s_per_tile_override=-1)
    assert fr(P, P, P, 0, 2, 32, 8, 128, 64, P, 64, 4, 1, 0, P, P, None, None, 0, ctypes.byref(ext), None) == -8
    # santa_prop_decode_ragged
    pr = lib.santa_prop_decode_ragged
    assert pr(P, P, P, 0, 2, 32, 8, 128, 64, None, 64, 4, 1, P, P, None, None, 0, None, None) == -8
    assert pr(P, P, P, 0, 2, 32, 8, 128, 64, P, 0, 4, 1, P, P, None, None, 0, None, None) == -3
    assert pr(P + 4, P, P, 0, 2, 32, 8, 128, 64, P, 64, 4, 1, P, P, None, None, 0, None, None) == -6
    # santa_rope_append: null tensor, D != 128, host position outside the cache, stride not a multiple of 4
    ra = lib.santa_rope_append
    assert ra(None, P, P, 0, 0, 0, P, P, 0, 2, 32, 8, 128, P, P, 64, 0, None, P, None, None, None) == -8
    assert ra(P, P, P, 0, 0, 0, P, P, 0, 2, 32, 8, 64, P, P, 64, 0, None, P, None, None, None) == -2
    assert ra(P, P, P, 0, 0, 0, P, P, 0, 2, 32, 8, 128, P, P, 64, 64, None, P, None, None, None) == -3
    assert ra(P, P, P, 6146, 0, 0, P, P, 0, 2, 32, 8, 128, P, P, 64, 0, None, P, None, None, None) == -6
    assert ra(P, P, P, 0, 0, 0, P, P, 3, 2, 32, 8, 128, P, P, 64, 0, None, P, None, None, None) == -1
    # host mirrors
    q = torch.zeros(2, 32, 128, dtype=torch.bfloat16)
    K = torch.zeros(2, 16, 8, 128, dtype=torch.bfloat16)
    with pytest.raises(RuntimeError, match="must be CUDA"):
        ops.prop_decode_ragged(q, K, K, [16, 16], 4)
    with pytest.raises(RuntimeError, match="q_h must be CUDA"):
        ops.flash_decode_ragged(q, K, K, [16, 16], 4)


def test_peer_exchange_layout_and_validation():
    lib = capi.lib()
    assert lib.santa_peer_exchange_bytes(0, 32) == 0 and lib.santa_peer_exchange_bytes(17, 32) == 0
    assert lib.santa_peer_exchange_bytes(2, 0) == 0
    for world, BH in ((1, 32), (2, 32), (8, 64), (16, 1024)):
        n = lib.santa_peer_exchange_bytes(world, BH)
        # control words, row flags [2][world][BH] int32 (padded to 256 bytes), rows [2][world][BH][130] fp32
        flags = (2 * world * BH * 4 + 255) // 256 * 256
        need = 256 + flags + 2 * world * BH * 130 * 4
        assert n % 256 == 0 and need <= n < need + 256
    assert lib.santa_peer_exchange_status(4096) == 4096 + 4 * 34 and lib.santa_peer_exchange_status(None) is None
    px = capi.PeerExchange(world=2, rank=0, epoch=1)
    px.peer_buffer[0], px.peer_buffer[1] = 256, 512
    cw = lib.santa_lse_combine_wait
    assert cw(ctypes.byref(px), 32, 64, 1, 0, 256, None, None, None) == -2           # D
    assert cw(ctypes.byref(px), 32, 128, 1, 9, 256, None, None, None) == -1          # dtype
    px.rank = 2
    assert cw(ctypes.byref(px), 32, 128, 1, 0, 256, None, None, None) == -8          # rank outside world
    # a decode call that names a malformed exchange is refused before any CUDA work
    px.rank, px.world = 0, 17
    ext = capi.FlashExt(batch_offset=0, tile_offset=0, s_per_tile_override=-1)
    ext.peer = ctypes.pointer(px)
    rc = lib.santa_flash_decode(256, 256, 256, 0, 1, 32, 8, 128, 16, 16, 4, 1, 0, None, None, None, None, 0,
                                ctypes.byref(ext), None)
    assert rc == -8
    # the combining form needs somewhere to put the combined result
    px.world, px.flags = 2, capi.SANTA_PEER_COMBINE
    rc = lib.santa_flash_decode(256, 256, 256, 0, 1, 32, 8, 128, 16, 16, 4, 1, 0, None, None, None, None, 0,
                                ctypes.byref(ext), None)
    assert rc == -8


def test_public_header_is_plain_c():
    """include/santa_b200.h is what a cgo / JNI / FFI binding includes: it must compile as C and as C++."""
    import shutil
    import subprocess
    hdr = os.path.join(ROOT, "include", "santa_b200.h")
    if shutil.which("gcc") is None:
        pytest.skip("no gcc")
    subprocess.check_call(["gcc", "-std=c11", "-Wall", "-Werror", "-fsyntax-only", "-x", "c", hdr])
    subprocess.check_call(["g++", "-std=c++17", "-Wall", "-Werror", "-fsyntax-only", "-x", "c++", hdr])


def test_library_is_self_contained():
    """The C-ABI library depends on neither PyTorch nor Python, and exports nothing but its santa_* API."""
    import shutil
    import subprocess
    if shutil.which("ldd") is None or shutil.which("nm") is None:
        pytest.skip("no binutils")
    deps = subprocess.check_output(["ldd", capi.LIB_PATH], text=True)
    for forbidden in ("torch", "c10", "python", "libcuda.so"):
        assert forbidden not in deps, deps
    syms = subprocess.check_output(["nm", "-D", "--defined-only", capi.LIB_PATH], text=True).split("\n")
    funcs = [ln.split()[-1] for ln in syms if " T " in ln]
    assert funcs and all(f.startswith("santa_") for f in funcs), funcs
    assert sorted(funcs) == sorted(capi.EXPORTS)


def test_work_split_arithmetic_of_the_kernels(tmp_path):
    """tests/split_host.cu compiles the kernels' own split functions (csrc/common.cuh) as host code and
    checks on random ragged batches that the weighted ranges of Prop's second pass tile the items exactly
    once, that none is empty, and that the merge kernel finds the owning range of every column."""
    import shutil
    import subprocess
    if shutil.which("nvcc") is None:
        pytest.skip("no nvcc on this machine")
    exe = str(tmp_path / "split_host")
    subprocess.check_call(["nvcc", "-gencode", "arch=compute_100a,code=sm_100a", "-O1", "-std=c++17", "-o", exe,
                           os.path.join(ROOT, "tests", "split_host.cu")])
    txt = subprocess.check_output([exe], text=True, timeout=300)
    assert txt.startswith("ok "), txt
