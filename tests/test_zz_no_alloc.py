"""The no-allocation entry point (santa_flash_decode_noalloc), called through the C ABI.

It serves callers that cannot give the library a workspace -- servers that hand all free device memory
to their KV-cache pool at start-up and forbid allocation while decoding, and C hosts without a device
allocator -- by keeping its scratch in a fixed array inside the library.  Here it must reproduce the
regular entry point on two calls in a row, because every call reuses the same scratch: within the
suite's output tolerance, and -- the kernels being the same and deterministic -- in fact bit for bit.
Its status word, reachable through santa_noalloc_status(), must stay zero, and problems whose scratch
need exceeds the fixed array must be refused.  This file sorts last so that a failure here cannot hide another
test's result in a run that stops at the first failure."""

import ctypes

import pytest
import torch

import cases

pytestmark = pytest.mark.gpu
MAX_ABS, MEAN_ABS = 2e-2, 2e-3


def _read_device_int32(addr):
    """One int32 at a raw device address (the CUDA runtime's cudaMemcpy, device to host)."""
    rt = None
    for name in ("libcudart.so", "libcudart.so.12", "/usr/local/cuda/lib64/libcudart.so"):
        try:
            rt = ctypes.CDLL(name)
            break
        except OSError:
            continue
    if rt is None:
        pytest.skip("no CUDA runtime library to read the word with")
    host = (ctypes.c_int32 * 1)()
    assert rt.cudaMemcpy(host, ctypes.c_void_p(addr), ctypes.c_size_t(4), ctypes.c_int(2)) == 0
    return int(host[0])


def _call_noalloc(lib, q, K, V, S, seed, valid_len, want_vrows=True):
    B, H, D = q.shape
    Ls, KVH = K.shape[1], K.shape[2]
    out = torch.empty_like(q)
    m_star = torch.empty(B, H, device=q.device, dtype=torch.float32)
    vrows = torch.empty(B, KVH, device=q.device, dtype=torch.int32)
    rc = lib.santa_flash_decode_noalloc(q.data_ptr(), K.data_ptr(), V.data_ptr(), 0, B, H, KVH, D, valid_len, Ls,
                                        S, seed, 0, out.data_ptr(), m_star.data_ptr(),
                                        vrows.data_ptr() if want_vrows else None, None,
                                        torch.cuda.current_stream().cuda_stream)
    return rc, out, m_star, vrows


def test_noalloc_entry_point_matches_workspace_entry_point():
    from santa_b200 import capi, ops

    lib = capi.lib()
    dev = torch.device("cuda:0")
    torch.cuda.set_device(dev)
    for rep, (B, L, Ls, KVH, S, seed) in enumerate([(2, 5000, 5100, 8, 256, 1690), (3, 700, 700, 2, 64, 7)]):
        q, K, V = cases.make_qkv(B, Ls, KVH, "bf16", 40 + rep, 1.0, True)
        q, K, V = q.to(dev), K.to(dev), V.to(dev)
        ref_out, ref_m, ref_v = ops.flash_decode(q, K, V, S, seed=seed, want_vrows=True, valid_len=L)
        for _ in range(2):  # two calls in a row share the library's scratch array
            rc, out, m_star, vrows = _call_noalloc(lib, q, K, V, S, seed, L)
            assert rc == 0, lib.santa_strerror(rc)
            torch.cuda.synchronize()
            d = (out.float() - ref_out.float()).abs()
            assert d.max().item() <= MAX_ABS and d.mean().item() <= MEAN_ABS
            assert torch.equal(out, ref_out)            # the same kernels in the same order: the same bits
            assert torch.equal(m_star, ref_m) and torch.equal(vrows, ref_v)
            # the scratch's status word: reachable once the entry point has run on this device, and zero
            addr = lib.santa_noalloc_status()
            assert addr
            assert _read_device_int32(addr) == 0


def test_noalloc_entry_point_rejects_oversized_problems():
    from santa_b200 import capi

    lib = capi.lib()
    torch.cuda.set_device(0)
    B, KVH, L = 4096, 8, 4096
    assert lib.santa_flash_workspace_bytes(B, KVH, L, 0) > (4 << 20)
    dummy = torch.zeros(64, device="cuda:0")
    rc = lib.santa_flash_decode_noalloc(dummy.data_ptr(), dummy.data_ptr(), dummy.data_ptr(), 0, B, 4 * KVH, KVH, 128,
                                        L, L, 16, 1, 0, dummy.data_ptr(), dummy.data_ptr(), None, None, None)
    assert rc == -9 and b"limit" in lib.santa_strerror(rc)
