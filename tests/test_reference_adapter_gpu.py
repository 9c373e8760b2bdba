"""The reference's own adapter layer, unmodified, driving this build's drop-in modules.

``tutorial_code/attention_backends.py`` of the reference imports ``santa_flash_batch_cuda`` /
``santa_prop_batch_cuda`` by name (:513-520) and calls them from ``_SantaBaseBackend.decode``
(:462-500).  When a checkout of the reference is reachable (environment variable
``SANTA_REFERENCE``) the file is imported as it lies there and its ``SantaFlashBackend`` /
``SantaPropBackend`` run ``smoke_test`` (:41-67) and ``decode`` against the modules of this build;
otherwise the test is skipped.  Nothing of the reference is copied."""
import importlib
import os
import sys

import pytest
import torch

pytestmark = pytest.mark.gpu

REFERENCE = os.environ.get("SANTA_REFERENCE", "/root/reference")
TUTORIAL = os.path.join(REFERENCE, "tutorial_code")


@pytest.mark.skipif(not os.path.exists(os.path.join(TUTORIAL, "attention_backends.py")),
                    reason="no reference checkout (set SANTA_REFERENCE)")
def test_unmodified_reference_adapter_drives_the_dropin_modules():
    import santa_b200
    from santa_b200 import ops

    sys.path.insert(0, os.path.dirname(os.path.abspath(__file__)))
    import cases

    santa_b200.enable_dropin()
    sys.path.insert(0, TUTORIAL)
    try:
        ab = importlib.import_module("attention_backends")
    finally:
        sys.path.remove(TUTORIAL)
    dev = torch.device("cuda:0")
    flash = ab.SantaFlashBackend(S=256, seed=1690, block_n=None)
    prop = ab.SantaPropBackend(S=256, seed=1690, block_n=None)
    assert flash.module_name == "santa_flash_batch_cuda" and prop.module_name == "santa_prop_batch_cuda"
    assert os.path.dirname(flash.module.__file__) == santa_b200.LIB_DIR       # this build's modules, not another's
    assert flash.supports_true_batch_decode and not prop.supports_true_batch_decode

    # the adapter's start-up check: two sequences of 16 cached tokens (32-row tiles, one tile)
    for be in (flash, prop):
        rep = be.smoke_test(device=dev, dtype=torch.bfloat16, num_heads=32, num_kv_heads=8, head_dim=128, valid_len=16)
        assert rep["output_shape"] == [2, 32, 128]
    assert flash.actual_mode == "batch" and prop.actual_mode == "single_loop_fallback"

    # decode() on caches longer than the valid prefix, against direct calls of the C-ABI mirror
    for L_valid in (700, 2500, 5000):
        q, K, V = cases.make_qkv(3, L_valid + 300, 8, "bf16", 31 + L_valid, 1.0, True)
        q, K, V = q.to(dev), K.to(dev), V.to(dev)
        out_f = flash.decode(q, K, V, L_valid)
        assert flash.actual_mode == "batch"
        want_f = ops.flash_decode(q, K, V, 256, seed=1690, valid_len=L_valid)[0]
        assert torch.equal(out_f, want_f)
        out_p = prop.decode(q, K, V, L_valid)
        assert prop.actual_mode == "single_loop_fallback"
        for b in range(3):
            want_p = ops.prop_decode(q[b], K[b, :L_valid].contiguous(), V[b, :L_valid].contiguous(), 256, seed=1690)[0]
            assert torch.equal(out_p[b], want_p)
        assert torch.isfinite(out_f.float()).all() and torch.isfinite(out_p.float()).all()
