"""GPU parity tests of the CUDA path (through the C ABI) against the reference's own kernels
(oracle/_ref), the golden fixtures and the CPU oracle.  Integer results are compared bit-for-bit;
attention outputs within max-abs 2e-2 / mean-abs 2e-3 (the tolerance the task states for bf16)."""
import os

import numpy as np
import pytest
import torch

import cases
from oracle import ref_gpu
from oracle import santa_oracle as so

pytestmark = pytest.mark.gpu

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
HERE = os.path.dirname(os.path.abspath(__file__))
MAX_ABS, MEAN_ABS = 2e-2, 2e-3
HAVE_REF = ref_gpu.available()
needs_ref = pytest.mark.skipif(not HAVE_REF, reason="oracle/_ref not built (needs the reference tree)")


def dev():
    return torch.device("cuda:0")


def ops():
    from santa_b200 import ops as _ops
    return _ops


def bits_eq(a, b):
    return bool((a.view(torch.int32) == b.view(torch.int32)).all())


def close(a, b):
    d = (a.float() - b.float()).abs()
    return d.max().item() <= MAX_ABS and d.mean().item() <= MEAN_ABS


def dense_counts(g, shape):
    c = np.zeros(int(np.prod(shape)), np.int16)
    c[g["ref_counts_idx"]] = g["ref_counts_val"]
    return c.reshape(shape)


def flash_eval_torch(counts, V, m_tiles, ell_tiles, bn, spt):
    """fp32 torch evaluation of the Flash estimator over a given count table (on the GPU)."""
    B, H, L = counts.shape
    KVH = V.shape[2]
    ms = m_tiles.max(-1, keepdim=True).values
    w = torch.exp(m_tiles - ms) * ell_tiles                     # [B,H,T_c]
    Z = w.sum(-1)
    wrow = w.repeat_interleave(bn, dim=-1)[..., :L]             # [B,H,L]
    cw = counts.float() * wrow
    out = torch.zeros(B, H, 128, device=counts.device)
    for kv in range(KVH):
        Vk = V[:, :L, kv].float()                               # [B,L,128]
        out[:, 4 * kv:4 * kv + 4] = torch.bmm(cw[:, 4 * kv:4 * kv + 4], Vk)
    return out / (Z * spt).clamp_min(1e-30)[..., None] if spt > 0 else out * 0


# ---------------------------------------------------------------- Flash
FLASH_SHAPES = [  # B, L, Ls, KVH, S, seed, dtype, block_n
    (1, 4096, 4096, 8, 32, 1690, "bf16", 0),
    (2, 4096, 4096, 8, 2048, 7, "bf16", 0),
    (3, 5000, 6000, 3, 300, 3, "bf16", 0),
    (2, 1, 4, 2, 64, 11, "bf16", 0),
    (2, 16, 16, 8, 2048, 11, "bf16", 0),
    (2, 31, 40, 2, 64, 11, "bf16", 0),
    (2, 33, 33, 2, 64, 11, "f16", 0),
    (2, 255, 300, 2, 64, 11, "bf16", 0),
    (2, 257, 257, 2, 64, 11, "bf16", 0),
    (1, 1536, 1536, 2, 256, 12, "bf16", 0),
    (1, 1537, 1537, 2, 256, 12, "f16", 0),
    (1, 3072, 3072, 2, 256, 12, "bf16", 0),
    (1, 3073, 3100, 2, 256, 12, "bf16", 0),
    (1, 2000, 2000, 4, 100, 5, "bf16", 256),
    (1, 9000, 9000, 8, 100, 5, "bf16", 32),
    (2, 8200, 8200, 8, 0, 5, "bf16", 0),
    (5, 7000, 7000, 1, 1, 5, "f16", 0),
]


@needs_ref
@pytest.mark.parametrize("B,L,Ls,KVH,S,seed,dtype,block_n", FLASH_SHAPES)
def test_flash_matches_reference_binary(B, L, Ls, KVH, S, seed, dtype, block_n):
    q, K, V = cases.make_qkv(B, Ls, KVH, dtype, 100 + L, 1.0, True)
    q, K, V = q.to(dev()), K.to(dev()), V.to(dev())
    out, m_star, vrows, tr = ops().flash_decode(q, K, V, S, seed=seed, block_n=block_n, want_vrows=True,
                                                valid_len=L, trace=True)
    ref_counts, _ = ref_gpu.flash_counts(q, K, S, seed=seed, block_n=block_n, valid_len=L)
    r = ref_gpu.flash_decode(q, K, V, S, seed=seed, block_n=block_n, want_vrows=True, valid_len=L)
    torch.cuda.synchronize()
    assert ops().workspace_status("flash", dev()) == 0
    assert (tr.block_n, tr.T_c, tr.S_per_tile) == (r.block_n, r.T_c, r.S_per_tile)
    assert (tr.counts.int() == ref_counts).all()            # sampled rows: bit-exact
    assert bits_eq(tr.m_tiles, r.m_tiles) and bits_eq(tr.ell_tiles, r.ell_tiles)
    assert bits_eq(m_star, r.m_star)
    assert (vrows == r.vrows).all() and (tr.rowmask == r.rowmask).all()
    assert close(out, r.out)
    if S == 0:
        assert (out == 0).all()


VALUE_RANGES = [  # kscale, qscale, L, dtype, block_n
    (0.0, 1.0, 5000, "bf16", 0),     # every score equal: all weights 1
    (6.0, 1.0, 5000, "bf16", 0),     # scores spread over +-70: most weights underflow (flush-to-zero territory)
    (6.0, 1.0, 700, "f16", 0),
    (12.0, 2.0, 3000, "bf16", 0),    # +-270: exp of the whole tile but its maximum is zero
    (1e-3, 1e-3, 4096, "bf16", 256),  # tiny scores: weights all within an ulp of 1
]


@needs_ref
@pytest.mark.parametrize("kscale,qscale,L,dtype,block_n", VALUE_RANGES)
def test_extreme_value_ranges_match_reference_binary(kscale, qscale, L, dtype, block_n):
    """Score distributions at the edges of the arithmetic (equal scores; weights that underflow, where the
    Flash build's flush-to-zero and the Prop build's denormals differ; tiny scores): both variants against the
    reference binary, bit for bit."""
    q, K, V = cases.make_qkv(2, L, 2, dtype, 900 + L, kscale, False)
    q = (q.float() * qscale).to(q.dtype)
    q, K, V = q.to(dev()), K.to(dev()), V.to(dev())
    S, seed = 128, 77
    out, m_star, vrows, tr = ops().flash_decode(q, K, V, S, seed=seed, block_n=block_n, want_vrows=True, trace=True)
    ref_counts, _ = ref_gpu.flash_counts(q, K, S, seed=seed, block_n=block_n)
    r = ref_gpu.flash_decode(q, K, V, S, seed=seed, block_n=block_n, want_vrows=True)
    torch.cuda.synchronize()
    assert ops().workspace_status("flash", dev()) == 0
    assert (tr.counts.int() == ref_counts).all()
    assert bits_eq(tr.m_tiles, r.m_tiles) and bits_eq(tr.ell_tiles, r.ell_tiles) and bits_eq(m_star, r.m_star)
    assert (vrows == r.vrows).all() and close(out, r.out)
    for b in range(2):
        po, pm, pv, pt = ops().prop_decode(q[b], K[b], V[b], S, seed=seed, block_n=block_n, want_vrows=True, trace=True)
        pr = ref_gpu.prop_decode(q[b], K[b], V[b], S, seed=seed, block_n=block_n, want_vrows=True)
        torch.cuda.synchronize()
        assert ops().workspace_status("prop", dev()) == 0
        assert bits_eq(pt.m_tiles, pr.m_tiles) and bits_eq(pt.ell_tiles, pr.ell_tiles) and bits_eq(pm, pr.m_star)
        assert (pt.u16 == pr.u_stash.view(torch.int16).t()).all()
        dS = (pt.S_tiles - pr.S_tiles).abs()     # the reference's Z is an unordered atomic sum
        assert dS.max().item() <= 1
        if dS.max().item() == 0:
            assert bits_eq(pt.invdelta, pr.invdelta) and (pv == pr.vrows).all()
            if L <= 4096:
                rc, _ = ref_gpu.prop_counts(q[b], K[b], S, seed=seed, block_n=block_n)
                assert (pt.counts.int() == rc).all()
        assert close(po, pr.out)


@pytest.mark.parametrize("name", list(cases.FLASH_CASES))
def test_flash_matches_golden_and_oracle(name):
    """No reference build needed: golden fixtures (from the reference kernels) + CPU oracle."""
    c = cases.FLASH_CASES[name]
    g = np.load(os.path.join(GOLDEN, f"flash_{name}.npz"))
    qc, Kc, Vc = cases.make_qkv(c["B"], c["Ls"], c["KVH"], c["dtype"], c["gen_seed"], c["kscale"], c["heavy"])
    q, K, V = qc.to(dev()), Kc.to(dev()), Vc.to(dev())
    out, m_star, vrows, tr = ops().flash_decode(q, K, V, c["S"], seed=c["seed"], block_n=c["block_n"],
                                                want_vrows=True, valid_len=c["L"], trace=True)
    torch.cuda.synchronize()
    H = 4 * c["KVH"]
    ref_counts = dense_counts(g, (c["B"], H, c["L"]))
    assert (tr.counts.cpu().numpy() == ref_counts).all()
    assert (tr.m_tiles.cpu().numpy().view(np.int32) == g["ref_m_tiles"].view(np.int32)).all()
    assert (tr.ell_tiles.cpu().numpy().view(np.int32) == g["ref_ell_tiles"].view(np.int32)).all()
    assert (tr.u16.cpu().numpy().view(np.uint16) == g["dev_u16"]).all()
    assert (vrows.cpu().numpy() == g["ref_vrows"]).all()
    assert (m_star.cpu().numpy().view(np.int32) == g["ref_m_star"].view(np.int32)).all()
    isb = c["dtype"] == "bf16"
    out_ref = torch.from_numpy(so.from16(g["ref_out"], isb))
    assert close(out.cpu(), out_ref)
    # CPU oracle fed with the device's approximate intermediates reproduces the device's counts
    r = so.flash_decode(cases.bits(qc), cases.bits(Kc), cases.bits(Vc), c["S"], seed=c["seed"],
                        block_n=c["block_n"], valid_len=c["L"], is_bf16=isb,
                        inject_u16=tr.u16.cpu().numpy().view(np.uint16), inject_ell=tr.ell_tiles.cpu().numpy(),
                        inject_invdel=tr.invdel.cpu().numpy())
    assert (r.counts == tr.counts.cpu().numpy()).all()
    assert (r.m_tiles.view(np.int32) == tr.m_tiles.cpu().numpy().view(np.int32)).all()
    assert close(out.cpu(), torch.from_numpy(r.out))


def test_flash_dropin_module_equals_c_abi_path():
    import santa_b200
    santa_b200.enable_dropin()
    import santa_flash_batch_cuda as mod
    q, K, V = cases.make_qkv(2, 5000, 8, "bf16", 9, 1.0, True)
    q, K, V = q.to(dev()), K.to(dev()), V.to(dev())
    a = ops().flash_decode(q, K, V, 256, seed=1690, want_vrows=True, valid_len=4500)
    # the reference adapter's call: positional q,K,V,S then keywords (attention_backends.py:464-473)
    b = mod.decode_systematic_batched(q.contiguous(), K, V, 256, seed=1690, want_vrows=True, valid_len=4500)
    assert torch.equal(a[0], b[0]) and torch.equal(a[1], b[1]) and torch.equal(a[2], b[2])
    assert b[0].shape == (2, 32, 128) and b[0].dtype == torch.bfloat16 and b[1].shape == (2, 32)
    # scalar alias, single sequence, no vrows -> empty int32 tensor of shape [0]
    c = mod.decode_systematic_scalar(q[0], K[0], V[0], 256, seed=1690, valid_len=4500)
    assert c[0].shape == (32, 128) and c[2].shape == (0,) and c[2].dtype == torch.int32
    s = ops().flash_decode(q[0], K[0], V[0], 256, seed=1690, valid_len=4500)
    assert torch.equal(c[0], s[0])
    # head index of the RNG key is b*H + h: sequence 0 of the batch equals the single call
    assert torch.equal(c[0], b[0][0])
    with pytest.raises(TypeError):
        mod.decode_systematic_batched(q, K, V, 256, seed=-1)
    with pytest.raises(RuntimeError, match="contiguous"):
        mod.decode_systematic_batched(q, K.transpose(1, 2), V.transpose(1, 2), 256)
    with pytest.raises(RuntimeError, match="valid_len exceeds storage length"):
        mod.decode_systematic_batched(q, K, V, 256, valid_len=6000)
    with pytest.raises(RuntimeError, match="block_n must be 0"):
        mod.decode_systematic_batched(q, K, V, 256, block_n=128)
    with pytest.raises(RuntimeError, match="GH=4"):
        mod.decode_systematic_batched(q[:, :16], K, V, 256)


def test_flash_full_size_properties():
    """Config 1 at full size (B=8, L=32768, S=256): size-independent properties."""
    q, K, V = cases.make_qkv(8, 32768, 8, "bf16", 1690, 1.0, True)
    q, K, V = q.to(dev()), K.to(dev()), V.to(dev())
    out, m_star, vrows, tr = ops().flash_decode(q, K, V, 256, seed=1690, want_vrows=True, trace=True)
    out2, _, vrows2 = ops().flash_decode(q, K, V, 256, seed=1690, want_vrows=True)
    torch.cuda.synchronize()
    assert torch.equal(out, out2) and torch.equal(vrows, vrows2)          # deterministic
    assert (tr.T_c, tr.S_per_tile) == (128, 2)
    per_tile = tr.counts.view(8, 32, 128, 256).sum(-1)
    assert per_tile.min() >= 1 and per_tile.max() <= 3                     # ~S_per_tile samples per (head, tile)
    flagged = (tr.counts.view(8, 8, 4, 32768) > 0).any(2)                  # a row is gathered iff some head drew it
    assert (flagged.sum(-1).int() == vrows).all()
    assert ((tr.rowmask != 0) == flagged).all()
    assert bits_eq(m_star, tr.m_tiles.max(-1).values)
    ev = flash_eval_torch(tr.counts, V, tr.m_tiles, tr.ell_tiles, 256, 2)   # fp32 evaluation over the op's counts
    assert close(out, ev)
    # offsets: a0[b,h,t] only depends on (seed, b*H+h, t)
    assert ops().workspace_status("flash", dev()) == 0
    if HAVE_REF:
        rc, _ = ref_gpu.flash_counts(q, K, 256, seed=1690)
        assert (tr.counts.int() == rc).all()


def test_flash_sharding_extensions():
    """Sequence shards (global tile index, global budget) + LSE combine == unsharded; batch shards with
    batch_offset == unsharded."""
    q, K, V = cases.make_qkv(2, 8192, 8, "bf16", 21, 1.0, True)
    q, K, V = q.to(dev()), K.to(dev()), V.to(dev())
    S, seed = 512, 1690
    out, m_star, vrows, tr = ops().flash_decode(q, K, V, S, seed=seed, want_vrows=True, trace=True)
    for G in (2, 4, 8):
        Lr = 8192 // G
        parts, cnts, vr = [], [], 0
        for r in range(G):
            Kr, Vr = K[:, r * Lr:(r + 1) * Lr].contiguous(), V[:, r * Lr:(r + 1) * Lr].contiguous()
            p_, _, v_, t_ = ops().flash_decode(q, Kr, Vr, S, seed=seed, block_n=tr.block_n, want_vrows=True,
                                               partial=True, trace=True, tile_offset=r * (Lr // 256),
                                               s_per_tile=tr.S_per_tile)
            parts.append(p_)
            cnts.append(t_.counts)
            vr = vr + v_
        assert torch.equal(torch.cat(cnts, dim=2), tr.counts)              # same samples as the unsharded call
        assert torch.equal(vr, vrows)
        o2, ms2 = ops().lse_combine(torch.stack(parts).contiguous(), tr.S_per_tile, torch.bfloat16)
        assert bits_eq(ms2, m_star)
        assert (o2.float() - out.float()).abs().max().item() <= 2 ** -7      # fp32 merge order + one bf16 rounding
        # CPU oracle of the merge rule
        oc, mc = so.merge_partials(torch.stack(parts)[:, 0].cpu().numpy(), tr.S_per_tile)
        assert np.abs(oc - o2[0].float().cpu().numpy()).max() <= 2 ** -7
    ob = [ops().flash_decode(q[b:b + 1], K[b:b + 1], V[b:b + 1], S, seed=seed, batch_offset=b)[0] for b in range(2)]
    assert torch.equal(torch.cat(ob), out)


# ---------------------------------------------------------------- Prop
PROP_SHAPES = [  # L, KVH, S, seed, dtype, block_n
    (4096, 8, 256, 1690, "bf16", 0), (3300, 2, 64, 7, "f16", 0), (600, 2, 48, 9, "bf16", 0),
    (2000, 4, 100, 10, "bf16", 0), (16, 8, 2048, 3, "bf16", 0), (1, 2, 5, 3, "bf16", 0),
    (257, 2, 64, 3, "bf16", 256), (1000, 2, 64, 3, "bf16", 128), (5000, 8, 0, 3, "bf16", 0),
    (9000, 8, 256, 1690, "bf16", 48), (23132, 8, 256, 1690, "bf16", 0), (8769, 8, 256, 1690, "bf16", 0),
    # more tiles than samples: most (head, tile) pairs get no budget and their scans are left out
    (40000, 2, 32, 5, "bf16", 0), (30000, 8, 16, 6, "f16", 0), (4096, 2, 3, 8, "bf16", 64),
]


@needs_ref
@pytest.mark.parametrize("L,KVH,S,seed,dtype,block_n", PROP_SHAPES)
def test_prop_matches_reference_binary(L, KVH, S, seed, dtype, block_n):
    q, K, V = cases.make_qkv(1, L, KVH, dtype, 200 + L, 1.0, True)
    q, K, V = q[0].to(dev()), K[0].to(dev()), V[0].to(dev())
    out, m_star, vrows, tr = ops().prop_decode(q, K, V, S, seed=seed, block_n=block_n, want_vrows=True, trace=True)
    r = ref_gpu.prop_decode(q, K, V, S, seed=seed, block_n=block_n, want_vrows=True)
    torch.cuda.synchronize()
    assert ops().workspace_status("prop", dev()) == 0
    assert (tr.block_n, tr.T_c) == (r.block_n, r.T_c)
    assert bits_eq(tr.m_tiles, r.m_tiles) and bits_eq(tr.ell_tiles, r.ell_tiles)
    assert (tr.u16 == r.u_stash.view(torch.int16).t()).all()
    assert bits_eq(m_star, r.m_star) and bits_eq(tr.a0, r.a0)
    # the reference sums Z with unordered atomics: budgets may differ by one sample on rare tiles
    dS = (tr.S_tiles - r.S_tiles).abs()
    assert dS.max().item() <= 1 and (dS != 0).float().mean().item() <= 0.01
    if dS.max().item() == 0:
        assert bits_eq(tr.invdelta, r.invdelta)
        assert (vrows == r.vrows).all() and (tr.rowmask == r.rowmask).all()
        if L <= 4096:
            rc, _ = ref_gpu.prop_counts(q, K, S, seed=seed, block_n=block_n)
            assert (tr.counts.int() == rc).all()
    assert close(out, r.out)
    if S == 0:
        assert (out == 0).all()


PROP_GENERIC_SHAPES = [  # L, KVH, GH, D, S, seed, dtype, block_n
    (4096, 8, 8, 128, 256, 1690, "bf16", 0),     # H=64: eight query heads per kv-head
    (4096, 8, 4, 64, 256, 1690, "bf16", 0),      # head_dim 64
    (700, 4, 2, 64, 64, 3, "f16", 0), (3000, 2, 1, 256, 100, 5, "bf16", 0),
    (2000, 3, 8, 80, 128, 9, "bf16", 0), (5000, 2, 3, 128, 64, 9, "bf16", 0),
    (9000, 2, 8, 128, 64, 4, "f16", 48), (33, 2, 2, 32, 16, 1, "bf16", 0), (5000, 4, 4, 64, 0, 1, "bf16", 0),
]


@needs_ref
@pytest.mark.parametrize("L,KVH,GH,D,S,seed,dtype,block_n", PROP_GENERIC_SHAPES)
def test_prop_generic_shapes_match_reference_binary(L, KVH, GH, D, S, seed, dtype, block_n):
    """Query-group sizes and head dimensions other than 4 / 128 (the reference's generic tensor-core first
    pass and generic second pass): the same bit-for-bit comparisons as for the vectorised shape."""
    q, K, V = cases.make_qkv(1, L, KVH, dtype, 500 + L + D, 1.0, True, GH=GH, D=D)
    q, K, V = q[0].to(dev()), K[0].to(dev()), V[0].to(dev())
    out, m_star, vrows, tr = ops().prop_decode(q, K, V, S, seed=seed, block_n=block_n, want_vrows=True, trace=True)
    r = ref_gpu.prop_decode(q, K, V, S, seed=seed, block_n=block_n, want_vrows=True)
    torch.cuda.synchronize()
    assert ops().workspace_status("prop", dev()) == 0
    assert (tr.block_n, tr.T_c) == (r.block_n, r.T_c) and tuple(out.shape) == (GH * KVH, D)
    assert bits_eq(tr.m_tiles, r.m_tiles) and bits_eq(tr.ell_tiles, r.ell_tiles)
    assert (tr.u16 == r.u_stash.view(torch.int16).t()).all()
    assert bits_eq(m_star, r.m_star) and bits_eq(tr.a0, r.a0)
    dS = (tr.S_tiles - r.S_tiles).abs()          # the reference's Z is an unordered atomic sum
    assert dS.max().item() <= 1 and (dS != 0).float().mean().item() <= 0.01
    if dS.max().item() == 0:
        assert bits_eq(tr.invdelta, r.invdelta)
        assert (vrows == r.vrows).all() and (tr.rowmask == r.rowmask).all()
        if L <= 4096:
            rc, _ = ref_gpu.prop_counts(q, K, S, seed=seed, block_n=block_n)
            assert (tr.counts.int() == rc).all()
    assert close(out, r.out)
    # the estimator over the op's own counts, fp32: out[h] = sum_n c[h,n] V[n,kv] / S
    ev = torch.zeros(GH * KVH, D, device=dev())
    for kv in range(KVH):
        ev[GH * kv:GH * (kv + 1)] = tr.counts[GH * kv:GH * (kv + 1)].float() @ V[:, kv].float()
    assert close(out, ev / S if S > 0 else ev * 0)
    out2 = ops().prop_decode(q, K, V, S, seed=seed, block_n=block_n)[0]
    assert torch.equal(out, out2)                # fixed summation order


@pytest.mark.parametrize("name", list(cases.PROP_CASES))
def test_prop_matches_golden_and_oracle(name):
    c = cases.PROP_CASES[name]
    g = np.load(os.path.join(GOLDEN, f"prop_{name}.npz"))
    qc, Kc, Vc = cases.make_qkv(1, c["L"], c["KVH"], c["dtype"], c["gen_seed"], c["kscale"], c["heavy"], GH=c["GH"])
    q, K, V = qc[0].to(dev()), Kc[0].to(dev()), Vc[0].to(dev())
    out, m_star, vrows, tr = ops().prop_decode(q, K, V, c["S"], seed=c["seed"], block_n=c["block_n"],
                                               want_vrows=True, trace=True)
    torch.cuda.synchronize()
    H = c["GH"] * c["KVH"]
    assert (tr.m_tiles.cpu().numpy().view(np.int32) == g["ref_m_tiles"].view(np.int32)).all()
    assert (tr.ell_tiles.cpu().numpy().view(np.int32) == g["ref_ell_tiles"].view(np.int32)).all()
    assert (tr.u16.cpu().numpy().view(np.uint16) == g["ref_u_stash"].T).all()
    assert (tr.S_tiles.cpu().numpy() == g["ref_S_tiles"]).all()
    assert (tr.invdelta.cpu().numpy().view(np.int32) == g["ref_invdelta"].view(np.int32)).all()
    assert (tr.a0.cpu().numpy().view(np.int32) == g["ref_a0"].view(np.int32)).all()
    assert (tr.counts.cpu().numpy() == dense_counts(g, (H, c["L"]))).all()
    assert (vrows.cpu().numpy() == g["ref_vrows"]).all()
    isb = c["dtype"] == "bf16"
    assert close(out.cpu(), torch.from_numpy(so.from16(g["ref_out"], isb)))
    # CPU oracle downstream of the device's tile statistics
    r = so.prop_decode(cases.bits(qc[0]), cases.bits(Kc[0]), cases.bits(Vc[0]), c["S"], seed=c["seed"],
                       block_n=c["block_n"], is_bf16=isb, inject_u16=tr.u16.cpu().numpy().view(np.uint16),
                       inject_ell=tr.ell_tiles.cpu().numpy(), inject_m=tr.m_tiles.cpu().numpy())
    assert (r.S_tiles == tr.S_tiles.cpu().numpy()).all()
    assert (r.counts == tr.counts.cpu().numpy()).all()
    assert close(out.cpu(), torch.from_numpy(r.out))
    ev = so.prop_eval_over_counts(tr.counts.cpu().numpy(), Vc[0].float().numpy(), c["S"])
    assert close(out.cpu(), torch.from_numpy(ev).float())


def test_prop_dropin_module_and_adapter_fallback():
    import santa_b200
    santa_b200.enable_dropin()
    import santa_prop_batch_cuda as mod
    assert not hasattr(mod, "decode_systematic_batched")
    q, K, V = cases.make_qkv(3, 6000, 8, "bf16", 31, 1.0, True)
    q, K, V = q.to(dev()), K.to(dev()), V.to(dev())
    valid_len = 5000
    # what _SantaBaseBackend.decode does (attention_backends.py:462-500)
    with pytest.raises(TypeError) as ei:
        mod.decode_systematic_scalar(q.contiguous(), K, V, 256, seed=7, want_vrows=False, valid_len=valid_len)
    assert "valid_len" in str(ei.value)
    outs = []
    for b in range(3):
        k_b, v_b = K[b, :valid_len].contiguous(), V[b, :valid_len].contiguous()
        o = mod.decode_systematic_scalar(q[b].contiguous(), k_b, v_b, 256, seed=7, want_vrows=False)
        assert o[2].shape == (0,) and o[1].shape == (32,)
        outs.append(o[0])
        o2 = ops().prop_decode(q[b], k_b, v_b, 256, seed=7)
        assert torch.equal(o[0], o2[0]) and torch.equal(o[1], o2[1])
    assert torch.stack(outs).shape == (3, 32, 128)
    # two identical calls give identical bits (fixed summation order)
    o3 = mod.decode_systematic_scalar(q[0].contiguous(), K[0, :valid_len].contiguous(), V[0, :valid_len].contiguous(),
                                      256, seed=7, want_vrows=True)
    assert torch.equal(o3[0], outs[0]) and o3[2].shape == (8,)
    with pytest.raises(RuntimeError, match="bad ranks"):
        mod.decode_systematic_scalar(q, K, V, 256)


def test_prop_ragged_batch_properties():
    """Config 2 lengths (seed-7 draw), S=256: budgets sum to S when the tile count is a power of two or
    at least never exceed it, counts per tile follow the budgets, output equals the fp32 evaluation."""
    lengths = torch.randint(8192, 65537, (16,), generator=torch.Generator().manual_seed(7)).tolist()
    assert lengths[:4] == [23132, 8769, 40428, 11428] and sum(lengths) == 562962
    for L in (lengths[1], lengths[5]):
        q, K, V = cases.make_qkv(1, L, 8, "bf16", L, 1.0, True)
        q, K, V = q[0].to(dev()), K[0].to(dev()), V[0].to(dev())
        out, m_star, vrows, tr = ops().prop_decode(q, K, V, 256, seed=1690, want_vrows=True, trace=True)
        torch.cuda.synchronize()
        assert (tr.S_tiles.sum(1) <= 256).all() and (tr.S_tiles.sum(1) >= 256 - tr.T_c).all()
        pad = tr.T_c * 256 - L
        cnt = torch.nn.functional.pad(tr.counts, (0, pad)).view(32, tr.T_c, 256).sum(-1)
        assert ((cnt - tr.S_tiles).abs() <= 1).all()
        flagged = (tr.counts.view(8, 4, L) > 0).any(1)
        assert (flagged.sum(-1).int() == vrows).all()
        ev = torch.zeros(32, 128, device=dev())
        for kv in range(8):
            ev[4 * kv:4 * kv + 4] = tr.counts[4 * kv:4 * kv + 4].float() @ V[:, kv].float()
        assert close(out, ev / 256)


RAGGED_SETS = [
    ([300, 5000, 1, 777, 4096], 5120, 256, "bf16", 8),
    ([256, 0, 513], 600, 64, "f16", 2),
    ([8769, 23132, 11428, 9000], 23132, 256, "bf16", 8),
    # very unequal lengths: the second pass cuts its ranges by weight (a unit of a short sequence costs more)
    ([8192, 0, 65536, 300, 9000, 256, 1, 40000], 65536, 32, "bf16", 2),
    ([300, 60000, 700, 512, 33000], 60000, 2048, "f16", 2),
]


@pytest.mark.parametrize("lengths,Ls,S,dtype,KVH", RAGGED_SETS)
def test_prop_ragged_entry_equals_per_sequence_calls(lengths, Ls, S, dtype, KVH):
    """One ragged launch sequence against one 256-row-tile call per sequence (what the reference adapter's
    loop does, attention_backends.py:491-500): tile statistics, budgets, sampled counts, vrows and m_star
    bit for bit; outputs in tolerance (the partial sums are added in a different order)."""
    B, H = len(lengths), 4 * KVH
    q, K, V = cases.make_qkv(B, Ls, KVH, dtype, 77 + B, 1.0, True)
    q, K, V = q.to(dev()), K.to(dev()), V.to(dev())
    lens = torch.tensor(lengths, dtype=torch.int32, device=dev())
    out, m_star, vrows, tr = ops().prop_decode_ragged(q, K, V, lens, S, seed=1690, want_vrows=True, trace=True)
    torch.cuda.synchronize()
    assert ops().workspace_status("prop_ragged", dev()) == 0
    assert out.shape == (B, H, 128) and m_star.shape == (B, H) and vrows.shape == (B, KVH)
    for b, L in enumerate(lengths):
        if L == 0:
            assert (out[b] == 0).all() and (vrows[b] == 0).all()
            continue
        o1, m1, v1, t1 = ops().prop_decode(q[b], K[b, :L].contiguous(), V[b, :L].contiguous(), S, seed=1690,
                                           block_n=256, want_vrows=True, trace=True)
        T = t1.T_c
        assert bits_eq(tr.m_tiles[b, :, :T], t1.m_tiles) and bits_eq(tr.ell_tiles[b, :, :T], t1.ell_tiles)
        assert torch.equal(tr.u16[b, :, :L], t1.u16)
        assert torch.equal(tr.S_tiles[b, :, :T], t1.S_tiles)
        assert bits_eq(tr.invdelta[b, :, :T], t1.invdelta) and bits_eq(tr.a0[b, :, :T], t1.a0)
        assert torch.equal(tr.counts[b, :, :L], t1.counts)
        assert (tr.counts[b, :, L:] == 0).all()
        assert torch.equal(tr.rowmask[b, :, :L], t1.rowmask)
        assert bits_eq(m_star[b], m1) and torch.equal(vrows[b], v1)
        assert close(out[b], o1)
    # lengths live on the device: changing them changes the next call without any host-side re-planning
    if B > 1 and lengths[0] > 1:
        lens2 = lens.clone()
        lens2[0] = lengths[0] - 1
        out2 = ops().prop_decode_ragged(q, K, V, lens2, S, seed=1690)[0]
        o1 = ops().prop_decode(q[0], K[0, :lengths[0] - 1].contiguous(), V[0, :lengths[0] - 1].contiguous(), S,
                               seed=1690, block_n=256)[0]
        assert close(out2[0], o1)
        assert torch.equal(out2[1:], out[1:])


def test_prop_ragged_module_function():
    import santa_b200
    santa_b200.enable_dropin()
    import santa_prop_batch_cuda as mod
    assert not hasattr(mod, "decode_systematic_batched")
    lengths = [4000, 3500, 6000]
    q, K, V = cases.make_qkv(3, 6000, 8, "bf16", 41, 1.0, True)
    q, K, V = q.to(dev()), K.to(dev()), V.to(dev())
    lens = torch.tensor(lengths, dtype=torch.int32)
    o = mod.decode_systematic_ragged(q, K, V, lens, 256, seed=7, want_vrows=True)   # host lengths are copied over
    o_dev = mod.decode_systematic_ragged(q, K, V, lens.to(dev()), 256, seed=7, want_vrows=True, max_len=6000)
    assert torch.equal(o[0], o_dev[0]) and torch.equal(o[1], o_dev[1]) and torch.equal(o[2], o_dev[2])
    o2 = ops().prop_decode_ragged(q, K, V, lengths, 256, seed=7, want_vrows=True)
    assert torch.equal(o[0], o2[0]) and torch.equal(o[2], o2[2])
    for b, L in enumerate(lengths):
        ob = mod.decode_systematic_scalar(q[b].contiguous(), K[b, :L].contiguous(), V[b, :L].contiguous(), 256,
                                          seed=7, want_vrows=True)
        assert close(o[0][b], ob[0]) and torch.equal(o[1][b], ob[1]) and torch.equal(o[2][b], ob[2])
    with pytest.raises(RuntimeError, match="Ragged path expects"):
        mod.decode_systematic_ragged(q[0], K, V, lens, 256)
    with pytest.raises(RuntimeError, match="one length per sequence"):
        mod.decode_systematic_ragged(q, K, V, lens[:2], 256)
    with pytest.raises(RuntimeError, match="max_len exceeds"):
        mod.decode_systematic_ragged(q, K, V, lens, 256, max_len=7000)


FLASH_RAGGED_SETS = [
    ([300, 5000, 1, 777, 4096], 5120, 256, "bf16", 8, 256),
    ([256, 0, 513, 100], 600, 64, "f16", 2, 32),
    ([2000, 1537, 3072], 3072, 100, "bf16", 4, 64),
    ([8769, 23132, 11428, 9000], 23132, 256, "bf16", 8, 0),
]


@pytest.mark.parametrize("lengths,Ls,S,dtype,KVH,block_n", FLASH_RAGGED_SETS)
def test_flash_ragged_entry_equals_per_sequence_calls(lengths, Ls, S, dtype, KVH, block_n):
    """Lengths from device memory against one uniform call per sequence (valid_len = its length,
    batch_offset = its index, same tile size): everything bit for bit, the output included -- the
    partial sums of a sequence are folded in the same order whenever its tiles are split the same way,
    and in tolerance otherwise."""
    B, H = len(lengths), 4 * KVH
    q, K, V = cases.make_qkv(B, Ls, KVH, dtype, 91 + B, 1.0, True)
    q, K, V = q.to(dev()), K.to(dev()), V.to(dev())
    lens = torch.tensor(lengths, dtype=torch.int32, device=dev())
    out, m_star, vrows, tr = ops().flash_decode_ragged(q, K, V, lens, S, seed=1690, block_n=block_n,
                                                       want_vrows=True, trace=True)
    torch.cuda.synchronize()
    assert ops().workspace_status("flash_ragged", dev()) == 0
    bn = tr.block_n
    for b, L in enumerate(lengths):
        if L == 0:
            assert (out[b] == 0).all() and (vrows[b] == 0).all()
            continue
        o1, m1, v1, t1 = ops().flash_decode(q[b:b + 1], K[b:b + 1], V[b:b + 1], S, seed=1690, block_n=bn,
                                            want_vrows=True, valid_len=L, batch_offset=b, trace=True)
        T = t1.T_c
        assert bits_eq(tr.m_tiles[b, :, :T], t1.m_tiles[0]) and bits_eq(tr.ell_tiles[b, :, :T], t1.ell_tiles[0])
        assert bits_eq(tr.invdel[b, :, :T], t1.invdel[0])
        assert torch.equal(tr.u16[b, :, :L], t1.u16[0]) and torch.equal(tr.counts[b, :, :L], t1.counts[0])
        assert (tr.counts[b, :, L:] == 0).all()
        assert torch.equal(tr.rowmask[b, :, :L], t1.rowmask[0])
        assert bits_eq(m_star[b], m1[0]) and torch.equal(vrows[b], v1[0])
        assert close(out[b], o1[0])


def test_flash_ragged_equal_lengths_is_the_uniform_call_and_graph_replay_follows_lengths():
    import santa_b200
    santa_b200.enable_dropin()
    import santa_flash_batch_cuda as mod
    B, Ls, L = 4, 9000, 8000
    q, K, V = cases.make_qkv(B, Ls, 8, "bf16", 55, 1.0, True)
    q, K, V = q.to(dev()), K.to(dev()), V.to(dev())
    lens = torch.full((B,), L, dtype=torch.int32, device=dev())
    o_u = mod.decode_systematic_batched(q, K, V, 256, seed=3, want_vrows=True, valid_len=L)
    o_r = mod.decode_systematic_ragged(q, K, V, lens, 256, seed=3, want_vrows=True)
    assert bits_eq(o_u[1], o_r[1]) and torch.equal(o_u[2], o_r[2]) and close(o_u[0], o_r[0])
    # capture once, replay after the lengths changed on the device
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        mod.decode_systematic_ragged(q, K, V, lens, 256, seed=3)
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        o_g = mod.decode_systematic_ragged(q, K, V, lens, 256, seed=3)
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(o_g[0], o_r[0])
    lens += 500            # the cache "grew": same graph, new lengths
    graph.replay()
    torch.cuda.synchronize()
    o_u2 = mod.decode_systematic_batched(q, K, V, 256, seed=3, valid_len=L + 500)
    assert bits_eq(o_g[1], o_u2[1]) and close(o_g[0], o_u2[0])
    with pytest.raises(RuntimeError, match="one length per sequence"):
        mod.decode_systematic_ragged(q, K, V, lens[:2], 256)


@pytest.mark.parametrize("name", list(cases.ROPE_CASES))
def test_rope_append_matches_reference_golden(name):
    """The fused RoPE + cache append + q pack launch against what the reference's tensor code produced
    (runtime_common.py:540-556, golden made by tests/golden/make_golden_rope.py): bit for bit."""
    from oracle import rope_append as ro
    c = cases.ROPE_CASES[name]
    g = np.load(os.path.join(GOLDEN, f"rope_{name}.npz"))
    dt = cases.torch_dtype(c["dtype"])
    B, pos = c["B"], c["pos"]
    q_proj, k_proj, v_proj, kc, vc = cases.make_rope_inputs(c)
    cos, sin = ro.rope_tables(torch.full((B,), pos), 128, dt)
    d = dev()
    kc_d, vc_d = kc.to(d), vc.to(d)
    q = ops().rope_append(q_proj.to(d), k_proj.to(d), v_proj.to(d), cos.to(d), sin.to(d), kc_d, vc_d, pos)
    torch.cuda.synchronize()
    assert (cases.bits(q) == g["ref_q"]).all()
    assert (cases.bits(kc_d[:, pos]) == g["ref_k_row"]).all()
    assert (cases.bits(vc_d[:, pos]) == g["ref_v_row"]).all()
    assert kc_d.float().abs().sum().item() == float(g["ref_k_cache_sum"])
    # the same with the three projections left in pinned host memory (read by the kernel over PCIe)
    kc_h, vc_h = kc.to(d), vc.to(d)
    q_h = ops().rope_append(q_proj.pin_memory(), k_proj.pin_memory(), v_proj.pin_memory(), cos.to(d), sin.to(d),
                            kc_h, vc_h, pos)
    torch.cuda.synchronize()
    assert torch.equal(q_h, q) and torch.equal(kc_h, kc_d) and torch.equal(vc_h, vc_d)
    with pytest.raises(RuntimeError, match="pinned host memory"):
        ops().rope_append(q_proj, k_proj.to(d), v_proj.to(d), cos.to(d), sin.to(d), kc_h, vc_h, pos)
    # device positions, one per sequence, with the new lengths written for the attention call
    q_proj, k_proj, v_proj, kc2, vc2 = cases.make_rope_inputs(c)
    plist = [(pos + 3 * b) % c["L"] for b in range(B)]
    cos2, sin2 = ro.rope_tables(torch.tensor(plist), 128, dt)
    q_ref = ro.rope_append_step(q_proj, k_proj, v_proj, cos2, sin2, kc2, vc2, plist)
    kc_d, vc_d = torch.full_like(kc_d, 0.5), torch.full_like(vc_d, -0.25)
    lens = torch.zeros(B, dtype=torch.int32, device=d)
    status = torch.zeros(1, dtype=torch.int32, device=d)
    q2 = ops().rope_append(q_proj.to(d), k_proj.to(d), v_proj.to(d), cos2.to(d), sin2.to(d), kc_d, vc_d,
                           torch.tensor(plist, dtype=torch.int32, device=d), seq_lens_out=lens, status=status)
    torch.cuda.synchronize()
    assert torch.equal(q2.cpu(), q_ref) and torch.equal(kc_d.cpu(), kc2) and torch.equal(vc_d.cpu(), vc2)
    assert lens.tolist() == [p + 1 for p in plist] and status.item() == 0
    # a position outside the cache is skipped and reported, nothing is written
    bad = torch.tensor([c["L"]] * B, dtype=torch.int32, device=d)
    before = kc_d.clone()
    ops().rope_append(q_proj.to(d), k_proj.to(d), v_proj.to(d), cos2.to(d), sin2.to(d), kc_d, vc_d, bad, status=status)
    torch.cuda.synchronize()
    assert status.item() == 3 and torch.equal(kc_d, before)
    with pytest.raises(RuntimeError, match="pos out of range"):
        ops().rope_append(q_proj.to(d), k_proj.to(d), v_proj.to(d), cos2.to(d), sin2.to(d), kc_d, vc_d, c["L"])


def test_sharded_module_path_equals_the_c_abi_mirror():
    """The compiled module's partial / combine functions (used by santa_b200.sharded) against the ctypes
    mirror, and the one-rank sequence-sharded call against the plain call."""
    import santa_b200
    from santa_b200 import sharded
    santa_b200.enable_dropin()
    import santa_flash_batch_cuda as mod
    q, K, V = cases.make_qkv(2, 9000, 8, "bf16", 61, 1.0, True)
    q, K, V = q.to(dev()), K.to(dev()), V.to(dev())
    L, S = 8700, 300
    bn, T_c, spt, plan = sharded.shard_plan(L, 3, S)
    parts = []
    for row0, row1, tile0 in plan:
        Ks, Vs = K[:, row0:row1].contiguous(), V[:, row0:row1].contiguous()
        p_mod = mod.decode_systematic_partial(q, Ks, Vs, S, seed=9, block_n=bn, valid_len=row1 - row0,
                                              tile_offset=tile0, s_per_tile=spt)
        p_ops = ops().flash_decode(q, Ks, Vs, S, seed=9, block_n=bn, valid_len=row1 - row0, tile_offset=tile0,
                                   s_per_tile=spt, partial=True)[0]
        assert torch.equal(p_mod, p_ops)
        parts.append(p_mod)
    buf = torch.stack(parts)
    o_mod, m_mod = mod.lse_combine(buf, spt, True)
    o_ops, m_ops = ops().lse_combine(buf, spt, torch.bfloat16)
    assert torch.equal(o_mod, o_ops) and torch.equal(m_mod, m_ops)
    full = ops().flash_decode(q, K, V, S, seed=9, valid_len=L)
    assert close(o_mod, full[0]) and bits_eq(m_mod, full[1])
    one = sharded.seq_sharded_flash_decode(q, K[:, :L].contiguous(), V[:, :L].contiguous(), S, 9, L)
    assert close(one[0], full[0]) and bits_eq(one[1], full[1])


def test_flash_config3_full_size_properties():
    """Config 3 at full size (B=1, L=524288, S=1024 => 2048 tiles, one sample per head and tile), whole
    and as four sequence shards through the module path: size-independent properties."""
    import santa_b200
    from santa_b200 import sharded
    santa_b200.enable_dropin()
    import santa_flash_batch_cuda as mod
    L, S = 524288, 1024
    g = torch.Generator(device=dev()).manual_seed(33)
    q = torch.randn(1, 32, 128, device=dev(), generator=g).to(torch.bfloat16)
    K = torch.randn(1, L, 8, 128, device=dev(), generator=g).to(torch.bfloat16)
    V = torch.randn(1, L, 8, 128, device=dev(), generator=g).to(torch.bfloat16)
    out, m_star, vrows, tr = ops().flash_decode(q, K, V, S, seed=1690, want_vrows=True, trace=True)
    torch.cuda.synchronize()
    assert ops().workspace_status("flash", dev()) == 0
    assert (tr.block_n, tr.T_c, tr.S_per_tile) == (256, 2048, 1)
    per_tile = tr.counts.view(1, 32, 2048, 256).sum(-1)
    assert per_tile.min() >= 0 and per_tile.max() <= 2 and abs(per_tile.float().mean().item() - 1.0) < 0.02
    flagged = (tr.counts.view(1, 8, 4, L) > 0).any(2)
    assert (flagged.sum(-1).int() == vrows).all() and ((tr.rowmask != 0) == flagged).all()
    assert bits_eq(m_star, tr.m_tiles.max(-1).values)
    assert close(out, flash_eval_torch(tr.counts, V, tr.m_tiles, tr.ell_tiles, 256, 1))
    bn, T_c, spt, plan = sharded.shard_plan(L, 4, S)
    assert (bn, T_c, spt) == (256, 2048, 1) and [p[2] for p in plan] == [0, 512, 1024, 1536]
    parts = [mod.decode_systematic_partial(q, K[:, r0:r1], V[:, r0:r1], S, seed=1690, block_n=bn,
                                           valid_len=r1 - r0, tile_offset=t0, s_per_tile=spt)
             for r0, r1, t0 in plan]
    o4, m4 = mod.lse_combine(torch.stack(parts), spt, True)
    assert bits_eq(m4, m_star) and close(o4, out)


def test_prop_config2_full_size_properties():
    """Config 2 at full size through the ragged entry: 16 sequences with the seed-7 lengths, S=256."""
    lengths = torch.randint(8192, 65537, (16,), generator=torch.Generator().manual_seed(7)).tolist()
    B, Ls, S = 16, 65536, 256
    g = torch.Generator(device=dev()).manual_seed(34)
    q = torch.randn(B, 32, 128, device=dev(), generator=g).to(torch.bfloat16)
    K = torch.randn(B, Ls, 8, 128, device=dev(), generator=g).to(torch.bfloat16)
    V = torch.randn(B, Ls, 8, 128, device=dev(), generator=g).to(torch.bfloat16)
    lens = torch.tensor(lengths, dtype=torch.int32, device=dev())
    out, m_star, vrows, tr = ops().prop_decode_ragged(q, K, V, lens, S, seed=1690, want_vrows=True, trace=True)
    out2 = ops().prop_decode_ragged(q, K, V, lens, S, seed=1690)[0]
    torch.cuda.synchronize()
    assert ops().workspace_status("prop_ragged", dev()) == 0
    assert torch.equal(out, out2)                                           # fixed summation order
    for b, Lb in enumerate(lengths):
        T = (Lb + 255) // 256
        St = tr.S_tiles[b, :, :T]
        assert (St.sum(1) <= S).all() and (St.sum(1) >= S - T).all() and (tr.S_tiles[b, :, T:] == 0).all()
        cnt = tr.counts[b].view(32, 256, 256).sum(-1)[:, :T]                # [H, tiles] (max_len = 256 tiles)
        assert ((cnt - St).abs() <= 1).all()
        assert (tr.counts[b, :, Lb:] == 0).all()
        flagged = (tr.counts[b].view(8, 4, Ls) > 0).any(1)
        assert (flagged.sum(-1).int() == vrows[b]).all()
        assert bits_eq(m_star[b], tr.m_tiles[b, :, :T].max(-1).values)
        ev = torch.zeros(32, 128, device=dev())
        for kv in range(8):
            ev[4 * kv:4 * kv + 4] = tr.counts[b, 4 * kv:4 * kv + 4, :Lb].float() @ V[b, :Lb, kv].float()
        assert close(out[b], ev / S)


def test_peer_exchange_on_one_device():
    """The peer-exchange path with every 'rank' on this GPU: three shards deliver their partials into
    three exchange buffers (all local), each buffer's owner then waits and combines.  Epochs alternate
    the buffer halves; a wait for a partial that nobody sent runs out and reports, without hanging."""
    import santa_b200
    from santa_b200 import capi, sharded
    santa_b200.enable_dropin()
    import santa_flash_batch_cuda as mod
    q, K, V = cases.make_qkv(2, 9000, 8, "bf16", 71, 1.0, True)
    q, K, V = q.to(dev()), K.to(dev()), V.to(dev())
    L, S, G, B, H = 8700, 300, 3, 2, 32
    bn, T_c, spt, plan = sharded.shard_plan(L, G, S)
    nbytes = capi.lib().santa_peer_exchange_bytes(G, B * H)
    bufs = [torch.zeros(nbytes, dtype=torch.uint8, device=dev()) for _ in range(G)]
    ptrs = [b.data_ptr() for b in bufs]
    status = torch.zeros(1, dtype=torch.int32, device=dev())
    full = ops().flash_decode(q, K, V, S, seed=9, valid_len=L)
    for epoch in (1, 2, 3):
        qe = q if epoch != 2 else (q * 0.5).to(torch.bfloat16)           # another step, other data
        ref = full if epoch != 2 else ops().flash_decode(qe, K, V, S, seed=9, valid_len=L)
        for r, (row0, row1, tile0) in enumerate(plan):
            mod.decode_systematic_exchange(qe, K[:, row0:row1].contiguous(), V[:, row0:row1].contiguous(), S, 9, bn,
                                           row1 - row0, 0, tile0, spt, ptrs, r, epoch)
        for r in range(G):
            o, m = mod.lse_combine_wait(ptrs, r, epoch, B, H, spt, True, status)
            assert close(o, ref[0]) and bits_eq(m, ref[1])
            if epoch == 1 and r == G - 1:
                sep = (o.clone(), m.clone())      # the separate wait-and-combine kernel's result for q
        assert status.item() == 0
    # nobody sends epoch 4: the wait gives up after its bound and says so
    o, m = mod.lse_combine_wait(ptrs, 0, 4, B, H, spt, True, status)
    torch.cuda.synchronize()
    assert status.item() == 4 and (o == 0).all()
    # device-counted epochs: the same two calls, captured once in a CUDA graph, serve every step
    bufs2 = [torch.zeros(nbytes, dtype=torch.uint8, device=dev()) for _ in range(G)]
    ptrs2 = [b.data_ptr() for b in bufs2]
    qs = q.clone()
    shards = [(K[:, r0:r1].contiguous(), V[:, r0:r1].contiguous(), r1 - r0, t0) for r0, r1, t0 in plan]

    def step_all_ranks():
        for r, (Ks, Vs, n, t0) in enumerate(shards):
            mod.decode_systematic_exchange(qs, Ks, Vs, S, 9, bn, n, 0, t0, spt, ptrs2, r, 0)
        return [mod.lse_combine_wait(ptrs2, r, 0, B, H, spt, True, status) for r in range(G)]

    status.zero_()
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        warm = step_all_ranks()                                            # step 1, eager
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    assert close(warm[0][0], full[0])
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph, stream=side):
        outs = step_all_ranks()
    for k in range(3):                                                     # steps 2, 3, 4: replays
        qs.copy_(q if k != 1 else (q * 0.5).to(torch.bfloat16))
        graph.replay()
        torch.cuda.synchronize()
        ref = full if k != 1 else ops().flash_decode(qs, K, V, S, seed=9, valid_len=L)
        for r in range(G):
            assert close(outs[r][0], ref[0]) and bits_eq(outs[r][1], ref[1])
    assert status.item() == 0
    steps_done = bufs2[0][4 * 33:4 * 34].view(torch.int32).item()
    assert steps_done == 4
    # receiving half inside the decode call (SANTA_PEER_COMBINE): the first two 'ranks' only send, the
    # third finds every row present and returns the combined result -- the same bits as the wait kernel's
    bufs3 = [torch.zeros(nbytes, dtype=torch.uint8, device=dev()) for _ in range(G)]
    ptrs3 = [b.data_ptr() for b in bufs3]
    for epoch in (1, 2):
        for r, (Ks, Vs, n, t0) in enumerate(shards):
            res = mod.decode_systematic_exchange(q, Ks, Vs, S, 9, bn, n, 0, t0, spt, ptrs3, r, epoch, r == G - 1)
        assert torch.equal(res[0], sep[0]) and torch.equal(res[1], sep[1])
        assert close(res[0], full[0]) and bits_eq(res[1], full[1])
    assert status.item() == 0 and bufs3[G - 1][4 * 34:4 * 35].view(torch.int32).item() == 0
    # ... and when the others never send, its bounded wait runs out: zeros and status 4, no hang
    Ks, Vs, n, t0 = shards[0]
    res = mod.decode_systematic_exchange(q, Ks, Vs, S, 9, bn, n, 0, t0, spt, ptrs3, 0, 3, True)
    torch.cuda.synchronize()
    assert (res[0] == 0).all() and bufs3[0][4 * 34:4 * 35].view(torch.int32).item() == 4
    # the one-rank object goes through the same kernels
    ex = sharded.PeerExchange(B, H, dev())
    one = sharded.seq_sharded_flash_decode(q, K[:, :L].contiguous(), V[:, :L].contiguous(), S, 9, L, exchange=ex)
    two = sharded.seq_sharded_flash_decode(q, K[:, :L].contiguous(), V[:, :L].contiguous(), S, 9, L, exchange=ex)
    ex.check()
    assert close(one[0], full[0]) and bits_eq(one[1], full[1]) and torch.equal(one[0], two[0])


def test_c_abi_from_a_plain_cxx_host(tmp_path):
    """tests/capi_host.cu -- a C++ program without PyTorch -- linked against libsanta_b200.so: its output
    equals the Python mirror's on the same generated bits."""
    import shutil
    import subprocess
    from santa_b200 import capi
    if shutil.which("nvcc") is None:
        pytest.skip("no nvcc on this box")
    exe = str(tmp_path / "capi_host")
    libdir = os.path.dirname(capi.LIB_PATH)
    subprocess.check_call(["nvcc", "-O1", "-std=c++17", "-o", exe, os.path.join(HERE, "capi_host.cu"),
                           "-L" + libdir, "-lsanta_b200", "-Xlinker", "-rpath," + libdir])
    B, L, KVH, S, seed = 2, 3000, 2, 96, 1690
    txt = subprocess.check_output([exe, str(B), str(L), str(KVH), str(S), str(seed)], text=True, timeout=120)
    lines = dict(ln.split(" ", 1) for ln in txt.strip().split("\n"))
    assert lines["status"] == "0"
    # the same recurrence in Python
    n = B * 4 * KVH * 128 + 2 * B * L * KVH * 128
    st, vals = 12345, np.empty(n, dtype=np.float32)
    for i in range(n):
        st = (st * 1664525 + 1013904223) & 0xffffffff
        vals[i] = (((st >> 16) & 0xff) - 128) / 64.0
    t = torch.from_numpy(vals).to(torch.bfloat16)
    nq, nk = B * 4 * KVH * 128, B * L * KVH * 128
    q = t[:nq].view(B, 4 * KVH, 128).to(dev())
    K = t[nq:nq + nk].view(B, L, KVH, 128).to(dev())
    V = t[nq + nk:].view(B, L, KVH, 128).to(dev())
    out, m_star, vrows = ops().flash_decode(q, K, V, S, seed=seed, want_vrows=True)
    assert [int(x) for x in lines["vrows"].split()] == vrows.flatten().tolist()
    got = np.array([int(x) for x in lines["out"].split()], dtype=np.uint16)
    assert (got == cases.bits(out).reshape(-1)).all()
