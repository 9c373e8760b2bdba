"""CPU-only checks of the oracle (oracle/santa_oracle.c) against known answers and
against the golden fixtures produced by the reference's own kernels."""
import math
import os
import struct

import numpy as np
import pytest
import torch

import cases
from oracle import santa_oracle as so

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def f32bits(x):
    return struct.unpack("<I", struct.pack("<f", float(x)))[0]


# splitmix64 offsets u01(seed=1690, h, t): values computed from the published
# splitmix64 finaliser with an independent big-integer implementation.
U01_KATS = [
    (0, 0, 0x3ED0C35F), (0, 1, 0x3E2857FF), (0, 127, 0x3EFCA861),
    (1, 0, 0x3F37C7CA), (1, 1, 0x3F306E37), (1, 127, 0x3F61BFD6),
    (31, 0, 0x3F0E8EA5), (31, 1, 0x3E449A44), (31, 127, 0x3DEA5904),
    (32, 0, 0x3F627ACF), (32, 1, 0x3F35E7BC), (32, 127, 0x3F2A89D6),
]


def _u01_bigint(seed, h, t):
    mask = (1 << 64) - 1
    x = (seed ^ (((h << 32) & mask) ^ (t & mask))) & mask
    z = (x + 0x9E3779B97F4A7C15) & mask
    z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & mask
    z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & mask
    z = z ^ (z >> 31)
    return np.float32((z >> 11) * (1.0 / 9007199254740992.0))


@pytest.mark.parametrize("h,t,bits", U01_KATS)
def test_u01_known_answers(h, t, bits):
    assert f32bits(so.u01(1690, h, t)) == bits
    assert f32bits(_u01_bigint(1690, h, t)) == bits


def test_u01_random_against_bigint():
    rng = np.random.default_rng(0)
    for _ in range(200):
        seed = int(rng.integers(0, 2**63)) * 2 + int(rng.integers(0, 2))
        h, t = int(rng.integers(0, 4096)), int(rng.integers(0, 1 << 20))
        assert f32bits(so.u01(seed, h, t)) == f32bits(_u01_bigint(seed, h, t))


BUDGET_KATS = [  # (L, S) -> (block_n, T_c, S_per_tile)
    ((16, 2048), (32, 1, 2048)), ((1536, 256), (32, 48, 5)), ((1537, 256), (64, 25, 10)),
    ((3072, 256), (64, 48, 5)), ((3073, 256), (256, 13, 19)), ((4096, 32), (256, 16, 2)),
    ((32768, 256), (256, 128, 2)), ((32769, 256), (256, 129, 1)), ((524288, 1024), (256, 2048, 1)),
    ((100, 0), (32, 4, 0)), ((5000, 1), (256, 20, 1)),
]


@pytest.mark.parametrize("inp,exp", BUDGET_KATS)
def test_budget_rule(inp, exp):
    L, S = inp
    bn = so.block_n_rule(L)
    assert (bn,) + so.flash_budget(L, bn, S) == exp


def test_explicit_block_n_wins():
    assert so.block_n_rule(100000, 64) == 64 and so.block_n_rule(10, 256) == 256


def test_16bit_conversions_match_torch():
    x = torch.randn(4096) * 3
    x[:8] = torch.tensor([0.0, -0.0, 1e-40, 65504.0, 1e38, float("inf"), -float("inf"), 1.0 + 2**-9])
    for isb, dt in ((True, torch.bfloat16), (False, torch.float16)):
        mine = so.to16(x.numpy(), isb)
        ref = x.to(dt).view(torch.int16).numpy().view(np.uint16)
        assert (mine == ref).all()
        assert (so.from16(mine, isb) == x.to(dt).float().numpy()).all()


def _dense_counts(g, shape):
    c = np.zeros(int(np.prod(shape)), np.int16)
    c[g["ref_counts_idx"]] = g["ref_counts_val"]
    return c.reshape(shape)


@pytest.mark.parametrize("name", list(cases.FLASH_CASES))
def test_flash_oracle_vs_reference_golden(name):
    """Oracle vs the reference kernels' own results: max scores, offsets and -- downstream of the
    two hardware-approximate intermediates -- sampled counts, gathered-row counts and m_star are
    bit-exact; ell and the estimator output agree to rounding."""
    c = cases.FLASH_CASES[name]
    g = np.load(os.path.join(GOLDEN, f"flash_{name}.npz"))
    q, K, V = cases.make_qkv(c["B"], c["Ls"], c["KVH"], c["dtype"], c["gen_seed"], c["kscale"], c["heavy"])
    isb = c["dtype"] == "bf16"
    q16, K16, V16 = cases.bits(q), cases.bits(K), cases.bits(V)
    H = 4 * c["KVH"]
    ref_counts = _dense_counts(g, (c["B"], H, c["L"]))

    r = so.flash_decode(q16, K16, V16, c["S"], seed=c["seed"], block_n=c["block_n"], valid_len=c["L"], is_bf16=isb)
    assert (r.block_n, r.T_c, r.S_per_tile) == (int(g["block_n"]), int(g["T_c"]), int(g["S_per_tile"]))
    # pure IEEE parts: bit-exact
    assert (r.m_tiles.view(np.int32) == g["ref_m_tiles"].view(np.int32)).all()
    assert (r.m_star.view(np.int32) == g["ref_m_star"].view(np.int32)).all()
    # parts behind exp2/approximate division: a few ulps
    assert np.abs(r.ell_tiles / g["ref_ell_tiles"] - 1).max() < 1e-6
    assert (r.u16 != g["dev_u16"]).mean() < 1e-3
    assert (r.counts != ref_counts).mean() < 1e-3

    # with the device's u16 / ell / step injected everything downstream is exact
    r2 = so.flash_decode(q16, K16, V16, c["S"], seed=c["seed"], block_n=c["block_n"], valid_len=c["L"], is_bf16=isb,
                         inject_u16=g["dev_u16"], inject_ell=g["ref_ell_tiles"], inject_invdel=g["dev_invdel"])
    assert (r2.counts == ref_counts).all()
    assert (r2.vrows == g["ref_vrows"]).all()
    out_ref = so.from16(g["ref_out"], isb)
    assert np.abs(r2.out - out_ref).max() <= 2e-2 and np.abs(r2.out - out_ref).mean() <= 2e-3
    # and the estimator identity evaluated in float64 over those counts
    for b in range(c["B"]):
        ev = so.flash_eval_over_counts(ref_counts[b], so.from16(V16[b], isb), g["ref_m_tiles"][b],
                                       g["ref_ell_tiles"][b], r.block_n, r.S_per_tile)
        assert np.abs(ev - out_ref[b]).max() <= 2e-2 and np.abs(ev - out_ref[b]).mean() <= 2e-3


@pytest.mark.parametrize("name", list(cases.PROP_CASES))
def test_prop_oracle_vs_reference_golden(name):
    c = cases.PROP_CASES[name]
    g = np.load(os.path.join(GOLDEN, f"prop_{name}.npz"))
    q, K, V = cases.make_qkv(1, c["L"], c["KVH"], c["dtype"], c["gen_seed"], c["kscale"], c["heavy"], GH=c["GH"])
    isb = c["dtype"] == "bf16"
    q16, K16, V16 = cases.bits(q[0]), cases.bits(K[0]), cases.bits(V[0])
    H = c["GH"] * c["KVH"]
    ref_counts = _dense_counts(g, (H, c["L"]))
    u_ref = np.ascontiguousarray(g["ref_u_stash"].T)

    r = so.prop_decode(q16, K16, V16, c["S"], seed=c["seed"], block_n=c["block_n"], is_bf16=isb)
    assert (r.block_n, r.T_c) == (int(g["block_n"]), int(g["T_c"]))
    if so.prop_uses_vec(H, c["KVH"], 128, r.block_n):
        assert (r.m_tiles.view(np.int32) == g["ref_m_tiles"].view(np.int32)).all()
    else:  # tensor-core accumulation order is hardware-defined
        assert np.abs(r.m_tiles - g["ref_m_tiles"]).max() < 1e-5
    assert np.abs(r.ell_tiles / g["ref_ell_tiles"] - 1).max() < 2e-6
    assert (r.u16 != u_ref).mean() < 1e-3

    # budgets, offsets and steps from the reference's own tile statistics: bit-exact
    for flags in (0, 3):
        m_star, S_tiles, invdelta, a0, _ = so.prop_budgets(g["ref_m_tiles"], g["ref_ell_tiles"], c["S"], c["seed"], flags)
        assert (S_tiles == g["ref_S_tiles"]).all()
        assert (invdelta.view(np.int32) == g["ref_invdelta"].view(np.int32)).all()
        assert (a0.view(np.int32) == g["ref_a0"].view(np.int32)).all()
        assert (m_star.view(np.int32) == g["ref_m_star"].view(np.int32)).all()
    # counts from the reference's stash and tables: bit-exact
    cnt = so.prop_counts(u_ref, isb, r.block_n, g["ref_invdelta"], g["ref_a0"])
    assert (cnt == ref_counts).all()
    assert (so.rowflags(cnt, c["KVH"])[1] == g["ref_vrows"]).all()
    # estimator: the reference adds tiles with atomics in no fixed order -> rounding-level agreement
    out, _ = so.prop_estimate(cnt, V16, isb, r.block_n, c["S"])
    out_ref = so.from16(g["ref_out"], isb)
    assert np.abs(out - out_ref).max() <= 2e-2 and np.abs(out - out_ref).mean() <= 2e-3
    ev = so.prop_eval_over_counts(ref_counts, so.from16(V16, isb), c["S"])
    assert np.abs(ev - out_ref).max() <= 2e-2


def test_config0_behaviour():
    """Config 0 (B=1, L=4096, S=32, seed 1690): two samples per (head, tile), ~3% of V rows, and the
    sampled estimate is far from the dense output by design."""
    g = torch.Generator().manual_seed(1690)
    q = torch.randn(1, 32, 128, generator=g)
    K = torch.randn(1, 4096, 8, 128, generator=g) / math.sqrt(128)
    V = torch.randn(1, 4096, 8, 128, generator=g)
    r = so.flash_decode(so.to16(q.numpy()), so.to16(K.numpy()), so.to16(V.numpy()), 32, seed=1690)
    assert (r.block_n, r.T_c, r.S_per_tile) == (256, 16, 2)
    per_tile = r.counts.reshape(1, 32, 16, 256).sum(-1)
    assert per_tile.min() == 2 and per_tile.max() == 2
    assert r.vrows.min() >= 120 and r.vrows.max() <= 128
    dense = torch.nn.functional.scaled_dot_product_attention(
        q.unsqueeze(2), K.permute(0, 2, 1, 3), V.permute(0, 2, 1, 3), enable_gqa=True)[:, :, 0]
    assert (torch.from_numpy(r.out) - dense).abs().mean() > 0.05


def test_prop_budgets_sum_and_dropped_entries():
    rng = np.random.default_rng(1)
    # power-of-two tile count: largest remainder hands out exactly S samples
    m = rng.normal(size=(8, 64)).astype(np.float32)
    ell = rng.uniform(1, 50, size=(8, 64)).astype(np.float32)
    _, S_tiles, invdelta, a0, _ = so.prop_budgets(m, ell, 200, 5)
    assert (S_tiles.sum(1) == 200).all() and (S_tiles >= 0).all()
    assert ((invdelta > 0) == (S_tiles > 0)).all()
    # S == 0 -> all zero, offsets still defined
    _, S0, inv0, a00, _ = so.prop_budgets(m, ell, 0, 5)
    assert (S0 == 0).all() and (inv0 == 0).all() and (a00 == a0).all()
    # non power of two: the network may drop entries; budgets never exceed S
    m3 = rng.normal(size=(4, 35)).astype(np.float32)
    ell3 = rng.uniform(1, 50, size=(4, 35)).astype(np.float32)
    _, S3, _, _, _ = so.prop_budgets(m3, ell3, 64, 9)
    assert (S3.sum(1) <= 64).all() and (S3.sum(1) >= 64 - 35).all()


def test_merge_of_sharded_partials_equals_unsharded():
    """Sequence sharding: per-shard (A, m, Z) partials merged with the log-sum-exp rule reproduce the
    single-call estimator when shards use global tile indices and the global S_per_tile."""
    q, K, V = cases.make_qkv(1, 2048, 2, "bf16", 77, 1.0, True)
    q16, K16, V16 = cases.bits(q), cases.bits(K), cases.bits(V)
    S, seed, bn = 64, 13, 256
    full = so.flash_decode(q16, K16, V16, S, seed=seed, block_n=bn)
    G = 4
    Lr = 2048 // G
    parts = np.zeros((G, 8, 130), np.float32)
    cnts = []
    for r in range(G):
        sh = so.flash_decode(q16, K16[:, r * Lr:(r + 1) * Lr], V16[:, r * Lr:(r + 1) * Lr], S, seed=seed, block_n=bn,
                             tile_offset=r * (Lr // bn), S_per_tile=full.S_per_tile)
        cnts.append(sh.counts)
        # rebuild the shard's unnormalised partial from its tiles
        for h in range(8):
            ms = sh.m_tiles[0, h].max()
            w = np.exp(sh.m_tiles[0, h].astype(np.float64) - ms) * sh.ell_tiles[0, h]
            parts[r, h, 129] = w.sum()
            parts[r, h, 128] = ms
            parts[r, h, :128] = sh.out[0, h].astype(np.float64) * w.sum() * full.S_per_tile
    assert (np.concatenate(cnts, axis=2) == full.counts).all()
    out, m_star = so.merge_partials(parts, full.S_per_tile)
    assert np.abs(out - full.out[0]).max() < 1e-5
    assert (m_star == full.m_star[0]).all()


@pytest.mark.parametrize("name", list(cases.ROPE_CASES))
def test_rope_oracle_matches_reference_golden(name):
    """The written-out roundings of oracle/rope_append.py against the outputs of the reference's own
    apply_rotary_pos_emb + cache copies (tests/golden/make_golden_rope.py), bit for bit."""
    from oracle import rope_append as ro
    c = cases.ROPE_CASES[name]
    g = np.load(os.path.join(GOLDEN, f"rope_{name}.npz"))
    dt = cases.torch_dtype(c["dtype"])
    q_proj, k_proj, v_proj, kc, vc = cases.make_rope_inputs(c)
    cos, sin = ro.rope_tables(torch.full((c["B"],), c["pos"]), 128, dt)
    assert (cases.bits(cos) == g["cos"]).all() and (cases.bits(sin) == g["sin"]).all()
    q = ro.rope_append_step(q_proj, k_proj, v_proj, cos, sin, kc, vc, c["pos"])
    assert (cases.bits(q) == g["ref_q"]).all()
    assert (cases.bits(kc[:, c["pos"]]) == g["ref_k_row"]).all()
    assert (cases.bits(vc[:, c["pos"]]) == g["ref_v_row"]).all()
    assert kc.float().abs().sum().item() == float(g["ref_k_cache_sum"])   # no other row was touched
    # per-sequence positions: each sequence equals the single-position step on it alone
    if c["B"] > 1:
        q_proj, k_proj, v_proj, kc2, vc2 = cases.make_rope_inputs(c)
        pos = [(c["pos"] + 3 * b) % c["L"] for b in range(c["B"])]
        cos2, sin2 = ro.rope_tables(torch.tensor(pos), 128, dt)
        q2 = ro.rope_append_step(q_proj, k_proj, v_proj, cos2, sin2, kc2, vc2, pos)
        assert (cases.bits(q2[0]) == g["ref_q"][0]).all()
        assert (cases.bits(kc2[0, pos[0]]) == g["ref_k_row"][0]).all()
