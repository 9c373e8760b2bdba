"""The opt-in tensor-core score mode (SANTA_SCORE_TENSOR) against the exact mode.

The exact mode's sampled counts equal the reference binary's bit for bit (tests/test_decode_gpu.py), so
the distance of the tensor-core mode from the exact mode IS its distance from the reference.  What is
asserted: the scores agree to fp32 accumulation noise (tile maxima within 1e-4), at most 0.5 % of the
sampled (row, head) count entries differ, the output evaluated in fp32 over the mode's OWN counts is
within max-abs 2e-2 / mean-abs 2e-3, and against the exact mode's output the mean-abs bound 2e-3 holds.
The max-abs distance to the exact output is only bounded loosely: with one or two samples per tile a
single sample that moves to a neighbouring row shifts a head's output by up to |V_a - V_b| / S, more
than 2e-2 for small S; the test prints the measured value."""
import pytest
import torch

import cases
from test_decode_gpu import close, dev, flash_eval_torch, ops

pytestmark = pytest.mark.gpu
MISMATCH_BOUND = 0.005

SHAPES = [  # B, L, Ls, KVH, S, seed, dtype, block_n
    (2, 5000, 5200, 8, 256, 1690, "bf16", 0),
    (2, 5000, 5000, 8, 2048, 3, "f16", 0),
    (1, 2500, 2500, 4, 300, 5, "bf16", 0),
    (3, 700, 768, 2, 64, 11, "f16", 0),
    (2, 1, 4, 2, 64, 11, "bf16", 0),
    (2, 257, 257, 2, 64, 11, "bf16", 0),
    (1, 40000, 40000, 8, 256, 7, "bf16", 0),
]


@pytest.mark.parametrize("B,L,Ls,KVH,S,seed,dtype,block_n", SHAPES)
def test_flash_tensor_scores_stay_close_to_the_exact_mode(B, L, Ls, KVH, S, seed, dtype, block_n):
    q, K, V = cases.make_qkv(B, Ls, KVH, dtype, 300 + L, 1.0, True)
    q, K, V = q.to(dev()), K.to(dev()), V.to(dev())
    kw = dict(seed=seed, block_n=block_n, want_vrows=True, valid_len=L, trace=True)
    o0, m0, v0, t0 = ops().flash_decode(q, K, V, S, **kw)
    o1, m1, v1, t1 = ops().flash_decode(q, K, V, S, score_mode=1, **kw)
    torch.cuda.synchronize()
    assert ops().workspace_status("flash", dev()) == 0
    assert (t0.m_tiles - t1.m_tiles).abs().max().item() <= 1e-4 and (m0 - m1).abs().max().item() <= 1e-4
    c0, c1 = t0.counts.int(), t1.counts.int()
    sampled = int((c0 > 0).sum().item())
    differing = int((c0 != c1).sum().item())
    assert differing <= max(2, MISMATCH_BOUND * sampled), (differing, sampled)
    assert (c1.sum(-1) - c0.sum(-1)).abs().max().item() <= 2          # the same budget per head, give or take a row
    # the estimator over the mode's own counts, in fp32
    ev = flash_eval_torch(t1.counts, V, t1.m_tiles, t1.ell_tiles, t1.block_n, t1.S_per_tile)
    assert close(o1, ev)
    d = (o0.float() - o1.float()).abs()
    print(f"tensor-vs-exact: {differing}/{sampled} count entries differ, out max-abs {d.max().item():.3e} "
          f"mean-abs {d.mean().item():.3e}")
    assert d.mean().item() <= 2e-3 and d.max().item() <= 0.25


def test_ragged_and_prop_entries_take_the_tensor_mode():
    """The ragged Flash call and both Prop calls accept the switch; results stay close to the exact mode and
    the Prop budgets -- sums over whole tiles, insensitive to single rows -- stay the same up to one sample."""
    q, K, V = cases.make_qkv(3, 9000, 8, "bf16", 77, 1.0, True)
    q, K, V = q.to(dev()), K.to(dev()), V.to(dev())
    lens = [9000, 4100, 6500]
    a = ops().flash_decode_ragged(q, K, V, lens, 256, seed=5, want_vrows=True)
    b = ops().flash_decode_ragged(q, K, V, lens, 256, seed=5, want_vrows=True, score_mode=1)
    d = (a[0].float() - b[0].float()).abs()
    assert d.mean().item() <= 2e-3 and (a[2] - b[2]).abs().max().item() <= 4
    pa = ops().prop_decode_ragged(q, K, V, lens, 256, seed=5, want_vrows=True, trace=True)
    pb = ops().prop_decode_ragged(q, K, V, lens, 256, seed=5, want_vrows=True, trace=True, score_mode=1)
    d = (pa[0].float() - pb[0].float()).abs()
    assert d.mean().item() <= 2e-3
    assert (pa[3].S_tiles - pb[3].S_tiles).abs().max().item() <= 1
    sampled = int((pa[3].counts > 0).sum().item())
    assert int((pa[3].counts != pb[3].counts).sum().item()) <= max(4, 0.02 * sampled)
    sa = ops().prop_decode(q[0], K[0, :7000].contiguous(), V[0, :7000].contiguous(), 128, seed=9)
    sb = ops().prop_decode(q[0], K[0, :7000].contiguous(), V[0, :7000].contiguous(), 128, seed=9, score_mode=1)
    torch.cuda.synchronize()
    assert (sa[0].float() - sb[0].float()).abs().mean().item() <= 2e-3
    assert ops().workspace_status("prop", dev()) == 0 and ops().workspace_status("prop_ragged", dev()) == 0
    # the drop-in modules take it as a keyword-only extra; the default is the reference's arithmetic
    import santa_b200
    santa_b200.enable_dropin()
    import santa_flash_batch_cuda as fm
    import santa_prop_batch_cuda as pm
    e = fm.decode_systematic_batched(q, K, V, 256, seed=5)[0]
    t = fm.decode_systematic_batched(q, K, V, 256, seed=5, score_mode=1)[0]
    assert torch.equal(e, ops().flash_decode(q, K, V, 256, seed=5)[0])
    assert torch.equal(t, ops().flash_decode(q, K, V, 256, seed=5, score_mode=1)[0])
    t = pm.decode_systematic_scalar(q[0], K[0, :7000].contiguous(), V[0, :7000].contiguous(), 128, seed=9, score_mode=1)[0]
    assert torch.equal(t, sb[0])
    with pytest.raises(TypeError):
        fm.decode_systematic_batched(q, K, V, 256, 5, 0, False, -1, 1)      # keyword-only
    # the backend objects and the decode runtime pass the switch on; unset, they make the reference's call
    from santa_b200 import backends
    fb0, fb1 = backends.make_backend("santa_flash", santa_s=256, santa_seed=5), \
        backends.make_backend("santa_flash", santa_s=256, santa_seed=5, score_mode=1)
    assert torch.equal(fb0.decode(q, K, V, 9000), e) and torch.equal(fb1.decode(q, K, V, 9000), t0 := fm.decode_systematic_batched(q, K, V, 256, seed=5, score_mode=1)[0])
    assert fb0.info()["score_mode"] == 0 and fb1.info()["score_mode"] == 1 and not torch.equal(e, t0)
    pb1 = backends.make_backend("santa_prop", santa_s=256, santa_seed=5, score_mode=1)
    lens_t = torch.tensor(lens, dtype=torch.int32, device=dev())
    assert torch.equal(pb1.decode(q, K, V, lens_t), pb[0])
