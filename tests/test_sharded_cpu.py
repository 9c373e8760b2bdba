"""Host-side logic of the multi-GPU paths, exercised with world_size-2 gloo ranks on CPU: the tile-aligned
shard plan, the all-gather of per-rank partials and the log-sum-exp merge rule.  The per-rank partials
come from the CPU oracle (the CUDA kernels need a GPU); the merged result must equal the unsharded
oracle result."""
import os

import numpy as np
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import cases
from oracle import santa_oracle as so
from santa_b200 import sharded


def test_shard_plan_covers_sequence_on_tile_boundaries():
    for L, world, S in [(524288, 8, 1024), (524288, 3, 1024), (4096, 2, 32), (1000, 4, 64), (300, 8, 16)]:
        bn, T_c, spt, plan = sharded.shard_plan(L, world, S)
        assert (T_c, spt) == so.flash_budget(L, bn, S)
        assert plan[0][0] == 0 and plan[-1][1] == L
        for (a0, a1, t0), (b0, b1, t1) in zip(plan, plan[1:]):
            assert a1 == b0 and a0 % bn == 0 and b0 % bn == 0 or a1 == L
            assert t1 == t0 + (a1 - a0 + bn - 1) // bn
    # the per-shard rule would give the wrong budget: the plan carries the global one
    assert sharded.shard_plan(524288, 8, 1024)[2] == 1


def _oracle_partial(q16, K16, V16, S, seed, bn, tile0, spt):
    """Unnormalised partial [H,130] of one shard, from the oracle's per-tile results."""
    r = so.flash_decode(q16, K16, V16, S, seed=seed, block_n=bn, tile_offset=tile0, S_per_tile=spt)
    H = q16.shape[1]
    part = np.zeros((H, 130), np.float32)
    for h in range(H):
        ms = r.m_tiles[0, h].max()
        w = np.exp(r.m_tiles[0, h].astype(np.float64) - ms) * r.ell_tiles[0, h]
        part[h, 128], part[h, 129] = ms, w.sum()
        part[h, :128] = r.out[0, h].astype(np.float64) * w.sum() * spt
    return part, r.counts


def _worker(rank, world, port, L, S, seed, ret):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        q, K, V = cases.make_qkv(1, L, 2, "bf16", 55, 1.0, True)
        q16, K16, V16 = cases.bits(q), cases.bits(K), cases.bits(V)
        bn, T_c, spt, plan = sharded.shard_plan(L, world, S, 256)
        row0, row1, tile0 = plan[rank]
        part, counts = _oracle_partial(q16, K16[:, row0:row1], V16[:, row0:row1], S, seed, bn, tile0, spt)
        mine = torch.from_numpy(part)[None]                      # [B=1,H,130]
        buf = torch.empty(world, *mine.shape)
        dist.all_gather_into_tensor(buf.view(world * mine.size(0), *mine.shape[1:]), mine)
        out, m_star = sharded.merge_partials_reference(buf, spt)
        cnt_all = [None] * world
        dist.all_gather_object(cnt_all, counts)
        if rank == 0:
            ret["out"], ret["m_star"], ret["counts"], ret["spt"] = out.numpy(), m_star.numpy(), np.concatenate(cnt_all, axis=2), spt
    finally:
        dist.destroy_process_group()


def test_two_rank_sequence_sharded_merge_equals_unsharded():
    L, S, seed = 2048, 64, 13
    mgr = mp.Manager()
    ret = mgr.dict()
    port = 29500 + (os.getpid() % 2000)
    mp.spawn(_worker, args=(2, port, L, S, seed, ret), nprocs=2, join=True)
    q, K, V = cases.make_qkv(1, L, 2, "bf16", 55, 1.0, True)
    full = so.flash_decode(cases.bits(q), cases.bits(K), cases.bits(V), S, seed=seed, block_n=256)
    assert ret["spt"] == full.S_per_tile
    assert (ret["counts"] == full.counts).all()          # same samples as the single-device call
    assert np.abs(ret["out"][0] - full.out[0]).max() < 1e-5
    assert (ret["m_star"][0] == full.m_star[0]).all()
    # the oracle's own merge agrees with the torch restatement used on the ranks
    assert np.abs(sharded.merge_partials_reference(torch.zeros(1, 1, 8, 130).fill_(1.0), 2)[0].numpy()
                  - so.merge_partials(np.ones((1, 8, 130), np.float32), 2)[0]).max() < 1e-6


def test_batch_sharding_offsets_reproduce_unsharded_counts():
    """Batch shards: rank r passes batch_offset = first global sequence index (RNG key b*H+h)."""
    q, K, V = cases.make_qkv(4, 600, 2, "bf16", 8, 1.0, False)
    q16, K16, V16 = cases.bits(q), cases.bits(K), cases.bits(V)
    full = so.flash_decode(q16, K16, V16, 64, seed=3)
    halves = [so.flash_decode(q16[o:o + 2], K16[o:o + 2], V16[o:o + 2], 64, seed=3, batch_offset=o) for o in (0, 2)]
    assert (np.concatenate([h.counts for h in halves]) == full.counts).all()
    wrong = so.flash_decode(q16[2:], K16[2:], V16[2:], 64, seed=3)      # without the offset the samples differ
    assert (wrong.counts != full.counts[2:]).any()
